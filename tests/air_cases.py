"""Seeded AIR cases: the package's own module (shared with the benchmark)."""
from zk_inference_prover_b200.air_cases import *  # noqa: F401,F403
from zk_inference_prover_b200.air_cases import _shift  # noqa: F401
