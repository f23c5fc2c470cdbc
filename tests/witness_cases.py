"""Seeded witness-generation cases: the package's own module (shared with the benchmark)."""
from zk_inference_prover_b200.witness_cases import *  # noqa: F401,F403
