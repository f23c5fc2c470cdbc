"""Seeded input generators shared by the tests: the package's own synthetic-input module."""
from zk_inference_prover_b200.synth import MASK, P, edge_m31_column, m31_column, qm31_array, splitmix64  # noqa: F401
