"""Generates tests/golden/proof_digests.json: SHA-256 digests of whole proofs (the word streams of
include/zkb200_prover.h) and of constraint-quotient accumulators (include/zkb200_air.h) produced by the CPU oracle
on seeded inputs.

The reference is Rust and cannot be run with this image's toolchains, so these vectors are outputs of
the oracle (which is pinned to the reference's own known-answer tests in tests/test_oracle_kats.py), not
of the reference binary. They serve two purposes: (1) the CUDA path is compared with them at sizes the
oracle needs minutes for (256 columns of 2^20 rows; one GKR instance of 2^24 fractions) without running
the oracle on the GPU machine; (2) a change of the oracle that alters any proof byte is caught on CPU.

    python tests/golden/make_golden.py            # small cases, seconds
    python tests/golden/make_golden.py --full     # adds the full-size cases, minutes and ~12 GiB of RAM
"""
import argparse
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, ".."))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

import oracle  # noqa: E402
from util import m31_column, qm31_array  # noqa: E402

OUT = os.path.join(HERE, "proof_digests.json")

# name -> (per-tree list of column log sizes, seed, prover parameters)
PCS_SMALL = {
    "pcs_1x2e6": ([[6]], 4000, dict(pow_bits=0, log_blowup=1, n_queries=3)),
    "pcs_default_config_3x2e5": ([[5, 5, 5]], 4000, dict(pow_bits=10, log_blowup=1, n_queries=3)),
    "pcs_mixed_sizes": ([[4, 6, 6, 5, 8, 8, 4]], 4000, dict(pow_bits=3, log_blowup=1, n_queries=20, two_sample_every=2)),
    "pcs_two_trees": ([[6, 6], [7, 5, 7, 3]], 4000, dict(pow_bits=0, log_blowup=1, n_queries=100)),
    "pcs_20cols_last_layer_2": ([[10] * 17 + [7] * 3], 4000, dict(pow_bits=5, log_blowup=2, n_queries=16, log_last_layer=2, two_sample_every=5)),
    "pcs_16x2e14_blowup4": ([[14] * 16], 0x5EED0001, dict(pow_bits=10, log_blowup=2, n_queries=3)),
}
# the benchmark workload: seeds 0x5EED0001 + column, default PcsConfig, blow-up 4
PCS_FULL = {
    "pcs_256x2e20_blowup4": ([[20] * 256], 0x5EED0001, dict(pow_bits=10, log_blowup=2, n_queries=3, cap=1 << 26)),
    # the same trace with the prover's own parameters (prover/src/util.rs:14-28): blow-up 2, 100 queries, no grinding
    "pcs_256x2e20_blowup2_pow0_q100": ([[20] * 256], 0x5EED0001, dict(pow_bits=0, log_blowup=1, n_queries=100, cap=1 << 26)),
}
# name -> (list of (kind, log size, seed), channel seed)
GKR_SMALL = {
    "gkr_grand_product_2e10": ([(0, 10, 5000)], 77),
    "gkr_logup_generic_2e9": ([(1, 9, 5010)], 78),
    "gkr_logup_multiplicities_2e12": ([(2, 12, 0x5EED0002)], 0x5EED0004),
    "gkr_logup_singles_2e8": ([(3, 8, 5030)], 79),
    "gkr_batch_mixed": ([(0, 7, 5040), (2, 11, 5050), (3, 4, 5060), (1, 9, 5070)], 80),
}
GKR_FULL = {
    "gkr_logup_multiplicities_2e24": ([(2, 24, 0x5EED0002)], 0x5EED0004),
}


# constraint quotients of an AIR (tests/air_cases.py): the accumulator's 4 x 2^eval_log words from the oracle's evaluator
# written against CpuDomainEvaluator. Small: index into air_cases.small_cases; full: the benchmark's two workloads.
AIR_SMALL = {f"air_small_{i}": i for i in range(8)}
AIR_FULL = {"air_wide_fibonacci_256x2e20": "wide_fibonacci", "air_freivalds_pk16_pq1_2mats_2e20": "freivalds"}


# whole STARK proofs of a wide Fibonacci component (oracle/stark.hpp): name -> (columns, trace log, prover parameters)
STARK_SMALL = {
    "stark_wide_fibonacci_10x2e6": (10, 6, dict(pow_bits=5, log_blowup=1, n_queries=7)),
    "stark_wide_fibonacci_24x2e10_blowup4": (24, 10, dict(pow_bits=10, log_blowup=2, n_queries=3)),
}
STARK_FULL = {
    "stark_wide_fibonacci_256x2e20_blowup4": (256, 20, dict(pow_bits=10, log_blowup=2, n_queries=3, cap=1 << 26)),
}


def stark_oracle(name):
    import air_cases

    n_cols, trace_log, kw = dict(STARK_SMALL, **STARK_FULL)[name]
    trace = air_cases.wide_fibonacci_trace(n_cols, trace_log)
    w, committed, at_point = oracle.stark_prove(0, [n_cols], np.zeros(4, np.uint32), [0, 0, n_cols, 0], trace, trace_log, trace_log + 1, **kw)
    assert (committed == at_point).all()
    return air_cases.stark_words(w, committed, at_point)


def air_case(name):
    import air_cases

    if name in AIR_SMALL:
        return air_cases.small_cases(oracle)[AIR_SMALL[name]]
    return air_cases.bench_case(oracle, AIR_FULL[name])


def pcs_trees(shape, seed):
    if seed == 0x5EED0001:  # the benchmark's convention: one seed per column index
        return [[m31_column(seed + c, 1 << lg) for c, lg in enumerate(logs)] for logs in shape]
    return [[m31_column(seed + 100 * t + c, 1 << lg) for c, lg in enumerate(logs)] for t, logs in enumerate(shape)]


def gkr_instance(kind, log_n, seed):
    n = 1 << log_n
    if kind == 2 and seed == 0x5EED0002:  # the benchmark's convention
        return kind, m31_column(seed, n), qm31_array(seed + 1, n, nonzero=True)
    den = qm31_array(seed, n, nonzero=True)
    num = qm31_array(seed + 1, n) if kind == 1 else m31_column(seed + 1, n) if kind == 2 else None
    return kind, num, den


def digest(words):
    words = np.ascontiguousarray(words, dtype=np.uint32)
    return {"words": int(words.size), "sha256": hashlib.sha256(words.tobytes()).hexdigest()}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--full", action="store_true")
    ap.add_argument("--only", default="", help="regenerate only the cases whose name starts with this")
    args = ap.parse_args()
    out = json.load(open(OUT)) if os.path.exists(OUT) else {}
    pcs = dict(PCS_SMALL, **(PCS_FULL if args.full else {}))
    gkr = dict(GKR_SMALL, **(GKR_FULL if args.full else {}))
    want = lambda name: name.startswith(args.only)
    for name, (shape, seed, kw) in pcs.items():
        if not want(name):
            continue
        out[name] = digest(oracle.pcs_prove(pcs_trees(shape, seed), **kw))
        print(name, out[name], flush=True)
    for name, (specs, seed) in gkr.items():
        if not want(name):
            continue
        cap = 1 << 22
        out[name] = digest(oracle.gkr_prove([gkr_instance(*s) for s in specs], seed, verify=max(s[1] for s in specs) <= 16, cap=cap))
        print(name, out[name], flush=True)
    import air_cases

    for name in list(AIR_SMALL) + (list(AIR_FULL) if args.full else []):
        if not want(name):
            continue
        out[name] = digest(air_cases.by_air(oracle, air_case(name)))
        print(name, out[name], flush=True)
    for name in list(STARK_SMALL) + (list(STARK_FULL) if args.full else []):
        if not want(name):
            continue
        out[name] = digest(stark_oracle(name))
        print(name, out[name], flush=True)
    json.dump(out, open(OUT, "w"), indent=1, sort_keys=True)


if __name__ == "__main__":
    main()
