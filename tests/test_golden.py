"""Committed proof digests (tests/golden/proof_digests.json, made by tests/golden/make_golden.py from
the CPU oracle): the oracle must still reproduce the small ones on CPU, and the CUDA path must reproduce
all of them, the full-size benchmark workloads included, through the C ABI."""
import hashlib
import importlib.util
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
_spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
mg = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(mg)
GOLDEN = json.load(open(os.path.join(HERE, "golden", "proof_digests.json")))


def _check(name, words):
    words = np.ascontiguousarray(words, dtype=np.uint32)
    assert name in GOLDEN, f"{name} is missing from proof_digests.json: run tests/golden/make_golden.py --full"
    assert int(words.size) == GOLDEN[name]["words"]
    assert hashlib.sha256(words.tobytes()).hexdigest() == GOLDEN[name]["sha256"]


@pytest.mark.parametrize("name", sorted(mg.PCS_SMALL))
def test_oracle_reproduces_pcs_digest(oracle, name):
    shape, seed, kw = mg.PCS_SMALL[name]
    _check(name, oracle.pcs_prove(mg.pcs_trees(shape, seed), **kw))


@pytest.mark.parametrize("name", sorted(mg.GKR_SMALL))
def test_oracle_reproduces_gkr_digest(oracle, name):
    specs, seed = mg.GKR_SMALL[name]
    _check(name, oracle.gkr_prove([mg.gkr_instance(*s) for s in specs], seed))


@pytest.mark.parametrize("name", sorted(mg.AIR_SMALL))
def test_oracle_reproduces_air_digest(oracle, name):
    import air_cases

    case = mg.air_case(name)
    _check(name, air_cases.by_air(oracle, case))
    _check(name, air_cases.by_ssa(oracle, case))


@pytest.mark.parametrize("name", sorted(mg.STARK_SMALL))
def test_oracle_reproduces_stark_digest(oracle, name):
    _check(name, mg.stark_oracle(name))


def test_every_golden_has_a_recipe():
    assert set(GOLDEN) == (set(mg.PCS_SMALL) | set(mg.PCS_FULL) | set(mg.GKR_SMALL) | set(mg.GKR_FULL) | set(mg.AIR_SMALL) | set(mg.AIR_FULL)
                           | set(mg.STARK_SMALL) | set(mg.STARK_FULL))


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(mg.STARK_SMALL) + sorted(mg.STARK_FULL))
def test_cuda_reproduces_stark_digest(ctx, name):
    import air_cases
    from zk_inference_prover_b200 import air

    n_cols, trace_log, kw = dict(mg.STARK_SMALL, **mg.STARK_FULL)[name]
    trace = air_cases.wide_fibonacci_trace(n_cols, trace_log)
    prog = ctx.air_compile(air.wide_fibonacci(air.ExprEvaluator(), n_cols).source()).specialize()
    w, committed, at_point, _ = ctx.stark_prove(prog, [[], [], trace, []], trace_log, host=True, **kw)
    assert (committed == at_point).all()
    _check(name, air_cases.stark_words(w, committed, at_point))


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(mg.AIR_SMALL) + sorted(mg.AIR_FULL))
def test_cuda_reproduces_air_digest(ctx, name):
    case = mg.air_case(name)
    prog = ctx.air_compile(case["source"])
    bufs = [ctx.upload(c) for c in case["cols"]]
    acc = [ctx.alloc(1 << case["eval_log"]) for _ in range(4)]
    for specialized in (False, True):
        if specialized:
            prog.specialize()
        ctx.constraint_quotients(prog, [b.ptr for b in bufs], case["rcp"], case["trace_log"], case["eval_log"], [a.ptr for a in acc],
                                 accumulate=False, cumsum_shift=case["cumsum_shift"])
        _check(name, np.stack([a.download() for a in acc]))


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(mg.PCS_SMALL) + sorted(mg.PCS_FULL))
def test_cuda_reproduces_pcs_digest(ctx, name):
    shape, seed, kw = dict(mg.PCS_SMALL, **mg.PCS_FULL)[name]
    _check(name, ctx.pcs_prove_host(mg.pcs_trees(shape, seed), **kw))


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(mg.GKR_SMALL) + sorted(mg.GKR_FULL))
def test_cuda_reproduces_gkr_digest(ctx, name):
    specs, seed = dict(mg.GKR_SMALL, **mg.GKR_FULL)[name]
    inst = []
    keep = []
    for s in specs:
        kind, num, den = mg.gkr_instance(*s)
        nb = ctx.upload(num) if num is not None else None
        db = ctx.upload(den)
        keep += [nb, db]
        inst.append((kind, nb.ptr if nb else 0, db.ptr, den.shape[0]))
    _check(name, ctx.gkr_prove_device(inst, seed))
