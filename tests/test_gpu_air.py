"""Constraint quotients of an AIR on the GPU (zkb_air_compile + zkb_constraint_quotients through the C ABI) against the
CPU oracle: the reference's AIRs written against CpuDomainEvaluator and the interpreter of the lowered program; random
programs; the reference's own wide-Fibonacci CUDA kernel; and, at full size, the property that a valid trace's quotient
is a polynomial."""
import numpy as np
import pytest

import air_cases
from util import P, m31_column, qm31_array

pytestmark = pytest.mark.gpu


def run_gpu(ctx, case, accum=None, prog=None):
    """Both device paths - the interpreter, then the kernel specialised with NVRTC - which must agree word for word."""
    prog = prog or ctx.air_compile(case["source"])
    n = 1 << case["eval_log"]
    bufs = [ctx.upload(c) for c in case["cols"]]
    out = []
    for specialized in (False, True):
        if specialized:
            prog.specialize()
            assert prog.stats["specialized"] == 1
        acc = [ctx.upload(accum[k]) if accum is not None else ctx.alloc(n) for k in range(4)]
        ctx.constraint_quotients(prog, [b.ptr for b in bufs], case["rcp"], case["trace_log"], case["eval_log"], [a.ptr for a in acc],
                                 accumulate=accum is not None, cumsum_shift=case["cumsum_shift"])
        out.append(np.stack([a.download() for a in acc]))
    prog.select(False)
    assert (out[0] == out[1]).all(), "the specialised kernel and the interpreter disagree"
    return out[0]


def test_reference_airs_match_oracle(ctx, oracle):
    for case in air_cases.small_cases(oracle):
        want = air_cases.by_air(oracle, case)
        got = run_gpu(ctx, case)
        assert (got == want).all(), case["name"]
        acc0 = qm31_array(19, 1 << case["eval_log"]).T.copy()
        assert (run_gpu(ctx, case, accum=acc0) == air_cases.by_air(oracle, case, accum=acc0)).all(), case["name"]


@pytest.mark.parametrize("make", [
    lambda o: air_cases.wide_fibonacci_case(o, 64, 12, 13, 1000),
    lambda o: air_cases.wide_fibonacci_case(o, 300, 9, 11, 1100),     # more live loads than one batch, long program
    lambda o: air_cases.plonk_case(o, 13, 14, 1200),
    lambda o: air_cases.freivalds_case(o, 16, 8, 3, 11, 12, 1300),
    lambda o: air_cases.freivalds_case(o, 48, 12, 3, 10, 11, 1400),   # a register file that needs a smaller CTA
    lambda o: air_cases.freivalds_case(o, 6, 7, 2, 12, 16, 1500, range_check=True),  # blow-up 16: 16 denominators
])
def test_larger_cases_match_oracle(ctx, oracle, make):
    case = make(oracle)
    prog = ctx.air_compile(case["source"])
    st = prog.stats
    assert st["smem_bytes"] <= 227 * 1024 and st["threads"] in (32, 64, 128, 256)
    got = run_gpu(ctx, case, prog=prog)
    assert (got == air_cases.by_ssa(oracle, case)).all(), (case["name"], st)
    assert (got == air_cases.by_air(oracle, case)).all(), (case["name"], st)


@pytest.mark.parametrize("seed,n_ops,eval_log", [(1, 60, 7), (2, 400, 9), (3, 2000, 10), (4, 5000, 8), (5, 300, 13)])
def test_random_programs_match_oracle(ctx, oracle, seed, n_ops, eval_log):
    tree_cols = [3, 0, 6, 4]
    src = air_cases.random_program(seed, n_ops, tree_cols, 5, 41, max_offset=3)
    trace_log = eval_log - 1 - seed % 2
    cols = [m31_column(70 + seed * 100 + c, 1 << eval_log) for c in range(sum(tree_cols))]
    rcp, shift = qm31_array(seed + 40, 41), qm31_array(seed + 41, 1)[0]
    want = oracle.constraint_quotients_ssa(src, cols, rcp, trace_log, eval_log, cumsum_shift=shift)
    prog = ctx.air_compile(src)
    bufs = [ctx.upload(c) for c in cols]
    acc = [ctx.alloc(1 << eval_log) for _ in range(4)]
    ctx.constraint_quotients(prog, [b.ptr for b in bufs], rcp, trace_log, eval_log, [a.ptr for a in acc], accumulate=False, cumsum_shift=shift)
    got = np.stack([a.download() for a in acc])
    assert (got == want).all(), prog.stats
    # the same program serves other scalars (the run-time blob) without recompiling
    sc2 = qm31_array(seed + 42, 5)
    want2 = oracle.constraint_quotients_ssa(src, cols, rcp, trace_log, eval_log, cumsum_shift=shift, scalars=sc2)
    ctx.constraint_quotients(prog, [b.ptr for b in bufs], rcp, trace_log, eval_log, [a.ptr for a in acc], accumulate=False, cumsum_shift=shift,
                             scalars=sc2)
    assert (np.stack([a.download() for a in acc]) == want2).all()
    # and the kernel specialised to the program gives the same words, for both sets of scalars
    prog.specialize()
    for sc, w in ((None, want), (sc2, want2)):
        ctx.constraint_quotients(prog, [b.ptr for b in bufs], rcp, trace_log, eval_log, [a.ptr for a in acc], accumulate=False, cumsum_shift=shift,
                                 scalars=sc)
        assert (np.stack([a.download() for a in acc]) == w).all()


def test_compile_rejects_bad_programs(ctx, zkb):
    from zk_inference_prover_b200 import air

    def src(ops, cons=(0,), trees=(1, 0, 1, 0), n_scalars=1):
        return air.AirSource(np.array(ops, np.uint32).reshape(-1, 5), np.array(cons, np.uint32), np.array(trees, np.uint32),
                             np.zeros((n_scalars, 4), np.uint32))

    good = [(air.LOAD, 2, 0, 0, 0), (air.SCALAR, 0, 0, 0, 0), (air.MUL_E, 0, 1, 0, 0)]
    ctx.air_compile(src(good, cons=(2,)))
    for bad, cons in [
        ([(air.LOAD, 2, 1, 0, 0)], (0,)),                                        # column outside the tree
        ([(air.LOAD, 1, 0, 0, 0)], (0,)),                                        # empty tree
        ([(air.LOAD, 2, 0, 0, 0), (air.ADD_B, 0, 1, 0, 0)], (1,)),               # operand is not an earlier instruction
        (good + [(air.ADD_B, 0, 2, 0, 0)], (3,)),                                # secure operand of a base instruction
        ([(air.CONST_M31, P, 0, 0, 0)], (0,)),                                   # not canonical
        ([(air.SCALAR, 1, 0, 0, 0)], (0,)),                                      # scalar slot out of range
        ([(air.LOAD, 2, 0, 5000, 0)], (0,)),                                     # offset out of range
        ([(99, 0, 0, 0, 0)], (0,)),                                              # unknown opcode
        (good, (7,)),                                                            # constraint is not an instruction
    ]:
        with pytest.raises(zkb.ZkbError) as e:
            ctx.air_compile(src(bad, cons=cons))
        assert e.value.code == -1, bad
    prog = ctx.air_compile(src(good, cons=(2,)))
    col, acc = ctx.alloc(16), [ctx.alloc(16) for _ in range(4)]
    with pytest.raises(zkb.ZkbError):  # the evaluation domain must be larger than the trace domain
        ctx.constraint_quotients(prog, [col.ptr, col.ptr], np.zeros(4, np.uint32), 4, 4, [a.ptr for a in acc], denom_inv=np.ones(1, np.uint32))


def test_too_many_live_values_is_an_error_not_a_fault(ctx, zkb):
    """A program whose live values cannot fit one CTA's shared memory is refused at compile time."""
    from zk_inference_prover_b200 import air

    ev = air.ExprEvaluator()
    vals = [ev.scalar([1, 2, 3, 4]) * ev.next_trace_mask() for _ in range(2000)]   # 2000 secure values alive at once
    acc = vals[0]
    for v in vals[1:]:
        acc = acc + v
    for v in vals:
        acc = acc * v
    ev.add_constraint(acc)
    with pytest.raises(zkb.ZkbError) as e:
        ctx.air_compile(ev.source())
    assert "shared memory" in str(e.value)


@pytest.mark.parametrize("n_cols,trace_log,eval_log", [(3, 4, 5), (16, 10, 11), (100, 12, 13), (32, 14, 16)])
def test_wide_fibonacci_matches_reference_cuda_kernel(ctx, oracle, n_cols, trace_log, eval_log):
    from oracle import ref_cuda

    if not ref_cuda.available():
        pytest.skip("oracle/_ref/libstwo_cuda_ref.so is not built (the reference checkout is needed to build it)")
    ref = ref_cuda.RefCudaAir()
    case = air_cases.wide_fibonacci_case(oracle, n_cols, trace_log, eval_log, 2000 + n_cols)
    denom = oracle.constraint_denom_inv(trace_log, eval_log)
    r_cols = [ref.upload(c) for c in case["cols"]]
    r_out = ref.wide_fibonacci_quotients(r_cols, case["rcp"], denom, trace_log, eval_log)
    want = np.stack([ref.download(p, 1 << eval_log) for p in r_out])
    for p in r_cols + r_out:
        ref.free(p)
    assert (run_gpu(ctx, case) == want).all()
    if eval_log <= 13:
        assert (air_cases.by_air(oracle, case) == want).all()


def test_full_size_wide_fibonacci_quotient_is_a_polynomial(ctx, oracle):
    """2^20 rows x 64 columns, blow-up 2: the quotient of a valid trace has no coefficient above index 2^20, and one
    corrupted trace cell gives it some."""
    trace_log, eval_log, n_cols = 20, 21, 64
    n, N = 1 << trace_log, 1 << eval_log
    a, b = m31_column(1, n).astype(np.uint64), m31_column(2, n).astype(np.uint64)
    trace = [a, b]
    for _ in range(2, n_cols):
        a, b = b, (a * a % P + b * b % P) % P
        trace.append(b)
    case = air_cases.wide_fibonacci_case(oracle, n_cols, 4, 5, 7)
    prog = ctx.air_compile(case["source"])
    rcp = qm31_array(77, n_cols - 2)
    for corrupt in (False, True):
        if corrupt:
            prog.specialize()   # the second pass runs the specialised kernel
        cols = [ctx.upload(c.astype(np.uint32)) for c in trace]
        if corrupt:
            bad = trace[9].astype(np.uint32)
            bad[12345] ^= 1
            cols[9].upload(bad)
        ctx.ifft_cols([c.ptr for c in cols], trace_log)
        ext = [ctx.alloc(N) for _ in range(n_cols)]
        ctx.lde_cols([c.ptr for c in cols], trace_log, [e.ptr for e in ext], eval_log)
        acc = [ctx.alloc(N) for _ in range(4)]
        ctx.constraint_quotients(prog, [e.ptr for e in ext], rcp, trace_log, eval_log, [x.ptr for x in acc], accumulate=False)
        ctx.ifft_cols([x.ptr for x in acc], eval_log)
        coeffs = np.stack([x.download() for x in acc])
        assert coeffs[:, :n].any()
        assert coeffs[:, n + 1:].any() == corrupt
        del cols, ext, acc


def test_freivalds_witness_satisfies_its_air(ctx, oracle):
    """The columns zkb_freivalds_scatter / zkb_freivalds_acc produce, extended to the evaluation domain, satisfy the
    component's constraints (prover/src/gadgets/freivalds/mod.rs:114-163): the quotient is a polynomial. This ties the
    witness kernels, the mask offsets (rows j-1 in coset order) and the constraint evaluator together. The constraint
    acc - acc_prev * notzero - (u * v) * last has degree 3, so its quotient has up to twice the trace size of
    coefficients; on an evaluation domain of four times the trace the upper half must vanish."""
    from test_freivalds import _case, layout
    from zk_inference_prover_b200 import air

    tokens, n_in, n_outs, chunks = 32, 64, [64, 48, 64], 16
    qx, qws = _case(31, tokens, n_in, n_outs)
    grid, pq, pk = layout(n_in, max(n_outs), tokens, chunks)
    trace_log, n_mats = grid[0], len(qws)
    eval_log, rows = trace_log + 2, 1 << trace_log
    d_qx, d_qw = ctx.upload_bytes(qx), [ctx.upload_bytes(w) for w in qws]
    base, pre = [ctx.alloc(rows) for _ in range(pq)], [ctx.alloc(rows) for _ in range(n_mats * pk + 4)]
    m_r8, off = ctx.alloc(256).zero(), ctx.alloc(2).zero()
    ctx.freivalds_scatter(d_qx.ptr, [w.ptr for w in d_qw], n_outs, grid, pq, pk, n_in, tokens, [b.ptr for b in base], [p.ptr for p in pre],
                          m_r8.ptr, 256, off.ptr)
    fp = air_cases.freivalds_params(oracle, pk, pq, n_mats, 3100)
    inter = [ctx.alloc(rows) for _ in range((1 + 2 * n_mats) * 4)]
    claims = ctx.freivalds_acc([b.ptr for b in base], [p.ptr for p in pre[:n_mats * pk]], grid, pq, pk, n_mats, fp["s"], fp["rv"],
                               [o.ptr for o in inter])
    # the AIR's column order: preprocessed = 4 selectors then the weights; trace = activations; interaction = v, (u_m, acc_m)
    trace_cols = pre[n_mats * pk:] + pre[:n_mats * pk] + base + inter
    src = air.freivalds(air.ExprEvaluator(), pk, pq, n_mats, fp["rv_pow"], fp["rv_step"], fp["s_pow"], fp["s_step"], claims, 128, None).source()
    assert int(sum(src.tree_cols)) == len(trace_cols)
    prog = ctx.air_compile(src)
    rcp = qm31_array(3200, src.n_constraints)
    for corrupt in (False, True):
        work = [ctx.alloc(rows) for _ in trace_cols]
        for w, c in zip(work, trace_cols):
            ctx.d2d(w.ptr, c.ptr, rows * 4)
        if corrupt:
            v = work[4 + n_mats * pk + pq].download()   # first coordinate of v
            v[77] = (int(v[77]) + 1) % P
            work[4 + n_mats * pk + pq].upload(v)
        ctx.ifft_cols([w.ptr for w in work], trace_log)
        ext = [ctx.alloc(4 * rows) for _ in work]
        ctx.lde_cols([w.ptr for w in work], trace_log, [e.ptr for e in ext], eval_log)
        acc = [ctx.alloc(4 * rows) for _ in range(4)]
        ctx.constraint_quotients(prog, [e.ptr for e in ext], rcp, trace_log, eval_log, [x.ptr for x in acc], accumulate=False)
        ctx.ifft_cols([x.ptr for x in acc], eval_log)
        coeffs = np.stack([x.download() for x in acc])
        assert coeffs[:, :rows].any()
        assert coeffs[:, 2 * rows + 1:].any() == corrupt


# ---------------------------------------------------------------------------------------------- whole proofs of one component

_wide_fibonacci_trace = air_cases.wide_fibonacci_trace


@pytest.mark.parametrize("n_cols,trace_log,log_blowup,specialize", [(10, 6, 1, False), (10, 6, 2, True), (40, 10, 1, True), (24, 12, 2, False)])
def test_stark_proof_of_wide_fibonacci_matches_oracle(ctx, oracle, n_cols, trace_log, log_blowup, specialize):
    """prove() end to end: every word of the proof (5 trees: the composition tree among them), the channel state after it, and
    the prover's sanity check equal the oracle's; a corrupted trace fails the check on both sides with the same values."""
    from zk_inference_prover_b200 import air

    trace = _wide_fibonacci_trace(n_cols, trace_log)
    prog = ctx.air_compile(air.wide_fibonacci(air.ExprEvaluator(), n_cols).source())
    if specialize:
        prog.specialize()
    kw = dict(pow_bits=5, log_blowup=log_blowup, n_queries=7)
    for corrupt in (False, True):
        if corrupt:
            trace[3] = trace[3].copy()
            trace[3][5] ^= 1
        want, w_committed, w_point = oracle.stark_prove(0, [n_cols], np.zeros(4, np.uint32), [0, 0, n_cols, 0], trace, trace_log, trace_log + 1, **kw)
        bufs = [ctx.upload(c) for c in trace]
        got, committed, at_point, _ = ctx.stark_prove(prog, [[], [], [b.ptr for b in bufs], []], trace_log, **kw)
        assert (committed == w_committed).all() and (at_point == w_point).all()
        assert (committed == at_point).all() != corrupt
        assert len(got) == len(want) and (got == want).all()
        got_h, c_h, p_h, _ = ctx.stark_prove(prog, [[], [], trace, []], trace_log, host=True, **kw)
        assert (got_h == want).all() and (c_h == w_committed).all() and (p_h == w_point).all()


def test_stark_proof_of_the_freivalds_component_matches_oracle(ctx, oracle):
    """The Freivalds component proved end to end from the witness the device kernels make: preprocessed selectors and
    weights, activations, and the Horner / accumulator columns as the interaction tree, masks at offsets -1 and 0."""
    from test_freivalds import _case, layout
    from zk_inference_prover_b200 import air

    tokens, n_in, n_outs, chunks = 9, 8, [8, 6], 4
    qx, qws = _case(41, tokens, n_in, n_outs)
    grid, pq, pk = layout(n_in, max(n_outs), tokens, chunks)
    trace_log, n_mats = grid[0], len(qws)
    base, pre, _, _ = oracle.freivalds_columns(qx, qws, grid, pq, pk)
    fp = air_cases.freivalds_params(oracle, pk, pq, n_mats, 4100)
    inter, claims = oracle.freivalds_acc(base, pre, n_mats, grid, pq, pk, fp["s"], fp["rv"])
    trees = [list(pre[n_mats * pk:]) + list(pre[:n_mats * pk]), [], list(base), list(inter)]
    rel = qm31_array(5, 2)
    qp = np.concatenate([fp["rv_pow"], fp["rv_step"][None], fp["s_pow"], fp["s_step"][None], claims, rel]).astype(np.uint32)
    src = air.freivalds(air.ExprEvaluator(), pk, pq, n_mats, fp["rv_pow"], fp["rv_step"], fp["s_pow"], fp["s_step"], claims, 128, None).source()
    assert [len(t) for t in trees] == list(src.tree_cols)
    prog = ctx.air_compile(src).specialize()
    kw = dict(pow_bits=3, log_blowup=2, n_queries=5)
    flat = [c for t in trees for c in t]
    want, w_committed, w_point = oracle.stark_prove(2, [pk, pq, n_mats, 128, 0], qp, list(src.tree_cols), flat, trace_log, trace_log + 1, **kw)
    assert (w_committed == w_point).all()
    bufs = [[ctx.upload(c) for c in t] for t in trees]
    got, committed, at_point, _ = ctx.stark_prove(prog, [[b.ptr for b in t] for t in bufs], trace_log, **kw)
    assert (committed == w_committed).all() and (at_point == w_point).all()
    assert len(got) == len(want) and (got == want).all()


def test_full_size_stark_proof_passes_its_own_check(ctx):
    """256 columns x 2^20 rows, blow-up 4 (the benchmark's trace shape) proved as a wide Fibonacci component: the composition
    polynomial's out-of-domain value from the committed halves equals the value from the constraints at the sampled masks."""
    from zk_inference_prover_b200 import air

    n_cols, trace_log = 256, 20
    trace = _wide_fibonacci_trace(n_cols, trace_log)
    prog = ctx.air_compile(air.wide_fibonacci(air.ExprEvaluator(), n_cols).source()).specialize()
    bufs = [ctx.upload(c) for c in trace]
    _, committed, at_point, _ = ctx.stark_prove(prog, [[], [], [b.ptr for b in bufs], []], trace_log, pow_bits=10, log_blowup=2, n_queries=3,
                                                cap=1 << 26)
    assert (committed == at_point).all() and committed.any()


def test_without_nvrtc_the_interpreter_still_serves(oracle):
    """When NVRTC cannot be loaded, zkb_air_specialize reports it and the program keeps working through the interpreter.
    (NVRTC is looked up once per process, so this runs in a child process with ZKB_NVRTC_LIB pointing nowhere.)"""
    import os
    import subprocess
    import sys

    code = r'''
import sys, numpy as np
sys.path.insert(0, "tests"); sys.path.insert(0, ".")
import oracle, air_cases
import zk_inference_prover_b200 as z
ctx = z.Context(device=0, max_log_size=10)
case = air_cases.wide_fibonacci_case(oracle, 8, 5, 6, 100)
prog = ctx.air_compile(case["source"])
try:
    prog.specialize()
    print("UNEXPECTED: specialised")
except z.ZkbError as e:
    assert "NVRTC" in str(e), str(e)
bufs = [ctx.upload(c) for c in case["cols"]]
acc = [ctx.alloc(64) for _ in range(4)]
ctx.constraint_quotients(prog, [b.ptr for b in bufs], case["rcp"], 5, 6, [a.ptr for a in acc], accumulate=False)
assert (np.stack([a.download() for a in acc]) == air_cases.by_air(oracle, case)).all()
print("OK")
'''
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, ZKB_NVRTC_LIB="/nonexistent/libnvrtc.so")
    r = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip().endswith("OK"), r.stdout + r.stderr


@pytest.mark.parametrize("log_blowup,logs,specialize", [(1, (6, 8), False), (2, (6, 8), True), (1, (9, 7, 9), True)])
def test_stark_proof_of_several_components_matches_oracle(ctx, oracle, log_blowup, logs, specialize):
    """A statement of wide Fibonacci components of different sizes and the Freivalds component: sub-accumulations per size,
    lifted and added; mask points in steps of the largest trace; one out-of-domain check through all components."""
    comps, sources, flat, tree_cols, per_comp = air_cases.mixed_components_case(oracle, logs=logs)
    kw = dict(pow_bits=3, log_blowup=log_blowup, n_queries=5)
    want, w_committed, w_point = oracle.stark_prove_multi(comps, tree_cols, flat, **kw)
    assert (w_committed == w_point).all()
    progs = [ctx.air_compile(s) for s in sources]
    if specialize:
        for p in progs:
            p.specialize()
    trees = [[c for pc in per_comp for c in pc[t]] for t in range(4)]
    bufs = [[ctx.upload(c) for c in t] for t in trees]
    components = [(p, c["trace_log"], None) for p, c in zip(progs, comps)]
    got, committed, at_point, _ = ctx.stark_prove_multi(components, [[b.ptr for b in t] for t in bufs], **kw)
    assert (committed == w_committed).all() and (at_point == w_point).all()
    assert len(got) == len(want) and (got == want).all()
    got_h, c_h, p_h, _ = ctx.stark_prove_multi(components, trees, host=True, **kw)
    assert (got_h == want).all() and (c_h == w_committed).all() and (p_h == w_point).all()
    # a corrupted cell of the middle component fails the check, with the oracle's values
    flat2 = [c.copy() for c in flat]
    flat2[12][3] ^= 1
    want2, w_c2, w_p2 = oracle.stark_prove_multi(comps, tree_cols, flat2, **kw)
    trees2, at = [], 0
    for t in trees:
        trees2.append(flat2[at:at + len(t)])
        at += len(t)
    got2, c2, p2, _ = ctx.stark_prove_multi(components, trees2, host=True, **kw)
    assert not (w_c2 == w_p2).all() and (c2 == w_c2).all() and (p2 == w_p2).all() and (got2 == want2).all()
