"""Constraint quotients of an AIR on the CPU: the oracle against the reference's known answers, and the two routes
through the oracle (AIRs written against CpuDomainEvaluator; the lowered single-assignment program) against each other."""
import numpy as np
import pytest

import air_cases
from util import P, m31_column, qm31_array


def test_previous_index_known_answer(oracle):
    """nitroo/crates/stwo/src/core/utils.rs:238-290: neighbours on the circle domain of log size 4."""
    log_size, n = 4, 16
    natural = np.arange(n)
    bit_reversed = oracle.bit_reverse(natural.astype(np.uint32))
    pairs = sorted((int(bit_reversed[i]), int(bit_reversed[oracle.offset_bit_reversed_circle_domain_index(i, log_size - 3, log_size, -1)]))
                   for i in range(n))
    expected = sorted([(0, 4), (15, 11), (1, 5), (14, 10), (2, 6), (13, 9), (3, 7), (12, 8), (4, 0), (11, 15), (5, 1), (10, 14), (6, 2),
                       (9, 13), (7, 3), (8, 12)])
    assert pairs == expected


def test_offset_composes(oracle):
    """core/utils.rs:214-236: offset -2 is two steps of -1."""
    f = oracle.offset_bit_reversed_circle_domain_index
    for i in range(64):
        assert f(i, 3, 6, -2) == f(f(i, 3, 6, -1), 3, 6, -1)
        assert f(f(i, 3, 6, 5), 3, 6, -5) == i


@pytest.mark.parametrize("trace_log,eval_log", [(3, 4), (4, 6), (5, 8), (1, 3), (2, 3)])
def test_denominator_inverses(oracle, zkb, trace_log, eval_log):
    """denom_inv[row >> trace_log] inverts the trace domain's vanishing polynomial at every row of the evaluation domain
    (core/constraints.rs:147-165 checks the same polynomial vanishes on its coset and nowhere else on the others)."""
    d = oracle.constraint_denom_inv(trace_log, eval_log)
    assert (d == zkb.capi.constraint_denom_inv(trace_log, eval_log)).all()
    n = 1 << eval_log
    rows = oracle.bit_reverse(np.arange(n, dtype=np.uint32))  # rows[r] = natural index of bit-reversed row r
    for r in range(n):
        x = int(oracle.domain_at(eval_log, int(rows[r]))[0])
        for _ in range(1, trace_log):
            x = (2 * x * x - 1) % P
        assert x != 0 and oracle.m31_mul(x, int(d[r >> trace_log])) == 1
    # and the same polynomial is zero on the trace domain itself
    for i in range(1 << trace_log):
        x = int(oracle.domain_at(trace_log, i)[0])
        for _ in range(1, trace_log):
            x = (2 * x * x - 1) % P
        assert x == 0


def test_lowered_program_equals_hand_written_air(oracle):
    for case in air_cases.small_cases(oracle):
        a, b = air_cases.by_air(oracle, case), air_cases.by_ssa(oracle, case)
        assert (a == b).all(), case["name"]
        assert a.any()
        acc0 = qm31_array(9, 1 << case["eval_log"]).T.copy()
        assert (air_cases.by_air(oracle, case, accum=acc0) == air_cases.by_ssa(oracle, case, accum=acc0)).all()
        # accumulation is addition of the overwrite result
        assert (air_cases.by_ssa(oracle, case, accum=acc0) == ((acc0.astype(np.uint64) + b) % P).astype(np.uint32)).all()


def test_wide_fibonacci_quotient_of_a_valid_trace_is_a_polynomial(oracle):
    """A trace that satisfies the constraints on the trace domain gives a quotient that is a polynomial of the trace's
    degree: its coefficients on the evaluation domain vanish above index 2^trace_log (the basis function at that index
    is the trace domain's own vanishing polynomial, which a degree-2 constraint can leave a multiple of)."""
    trace_log, eval_log, n_cols = 6, 7, 12
    n = 1 << trace_log
    a, b = m31_column(1, n).astype(object), m31_column(2, n).astype(object)
    trace = [a, b]
    for _ in range(2, n_cols):
        a, b = b, (a * a + b * b) % P
        trace.append(b)
    trace = [np.array(c, dtype=np.uint32) for c in trace]
    coeffs = oracle.interpolate_cols(trace, trace_log)
    cols = oracle.evaluate_cols(coeffs, trace_log, eval_log)
    case = air_cases.wide_fibonacci_case(oracle, n_cols, trace_log, eval_log, 5)
    case["cols"] = list(cols)
    q = air_cases.by_air(oracle, case)
    assert (q == air_cases.by_ssa(oracle, case)).all()
    qc = np.stack(oracle.interpolate_cols(list(q), eval_log))
    assert qc[:, :n].any() and not qc[:, n + 1:].any()
    # a single corrupted cell breaks it
    trace[5][3] ^= 1
    cols = oracle.evaluate_cols(oracle.interpolate_cols(trace, trace_log), trace_log, eval_log)
    case["cols"] = list(cols)
    qc = np.stack(oracle.interpolate_cols(list(air_cases.by_air(oracle, case)), eval_log))
    assert qc[:, n + 1:].any()


def test_random_programs_interpret(oracle):
    """The fuzz generator used on the GPU produces programs the oracle accepts (all opcodes, offsets, dead code)."""
    src = air_cases.random_program(3, 200, [3, 0, 5, 4], 6, 9)
    cols = [m31_column(50 + c, 1 << 6) for c in range(12)]
    out = oracle.constraint_quotients_ssa(src, cols, qm31_array(4, 9), 4, 6, cumsum_shift=[1, 2, 3, 4])
    assert out.any()


def test_whole_proof_passes_the_provers_own_check(oracle):
    """prove() end to end in the oracle (oracle/stark.hpp): for a valid trace the composition polynomial's out-of-domain
    value from the committed halves equals the value from the constraints at the sampled mask values
    (nitroo/crates/stwo/src/prover/mod.rs:141-166); one corrupted cell breaks the equality."""
    n_cols, trace_log = 12, 6
    trace = air_cases.wide_fibonacci_trace(n_cols, trace_log)
    args = (0, [n_cols], np.zeros(4, np.uint32), [0, 0, n_cols, 0])
    for log_blowup in (1, 2):
        w, committed, at_point = oracle.stark_prove(*args, trace, trace_log, trace_log + 1, log_blowup=log_blowup, pow_bits=4, n_queries=5)
        assert (committed == at_point).all() and committed.any() and len(w) > 500
    bad = [c.copy() for c in trace]
    bad[7][9] ^= 1
    _, committed, at_point = oracle.stark_prove(*args, bad, trace_log, trace_log + 1, pow_bits=4, n_queries=5)
    assert not (committed == at_point).all()


def test_whole_proof_of_the_freivalds_component(oracle):
    """The Freivalds witness (masks at offsets -1 and 0 in the interaction tree, four preprocessed selectors) passes the check."""
    from test_freivalds import _case, layout

    tokens, n_in, n_outs, chunks = 5, 6, [7, 5], 4
    qx, qws = _case(31, tokens, n_in, n_outs)
    grid, pq, pk = layout(n_in, max(n_outs), tokens, chunks)
    trace_log, n_mats = grid[0], len(qws)
    base, pre, _, _ = oracle.freivalds_columns(qx, qws, grid, pq, pk)
    fp = air_cases.freivalds_params(oracle, pk, pq, n_mats, 3100)
    inter, claims = oracle.freivalds_acc(base, pre, n_mats, grid, pq, pk, fp["s"], fp["rv"])
    cols = list(pre[n_mats * pk:]) + list(pre[:n_mats * pk]) + list(base) + list(inter)
    qp = np.concatenate([fp["rv_pow"], fp["rv_step"][None], fp["s_pow"], fp["s_step"][None], claims, qm31_array(5, 2)]).astype(np.uint32)
    tree_cols = [4 + n_mats * pk, 0, pq, 4 * (1 + 2 * n_mats)]
    _, committed, at_point = oracle.stark_prove(2, [pk, pq, n_mats, 128, 0], qp, tree_cols, cols, trace_log, trace_log + 1, log_blowup=2)
    assert (committed == at_point).all()
    cols[-3] = cols[-3].copy()
    cols[-3][3] ^= 1
    _, committed, at_point = oracle.stark_prove(2, [pk, pq, n_mats, 128, 0], qp, tree_cols, cols, trace_log, trace_log + 1, log_blowup=2)
    assert not (committed == at_point).all()


# ---------------------------------------------------------------------------------------------- the product's compiler, on the host

def test_compiler_report_for_the_reference_airs(oracle, zkb):
    """zkb_air_analyze (host only): what the lowering to bytecode makes of the three AIRs."""
    from zk_inference_prover_b200 import air

    wf = zkb.air_analyze(air.wide_fibonacci(air.ExprEvaluator(), 100).source())
    assert wf["n_loads"] == 100 and wf["n_columns_read"] == 100 and wf["n_uniform"] == 0
    assert wf["m31_mults"] == 98 * 6          # two squares and a coefficient of four words per constraint
    assert wf["reg_words"] <= 16 and wf["rows_per_thread"] == 4 and wf["threads"] == 256
    assert wf["n_instr"] < wf["n_live_ops"]   # multiplications folded, constraints accumulated where they are computed
    case = air_cases.freivalds_case(oracle, 16, 1, 2, 5, 6, 1)
    fr = zkb.air_analyze(case["source"])
    assert fr["n_columns_read"] == int(sum(case["tree_cols"])) and fr["n_loads"] > fr["n_columns_read"]   # masks at -1 and 0
    assert fr["n_uniform"] > 0 and fr["smem_bytes"] <= 227 * 1024
    pl = zkb.air_analyze(air_cases.plonk_case(oracle, 5, 6, 2)["source"])
    assert pl["n_columns_read"] == 16 and pl["n_loads"] == 20


def test_compiler_rejects_bad_programs_on_the_host(zkb):
    from zk_inference_prover_b200 import air

    def src(ops, cons=(0,), trees=(1, 0, 1, 0), n_scalars=1):
        return air.AirSource(np.array(ops, np.uint32).reshape(-1, 5), np.array(cons, np.uint32), np.array(trees, np.uint32),
                             np.zeros((n_scalars, 4), np.uint32))

    good = [(air.LOAD, 2, 0, 0, 0), (air.SCALAR, 0, 0, 0, 0), (air.MUL_E, 0, 1, 0, 0)]
    assert zkb.air_analyze(src(good, cons=(2,)))["n_instr"] >= 2
    for bad, cons, needle in [
        ([(air.LOAD, 2, 1, 0, 0)], (0,), "outside the trees"),
        ([(air.LOAD, 2, 0, 0, 0), (air.ADD_B, 0, 1, 0, 0)], (1,), "not an earlier instruction"),
        (good + [(air.ADD_B, 0, 2, 0, 0)], (3,), "secure-field operand"),
        ([(air.CONST_M31, P, 0, 0, 0)], (0,), "canonical"),
        ([(air.SCALAR, 1, 0, 0, 0)], (0,), "scalar slot"),
        ([(air.LOAD, 2, 0, 5000, 0)], (0,), "offset"),
        ([(99, 0, 0, 0, 0)], (0,), "opcode"),
        (good, (7,), "constraint 0"),
    ]:
        with pytest.raises(zkb.ZkbError) as e:
            zkb.air_analyze(src(bad, cons=cons))
        assert e.value.code == -1 and needle in str(e.value), (bad, str(e.value))
    ev = air.ExprEvaluator()
    vals = [ev.scalar([1, 2, 3, 4]) * ev.next_trace_mask() for _ in range(2000)]
    acc = vals[0]
    for v in vals[1:]:
        acc = acc + v
    for v in vals:
        acc = acc * v
    ev.add_constraint(acc)
    with pytest.raises(zkb.ZkbError) as e:
        zkb.air_analyze(ev.source())
    assert "shared memory" in str(e.value)


def test_specialised_kernel_source_compiles_without_a_gpu(oracle, zkb):
    """The code generator's output goes through NVRTC for sm_100a on the host (no device is needed to compile)."""
    case = air_cases.freivalds_case(oracle, 8, 3, 2, 5, 6, 1)
    try:
        st = zkb.air_analyze(case["source"], check_specialized=True)
    except zkb.ZkbError as e:
        if "could not be loaded" in str(e):
            pytest.skip("NVRTC is not installed here")
        raise
    assert st["specialized"] == 1 and 16 <= st["specialized_regs"] <= 255


def test_whole_proof_of_several_components_of_different_sizes(oracle):
    """Three components on traces of 2^6, 2^8 and 2^5 rows: per-size accumulations lifted and added, mask points in steps of
    the largest trace, one out-of-domain check running through all of them."""
    comps, _, flat, tree_cols, _ = air_cases.mixed_components_case(oracle)
    for log_blowup in (1, 2):
        _, committed, at_point = oracle.stark_prove_multi(comps, tree_cols, flat, pow_bits=3, log_blowup=log_blowup, n_queries=5)
        assert (committed == at_point).all() and committed.any()
    flat[12] = flat[12].copy()
    flat[12][3] ^= 1
    _, committed, at_point = oracle.stark_prove_multi(comps, tree_cols, flat, pow_bits=3, log_blowup=1, n_queries=5)
    assert not (committed == at_point).all()
