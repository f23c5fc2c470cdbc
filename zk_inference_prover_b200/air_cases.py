"""Seeded AIR cases shared by the CPU tests, the GPU tests and the golden-vector generator.

A case holds the lowered program (built with the package's ExprEvaluator), the parameters of the same AIR for the
oracle's hand-written evaluator, the columns on the evaluation domain and the random-coefficient powers."""
import numpy as np

from zk_inference_prover_b200.synth import P, m31_column, qm31_array
from zk_inference_prover_b200 import air


def _shift(oracle, claimed_sum, trace_log):
    """LogupAtRow::new (constraint-framework/src/logup.rs:33-41): claimed_sum / 2^log_size."""
    return oracle.qm31_mul(claimed_sum, oracle.qm31_inv([1 << trace_log, 0, 0, 0]))


def _random_cols(seed, n_cols, eval_log):
    return [m31_column(seed + 7 * c, 1 << eval_log) for c in range(n_cols)]


def wide_fibonacci_case(oracle, n_cols, trace_log, eval_log, seed):
    src = air.wide_fibonacci(air.ExprEvaluator(), n_cols).source()
    return dict(name=f"wide_fibonacci_{n_cols}", source=src, air=0, ip=[n_cols], qp=np.zeros((1, 4), np.uint32), tree_cols=[0, 0, n_cols, 0],
                cols=_random_cols(seed, n_cols, eval_log), rcp=qm31_array(seed + 1, src.n_constraints), trace_log=trace_log,
                eval_log=eval_log, claimed_sum=None, cumsum_shift=None)


def plonk_case(oracle, trace_log, eval_log, seed):
    z, alphas = qm31_array(seed + 2, 1)[0], qm31_array(seed + 3, 2)
    src = air.plonk(air.ExprEvaluator(), z, alphas).source()
    assert list(src.tree_cols) == [4, 0, 4, 8] and src.n_constraints == 3
    claimed = qm31_array(seed + 4, 1)[0]
    return dict(name="plonk", source=src, air=1, ip=[0], qp=np.concatenate([z[None], alphas]), tree_cols=list(src.tree_cols),
                cols=_random_cols(seed, 16, eval_log), rcp=qm31_array(seed + 1, 3), trace_log=trace_log, eval_log=eval_log,
                claimed_sum=claimed, cumsum_shift=_shift(oracle, claimed, trace_log))


def freivalds_params(oracle, pk, pq, n_mats, seed):
    s, rv = qm31_array(seed + 5, 1)[0], qm31_array(seed + 6, 1)[0]
    rv_all, s_all = oracle.secure_powers(rv, pk + 1), oracle.secure_powers(s, pq + 1)
    return dict(rv_pow=rv_all[:pk], rv_step=rv_all[pk], s_pow=s_all[:pq], s_step=s_all[pq], s=s, rv=rv)


def freivalds_case(oracle, pk, pq, n_mats, trace_log, eval_log, seed, range_check=True, act_off=128):
    fp = freivalds_params(oracle, pk, pq, n_mats, seed)
    claimed = qm31_array(seed + 8, n_mats)
    rel = qm31_array(seed + 9, 2)  # z, alpha^0
    src = air.freivalds(air.ExprEvaluator(), pk, pq, n_mats, fp["rv_pow"], fp["rv_step"], fp["s_pow"], fp["s_step"], claimed, act_off,
                        (rel[0], rel[1]) if range_check else None).source()
    n_inter = 4 * (1 + 2 * n_mats) + (4 * ((pq + 1) // 2) if range_check else 0)
    assert list(src.tree_cols) == [4 + n_mats * pk, 0, pq, n_inter]
    qp = np.concatenate([fp["rv_pow"], fp["rv_step"][None], fp["s_pow"], fp["s_step"][None], claimed, rel]).astype(np.uint32)
    claimed_sum = qm31_array(seed + 10, 1)[0]
    return dict(name=f"freivalds_pk{pk}_pq{pq}_m{n_mats}", source=src, air=2, ip=[pk, pq, n_mats, act_off, int(range_check)], qp=qp,
                tree_cols=list(src.tree_cols), cols=_random_cols(seed, int(sum(src.tree_cols)), eval_log),
                rcp=qm31_array(seed + 1, src.n_constraints), trace_log=trace_log, eval_log=eval_log, claimed_sum=claimed_sum,
                cumsum_shift=_shift(oracle, claimed_sum, trace_log))


def small_cases(oracle):
    return [
        wide_fibonacci_case(oracle, 8, 5, 6, 100),
        wide_fibonacci_case(oracle, 100, 4, 6, 200),
        wide_fibonacci_case(oracle, 3, 3, 4, 300),
        plonk_case(oracle, 5, 6, 400),
        plonk_case(oracle, 4, 7, 500),
        freivalds_case(oracle, 3, 2, 2, 5, 6, 600),
        freivalds_case(oracle, 8, 5, 3, 6, 7, 700),
        freivalds_case(oracle, 4, 4, 1, 5, 7, 800, range_check=False),
    ]


def bench_case(oracle, which, trace_log=20, n_cols=256):
    """The benchmark's two workloads (bench.py --mode constraints), evaluation domain twice the trace: the wide
    Fibonacci AIR with n_cols columns, and the Freivalds component at pk = 16, pq = 1, two matrices, with its range check.
    Columns are m31_column(0x5EED0100 + c), the random-coefficient powers qm31_array(0x5EED0101)."""
    eval_log = trace_log + 1
    if which == "wide_fibonacci":
        case = wide_fibonacci_case(oracle, n_cols, trace_log, eval_log, 0)
        case["name"] = f"air_wide_fibonacci_{n_cols}x2e{trace_log}"
    else:
        pk, pq, n_mats = 16, 1, 2
        fp = freivalds_params(oracle, pk, pq, n_mats, 0x5EED0102)
        rel, claimed = qm31_array(0x5EED0103, 2), qm31_array(0x5EED0104, n_mats)
        src = air.freivalds(air.ExprEvaluator(), pk, pq, n_mats, fp["rv_pow"], fp["rv_step"], fp["s_pow"], fp["s_step"], claimed, 128,
                            (rel[0], rel[1])).source()
        qp = np.concatenate([fp["rv_pow"], fp["rv_step"][None], fp["s_pow"], fp["s_step"][None], claimed, rel]).astype(np.uint32)
        claimed_sum = qm31_array(0x5EED0105, 1)[0]
        case = dict(name=f"air_freivalds_pk16_pq1_2mats_2e{trace_log}", source=src, air=2, ip=[pk, pq, n_mats, 128, 1], qp=qp,
                    tree_cols=list(src.tree_cols), trace_log=trace_log, eval_log=eval_log, claimed_sum=claimed_sum,
                    cumsum_shift=_shift(oracle, claimed_sum, trace_log))
    n_total = int(sum(case["tree_cols"]))
    case["cols"] = [m31_column(0x5EED0100 + c, 1 << eval_log) for c in range(n_total)]
    case["rcp"] = qm31_array(0x5EED0101, case["source"].n_constraints)
    return case


def by_air(oracle, case, accum=None):
    """The oracle's hand-written evaluator of the case's AIR."""
    return oracle.constraint_quotients_air(case["air"], case["ip"], case["qp"], case["tree_cols"], case["cols"], case["rcp"],
                                           case["trace_log"], case["eval_log"], accum=accum, claimed_sum=case["claimed_sum"])


def by_ssa(oracle, case, accum=None):
    """The oracle's interpreter of the lowered program."""
    return oracle.constraint_quotients_ssa(case["source"], case["cols"], case["rcp"], case["trace_log"], case["eval_log"], accum=accum,
                                           cumsum_shift=case["cumsum_shift"])


def random_program(seed, n_ops, tree_cols, n_scalars, n_constraints, max_offset=2):
    """A random well-typed single-assignment program exercising every opcode, with row-independent subexpressions,
    repeated loads, PACK of literal zeros and dead code."""
    rng = np.random.default_rng(seed)
    ops, ext = [], []
    B, E = [], []

    def push(op, a=0, b=0, c=0, d=0, e=False):
        ops.append((op, a & 0xffffffff, b & 0xffffffff, c & 0xffffffff, d & 0xffffffff))
        ext.append(e)
        (E if e else B).append(len(ops) - 1)

    push(air.CONST_M31, 0)
    push(air.CONST_M31, 1)
    push(air.CONST_M31, P - 1)
    trees = [t for t, n in enumerate(tree_cols) if n]
    for _ in range(4):
        t = int(rng.choice(trees))
        push(air.LOAD, t, int(rng.integers(tree_cols[t])), int(rng.integers(-max_offset, max_offset + 1)))
    push(air.SCALAR, 0, e=True)
    push(air.CUMSUM_SHIFT, e=True)
    while len(ops) < n_ops:
        k = int(rng.integers(0, 20))
        pick_b = lambda: int(rng.choice(B))
        pick_any = lambda: int(rng.choice(B + E)) if rng.random() < 0.4 else int(rng.choice(E))
        if k < 4:
            t = int(rng.choice(trees))
            push(air.LOAD, t, int(rng.integers(tree_cols[t])), int(rng.integers(-max_offset, max_offset + 1)))
        elif k == 4:
            push(air.CONST_M31, int(rng.integers(P)))
        elif k == 5:
            push(air.SCALAR, int(rng.integers(n_scalars)), e=True)
        elif k < 9:
            push(int(rng.choice([air.ADD_B, air.SUB_B, air.MUL_B])), pick_b(), pick_b())
        elif k == 9:
            push(air.NEG_B, pick_b())
        elif k == 10:
            push(air.INV_B, pick_b())
        elif k < 16:
            a, b = pick_any(), pick_any()
            push(int(rng.choice([air.ADD_E, air.SUB_E, air.MUL_E])), a, b, e=ext[a] or ext[b])
        elif k == 16:
            a = pick_any()
            push(air.NEG_E, a, e=ext[a])
        elif k == 17:
            push(air.PACK, pick_b(), 0, 0, 0, e=False)  # (x, 0, 0, 0): a base value in secure clothing
        else:
            push(air.PACK, pick_b(), pick_b(), pick_b(), pick_b(), e=True)
    cons = rng.integers(len(ops) // 2, len(ops), n_constraints)
    cons[0] = 1          # a row-independent constraint
    cons[-1] = 3         # a bare column
    scalars = qm31_array(seed + 11, n_scalars)
    return air.AirSource(np.array(ops, np.uint32).reshape(-1, 5), cons.astype(np.uint32), np.array(tree_cols, np.uint32), scalars)


def wide_fibonacci_trace(n_cols, trace_log, seed=1):
    """A trace that satisfies the wide Fibonacci AIR: every row its own sequence from two seeded values."""
    n = 1 << trace_log
    a, b = m31_column(seed, n).astype(np.uint64), m31_column(seed + 1, n).astype(np.uint64)
    trace = [a, b]
    for _ in range(2, n_cols):
        a, b = b, (a * a % P + b * b % P) % P
        trace.append(b)
    return [c.astype(np.uint32) for c in trace]


def stark_words(words, committed, at_point):
    """The proof words followed by the two out-of-domain values: what the golden digests of whole proofs cover."""
    return np.concatenate([words, committed, at_point]).astype(np.uint32)


def mixed_components_case(oracle, logs=(6, 8), freivalds=True):
    """A statement of several components of different sizes: wide Fibonacci components with 10, 5, ... columns on traces
    of the given sizes and, optionally, the Freivalds component on the witness of a small matrix product. Returns
    (components for the oracle, lowered sources, flat columns (trees concatenated), columns per tree, columns as trees per component)."""
    from test_freivalds import _case, layout

    comps, sources, per_comp = [], [], []
    for i, lg in enumerate(logs):
        n_cols = 10 - 5 * (i % 2)
        comps.append(dict(air=0, ip=[n_cols], qp=np.zeros((1, 4), np.uint32), trace_log=lg, claimed_sum=None))
        sources.append(air.wide_fibonacci(air.ExprEvaluator(), n_cols).source())
        per_comp.append([[], [], wide_fibonacci_trace(n_cols, lg, seed=11 + i), []])
    if freivalds:
        tokens, n_in, n_outs, chunks = 5, 6, [7, 5], 4
        qx, qws = _case(31, tokens, n_in, n_outs)
        grid, pq, pk = layout(n_in, max(n_outs), tokens, chunks)
        trace_log, n_mats = grid[0], len(qws)
        base, pre, _, _ = oracle.freivalds_columns(qx, qws, grid, pq, pk)
        fp = freivalds_params(oracle, pk, pq, n_mats, 3100)
        inter, claims = oracle.freivalds_acc(base, pre, n_mats, grid, pq, pk, fp["s"], fp["rv"])
        qp = np.concatenate([fp["rv_pow"], fp["rv_step"][None], fp["s_pow"], fp["s_step"][None], claims, qm31_array(5, 2)]).astype(np.uint32)
        comps.append(dict(air=2, ip=[pk, pq, n_mats, 128, 0], qp=qp, trace_log=trace_log, claimed_sum=None))
        sources.append(air.freivalds(air.ExprEvaluator(), pk, pq, n_mats, fp["rv_pow"], fp["rv_step"], fp["s_pow"], fp["s_step"], claims, 128,
                                     None).source())
        per_comp.append([list(pre[n_mats * pk:]) + list(pre[:n_mats * pk]), [], list(base), list(inter)])
    trees = [[c for pc in per_comp for c in pc[t]] for t in range(4)]
    flat = [c for t in trees for c in t]
    return comps, sources, flat, [len(t) for t in trees], per_comp
