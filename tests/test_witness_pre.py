"""Device witness generation of the shared bf16 tables, the key tile selectors and the residual-stream component
(zkb_witness_pre_table, zkb_key_tile_flags, zkb_witness_selectors, zkb_witness_residual_stream) against the oracle's
restatement of the reference's host code (oracle/witness_pre.hpp), and the oracle itself against independent statements:
the tables against the second, separately written builders of zk_inference_prover_b200/witness_cases.py, and the
residual stream's outputs against IEEE float arithmetic rounded once to bf16."""
import numpy as np
import pytest

from zk_inference_prover_b200 import witness_cases as wc

ROUNDS = {"even": 0, "away": 1, "zero": 2}


def _natural(oracle, col, log_rows):
    """A committed-order column back in natural row order (the permutation is an involution)."""
    perm = np.array([oracle.coset_perm(i, log_rows) for i in range(1 << log_rows)]) if log_rows <= 12 else None
    if perm is None:
        i = np.arange(1 << log_rows, dtype=np.uint64)
        n = np.uint64(1 << log_rows)
        c = np.where(i & 1 == 1, (2 * n - i - 1) >> 1, i >> 1).astype(np.uint64)
        rev = np.zeros_like(c)
        for b in range(log_rows):
            rev |= ((c >> np.uint64(b)) & np.uint64(1)) << np.uint64(log_rows - 1 - b)
        perm = rev.astype(np.int64)
    out = np.zeros_like(col)
    out[perm] = col
    return out


# ---- the oracle against independent statements (CPU) -----------------------------------------------------------------

@pytest.mark.parametrize("kmax,round_mode", [(13, "even"), (16, "even"), (13, "away")])
def test_oracle_norm_table_matches_second_builder(oracle, kmax, round_mode):
    sticky = round_mode == "even"
    second = wc.norm_table(kmax, sticky) if sticky else wc._norm_table_away(kmax)
    log_rows = int(len(second) - 1).bit_length()
    cols, _ = oracle.witness_pre_table(0, log_rows, kmax, ROUNDS[round_mode], with_m=False)
    nat = np.stack([_natural(oracle, c, log_rows) for c in cols])
    assert np.array_equal(nat[3:6, :len(second)].T, second)
    assert not nat[:, len(second):].any()
    # the key columns are the decomposition the row stands for: mag = m2 * ph + r with st = (r != 0)
    m2, ph, st = nat[0, :len(second)], nat[1, :len(second)], nat[2, :len(second)]
    assert m2[0] == 0 and np.array_equal(m2[1:256], np.arange(1, 256)) and set(ph[1:256]) == {1}
    assert set(np.unique(ph[256:])) == {1 << k for k in range(kmax + 1)} and st.max() == (1 if sticky else 0)


def test_oracle_mul_and_frac_tables(oracle):
    cols, _ = oracle.witness_pre_table(2, 14, 13, 0, with_m=False)
    nat = np.stack([_natural(oracle, c, 14) for c in cols])
    assert np.array_equal(nat[2:4].T, wc.mul_table())
    assert np.array_equal(nat[0], np.arange(1 << 14) >> 7) and np.array_equal(nat[1], np.arange(1 << 14) & 127)
    cols, _ = oracle.witness_pre_table(1, 15, 13, 0, with_m=False)
    ph, r, st = (_natural(oracle, c, 15) for c in cols)
    d = np.arange(1, 1 << 14)
    assert np.array_equal(ph[1:1 << 14] + r[1:1 << 14], d) and np.all(r[1:1 << 14] < ph[1:1 << 14]) and np.array_equal(st[1:1 << 14], (r[1:1 << 14] != 0))
    assert not ph[1 << 14:].any() and ph[0] == 0


def _bf16_to_f32(pat):
    return (pat.astype(np.uint32) << 16).view(np.float32)


def _f32_to_bf16(x):
    u = x.astype(np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint32)


@pytest.mark.parametrize("kind", [0, 1])
def test_oracle_residual_stream_agrees_with_float_arithmetic(oracle, kind):
    """n independent adds (multiplies) of two bf16 inputs: the reported pattern is the IEEE sum (product) rounded once to
    bf16, to nearest even. Sums are exact in float32 when the exponents differ by at most 12 bits, and an operand more than
    12 bits below the other is dropped by the component and invisible to a correctly rounded sum alike."""
    case = wc.residual_stream_case(7 + kind, "pairs", 6, 8, 200, kind=kind, spread=10)
    out = oracle.witness_residual_stream(case)
    assert list(out["counts"]) == [0, 0, 0]
    wit = case["wit"].reshape(200, 12)
    finite = lambda p: np.where((((p >> 7) & 0xFF) == 0) | (((p >> 7) & 0xFF) == 0xFF), 0, p)  # zeros, infinities, NaNs read as +0
    a, b = _bf16_to_f32(finite(wit[:, :6])), _bf16_to_f32(finite(wit[:, 6:]))
    want = _f32_to_bf16(a + b if kind == 0 else a * b)
    want = np.where((want & 0x7FFF) == 0, 0, want)  # the component has one zero
    got = out["out_pat"].reshape(256, 6)[:200]
    assert np.array_equal(got, want)
    assert not out["out_pat"].reshape(256, 6)[200:].any()


def test_oracle_tree_sums_in_tree_order(oracle):
    case = wc.residual_stream_case(11, "tree", 5, 6, 40, pad=8, spread=3)
    out = oracle.witness_residual_stream(case)
    wit = case["wit"].reshape(40, 5)
    finite = lambda p: np.where((((p >> 7) & 0xFF) == 0) | (((p >> 7) & 0xFF) == 0xFF), 0, p)
    x = [_bf16_to_f32(finite(wit[:, i])) for i in range(5)]
    rnd = lambda v: _bf16_to_f32(np.where((_f32_to_bf16(v) & 0x7FFF) == 0, 0, _f32_to_bf16(v)))
    # pad 8: x0+x4, then (x0+x4)+x2 and x1+x3, then their sum
    root = rnd(rnd(rnd(x[0] + x[4]) + x[2]) + rnd(x[1] + x[3]))
    assert np.array_equal(out["out_pat"][:40], _f32_to_bf16(root) & np.where(root == 0, 0, 0xFFFF))


def test_oracle_key_tile_flags_and_selectors(oracle):
    # 3 instances x 4 channels, 5 chunks each, 4 lead rows: 64 rows
    flags = oracle.key_tile_flags(0, 6, 12, 5, 4, 1, 4, 0)
    assert not flags[:4].any() and np.all(flags[4:] & 1)
    grp_first = np.arange(4, 64, 5)
    assert not (flags[grp_first] & 2).any() and np.all(flags[np.setdiff1d(np.arange(4, 64), grp_first)] & 2)
    assert np.array_equal(np.nonzero(flags & 4)[0], grp_first + 4)
    # descending groups 11..0; instance starts where group % 4 == 3: rows of groups 11, 7, 3, except row 0
    assert np.array_equal(np.nonzero(flags & 8)[0], [4, 24, 44])
    cols = oracle.witness_selectors(0, 6, 12, 5, 4, 1, flags, [], 1, False, 5)
    nat = np.stack([_natural(oracle, c, 6) for c in cols])
    assert np.array_equal(nat[0], (flags >> 1) & 1) and np.array_equal(nat[1], (flags >> 2) & 1) and np.array_equal(nat[4], (flags >> 3) & 1)
    assert np.array_equal(nat[2], np.arange(64) > 0) and np.array_equal(nat[3], np.arange(64) == 63)


# ---- the CUDA path against the oracle (GPU) -----------------------------------------------------------------------------

def run_pre_table(ctx, kind, log_rows, kmax, round_mode, counters, patch_idx, patch_val, with_m=True):
    rows, n_cols = 1 << log_rows, {0: 6, 1: 3, 2: 4, 3: 2, 4: 1}[kind]
    d_cnt = [ctx.upload(c) for c in counters]
    cols = [ctx.alloc(rows) for _ in range(n_cols)]
    m = ctx.alloc(rows).zero()
    d_pi = ctx.upload(patch_idx) if len(patch_idx) else None
    d_pv = ctx.upload(np.ascontiguousarray(patch_val).reshape(-1)) if len(patch_idx) else None
    ctx.witness_pre_table(kind, log_rows, kmax, round_mode, [c.ptr for c in d_cnt], [c.ptr for c in cols], m.ptr if with_m else 0,
                          d_pi.ptr if d_pi else 0, d_pv.ptr if d_pv else 0, len(patch_idx))
    return np.stack([c.download() for c in cols]), m.download()


@pytest.mark.gpu
@pytest.mark.parametrize("kind,log_rows,kmax,round_mode,n_counters,n_patch", [
    (0, 13, 13, "even", 2, 1), (0, 12, 13, "away", 1, 0), (0, 14, 21, "zero", 0, 0), (0, 15, 21, "even", 3, 2), (1, 14, 13, "even", 1, 0),
    (1, 16, 14, "away", 2, 1), (2, 14, 13, "even", 2, 0), (2, 15, 13, "zero", 1, 3), (3, 8, 0, "even", 1, 0), (4, 1, 0, "even", 1, 0),
    (4, 16, 0, "even", 2, 0), (4, 20, 0, "even", 1, 0)])
def test_pre_tables_match_oracle(ctx, oracle, kind, log_rows, kmax, round_mode, n_counters, n_patch):
    counters, pi, pv = wc.pre_table_case(500 + 7 * kind + log_rows, kind, log_rows, n_counters, n_patch)
    got_cols, got_m = run_pre_table(ctx, kind, log_rows, kmax, ROUNDS[round_mode], counters, pi, pv, with_m=n_counters > 0)
    want_cols, want_m = oracle.witness_pre_table(kind, log_rows, kmax, ROUNDS[round_mode], counters, pi, pv, with_m=n_counters > 0)
    assert np.array_equal(got_cols, want_cols)
    if n_counters:
        assert np.array_equal(got_m, want_m)


@pytest.mark.gpu
def test_pre_table_refuses_a_table_taller_than_its_column(ctx, zkb):
    cols = [ctx.alloc(1 << 10) for _ in range(6)]
    with pytest.raises(zkb.ZkbError):
        ctx.witness_pre_table(0, 10, 13, 0, [], [c.ptr for c in cols])
    with pytest.raises(zkb.ZkbError):
        ctx.witness_pre_table(1, 14, 13, 0, [], [c.ptr for c in cols])  # wrong column count for the kind


TILE_CASES = [  # shape, log_rows, groups, chunks, lead, descending, modulus, rw, ctx_len, n_cols, with_scale
    (0, 6, 12, 5, 4, 1, 4, 0, 1, 5, False), (0, 10, 128, 8, 0, 1, 16, 0, 1, 5, False), (1, 8, 30, 8, 16, 1, 10, 0, 10, 8, True),
    (1, 12, 512, 7, 512, 1, 64, 0, 64, 9, True), (1, 9, 64, 8, 0, 0, 16, 0, 16, 8, False), (2, 7, 0, 0, 0, 0, 32, 4, 1, 3, False),
    (2, 11, 0, 0, 0, 0, 96, 3, 1, 3, False)]


@pytest.mark.gpu
@pytest.mark.parametrize("shape,log_rows,groups,chunks,lead,desc,modulus,rw,ctx_len,n_cols,with_scale", TILE_CASES)
def test_key_tile_flags_and_selectors_match_oracle(ctx, oracle, shape, log_rows, groups, chunks, lead, desc, modulus, rw, ctx_len, n_cols, with_scale):
    rows = 1 << log_rows
    d_flags = ctx.alloc(rows)
    ctx.key_tile_flags(shape, log_rows, groups, chunks, lead, desc, modulus, rw, d_flags.ptr)
    flags = d_flags.download()
    assert np.array_equal(flags, oracle.key_tile_flags(shape, log_rows, groups, chunks, lead, desc, modulus, rw))
    n_insts = (groups + ctx_len - 1) // ctx_len if shape == 1 else 0
    scale = np.random.default_rng(log_rows).integers(1, 2**31 - 1, max(1, n_insts), dtype=np.uint32)
    cols = [ctx.alloc(rows) for _ in range(n_cols)]
    ctx.witness_selectors(shape, log_rows, groups, chunks, lead, desc, d_flags.ptr, ctx.upload(scale).ptr, ctx_len, n_insts, with_scale,
                          [c.ptr for c in cols])
    want = oracle.witness_selectors(shape, log_rows, groups, chunks, lead, desc, flags, scale, ctx_len, with_scale, n_cols)
    assert np.array_equal(np.stack([c.download() for c in cols]), want)


def run_residual_stream(ctx, case):
    """Runs zkb_witness_residual_stream on zeroed buffers; returns the same dict as oracle.witness_residual_stream."""
    rows, n_leaves, n_cols, out_w = 1 << case["log_rows"], case["n_leaves"], case["n_cols"], len(case["out_slot"])
    upi = lambda a: ctx.upload_bytes(np.ascontiguousarray(a, np.int32))
    d_wit, d_norm, d_smul = ctx.upload(case["wit"]), ctx.upload(case["norm3"]), upi(case["smul3"])
    d_un = [upi(u) for u in case["un2"]]
    cols = [ctx.alloc(rows).zero() for _ in range(n_cols)]
    out_pat, out_nat, in_nat = ctx.alloc(max(1, rows * out_w)).zero(), ctx.alloc(max(1, rows * out_w * 2)).zero(), ctx.alloc(rows * n_leaves * 2).zero()
    ml = case["m_len"]
    ms = {k: ctx.alloc(ml[k]).zero() for k in ("pow", "norm", "val", "frac", "smul")}
    m_un = [ctx.alloc(ml["un"]).zero() for _ in d_un]
    counts = ctx.alloc(4).zero()
    ctx.witness_residual_stream(case["lowered_groups"], case["lowered_slots"], case["out_slot"], case["kind"], case["sticky"], case["kmax"],
                                d_norm.ptr, len(case["norm3"]) // 3, d_smul.ptr, len(case["smul3"]) // 3, [u.ptr for u in d_un], case["n_val"],
                                d_wit.ptr, case["live_rows"], case["log_rows"], [c.ptr for c in cols], out_pat.ptr, out_nat.ptr, in_nat.ptr,
                                {k: (v.ptr, ml[k]) for k, v in ms.items()}, [(m.ptr, ml["un"]) for m in m_un], counts.ptr)
    return {"cols": np.stack([c.download() for c in cols]), "out_pat": out_pat.download()[:rows * out_w],
            "out_nat": out_nat.download()[:rows * out_w * 2].view(np.int32), "in_nat": in_nat.download().view(np.int32),
            "m_pow": ms["pow"].download(), "m_norm": ms["norm"].download(), "m_val": ms["val"].download(), "m_frac": ms["frac"].download(),
            "m_smul": ms["smul"].download(), "m_un": np.stack([m.download() for m in m_un]) if m_un else np.zeros((0, ml["un"]), np.uint32),
            "counts": counts.download()[:3]}


RS_CASES = [  # shape, n, log_rows, live_rows, pad, un, kind, sticky, kmax, spread
    ("pairs", 4, 5, 32, None, (0, 0), 0, True, 13, 6), ("pairs", 16, 9, 500, None, (0, 0), 1, True, 13, 130), ("pairs", 8, 8, 256, None, (1, 0), 0, True, 16, 9),
    ("pairs", 8, 7, 100, None, (1, 2), 1, True, 13, 30), ("tree", 5, 6, 40, 8, (0, 0), 0, True, 13, 3), ("tree", 64, 10, 1000, 64, (1, 0), 0, True, 21, 14),
    ("tree", 33, 8, 256, 64, (0, 0), 0, False, 13, 6), ("pairs", 128, 12, 4000, None, (0, 0), 0, True, 13, 70), ("pairs", 3, 1, 2, None, (0, 0), 1, False, 13, 130)]


@pytest.mark.gpu
@pytest.mark.parametrize("shape,n,log_rows,live_rows,pad,un,kind,sticky,kmax,spread", RS_CASES)
def test_residual_stream_matches_oracle(ctx, oracle, shape, n, log_rows, live_rows, pad, un, kind, sticky, kmax, spread):
    case = wc.residual_stream_case(900 + n + log_rows, shape, n, log_rows, live_rows, pad=pad, un=un, kind=kind, sticky=sticky, kmax=kmax, spread=spread)
    got, want = run_residual_stream(ctx, case), oracle.witness_residual_stream(case)
    for k in want:
        assert np.array_equal(got[k], want[k]), k
    if kind == 1 and spread > 100 and live_rows >= 100:
        assert want["counts"][1] > 0  # products of extreme exponents leave bf16's normal range: the counter is exercised


@pytest.mark.gpu
def test_residual_stream_refuses_a_column_outside_the_trace(ctx, zkb):
    case = wc.residual_stream_case(1, "pairs", 4, 5, 32)
    bad = dict(case)
    bad["lowered_slots"] = case["lowered_slots"].copy()
    bad["lowered_slots"][2, 4] = case["n_cols"]  # a slot whose cells start past the last column
    with pytest.raises(zkb.ZkbError):
        run_residual_stream(ctx, bad)
