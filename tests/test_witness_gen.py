"""Witness generation of the tables' own columns and of the matmul dequantize component.

CPU: the oracle's restatement of the reference's host code (oracle/witness.hpp) is pinned to facts that do not depend on it:
the x column is the coset permutation itself; the y column's bf16 patterns equal torch's float32 -> bfloat16 conversion; with an
honest normalisation table and an honest mantissa-product table the integer dequantisation agrees with the IEEE double-precision
cross-check on every slot (the property the reference's own cross-check exists to assert), for both scale variants.
GPU: zkb_witness_tables / zkb_witness_dequant against the oracle, every cell, every multiplicity and every counter. The reference's
own device kernels are compared on the same inputs in test_gpu_reference_cuda.py."""
import numpy as np
import pytest

from witness_cases import dequant_case, tables_case


def test_tables_oracle_x_is_the_coset_permutation_and_y_is_bf16_of_the_scaled_row(oracle):
    import torch

    log_rows, frac = 12, 5.0
    expmap, counters, _, _ = tables_case(1, log_rows, 2)
    expmap = np.arange(1 << 16, dtype=np.uint32)  # identity map: y is then the pattern itself
    x, y, m = oracle.witness_tables(expmap, counters, log_rows, False, 2.0 ** frac)
    perm = np.array([oracle.coset_perm(i, log_rows) for i in range(1 << log_rows)])
    assert np.array_equal(x, perm)
    assert np.array_equal(np.sort(x), np.arange(1 << log_rows))
    want = torch.tensor(-perm.astype(np.float64) / 2.0 ** frac, dtype=torch.float32).to(torch.bfloat16).view(torch.int16).numpy().astype(np.uint16)
    assert np.array_equal(y, want.astype(np.uint32))
    assert np.array_equal(m, (counters[0] + counters[1])[perm])
    xb, yb, _ = oracle.witness_tables(expmap, [], log_rows, True, 1.0, patch_idx=[5], patch_val=[77])
    assert np.array_equal(yb[xb != 5], xb[xb != 5] & 0xFFFF) and yb[xb == 5][0] == 77


@pytest.mark.parametrize("variant", [0, 1])
def test_dequant_oracle_agrees_with_ieee_cross_check_on_honest_tables(oracle, variant):
    case = dequant_case(10 + variant, variant, tokens=16, chunks=8, per_row=6, kmax=16, sticky=1, do_ref=1)
    out = oracle.witness_dequant(case["acc"], case["jx"], case["jw"], case["sx"], case["sw"], case["norm3"], case["mul2"], case["n_base"],
                                 case["n_pre"], case["cfg"])
    assert out["counts"].tolist() == [0, 0, 0]  # nothing off the range table, no cross-check disagreement, every slot described
    cfg = case["cfg"]
    slots = case["rows"] * cfg["per_row"]
    assert out["m_norm"].sum() == slots and out["m_frac"].sum() == slots
    assert out["m_r8"].sum() == slots * (2 if variant else 1)
    # the accumulator column, read back through the permutation, is the input
    perm = np.array([oracle.coset_perm(i, cfg["log_rows"]) for i in range(case["rows"])])
    j = perm
    t, b = cfg["tokens"] - 1 - j // cfg["chunks"], cfg["chunks"] - 1 - j % cfg["chunks"]
    col = out["base"][cfg["slot0"] + 2 * cfg["per_slot"] + cfg["f_acc"]]
    want = case["acc"][t, b * cfg["per_row"] + 2].astype(np.int64) % ((1 << 31) - 1)
    assert np.array_equal(col, want.astype(np.uint32))


def test_dequant_oracle_counts_what_the_tables_cannot_describe(oracle):
    case = dequant_case(20, 0, tokens=8, chunks=4, per_row=4, kmax=12, wide=True)
    out = oracle.witness_dequant(case["acc"], case["jx"], case["jw"], case["sx"], case["sw"], case["norm3"], case["mul2"], case["n_base"],
                                 case["n_pre"], case["cfg"])
    assert out["counts"][2] >= 1 and out["counts"][0] >= 1


# ---------------------------------------------------------------------------------------------- GPU
def _run_tables(ctx, expmap, counters, log_rows, bf16x, two_pow, patch_idx, patch_val, with_m=True):
    rows = 1 << log_rows
    d_map = ctx.upload(expmap)
    d_cnt = [ctx.upload(c) for c in counters]
    x, y, m = ctx.alloc(rows), ctx.alloc(rows), ctx.alloc(rows).zero()
    d_pi = ctx.upload(patch_idx) if len(patch_idx) else None
    d_pv = ctx.upload(patch_val) if len(patch_idx) else None
    ctx.witness_tables(d_map.ptr, [c.ptr for c in d_cnt], log_rows, bf16x, two_pow, x.ptr, y.ptr, m.ptr if with_m else 0,
                       d_pi.ptr if d_pi else 0, d_pv.ptr if d_pv else 0, len(patch_idx))
    return x.download(), y.download(), m.download()


@pytest.mark.gpu
@pytest.mark.parametrize("log_rows,n_counters,bf16x,n_patch", [(4, 1, False, 0), (10, 3, False, 2), (11, 1, False, 1), (12, 2, True, 0),
                                                                 (13, 0, False, 0), (16, 4, False, 3), (20, 2, False, 1), (22, 1, False, 0)])
def test_tables_match_oracle(ctx, oracle, log_rows, n_counters, bf16x, n_patch):
    expmap, counters, pi, pv = tables_case(100 + log_rows, log_rows, n_counters, n_patch)
    two_pow = 2.0 ** 7
    got = _run_tables(ctx, expmap, counters, log_rows, bf16x, two_pow, pi, pv, with_m=n_counters > 0)
    want = oracle.witness_tables(expmap, counters, log_rows, bf16x, two_pow, pi, pv)
    for g, w, name in zip(got, want, "xym"):
        assert np.array_equal(g, w), name


def run_dequant(ctx, case):
    """Runs zkb_witness_dequant on zeroed buffers; returns the same dict as oracle.witness_dequant."""
    cfg, rows = case["cfg"], case["rows"]
    chain = cfg["variant"] == 1
    up = lambda a: ctx.upload_bytes(np.ascontiguousarray(a))
    d_acc, d_norm, d_mul = up(case["acc"]), ctx.upload(case["norm3"]), ctx.upload(case["mul2"])
    d_jx, d_jw, d_sx, d_sw = up(case["jx"]), up(case["jw"]), ctx.upload(case["sx"]), ctx.upload(case["sw"])
    base = [ctx.alloc(rows).zero() for _ in range(case["n_base"])]
    pre = [ctx.alloc(rows).zero() for _ in range(case["n_pre"])]
    m_norm, m_frac = ctx.alloc(cfg["n_norm"]).zero(), ctx.alloc(cfg["n_frac"]).zero()
    m_mul, m_r8, counts = ctx.alloc(cfg["n_mul"]).zero(), ctx.alloc(cfg["n_r8"]).zero(), ctx.alloc(3).zero()
    want = ctx.alloc(rows * cfg["per_row"]).zero()
    ctx.witness_dequant(cfg, d_acc.ptr, 0 if chain else d_jx.ptr, 0 if chain else d_jw.ptr, d_sx.ptr if chain else 0, d_sw.ptr if chain else 0,
                        d_norm.ptr, d_mul.ptr, [b.ptr for b in base], [p.ptr for p in pre], m_norm.ptr, m_frac.ptr, m_mul.ptr, m_r8.ptr,
                        counts.ptr, want.ptr)
    return {"base": np.stack([b.download() for b in base]), "pre": np.stack([p.download() for p in pre]), "m_norm": m_norm.download(),
            "m_frac": m_frac.download(), "m_mul": m_mul.download(), "m_r8": m_r8.download(), "counts": counts.download(), "want": want.download()}


DEQUANT_SHAPES = [  # (variant, tokens, chunks, per_row, kmax, sticky, do_ref, wide)
    (0, 4, 4, 1, 16, 1, 1, False), (0, 32, 8, 16, 16, 1, 1, False), (0, 32, 64, 9, 19, 0, 0, False), (0, 16, 16, 5, 12, 1, 1, True),
    (1, 4, 4, 3, 16, 1, 1, False), (1, 32, 16, 16, 16, 1, 1, False), (1, 64, 32, 7, 19, 0, 0, False), (1, 16, 8, 4, 10, 1, 1, True),
    (1, 512, 256, 16, 19, 1, 1, False),
]


@pytest.mark.gpu
@pytest.mark.parametrize("variant,tokens,chunks,per_row,kmax,sticky,do_ref,wide", DEQUANT_SHAPES)
def test_dequant_matches_oracle(ctx, oracle, variant, tokens, chunks, per_row, kmax, sticky, do_ref, wide):
    case = dequant_case(1000 + tokens + per_row, variant, tokens, chunks, per_row, kmax, sticky, do_ref, wide)
    got = run_dequant(ctx, case)
    want = oracle.witness_dequant(case["acc"], case["jx"], case["jw"], case["sx"], case["sw"], case["norm3"], case["mul2"], case["n_base"],
                                  case["n_pre"], case["cfg"])
    if not do_ref:
        want["want"][:] = 0
    for k in ("counts", "m_norm", "m_frac", "m_mul", "m_r8", "pre", "base", "want"):
        assert np.array_equal(got[k], want[k]), k
    if wide:
        assert want["counts"][2] >= 1


@pytest.mark.gpu
def test_witness_entry_points_reject_bad_shapes(zkb, ctx):
    case = dequant_case(1, 0, 8, 4, 4)
    bad = dict(case["cfg"], tokens=7)  # tokens * chunks is no longer the row count
    buf = ctx.alloc(64)
    with pytest.raises(zkb.ZkbError):
        ctx.witness_dequant(bad, buf.ptr, buf.ptr, buf.ptr, 0, 0, buf.ptr, 0, [buf.ptr] * case["n_base"], [buf.ptr] * case["n_pre"], buf.ptr,
                            buf.ptr, 0, buf.ptr, buf.ptr)
    with pytest.raises(zkb.ZkbError):
        ctx.witness_tables(buf.ptr, [], 0, False, 1.0, buf.ptr, buf.ptr, 0)
