"""The Freivalds attention-witness component: columns (scatter) and Horner accumulators.

CPU: the oracle's restatement of prover/src/gadgets/freivalds/{trace,claims}.rs is pinned to the
identity the component exists to prove: the claim of matrix m equals
sum_{t,i} s^t rv^i (X W_m)[t, i] with the integer product X W_m computed independently.
GPU: zkb_freivalds_scatter / zkb_freivalds_acc against the oracle, every cell."""
import numpy as np
import pytest

from util import P, qm31_array


def layout(n_in, n_out_max, tokens, chunks):
    """FreivaldsLayout for a given chunk count (prover/src/gadgets/freivalds/layout.rs:22-46)."""
    pk = -(-n_out_max // chunks)
    pq = -(-tokens // chunks)
    rows = n_in * chunks
    log_rows = max(4, (rows - 1).bit_length())
    return (log_rows, n_in, chunks, (1 << log_rows) - rows), pq, pk


def _case(seed, tokens, n_in, n_outs):
    rng = np.random.default_rng(seed)
    qx = rng.integers(-128, 128, (tokens, n_in), dtype=np.int8)
    qws = [rng.integers(-128, 128, (n_in, no), dtype=np.int8) for no in n_outs]
    return qx, qws


def _qm31_pow_sum(oracle, coeffs_2d, s, rv):
    """sum_{t,i} s^t rv^i c[t,i] over QM31 for an integer matrix c."""
    acc = np.zeros(4, np.uint32)
    sp = oracle.secure_powers(s, coeffs_2d.shape[0])
    rp = oracle.secure_powers(rv, coeffs_2d.shape[1])
    for t in range(coeffs_2d.shape[0]):
        row = np.zeros(4, np.uint32)
        for i in range(coeffs_2d.shape[1]):
            c = int(coeffs_2d[t, i]) % P
            term = oracle.qm31_mul(rp[i], [c, 0, 0, 0])
            row = ((row.astype(np.uint64) + term) % P).astype(np.uint32)
        acc = ((acc.astype(np.uint64) + oracle.qm31_mul(sp[t], row)) % P).astype(np.uint32)
    return acc


@pytest.mark.parametrize("tokens,n_in,n_outs,chunks", [(5, 6, [7, 5], 4), (3, 8, [8], 2), (9, 4, [4, 6, 2], 3), (1, 16, [5], 1)])
def test_oracle_claims_are_the_freivalds_identity(oracle, tokens, n_in, n_outs, chunks):
    qx, qws = _case(11, tokens, n_in, n_outs)
    grid, pq, pk = layout(n_in, max(n_outs), tokens, chunks)
    base, pre, m_r8, off = oracle.freivalds_columns(qx, qws, grid, pq, pk)
    assert off == 0 and m_r8.sum() == pq << grid[0]
    s, rv = qm31_array(21, 1)[0], qm31_array(22, 1)[0]
    cols, claims = oracle.freivalds_acc(base, pre, len(qws), grid, pq, pk, s, rv)
    for m, w in enumerate(qws):
        y = qx.astype(np.int64) @ w.astype(np.int64)
        assert (claims[m] == _qm31_pow_sum(oracle, y, s, rv)).all()
    # the last committed row of acc_m carries the claim (coset row rows-1 sits at index coset_perm(rows-1))
    last = oracle.coset_perm((1 << grid[0]) - 1, grid[0])
    for m in range(len(qws)):
        assert (cols[8 + 8 * m:12 + 8 * m, last] == claims[m]).all()


@pytest.mark.gpu
@pytest.mark.parametrize("tokens,n_in,n_outs,chunks", [(5, 6, [7, 5], 4), (3, 8, [8], 2), (9, 4, [4, 6, 2], 3), (1, 16, [5], 1),
                                                      (32, 64, [64, 48, 64], 16), (17, 128, [96], 64)])
def test_freivalds_device_matches_oracle(ctx, oracle, tokens, n_in, n_outs, chunks):
    qx, qws = _case(12, tokens, n_in, n_outs)
    grid, pq, pk = layout(n_in, max(n_outs), tokens, chunks)
    rows = 1 << grid[0]
    n_mats = len(qws)
    want_base, want_pre, want_m, want_off = oracle.freivalds_columns(qx, qws, grid, pq, pk)
    d_qx = ctx.upload_bytes(qx)
    d_qw = [ctx.upload_bytes(w) for w in qws]
    base = [ctx.alloc(rows) for _ in range(pq)]
    pre = [ctx.alloc(rows) for _ in range(n_mats * pk + 4)]
    m_r8 = ctx.alloc(256).zero()
    off = ctx.alloc(2).zero()
    ctx.freivalds_scatter(d_qx.ptr, [w.ptr for w in d_qw], n_outs, grid, pq, pk, n_in, tokens, [b.ptr for b in base],
                          [p.ptr for p in pre], m_r8.ptr, 256, off.ptr)
    assert (np.stack([b.download() for b in base]) == want_base).all()
    assert (np.stack([p.download() for p in pre]) == want_pre).all()
    assert (m_r8.download() == want_m).all()
    assert int(off.download()[0]) == want_off
    s, rv = qm31_array(31, 1)[0], qm31_array(32, 1)[0]
    want_cols, want_claims = oracle.freivalds_acc(want_base, want_pre, n_mats, grid, pq, pk, s, rv)
    out = [ctx.alloc(rows) for _ in range((1 + 2 * n_mats) * 4)]
    claims = ctx.freivalds_acc([b.ptr for b in base], [p.ptr for p in pre[:n_mats * pk]], grid, pq, pk, n_mats, s, rv, [o.ptr for o in out])
    assert (np.stack([o.download() for o in out]) == want_cols).all()
    assert (claims == want_claims).all()
