"""Parity of every CUDA operator with the CPU oracle, bit for bit, through the C ABI.

The shape of each test follows the reference's backend-vs-CpuBackend tests
(nitroo/crates/stwo/src/prover/backend/simd/{fft,fri,quotients,blake2s,bit_reverse}.rs test modules,
backend/cuda/*.rs test modules): same seeded input to both, assert equality of every word."""
import numpy as np
import pytest

from util import P, edge_m31_column, m31_column, qm31_array

pytestmark = pytest.mark.gpu


def up_cols(ctx, arr2d):
    bufs = [ctx.upload(c) for c in arr2d]
    return bufs, [b.ptr for b in bufs]


def secure_bufs(ctx, arr4):
    bufs = [ctx.upload(c) for c in arr4]
    return bufs, [b.ptr for b in bufs]


def down4(bufs, n):
    return np.stack([b.download(n) for b in bufs])


# ------------------------------------------------------------------ twiddles (A1)
@pytest.mark.parametrize("log_size", [1, 2, 5, 12, 17])
def test_twiddle_tower(ctx, oracle, log_size):
    tw, itw = ctx.twiddles(log_size)
    otw, oitw = oracle.twiddles(log_size)
    assert (tw == otw).all()
    assert (itw == oitw).all()


# ------------------------------------------------------------------ interpolate (A2)
@pytest.mark.parametrize("log_n,ncols", [(1, 3), (2, 2), (3, 5), (4, 1), (7, 17), (10, 4), (12, 3), (13, 2), (16, 2), (20, 1)])
def test_ifft_matches_oracle(ctx, oracle, log_n, ncols):
    vals = np.stack([edge_m31_column(100 + c, 1 << log_n) for c in range(ncols)])
    bufs, ptrs = up_cols(ctx, vals)
    ctx.ifft_cols(ptrs, log_n)
    got = np.stack([b.download() for b in bufs])
    want = oracle.interpolate_cols(vals, log_n)
    assert (got == want).all()


def test_ifft_zero_columns(ctx):
    ctx.ifft_cols([], 8)


# ------------------------------------------------------------------ LDE (A3)
@pytest.mark.parametrize(
    "log_n,log_out,ncols",
    [(0, 1, 2), (1, 1, 1), (1, 2, 3), (2, 2, 2), (0, 5, 2), (1, 4, 1), (3, 3, 2), (3, 5, 7), (6, 8, 3), (10, 11, 2),
     (12, 14, 3), (13, 13, 1), (14, 16, 2), (16, 18, 1), (18, 20, 1), (20, 22, 1)],
)
def test_lde_matches_oracle(ctx, oracle, log_n, log_out, ncols):
    coeffs = np.stack([edge_m31_column(200 + c, 1 << log_n) for c in range(ncols)])
    bufs, ptrs = up_cols(ctx, coeffs)
    outs = [ctx.alloc(1 << log_out) for _ in range(ncols)]
    ctx.lde_cols(ptrs, log_n, [o.ptr for o in outs], log_out)
    got = np.stack([o.download() for o in outs])
    want = oracle.evaluate_cols(coeffs, log_n, log_out)
    assert (got == want).all()
    # inputs are left untouched
    assert (np.stack([b.download() for b in bufs]) == coeffs).all()


def test_lde_then_ifft_roundtrip_large(ctx):
    # size-independent property at a size the oracle would take long for: interpolate(evaluate(c)) == c
    log_n = 21
    coeffs = m31_column(7, 1 << log_n)
    src = ctx.upload(coeffs)
    out = ctx.alloc(1 << log_n)
    ctx.lde_cols([src.ptr], log_n, [out.ptr], log_n)
    ctx.ifft_cols([out.ptr], log_n)
    assert (out.download() == coeffs).all()


# ------------------------------------------------------------------ eval_at_point
@pytest.mark.parametrize("log_n,ncols", [(0, 2), (1, 1), (3, 3), (8, 2), (11, 2), (12, 3), (16, 2)])
def test_eval_at_point(ctx, oracle, log_n, ncols):
    coeffs = np.stack([m31_column(300 + c, 1 << log_n) for c in range(ncols)])
    bufs, ptrs = up_cols(ctx, coeffs)
    point = oracle.secure_circle_mul(0x1234567 + log_n)
    got = ctx.eval_at_point_cols(ptrs, log_n, point)
    want = np.stack([oracle.eval_at_point(c, point) for c in coeffs])
    assert (got == want).all()


# ------------------------------------------------------------------ bit reverse (A4)
@pytest.mark.parametrize("log_n", [1, 2, 3, 9, 10, 11, 12, 15, 20])
def test_bit_reverse_m31(ctx, oracle, log_n):
    v = m31_column(400 + log_n, 1 << log_n)
    b = ctx.upload(v)
    ctx.bit_reverse_m31(b.ptr, log_n)
    got = b.download()
    assert (got == oracle.bit_reverse(v)).all()
    ctx.bit_reverse_m31(b.ptr, log_n)  # an involution
    assert (b.download() == v).all()


def test_bit_reverse_literal(ctx):
    # nitroo/crates/stwo/src/prover/backend/cpu/mod.rs:86-90
    b = ctx.upload(np.arange(8))
    ctx.bit_reverse_m31(b.ptr, 3)
    assert list(b.download()) == [0, 4, 2, 6, 1, 5, 3, 7]


@pytest.mark.parametrize("log_n", [1, 4, 10, 13])
def test_bit_reverse_qm31(ctx, log_n):
    v = qm31_array(500 + log_n, 1 << log_n)
    b = ctx.upload(v)
    ctx.bit_reverse_qm31(b.ptr, log_n)
    got = b.download(shape=(-1, 4))
    idx = np.array([int(f"{i:0{log_n}b}"[::-1], 2) for i in range(1 << log_n)])
    assert (got == v[idx]).all()


# ------------------------------------------------------------------ Merkle (A5)
@pytest.mark.parametrize("m31", [True, False])
@pytest.mark.parametrize("log_size,ncols,with_prev", [(0, 0, False), (0, 3, False), (3, 1, False), (4, 16, False), (5, 17, True),
                                                      (6, 0, True), (6, 15, True), (7, 32, False), (8, 33, True), (10, 100, False),
                                                      (12, 256, False), (3, 4, True),
                                                      # few rows, many columns: the variant that requests the next block's words ahead (merkle_layer_prefetch_kernel)
                                                      (0, 64, False), (2, 65, True), (5, 80, False), (6, 127, True), (7, 128, True),
                                                      (9, 1000, True), (11, 300, False), (13, 64, True), (15, 97, True), (17, 66, False)])
def test_merkle_layer(ctx, oracle, log_size, ncols, with_prev, m31):
    n = 1 << log_size
    cols = [edge_m31_column(600 + c, n) for c in range(ncols)]
    prev = m31_column(699, 2 * n * 8).reshape(2 * n, 8) if with_prev else None
    if prev is not None and m31:
        prev = prev % np.uint32(P)
    bufs = [ctx.upload(c) for c in cols]
    pbuf = ctx.upload(prev) if prev is not None else None
    out = ctx.alloc(n * 8)
    ctx.merkle_layer(log_size, pbuf.ptr if pbuf else 0, [b.ptr for b in bufs], out.ptr, m31_out=m31)
    got = out.download(shape=(n, 8))
    want = oracle.commit_on_layer(log_size, prev, cols, m31=m31)
    assert (got == want).all()


def test_merkle_tree_root_mixed_heights(ctx, oracle):
    # MerkleProver::commit order (nitroo/crates/stwo/src/prover/vcs/prover.rs:39-64): largest layer first,
    # columns injected at the layer of their own height.
    heights = {6: 3, 4: 2, 3: 1, 0: 1}
    cols = {h: [m31_column(700 + 10 * h + c, 1 << h) for c in range(k)] for h, k in heights.items()}
    prev_g, prev_o = None, None
    keep = []
    for log in range(6, -1, -1):
        layer_cols = cols.get(log, [])
        bufs = [ctx.upload(c) for c in layer_cols]
        out = ctx.alloc((1 << log) * 8)
        ctx.merkle_layer(log, prev_g.ptr if prev_g else 0, [b.ptr for b in bufs], out.ptr)
        keep.append((bufs, out))
        prev_g = out
        prev_o = oracle.commit_on_layer(log, prev_o, layer_cols)
    assert (prev_g.download(shape=(1, 8)) == prev_o).all()


# ------------------------------------------------------------------ FRI folds (A7, A8)
@pytest.mark.parametrize("log_n", [1, 2, 3, 5, 10, 16])
def test_fold_line(ctx, oracle, log_n):
    n = 1 << log_n
    ev = np.stack([edge_m31_column(800 + k, n) for k in range(4)])
    alpha = qm31_array(801, 1)[0]
    ib, ip = secure_bufs(ctx, ev)
    ob = [ctx.alloc(n // 2) for _ in range(4)]
    ctx.fold_line([o.ptr for o in ob], ip, log_n, alpha)
    assert (down4(ob, n // 2) == oracle.fold_line(ev, alpha)).all()


@pytest.mark.parametrize("log_n", [1, 2, 3, 4, 8, 15])
def test_fold_circle_into_line(ctx, oracle, log_n):
    n = 1 << log_n
    src = np.stack([edge_m31_column(810 + k, n) for k in range(4)])
    dst = np.stack([edge_m31_column(820 + k, n // 2) for k in range(4)])
    alpha = qm31_array(811, 1)[0]
    sb, sp = secure_bufs(ctx, src)
    db, dp = secure_bufs(ctx, dst)
    ctx.fold_circle_into_line(dp, sp, log_n, alpha)
    assert (down4(db, n // 2) == oracle.fold_circle_into_line(dst, src, alpha)).all()


# ------------------------------------------------------------------ quotients (A9, A10, A11)
@pytest.mark.parametrize("log_n,ncols,k", [(1, 1, 1), (3, 4, 4), (5, 7, 7), (8, 20, 13), (10, 33, 50), (12, 5, 0),
                                           # short and wide: the columns are split over the grid (partial sums, then one addition pass)
                                           (1, 40, 1500), (5, 300, 1100), (9, 1400, 1400), (12, 64, 2049)])
def test_quot_numerators(ctx, oracle, log_n, ncols, k):
    n = 1 << log_n
    cols = [edge_m31_column(900 + c, n) for c in range(ncols)]
    rng = np.random.default_rng(log_n)
    col_idx = rng.integers(0, ncols, size=k).astype(np.uint32)
    point = oracle.secure_circle_mul(987654321 + k)
    values = qm31_array(901, max(k, 1))[:k]
    rands = qm31_array(902, max(k, 1))[:k]
    want, first = oracle.quot_numerators(cols, point, col_idx, values, rands)
    lc = np.stack([oracle.line_coeffs(point, values[j], rands[j]) for j in range(k)]) if k else np.zeros((0, 3, 4), np.uint32)
    bufs = [ctx.upload(c) for c in cols]
    ob = [ctx.alloc(n) for _ in range(4)]
    ctx.quot_numerators([b.ptr for b in bufs], log_n, col_idx, lc[:, 1, :], lc[:, 2, :], [o.ptr for o in ob])
    assert (down4(ob, n) == want).all()


@pytest.mark.parametrize("lifting_log,acc_logs", [(1, [1]), (2, [1, 2]), (3, [3]), (5, [2, 5]), (8, [8, 4, 8]), (10, [3, 5, 7, 10, 10, 9, 8, 6, 4, 10])])
def test_quot_combine(ctx, oracle, lifting_log, acc_logs):
    accs = [np.stack([m31_column(1000 + 10 * i + k, 1 << lg) for k in range(4)]) for i, lg in enumerate(acc_logs)]
    first_lin = qm31_array(1001, len(acc_logs))
    points = np.stack([oracle.secure_circle_mul(55555 + 977 * i) for i in range(len(acc_logs))])
    want = oracle.quot_combine(accs, first_lin, points, lifting_log)
    bufs = [[ctx.upload(a[k]) for k in range(4)] for a in accs]
    ob = [ctx.alloc(1 << lifting_log) for _ in range(4)]
    ctx.quot_combine([b.ptr for a in bufs for b in a], acc_logs, first_lin, points, lifting_log, [o.ptr for o in ob])
    assert (down4(ob, 1 << lifting_log) == want).all()


def test_accumulate_and_lift(ctx, oracle):
    a = np.stack([edge_m31_column(1100 + k, 256) for k in range(4)])
    b = np.stack([edge_m31_column(1110 + k, 256) for k in range(4)])
    ab, ap = secure_bufs(ctx, a)
    bb, bp = secure_bufs(ctx, b)
    ctx.accumulate(ap, bp, 256)
    assert (down4(ab, 256) == oracle.accumulate(a, b)).all()
    # lift_and_accumulate over ascending sizes as a chain of lift_accumulate calls
    cols = [np.stack([m31_column(1120 + 10 * i + k, 1 << lg) for k in range(4)]) for i, lg in enumerate([1, 3, 3, 6])]
    want = oracle.lift_and_accumulate(cols)
    bufs = [secure_bufs(ctx, c) for c in cols]
    for i in range(1, len(cols)):
        ctx.lift_accumulate(bufs[i][1], [1, 3, 3, 6][i], bufs[i - 1][1], [1, 3, 3, 6][i - 1])
    assert (down4(bufs[-1][0], 64) == want).all()


def test_secure_powers(ctx, oracle):
    f = qm31_array(1200, 1)[0]
    assert (ctx.secure_powers(f, 9) == oracle.secure_powers(f, 9)).all()


# ------------------------------------------------------------------ GKR / MLE (A12-A15)
@pytest.mark.parametrize("ny", [0, 1, 2, 5, 11])
def test_gkr_eq_evals(ctx, oracle, ny):
    y = qm31_array(1300, max(ny, 1))[:ny]
    v = qm31_array(1301, 1)[0]
    out = ctx.alloc(4 << ny)
    ctx.gkr_eq_evals(y, v, out.ptr)
    assert (out.download(shape=(-1, 4)) == oracle.gkr_eq_evals(y, v)).all()


def _layer(kind, n, seed):
    den = qm31_array(seed, n, nonzero=True)
    if kind == 1:
        num = qm31_array(seed + 1, n)
    elif kind == 2:
        num = m31_column(seed + 1, n)
    else:
        num = None
    return num, den


@pytest.mark.parametrize("kind", [0, 1, 2, 3])
@pytest.mark.parametrize("log_n", [1, 2, 6, 13])
def test_gkr_next_layer(ctx, oracle, kind, log_n):
    n = 1 << log_n
    num, den = _layer(kind, n, 1400 + kind)
    nb = ctx.upload(num) if num is not None else None
    db = ctx.upload(den)
    no, do = ctx.alloc(2 * n), ctx.alloc(2 * n)
    ctx.gkr_next_layer(kind, nb.ptr if nb else 0, db.ptr, n, no.ptr, do.ptr)
    wn, wd = oracle.gkr_next_layer(kind, num, den)
    assert (do.download(shape=(-1, 4)) == wd).all()
    if kind != 0:
        assert (no.download(shape=(-1, 4)) == wn).all()


@pytest.mark.parametrize("kind", [0, 1, 2, 3])
@pytest.mark.parametrize("log_n", [2, 3, 9, 14, 18])
def test_gkr_sum(ctx, oracle, kind, log_n):
    n = 1 << log_n
    num, den = _layer(kind, n, 1500 + kind)
    eq = qm31_array(1510, n // 4)
    lam = qm31_array(1511, 1)[0]
    nb = ctx.upload(num) if num is not None else None
    db, eb = ctx.upload(den), ctx.upload(eq)
    got = ctx.gkr_sum(kind, nb.ptr if nb else 0, db.ptr, n, eb.ptr, lam)
    assert (got == oracle.gkr_round_sums(kind, num, den, eq, lam)).all()
    # the ticket is reset: a second call gives the same answer
    assert (ctx.gkr_sum(kind, nb.ptr if nb else 0, db.ptr, n, eb.ptr, lam) == got).all()


@pytest.mark.parametrize("log_n", [1, 4, 12])
def test_mle_fix_first_variable(ctx, oracle, log_n):
    n = 1 << log_n
    r = qm31_array(1600, 1)[0]
    q = qm31_array(1601, n)
    qb, ob = ctx.upload(q), ctx.alloc(2 * n)
    ctx.mle_fix_qm31(qb.ptr, n, r, ob.ptr)
    assert (ob.download(shape=(-1, 4)) == oracle.mle_fix_first(q, r)).all()
    ctx.mle_fix_qm31(qb.ptr, n, r, qb.ptr)  # in place
    assert (qb.download(2 * n, shape=(-1, 4)) == oracle.mle_fix_first(q, r)).all()
    m = edge_m31_column(1602, n)
    mb = ctx.upload(m)
    ctx.mle_fix_m31(mb.ptr, n, r, ob.ptr)
    assert (ob.download(shape=(-1, 4)) == oracle.mle_fix_first(m, r)).all()


# ------------------------------------------------------------------ gather / errors
def test_gather_multi(ctx):
    cols = [m31_column(1700 + c, 64) for c in range(5)]
    bufs = [ctx.upload(c) for c in cols]
    idx = [3, 0, 63, 17]
    got = ctx.gather_multi([b.ptr for b in bufs], idx)
    want = np.array([[c[i] for c in cols] for i in idx], np.uint32)
    assert (got == want).all()


def test_invalid_arguments_return_status(ctx, zkb):
    with pytest.raises(zkb.ZkbError) as e:
        ctx.ifft_cols([1234], 40)
    assert e.value.code == -1
    with pytest.raises(zkb.ZkbError):
        ctx.lde_cols([16], 5, [16], 6)  # aliasing input and output
    # the context is still usable
    b = ctx.upload(np.arange(8))
    ctx.bit_reverse_m31(b.ptr, 3)
    assert list(b.download()) == [0, 4, 2, 6, 1, 5, 3, 7]


@pytest.mark.parametrize("top_log", [1, 3, 6, 10])
def test_merkle_top_equals_layer_by_layer(ctx, oracle, top_log):
    top = m31_column(1800 + top_log, (1 << top_log) * 8).reshape(-1, 8)
    tb = ctx.upload(top)
    lowers = [ctx.alloc(8 << k) for k in range(top_log)]
    ctx.merkle_top(top_log, tb.ptr, [b.ptr for b in lowers])
    prev = top
    for k in range(top_log - 1, -1, -1):
        prev = oracle.commit_on_layer(k, prev, [], m31=True)
        assert (lowers[k].download(shape=(-1, 8)) == prev).all()


@pytest.mark.parametrize("ny", [12, 13, 17, 22])
def test_gkr_eq_evals_two_table_path(ctx, oracle, ny):
    y = qm31_array(1900 + ny, ny)
    v = qm31_array(1901, 1)[0]
    out = ctx.alloc(4 << ny)
    ctx.gkr_eq_evals(y, v, out.ptr)
    assert (out.download(shape=(-1, 4)) == oracle.gkr_eq_evals(y, v)).all()


@pytest.mark.parametrize("kind", [0, 1, 2, 3])
@pytest.mark.parametrize("log_n", [3, 4, 10, 17])
def test_gkr_fix_and_sum(ctx, oracle, kind, log_n):
    n = 1 << log_n
    num, den = _layer(kind, n, 2000 + kind)
    eq = qm31_array(2010, max(n // 8, 1))
    lam, r = qm31_array(2011, 1)[0], qm31_array(2012, 1)[0]
    nb = ctx.upload(num) if num is not None else None
    db, eb = ctx.upload(den), ctx.upload(eq)
    no, do = ctx.alloc(2 * n), ctx.alloc(2 * n)
    got = ctx.gkr_fix_and_sum(kind, nb.ptr if nb else 0, db.ptr, n, r, eb.ptr, lam, no.ptr, do.ptr)
    fden = oracle.mle_fix_first(den, r)
    fnum = oracle.mle_fix_first(num, r) if num is not None else None
    assert (do.download(shape=(-1, 4)) == fden).all()
    if fnum is not None:
        assert (no.download(shape=(-1, 4)) == fnum).all()
    out_kind = 1 if kind == 2 else kind
    assert (got == oracle.gkr_round_sums(out_kind, fnum, fden, eq, lam)).all()


@pytest.mark.parametrize("m31", [True, False])
@pytest.mark.parametrize("log_size,runs", [(5, [1]), (6, [16]), (4, [16, 1]), (7, [16, 16]), (9, [32, 16, 7]), (3, [48, 16]),
                                           (10, [16, 16, 16, 16, 3])])
def test_merkle_leaves_in_runs_of_columns(ctx, oracle, zkb, log_size, runs, m31):
    n, total = 1 << log_size, sum(runs)
    cols = [edge_m31_column(2100 + c, n) for c in range(total)]
    bufs = [ctx.upload(c) for c in cols]
    out = ctx.alloc(n * 8)
    before = 0
    for r in runs:
        ctx.merkle_leaves_partial(log_size, [b.ptr for b in bufs[before:before + r]], before, total, out.ptr, m31_out=m31)
        before += r
    assert (out.download(shape=(n, 8)) == oracle.commit_on_layer(log_size, None, cols, m31=m31)).all()
    # a run that is not the last one must hold whole blocks
    with pytest.raises(zkb.ZkbError):
        ctx.merkle_leaves_partial(log_size, [bufs[0].ptr], 0, total + 1, out.ptr)


def test_device_channel_step_and_folds_with_device_challenge(ctx, oracle):
    # Three chained steps of mix_root + draw_secure_felt on the device against the oracle's channel, then both
    # folds with the challenge read from device memory against the by-value folds.
    ch = oracle.Channel()
    ch.mix_u64(0xC0FFEE)
    ch.draw_secure_felt()                      # a channel that has already drawn (n_draws = 1)
    state = np.zeros(16, np.uint32)
    state[:8] = np.frombuffer(ch.digest(), np.uint32)
    state[8] = 1
    d_chan = ctx.upload(state)
    d_alpha, d_copy = ctx.alloc(4 * 3), ctx.alloc(8 * 3)
    alphas = []
    for k in range(3):
        root = m31_column(2200 + k, 8)
        d_root = ctx.upload(root)
        ctx.channel_mix_root_draw(d_chan.ptr, d_root.ptr, d_alpha.ptr + 16 * k, d_copy.ptr + 32 * k)
        ch.mix_root(root)
        alphas.append(ch.draw_secure_felt())
        assert (d_copy.download(shape=(3, 8))[k] == root).all()
    got = d_alpha.download(shape=(3, 4))
    assert (got == np.array(alphas, np.uint32)).all()
    st = d_chan.download(16)
    assert (st[:8] == np.frombuffer(ch.digest(), np.uint32)).all() and st[8] == 1
    for log_n in (1, 2, 3, 9):
        n = 1 << log_n
        ev = np.stack([edge_m31_column(2210 + k, n) for k in range(4)])
        bi = [ctx.upload(c) for c in ev]
        o1, o2 = [ctx.alloc(n // 2) for _ in range(4)], [ctx.alloc(n // 2) for _ in range(4)]
        ctx.fold_line([b.ptr for b in o1], [b.ptr for b in bi], log_n, alphas[1])
        ctx.fold_line_dalpha([b.ptr for b in o2], [b.ptr for b in bi], log_n, d_alpha.ptr + 16)
        assert all((a.download() == b.download()).all() for a, b in zip(o1, o2))
        dst = np.stack([edge_m31_column(2220 + k, n // 2) for k in range(4)])
        c1, c2 = [ctx.upload(c) for c in dst], [ctx.upload(c) for c in dst]
        ctx.fold_circle_into_line([b.ptr for b in c1], [b.ptr for b in bi], log_n, alphas[2])
        ctx.fold_circle_into_line_dalpha([b.ptr for b in c2], [b.ptr for b in bi], log_n, d_alpha.ptr + 32)
        assert all((a.download() == b.download()).all() for a, b in zip(c1, c2))
        # the variants that also hash the folded layer's Merkle leaves
        o3, lv, want_lv = [ctx.alloc(n // 2) for _ in range(4)], ctx.alloc(4 * n), ctx.alloc(4 * n)
        ctx.fold_line_dalpha_leaves([b.ptr for b in o3], [b.ptr for b in bi], log_n, d_alpha.ptr + 16, lv.ptr)
        ctx.merkle_layer(log_n - 1, 0, [b.ptr for b in o1], want_lv.ptr)
        assert all((a.download() == b.download()).all() for a, b in zip(o1, o3)) and (lv.download() == want_lv.download()).all()
        if log_n >= 3:
            c3 = [ctx.upload(c) for c in dst]
            ctx.fold_circle_into_line_dalpha_leaves([b.ptr for b in c3], [b.ptr for b in bi], log_n, d_alpha.ptr + 32, lv.ptr)
            ctx.merkle_layer(log_n - 1, 0, [b.ptr for b in c1], want_lv.ptr)
            assert all((a.download() == b.download()).all() for a, b in zip(c1, c3)) and (lv.download() == want_lv.download()).all()


# ------------------------------------------------------------------ PolyOps from evaluations (barycentric, folding)
@pytest.mark.parametrize("log_n", [3, 4, 7, 10, 14])
def test_barycentric_and_folding_evaluation(ctx, oracle, log_n):
    vals = edge_m31_column(8800 + log_n, 1 << log_n)
    point = oracle.secure_circle_mul(0x2468ACE + log_n)
    ev = ctx.upload(vals)
    w = ctx.barycentric_weights(log_n, point)
    want_w = oracle.barycentric_weights(log_n, point)
    assert (w.download(shape=(-1, 4)) == want_w).all()
    got = ctx.barycentric_eval_at_point(ev.ptr, w.ptr, log_n)
    assert (got == oracle.barycentric_eval_at_point(vals, want_w)).all()
    by_folding = ctx.eval_at_point_by_folding(ev.ptr, log_n, point)
    assert (by_folding == oracle.eval_at_point_by_folding(vals, point)).all()
    # the relation the reference's own tests check: all routes give the polynomial's value at the point
    coeffs = oracle.interpolate_cols([vals], log_n)[0]
    assert (got == oracle.eval_at_point(coeffs, point)).all() and (by_folding == got).all()
    assert (ev.download() == vals).all()


def test_fri_decompose_is_refused(ctx, zkb):
    import ctypes as C

    buf = ctx.alloc(64)
    arr = (C.c_void_p * 4)(*[buf.ptr] * 4)
    lam = np.zeros(4, np.uint32)
    rc = ctx.lib.zkb_fri_decompose(ctx.h, arr, C.c_int(4), arr, lam.ctypes.data_as(C.c_void_p))
    assert rc == -1 and b"decompose" in ctx.lib.zkb_last_error(ctx.h)
