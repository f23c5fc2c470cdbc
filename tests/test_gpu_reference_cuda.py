"""The reference's own CUDA backend (compiled unmodified by oracle/Makefile.ref_cuda from the reference checkout)
run on the same GPU and the same seeded inputs as this repository's kernels: every word must agree, and both
must agree with the CPU oracle. This pins the oracle and the product to outputs of the reference's code itself
for the commitment path: precompute_twiddles, interpolate_columns, evaluate_polynomials (LDE) and
MerkleOps<Blake2sM31MerkleHasher>::commit_on_layer."""
import numpy as np
import pytest

from util import m31_column, edge_m31_column

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    from oracle import ref_cuda

    if not ref_cuda.available():
        pytest.skip("oracle/_ref/libstwo_cuda_ref.so is not built (the reference checkout is needed to build it)")
    return ref_cuda.RefCuda()


@pytest.mark.parametrize("log_n,log_blowup,ncols", [(4, 1, 3), (7, 2, 2), (10, 2, 4), (12, 1, 3), (13, 1, 5), (16, 2, 3), (19, 1, 2), (20, 2, 2)])
def test_commit_path_matches_reference_cuda(ctx, oracle, ref, log_n, log_blowup, ncols):
    log_out = log_n + log_blowup
    n, N = 1 << log_n, 1 << log_out
    cols = [edge_m31_column(9000 + 17 * log_n + c, n) for c in range(ncols)]
    tree = ref.twiddle_tree(log_out - 1)  # CanonicCoset(log_out).circle_domain().half_coset

    # interpolate
    r_cols = [ref.upload(c) for c in cols]
    ref.interpolate_columns(r_cols, log_n, tree)
    r_coeffs = [ref.download(p, n) for p in r_cols]
    bufs = [ctx.upload(c) for c in cols]
    ctx.ifft_cols([b.ptr for b in bufs], log_n)
    for c in range(ncols):
        assert (bufs[c].download(n) == r_coeffs[c]).all()
    if log_n <= 16:
        want = oracle.interpolate_cols(cols, log_n)
        for c in range(ncols):
            assert (r_coeffs[c] == want[c]).all()

    # low-degree extension
    r_ext = ref.extend_columns(r_cols, log_n, log_out)
    ref.evaluate_extended(r_ext, log_out, tree)
    r_evals = [ref.download(p, N) for p in r_ext]
    outs = [ctx.alloc(N) for _ in range(ncols)]
    ctx.lde_cols([b.ptr for b in bufs], log_n, [o.ptr for o in outs], log_out)
    for c in range(ncols):
        assert (outs[c].download(N) == r_evals[c]).all()

    # Merkle: leaf layer and the two layers above it
    r_leaf = ref.commit_on_layer(log_out, None, r_ext)
    r_l1 = ref.commit_on_layer(log_out - 1, r_leaf, [])
    r_l2 = ref.commit_on_layer(log_out - 2, r_l1, [])
    leaf, l1, l2 = ctx.alloc(8 * N), ctx.alloc(4 * N), ctx.alloc(2 * N)
    ctx.merkle_layer(log_out, 0, [o.ptr for o in outs], leaf.ptr)
    ctx.merkle_layer(log_out - 1, leaf.ptr, [], l1.ptr)
    ctx.merkle_layer(log_out - 2, l1.ptr, [], l2.ptr)
    assert (leaf.download(shape=(N, 8)) == ref.download_hashes(r_leaf, N)).all()
    assert (l1.download(shape=(N // 2, 8)) == ref.download_hashes(r_l1, N // 2)).all()
    assert (l2.download(shape=(N // 4, 8)) == ref.download_hashes(r_l2, N // 4)).all()
    for p in r_cols + r_ext + [r_leaf, r_l1, r_l2, tree["tw"], tree["itw"]]:
        ref.free(p)


def test_merkle_layer_with_columns_and_children_matches_reference_cuda(ctx, ref):
    log = 9
    n = 1 << log
    prev = m31_column(9900, 2 * n * 8).reshape(2 * n, 8)
    cols = [edge_m31_column(9901 + c, n) for c in range(21)]
    r_prev, r_cols = ref.upload(prev), [ref.upload(c) for c in cols]
    r_out = ref.commit_on_layer(log, r_prev, r_cols)
    pb, bufs, out = ctx.upload(prev), [ctx.upload(c) for c in cols], ctx.alloc(8 * n)
    ctx.merkle_layer(log, pb.ptr, [b.ptr for b in bufs], out.ptr)
    assert (out.download(shape=(n, 8)) == ref.download_hashes(r_out, n)).all()
    for p in r_cols + [r_prev, r_out]:
        ref.free(p)


@pytest.fixture(scope="module")
def refops():
    from oracle import ref_cuda

    if not ref_cuda.available():
        pytest.skip("oracle/_ref/libstwo_cuda_ref.so is not built (the reference checkout is needed to build it)")
    return ref_cuda.RefCudaOps()


def _secure(seed, n):
    return [edge_m31_column(seed + k, n) for k in range(4)]


# From 8 points up: on a 4-point circle domain the reference's CUDA fold takes its y twiddle from the pad word of
# the twiddle slice (stwo_cuda/cuda/poly_utils.cuh:7-18 on a slice of 2 words); its FFTs fall back to the CPU
# below 16 points (backend/cuda/poly.rs:184-196) and FRI never folds a circle that small. At 4 points it is this
# library that equals CpuBackend (backend/cpu/fri.rs:95-123): tests/test_gpu_ops.py compares the fold with the CPU
# oracle from a 2^2 domain up, and the oracle restates exactly that function; the reference's CUDA kernel is the
# side that differs there.
@pytest.mark.parametrize("log_n", [3, 5, 11, 17])
def test_fri_folds_match_reference_cuda(ctx, refops, log_n):
    from util import qm31_array

    n = 1 << log_n
    alpha = qm31_array(9100 + log_n, 1)[0]
    tree = refops.twiddle_tree(max(log_n, 5))
    # fold_line on LineDomain(half_odds(log_n))
    ev = _secure(9110, n)
    r_in = [refops.upload(c) for c in ev]
    r_out = refops.fold_line(r_in, log_n, alpha, tree)
    bi, bo = [ctx.upload(c) for c in ev], [ctx.alloc(n // 2) for _ in range(4)]
    ctx.fold_line([b.ptr for b in bo], [b.ptr for b in bi], log_n, alpha)
    for k in range(4):
        assert (bo[k].download(n // 2) == refops.download(r_out[k], n // 2)).all()
    # fold_circle_into_line from CanonicCoset(log_n).circle_domain() into a non-zero destination
    dst = _secure(9120, n // 2)
    r_dst = [refops.upload(c) for c in dst]
    refops.fold_circle_into_line(r_dst, r_in, log_n, alpha, tree)
    bd = [ctx.upload(c) for c in dst]
    ctx.fold_circle_into_line([b.ptr for b in bd], [b.ptr for b in bi], log_n, alpha)
    for k in range(4):
        assert (bd[k].download(n // 2) == refops.download(r_dst[k], n // 2)).all()
    for p in r_in + r_out + r_dst + [tree["tw"], tree["itw"]]:
        refops.free(p)


@pytest.mark.parametrize("log_n,k", [(4, 1), (9, 7), (14, 33)])
def test_quotients_match_reference_cuda(ctx, refops, log_n, k):
    from util import qm31_array

    n = 1 << log_n
    ncols = k + 2
    cols = [edge_m31_column(9200 + c, n) for c in range(ncols)]
    idx = np.array([(3 * j + 1) % ncols for j in range(k)], np.uint32)
    b, c = qm31_array(9210, k), qm31_array(9211, k)
    r_cols = [refops.upload(x) for x in cols]
    r_acc = refops.quot_numerators(r_cols, log_n, idx, b, c)
    bufs = [ctx.upload(x) for x in cols]
    acc = [ctx.alloc(n) for _ in range(4)]
    ctx.quot_numerators([x.ptr for x in bufs], log_n, idx, b, c, [a.ptr for a in acc])
    for q in range(4):
        assert (acc[q].download(n) == refops.download(r_acc[q], n)).all()
    # combine three accumulations of different sizes (lifting) at distinct sample points
    logs = [log_n, max(log_n - 2, 1), log_n]
    accs = [_secure(9220 + 10 * a, 1 << lg) for a, lg in enumerate(logs)]
    first_lin, points = qm31_array(9250, 3), qm31_array(9251, 6).reshape(3, 8)
    r_accs = [[refops.upload(x) for x in a] for a in accs]
    r_out = refops.quot_combine(r_accs, logs, first_lin, points, log_n)
    g_accs = [[ctx.upload(x) for x in a] for a in accs]
    out = [ctx.alloc(n) for _ in range(4)]
    ctx.quot_combine([x.ptr for a in g_accs for x in a], logs, first_lin, points, log_n, [o.ptr for o in out])
    for q in range(4):
        assert (out[q].download(n) == refops.download(r_out[q], n)).all()
    for p in r_cols + r_acc + r_out + [x for a in r_accs for x in a]:
        refops.free(p)


@pytest.mark.parametrize("kind", [0, 1, 2, 3])
@pytest.mark.parametrize("log_n", [3, 10, 15])
def test_gkr_ops_match_reference_cuda(ctx, refops, kind, log_n):
    from util import qm31_array

    n = 1 << log_n
    den = qm31_array(9300 + kind, n, nonzero=True)
    num = qm31_array(9310 + kind, n) if kind == 1 else m31_column(9310 + kind, n) if kind == 2 else None
    lam, r = qm31_array(9320, 1)[0], qm31_array(9321, 1)[0]
    y = qm31_array(9322, log_n - 2)
    r_den, r_num = refops.upload(den), (refops.upload(num) if num is not None else None)
    g_den, g_num = ctx.upload(den), (ctx.upload(num) if num is not None else None)
    # gen_eq_evals
    r_eq = refops.gen_eq_evals(y, lam)
    g_eq = ctx.alloc(n)
    ctx.gkr_eq_evals(y, lam, g_eq.ptr)
    assert (g_eq.download(n) == refops.download(r_eq, n)).all()
    # next_layer
    r_no, r_do = refops.next_layer(kind, r_num, r_den, n)
    g_no, g_do = ctx.alloc(2 * n), ctx.alloc(2 * n)
    ctx.gkr_next_layer(kind, g_num.ptr if g_num else 0, g_den.ptr, n, g_no.ptr, g_do.ptr)
    assert (g_do.download(2 * n) == refops.download(r_do, 2 * n)).all()
    if kind != 0:
        assert (g_no.download(2 * n) == refops.download(r_no, 2 * n)).all()
    # sum_as_poly_in_first_variable: the sums at t = 0 and t = 2
    want = refops.round_sums(kind, r_num, r_den, n, r_eq, lam)
    got = ctx.gkr_sum(kind, g_num.ptr if g_num else 0, g_den.ptr, n, g_eq.ptr, lam)
    assert (got == want).all()
    # fix_first_variable on the denominators (QM31) and, for multiplicities, the M31 numerators
    r_fx = refops.fix_first_variable(r_den, n, r, base=False)
    g_fx = ctx.alloc(2 * n)
    ctx.mle_fix_qm31(g_den.ptr, n, r, g_fx.ptr)
    assert (g_fx.download(2 * n) == refops.download(r_fx, 2 * n)).all()
    if kind == 2:
        r_fb = refops.fix_first_variable(r_num, n, r, base=True)
        ctx.mle_fix_m31(g_num.ptr, n, r, g_fx.ptr)
        assert (g_fx.download(2 * n) == refops.download(r_fb, 2 * n)).all()
        refops.free(r_fb)
    for p in [r_den, r_eq, r_no, r_do, r_fx] + ([r_num] if r_num else []):
        refops.free(p)


@pytest.mark.parametrize("log_n", [4, 12, 20])
def test_bit_reverse_matches_reference_cuda(ctx, refops, log_n):
    n = 1 << log_n
    v = m31_column(9400 + log_n, n)
    r = refops.upload(v)
    refops.bit_reverse(r, n)
    b = ctx.upload(v)
    ctx.bit_reverse_m31(b.ptr, log_n)
    assert (b.download(n) == refops.download(r, n)).all()
    refops.free(r)


@pytest.fixture(scope="module")
def refmore():
    from oracle import ref_cuda

    if not ref_cuda.available():
        pytest.skip("oracle/_ref/libstwo_cuda_ref.so is not built (the reference checkout is needed to build it)")
    return ref_cuda.RefCudaMore()


def test_accumulation_matches_reference_cuda(ctx, refmore):
    log_dst, log_src = 12, 9
    n, m = 1 << log_dst, 1 << log_src
    a, b, small = _secure(9500, n), _secure(9510, n), _secure(9520, m)
    ra, rb, rs = [refmore.upload(x) for x in a], [refmore.upload(x) for x in b], [refmore.upload(x) for x in small]
    refmore.accumulate(ra, rb, n)
    refmore.lift_and_accumulate(ra, log_dst, rs, log_src)
    ga, gb, gs = [ctx.upload(x) for x in a], [ctx.upload(x) for x in b], [ctx.upload(x) for x in small]
    ctx.accumulate([x.ptr for x in ga], [x.ptr for x in gb], n)
    ctx.lift_accumulate([x.ptr for x in ga], log_dst, [x.ptr for x in gs], log_src)
    for q in range(4):
        assert (ga[q].download(n) == refmore.download(ra[q], n)).all()
    for p in ra + rb + rs:
        refmore.free(p)


@pytest.mark.parametrize("log_n,ncols", [(10, 3), (16, 5), (20, 2)])
def test_batch_eval_at_point_matches_reference_cuda(ctx, refmore, log_n, ncols):
    from util import qm31_array

    n = 1 << log_n
    coeffs = [edge_m31_column(9600 + c, n) for c in range(ncols)]
    point = qm31_array(9610 + log_n, 2).reshape(8)  # the evaluation is algebraic: any (x, y) pair will do
    r = [refmore.upload(c) for c in coeffs]
    want = refmore.batch_eval_at_point(r, log_n, point)
    bufs = [ctx.upload(c) for c in coeffs]
    got = ctx.eval_at_point_cols([b.ptr for b in bufs], log_n, point)
    assert (got == want).all()
    for p in r:
        refmore.free(p)


@pytest.mark.parametrize("pow_bits", [0, 5, 12, 20])
def test_grind_matches_reference_cuda(ctx, refmore, pow_bits):
    digest = m31_column(9700 + pow_bits, 8)
    # the reference's kernel tests the raw first word of the digest (stwo_cuda/cuda/grind_blake2s.cu:105-112)
    assert ctx.grind(digest, pow_bits, m31_out=False) == refmore.grind(digest, pow_bits)


@pytest.mark.parametrize("tokens,n_in,n_outs,chunks", [(5, 6, [7, 5], 4), (9, 4, [4, 6, 2], 3), (32, 64, [64, 48, 64], 16), (17, 128, [96], 64)])
def test_freivalds_component_matches_reference_cuda(ctx, oracle, tokens, n_in, n_outs, chunks):
    from oracle import ref_cuda
    from test_freivalds import _case, layout
    from util import qm31_array

    if not ref_cuda.available():
        pytest.skip("oracle/_ref/libstwo_cuda_ref.so is not built (the reference checkout is needed to build it)")
    ref = ref_cuda.RefCudaFreivalds()
    qx, qws = _case(13, tokens, n_in, n_outs)
    grid, pq, pk = layout(n_in, max(n_outs), tokens, chunks)
    rows, n_mats = 1 << grid[0], len(qws)
    # witness scatter
    r_base, r_pre, r_m, r_counts = ref.scatter(qx, qws, grid, pq, pk)
    d_qx, d_qw = ctx.upload_bytes(qx), [ctx.upload_bytes(w) for w in qws]
    base, pre = [ctx.alloc(rows) for _ in range(pq)], [ctx.alloc(rows) for _ in range(n_mats * pk + 4)]
    m_r8, off = ctx.alloc(256).zero(), ctx.alloc(2).zero()
    ctx.freivalds_scatter(d_qx.ptr, [w.ptr for w in d_qw], n_outs, grid, pq, pk, n_in, tokens, [b.ptr for b in base],
                          [p.ptr for p in pre], m_r8.ptr, 256, off.ptr)
    for c in range(pq):
        assert (base[c].download() == ref.download(r_base[c], rows)).all()
    for c in range(n_mats * pk + 4):
        assert (pre[c].download() == ref.download(r_pre[c], rows)).all()
    assert (m_r8.download() == ref.download(r_m, 256)).all()
    assert int(off.download()[0]) == int(ref.download(r_counts, 3)[0])
    # accumulators: v, then (u_m, acc_m) per matrix, and the claims
    s, rv = qm31_array(41, 1)[0], qm31_array(42, 1)[0]
    s_pow, rv_pow = oracle.secure_powers(s, pq + 1), oracle.secure_powers(rv, pk + 1)
    r_out, r_claims = ref.acc(r_base, r_pre, grid, pq, pk, n_mats, s, rv, s_pow[:pq], rv_pow[:pk], s_pow[pq], rv_pow[pk])
    out = [ctx.alloc(rows) for _ in range((1 + 2 * n_mats) * 4)]
    claims = ctx.freivalds_acc([b.ptr for b in base], [p.ptr for p in pre[:n_mats * pk]], grid, pq, pk, n_mats, s, rv, [o.ptr for o in out])
    for c in range(len(out)):
        assert (out[c].download() == ref.download(r_out[c], rows)).all()
    assert (claims == r_claims).all()
    for p in r_base + r_pre + r_out + [r_m, r_counts]:
        ref.free(p)


@pytest.fixture(scope="module")
def refwit():
    from oracle import ref_cuda

    if not ref_cuda.available():
        pytest.skip("oracle/_ref/libstwo_cuda_ref.so is not built (the reference checkout is needed to build it)")
    try:
        return ref_cuda.RefCudaWitness()
    except AttributeError:
        pytest.skip("oracle/_ref/libstwo_cuda_ref.so predates the witness-generation kernels; rebuild it")


@pytest.mark.parametrize("log_rows,n_counters,bf16x,n_patch", [(5, 1, False, 0), (11, 2, False, 1), (14, 3, True, 2), (20, 2, False, 1)])
def test_witness_tables_match_reference_cuda(ctx, oracle, refwit, log_rows, n_counters, bf16x, n_patch):
    """zk_witness_gen_tables (stwo_cuda/cuda/zk_table_witness_gen.cu) against zkb_witness_tables and the oracle."""
    from test_witness_gen import _run_tables
    from witness_cases import tables_case

    expmap, counters, pi, pv = tables_case(300 + log_rows, log_rows, n_counters, n_patch)
    two_pow = 2.0 ** 6
    ref = refwit.tables(expmap, counters, log_rows, bf16x, two_pow, pi, pv)
    got = _run_tables(ctx, expmap, counters, log_rows, bf16x, two_pow, pi, pv)
    want = oracle.witness_tables(expmap, counters, log_rows, bf16x, two_pow, pi, pv)
    for r, g, w, name in zip(ref, got, want, "xym"):
        assert np.array_equal(r, g) and np.array_equal(r, w), name


@pytest.mark.parametrize("variant,tokens,chunks,per_row,kmax,sticky,do_ref,wide", [
    (0, 8, 4, 3, 16, 1, 1, False), (0, 32, 32, 16, 19, 1, 1, False), (0, 16, 16, 5, 12, 0, 0, True),
    (1, 8, 4, 3, 16, 1, 1, False), (1, 64, 64, 16, 19, 1, 1, False), (1, 16, 8, 4, 10, 1, 1, True)])
def test_witness_dequant_matches_reference_cuda(ctx, oracle, refwit, variant, tokens, chunks, per_row, kmax, sticky, do_ref, wide):
    """zk_witness_gen_dequant (stwo_cuda/cuda/zk_dequant_witness_gen.cu) against zkb_witness_dequant and the oracle: every
    committed and preprocessed cell, the four multiplicity arrays, the three counters and the cross-check patterns."""
    from test_witness_gen import run_dequant
    from witness_cases import dequant_case

    case = dequant_case(2000 + tokens + per_row, variant, tokens, chunks, per_row, kmax, sticky, do_ref, wide)
    ref = refwit.dequant(case)
    got = run_dequant(ctx, case)
    want = oracle.witness_dequant(case["acc"], case["jx"], case["jw"], case["sx"], case["sw"], case["norm3"], case["mul2"], case["n_base"],
                                  case["n_pre"], case["cfg"])
    if not do_ref:
        want["want"][:] = 0
    for k in ("counts", "m_norm", "m_frac", "m_mul", "m_r8", "pre", "base", "want"):
        assert np.array_equal(ref[k], got[k]), k
        assert np.array_equal(ref[k], want[k]), k


@pytest.fixture(scope="module")
def refpre():
    from oracle import ref_cuda

    if not ref_cuda.available():
        pytest.skip("oracle/_ref/libstwo_cuda_ref.so is not built (the reference checkout is needed to build it)")
    try:
        return ref_cuda.RefCudaWitnessPre()
    except AttributeError:
        pytest.skip("oracle/_ref/libstwo_cuda_ref.so predates the shared-table and residual-stream kernels; rebuild it")


@pytest.mark.parametrize("kind,log_rows,kmax,round_mode,n_counters,n_patch", [
    (0, 13, 13, 0, 2, 1), (0, 12, 13, 1, 1, 0), (0, 15, 21, 0, 3, 2), (1, 14, 13, 0, 1, 0), (1, 16, 14, 1, 2, 1), (2, 14, 13, 0, 2, 0),
    (2, 15, 13, 2, 1, 3), (3, 8, 0, 0, 1, 0), (4, 16, 0, 0, 2, 0)])
def test_pre_tables_match_reference_cuda(ctx, oracle, refpre, kind, log_rows, kmax, round_mode, n_counters, n_patch):
    """zk_witness_gen_pre_table (stwo_cuda/cuda/zk_pre_witness_gen.cu) against zkb_witness_pre_table and the oracle: every
    preprocessed column of the five shared tables and their multiplicity columns."""
    from test_witness_pre import run_pre_table
    from witness_cases import pre_table_case

    counters, pi, pv = pre_table_case(40 + 3 * kind + log_rows, kind, log_rows, n_counters, n_patch)
    ref_cols, ref_m = refpre.pre_table(kind, log_rows, kmax, round_mode, counters, pi, pv)
    got_cols, got_m = run_pre_table(ctx, kind, log_rows, kmax, round_mode, counters, pi, pv)
    want_cols, want_m = oracle.witness_pre_table(kind, log_rows, kmax, round_mode, counters, pi, pv)
    assert np.array_equal(ref_cols, got_cols) and np.array_equal(ref_cols, want_cols)
    assert np.array_equal(ref_m, got_m) and np.array_equal(ref_m, want_m)


def test_key_tile_selectors_match_reference_cuda(ctx, oracle, refpre):
    """zk_flags_key_tile (zk_acc.cu) and zk_witness_gen_sel (zk_pre_witness_gen.cu) against zkb_key_tile_flags,
    zkb_witness_selectors and the oracle, for the three sub-component shapes."""
    from test_witness_pre import TILE_CASES

    for shape, log_rows, groups, chunks, lead, desc, modulus, rw, ctx_len, n_cols, with_scale in TILE_CASES:
        rows = 1 << log_rows
        n_insts = (groups + ctx_len - 1) // ctx_len if shape == 1 else 0
        scale = np.random.default_rng(log_rows).integers(1, 2**31 - 1, max(1, n_insts), dtype=np.uint32)
        ref_flags, ref_cols = refpre.flags_and_selectors(shape, log_rows, groups, chunks, lead, desc, modulus, rw, scale, ctx_len, n_insts,
                                                         with_scale, n_cols)
        d_flags = ctx.alloc(rows)
        ctx.key_tile_flags(shape, log_rows, groups, chunks, lead, desc, modulus, rw, d_flags.ptr)
        cols = [ctx.alloc(rows) for _ in range(n_cols)]
        ctx.witness_selectors(shape, log_rows, groups, chunks, lead, desc, d_flags.ptr, ctx.upload(scale).ptr, ctx_len, n_insts, with_scale,
                              [c.ptr for c in cols])
        assert np.array_equal(ref_flags, d_flags.download()), (shape, log_rows)
        assert np.array_equal(ref_flags, oracle.key_tile_flags(shape, log_rows, groups, chunks, lead, desc, modulus, rw))
        assert np.array_equal(ref_cols, np.stack([c.download() for c in cols])), (shape, log_rows)
        assert np.array_equal(ref_cols, oracle.witness_selectors(shape, log_rows, groups, chunks, lead, desc, ref_flags, scale, ctx_len,
                                                                 with_scale, n_cols))


def test_residual_stream_matches_reference_cuda(ctx, oracle, refpre):
    """zk_witness_gen_residual_stream (stwo_cuda/cuda/zk_residual_stream_witness_gen.cu) against zkb_witness_residual_stream and
    the oracle: every committed cell, the natural-order outputs, every multiplicity array and the three counters."""
    from test_witness_pre import RS_CASES, run_residual_stream
    from witness_cases import residual_stream_case

    for shape, n, log_rows, live_rows, pad, un, kind, sticky, kmax, spread in RS_CASES:
        case = residual_stream_case(70 + n + log_rows, shape, n, log_rows, live_rows, pad=pad, un=un, kind=kind, sticky=sticky, kmax=kmax,
                                    spread=spread)
        ref, got, want = refpre.residual_stream(case), run_residual_stream(ctx, case), oracle.witness_residual_stream(case)
        for k in want:
            assert np.array_equal(ref[k], got[k]), (shape, n, log_rows, k)
            assert np.array_equal(ref[k], want[k]), (shape, n, log_rows, k)
