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
