// The three PolyOps methods that evaluate a polynomial from its EVALUATIONS on a canonic circle domain, in their
// simplest correct form (they are off the prover's path: the prover stores coefficients and samples with
// batch_eval_at_point): barycentric_weights, barycentric_eval_at_point, eval_at_point_by_folding
// (nitroo/crates/stwo/src/prover/poly/circle/ops.rs:59-86; CPU statements backend/cpu/circle.rs:101-180), and the
// FriOps::decompose the reference's own CUDA backend leaves unimplemented (backend/cuda/fri.rs:71-77).
#include <vector>

#include "common.cuh"

namespace zk {

struct BaryArgs {
    cpoint shift[31];  // -initial + step/2 of CanonicCoset(k).coset, k = 1..30 (index k)
    int log_size;
    uint32_t four_pow;  // 4^(log_size - 1)
    qm31 px, py, vn_p;
};

// weight_i = vn(p) / (s_i * v_i(p)),  s_i = -2 y_i * vanishing'(point_i),  v_i(p) = h.y / (1 + h.x), h = p - point_i
// (core/constraints.rs:38-55, 87-93). Row i of the bit-reversed canonic domain: point of half_odds(L-1) or its conjugate.
__global__ void __launch_bounds__(256) bary_weights_kernel(BaryArgs a, const uint32_t* __restrict__ tw, uint32_t* __restrict__ out) {
    const size_t row = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= ((size_t)1 << a.log_size)) return;
    uint32_t x, y;
    half_coset_point(tw, a.log_size, (uint32_t)(row >> 1), x, y);
    if (row & 1) y = m31_neg(y);
    uint32_t prod = 1u;
    for (int k = 1; k < a.log_size; k++) {
        cpoint q = cpoint_add(cpoint{x, y}, a.shift[k]);
        uint32_t v = q.x;
        for (int j = 1; j < k; j++) v = m31_sub(m31_dbl(m31_sqr(v)), 1u);
        prod = m31_mul(prod, v);
    }
    const uint32_t si = m31_mul(m31_mul(m31_neg(m31_dbl(y)), a.four_pow), prod);
    // h = p + conj(point_i)
    const qm31 hx = qm31_add(qm31_mul_m31(a.px, x), qm31_mul_m31(a.py, y));
    const qm31 hy = qm31_sub(qm31_mul_m31(a.py, x), qm31_mul_m31(a.px, y));
    const qm31 num = qm31_mul(a.vn_p, qm31_add(qm31_one(), hx));
    const qm31 w = qm31_mul(num, qm31_inv(qm31_mul_m31(hy, si)));
    reinterpret_cast<uint4*>(out)[row] = make_uint4(w.c[0], w.c[1], w.c[2], w.c[3]);
}

// partial[b] = sum over the block's rows of evals[i] * weights[i] (cpu/circle.rs:134-141); the host adds the partials.
__global__ void __launch_bounds__(256) bary_dot_kernel(const uint32_t* __restrict__ evals, const uint32_t* __restrict__ weights, size_t n,
                                                       uint32_t* __restrict__ partial) {
    __shared__ uint32_t red[4][256];
    qm31 acc = qm31_zero();
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) {
        const uint4 w = reinterpret_cast<const uint4*>(weights)[i];
        acc = qm31_add(acc, qm31_mul_m31(qm31{{w.x, w.y, w.z, w.w}}, evals[i]));
    }
    for (int k = 0; k < 4; k++) red[k][threadIdx.x] = acc.c[k];
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if ((int)threadIdx.x < s)
            for (int k = 0; k < 4; k++) red[k][threadIdx.x] = m31_add(red[k][threadIdx.x], red[k][threadIdx.x + s]);
        __syncthreads();
    }
    if (threadIdx.x < 4) partial[4 * blockIdx.x + threadIdx.x] = red[threadIdx.x][0];
}

static cpoint host_pt(uint32_t index) {
    cpoint g{2u, 1268011823u}, r{1u, 0u};
    for (int b = 0; b < 31; b++) {
        if ((index >> b) & 1u) r = cpoint_add(r, g);
        g = cpoint_add(g, g);
    }
    return r;
}
// -initial + step/2 of CanonicCoset(k).coset = Coset::odds(k): initial index 2^(30-k), step index 2^(31-k)
static cpoint canonic_shift(int k) {
    const uint32_t initial = 1u << (30 - k), half_step = 1u << (30 - k);
    cpoint i = host_pt(initial);
    return cpoint_add(cpoint{i.x, m31_neg(i.y)}, host_pt(half_step));
}
// coset_vanishing(CanonicCoset(log).coset, p) at a secure point (core/constraints.rs:12-35)
static qm31 host_coset_vanishing(int log, qm31 px, qm31 py) {
    cpoint s = canonic_shift(log);
    qm31 x = qm31_sub(qm31_mul_m31(px, s.x), qm31_mul_m31(py, s.y));
    for (int k = 1; k < log; k++) x = qm31_double_x(x);
    return x;
}

}  // namespace zk

using namespace zk;

extern "C" {

int zkb_barycentric_weights(zkb_ctx* ctx, int log_size, const uint32_t h_point[8], uint32_t* d_weights) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, h_point && d_weights && log_size >= 3 && log_size <= ctx->max_log && log_size <= 30);
    ZKB_CHECK_ARG(ctx, ((uintptr_t)d_weights & 15) == 0);
    BaryArgs a;
    memset(&a, 0, sizeof(a));
    for (int k = 1; k < log_size; k++) a.shift[k] = canonic_shift(k);
    a.log_size = log_size;
    a.four_pow = 1u;
    for (int k = 1; k < log_size; k++) a.four_pow = m31_mul(a.four_pow, 4u);
    memcpy(a.px.c, h_point, 16);
    memcpy(a.py.c, h_point + 4, 16);
    a.vn_p = host_coset_vanishing(log_size, a.px, a.py);
    DeviceGuard g(ctx);
    const size_t n = (size_t)1 << log_size;
    bary_weights_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(a, ctx->tw, d_weights);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

int zkb_barycentric_eval_at_point(zkb_ctx* ctx, const uint32_t* d_evals, const uint32_t* d_weights, int log_size, uint32_t h_out[4]) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, d_evals && d_weights && h_out && log_size >= 0 && log_size <= 30 && ((uintptr_t)d_weights & 15) == 0);
    DeviceGuard g(ctx);
    const size_t n = (size_t)1 << log_size;
    unsigned blocks = (unsigned)((n + 255) / 256);
    if (blocks > 512u) blocks = 512u;
    bary_dot_kernel<<<blocks, 256, 0, ctx->stream>>>(d_evals, d_weights, n, ctx->scratch);
    ZKB_LAUNCH_CHECK(ctx);
    std::vector<uint32_t> part(4 * (size_t)blocks);
    ZKB_CUDA(ctx, cudaMemcpyAsync(part.data(), ctx->scratch, part.size() * 4, cudaMemcpyDeviceToHost, ctx->stream));
    ZKB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    qm31 acc = qm31_zero();
    for (unsigned b = 0; b < blocks; b++) acc = qm31_add(acc, qm31{{part[4 * b], part[4 * b + 1], part[4 * b + 2], part[4 * b + 3]}});
    memcpy(h_out, acc.c, 16);
    return ZKB_OK;
}

int zkb_eval_at_point_by_folding(zkb_ctx* ctx, const uint32_t* d_evals, int log_size, const uint32_t h_point[8], uint32_t h_out[4]) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, d_evals && h_point && h_out && log_size >= 2 && log_size <= ctx->max_log && log_size <= 30);
    // get_folding_alphas (core/poly/utils.rs:45-70): y first, then x, pi(x), pi(pi(x)), ...
    qm31 px, py;
    memcpy(px.c, h_point, 16);
    memcpy(py.c, h_point + 4, 16);
    const size_t n = (size_t)1 << log_size;
    uint32_t *zero = nullptr, *layers = nullptr;
    int rc = zkb_malloc(ctx, n * 4, (void**)&zero);
    if (rc) return rc;
    rc = zkb_malloc(ctx, 2 * n * 4 * 4 / 2, (void**)&layers);  // two ping-pong secure layers of n / 2 rows
    if (rc) { zkb_free(ctx, zero); return rc; }
    auto fail = [&](int code) { zkb_free(ctx, zero); zkb_free(ctx, layers); return code; };
    if ((rc = zkb_memset_zero(ctx, zero, n * 4))) return fail(rc);
    if ((rc = zkb_memset_zero(ctx, layers, 2 * n * 4 * 4 / 2))) return fail(rc);
    const size_t half = n / 2;
    uint32_t* a[4] = {layers, layers + half, layers + 2 * half, layers + 3 * half};
    uint32_t* b[4] = {layers + 4 * half, layers + 5 * half, layers + 6 * half, layers + 7 * half};
    const uint32_t* src[4] = {d_evals, zero, zero, zero};  // the base-field evaluations as a secure column
    if ((rc = zkb_fold_circle_into_line(ctx, a, src, log_size, py.c))) return fail(rc);
    qm31 alpha = px;
    uint32_t** cur = a;
    uint32_t** nxt = b;
    for (int log = log_size - 1; log >= 1; log--) {
        const uint32_t* in[4] = {cur[0], cur[1], cur[2], cur[3]};
        if ((rc = zkb_fold_line(ctx, nxt, in, log, alpha.c))) return fail(rc);
        alpha = qm31_double_x(alpha);
        std::swap(cur, nxt);
    }
    uint32_t v[4];
    for (int k = 0; k < 4; k++)
        if ((rc = zkb_d2h(ctx, &v[k], cur[k], 4))) return fail(rc);
    const qm31 r = qm31_mul_m31(qm31{{v[0], v[1], v[2], v[3]}}, m31_inv(1u << log_size));
    memcpy(h_out, r.c, 16);
    return fail(ZKB_OK);
}

int zkb_fri_decompose(zkb_ctx* ctx, const uint32_t* const d_eval[4], int log_size, uint32_t* const d_out[4], uint32_t h_lambda[4]) {
    (void)d_eval; (void)log_size; (void)d_out; (void)h_lambda;
    if (!ctx) return ZKB_EINVAL;
    return set_error(ctx, ZKB_EINVAL,
                     "zkb_fri_decompose: FriOps::decompose is not used by the prover (every polynomial that enters FRI already lies in the "
                     "FFT space) and the reference's own device backend leaves it unimplemented; it is not provided");
}

}  // extern "C"
