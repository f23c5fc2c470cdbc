// FriOps: fold_line and fold_circle_into_line on secure columns in coordinate layout.
//
// Both fold adjacent pairs (2i, 2i+1) of a bit-reversed evaluation:
//   f0 = a + b,  f1 = (a - b) * t^-1,  folded = f0 + alpha * f1
// with t the x-coordinate (line) or y-coordinate (circle) of the pair's domain point
// (nitroo/crates/stwo/src/prover/backend/cpu/fri.rs:67-123). The inverse coordinates come from the
// inverse twiddle tower: pair i of the line domain Coset::half_odds(k) uses T_k^-1[i]; pair i of
// the canonic circle domain of log size L uses the y of point i of Coset::half_odds(L-1).
#include "blake2s.cuh"
#include "common.cuh"

namespace zk {

struct Secure4 { uint32_t* c[4]; };
struct Secure4C { const uint32_t* c[4]; };

__device__ __forceinline__ qm31 fold_pair(const Secure4C& in, size_t i, uint32_t itw, qm31 alpha) {
    qm31 a, b;
#pragma unroll
    for (int k = 0; k < 4; k++) {
        uint2 v = reinterpret_cast<const uint2*>(in.c[k])[i];
        a.c[k] = v.x;
        b.c[k] = v.y;
    }
    qm31 f0 = qm31_add(a, b);
    qm31 f1 = qm31_mul_m31(qm31_sub(a, b), itw);
    return qm31_add(f0, qm31_mul(alpha, f1));
}

// The folding challenge comes by value or, when d_alpha is given, from device memory (written by the
// channel kernel of the previous step, so that a whole FRI commit phase runs without a host round trip).
__device__ __forceinline__ qm31 load_alpha(const uint32_t* __restrict__ d_alpha, qm31 alpha) {
    if (d_alpha) {
        uint4 v = *reinterpret_cast<const uint4*>(d_alpha);
        return qm31{{v.x, v.y, v.z, v.w}};
    }
    return alpha;
}

// The folded value is the next FRI layer's Merkle leaf (its four coordinates are the layer's four columns,
// prover/fri.rs:169-188): hashing it here saves the leaf launch and the re-read of the layer.
__device__ __forceinline__ void store_leaf(uint32_t* __restrict__ leaves, size_t i, qm31 r) {
    uint32_t h[8], m[16];
    blake2s_init(h);
#pragma unroll
    for (int k = 0; k < 4; k++) m[k] = r.c[k];
#pragma unroll
    for (int k = 4; k < 16; k++) m[k] = 0u;
    blake2s_compress(h, m, 16u, true);
    uint4* o = reinterpret_cast<uint4*>(leaves + 8 * i);
    o[0] = make_uint4(reduce_word_m31(h[0]), reduce_word_m31(h[1]), reduce_word_m31(h[2]), reduce_word_m31(h[3]));
    o[1] = make_uint4(reduce_word_m31(h[4]), reduce_word_m31(h[5]), reduce_word_m31(h[6]), reduce_word_m31(h[7]));
}

__global__ void __launch_bounds__(256) fold_line_kernel(Secure4 out, Secure4C in, int log_n, qm31 alpha,
                                                        const uint32_t* __restrict__ d_alpha, const uint32_t* __restrict__ itw,
                                                        uint32_t* __restrict__ leaves = nullptr) {
    alpha = load_alpha(d_alpha, alpha);
    size_t half = (size_t)1 << (log_n - 1);
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= half) return;
    uint32_t t = itw[half + i];  // T_k^-1 starts at 2^(k-1)
    qm31 r = fold_pair(in, i, t, alpha);
#pragma unroll
    for (int k = 0; k < 4; k++) out.c[k][i] = r.c[k];
    if (leaves) store_leaf(leaves, i, r);
}

// Two output elements per thread: one 16-byte load per coordinate column brings both pairs, and twice the bytes
// are in flight per thread (these kernels wait on memory, not on arithmetic).
__device__ __forceinline__ void fold_pair2(const Secure4C& in, size_t i2, uint32_t t0, uint32_t t1, qm31 alpha, qm31& r0, qm31& r1) {
    qm31 a0, b0, a1, b1;
#pragma unroll
    for (int k = 0; k < 4; k++) {
        uint4 v = reinterpret_cast<const uint4*>(in.c[k])[i2];
        a0.c[k] = v.x; b0.c[k] = v.y; a1.c[k] = v.z; b1.c[k] = v.w;
    }
    r0 = qm31_add(qm31_add(a0, b0), qm31_mul(alpha, qm31_mul_m31(qm31_sub(a0, b0), t0)));
    r1 = qm31_add(qm31_add(a1, b1), qm31_mul(alpha, qm31_mul_m31(qm31_sub(a1, b1), t1)));
}

__global__ void __launch_bounds__(256) fold_line_kernel2(Secure4 out, Secure4C in, int log_n, qm31 alpha,
                                                         const uint32_t* __restrict__ d_alpha, const uint32_t* __restrict__ itw,
                                                         uint32_t* __restrict__ leaves) {
    alpha = load_alpha(d_alpha, alpha);
    const size_t half = (size_t)1 << (log_n - 1);
    const size_t i2 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (2 * i2 >= half) return;
    const uint2 t = reinterpret_cast<const uint2*>(itw + half)[i2];
    qm31 r0, r1;
    fold_pair2(in, i2, t.x, t.y, alpha, r0, r1);
#pragma unroll
    for (int k = 0; k < 4; k++) reinterpret_cast<uint2*>(out.c[k])[i2] = make_uint2(r0.c[k], r1.c[k]);
    if (leaves) { store_leaf(leaves, 2 * i2, r0); store_leaf(leaves, 2 * i2 + 1, r1); }
}

// Four output elements per thread (the variant without leaf hashing): eight 16-byte loads in flight per thread and one
// 16-byte store per coordinate column. A fold moves 26 (line) or 34 (circle) bytes per output pair and does about 60
// instructions for them; what limits it is the number of bytes each thread keeps in flight.
__device__ __forceinline__ void fold_quad(const Secure4C& in, size_t i4, const uint32_t t[4], qm31 alpha, qm31 r[4]) {
    qm31 a[4], b[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const uint4 v = reinterpret_cast<const uint4*>(in.c[k])[2 * i4], w = reinterpret_cast<const uint4*>(in.c[k])[2 * i4 + 1];
        a[0].c[k] = v.x; b[0].c[k] = v.y; a[1].c[k] = v.z; b[1].c[k] = v.w;
        a[2].c[k] = w.x; b[2].c[k] = w.y; a[3].c[k] = w.z; b[3].c[k] = w.w;
    }
#pragma unroll
    for (int e = 0; e < 4; e++) r[e] = qm31_add(qm31_add(a[e], b[e]), qm31_mul(alpha, qm31_mul_m31(qm31_sub(a[e], b[e]), t[e])));
}

__global__ void __launch_bounds__(256) fold_line_kernel4(Secure4 out, Secure4C in, int log_n, qm31 alpha,
                                                         const uint32_t* __restrict__ d_alpha, const uint32_t* __restrict__ itw) {
    alpha = load_alpha(d_alpha, alpha);
    const size_t half = (size_t)1 << (log_n - 1);
    const size_t i4 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (4 * i4 >= half) return;
    const uint4 tw = reinterpret_cast<const uint4*>(itw + half)[i4];
    const uint32_t t[4] = {tw.x, tw.y, tw.z, tw.w};
    qm31 r[4];
    fold_quad(in, i4, t, alpha, r);
#pragma unroll
    for (int k = 0; k < 4; k++) reinterpret_cast<uint4*>(out.c[k])[i4] = make_uint4(r[0].c[k], r[1].c[k], r[2].c[k], r[3].c[k]);
}

__global__ void __launch_bounds__(256) fold_circle_kernel4(Secure4 dst, Secure4C src, int log_n_src, qm31 alpha,
                                                           const uint32_t* __restrict__ d_alpha, const uint32_t* __restrict__ itw) {
    alpha = load_alpha(d_alpha, alpha);
    const qm31 alpha_sq = qm31_sqr(alpha);
    const size_t half = (size_t)1 << (log_n_src - 1);
    const size_t i4 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (4 * i4 >= half) return;
    uint32_t ix, t[4];
#pragma unroll
    for (int e = 0; e < 4; e++) half_coset_point(itw, log_n_src, (uint32_t)(4 * i4 + e), ix, t[e]);
    qm31 f[4];
    fold_quad(src, i4, t, alpha, f);
    uint4 d[4];
#pragma unroll
    for (int k = 0; k < 4; k++) d[k] = reinterpret_cast<const uint4*>(dst.c[k])[i4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const qm31 de{{(&d[0].x)[e], (&d[1].x)[e], (&d[2].x)[e], (&d[3].x)[e]}};
        f[e] = qm31_add(qm31_mul(de, alpha_sq), f[e]);
    }
#pragma unroll
    for (int k = 0; k < 4; k++) reinterpret_cast<uint4*>(dst.c[k])[i4] = make_uint4(f[0].c[k], f[1].c[k], f[2].c[k], f[3].c[k]);
}

__global__ void __launch_bounds__(256) fold_circle_kernel2(Secure4 dst, Secure4C src, int log_n_src, qm31 alpha,
                                                           const uint32_t* __restrict__ d_alpha, const uint32_t* __restrict__ itw,
                                                           uint32_t* __restrict__ leaves) {
    alpha = load_alpha(d_alpha, alpha);
    const qm31 alpha_sq = qm31_sqr(alpha);
    const size_t half = (size_t)1 << (log_n_src - 1);
    const size_t i2 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (2 * i2 >= half) return;
    uint32_t ix, iy0, iy1;
    half_coset_point(itw, log_n_src, (uint32_t)(2 * i2), ix, iy0);
    half_coset_point(itw, log_n_src, (uint32_t)(2 * i2 + 1), ix, iy1);
    qm31 f0, f1;
    fold_pair2(src, i2, iy0, iy1, alpha, f0, f1);
    qm31 d0, d1;
#pragma unroll
    for (int k = 0; k < 4; k++) {
        uint2 v = reinterpret_cast<const uint2*>(dst.c[k])[i2];
        d0.c[k] = v.x; d1.c[k] = v.y;
    }
    const qm31 r0 = qm31_add(qm31_mul(d0, alpha_sq), f0), r1 = qm31_add(qm31_mul(d1, alpha_sq), f1);
#pragma unroll
    for (int k = 0; k < 4; k++) reinterpret_cast<uint2*>(dst.c[k])[i2] = make_uint2(r0.c[k], r1.c[k]);
    if (leaves) { store_leaf(leaves, 2 * i2, r0); store_leaf(leaves, 2 * i2 + 1, r1); }
}

// log_n == 1, 2 of the line fold and small circle domains need points that are not in the tower
// (T_k holds only half of each coset and starts at k = 1); they are passed in by the host.
__global__ void fold_small_kernel(Secure4 out, Secure4C in, int n_out, qm31 alpha, const uint32_t* __restrict__ d_alpha,
                                  int accumulate, uint32_t it0, uint32_t it1, uint32_t it2, uint32_t it3) {
    alpha = load_alpha(d_alpha, alpha);
    const qm31 alpha_sq = qm31_sqr(alpha);
    int i = threadIdx.x;
    if (i >= n_out) return;
    uint32_t its[4] = {it0, it1, it2, it3};
    qm31 r = fold_pair(in, i, its[i], alpha);
    if (accumulate) {
        qm31 d{{out.c[0][i], out.c[1][i], out.c[2][i], out.c[3][i]}};
        r = qm31_add(qm31_mul(d, alpha_sq), r);
    }
#pragma unroll
    for (int k = 0; k < 4; k++) out.c[k][i] = r.c[k];
}

__global__ void __launch_bounds__(256) fold_circle_kernel(Secure4 dst, Secure4C src, int log_n_src, qm31 alpha,
                                                          const uint32_t* __restrict__ d_alpha, const uint32_t* __restrict__ itw,
                                                          uint32_t* __restrict__ leaves = nullptr) {
    alpha = load_alpha(d_alpha, alpha);
    const qm31 alpha_sq = qm31_sqr(alpha);
    size_t half = (size_t)1 << (log_n_src - 1);
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= half) return;
    uint32_t ix, iy;
    half_coset_point(itw, log_n_src, (uint32_t)i, ix, iy);
    qm31 f = fold_pair(src, i, iy, alpha);
    qm31 d{{dst.c[0][i], dst.c[1][i], dst.c[2][i], dst.c[3][i]}};
    qm31 r = qm31_add(qm31_mul(d, alpha_sq), f);
#pragma unroll
    for (int k = 0; k < 4; k++) dst.c[k][i] = r.c[k];
    if (leaves) store_leaf(leaves, i, r);
}

}  // namespace zk

using namespace zk;

// Host-side point of the order-2^31 group: index -> (x, y).
static cpoint host_point(uint32_t index) {
    cpoint g{2u, 1268011823u}, r{1u, 0u};
    for (int b = 0; b < 31; b++) {
        if ((index >> b) & 1u) r = cpoint_add(r, g);
        g = cpoint_add(g, g);
    }
    return r;
}
static uint32_t host_bitrev(uint32_t i, int bits) {
    uint32_t r = 0;
    for (int b = 0; b < bits; b++) r |= ((i >> b) & 1u) << (bits - 1 - b);
    return r;
}

static int fold_line_impl(zkb_ctx* ctx, uint32_t* const out[4], const uint32_t* const in[4], int log_n,
                          const uint32_t* h_alpha, const uint32_t* d_alpha, uint32_t* leaves = nullptr) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, out && in && (h_alpha || d_alpha) && log_n >= 1 && log_n <= ctx->max_log - 1);
    ZKB_CHECK_ARG(ctx, ((uintptr_t)d_alpha & 15) == 0);
    Secure4 o;
    Secure4C s;
    for (int k = 0; k < 4; k++) {
        ZKB_CHECK_ARG(ctx, out[k] != nullptr && in[k] != nullptr && ((uintptr_t)in[k] & 7) == 0);
        o.c[k] = out[k];
        s.c[k] = in[k];
    }
    qm31 alpha = qm31_zero();
    if (h_alpha) alpha = qm31{{h_alpha[0], h_alpha[1], h_alpha[2], h_alpha[3]}};
    DeviceGuard g(ctx);
    size_t half = (size_t)1 << (log_n - 1);
    bool wide = log_n >= 3;
    for (int k = 0; k < 4; k++) wide = wide && ((uintptr_t)in[k] & 15) == 0 && ((uintptr_t)out[k] & 7) == 0;
    ProfScope prof(ctx, "fold_line_kernel");
    bool quad = wide && log_n >= 4 && !leaves;
    for (int k = 0; k < 4; k++) quad = quad && ((uintptr_t)out[k] & 15) == 0;
    if (quad)
        fold_line_kernel4<<<(unsigned)((half / 4 + 255) / 256), 256, 0, ctx->stream>>>(o, s, log_n, alpha, d_alpha, ctx->itw);
    else if (wide)
        fold_line_kernel2<<<(unsigned)((half / 2 + 255) / 256), 256, 0, ctx->stream>>>(o, s, log_n, alpha, d_alpha, ctx->itw, leaves);
    else
        fold_line_kernel<<<(unsigned)((half + 255) / 256), 256, 0, ctx->stream>>>(o, s, log_n, alpha, d_alpha, ctx->itw, leaves);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

static int fold_circle_impl(zkb_ctx* ctx, uint32_t* const dst[4], const uint32_t* const src[4], int log_n_src,
                            const uint32_t* h_alpha, const uint32_t* d_alpha, uint32_t* leaves = nullptr) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, dst && src && (h_alpha || d_alpha) && log_n_src >= 1 && log_n_src <= ctx->max_log);
    ZKB_CHECK_ARG(ctx, ((uintptr_t)d_alpha & 15) == 0);
    Secure4 o;
    Secure4C s;
    for (int k = 0; k < 4; k++) {
        ZKB_CHECK_ARG(ctx, dst[k] != nullptr && src[k] != nullptr && ((uintptr_t)src[k] & 7) == 0);
        o.c[k] = dst[k];
        s.c[k] = src[k];
    }
    qm31 alpha = qm31_zero();
    if (h_alpha) alpha = qm31{{h_alpha[0], h_alpha[1], h_alpha[2], h_alpha[3]}};
    DeviceGuard g(ctx);
    if (log_n_src <= 2 && leaves) return set_error(ctx, ZKB_EINVAL, "fold with leaf hashing needs at least 8 source points");
    if (log_n_src <= 2) {
        // Points i of Coset::half_odds(log_n_src - 1), bit-reversed: index 2^(31-(L-1)-2) + j * 2^(31-(L-1)).
        int hl = log_n_src - 1;
        uint32_t it[4] = {0, 0, 0, 0};
        for (uint32_t i = 0; i < (1u << hl); i++) {
            uint32_t j = host_bitrev(i, hl);
            cpoint p = host_point(((1u << (29 - hl)) + (j << (31 - hl))) & 0x7fffffffu);
            it[i] = m31_inv(p.y);
        }
        fold_small_kernel<<<1, 32, 0, ctx->stream>>>(o, s, 1 << hl, alpha, d_alpha, 1, it[0], it[1], it[2], it[3]);
        ZKB_LAUNCH_CHECK(ctx);
        return ZKB_OK;
    }
    size_t half = (size_t)1 << (log_n_src - 1);
    bool wide = log_n_src >= 4;
    for (int k = 0; k < 4; k++) wide = wide && ((uintptr_t)src[k] & 15) == 0 && ((uintptr_t)dst[k] & 7) == 0;
    ProfScope prof(ctx, "fold_circle_kernel");
    bool quad = wide && log_n_src >= 5 && !leaves;
    for (int k = 0; k < 4; k++) quad = quad && ((uintptr_t)dst[k] & 15) == 0;
    if (quad)
        fold_circle_kernel4<<<(unsigned)((half / 4 + 255) / 256), 256, 0, ctx->stream>>>(o, s, log_n_src, alpha, d_alpha, ctx->itw);
    else if (wide)
        fold_circle_kernel2<<<(unsigned)((half / 2 + 255) / 256), 256, 0, ctx->stream>>>(o, s, log_n_src, alpha, d_alpha, ctx->itw, leaves);
    else
        fold_circle_kernel<<<(unsigned)((half + 255) / 256), 256, 0, ctx->stream>>>(o, s, log_n_src, alpha, d_alpha, ctx->itw, leaves);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

extern "C" {

int zkb_fold_line(zkb_ctx* ctx, uint32_t* const out[4], const uint32_t* const in[4], int log_n, const uint32_t h_alpha[4]) {
    if (ctx && !h_alpha) return zk::set_error(ctx, ZKB_EINVAL, "zkb_fold_line: null alpha");
    return fold_line_impl(ctx, out, in, log_n, h_alpha, nullptr);
}
int zkb_fold_line_dalpha(zkb_ctx* ctx, uint32_t* const out[4], const uint32_t* const in[4], int log_n, const uint32_t* d_alpha) {
    if (ctx && !d_alpha) return zk::set_error(ctx, ZKB_EINVAL, "zkb_fold_line_dalpha: null alpha");
    return fold_line_impl(ctx, out, in, log_n, nullptr, d_alpha);
}
int zkb_fold_circle_into_line(zkb_ctx* ctx, uint32_t* const dst[4], const uint32_t* const src[4], int log_n_src,
                              const uint32_t h_alpha[4]) {
    if (ctx && !h_alpha) return zk::set_error(ctx, ZKB_EINVAL, "zkb_fold_circle_into_line: null alpha");
    return fold_circle_impl(ctx, dst, src, log_n_src, h_alpha, nullptr);
}
int zkb_fold_circle_into_line_dalpha(zkb_ctx* ctx, uint32_t* const dst[4], const uint32_t* const src[4], int log_n_src,
                                     const uint32_t* d_alpha) {
    if (ctx && !d_alpha) return zk::set_error(ctx, ZKB_EINVAL, "zkb_fold_circle_into_line_dalpha: null alpha");
    return fold_circle_impl(ctx, dst, src, log_n_src, nullptr, d_alpha);
}

int zkb_fold_line_dalpha_leaves(zkb_ctx* ctx, uint32_t* const out[4], const uint32_t* const in[4], int log_n, const uint32_t* d_alpha,
                                uint32_t* leaves) {
    if (ctx && (!d_alpha || !leaves || ((uintptr_t)leaves & 15))) return zk::set_error(ctx, ZKB_EINVAL, "zkb_fold_line_dalpha_leaves: bad argument");
    return fold_line_impl(ctx, out, in, log_n, nullptr, d_alpha, leaves);
}
int zkb_fold_circle_into_line_dalpha_leaves(zkb_ctx* ctx, uint32_t* const dst[4], const uint32_t* const src[4], int log_n_src,
                                            const uint32_t* d_alpha, uint32_t* leaves) {
    if (ctx && (!d_alpha || !leaves || ((uintptr_t)leaves & 15))) return zk::set_error(ctx, ZKB_EINVAL, "zkb_fold_circle_into_line_dalpha_leaves: bad argument");
    return fold_circle_impl(ctx, dst, src, log_n_src, nullptr, d_alpha, leaves);
}

}  // extern "C"
