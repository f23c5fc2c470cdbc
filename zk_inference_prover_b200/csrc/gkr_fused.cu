// Launch-count reductions for the GKR / sum-check loop, which is bound by launch and host
// round-trip latency, not by bandwidth (one layer of 2^24 fractions needs 276 rounds):
//
//  * fold_sum_kernel: MleOps::fix_first_variable on every column of a layer AND the next round's
//    sum_as_poly_in_first_variable sums, in one pass over the data. A round is then one launch and
//    one 32-byte read-back instead of three launches (nitroo/crates/stwo/src/prover/lookups/
//    sumcheck.rs:115-171 asks for the sums, draws the challenge, then fixes the variable; the sums
//    of the NEXT round only depend on the fixed layer, so they can be produced with it).
//  * gen_eq_evals as a product of two small tables instead of one launch per variable:
//    eq[x] = A[low bits of x] * B[high bits of x] (cpu/lookups/gkr.rs:216-231 doubles the table once
//    per variable; the values are the same field elements).
#include "common.cuh"

namespace zk {

__device__ __forceinline__ qm31 ldq2(const uint32_t* __restrict__ p, size_t i) {
    uint4 v = reinterpret_cast<const uint4*>(p)[i];
    return {{v.x, v.y, v.z, v.w}};
}
__device__ __forceinline__ void stq2(uint32_t* __restrict__ p, size_t i, qm31 v) {
    reinterpret_cast<uint4*>(p)[i] = make_uint4(v.c[0], v.c[1], v.c[2], v.c[3]);
}
__device__ __forceinline__ qm31 fold_q(qm31 r, qm31 a, qm31 b) { return qm31_add(qm31_mul(r, qm31_sub(b, a)), a); }

__device__ __forceinline__ qm31 warp_sum2(qm31 v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        qm31 o;
#pragma unroll
        for (int k = 0; k < 4; k++) o.c[k] = __shfl_down_sync(0xffffffffu, v.c[k], off);
        v = qm31_add(v, o);
    }
    return v;
}

// KIND is the INPUT layer's kind; LogUpMultiplicities folds into LogUpGeneric.
template <int KIND>
__global__ void __launch_bounds__(256) fold_sum_kernel(const uint32_t* __restrict__ num, const uint32_t* __restrict__ den, size_t n, qm31 r,
                                                       const uint32_t* __restrict__ eq_evals, qm31 lambda, uint32_t* __restrict__ num_out,
                                                       uint32_t* __restrict__ den_out, uint32_t* __restrict__ partials,
                                                       unsigned int* __restrict__ ticket, uint32_t* __restrict__ result,
                                                       const uint32_t* __restrict__ d_r = nullptr,
                                                       const uint32_t* __restrict__ d_lambda = nullptr) {
    if (d_r) r = ldq2(d_r, 0);  // challenges of a device-resident transcript
    if (d_lambda) lambda = ldq2(d_lambda, 0);
    const size_t half = n / 2, nt = half / 4;
    qm31 s0 = qm31_zero(), s2 = qm31_zero();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nt; i += (size_t)gridDim.x * blockDim.x) {
        const size_t o[4] = {2 * i, 2 * i + 1, 2 * (nt + i), 2 * (nt + i) + 1};
        qm31 d[4], nu[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            d[q] = fold_q(r, ldq2(den, o[q]), ldq2(den, o[q] + half));
            stq2(den_out, o[q], d[q]);
            if (KIND == ZKB_GKR_LOGUP_GENERIC) {
                nu[q] = fold_q(r, ldq2(num, o[q]), ldq2(num, o[q] + half));
                stq2(num_out, o[q], nu[q]);
            } else if (KIND == ZKB_GKR_LOGUP_MULTIPLICITIES) {
                uint32_t a = num[o[q]], b = num[o[q] + half];
                nu[q] = qm31_mul_m31(r, m31_sub(b, a));
                nu[q].c[0] = m31_add(nu[q].c[0], a);
                stq2(num_out, o[q], nu[q]);
            }
        }
        // round sums of the folded layer: values at (r', 0, i, {0,1}) = d[0], d[1]; (r', 1, i, {0,1}) = d[2], d[3]
        qm31 d20 = qm31_sub(qm31_dbl(d[2]), d[0]), d21 = qm31_sub(qm31_dbl(d[3]), d[1]);
        qm31 t0, t2;
        if (KIND == ZKB_GKR_GRAND_PRODUCT) {
            t0 = qm31_mul(d[0], d[1]);
            t2 = qm31_mul(d20, d21);
        } else {
            qm31 n0, n2;
            if (KIND == ZKB_GKR_LOGUP_SINGLES) {
                n0 = qm31_add(d[0], d[1]);
                n2 = qm31_add(d20, d21);
            } else {
                qm31 n20 = qm31_sub(qm31_dbl(nu[2]), nu[0]), n21 = qm31_sub(qm31_dbl(nu[3]), nu[1]);
                n0 = qm31_add(qm31_mul(d[1], nu[0]), qm31_mul(d[0], nu[1]));
                n2 = qm31_add(qm31_mul(d21, n20), qm31_mul(d20, n21));
            }
            t0 = qm31_add(n0, qm31_mul(lambda, qm31_mul(d[0], d[1])));
            t2 = qm31_add(n2, qm31_mul(lambda, qm31_mul(d20, d21)));
        }
        qm31 e = ldq2(eq_evals, i);
        s0 = qm31_add(s0, qm31_mul(e, t0));
        s2 = qm31_add(s2, qm31_mul(e, t2));
    }
    __shared__ uint32_t sh[8][8];
    __shared__ bool is_last;
    s0 = warp_sum2(s0);
    s2 = warp_sum2(s2);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < 4; k++) { sh[warp][k] = s0.c[k]; sh[warp][4 + k] = s2.c[k]; }
    }
    __syncthreads();
    if (threadIdx.x < 8) {
        uint32_t acc = 0;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) acc = m31_add(acc, sh[w][threadIdx.x]);
        partials[8 * blockIdx.x + threadIdx.x] = acc;
        __threadfence();
    }
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
    __syncthreads();
    if (is_last) {
        __threadfence();
        if (threadIdx.x < 8) {
            uint32_t acc = 0;
            for (unsigned b = 0; b < gridDim.x; b++) acc = m31_add(acc, __ldcg(&partials[8 * b + threadIdx.x]));
            result[threadIdx.x] = acc;
        }
        if (threadIdx.x == 0) *ticket = 0u;
    }
}

// table[x] = v * prod_k (bit k of x ? y_k : 1 - y_k), x < 2^m, m <= 11; ys[k] pairs with bit k. One CTA.
struct EqYs { qm31 y[12]; };
// With d_y, the variables come from device memory instead: step k uses d_y[ny - 1 - (first_bit + k)], and the
// scale is d_v (or one when d_v is null and use_one is set).
__global__ void __launch_bounds__(1024) eq_table_kernel(EqYs ys, int m, qm31 v, uint32_t* __restrict__ out,
                                                        const uint32_t* __restrict__ d_y = nullptr, int ny = 0, int first_bit = 0,
                                                        const uint32_t* __restrict__ d_v = nullptr) {
    __shared__ uint32_t s[4][2048];
    if (d_y) {
        for (int k = 0; k < m; k++) ys.y[k] = ldq2(d_y, ny - 1 - (first_bit + k));
        if (d_v) v = ldq2(d_v, 0);
    }
    if (threadIdx.x == 0) { s[0][0] = v.c[0]; s[1][0] = v.c[1]; s[2][0] = v.c[2]; s[3][0] = v.c[3]; }
    __syncthreads();
    // step k of the doubling appends index bit k
    for (int step = 0; step < m; step++) {
        const uint32_t len = 1u << step;
        const qm31 y = ys.y[step];
        for (uint32_t j = threadIdx.x; j < len; j += blockDim.x) {
            qm31 e{{s[0][j], s[1][j], s[2][j], s[3][j]}};
            qm31 t = qm31_mul(e, y);
            qm31 lo = qm31_sub(e, t);
            s[0][j] = lo.c[0]; s[1][j] = lo.c[1]; s[2][j] = lo.c[2]; s[3][j] = lo.c[3];
            s[0][j + len] = t.c[0]; s[1][j + len] = t.c[1]; s[2][j + len] = t.c[2]; s[3][j + len] = t.c[3];
        }
        __syncthreads();
    }
    for (uint32_t j = threadIdx.x; j < (1u << m); j += blockDim.x)
        reinterpret_cast<uint4*>(out)[j] = make_uint4(s[0][j], s[1][j], s[2][j], s[3][j]);
}

// out[x] = A[x & (2^a - 1)] * B[x >> a]
__global__ void __launch_bounds__(256) eq_product_kernel(const uint32_t* __restrict__ A, const uint32_t* __restrict__ B, int a, size_t n,
                                                         uint32_t* __restrict__ out) {
    size_t x = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (x >= n) return;
    stq2(out, x, qm31_mul(ldq2(A, x & (((size_t)1 << a) - 1)), ldq2(B, x >> a)));
}

int gkr_eq_evals_launch(zkb_ctx* ctx, const uint32_t* d_y, int ny, const uint32_t* d_v, uint32_t* out) {
    EqYs ys;
    memset(&ys, 0, sizeof(ys));
    auto table = [&](int first_bit, int bits, const uint32_t* dv, qm31 v, uint32_t* dst) {
        ProfScope prof(ctx, "eq_table_kernel");
        eq_table_kernel<<<1, bits >= 10 ? 1024 : (bits >= 5 ? 1 << bits : 32), 0, ctx->stream>>>(ys, bits, v, dst, d_y ? d_y : out, ny,
                                                                                                  first_bit, dv);
    };
    if (ny <= 11) {
        table(0, ny, d_v, qm31_one(), out);
        ZKB_LAUNCH_CHECK(ctx);
        return ZKB_OK;
    }
    if (ny > 22) return set_error(ctx, ZKB_EINVAL, "gkr_eq_evals: more than 22 variables");
    const int a = 11, b = ny - 11;
    uint32_t* A = ctx->scratch;
    uint32_t* B = ctx->scratch + (4u << 11);
    table(0, a, d_v, qm31_one(), A);
    table(a, b, nullptr, qm31_one(), B);
    size_t n = (size_t)1 << ny;
    {
        ProfScope prof(ctx, "eq_product_kernel");
        eq_product_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(A, B, a, n, out);
    }
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

int gkr_fold_sum_launch(zkb_ctx* ctx, int kind, const uint32_t* num, const uint32_t* den, size_t n, const uint32_t* d_r,
                        const uint32_t* eq_evals, const uint32_t* d_lambda, uint32_t* num_out, uint32_t* den_out, uint32_t* d_result) {
    const size_t nt = n / 8;
    unsigned blocks = (unsigned)((nt + 255) / 256);
    if (blocks > 148u * 8u) blocks = 148u * 8u;
    uint32_t* partials = ctx->scratch + (8u << 11);  // clear of the two eq tables
    qm31 z = qm31_zero();
    {
        ProfScope prof(ctx, "fold_sum_kernel");
        switch (kind) {
            case ZKB_GKR_GRAND_PRODUCT: fold_sum_kernel<0><<<blocks, 256, 0, ctx->stream>>>(num, den, n, z, eq_evals, z, num_out, den_out, partials, ctx->ticket, d_result, d_r, d_lambda); break;
            case ZKB_GKR_LOGUP_GENERIC: fold_sum_kernel<1><<<blocks, 256, 0, ctx->stream>>>(num, den, n, z, eq_evals, z, num_out, den_out, partials, ctx->ticket, d_result, d_r, d_lambda); break;
            case ZKB_GKR_LOGUP_MULTIPLICITIES: fold_sum_kernel<2><<<blocks, 256, 0, ctx->stream>>>(num, den, n, z, eq_evals, z, num_out, den_out, partials, ctx->ticket, d_result, d_r, d_lambda); break;
            default: fold_sum_kernel<3><<<blocks, 256, 0, ctx->stream>>>(num, den, n, z, eq_evals, z, num_out, den_out, partials, ctx->ticket, d_result, d_r, d_lambda); break;
        }
    }
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

}  // namespace zk

using namespace zk;

static inline qm31 qq4(const uint32_t* p) { return qm31{{p[0], p[1], p[2], p[3]}}; }

extern "C" {

int zkb_gkr_eq_evals(zkb_ctx* ctx, const uint32_t* h_y, int ny, const uint32_t h_v[4], uint32_t* out) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, ny >= 0 && ny <= 28 && h_v && out && (ny == 0 || h_y) && ((uintptr_t)out & 15) == 0);
    DeviceGuard g(ctx);
    // Index bit k pairs with y[ny-1-k]; the doubling of the reference appends one index bit per
    // variable, starting from y[ny-1] at bit 0.
    auto table = [&](int first_bit, int bits, qm31 v, uint32_t* dst) {
        EqYs ys;
        memset(&ys, 0, sizeof(ys));
        for (int k = 0; k < bits; k++) ys.y[k] = qq4(h_y + 4 * (ny - 1 - (first_bit + k)));
        ProfScope prof(ctx, "eq_table_kernel");
        eq_table_kernel<<<1, bits >= 10 ? 1024 : (bits >= 5 ? 1 << bits : 32), 0, ctx->stream>>>(ys, bits, v, dst);
    };
    if (ny <= 11) {
        table(0, ny, qq4(h_v), out);
        ZKB_LAUNCH_CHECK(ctx);
        return ZKB_OK;
    }
    ZKB_CHECK_ARG(ctx, ny <= 22);  // two tables of at most 2^11 entries
    const int a = 11, b = ny - 11;
    uint32_t* A = ctx->scratch;
    uint32_t* B = ctx->scratch + (4u << 11);
    table(0, a, qq4(h_v), A);
    table(a, b, qm31_one(), B);
    size_t n = (size_t)1 << ny;
    {
        ProfScope prof(ctx, "eq_product_kernel");
        eq_product_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(A, B, a, n, out);
    }
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

int zkb_gkr_fix_and_sum(zkb_ctx* ctx, int kind, const uint32_t* num, const uint32_t* den, size_t n, const uint32_t h_r[4],
                        const uint32_t* eq_evals, const uint32_t h_lambda[4], uint32_t* num_out, uint32_t* den_out, uint32_t h_out[8]) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, kind >= 0 && kind <= 3 && den && den_out && h_r && eq_evals && h_lambda && h_out);
    ZKB_CHECK_ARG(ctx, n >= 8 && (n & (n - 1)) == 0);
    const bool has_num = kind == ZKB_GKR_LOGUP_GENERIC || kind == ZKB_GKR_LOGUP_MULTIPLICITIES;
    ZKB_CHECK_ARG(ctx, !has_num || (num != nullptr && num_out != nullptr));
    ZKB_CHECK_ARG(ctx, ((uintptr_t)den & 15) == 0 && ((uintptr_t)den_out & 15) == 0 && ((uintptr_t)num_out & 15) == 0);
    DeviceGuard g(ctx);
    const size_t nt = n / 8;
    unsigned blocks = (unsigned)((nt + 255) / 256);
    if (blocks > 148u * 8u) blocks = 148u * 8u;
    uint32_t* partials = ctx->scratch;
    uint32_t* result = ctx->scratch + 8 * (size_t)blocks;
    qm31 r = qq4(h_r), lam = qq4(h_lambda);
    {
        ProfScope prof(ctx, "fold_sum_kernel");
        switch (kind) {
            case ZKB_GKR_GRAND_PRODUCT: fold_sum_kernel<0><<<blocks, 256, 0, ctx->stream>>>(num, den, n, r, eq_evals, lam, num_out, den_out, partials, ctx->ticket, result); break;
            case ZKB_GKR_LOGUP_GENERIC: fold_sum_kernel<1><<<blocks, 256, 0, ctx->stream>>>(num, den, n, r, eq_evals, lam, num_out, den_out, partials, ctx->ticket, result); break;
            case ZKB_GKR_LOGUP_MULTIPLICITIES: fold_sum_kernel<2><<<blocks, 256, 0, ctx->stream>>>(num, den, n, r, eq_evals, lam, num_out, den_out, partials, ctx->ticket, result); break;
            default: fold_sum_kernel<3><<<blocks, 256, 0, ctx->stream>>>(num, den, n, r, eq_evals, lam, num_out, den_out, partials, ctx->ticket, result); break;
        }
    }
    ZKB_LAUNCH_CHECK(ctx);
    ZKB_CUDA(ctx, cudaMemcpyAsync(ctx->h_small, result, 32, cudaMemcpyDeviceToHost, ctx->stream));
    ZKB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    memcpy(h_out, ctx->h_small, 32);
    return ZKB_OK;
}

}  // extern "C"
