// QuotientOps and AccumulationOps.
//
// accumulate_numerators, per row: sum_j (c_j * col_{idx_j}[row] - b_j) with QM31 coefficients and
// M31 column values (nitroo/crates/stwo/src/core/pcs/quotients.rs:217-229). The b_j do not depend
// on the row, so their sum is taken once on the host; the c_j * value products are accumulated
// unreduced in 64 bits (four 62-bit products fit) and folded every four columns.
//
// compute_quotients_and_combine, per row: sum over sample points z of
//   (acc_z[lift(row)] - A_z * p.y) * ((Re z.x - p.x) * Im z.y - (Re z.y - p.y) * Im z.x)^-1
// with p the row's domain point (prover/backend/cpu/quotients.rs:47-75). p comes from the twiddle
// tower; the CM31 inverses of one row are taken with one M31 inversion (Montgomery's trick on the
// norms), which is exact because inverses are unique.
#include <vector>

#include "common.cuh"

namespace zk {

struct Secure4 { uint32_t* c[4]; };
struct Secure4C { const uint32_t* c[4]; };

// Partially folds a 64-bit accumulator to below 2^34 without changing its residue.
__device__ __forceinline__ uint64_t fold64(uint64_t v) { return (v & P) + (v >> 31); }

// R consecutive rows per thread (one 8- or 16-byte load per column). The column addresses and the
// coefficients of a tile of columns are resolved once per CTA into shared memory, so the inner loop
// is one independent streaming load per column and 4 R multiply-adds: the kernel is bound by HBM.
constexpr int NUM_TILE = 128;

template <int R>
__global__ void __launch_bounds__(256) quot_numerators_kernel(const uint32_t* const* __restrict__ cols,
                                                              const uint32_t* __restrict__ col_idx,
                                                              const uint4* __restrict__ coeff_c, int k, qm31 b_sum,
                                                              size_t n, Secure4 out, int chunk = 0,
                                                              uint32_t* __restrict__ partial = nullptr) {
    // With `partial`, CTA row blockIdx.y takes the columns [y * chunk, (y + 1) * chunk) and leaves its reduced sums in
    // partial[(y * 4 + coordinate) * n + row]; quot_partial_sum_kernel adds the rows up. Short, wide groups (thousands of
    // columns of a few hundred rows) would otherwise run on one or two CTAs.
    const int k_begin = partial ? (int)blockIdx.y * chunk : 0;
    const int k_end = partial ? (k_begin + chunk < k ? k_begin + chunk : k) : k;
    __shared__ const uint32_t* s_col[NUM_TILE];
    __shared__ uint4 s_c[NUM_TILE];
    const size_t row0 = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * R;
    const bool live = row0 < n;
    uint64_t acc[R][4];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int q = 0; q < 4; q++) acc[r][q] = 0;
    auto load = [&](const uint32_t* col, uint32_t (&v)[R]) {
        if constexpr (R == 4) {
            uint4 x = __ldcs(reinterpret_cast<const uint4*>(col + row0));
            v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
        } else {
            uint2 x = __ldcs(reinterpret_cast<const uint2*>(col + row0));
            v[0] = x.x; v[1] = x.y;
        }
    };
    auto mac = [&](const uint4& c, const uint32_t (&v)[R]) {
#pragma unroll
        for (int r = 0; r < R; r++) {
            acc[r][0] += (uint64_t)c.x * v[r]; acc[r][1] += (uint64_t)c.y * v[r];
            acc[r][2] += (uint64_t)c.z * v[r]; acc[r][3] += (uint64_t)c.w * v[r];
        }
    };
    for (int tile0 = k_begin; tile0 < k_end; tile0 += NUM_TILE) {
        const int tk = k_end - tile0 < NUM_TILE ? k_end - tile0 : NUM_TILE;
        __syncthreads();
        if ((int)threadIdx.x < tk) {
            s_col[threadIdx.x] = cols[col_idx[tile0 + threadIdx.x]];
            s_c[threadIdx.x] = coeff_c[tile0 + threadIdx.x];
        }
        __syncthreads();
        if (!live) continue;
        int j = 0;
        for (; j + 4 <= tk; j += 4) {
            uint32_t v[4][R];
#pragma unroll
            for (int u = 0; u < 4; u++) load(s_col[j + u], v[u]);
#pragma unroll
            for (int u = 0; u < 4; u++) mac(s_c[j + u], v[u]);
            // four 62-bit products on top of a folded (< 2^34) accumulator fit in 64 bits
#pragma unroll
            for (int r = 0; r < R; r++)
#pragma unroll
                for (int q = 0; q < 4; q++) acc[r][q] = fold64(acc[r][q]);
        }
        for (; j < tk; j++) {  // at most 3 tail products
            uint32_t v[R];
            load(s_col[j], v);
            mac(s_c[j], v);
        }
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int q = 0; q < 4; q++) acc[r][q] = fold64(acc[r][q]);
    }
    if (!live) return;
    uint32_t res[R][4];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int q = 0; q < 4; q++) res[r][q] = partial ? m31_reduce64(acc[r][q]) : m31_sub(m31_reduce64(acc[r][q]), b_sum.c[q]);
    if (partial) {
#pragma unroll
        for (int q = 0; q < 4; q++) {
            uint32_t* dst = partial + ((size_t)blockIdx.y * 4 + q) * n + row0;
            if constexpr (R == 4) *reinterpret_cast<uint4*>(dst) = make_uint4(res[0][q], res[1][q], res[2][q], res[3][q]);
            else *reinterpret_cast<uint2*>(dst) = make_uint2(res[0][q], res[1][q]);
        }
        return;
    }
#pragma unroll
    for (int q = 0; q < 4; q++) {
        if constexpr (R == 4) *reinterpret_cast<uint4*>(out.c[q] + row0) = make_uint4(res[0][q], res[1][q], res[2][q], res[3][q]);
        else *reinterpret_cast<uint2*>(out.c[q] + row0) = make_uint2(res[0][q], res[1][q]);
    }
}

// out[q][row] = sum over the S column chunks of partial[(s * 4 + q) * n + row], minus b_sum.
__global__ void __launch_bounds__(256) quot_partial_sum_kernel(const uint32_t* __restrict__ partial, int S, size_t n, qm31 b_sum, Secure4 out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // over 4 * n (coordinate-major)
    if (i >= 4 * n) return;
    const int q = (int)(i / n);
    const size_t row = i - (size_t)q * n;
    uint64_t acc = 0;
    for (int s = 0; s < S; s++) acc += partial[((size_t)s * 4 + q) * n + row];  // 31-bit terms: the 64-bit sum cannot overflow
    out.c[q][row] = m31_sub(m31_reduce64(acc), b_sum.c[q]);
}

constexpr int MAX_ACCS = 8;
struct CombineArgs {
    const uint32_t* acc[MAX_ACCS][4];
    int log_ratio[MAX_ACCS];
    qm31 first_lin[MAX_ACCS];
    cm31 prx[MAX_ACCS], pry[MAX_ACCS], pix[MAX_ACCS], piy[MAX_ACCS];
    int n_acc;
    int first;  // 1: overwrite out, 0: add to out (more than MAX_ACCS accumulations)
};

// Rows [row_begin, row_begin + n_rows) of the lifting domain; the accumulations and `out` are indexed from row_begin
// (a row shard holds only its own rows; the whole domain is row_begin = 0, n_rows = 2^lifting_log).
__global__ void __launch_bounds__(256) quot_combine_kernel(CombineArgs a, int lifting_log, Secure4 out,
                                                           const uint32_t* __restrict__ tw, size_t row_begin, size_t n_rows) {
    const size_t local = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (local >= n_rows) return;
    const size_t row = row_begin + local;
    uint32_t px, py;
    half_coset_point(tw, lifting_log, (uint32_t)(row >> 1), px, py);
    if (row & 1) py = m31_neg(py);  // odd rows hold the conjugate point
    cm31 den[MAX_ACCS];
    uint32_t norm[MAX_ACCS], pref[MAX_ACCS];
    uint32_t run = 1u;
#pragma unroll
    for (int z = 0; z < MAX_ACCS; z++) {
        if (z < a.n_acc) {
            cm31 dx = {m31_sub(a.prx[z].a, px), a.prx[z].b};
            cm31 dy = {m31_sub(a.pry[z].a, py), a.pry[z].b};
            den[z] = cm31_sub(cm31_mul(dx, a.piy[z]), cm31_mul(dy, a.pix[z]));
            norm[z] = m31_reduce64((uint64_t)den[z].a * den[z].a + (uint64_t)den[z].b * den[z].b);
            pref[z] = run;
            run = m31_mul(run, norm[z]);
        }
    }
    uint32_t inv = m31_inv(run);
    qm31 q = qm31_zero();
#pragma unroll
    for (int z = MAX_ACCS - 1; z >= 0; z--) {
        if (z < a.n_acc) {
            uint32_t ninv = m31_mul(inv, pref[z]);
            inv = m31_mul(inv, norm[z]);
            cm31 dinv = {m31_mul(den[z].a, ninv), m31_mul(m31_neg(den[z].b), ninv)};
            const size_t li = ((row >> (a.log_ratio[z] + 1)) << 1) + (row & 1) - (((row_begin >> (a.log_ratio[z] + 1)) << 1));
            qm31 num{{a.acc[z][0][li], a.acc[z][1][li], a.acc[z][2][li], a.acc[z][3][li]}};
            num = qm31_sub(num, qm31_mul_m31(a.first_lin[z], py));
            q = qm31_add(q, qm31_mul_cm31(num, dinv));
        }
    }
    if (!a.first) {
        qm31 o{{out.c[0][local], out.c[1][local], out.c[2][local], out.c[3][local]}};
        q = qm31_add(q, o);
    }
#pragma unroll
    for (int k = 0; k < 4; k++) out.c[k][local] = q.c[k];
}

// Slow path for lifting domains of log size 1 and 2, whose points are not in the tower.
__global__ void quot_combine_small_kernel(CombineArgs a, int lifting_log, Secure4 out, uint32_t x0, uint32_t y0,
                                          uint32_t x1, uint32_t y1) {
    int row = threadIdx.x;
    if (row >= (1 << lifting_log)) return;
    uint32_t px = (row >> 1) ? x1 : x0, py = (row >> 1) ? y1 : y0;
    if (row & 1) py = m31_neg(py);
    qm31 q = qm31_zero();
    for (int z = 0; z < a.n_acc; z++) {
        cm31 dx = {m31_sub(a.prx[z].a, px), a.prx[z].b};
        cm31 dy = {m31_sub(a.pry[z].a, py), a.pry[z].b};
        cm31 dinv = cm31_inv(cm31_sub(cm31_mul(dx, a.piy[z]), cm31_mul(dy, a.pix[z])));
        int li = ((row >> (a.log_ratio[z] + 1)) << 1) + (row & 1);
        qm31 num{{a.acc[z][0][li], a.acc[z][1][li], a.acc[z][2][li], a.acc[z][3][li]}};
        num = qm31_sub(num, qm31_mul_m31(a.first_lin[z], py));
        q = qm31_add(q, qm31_mul_cm31(num, dinv));
    }
    if (!a.first) {
        qm31 o{{out.c[0][row], out.c[1][row], out.c[2][row], out.c[3][row]}};
        q = qm31_add(q, o);
    }
    for (int k = 0; k < 4; k++) out.c[k][row] = q.c[k];
}

__global__ void __launch_bounds__(256) accumulate_kernel(Secure4 col, Secure4C other, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
#pragma unroll
    for (int k = 0; k < 4; k++) col.c[k][i] = m31_add(col.c[k][i], other.c[k][i]);
}

__global__ void __launch_bounds__(256) lift_accumulate_kernel(Secure4 dst, int log_dst, Secure4C src, int log_ratio) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= ((size_t)1 << log_dst)) return;
    size_t li = ((i >> (log_ratio + 1)) << 1) + (i & 1);
#pragma unroll
    for (int k = 0; k < 4; k++) dst.c[k][i] = m31_add(dst.c[k][i], src.c[k][li]);
}

}  // namespace zk

using namespace zk;

static cpoint host_point_q(uint32_t index) {
    cpoint g{2u, 1268011823u}, r{1u, 0u};
    for (int b = 0; b < 31; b++) {
        if ((index >> b) & 1u) r = cpoint_add(r, g);
        g = cpoint_add(g, g);
    }
    return r;
}

extern "C" {

int zkb_quot_numerators(zkb_ctx* ctx, const uint32_t* const* cols, int ncols, int log_n, const uint32_t* h_col_idx,
                        const uint32_t* h_b, const uint32_t* h_c, int k, uint32_t* const out[4]) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, cols && ncols > 0 && log_n >= 1 && log_n <= 30 && k >= 0 && out);
    ZKB_CHECK_ARG(ctx, k == 0 || (h_col_idx && h_b && h_c));
    ZKB_CHECK_ARG(ctx, (size_t)k * 5 <= ctx->scratch_words);
    Secure4 o;
    for (int q = 0; q < 4; q++) {
        ZKB_CHECK_ARG(ctx, out[q] != nullptr && ((uintptr_t)out[q] & 7) == 0);
        o.c[q] = out[q];
    }
    for (int j = 0; j < k; j++) ZKB_CHECK_ARG(ctx, h_col_idx[j] < (uint32_t)ncols);
    for (int c = 0; c < ncols; c++) ZKB_CHECK_ARG(ctx, cols[c] != nullptr && ((uintptr_t)cols[c] & 7) == 0);
    qm31 b_sum = qm31_zero();
    for (int j = 0; j < k; j++) b_sum = qm31_add(b_sum, qm31{{h_b[4 * j], h_b[4 * j + 1], h_b[4 * j + 2], h_b[4 * j + 3]}});
    DeviceGuard g(ctx);
    void** d_cols;
    int rc = stage_ptrs(ctx, (const void* const*)cols, ncols, &d_cols);
    if (rc) return rc;
    // coefficient table and column indices go through the scratch buffer
    uint32_t* d_c = ctx->scratch;
    uint32_t* d_idx = ctx->scratch + (size_t)4 * k;
    if (k) {
        ZKB_CUDA(ctx, cudaMemcpyAsync(d_c, h_c, (size_t)k * 16, cudaMemcpyHostToDevice, ctx->stream));
        ZKB_CUDA(ctx, cudaMemcpyAsync(d_idx, h_col_idx, (size_t)k * 4, cudaMemcpyHostToDevice, ctx->stream));
    }
    size_t n = (size_t)1 << log_n;
    bool wide = n >= 4;
    for (int q = 0; q < 4; q++) wide = wide && ((uintptr_t)out[q] & 15) == 0;
    for (int c = 0; c < ncols; c++) wide = wide && ((uintptr_t)cols[c] & 15) == 0;
    ProfScope prof(ctx, "quot_numerators_kernel");
    // Few rows and many columns: split the columns over the grid's second dimension.
    const unsigned row_blocks = (unsigned)((n / (wide ? 4 : 2) + 255) / 256);
    const size_t scratch_free = ctx->scratch_words - (size_t)5 * k;
    if (row_blocks < 148u && k >= 8 * NUM_TILE && 4 * n * 2 <= scratch_free) {
        int S = (int)((2u * 148u + row_blocks - 1) / row_blocks);            // about two CTAs per SM
        int chunk = ((k + S - 1) / S + NUM_TILE - 1) / NUM_TILE * NUM_TILE;  // whole tiles of columns
        S = (k + chunk - 1) / chunk;
        while ((size_t)S * 4 * n + 4 > scratch_free) { chunk += NUM_TILE; S = (k + chunk - 1) / chunk; }
        uint32_t* partial = ctx->scratch + (size_t)5 * k + ((4 - ((size_t)5 * k & 3)) & 3);  // 16-byte aligned
        dim3 grid(row_blocks, (unsigned)S);
        if (wide)
            quot_numerators_kernel<4><<<grid, 256, 0, ctx->stream>>>((const uint32_t* const*)d_cols, d_idx, reinterpret_cast<const uint4*>(d_c), k,
                                                                     b_sum, n, o, chunk, partial);
        else
            quot_numerators_kernel<2><<<grid, 256, 0, ctx->stream>>>((const uint32_t* const*)d_cols, d_idx, reinterpret_cast<const uint4*>(d_c), k,
                                                                     b_sum, n, o, chunk, partial);
        ZKB_LAUNCH_CHECK(ctx);
        quot_partial_sum_kernel<<<(unsigned)((4 * n + 255) / 256), 256, 0, ctx->stream>>>(partial, S, n, b_sum, o);
        ZKB_LAUNCH_CHECK(ctx);
        return ZKB_OK;
    }
    if (wide)
        quot_numerators_kernel<4><<<(unsigned)((n / 4 + 255) / 256), 256, 0, ctx->stream>>>(
            (const uint32_t* const*)d_cols, d_idx, reinterpret_cast<const uint4*>(d_c), k, b_sum, n, o);
    else
        quot_numerators_kernel<2><<<(unsigned)((n / 2 + 255) / 256), 256, 0, ctx->stream>>>(
            (const uint32_t* const*)d_cols, d_idx, reinterpret_cast<const uint4*>(d_c), k, b_sum, n, o);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

int zkb_quot_combine(zkb_ctx* ctx, int n_acc, const uint32_t* const* acc_cols, const int* h_acc_log,
                     const uint32_t* h_first_lin, const uint32_t* h_points, int lifting_log, uint32_t* const out[4]) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, lifting_log >= 1 && lifting_log <= ctx->max_log);
    return zkb_quot_combine_rows(ctx, n_acc, acc_cols, h_acc_log, h_first_lin, h_points, lifting_log, 0, (size_t)1 << lifting_log, out);
}

int zkb_quot_combine_rows(zkb_ctx* ctx, int n_acc, const uint32_t* const* acc_cols, const int* h_acc_log, const uint32_t* h_first_lin,
                          const uint32_t* h_points, int lifting_log, size_t row_begin, size_t n_rows, uint32_t* const out[4]) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, n_acc >= 1 && acc_cols && h_acc_log && h_first_lin && h_points && out);
    ZKB_CHECK_ARG(ctx, lifting_log >= 1 && lifting_log <= ctx->max_log);
    ZKB_CHECK_ARG(ctx, n_rows >= 1 && row_begin + n_rows <= ((size_t)1 << lifting_log));
    const bool whole = row_begin == 0 && n_rows == ((size_t)1 << lifting_log);
    // a shard starts on a row that every lifted accumulation starts a pair on, and small domains are not sharded
    ZKB_CHECK_ARG(ctx, whole || (lifting_log > 2 && (row_begin & 1) == 0 && (n_rows & 1) == 0));
    Secure4 o;
    for (int q = 0; q < 4; q++) {
        ZKB_CHECK_ARG(ctx, out[q] != nullptr);
        o.c[q] = out[q];
    }
    for (int a = 0; a < n_acc; a++) ZKB_CHECK_ARG(ctx, h_acc_log[a] >= 1 && h_acc_log[a] <= lifting_log);
    for (int a = 0; a < n_acc; a++)
        ZKB_CHECK_ARG(ctx, whole || (row_begin & (((size_t)2 << (lifting_log - h_acc_log[a])) - 1)) == 0);
    DeviceGuard g(ctx);
    size_t n = n_rows;
    for (int base = 0; base < n_acc; base += MAX_ACCS) {
        CombineArgs args;
        memset(&args, 0, sizeof(args));
        args.n_acc = n_acc - base < MAX_ACCS ? n_acc - base : MAX_ACCS;
        args.first = base == 0;
        for (int z = 0; z < args.n_acc; z++) {
            int a = base + z;
            for (int q = 0; q < 4; q++) {
                ZKB_CHECK_ARG(ctx, acc_cols[4 * a + q] != nullptr);
                args.acc[z][q] = acc_cols[4 * a + q];
            }
            args.log_ratio[z] = lifting_log - h_acc_log[a];
            for (int q = 0; q < 4; q++) args.first_lin[z].c[q] = h_first_lin[4 * a + q];
            const uint32_t* pt = h_points + 8 * a;  // x[4], y[4]
            args.prx[z] = {pt[0], pt[1]};
            args.pix[z] = {pt[2], pt[3]};
            args.pry[z] = {pt[4], pt[5]};
            args.piy[z] = {pt[6], pt[7]};
        }
        if (lifting_log <= 2) {
            int hl = lifting_log - 1;
            cpoint p0 = host_point_q((1u << (29 - hl)) & 0x7fffffffu);
            cpoint p1 = hl ? host_point_q(((1u << (29 - hl)) + (1u << (31 - hl))) & 0x7fffffffu) : p0;
            quot_combine_small_kernel<<<1, 32, 0, ctx->stream>>>(args, lifting_log, o, p0.x, p0.y, p1.x, p1.y);
        } else {
            ProfScope prof(ctx, "quot_combine_kernel");
            quot_combine_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(args, lifting_log, o, ctx->tw, row_begin, n_rows);
        }
        ZKB_LAUNCH_CHECK(ctx);
    }
    return ZKB_OK;
}

int zkb_accumulate(zkb_ctx* ctx, uint32_t* const col[4], const uint32_t* const other[4], size_t n) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, col && other);
    if (n == 0) return ZKB_OK;
    Secure4 a;
    Secure4C b;
    for (int q = 0; q < 4; q++) {
        ZKB_CHECK_ARG(ctx, col[q] != nullptr && other[q] != nullptr);
        a.c[q] = col[q];
        b.c[q] = other[q];
    }
    DeviceGuard g(ctx);
    accumulate_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(a, b, n);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

int zkb_lift_accumulate(zkb_ctx* ctx, uint32_t* const dst[4], int log_dst, const uint32_t* const src[4], int log_src) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, dst && src && log_src >= 1 && log_src <= log_dst && log_dst <= 30);
    Secure4 a;
    Secure4C b;
    for (int q = 0; q < 4; q++) {
        ZKB_CHECK_ARG(ctx, dst[q] != nullptr && src[q] != nullptr);
        a.c[q] = dst[q];
        b.c[q] = src[q];
    }
    DeviceGuard g(ctx);
    size_t n = (size_t)1 << log_dst;
    ProfScope prof(ctx, "lift_accumulate_kernel");
    lift_accumulate_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(a, log_dst, b, log_dst - log_src);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

}  // extern "C"
