// PolyOps::eval_at_point / batch_eval_at_point: the value of each column's polynomial (FFT-basis
// coefficients) at one QM31 circle point.
//
// The reference folds the coefficient array as a binary tree
// (nitroo/crates/stwo/src/prover/backend/cpu/circle.rs:82-100, core/poly/utils.rs:11-23):
// level k joins blocks of 2^k values as lhs + rhs * m_k with m_0 = y, m_1 = x, m_{k+1} = pi(m_k).
// Field arithmetic is exact and distributive, so the tree equals sum_i c_i * prod_{k: bit k of i} m_k.
// The lowest 11 levels are evaluated as that weighted sum: a CTA takes 2048 coefficients, every
// thread multiplies its 8 coefficients (M31) by weights it keeps in registers (QM31), accumulating
// unreduced in 64 bits, and the CTA adds the 256 partial sums. What remains per column is a short
// array of partials, folded level by level in shared memory with the remaining factors.
#include <vector>

#include "common.cuh"

namespace zk {

constexpr int EVAL_CHUNK_LOG = 11;
constexpr int EVAL_MAX_LEVELS = 32;

struct EvalFactors { qm31 m[EVAL_MAX_LEVELS]; };

// weights[i] = prod over set bits k of i of m_k, i < 2^EVAL_CHUNK_LOG.
__global__ void eval_weights_kernel(EvalFactors f, int bits, uint32_t* __restrict__ weights) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (1u << bits)) return;
    qm31 w = qm31_one();
    for (int k = 0; k < bits; k++)
        if ((i >> k) & 1u) w = qm31_mul(w, f.m[k]);
    reinterpret_cast<uint4*>(weights)[i] = make_uint4(w.c[0], w.c[1], w.c[2], w.c[3]);
}

__device__ __forceinline__ uint64_t fold64_eval(uint64_t v) { return (v & P) + (v >> 31); }

// out[col][chunk] = sum_{e < 2048} cols[col][2048 chunk + e] * weights[e]
// Thread t owns elements 4t..4t+3 and 1024+4t..1024+4t+3 of every chunk (two 16-byte loads) and keeps
// their eight weights in registers. DOT_CHUNKS chunks are in flight per iteration; their per-warp sums
// use the hardware warp reduction on 16-bit halves (32 x 2^16 fits a word) and meet in shared memory
// once per iteration.
constexpr int DOT_CHUNKS = 4;
__global__ void __launch_bounds__(256) eval_dot_kernel(const uint32_t* const* __restrict__ cols, int ncols, int log_n,
                                                       const uint32_t* __restrict__ weights, uint32_t* __restrict__ out) {
    __shared__ uint32_t red[DOT_CHUNKS][4][2][8];  // [chunk][component][lo/hi][warp]
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    uint4 w[8];
#pragma unroll
    for (int u = 0; u < 8; u++) w[u] = reinterpret_cast<const uint4*>(weights)[(u >> 2) * 1024 + 4 * t + (u & 3)];
    const size_t chunks = (size_t)1 << (log_n - EVAL_CHUNK_LOG);
    const size_t groups = (chunks + DOT_CHUNKS - 1) / DOT_CHUNKS;
    // persistent CTAs over (column, group of chunks): the weights are read once per CTA
    for (size_t item = blockIdx.x; item < groups * (size_t)ncols; item += gridDim.x) {
        const size_t col = item / groups, chunk0 = (item % groups) * DOT_CHUNKS;
        const uint32_t* __restrict__ c = cols[col];
        uint4 v[DOT_CHUNKS][2];
#pragma unroll
        for (int g = 0; g < DOT_CHUNKS; g++) {
            if (chunk0 + g < chunks) {
                const uint4* p = reinterpret_cast<const uint4*>(c + ((chunk0 + g) << EVAL_CHUNK_LOG));
                v[g][0] = __ldcs(p + t);
                v[g][1] = __ldcs(p + 256 + t);
            } else {
                v[g][0] = v[g][1] = make_uint4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int g = 0; g < DOT_CHUNKS; g++) {
            const uint32_t e[8] = {v[g][0].x, v[g][0].y, v[g][0].z, v[g][0].w, v[g][1].x, v[g][1].y, v[g][1].z, v[g][1].w};
            uint64_t a0 = 0, a1 = 0, a2 = 0, a3 = 0;
#pragma unroll
            for (int u = 0; u < 8; u++) {
                a0 += (uint64_t)e[u] * w[u].x; a1 += (uint64_t)e[u] * w[u].y;
                a2 += (uint64_t)e[u] * w[u].z; a3 += (uint64_t)e[u] * w[u].w;
                if (u == 3) { a0 = fold64_eval(a0); a1 = fold64_eval(a1); a2 = fold64_eval(a2); a3 = fold64_eval(a3); }
            }
            const uint32_t r[4] = {m31_reduce64(a0), m31_reduce64(a1), m31_reduce64(a2), m31_reduce64(a3)};
#pragma unroll
            for (int k = 0; k < 4; k++) {
                uint32_t lo = __reduce_add_sync(0xffffffffu, r[k] & 0xffffu);
                uint32_t hi = __reduce_add_sync(0xffffffffu, r[k] >> 16);
                if (lane == 0) { red[g][k][0][warp] = lo; red[g][k][1][warp] = hi; }
            }
        }
        __syncthreads();
        if (t < 4 * DOT_CHUNKS) {
            const int g = t >> 2, k = t & 3;
            if (chunk0 + g < chunks) {
                uint64_t lo = 0, hi = 0;
#pragma unroll
                for (int wv = 0; wv < 8; wv++) { lo += red[g][k][0][wv]; hi += red[g][k][1][wv]; }
                out[4 * ((size_t)col * chunks + chunk0 + g) + k] = m31_reduce64(lo + (hi << 16));
            }
        }
        __syncthreads();
    }
}

// in: either a table of M31 columns (IS_BASE) or a dense [ncols][2^log_in] array of QM31.
// out: dense [ncols][2^(log_in - chunk_log)] QM31.
template <bool IS_BASE>
__global__ void __launch_bounds__(256) eval_fold_kernel(const uint32_t* const* __restrict__ base_cols,
                                                        const uint32_t* __restrict__ ext_in, int log_in, int chunk_log,
                                                        int level0, EvalFactors f, uint32_t* __restrict__ out) {
    __shared__ uint32_t s[4][1 << EVAL_CHUNK_LOG];
    const uint32_t E = 1u << chunk_log;
    const size_t chunk = blockIdx.x;
    const int col = blockIdx.y;
    const size_t n_in = (size_t)1 << log_in;
    for (uint32_t e = threadIdx.x; e < E; e += blockDim.x) {
        size_t idx = chunk * E + e;
        if (IS_BASE) {
            s[0][e] = base_cols[col][idx];
            s[1][e] = 0; s[2][e] = 0; s[3][e] = 0;
        } else {
            uint4 v = reinterpret_cast<const uint4*>(ext_in)[(size_t)col * n_in + idx];
            s[0][e] = v.x; s[1][e] = v.y; s[2][e] = v.z; s[3][e] = v.w;
        }
    }
    __syncthreads();
    for (int k = 0; k < chunk_log; k++) {
        const qm31 m = f.m[level0 + k];
        for (uint32_t t = threadIdx.x; t < (E >> (k + 1)); t += blockDim.x) {
            uint32_t i0 = t << (k + 1), i1 = i0 + (1u << k);
            qm31 a{{s[0][i0], s[1][i0], s[2][i0], s[3][i0]}}, b{{s[0][i1], s[1][i1], s[2][i1], s[3][i1]}};
            qm31 r = qm31_add(a, qm31_mul(b, m));
            s[0][i0] = r.c[0]; s[1][i0] = r.c[1]; s[2][i0] = r.c[2]; s[3][i0] = r.c[3];
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        size_t n_out = n_in >> chunk_log;
        reinterpret_cast<uint4*>(out)[(size_t)col * n_out + chunk] = make_uint4(s[0][0], s[1][0], s[2][0], s[3][0]);
    }
}

}  // namespace zk

using namespace zk;

extern "C" {

int zkb_eval_at_point_cols(zkb_ctx* ctx, const uint32_t* const* coeffs, int ncols, int log_n, const uint32_t* h_point,
                           uint32_t* h_out) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, ncols >= 0 && log_n >= 0 && log_n <= 30);
    if (ncols == 0) return ZKB_OK;
    ZKB_CHECK_ARG(ctx, coeffs && h_point && h_out);
    DeviceGuard g(ctx);
    // factors m_0 = y, m_1 = x, m_{k+1} = 2 m_k^2 - 1
    EvalFactors f;
    memset(&f, 0, sizeof(f));
    qm31 x{{h_point[0], h_point[1], h_point[2], h_point[3]}}, y{{h_point[4], h_point[5], h_point[6], h_point[7]}};
    f.m[0] = y;
    for (int k = 1; k < log_n; k++) {
        f.m[k] = x;
        x = qm31_double_x(x);
    }
    // Scratch: [weights: 2048 QM31] [ping] [pong]; columns go in batches whose partials fit.
    bool use_dot = log_n >= EVAL_CHUNK_LOG;
    for (int c = 0; c < ncols; c++) use_dot = use_dot && ((uintptr_t)coeffs[c] & 15) == 0;  // 16-byte loads
    int first_chunk = log_n < EVAL_CHUNK_LOG ? log_n : EVAL_CHUNK_LOG;
    size_t partials_per_col = (size_t)1 << (log_n - first_chunk);
    uint32_t* weights = ctx->scratch;
    const size_t weights_words = (size_t)4 << EVAL_CHUNK_LOG;
    size_t half_words = (ctx->scratch_words - weights_words) / 2;
    size_t max_cols = half_words / (4 * partials_per_col);
    ZKB_CHECK_ARG(ctx, max_cols >= 1);
    if (max_cols > 32768) max_cols = 32768;
    if (use_dot) {
        eval_weights_kernel<<<(1 << EVAL_CHUNK_LOG) / 256, 256, 0, ctx->stream>>>(f, EVAL_CHUNK_LOG, weights);
        ZKB_LAUNCH_CHECK(ctx);
    }
    for (int c0 = 0; c0 < ncols; c0 += (int)max_cols) {
        int nc = ncols - c0 < (int)max_cols ? ncols - c0 : (int)max_cols;
        void** d_cols;
        int rc = stage_ptrs(ctx, (const void* const*)(coeffs + c0), nc, &d_cols);
        if (rc) return rc;
        uint32_t* bufA = ctx->scratch + weights_words;
        uint32_t* bufB = bufA + half_words;
        int log_cur = log_n, level = 0;
        if (use_dot) {
            size_t items = (partials_per_col + DOT_CHUNKS - 1) / DOT_CHUNKS * (size_t)nc;
            unsigned grid = (unsigned)(items < 2 * 148 ? items : 2 * 148);
            ProfScope prof(ctx, "eval_dot_kernel");
            eval_dot_kernel<<<grid, 256, 0, ctx->stream>>>((const uint32_t* const*)d_cols, nc, log_n, weights, bufA);
            ZKB_LAUNCH_CHECK(ctx);
        } else {
            unsigned threads = first_chunk >= 9 ? 256 : 32;
            dim3 grid((unsigned)partials_per_col, nc);
            eval_fold_kernel<true><<<grid, threads, 0, ctx->stream>>>((const uint32_t* const*)d_cols, nullptr, log_cur,
                                                                      first_chunk, level, f, bufA);
            ZKB_LAUNCH_CHECK(ctx);
        }
        log_cur -= first_chunk;
        level += first_chunk;
        while (log_cur > 0) {
            int ch = log_cur < EVAL_CHUNK_LOG ? log_cur : EVAL_CHUNK_LOG;
            unsigned threads = ch >= 9 ? 256 : 32;
            dim3 grid(1u << (log_cur - ch), nc);
            eval_fold_kernel<false><<<grid, threads, 0, ctx->stream>>>(nullptr, bufA, log_cur, ch, level, f, bufB);
            ZKB_LAUNCH_CHECK(ctx);
            log_cur -= ch;
            level += ch;
            uint32_t* t = bufA; bufA = bufB; bufB = t;
        }
        ZKB_CUDA(ctx, cudaMemcpyAsync(h_out + 4 * (size_t)c0, bufA, (size_t)nc * 16, cudaMemcpyDeviceToHost, ctx->stream));
        ZKB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
    return ZKB_OK;
}

}  // extern "C"
