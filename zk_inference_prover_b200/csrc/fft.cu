// Circle FFT over M31: interpolate (evaluations -> coefficients) and low-degree extension
// (coefficients -> evaluations on a larger canonic domain), batched over columns.
//
// The transform is the one of nitroo/crates/stwo/src/prover/backend/cpu/circle.rs:28-80 (inverse)
// and :182-228 (forward): layer i pairs indices that differ in bit i; the twiddle of a pair is
// indexed by the bits above i. Here the layers are grouped into passes; a pass stages a tile in
// shared memory, runs its layers there and writes the tile back.
//
// A pass covers layers [lo, lo + nlayers). Its tile is 2^kbits rows (bits lo .. lo+kbits-1 of the
// element index, kbits >= nlayers) by 2^logw consecutive low indices (logw <= lo), so global
// accesses are runs of 2^logw words. Zero-extension in the forward direction is implicit: the
// layers above the coefficient count only copy, so the first pass reads coeffs[idx mod n].
#include <cstdlib>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "fft_internal.hpp"
#include "fft_r32.cuh"

namespace zk {

constexpr int FFT_MAX_TILE_LOG = 13;    // 8192 words = 32 KiB of shared memory
constexpr int FFT_CONTIG_LOG = 12;      // layers handled by the contiguous pass
constexpr int FFT_STRIDED_LAYERS = 10;  // most layers in one strided pass
constexpr int R32_MAX_DEVICES = 64;     // per-device launch set-up is cached for this many devices

struct FftPass {
    int lo, kbits, nlayers, logw;
};

// Twiddle for layer i (>= 1) of the domain of log size L: T_{L-i}[h].
__device__ __forceinline__ uint32_t line_twiddle(const uint32_t* __restrict__ tower, int L, int i, uint32_t h) {
    return tower[(1u << (L - i - 1)) + h];
}
// Twiddle for layer 0: [y, -y, -x, x] per pair (x, y) of T_{L-1} (cpu/circle.rs:312-332).
__device__ __forceinline__ uint32_t circle_twiddle(const uint32_t* __restrict__ tower, int L, uint32_t h) {
    const uint32_t* T = tower + (1u << (L - 2));
    uint32_t q = h >> 2, r = h & 3;
    uint32_t v = T[2 * q + ((r & 2) ? 0 : 1)];  // r=0,1 -> y ; r=2,3 -> x
    return (r == 1 || r == 2) ? m31_neg(v) : v;
}

template <bool INVERSE>
__global__ void __launch_bounds__(512) fft_pass_kernel(uint32_t* const* __restrict__ dst_cols,
                                                       const uint32_t* const* __restrict__ src_cols, uint32_t src_mask,
                                                       int ncols, int log_n, int dom_log, FftPass ps,
                                                       const uint32_t* __restrict__ tower, uint32_t scale) {
    extern __shared__ uint32_t s[];
    const int tile_log = ps.kbits + ps.logw;
    const uint32_t E = 1u << tile_log;
    const uint32_t W = 1u << ps.logw;
    const uint32_t tile = blockIdx.x;
    const uint32_t wb = tile & ((1u << (ps.lo - ps.logw)) - 1u);
    const uint32_t a = tile >> (ps.lo - ps.logw);
    const uint32_t base = (a << (ps.lo + ps.kbits)) | (wb << ps.logw);

    for (int col = blockIdx.y; col < ncols; col += gridDim.y) {
        const uint32_t* __restrict__ src = src_cols[col];
        uint32_t* __restrict__ dst = dst_cols[col];
        for (uint32_t e = threadIdx.x; e < E; e += blockDim.x) {
            uint32_t m = e >> ps.logw, w = e & (W - 1u);
            uint32_t idx = base | (m << ps.lo) | w;
            s[e] = src[idx & src_mask];
        }
        __syncthreads();
        for (int step = 0; step < ps.nlayers; step++) {
            const int j = INVERSE ? step : ps.nlayers - 1 - step;
            const int i = ps.lo + j;
            for (uint32_t t = threadIdx.x; t < E / 2; t += blockDim.x) {
                uint32_t w = t & (W - 1u), q = t >> ps.logw;
                uint32_t m0 = ((q >> j) << (j + 1)) | (q & ((1u << j) - 1u));
                uint32_t m1 = m0 | (1u << j);
                uint32_t h = (a << (ps.kbits - 1 - j)) | (q >> j);
                uint32_t tw = (i == 0) ? circle_twiddle(tower, dom_log, h) : line_twiddle(tower, dom_log, i, h);
                uint32_t v0 = s[(m0 << ps.logw) | w], v1 = s[(m1 << ps.logw) | w];
                if (INVERSE) {
                    s[(m0 << ps.logw) | w] = m31_add(v0, v1);
                    s[(m1 << ps.logw) | w] = m31_mul(m31_sub(v0, v1), tw);
                } else {
                    uint32_t p = m31_mul(v1, tw);
                    s[(m0 << ps.logw) | w] = m31_add(v0, p);
                    s[(m1 << ps.logw) | w] = m31_sub(v0, p);
                }
            }
            __syncthreads();
        }
        for (uint32_t e = threadIdx.x; e < E; e += blockDim.x) {
            uint32_t m = e >> ps.logw, w = e & (W - 1u);
            uint32_t idx = base | (m << ps.lo) | w;
            uint32_t v = s[e];
            dst[idx] = scale ? m31_mul(v, scale) : v;
        }
        __syncthreads();
    }
}

// Domains of log size 1 and 2 (cpu/circle.rs:36-58 and :200-214). One thread per column.
// consts = {x, y} of the half-coset's first point for the forward direction, or
// {x_inv, y_inv, n_inv} for the inverse.
template <bool INVERSE>
__global__ void fft_small_kernel(uint32_t* const* __restrict__ dst_cols, const uint32_t* const* __restrict__ src_cols,
                                 int n_src, int ncols, int dom_log, uint32_t c0, uint32_t c1, uint32_t c2) {
    int col = blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= ncols) return;
    const uint32_t* src = src_cols[col];
    uint32_t* dst = dst_cols[col];
    uint32_t v[4] = {0, 0, 0, 0};
    int n = 1 << dom_log;
    for (int k = 0; k < n && k < n_src; k++) v[k] = src[k];
    auto bf = [](uint32_t& a, uint32_t& b, uint32_t t) { uint32_t p = m31_mul(b, t); b = m31_sub(a, p); a = m31_add(a, p); };
    auto ibf = [](uint32_t& a, uint32_t& b, uint32_t t) { uint32_t tmp = a; a = m31_add(tmp, b); b = m31_mul(m31_sub(tmp, b), t); };
    if (!INVERSE) {
        if (dom_log == 1) {
            bf(v[0], v[1], c1);
        } else {
            bf(v[0], v[2], c0); bf(v[1], v[3], c0);
            bf(v[0], v[1], c1); bf(v[2], v[3], m31_neg(c1));
        }
    } else {
        if (dom_log == 1) {
            ibf(v[0], v[1], c1);
        } else {
            ibf(v[0], v[1], c1); ibf(v[2], v[3], m31_neg(c1));
            ibf(v[0], v[2], c0); ibf(v[1], v[3], c0);
        }
        for (int k = 0; k < n; k++) v[k] = m31_mul(v[k], c2);
    }
    for (int k = 0; k < n; k++) dst[k] = v[k];
}

// One launch of the plan.
struct FftStep {
    int kind;  // 0: generic, 1: radix-32 contiguous (10 layers), 3: contiguous over 12 layers, 4: wide strided (8 layers)
    FftPass generic;
    R32Pass r32;
};

// Splits layers [0, nl) of an array of 2^log_n words into launches, lowest layers first.
// From 2^12 words up (16-byte aligned columns): the twelve-layer contiguous pass, then wide strided passes
// of up to eight layers (their window slides down over layers already done when the array is short; those
// layers are switched off). 2^10 and 2^11 words: the ten-layer contiguous pass and a generic pass for the
// rest. Everything else goes through the generic pass.
static std::vector<FftStep> plan_steps(int nl, int log_n, bool aligned) {
    std::vector<FftStep> v;
    if (log_n < 10 || !aligned) {
        int kb = log_n < FFT_CONTIG_LOG ? log_n : FFT_CONTIG_LOG;
        int kf = nl < kb ? nl : kb;
        v.push_back({0, {0, kb, kf, 0}, {}});
        int r = nl - kf, lo = kf;
        if (r > 0) {
            int np = (r + FFT_STRIDED_LAYERS - 1) / FFT_STRIDED_LAYERS;
            for (int p = 0; p < np; p++) {
                int k = r / np + (p < r % np ? 1 : 0);
                int logw = FFT_MAX_TILE_LOG - k;
                if (logw > 5) logw = 5;
                if (logw > lo) logw = lo;
                v.push_back({0, {lo, k, k, logw}, {}});
                lo += k;
            }
        }
        return v;
    }
    if (log_n < 12) {
        int covered = nl < 10 ? nl : 10;
        v.push_back({1, {}, {0, 0, covered}});
        if (covered < nl) {  // log_n = 11, one layer left
            int take = nl - covered;
            int logw = FFT_MAX_TILE_LOG - take;
            if (logw > 5) logw = 5;
            if (logw > covered) logw = covered;
            v.push_back({0, {covered, take, take, logw}, {}});
        }
        return v;
    }
    int covered = nl < 12 ? nl : 12;
    v.push_back({3, {}, {0, 0, covered}});
    while (covered < nl) {  // here log_n >= 13
        int take = nl - covered < 8 ? nl - covered : 8;
        int lo = covered;
        if (lo + 8 > log_n) lo = log_n - 8;
        v.push_back({4, {}, {lo, covered - lo, covered - lo + take}});
        covered += take;
    }
    return v;
}

template <bool INVERSE>
static int launch_pass(zkb_ctx* ctx, uint32_t* const* d_dst, const uint32_t* const* d_src, uint32_t src_mask, int ncols,
                       int log_n, int dom_log, const FftPass& ps, uint32_t scale) {
    int tile_log = ps.kbits + ps.logw;
    unsigned tiles = 1u << (log_n - tile_log);
    unsigned threads = 1u << (tile_log > 1 ? tile_log - 1 : 0);
    if (threads > 512) threads = 512;
    if (threads < 32) threads = 32;
    unsigned gy = ncols < 32768 ? ncols : 32768;
    size_t smem = (size_t)4 << tile_log;
    dim3 grid(tiles, gy);
    ProfScope prof(ctx, INVERSE ? "fft_pass_kernel<inverse>" : "fft_pass_kernel<forward>");
    fft_pass_kernel<INVERSE><<<grid, threads, smem, ctx->stream>>>(d_dst, d_src, src_mask, ncols, log_n, dom_log, ps,
                                                                   INVERSE ? ctx->itw : ctx->tw, scale);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

template <bool INVERSE>
static int launch_step(zkb_ctx* ctx, uint32_t* const* d_dst, const uint32_t* const* d_src, uint32_t src_mask, int ncols,
                       int log_n, int dom_log, const FftStep& st, uint32_t scale, RowBlocks rb = {31, 0u}, bool src_blocked = false) {
    if (st.kind == 0) return launch_pass<INVERSE>(ctx, d_dst, d_src, src_mask, ncols, log_n, dom_log, st.generic, scale);
    // Persistent launch: as many CTAs as fit on the device at once, each walking over work items.
    // The opt-in shared-memory size is a per-device function attribute and the SM count differs between
    // devices, so both are looked up once per device (under a lock: contexts on several devices may be
    // driven from several host threads).
    const int which = st.kind == 1 ? 0 : st.kind == 3 ? 1 : 2;
    const size_t smem = which == 0 ? r32_contig_smem(INVERSE) : which == 1 ? r32_c12_smem() : r32_wide_smem();
    const void* fn = which == 0   ? (const void*)fft_r32_contig_kernel<INVERSE>
                     : which == 1 ? (const void*)fft_r32_contig12_kernel<INVERSE>
                                  : (const void*)fft_r32_wide_kernel<INVERSE>;
    const int threads = which == 0 ? 32 * R32_CONTIG_WARPS : which == 1 ? 32 * R32_C12_WARPS : 256;
    int ctas = 0, n_sms = 0;
    {
        static std::mutex mu;
        static int s_ctas[R32_MAX_DEVICES][3][2];  // [device][kernel][forward/inverse]; 0 = not set up
        static int s_sms[R32_MAX_DEVICES];
        ZKB_CHECK_ARG(ctx, ctx->device >= 0 && ctx->device < R32_MAX_DEVICES);
        std::lock_guard<std::mutex> lock(mu);
        if (s_ctas[ctx->device][which][INVERSE] == 0) {
            ZKB_CUDA(ctx, cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            int k = 0;
            ZKB_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&k, fn, threads, smem));
            ZKB_CUDA(ctx, cudaDeviceGetAttribute(&s_sms[ctx->device], cudaDevAttrMultiProcessorCount, ctx->device));
            s_ctas[ctx->device][which][INVERSE] = k > 0 ? k : 1;
        }
        ctas = s_ctas[ctx->device][which][INVERSE];
        n_sms = s_sms[ctx->device];
    }
    size_t items = which == 0   ? (((size_t)ncols << (log_n - 10)) + R32_CONTIG_WARPS - 1) / R32_CONTIG_WARPS
                   : which == 1 ? ((size_t)ncols << (log_n - 12))
                                : ((size_t)ncols << (log_n - 13));
    size_t max_ctas = (size_t)n_sms * ctas;
    unsigned grid = (unsigned)(items < max_ctas ? items : max_ctas);
    if (which == 2) {
        // a grid that is a multiple of the number of tile rows above the window lets every CTA keep one twiddle table
        const unsigned n_a = 1u << (log_n - st.r32.lo - 8);
        if (grid >= n_a) grid -= grid % n_a;
    }
    const uint32_t* tower = INVERSE ? ctx->itw2 : ctx->tw2;
    ProfScope prof(ctx, which == 2 ? (INVERSE ? "fft_r32_wide_kernel<inverse>" : "fft_r32_wide_kernel<forward>")
                                   : (INVERSE ? "fft_r32_contig_kernel<inverse>" : "fft_r32_contig_kernel<forward>"));
    if (which == 0)
        fft_r32_contig_kernel<INVERSE><<<grid, threads, smem, ctx->stream>>>(d_dst, d_src, src_mask, ncols, log_n, dom_log, st.r32, tower, scale);
    else if (which == 1)
        fft_r32_contig12_kernel<INVERSE><<<grid, threads, smem, ctx->stream>>>(d_dst, d_src, src_mask, ncols, log_n, dom_log, st.r32, tower, scale,
                                                                                 rb, src_blocked ? 1 : 0);
    else
        fft_r32_wide_kernel<INVERSE><<<grid, threads, smem, ctx->stream>>>(d_dst, d_src, src_mask, ncols, log_n, dom_log, st.r32, tower, scale, rb);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

// The butterfly arithmetic alone: 32 values per thread, five layers per round, twiddles from shared memory,
// no global traffic inside the loop. What this kernel reaches is the ceiling the FFT passes are bound by.
__global__ void __launch_bounds__(256, 2) butterfly_ceiling_kernel(uint32_t* __restrict__ out, const uint32_t* __restrict__ tower, int rounds) {
    __shared__ __align__(16) uint32_t tw[32];
    if (threadIdx.x < 32) tw[threadIdx.x] = tower[32 + threadIdx.x];
    __syncthreads();
    uint32_t v[32];
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = tower[(threadIdx.x * 32 + i) & 1023] >> 1;
    const uint32_t* const tb[5] = {tw, tw + 16, tw + 24, tw + 28, tw + 30};
    for (int r = 0; r < rounds; r++) radix32_stage<false, false, true>(v, tb, 0, 0, 5);
    uint32_t acc = 0;
#pragma unroll
    for (int i = 0; i < 32; i++) acc ^= v[i];
    out[(size_t)blockIdx.x * 256 + threadIdx.x] = acc;
}

// First point of Coset::half_odds(log) on the host: index 2^(31 - log - 2).
static cpoint host_half_odds_initial_zk(int log) {
    cpoint g{2u, 1268011823u};
    for (int b = 0; b < 31 - log - 2; b++) g = cpoint_add(g, g);
    return g;
}

// zkb_lde_cols with the output columns laid out in row blocks (see RowBlocks): out[c] is the base of column c, block b of
// it starts blk_stride words further per block. blk_log = 31: plain columns. Blocked output needs the radix-32 plan
// (2^13 words or more per column, 16-byte aligned) and blocks of at least 4096 words; lde_blocked_supported says so.
bool lde_blocked_supported(int log_n, int log_out, int blk_log) {
    // one wide pass at most (the second one of a longer transform would have to read blocked input too)
    return log_n >= 2 && log_n <= 20 && log_out >= 13 && blk_log >= 12 && blk_log <= log_out;
}

__global__ void repack_row_blocks_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, int ncols, int log_out, int blk_log) {
    const size_t total = ((size_t)ncols << log_out) >> 2;  // 16-byte pieces
    for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
        const size_t w = t << 2, c = w >> log_out, idx = w & (((size_t)1 << log_out) - 1);
        const size_t b = idx >> blk_log, i = idx & (((size_t)1 << blk_log) - 1);
        out[((((b * ncols + c) << blk_log) + i)) >> 2] = in[t];
    }
}

int repack_row_blocks(zkb_ctx* ctx, const uint32_t* in, uint32_t* out, int ncols, int log_out, int blk_log) {
    ZKB_CHECK_ARG(ctx, in && out && ncols > 0 && blk_log >= 2 && blk_log <= log_out && (((uintptr_t)in | (uintptr_t)out) & 15) == 0);
    DeviceGuard g(ctx);
    repack_row_blocks_kernel<<<148 * 8, 256, 0, ctx->stream>>>((const uint4*)in, (uint4*)out, ncols, log_out, blk_log);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

int lde_cols_blocked(zkb_ctx* ctx, const uint32_t* const* coeffs, int ncols, int log_n, uint32_t* const* out, int log_out, int blk_log,
                     uint32_t blk_stride) {
    const bool plain = blk_log >= 31;
    const RowBlocks rb{plain ? 31 : blk_log, plain ? 0u : blk_stride};
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, ncols >= 0 && log_n >= 0 && log_out >= 1 && log_n <= log_out && log_out <= ctx->max_log);
    if (ncols == 0) return ZKB_OK;
    ZKB_CHECK_ARG(ctx, coeffs != nullptr && out != nullptr);
    for (int c = 0; c < ncols; c++) ZKB_CHECK_ARG(ctx, (const void*)coeffs[c] != (const void*)out[c]);
    DeviceGuard g(ctx);
    void **d_src, **d_dst;
    int rc = stage_ptrs(ctx, (const void* const*)coeffs, ncols, &d_src);
    if (rc) return rc;
    rc = stage_ptrs(ctx, (const void* const*)out, ncols, &d_dst);
    if (rc) return rc;
    if (log_out <= 2) {
        cpoint p = host_half_odds_initial_zk(log_out - 1);
        fft_small_kernel<false><<<(ncols + 127) / 128, 128, 0, ctx->stream>>>(
            (uint32_t* const*)d_dst, (const uint32_t* const*)d_src, 1 << log_n, ncols, log_out, p.x, p.y, 0u);
        ZKB_LAUNCH_CHECK(ctx);
        return ZKB_OK;
    }
    bool aligned = true;
    for (int c = 0; c < ncols; c++) aligned = aligned && (((uintptr_t)out[c] | (uintptr_t)coeffs[c]) & 15) == 0;
    if (log_n < 2) aligned = false;  // the staged copies move 16 bytes at a time
    if (!plain) ZKB_CHECK_ARG(ctx, aligned && lde_blocked_supported(log_n, log_out, blk_log) && (blk_stride & 3u) == 0);
    auto steps = plan_steps(log_n, log_out, aligned);
    uint32_t src_mask = (1u << log_n) - 1u;
    // ZKB_LDE_CHUNK=k runs all passes over k columns at a time, so that the array between two passes (2^log_out
    // words per column) is still in the L2 cache when the next pass reads it. Off by default: at 256 x 2^22 the
    // DRAM traffic drops but the many short launches cost more time than the traffic saves (the passes are bound
    // by instruction issue, not by DRAM).
    static const int env_chunk = []() { const char* e = getenv("ZKB_LDE_CHUNK"); return e ? atoi(e) : 0; }();
    const int chunk = env_chunk > 0 && steps.size() > 1 ? env_chunk : ncols;
    for (int c0 = 0; c0 < ncols; c0 += chunk) {
        const int nc = ncols - c0 < chunk ? ncols - c0 : chunk;
        for (size_t p = steps.size(); p-- > 0;) {
            bool first = p + 1 == steps.size();
            rc = launch_step<false>(ctx, (uint32_t* const*)d_dst + c0,
                                    (first ? (const uint32_t* const*)d_src : (const uint32_t* const*)d_dst) + c0,
                                    first ? src_mask : 0xffffffffu, nc, log_out, log_out, steps[p], 0u, rb, !first && !plain);
            if (rc) return rc;
        }
    }
    return ZKB_OK;
}


}  // namespace zk

using namespace zk;

// First point of Coset::half_odds(log) on the host: index 2^(31 - log - 2).
static cpoint host_half_odds_initial(int log) {
    cpoint g{2u, 1268011823u};
    for (int b = 0; b < 31 - log - 2; b++) g = cpoint_add(g, g);
    return g;
}

extern "C" {

int zkb_fft_arith_ceiling(zkb_ctx* ctx, double* h_butterflies_per_s) {
    if (!ctx || !h_butterflies_per_s) return ZKB_EINVAL;
    DeviceGuard g(ctx);
    int n_sms = 0;
    ZKB_CUDA(ctx, cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, ctx->device));
    const int grid = n_sms * 2, rounds = 400;
    ZKB_CHECK_ARG(ctx, (size_t)grid * 256 <= ctx->scratch_words && ctx->tw_len >= 1024);
    if (!ctx->events[62]) { ZKB_CUDA(ctx, cudaEventCreate(&ctx->events[62])); }
    if (!ctx->events[63]) { ZKB_CUDA(ctx, cudaEventCreate(&ctx->events[63])); }
    butterfly_ceiling_kernel<<<grid, 256, 0, ctx->stream>>>(ctx->scratch, ctx->tw2, 20);  // warm-up
    ZKB_CUDA(ctx, cudaEventRecord(ctx->events[62], ctx->stream));
    butterfly_ceiling_kernel<<<grid, 256, 0, ctx->stream>>>(ctx->scratch, ctx->tw2, rounds);
    ZKB_CUDA(ctx, cudaEventRecord(ctx->events[63], ctx->stream));
    ZKB_LAUNCH_CHECK(ctx);
    ZKB_CUDA(ctx, cudaEventSynchronize(ctx->events[63]));
    float ms = 0.f;
    ZKB_CUDA(ctx, cudaEventElapsedTime(&ms, ctx->events[62], ctx->events[63]));
    *h_butterflies_per_s = (double)grid * 256 * 80.0 * rounds / ((double)ms * 1e-3);
    return ZKB_OK;
}

int zkb_ifft_cols(zkb_ctx* ctx, uint32_t* const* cols, int ncols, int log_n) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, ncols >= 0 && log_n >= 1 && log_n <= ctx->max_log);
    if (ncols == 0) return ZKB_OK;
    ZKB_CHECK_ARG(ctx, cols != nullptr);
    DeviceGuard g(ctx);
    void** d_cols;
    int rc = stage_ptrs(ctx, (const void* const*)cols, ncols, &d_cols);
    if (rc) return rc;
    uint32_t* const* dc = (uint32_t* const*)d_cols;
    if (log_n <= 2) {
        cpoint p = host_half_odds_initial(log_n - 1);
        uint32_t n = 1u << log_n;
        uint32_t xi = log_n == 2 ? m31_inv(p.x) : 0u, yi = m31_inv(p.y), ni = m31_inv(n);
        fft_small_kernel<true><<<(ncols + 127) / 128, 128, 0, ctx->stream>>>(dc, (const uint32_t* const*)dc, (int)n, ncols,
                                                                            log_n, xi, yi, ni);
        ZKB_LAUNCH_CHECK(ctx);
        return ZKB_OK;
    }
    bool aligned = true;
    for (int c = 0; c < ncols; c++) aligned = aligned && ((uintptr_t)cols[c] & 15) == 0;
    auto steps = plan_steps(log_n, log_n, aligned);
    uint32_t n_inv = m31_inv(1u << log_n);
    for (size_t p = 0; p < steps.size(); p++) {
        rc = launch_step<true>(ctx, dc, (const uint32_t* const*)dc, 0xffffffffu, ncols, log_n, log_n, steps[p],
                               p + 1 == steps.size() ? n_inv : 0u);
        if (rc) return rc;
    }
    return ZKB_OK;
}

int zkb_lde_cols(zkb_ctx* ctx, const uint32_t* const* coeffs, int ncols, int log_n, uint32_t* const* out, int log_out) {
    return zk::lde_cols_blocked(ctx, coeffs, ncols, log_n, out, log_out, 31, 0u);
}

}  // extern "C"
