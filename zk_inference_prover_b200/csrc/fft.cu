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

// One launch of the plan: either a radix-32 window pass or a generic shared-memory pass.
struct FftStep {
    int kind;  // 0: generic, 1: radix-32 contiguous, 2: radix-32 strided
    FftPass generic;
    R32Pass r32;
};

// Splits layers [0, nl) of an array of 2^log_n words into launches, lowest layers first.
// Radix-32 windows need 2^10 rows (log_n >= 10) and 16-byte aligned columns; everything else
// goes through the generic pass.
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
    int covered = nl < 10 ? nl : 10;
    v.push_back({1, {}, {0, 0, covered}});
    while (covered < nl) {
        int take = nl - covered < 10 ? nl - covered : 10;
        int lo = covered;
        if (lo + 10 > log_n) lo = log_n - 10;
        if (lo >= 3) {
            v.push_back({2, {}, {lo, covered - lo, covered - lo + take}});
        } else {
            int logw = FFT_MAX_TILE_LOG - take;
            if (logw > 5) logw = 5;
            if (logw > covered) logw = covered;
            v.push_back({0, {covered, take, take, logw}, {}});
        }
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
                       int log_n, int dom_log, const FftStep& st, uint32_t scale) {
    if (st.kind == 0) return launch_pass<INVERSE>(ctx, d_dst, d_src, src_mask, ncols, log_n, dom_log, st.generic, scale);
    // Persistent launch: as many CTAs as fit on the device at once, each walking over work items.
    // The opt-in shared-memory size is a per-device function attribute and the SM count differs between
    // devices, so both are looked up once per device (under a lock: contexts on several devices may be
    // driven from several host threads).
    static const int lw = []() { const char* e = getenv("ZKB_FFT_LW"); return e && e[0] == '2' ? 2 : e && e[0] == '4' ? 4 : 3; }();
    const size_t smem = st.kind == 1 ? r32_contig_smem(INVERSE) : r32_strided_smem(lw);
    const int which = st.kind == 1 ? 0 : 1;
    const void* fn = st.kind == 1 ? (const void*)fft_r32_contig_kernel<INVERSE>
                     : lw == 3   ? (const void*)fft_r32_strided_kernel<INVERSE, 3>
                     : lw == 4   ? (const void*)fft_r32_strided_kernel<INVERSE, 4>
                                 : (const void*)fft_r32_strided_kernel<INVERSE, 2>;
    const int threads = st.kind == 1 ? 32 * R32_CONTIG_WARPS : 32 << lw;
    int ctas = 0, n_sms = 0;
    {
        static std::mutex mu;
        static int s_ctas[R32_MAX_DEVICES][2][2];  // [device][contiguous/strided][forward/inverse]; 0 = not set up
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
    size_t items = st.kind == 1 ? (((size_t)ncols << (log_n - 10)) + R32_CONTIG_WARPS - 1) / R32_CONTIG_WARPS
                                : ((size_t)ncols << (log_n - 10 - lw));
    size_t max_ctas = (size_t)n_sms * ctas;
    unsigned grid = (unsigned)(items < max_ctas ? items : max_ctas);
    if (st.kind == 2) {
        // a grid that is a multiple of the number of tile rows above the window lets every CTA keep one twiddle table
        const unsigned n_a = 1u << (log_n - st.r32.lo - 10);
        if (grid >= n_a) grid -= grid % n_a;
    }
    ProfScope prof(ctx, st.kind == 1 ? (INVERSE ? "fft_r32_contig_kernel<inverse>" : "fft_r32_contig_kernel<forward>")
                                     : (INVERSE ? "fft_r32_strided_kernel<inverse>" : "fft_r32_strided_kernel<forward>"));
    if (st.kind == 1)
        fft_r32_contig_kernel<INVERSE><<<grid, threads, smem, ctx->stream>>>(d_dst, d_src, src_mask, ncols, log_n, dom_log,
                                                                              st.r32, INVERSE ? ctx->itw2 : ctx->tw2, scale);
    else if (lw == 3)
        fft_r32_strided_kernel<INVERSE, 3><<<grid, threads, smem, ctx->stream>>>(d_dst, d_src, src_mask, ncols, log_n, dom_log,
                                                                                  st.r32, INVERSE ? ctx->itw2 : ctx->tw2, scale);
    else if (lw == 4)
        fft_r32_strided_kernel<INVERSE, 4><<<grid, threads, smem, ctx->stream>>>(d_dst, d_src, src_mask, ncols, log_n, dom_log,
                                                                                  st.r32, INVERSE ? ctx->itw2 : ctx->tw2, scale);
    else
        fft_r32_strided_kernel<INVERSE, 2><<<grid, threads, smem, ctx->stream>>>(d_dst, d_src, src_mask, ncols, log_n, dom_log,
                                                                                  st.r32, INVERSE ? ctx->itw2 : ctx->tw2, scale);
    ZKB_LAUNCH_CHECK(ctx);
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
        cpoint p = host_half_odds_initial(log_out - 1);
        fft_small_kernel<false><<<(ncols + 127) / 128, 128, 0, ctx->stream>>>(
            (uint32_t* const*)d_dst, (const uint32_t* const*)d_src, 1 << log_n, ncols, log_out, p.x, p.y, 0u);
        ZKB_LAUNCH_CHECK(ctx);
        return ZKB_OK;
    }
    bool aligned = true;
    for (int c = 0; c < ncols; c++) aligned = aligned && (((uintptr_t)out[c] | (uintptr_t)coeffs[c]) & 15) == 0;
    if (log_n < 2) aligned = false;  // the staged copies move 16 bytes at a time
    auto steps = plan_steps(log_n, log_out, aligned);
    uint32_t src_mask = (1u << log_n) - 1u;
    for (size_t p = steps.size(); p-- > 0;) {
        bool first = p + 1 == steps.size();
        rc = launch_step<false>(ctx, (uint32_t* const*)d_dst,
                                first ? (const uint32_t* const*)d_src : (const uint32_t* const*)d_dst,
                                first ? src_mask : 0xffffffffu, ncols, log_out, log_out, steps[p], 0u);
        if (rc) return rc;
    }
    return ZKB_OK;
}

}  // extern "C"
