// Witness generation on the device for two more column families of the prover: the shared lookup tables'
// own columns and the matmul dequantize component. Both write every column directly in committed order
// (row j of the natural order lands at index coset_perm(j), prover/src/common.rs:76-80), so the host never
// shuffles, packs or uploads a trace column.
//
// The reference's device originals are zk_witness_gen_tables (stwo_cuda/cuda/zk_table_witness_gen.cu,
// called from prover/src/devtab.rs:267) and zk_witness_gen_dequant (stwo_cuda/cuda/zk_dequant_witness_gen.cu,
// called from prover/src/gadgets/dequant/device.rs:330); the per-row arithmetic of the dequantize
// component is witness_gen_mat_row, prover/src/gadgets/dequant/trace.rs:503-690 (pow2 and chain arms).
// The reference kernels' "mutate" arguments are deliberate defects for its negative controls; they are not
// part of the operator and are not built here.
#include <vector>

#include "common.cuh"

namespace zk {

constexpr uint32_t NONE = 0xffffffffu;

// The committed index i holds natural (coset-order) row coset_perm(i); the map is an involution.
__device__ __forceinline__ uint32_t coset_perm(uint32_t i, uint32_t log_n) {
    uint32_t c = (i & 1u) ? (((2u << log_n) - i - 1u) >> 1) : (i >> 1);
    return __brev(c) >> (32u - log_n);
}

// A possibly negative integer as a field element (attn_trace::m31_of).
__device__ __forceinline__ uint32_t m31_of(long long v) {
    // two folds of 31 bits bring any |v| < 2^62 below 2p (2^31 = 1 mod p); no 64-bit division
    unsigned long long u = (unsigned long long)(v < 0 ? -v : v);
    u = (u & P) + (u >> 31);
    u = (u & P) + (u >> 31);
    uint32_t r = (uint32_t)u;
    if (r >= P) r -= P;
    return (v < 0 && r) ? P - r : r;
}

// ---------------------------------------------------------------------------------------------------
// Tables: x = row index, y = exp table (a gather out of the 2^16-entry map of bf16 patterns), m = the
// multiplicities summed over every key tile's counter.
//
// Committed rows 2q and 2q+1 hold natural rows brev(q) and brev(~q): a pair of reads at mirrored
// addresses. A CTA takes a 32 x 32 tile of q (5 high bits x 5 low bits, the middle bits fixed): the
// counter reads then run along the 5 high bits of q, which are the 5 low bits of the natural row, so
// every read of a warp is one 128-byte line (and its mirror), and the writes are 256-byte runs of
// committed rows. Tiles go through shared memory; nothing is read twice.
// ---------------------------------------------------------------------------------------------------
struct TabCfg {
    uint32_t log_rows, n_counters, bf16x;
    double two_pow;
};

__device__ __forceinline__ uint32_t exp_pattern(uint32_t d, const TabCfg& cfg) {
    if (cfg.bf16x) return d & 0xffffu;
    // bf16(-d / 2^frac), round to nearest even (prover/src/bf16.rs:36-43; the argument is finite)
    float x = (float)(-(double)d / cfg.two_pow);
    uint32_t u = __float_as_uint(x);
    return ((u + 0x7fffu + ((u >> 16) & 1u)) >> 16) & 0xffffu;
}

__global__ void __launch_bounds__(256) tables_tiled_kernel(const uint32_t* __restrict__ expmap, const uint32_t* const* __restrict__ counters,
                                                           uint32_t* __restrict__ x_col, uint32_t* __restrict__ y_col,
                                                           uint32_t* __restrict__ m_col, TabCfg cfg) {
    // q has log_rows - 1 bits: [hi:5 | mid | lo:5]; natural row of committed 2q is brev_{log_rows}(q) (top bit of c is 0),
    // of committed 2q+1 it is the complement within log_rows bits.
    __shared__ uint32_t even_m[32][33], odd_m[32][33];
    const uint32_t L = cfg.log_rows, qbits = L - 1, mid_bits = qbits - 10;
    const uint32_t mask = (1u << L) - 1u;
    const uint32_t n_tiles = 1u << mid_bits;
    const uint32_t lane = threadIdx.x & 31u, w = threadIdx.x >> 5;  // 8 warps
    // Tile `mid` and tile `~mid` read the even and the odd words of the same two address ranges, so a CTA takes them
    // back to back and the second one finds its lines in L2.
    const uint32_t n_items = n_tiles > 1 ? n_tiles : 2;
    for (uint32_t item = 2 * blockIdx.x; item < n_items; item += 2 * gridDim.x)
    for (uint32_t half = 0; half < 2; half++) {
        const uint32_t tile = half ? n_tiles - 1u - (item >> 1) : (item >> 1);
        if (half && n_tiles == 1) break;
        if (m_col) {
            // read phase: warp w covers lo = w, w+8, ...; lanes run over hi, i.e. over consecutive natural rows
            for (uint32_t lo = w; lo < 32; lo += 8) {
                uint32_t q = (lane << (qbits - 5)) | (tile << 5) | lo;
                uint32_t j0 = __brev(q) >> (32u - L);  // natural row of committed 2q
                uint32_t j1 = (~j0) & mask;           // natural row of committed 2q+1
                uint32_t s0 = 0, s1 = 0;
                for (uint32_t c = 0; c < cfg.n_counters; c++) {
                    const uint32_t* cnt = counters[c];
                    s0 += __ldg(cnt + j0);
                    s1 += __ldg(cnt + j1);
                }
                even_m[lane][lo] = s0;
                odd_m[lane][lo] = s1;
            }
            __syncthreads();
        }
        // write phase: warp w covers hi = w, w+8, ...; a warp writes 64 consecutive committed rows
        for (uint32_t hi = w; hi < 32; hi += 8) {
            uint32_t q = (hi << (qbits - 5)) | (tile << 5) | lane;
            uint32_t j0 = __brev(q) >> (32u - L), j1 = (~j0) & mask;
            uint2 xv = make_uint2(j0, j1);
            uint2 yv = make_uint2(__ldg(expmap + exp_pattern(j0, cfg)), __ldg(expmap + exp_pattern(j1, cfg)));
            reinterpret_cast<uint2*>(x_col)[q] = xv;
            reinterpret_cast<uint2*>(y_col)[q] = yv;
            if (m_col) reinterpret_cast<uint2*>(m_col)[q] = make_uint2(even_m[hi][lane], odd_m[hi][lane]);
        }
        if (m_col) __syncthreads();
    }
}

// Small tables (fewer than 2^11 rows): one thread per committed row.
__global__ void tables_small_kernel(const uint32_t* __restrict__ expmap, const uint32_t* const* __restrict__ counters,
                                    uint32_t* __restrict__ x_col, uint32_t* __restrict__ y_col, uint32_t* __restrict__ m_col, TabCfg cfg) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >> cfg.log_rows) return;
    uint32_t j = coset_perm(i, cfg.log_rows);
    x_col[i] = j;
    y_col[i] = __ldg(expmap + exp_pattern(j, cfg));
    if (m_col) {
        uint32_t s = 0;
        for (uint32_t c = 0; c < cfg.n_counters; c++) s += __ldg(counters[c] + j);
        m_col[i] = s;
    }
}

// Rows where this witness's own table differs from the closed form (one entry for the reference's corrupted-table
// probe, none otherwise): natural row idx[t] takes val[t].
__global__ void tables_patch_kernel(const uint32_t* __restrict__ idx, const uint32_t* __restrict__ val, uint32_t n, uint32_t* __restrict__ y_col,
                                    uint32_t log_rows) {
    uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n) y_col[coset_perm(idx[t], log_rows)] = val[t];
}

// ---------------------------------------------------------------------------------------------------
// Dequantize component. One thread owns one committed row and a tile of its slots; a warp therefore
// writes 128 consecutive bytes of every column it touches; the accumulators of a row's slots are
// consecutive in memory, so a thread walks one or two sectors of them. Multiplicities:
// the 8-bit range table is a shared-memory histogram flushed once per CTA; the three large tables take
// warp-aggregated atomics (lanes hitting the same row add once).
// ---------------------------------------------------------------------------------------------------
struct DeqArgs {
    const int32_t *acc, *jx, *jw;
    const uint32_t *sx, *sw, *norm3, *mul2;
    uint32_t* const* base;
    uint32_t* const* pre;
    uint32_t *m_norm, *m_frac, *m_mul, *m_r8, *counts, *want;
    zkb_dequant_cfg c;
    uint32_t slot_tile;
};

__device__ __forceinline__ void bump_agg(uint32_t* m, uint32_t idx) {
    uint32_t peers = __match_any_sync(__activemask(), idx);
    if ((threadIdx.x & 31u) == (uint32_t)(__ffs(peers) - 1)) atomicAdd(m + idx, (uint32_t)__popc(peers));
}

__device__ __forceinline__ uint32_t bf16_bits(uint32_t sg, uint32_t ef, uint32_t m7) { return ((sg << 15) | (ef << 7) | m7) & 0xffffu; }
__device__ __forceinline__ double bf16_value(uint32_t bits) { return (double)__uint_as_float(bits << 16); }

// One IEEE rounding of a normal double to bf16, ties to even (prover/src/bf16.rs:197-230, the in-range part).
__device__ __forceinline__ uint32_t bf16_round_f64(double x) {
    if (x == 0.0) return signbit(x) ? 0x8000u : 0u;
    unsigned long long u = (unsigned long long)__double_as_longlong(x);
    int e = (int)((u >> 52) & 0x7ffull) - 1023;
    unsigned long long man = u & ((1ull << 52) - 1ull);
    unsigned long long keep = man >> 45;
    bool round_bit = (man >> 44) & 1ull, sticky = (man & ((1ull << 44) - 1ull)) != 0ull;
    if (round_bit && (sticky || (keep & 1ull))) keep++;
    if (keep == 128ull) { keep = 0; e++; }
    return bf16_bits((uint32_t)(u >> 63), (uint32_t)(e + 127), (uint32_t)keep);
}

template <int CHAIN>
__global__ void __launch_bounds__(128) dequant_kernel(const DeqArgs a) {
    extern __shared__ __align__(16) uint32_t r8_hist[];
    const zkb_dequant_cfg& c = a.c;
    for (uint32_t k = threadIdx.x; k < c.n_r8; k += blockDim.x) r8_hist[k] = 0;
    // The column addresses of this CTA's slots, once per CTA: every store of every thread would otherwise start with a
    // dependent read of the pointer table.
    uint32_t** s_base = reinterpret_cast<uint32_t**>(r8_hist + ((c.n_r8 + 3u) & ~3u));  // [slot in tile][field]
    uint32_t** s_pre = s_base + a.slot_tile * c.per_slot;                               // [slot in tile][scale column]
    {
        const uint32_t s0 = blockIdx.y * a.slot_tile, ns = min(c.per_row - s0, a.slot_tile);
        for (uint32_t k = threadIdx.x; k < ns * c.per_slot; k += blockDim.x) s_base[k] = a.base[c.slot0 + s0 * c.per_slot + k];
        for (uint32_t k = threadIdx.x; k < ns * c.chan_w; k += blockDim.x) s_pre[k] = a.pre[c.chan_w * s0 + k];
    }
    __syncthreads();
    const uint32_t rows = 1u << c.log_rows;
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    uint32_t off_table = 0, ref_bad = 0, no_row = 0;
    if (i < rows) {
        const uint32_t j = coset_perm(i, c.log_rows);
        const uint32_t t = c.tokens - 1u - j / c.chunks, jm = j % c.chunks, b = c.chunks - 1u - jm;
        const uint32_t s_begin = blockIdx.y * a.slot_tile, s_end = min(c.per_row, s_begin + a.slot_tile);
        uint32_t sx_m = 0, sx_e = 0;
        int jx_t = 0;
        if (CHAIN) { sx_m = __ldg(a.sx + 2u * t); sx_e = __ldg(a.sx + 2u * t + 1u); }
        else jx_t = __ldg(a.jx + t);
        if (blockIdx.y == 0) {
            // the row's shared columns (the activation's scale) and the five selectors that close the preprocessed columns
            if (CHAIN) { a.base[c.sh0][i] = sx_m; a.base[c.sh1][i] = sx_e; }
            else a.base[c.sh0][i] = m31_of(jx_t);
            const uint32_t last = jm == c.chunks - 1u, sel0 = c.chan_w * c.per_row;
            a.pre[sel0 + 0][i] = jm != 0u;
            a.pre[sel0 + 1][i] = last;
            a.pre[sel0 + 2][i] = j > 0u && !last;
            a.pre[sel0 + 3][i] = j > 0u && last;
            a.pre[sel0 + 4][i] = j + 1u == rows;
        }
        const int32_t* acc_row = a.acc + (size_t)t * c.n_out + (size_t)b * c.per_row;
        for (uint32_t s = s_begin; s < s_end; s++) {
            const uint32_t ch = b * c.per_row + s;
            uint32_t* const* col = s_base + (s - s_begin) * c.per_slot;  // col[field] is the slot's column of that field
            uint32_t* const* pcol = s_pre + (s - s_begin) * c.chan_w;
            uint32_t sw_m = 0, sw_e = 0;
            int jw_c = 0;
            if (CHAIN) {
                sw_m = __ldg(a.sw + 2u * ch);
                sw_e = __ldg(a.sw + 2u * ch + 1u);
                pcol[0][i] = sw_m;
                pcol[1][i] = sw_e;
            } else {
                jw_c = __ldg(a.jw + ch);
                pcol[0][i] = m31_of(jw_c);
            }
            const long long av = __ldg(acc_row + s);
            col[c.f_acc][i] = m31_of(av);
            const uint32_t sg = av < 0;
            const unsigned long long mag = (unsigned long long)(av < 0 ? -av : av);
            // mag = m2 * ph + r with a 9-bit extended significand m2 (prover/src/bf16.rs:300-316)
            uint32_t m2 = 0, ph = 0, st = 0, k = 0;
            unsigned long long r = 0;
            if (mag) {
                uint32_t bits = 64u - (uint32_t)__clzll((long long)mag);
                k = bits > 9u ? bits - 9u : 0u;
                ph = 1u << (k & 31u);
                m2 = (uint32_t)(mag >> k);
                r = mag & ((1ull << k) - 1ull);
                st = (r != 0ull) && c.sticky;
            }
            // row indices of the normalisation and fraction tables (prover/src/layer.rs:2042-2068)
            uint32_t ri = NONE, fi = NONE;
            if (k <= c.kmax) {
                if (!mag) ri = 0;
                else if (m2 < 256u) ri = m2;  // then k = 0, ph = 1, r = 0
                else ri = 256u + (k * 256u + (m2 - 256u)) * (1u + c.sticky) + st;
                fi = ph + (uint32_t)r;
            }
            if (ri >= c.n_norm || fi >= c.n_frac) { no_row++; continue; }
            const uint32_t n_m7 = __ldg(a.norm3 + 3u * ri), n_ef = __ldg(a.norm3 + 3u * ri + 1u), n_nz = __ldg(a.norm3 + 3u * ri + 2u);
            bump_agg(a.m_norm, ri);
            bump_agg(a.m_frac, fi);
            col[c.f_sg][i] = sg;
            col[c.f_m2][i] = m2;
            col[c.f_ph][i] = ph;
            if (c.sticky) col[c.f_st][i] = st;
            col[c.f_r][i] = (uint32_t)r;
            col[c.f_m7][i] = n_m7;
            col[c.f_ef][i] = n_ef;
            col[c.f_nz][i] = n_nz;
            uint32_t got;
            if (!CHAIN) {
                const long long shift = (long long)jx_t + jw_c;
                const long long eo = n_nz == 1u ? (long long)n_ef + shift : 0;
                col[c.f_eo][i] = m31_of(eo);
                if (eo >= 0 && eo < (long long)c.n_r8) atomicAdd(&r8_hist[eo], 1u); else off_table++;
                got = bf16_bits(sg, (uint32_t)(eo > 0 ? eo : 0), n_m7);
                if (c.do_ref) {
                    // the accumulator times a power of two is exact in double, so this is one rounding
                    uint32_t want = bf16_round_f64(ldexp((double)av, (int)shift));
                    ref_bad += want != got;
                    if (a.want) a.want[(size_t)j * c.per_row + s] = want;
                }
            } else {
                uint32_t m_in = n_m7;
                long long e_in = n_ef;
                for (uint32_t step = 0; step < 2u; step++) {
                    const uint32_t ms = step ? sw_m : sx_m;
                    const long long es = step ? sw_e : sx_e;
                    const uint32_t mi = m_in * 128u + ms;
                    if (mi >= c.n_mul) { no_row++; break; }
                    uint32_t po = 0, ca = 0;
                    if (n_nz == 1u) { po = __ldg(a.mul2 + 2u * mi); ca = __ldg(a.mul2 + 2u * mi + 1u); }
                    const long long eo = n_nz == 1u ? e_in + es - 127 + (long long)ca : 0;
                    col[c.f_mul[3u * step + 0u]][i] = po;
                    col[c.f_mul[3u * step + 1u]][i] = ca;
                    col[c.f_mul[3u * step + 2u]][i] = m31_of(eo);
                    if (n_nz == 1u) bump_agg(a.m_mul, mi);
                    if (eo >= 0 && eo < (long long)c.n_r8) atomicAdd(&r8_hist[eo], 1u); else off_table++;
                    m_in = po;
                    e_in = eo;
                }
                got = bf16_bits(sg, (uint32_t)(e_in > 0 ? e_in : 0), m_in);
                if (c.do_ref) {
                    // two double products, each rounded to bf16 (no addition that could contract into an FMA)
                    double y0 = bf16_value(bf16_round_f64((double)(long long)mag));
                    double t1 = bf16_value(bf16_round_f64(__dmul_rn(y0, bf16_value(bf16_bits(0, sx_e, sx_m)))));
                    uint32_t want = bf16_round_f64(__dmul_rn(t1, bf16_value(bf16_bits(0, sw_e, sw_m)))) | (sg << 15);
                    ref_bad += want != got;
                    if (a.want) a.want[(size_t)j * c.per_row + s] = want;
                }
            }
        }
    }
    if (off_table) atomicAdd(a.counts + 0, off_table);
    if (ref_bad) atomicAdd(a.counts + 1, ref_bad);
    if (no_row) atomicAdd(a.counts + 2, no_row);
    __syncthreads();
    for (uint32_t k = threadIdx.x; k < c.n_r8; k += blockDim.x)
        if (r8_hist[k]) atomicAdd(a.m_r8 + k, r8_hist[k]);
}

}  // namespace zk

using namespace zk;

extern "C" {

int zkb_witness_tables(zkb_ctx* ctx, const uint32_t* expmap, const uint32_t* const* counters, uint32_t n_counters, const uint32_t* patch_idx,
                       const uint32_t* patch_val, uint32_t n_patch, uint32_t log_rows, int bf16x, double two_pow, uint32_t* x_col,
                       uint32_t* y_col, uint32_t* m_col) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, expmap && x_col && y_col && log_rows >= 1 && log_rows <= 30);
    ZKB_CHECK_ARG(ctx, (n_counters == 0 || counters) && n_counters <= 4096 && (n_patch == 0 || (patch_idx && patch_val)));
    ZKB_CHECK_ARG(ctx, bf16x || two_pow > 0.0);
    DeviceGuard g(ctx);
    void** d_cnt = nullptr;
    if (n_counters) {
        for (uint32_t c = 0; c < n_counters; c++) ZKB_CHECK_ARG(ctx, counters[c] != nullptr);
        int rc = stage_ptrs(ctx, (const void* const*)counters, (int)n_counters, &d_cnt);
        if (rc) return rc;
    }
    TabCfg cfg{log_rows, n_counters, bf16x ? 1u : 0u, two_pow};
    {
        ProfScope prof(ctx, "witness_tables_kernel");
        if (log_rows >= 11) {
            uint32_t n_pairs = log_rows > 11 ? 1u << (log_rows - 12) : 1u;
            uint32_t grid = n_pairs < 148u * 8u ? n_pairs : 148u * 8u;
            tables_tiled_kernel<<<grid, 256, 0, ctx->stream>>>(expmap, (const uint32_t* const*)d_cnt, x_col, y_col, m_col, cfg);
        } else {
            uint32_t rows = 1u << log_rows;
            tables_small_kernel<<<(rows + 255) / 256, 256, 0, ctx->stream>>>(expmap, (const uint32_t* const*)d_cnt, x_col, y_col, m_col, cfg);
        }
        ZKB_LAUNCH_CHECK(ctx);
    }
    if (n_patch) {
        tables_patch_kernel<<<(n_patch + 255) / 256, 256, 0, ctx->stream>>>(patch_idx, patch_val, n_patch, y_col, log_rows);
        ZKB_LAUNCH_CHECK(ctx);
    }
    return ZKB_OK;
}

int zkb_witness_dequant(zkb_ctx* ctx, const int32_t* acc, const int32_t* jx, const int32_t* jw, const uint32_t* sx, const uint32_t* sw,
                        const uint32_t* norm3, const uint32_t* mul2, uint32_t* const* base_cols, uint32_t n_base, uint32_t* const* pre_cols,
                        uint32_t n_pre, uint32_t* m_norm, uint32_t* m_frac, uint32_t* m_mul, uint32_t* m_r8, uint32_t* counts,
                        uint32_t* want_out, const zkb_dequant_cfg* cfg) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, cfg && acc && norm3 && base_cols && pre_cols && m_norm && m_frac && m_r8 && counts);
    const zkb_dequant_cfg& c = *cfg;
    ZKB_CHECK_ARG(ctx, c.variant <= 1 && c.log_rows >= 1 && c.log_rows <= 30 && c.per_row >= 1 && c.chunks >= 1 && c.tokens >= 1);
    ZKB_CHECK_ARG(ctx, (uint64_t)c.tokens * c.chunks == (1ull << c.log_rows) && (uint64_t)c.chunks * c.per_row == c.n_out);
    ZKB_CHECK_ARG(ctx, c.variant == 1 ? (sx && sw && mul2 && m_mul && c.chan_w == 2) : (jx && jw && c.chan_w == 1));
    ZKB_CHECK_ARG(ctx, c.n_r8 >= 1 && c.n_r8 <= 8192 && c.kmax <= 30 && c.sticky <= 1);
    ZKB_CHECK_ARG(ctx, n_pre == c.chan_w * c.per_row + 5 && (uint64_t)c.slot0 + (uint64_t)c.per_row * c.per_slot <= n_base);
    const uint32_t fields[] = {c.f_acc, c.f_sg, c.f_m2, c.f_ph, c.f_r, c.f_m7, c.f_ef, c.f_nz};
    for (uint32_t f : fields) ZKB_CHECK_ARG(ctx, f < c.per_slot);
    ZKB_CHECK_ARG(ctx, (!c.sticky || c.f_st < c.per_slot) && c.sh0 < n_base && (c.variant == 0 || c.sh1 < n_base));
    if (c.variant == 0) ZKB_CHECK_ARG(ctx, c.f_eo < c.per_slot);
    else for (int k = 0; k < 6; k++) ZKB_CHECK_ARG(ctx, c.f_mul[k] < c.per_slot);
    DeviceGuard g(ctx);
    void **d_base, **d_pre;
    int rc = stage_ptrs(ctx, (const void* const*)base_cols, (int)n_base, &d_base);
    if (rc) return rc;
    rc = stage_ptrs(ctx, (const void* const*)pre_cols, (int)n_pre, &d_pre);
    if (rc) return rc;
    const uint32_t rows = 1u << c.log_rows, gx = (rows + 127) / 128;
    // Slots per thread. A slot is a chain of dependent table reads, so the kernel lives on the number of warps in flight:
    // as few slots per thread as it takes to reach 32 CTAs (128 warps) per SM, and never more than four.
    uint32_t slot_tile = c.per_row < 4 ? c.per_row : 4;
    while (slot_tile > 1 && (uint64_t)gx * ((c.per_row + slot_tile - 1) / slot_tile) < 148u * 32u) slot_tile = (slot_tile + 1) / 2;
    DeqArgs a{acc, jx, jw, sx, sw, norm3, mul2, (uint32_t* const*)d_base, (uint32_t* const*)d_pre, m_norm, m_frac, m_mul, m_r8, counts,
              want_out, c, slot_tile};
    dim3 grid(gx, (c.per_row + slot_tile - 1) / slot_tile);
    ProfScope prof(ctx, "witness_dequant_kernel");
    const size_t smem = (size_t)((c.n_r8 + 3u) & ~3u) * 4 + (size_t)slot_tile * (c.per_slot + c.chan_w) * sizeof(uint32_t*);
    if (c.variant == 1) dequant_kernel<1><<<grid, 128, smem, ctx->stream>>>(a);
    else dequant_kernel<0><<<grid, 128, smem, ctx->stream>>>(a);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

}  // extern "C"
