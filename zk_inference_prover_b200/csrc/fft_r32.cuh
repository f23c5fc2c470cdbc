// Radix-32 register stages for the circle FFT.
//
// A pass covers a window of 10 index bits [lo, lo+10): 1024 "rows" m. Every thread keeps 32 values
// in registers and runs up to 5 butterfly layers on them without touching memory; one exchange
// through shared memory sits between the two stages of a pass:
//   stage 1 (window bits 5..9): the thread holds rows m = tm + 32 p, p = 0..31
//   stage 2 (window bits 0..4): the thread holds rows m = 32 tm + p
// In stage 1 the twiddle of a butterfly depends only on p and on the bits above the window, so it is
// the same for every thread of the CTA; in stage 2 it depends on tm. Either way a thread loads each
// twiddle once (31 + 15 loads for 160 butterflies).
//
// Two thread mappings share the per-thread code:
//   contiguous pass (lo = 0): one warp owns 1024 consecutive words of one column; the exchange is
//     warp-private (33-word row pitch, no bank conflicts, __syncwarp only);
//   strided pass (lo >= 3): a CTA of 256 threads owns 1024 rows x 8 consecutive words; thread
//     (tm = tid / 8, w = tid % 8); global accesses are runs of 32 bytes.
//
// The butterfly multiplies by a pre-doubled twiddle: with t2 = 2t, the 64-bit product t2 * v splits
// as hi = (t v) >> 31 and lo / 2 = (t v) mod 2^31, whose sum is congruent to t v and below 2p.
#pragma once
#include <type_traits>

#include "common.cuh"

namespace zk {

__device__ __forceinline__ uint32_t m31_mul_dbl(uint32_t v, uint32_t t2) {
    uint64_t p = (uint64_t)v * t2;
    uint32_t s = (uint32_t)(p >> 32) + ((uint32_t)p >> 1);
    return umin32(s, s - P);
}

// Forward: (a, b) -> (a + t b, a - t b); with NEG the twiddle is -t.
template <bool NEG>
__device__ __forceinline__ void bf_fwd(uint32_t& a, uint32_t& b, uint32_t t2) {
    uint32_t s = m31_mul_dbl(b, t2);
    uint32_t x = m31_add(a, s), y = m31_sub(a, s);
    a = NEG ? y : x;
    b = NEG ? x : y;
}
// Inverse: (a, b) -> (a + b, (a - b) t); with NEG the twiddle is -t.
template <bool NEG>
__device__ __forceinline__ void bf_inv(uint32_t& a, uint32_t& b, uint32_t t2) {
    uint32_t d = NEG ? m31_sub(b, a) : m31_sub(a, b);
    a = m31_add(a, b);
    b = m31_mul_dbl(d, t2);
}

// CNT consecutive twiddles, fetched with the widest loads (the tables are aligned to their length).
template <int CNT>
__device__ __forceinline__ void load_tw(const uint32_t* __restrict__ p, uint32_t (&t)[16]) {
    if constexpr (CNT >= 4) {
#pragma unroll
        for (int q = 0; q < CNT / 4; q++) {
            uint4 x = reinterpret_cast<const uint4*>(p)[q];
            t[4 * q] = x.x; t[4 * q + 1] = x.y; t[4 * q + 2] = x.z; t[4 * q + 3] = x.w;
        }
    } else if constexpr (CNT == 2) {
        uint2 x = *reinterpret_cast<const uint2*>(p);
        t[0] = x.x; t[1] = x.y;
    } else {
        t[0] = p[0];
    }
}

// Five layers on 32 registers. Layer jj pairs p with p + 2^jj and uses the 16 >> jj twiddles at
// tb[jj] (global or shared memory): tb[jj][p >> (jj+1)].
// Layers outside [act_lo, act_hi) (window-local numbering, this stage starts at `first`) are skipped.
// When CIRCLE, layer jj = 0 is the circle layer (global layer 0): its twiddles are [y, -y, -x, x]
// for each pair (x, y) of the eight layer-1 twiddles at tb[0] (cpu/circle.rs:312-332).
// With DBL the table already holds doubled twiddles (2t) and nothing is shifted here.
template <bool INVERSE, bool CIRCLE, bool DBL = false>
__device__ __forceinline__ void radix32_stage(uint32_t (&v)[32], const uint32_t* const (&tb)[5], int first, int act_lo, int act_hi) {
    uint32_t t[16];
    auto layer = [&](auto JJ) {
        constexpr int jj = decltype(JJ)::value;
        if (first + jj < act_lo || first + jj >= act_hi) return;
        if constexpr (CIRCLE && jj == 0) {
            load_tw<8>(tb[0], t);
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const uint32_t x2 = DBL ? t[2 * q] : t[2 * q] << 1, y2 = DBL ? t[2 * q + 1] : t[2 * q + 1] << 1;
                if (INVERSE) {
                    bf_inv<false>(v[8 * q + 0], v[8 * q + 1], y2);
                    bf_inv<true>(v[8 * q + 2], v[8 * q + 3], y2);
                    bf_inv<true>(v[8 * q + 4], v[8 * q + 5], x2);
                    bf_inv<false>(v[8 * q + 6], v[8 * q + 7], x2);
                } else {
                    bf_fwd<false>(v[8 * q + 0], v[8 * q + 1], y2);
                    bf_fwd<true>(v[8 * q + 2], v[8 * q + 3], y2);
                    bf_fwd<true>(v[8 * q + 4], v[8 * q + 5], x2);
                    bf_fwd<false>(v[8 * q + 6], v[8 * q + 7], x2);
                }
            }
        } else {
            load_tw<(16 >> jj)>(tb[jj], t);
#pragma unroll
            for (int h = 0; h < (16 >> jj); h++) {
                const uint32_t t2 = DBL ? t[h] : t[h] << 1;
#pragma unroll
                for (int l = 0; l < (1 << jj); l++) {
                    const int p0 = (h << (jj + 1)) | l, p1 = p0 | (1 << jj);
                    if (INVERSE) bf_inv<false>(v[p0], v[p1], t2);
                    else bf_fwd<false>(v[p0], v[p1], t2);
                }
            }
        }
    };
    if (INVERSE) {
        layer(std::integral_constant<int, 0>{}); layer(std::integral_constant<int, 1>{}); layer(std::integral_constant<int, 2>{});
        layer(std::integral_constant<int, 3>{}); layer(std::integral_constant<int, 4>{});
    } else {
        layer(std::integral_constant<int, 4>{}); layer(std::integral_constant<int, 3>{}); layer(std::integral_constant<int, 2>{});
        layer(std::integral_constant<int, 1>{}); layer(std::integral_constant<int, 0>{});
    }
}

// ---- asynchronous global -> shared copies (16 bytes each), grouped and waited on per thread
__device__ __forceinline__ void cp_async16(uint32_t* smem_dst, const uint32_t* gmem_src) {
    unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t* smem_dst, const uint32_t* gmem_src) {
    unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

constexpr int R32_CONTIG_WARPS = 8;    // warps per CTA of the contiguous pass; each runs its own pipeline
constexpr int R32_PITCH = 36;          // words per staged row of 32 in the contiguous pass
// Every pass also stages the twiddles of the next work item (cp.async, same group as its data): the
// twiddles a thread needs are short consecutive runs of the tower, different for every item.
//   contiguous: [0,480) the per-thread stage (layers 1..4: 256 + 128 + 64 + 32 words; the circle layer reuses
//               the layer-1 run), [480,511) the CTA-uniform stage (layers 5..9: 16 + 8 + 4 + 2 + 1 words)
//   strided:    [0,992) the per-thread stage (512 + 256 + 128 + 64 + 32), [992,1023) the uniform stage
constexpr int R32_TW_CONTIG = 512;
constexpr int R32_TW_STRIDED = 1024;
__host__ __device__ constexpr size_t r32_contig_smem(bool inverse) {
    (void)inverse;
    return (size_t)R32_CONTIG_WARPS * 2 * (R32_PITCH * 32 + R32_TW_CONTIG) * sizeof(uint32_t);
}
__host__ __device__ constexpr size_t r32_strided_smem(int lw) {
    return (size_t)(2 * 33 * 32 * (1 << lw) + R32_TW_STRIDED) * sizeof(uint32_t);
}
// Word k (0..30) of a uniform-stage block: layer jj and index h within its run of 16 >> jj.
__device__ __forceinline__ void uniform_slot(int k, int& jj, int& h) {
    jj = (k >= 16) + (k >= 24) + (k >= 28) + (k >= 30);
    h = k - (32 - (32 >> jj));
}

struct R32Pass {
    int lo;              // first index bit of the window
    int act_lo, act_hi;  // active layers, window-local: [act_lo, act_hi) within 0..10
};

// Both kernels are persistent: a CTA (strided) or a warp (contiguous) walks over work items
// (tile, column) and, while it computes one item from shared memory, the next item's words are
// already on their way from HBM (cp.async into the other staging buffer). The buffer an item
// arrived in is reused for that item's stage exchange once every value has been read from it.

// Contiguous pass: window bits [0, 10). One warp per 1024 consecutive words.
// Staging layout: the unit's 32 rows of 32 words at a pitch of 36 words (R32_PITCH). Both access patterns of
// the two register stages are then free of bank conflicts: (row p, word tm) at word 36 p + tm hits 32
// distinct banks, and row tm read as eight 16-byte chunks (chunk q at 36 tm + 4 q) puts the eight lanes of a
// quarter-warp on eight distinct 4-bank groups (36 = 4 mod 32). The exchange between the stages and, in the
// forward direction, the transposition of the output run in place in the buffer the unit arrived in.
// Forward output: after the last stage a lane holds 32 consecutive words; storing them directly would touch
// 32 different 128-byte lines per instruction, so the rows go back to shared memory and are written out with
// eight lanes per line (lane 8 j + c stores chunk c of row 4 s + j): four full lines per store instruction.
// `tower` holds doubled twiddles (2t).
template <bool INVERSE>
__global__ void __launch_bounds__(32 * R32_CONTIG_WARPS, 16 / R32_CONTIG_WARPS)
    fft_r32_contig_kernel(uint32_t* const* __restrict__ dst_cols, const uint32_t* const* __restrict__ src_cols,
                          uint32_t src_mask, int ncols, int log_n, int dom_log, R32Pass ps,
                          const uint32_t* __restrict__ tower, uint32_t scale) {
    extern __shared__ __align__(16) uint32_t dyn_smem[];
    const int warp = threadIdx.x >> 5, tm = threadIdx.x & 31;
    constexpr int BUF = R32_PITCH * 32;
    uint32_t* const buf0 = dyn_smem + (2 * warp) * BUF;
    uint32_t* const tw0 = dyn_smem + 2 * R32_CONTIG_WARPS * BUF + (2 * warp) * R32_TW_CONTIG;
    const int unit_bits = log_n - 10;
    const size_t total = (size_t)ncols << unit_bits;
    // Items are ordered column-major (unit index fastest) and dealt round-robin, so at any time
    // the whole grid streams through neighbouring units of the same few columns. (Dealing each
    // worker a run of columns of one unit instead measured 1.5x slower: every access then lands
    // in a different 16 MiB column.)
    const size_t stride = (size_t)gridDim.x * R32_CONTIG_WARPS;
    size_t item = (size_t)blockIdx.x * R32_CONTIG_WARPS + warp;
    const size_t item_end = total;

    auto prefetch = [&](int b, size_t it) {
        uint32_t* buf = buf0 + b * BUF;
        const uint32_t* __restrict__ src = src_cols[it >> unit_bits];
        const uint32_t un = (uint32_t)(it & (((size_t)1 << unit_bits) - 1));
        const uint32_t base = un << 10;
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const int r = k * 4 + (tm >> 3), q = tm & 7;  // chunk c = 32 k + tm: row c / 8, chunk c % 8
            cp_async16(buf + r * R32_PITCH + (q << 2), src + ((base + r * 32 + q * 4) & src_mask));
        }
        {
            uint32_t* tw = tw0 + b * R32_TW_CONTIG;
            // per-thread stage: chunk c of 120 (16 bytes each): layers 1, 2, 3, 4 hold 64, 32, 16, 8 chunks
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int c = 32 * k + tm;
                if (c < 120) {
                    const int jj = 1 + (c >= 64) + (c >= 96) + (c >= 112);
                    const int cc = c - (128 - (256 >> jj));
                    cp_async16(tw + 4 * c, tower + (1u << (dom_log - jj - 1)) + (un << (9 - jj)) + 4 * cc);
                }
            }
            if (tm < 31) {
                int jj, h;
                uniform_slot(tm, jj, h);
                cp_async4(tw + 480 + tm, tower + (1u << (dom_log - 5 - jj - 1)) + (un << (4 - jj)) + h);
            }
        }
    };

    int cur = 0;
    if (item < item_end) prefetch(0, item);
    cp_async_commit();
    for (; item < item_end; item += stride) {
        if (item + stride < item_end) prefetch(cur ^ 1, item + stride);
        cp_async_commit();
        cp_async_wait<1>();
        __syncwarp();
        uint32_t* __restrict__ s = buf0 + cur * BUF;
        uint32_t* __restrict__ dst = dst_cols[item >> unit_bits];
        const uint32_t unit = (uint32_t)(item & (((size_t)1 << unit_bits) - 1));
        const uint32_t base = unit << 10;
        const uint32_t* tw = tw0 + cur * R32_TW_CONTIG;
        const uint32_t* const tb_uni[5] = {tw + 480, tw + 496, tw + 504, tw + 508, tw + 510};
        const uint32_t* const tb_lane[5] = {tw + 8 * tm, tw + 8 * tm, tw + 256 + 4 * tm, tw + 384 + 2 * tm, tw + 448 + tm};
        uint4* const row = reinterpret_cast<uint4*>(s + R32_PITCH * tm);
        uint32_t v[32];
        if (!INVERSE) {
#pragma unroll
            for (int p = 0; p < 32; p++) v[p] = s[R32_PITCH * p + tm];
            radix32_stage<false, false, true>(v, tb_uni, 5, ps.act_lo, ps.act_hi);
#pragma unroll
            for (int p = 0; p < 32; p++) s[R32_PITCH * p + tm] = v[p];  // the words this lane read itself
            __syncwarp();
#pragma unroll
            for (int q = 0; q < 8; q++) {
                uint4 x = row[q];
                v[4 * q] = x.x; v[4 * q + 1] = x.y; v[4 * q + 2] = x.z; v[4 * q + 3] = x.w;
            }
            radix32_stage<false, true, true>(v, tb_lane, 0, ps.act_lo, ps.act_hi);
#pragma unroll
            for (int q = 0; q < 8; q++) row[q] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            __syncwarp();
            const int j = tm >> 3, c = tm & 7;
#pragma unroll
            for (int st = 0; st < 8; st++) {
                const int r = 4 * st + j;
                const uint4 x = *reinterpret_cast<const uint4*>(s + R32_PITCH * r + 4 * c);
                *reinterpret_cast<uint4*>(dst + base + 32 * r + 4 * c) = x;
            }
        } else {
#pragma unroll
            for (int q = 0; q < 8; q++) {
                uint4 x = row[q];
                v[4 * q] = x.x; v[4 * q + 1] = x.y; v[4 * q + 2] = x.z; v[4 * q + 3] = x.w;
            }
            radix32_stage<true, true, true>(v, tb_lane, 0, ps.act_lo, ps.act_hi);
#pragma unroll
            for (int q = 0; q < 8; q++) row[q] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            __syncwarp();
#pragma unroll
            for (int p = 0; p < 32; p++) v[p] = s[R32_PITCH * p + tm];
            radix32_stage<true, false, true>(v, tb_uni, 5, ps.act_lo, ps.act_hi);
#pragma unroll
            for (int p = 0; p < 32; p++) dst[base + tm + 32 * p] = scale ? m31_mul(v[p], scale) : v[p];
        }
        __syncwarp();  // the exchange reads are done before this buffer is refilled
        cur ^= 1;
    }
    cp_async_wait<0>();
}

__host__ __device__ constexpr int r32_strided_min_ctas(bool inverse, int lw) {
    return lw >= 4 ? 1 : lw == 3 ? (inverse ? 3 : 2) : (inverse ? 6 : 4);
}
// Strided pass: window bits [lo, lo+10), lo >= LW. CTA = 1024 rows x W = 2^LW consecutive words (W = 8 or 4).
// Staging and exchange share one layout: row m at word W m + W (m / 32).
// The twiddles of a tile depend only on the bits above the window (`a`), so a CTA keeps one value of `a` for
// its whole life whenever the grid allows it (blockIdx mod the number of values) and loads that table of
// 1023 doubled twiddles into shared memory once; otherwise it reloads the table when `a` changes.
template <bool INVERSE, int LW>
__global__ void __launch_bounds__(32 << LW, r32_strided_min_ctas(INVERSE, LW))
    fft_r32_strided_kernel(uint32_t* const* __restrict__ dst_cols, const uint32_t* const* __restrict__ src_cols,
                           uint32_t src_mask, int ncols, int log_n, int dom_log, R32Pass ps,
                           const uint32_t* __restrict__ tower, uint32_t scale) {
    extern __shared__ __align__(16) uint32_t dyn_smem[];
    uint32_t* const buf0 = dyn_smem;
    constexpr int W = 1 << LW, NT = 32 << LW;  // words per row of the tile, threads of the CTA
    constexpr int BUF = 33 * 32 * W;            // row m at word W m + W (m / 32)
    uint32_t* const tw = dyn_smem + 2 * BUF;
    const uint32_t w = threadIdx.x & (W - 1), tm = threadIdx.x >> LW;
    const int wb_bits = ps.lo - LW;                // tiles across the words below the window
    const int a_bits = log_n - ps.lo - 10;         // values of the bits above the window
    const uint32_t n_a = 1u << a_bits;
    // Work space: (column, wb) pairs for a fixed `a` when the grid is a multiple of n_a, else (column, a, wb).
    const bool stationary = (gridDim.x % n_a) == 0;
    const size_t per_a = (size_t)ncols << wb_bits;
    const size_t total = stationary ? per_a : per_a << a_bits;
    const size_t stride = stationary ? gridDim.x / n_a : gridDim.x;
    size_t item = stationary ? blockIdx.x / n_a : blockIdx.x;
    const uint32_t a_fixed = blockIdx.x % n_a;

    auto decode = [&](size_t it, uint32_t& col, uint32_t& a) {
        uint32_t wb;
        if (stationary) {
            col = (uint32_t)(it >> wb_bits);
            wb = (uint32_t)it & ((1u << wb_bits) - 1u);
            a = a_fixed;
        } else {
            col = (uint32_t)(it >> (wb_bits + a_bits));
            const uint32_t tile = (uint32_t)it & ((1u << (wb_bits + a_bits)) - 1u);
            wb = tile & ((1u << wb_bits) - 1u);
            a = tile >> wb_bits;
        }
        return (a << (ps.lo + 10)) | (wb << LW);
    };
    auto prefetch = [&](int b, size_t it) {
        uint32_t* buf = buf0 + b * BUF;
        uint32_t col, a;
        const uint32_t base = decode(it, col, a);
        const uint32_t* __restrict__ src = src_cols[col];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const uint32_t c = k * NT + threadIdx.x;  // 16-byte chunk: row c / (W/4), part c % (W/4)
            const uint32_t m = c / (W / 4), part = c % (W / 4);
            cp_async16(buf + W * m + W * (m >> 5) + 4 * part, src + ((base | (m << ps.lo) | (part << 2)) & src_mask));
        }
    };
    // [0,992) the per-thread stage (layers lo+0..lo+4: 512 + 256 + 128 + 64 + 32 words), [992,1023) the uniform stage
    auto load_twiddles = [&](uint32_t a) {
        for (int c = threadIdx.x; c < 248; c += NT) {  // chunk c of 248: layers lo+0..lo+4 hold 128, 64, 32, 16, 8 chunks
            const int jj = (c >= 128) + (c >= 192) + (c >= 224) + (c >= 240);
            const int cc = c - (256 - (256 >> jj));
            *reinterpret_cast<uint4*>(tw + 4 * c) =
                *reinterpret_cast<const uint4*>(tower + (1u << (dom_log - ps.lo - jj - 1)) + (a << (9 - jj)) + 4 * cc);
        }
        if (threadIdx.x < 31) {
            const int c = threadIdx.x;
            int jj, h;
            uniform_slot(c, jj, h);
            tw[992 + c] = tower[(1u << (dom_log - ps.lo - 5 - jj - 1)) + (a << (4 - jj)) + h];
        }
    };

    int cur = 0;
    uint32_t cur_a = 0xffffffffu;
    if (item < total) prefetch(0, item);
    cp_async_commit();
    for (; item < total; item += stride) {
        if (item + stride < total) prefetch(cur ^ 1, item + stride);
        cp_async_commit();
        uint32_t col, a;
        const uint32_t base = decode(item, col, a) | w;
        if (a != cur_a) {  // uniform over the CTA; the previous item's last barrier ordered every read of the old table
            load_twiddles(a);
            cur_a = a;
        }
        cp_async_wait<1>();
        __syncthreads();
        uint32_t* __restrict__ s = buf0 + cur * BUF;
        uint32_t* __restrict__ dst = dst_cols[col];
        const uint32_t* const tb_uni[5] = {tw + 992, tw + 1008, tw + 1016, tw + 1020, tw + 1022};
        const uint32_t* const tb_lane[5] = {tw + 16 * tm, tw + 512 + 8 * tm, tw + 768 + 4 * tm, tw + 896 + 2 * tm, tw + 960 + tm};
        uint32_t v[32];
        if (!INVERSE) {
#pragma unroll
            for (int p = 0; p < 32; p++) v[p] = s[33 * W * p + W * tm + w];
            radix32_stage<false, false, true>(v, tb_uni, 5, ps.act_lo, ps.act_hi);
            // each thread writes back exactly the words it read: no barrier needed before the write
#pragma unroll
            for (int p = 0; p < 32; p++) s[33 * W * p + W * tm + w] = v[p];
            __syncthreads();
#pragma unroll
            for (int p = 0; p < 32; p++) v[p] = s[33 * W * tm + W * p + w];
            radix32_stage<false, false, true>(v, tb_lane, 0, ps.act_lo, ps.act_hi);
#pragma unroll
            for (int p = 0; p < 32; p++) dst[base | ((32u * tm + p) << ps.lo)] = v[p];
        } else {
#pragma unroll
            for (int p = 0; p < 32; p++) v[p] = s[33 * W * tm + W * p + w];
            radix32_stage<true, false, true>(v, tb_lane, 0, ps.act_lo, ps.act_hi);
#pragma unroll
            for (int p = 0; p < 32; p++) s[33 * W * tm + W * p + w] = v[p];
            __syncthreads();
#pragma unroll
            for (int p = 0; p < 32; p++) v[p] = s[33 * W * p + W * tm + w];
            radix32_stage<true, false, true>(v, tb_uni, 5, ps.act_lo, ps.act_hi);
#pragma unroll
            for (int p = 0; p < 32; p++) {
                uint32_t x = scale ? m31_mul(v[p], scale) : v[p];
                dst[base | ((tm + 32u * p) << ps.lo)] = x;
            }
        }
        __syncthreads();  // exchange reads are done before this buffer is refilled
        cur ^= 1;
    }
    cp_async_wait<0>();
}

}  // namespace zk
