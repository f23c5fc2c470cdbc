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
__host__ __device__ constexpr size_t r32_contig_smem(bool inverse) {
    (void)inverse;
    return (size_t)R32_CONTIG_WARPS * 2 * (R32_PITCH * 32 + R32_TW_CONTIG) * sizeof(uint32_t);
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
// Destination layout in row blocks: word idx of a column lies at (idx >> log) * stride + (idx mod 2^log) from the
// column's base, i.e. consecutive blocks of 2^log rows are `stride` words apart (a sharded commitment lays the
// extended columns out by destination rank this way). log = 31 is the plain contiguous column. A block is at least
// 4096 words, so a tile row or a unit never straddles two blocks.
struct RowBlocks {
    int log;
    uint32_t stride;
};
__device__ __forceinline__ size_t blocked(uint32_t idx, RowBlocks rb) {
    return (size_t)(idx >> rb.log) * rb.stride + (idx & ((1u << rb.log) - 1u));
}

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

// ---------------------------------------------------------------------------------------------------------
// Wide strided pass: window bits [lo, lo+8), lo >= 5. A CTA of 256 threads owns a tile of 256 rows x 32
// consecutive words, so every global access is a full 128-byte line (a row of the tile), in both directions.
//   stage A (window bits 3..7, five layers): thread (warp, lane) holds rows warp + 8 p, p = 0..31, word lane;
//     its twiddles depend only on p and on the bits above the window;
//   stage B (window bits 0..2, three layers): thread (R = tid / 8, c = tid % 8) holds rows 8 R + q, q = 0..7,
//     as 16-byte chunks (words 4 c .. 4 c + 3): 128-bit shared loads and 128-bit global stores, eight lanes per line.
// The tile sits in shared memory densely (row m at word 32 m): stage A reads a row with one access per lane,
// stage B reads a row with a quarter-warp, so neither pattern has a bank conflict and nothing is padded.
// The twiddles of a tile depend only on the bits above the window (`a`): 255 words. A CTA keeps one value of
// `a` for its whole life whenever the grid is a multiple of the number of values, else it reloads on change.
constexpr int R32_WIDE_TILE = 256 * 32;  // words
#ifndef R32_WIDE_CTAS
#define R32_WIDE_CTAS 3
#endif
constexpr int R32_WIDE_TW = 256;         // [0,128) [128,192) [192,224): layers lo+0..lo+2; [224,255): layers lo+3..lo+7
__host__ __device__ constexpr size_t r32_wide_smem() { return (size_t)(2 * R32_WIDE_TILE + R32_WIDE_TW) * sizeof(uint32_t); }

// Three layers over the row index q of v[4 q + j] (eight rows x four words). tw0: 4, tw1: 2, tw2: 1 doubled twiddles.
template <bool INVERSE>
__device__ __forceinline__ void radix8x4_stage(uint32_t (&v)[32], const uint32_t* tw0, const uint32_t* tw1, const uint32_t* tw2,
                                               int act_lo, int act_hi) {
    auto layer = [&](auto JJ, const uint32_t* tw) {
        constexpr int jj = decltype(JJ)::value;
        if (jj < act_lo || jj >= act_hi) return;
        uint32_t t[4];
        if constexpr (jj == 0) { uint4 x = *reinterpret_cast<const uint4*>(tw); t[0] = x.x; t[1] = x.y; t[2] = x.z; t[3] = x.w; }
        else if constexpr (jj == 1) { uint2 x = *reinterpret_cast<const uint2*>(tw); t[0] = x.x; t[1] = x.y; }
        else t[0] = tw[0];
#pragma unroll
        for (int h = 0; h < (4 >> jj); h++) {
#pragma unroll
            for (int l = 0; l < (1 << jj); l++) {
                const int q0 = (h << (jj + 1)) | l, q1 = q0 | (1 << jj);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    if (INVERSE) bf_inv<false>(v[4 * q0 + j], v[4 * q1 + j], t[h]);
                    else bf_fwd<false>(v[4 * q0 + j], v[4 * q1 + j], t[h]);
                }
            }
        }
    };
    if (INVERSE) {
        layer(std::integral_constant<int, 0>{}, tw0); layer(std::integral_constant<int, 1>{}, tw1); layer(std::integral_constant<int, 2>{}, tw2);
    } else {
        layer(std::integral_constant<int, 2>{}, tw2); layer(std::integral_constant<int, 1>{}, tw1); layer(std::integral_constant<int, 0>{}, tw0);
    }
}

template <bool INVERSE>
__global__ void __launch_bounds__(256, R32_WIDE_CTAS)
    fft_r32_wide_kernel(uint32_t* const* __restrict__ dst_cols, const uint32_t* const* __restrict__ src_cols, uint32_t src_mask,
                        int ncols, int log_n, int dom_log, R32Pass ps, const uint32_t* __restrict__ tower, uint32_t scale, RowBlocks rb) {
    extern __shared__ __align__(16) uint32_t dyn_smem[];
    uint32_t* const buf0 = dyn_smem;
    constexpr int BUF = R32_WIDE_TILE;
    uint32_t* const tw = dyn_smem + 2 * BUF;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;  // stage A
    const uint32_t R = threadIdx.x >> 3, c = threadIdx.x & 7;         // stage B
    const int wb_bits = ps.lo - 5;          // tiles across the words below the window
    const int a_bits = log_n - ps.lo - 8;   // values of the bits above the window
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
        return (a << (ps.lo + 8)) | (wb << 5);
    };
    auto prefetch = [&](int b, size_t it) {
        uint32_t* buf = buf0 + b * BUF;
        uint32_t col, a;
        const uint32_t base = decode(it, col, a);
        const uint32_t* __restrict__ src = src_cols[col];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const uint32_t ch = k * 256 + threadIdx.x;  // 16-byte chunk: row ch / 8, part ch % 8
            const uint32_t m = ch >> 3, q = ch & 7;
            cp_async16(buf + 32 * m + 4 * q, src + ((base | (m << ps.lo) | (q << 2)) & src_mask));
        }
    };
    auto load_twiddles = [&](uint32_t a) {
        const int t = threadIdx.x;
        if (t < 224) {
            const int jj = (t >= 128) + (t >= 192);
            const int h = t - (256 - (256 >> jj));
            tw[t] = tower[(1u << (dom_log - ps.lo - jj - 1)) + (a << (7 - jj)) + h];
        } else if (t < 255) {
            int jj, h;
            uniform_slot(t - 224, jj, h);
            tw[t] = tower[(1u << (dom_log - ps.lo - 3 - jj - 1)) + (a << (4 - jj)) + h];
        }
    };

    int cur = 0;
    uint32_t cur_a = 0xffffffffu;
    if (item < total) prefetch(0, item);
    cp_async_commit();
    for (; item < total; item += stride) {
        uint32_t col, a;
        const uint32_t base = decode(item, col, a);
        cp_async_wait<0>();
        __syncthreads();
        // Past this barrier every thread has finished the previous tile, so the other buffer (and, when `a`
        // changes, the twiddle table) may be overwritten.
        if (item + stride < total) prefetch(cur ^ 1, item + stride);
        cp_async_commit();
        if (a != cur_a) {  // uniform over the CTA
            load_twiddles(a);
            cur_a = a;
            __syncthreads();
        }
        uint32_t* __restrict__ s = buf0 + cur * BUF;
        uint32_t* __restrict__ dst = dst_cols[col];
        const uint32_t* const tb_uni[5] = {tw + 224, tw + 240, tw + 248, tw + 252, tw + 254};
        uint32_t v[32];
        if (!INVERSE) {
#pragma unroll
            for (int p = 0; p < 32; p++) v[p] = s[32 * (warp + 8 * p) + lane];
            radix32_stage<false, false, true>(v, tb_uni, 3, ps.act_lo, ps.act_hi);
#pragma unroll
            for (int p = 0; p < 32; p++) s[32 * (warp + 8 * p) + lane] = v[p];  // the words this thread read itself
            __syncthreads();
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const uint4 x = *reinterpret_cast<const uint4*>(s + 32 * (8 * R + q) + 4 * c);
                v[4 * q] = x.x; v[4 * q + 1] = x.y; v[4 * q + 2] = x.z; v[4 * q + 3] = x.w;
            }
            radix8x4_stage<false>(v, tw + 4 * R, tw + 128 + 2 * R, tw + 192 + R, ps.act_lo, ps.act_hi);
#pragma unroll
            for (int q = 0; q < 8; q++)
                *reinterpret_cast<uint4*>(dst + blocked(base | ((8 * R + q) << ps.lo), rb) + 4 * c) =
                    make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        } else {
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const uint4 x = *reinterpret_cast<const uint4*>(s + 32 * (8 * R + q) + 4 * c);
                v[4 * q] = x.x; v[4 * q + 1] = x.y; v[4 * q + 2] = x.z; v[4 * q + 3] = x.w;
            }
            radix8x4_stage<true>(v, tw + 4 * R, tw + 128 + 2 * R, tw + 192 + R, ps.act_lo, ps.act_hi);
#pragma unroll
            for (int q = 0; q < 8; q++)
                *reinterpret_cast<uint4*>(s + 32 * (8 * R + q) + 4 * c) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            __syncthreads();
#pragma unroll
            for (int p = 0; p < 32; p++) v[p] = s[32 * (warp + 8 * p) + lane];
            radix32_stage<true, false, true>(v, tb_uni, 3, ps.act_lo, ps.act_hi);
#pragma unroll
            for (int p = 0; p < 32; p++) dst[(base | ((warp + 8 * p) << ps.lo)) + lane] = scale ? m31_mul(v[p], scale) : v[p];
        }
        cur ^= 1;
    }
    cp_async_wait<0>();
}

// ---------------------------------------------------------------------------------------------------------
// Contiguous pass over twelve layers: window bits [0, 12). A CTA of four warps owns 4096 consecutive words:
// four blocks of 1024, staged in the padded-row layout of the ten-layer pass (block b at b * 36 * 32). Layers
// 10 and 11 pair words 1024 and 2048 apart: every thread runs them as radix-4 butterflies on the four blocks'
// words at its own eight offsets (in place in shared memory); between that step and the ten layers each warp
// then runs on its own block (as in fft_r32_contig_kernel) sits one barrier of the four warps.
// Twiddles of the unit: layers 1..11 are runs of 1024 .. 1 words of the (doubled) tower, 2047 words in all.
constexpr int R32_C12_WARPS = 4;
constexpr int R32_C12_BUF = R32_C12_WARPS * R32_PITCH * 32;
constexpr int R32_C12_TW = 2048;
__host__ __device__ constexpr size_t r32_c12_smem() { return (size_t)2 * (R32_C12_BUF + R32_C12_TW) * sizeof(uint32_t); }

template <bool INVERSE>
__global__ void __launch_bounds__(32 * R32_C12_WARPS, 4)
    fft_r32_contig12_kernel(uint32_t* const* __restrict__ dst_cols, const uint32_t* const* __restrict__ src_cols, uint32_t src_mask,
                            int ncols, int log_n, int dom_log, R32Pass ps, const uint32_t* __restrict__ tower, uint32_t scale, RowBlocks rb,
                            int src_blocked) {
    extern __shared__ __align__(16) uint32_t dyn_smem[];
    constexpr int BLK = R32_PITCH * 32, BUF = R32_C12_BUF, NT = 32 * R32_C12_WARPS;
    uint32_t* const buf0 = dyn_smem;
    uint32_t* const tw0 = dyn_smem + 2 * BUF;
    const int warp = threadIdx.x >> 5, tm = threadIdx.x & 31, tid = threadIdx.x;
    const int unit_bits = log_n - 12;
    const size_t total = (size_t)ncols << unit_bits, stride = gridDim.x;
    size_t item = blockIdx.x;

    auto prefetch = [&](int b, size_t it) {
        uint32_t* buf = buf0 + b * BUF;
        const uint32_t* __restrict__ src = src_cols[it >> unit_bits];
        const uint32_t un = (uint32_t)(it & (((size_t)1 << unit_bits) - 1));
        const uint32_t base = un << 12;
        // an in-place pass over a column laid out in row blocks reads the unit where the pass before it wrote it
        const uint32_t* __restrict__ usrc = src_blocked ? src + blocked(base, rb) - base : src;
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const int ch = k * NT + tid;  // 16-byte chunk: block ch / 256, row (ch / 8) % 32, part ch % 8
            const int blk = ch >> 8, r = (ch >> 3) & 31, q = ch & 7;
            cp_async16(buf + blk * BLK + R32_PITCH * r + 4 * q, usrc + ((base + (blk << 10) + 32 * r + 4 * q) & src_mask));
        }
        uint32_t* tw = tw0 + b * R32_C12_TW;
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int ch = k * NT + tid;  // chunk of layers 1..9: layer jj holds 256 >> (jj - 1) chunks
            if (ch < 511) {
                const int jj = 9 - (31 - __clz(511 - ch));
                const int cc = ch - (512 - (512 >> (jj - 1)));
                cp_async16(tw + 4 * ch, tower + (1u << (dom_log - jj - 1)) + (un << (11 - jj)) + 4 * cc);
            }
        }
        if (tid < 2) cp_async4(tw + 2044 + tid, tower + (1u << (dom_log - 11)) + (un << 1) + tid);
        else if (tid == 2) cp_async4(tw + 2046, tower + (1u << (dom_log - 12)) + un);
    };
    // Layers 10 and 11 on the four blocks' words at offset o of a block.
    auto cross_blocks = [&](uint32_t* s, const uint32_t* tw, uint32_t* out, uint32_t out_scale) {
        const bool on10 = 10 >= ps.act_lo && 10 < ps.act_hi, on11 = 11 >= ps.act_lo && 11 < ps.act_hi;
        const uint32_t t10a = tw[2044], t10b = tw[2045], t11 = tw[2046];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int o = tid + NT * i;
            const int pos = R32_PITCH * (o >> 5) + (o & 31);
            uint32_t x0 = s[pos], x1 = s[BLK + pos], x2 = s[2 * BLK + pos], x3 = s[3 * BLK + pos];
            if (!INVERSE) {
                if (on11) { bf_fwd<false>(x0, x2, t11); bf_fwd<false>(x1, x3, t11); }
                if (on10) { bf_fwd<false>(x0, x1, t10a); bf_fwd<false>(x2, x3, t10b); }
                s[pos] = x0; s[BLK + pos] = x1; s[2 * BLK + pos] = x2; s[3 * BLK + pos] = x3;
            } else {
                if (on10) { bf_inv<false>(x0, x1, t10a); bf_inv<false>(x2, x3, t10b); }
                if (on11) { bf_inv<false>(x0, x2, t11); bf_inv<false>(x1, x3, t11); }
                if (out_scale) { x0 = m31_mul(x0, out_scale); x1 = m31_mul(x1, out_scale); x2 = m31_mul(x2, out_scale); x3 = m31_mul(x3, out_scale); }
                out[o] = x0; out[1024 + o] = x1; out[2048 + o] = x2; out[3072 + o] = x3;
            }
        }
    };

    int cur = 0;
    if (item < total) prefetch(0, item);
    cp_async_commit();
    for (; item < total; item += stride) {
        cp_async_wait<0>();
        __syncthreads();
        // past this barrier every thread has finished the previous unit: the other buffer may be refilled
        if (item + stride < total) prefetch(cur ^ 1, item + stride);
        cp_async_commit();
        uint32_t* __restrict__ sb = buf0 + cur * BUF;
        uint32_t* __restrict__ s = sb + warp * BLK;
        uint32_t* __restrict__ dst = dst_cols[item >> unit_bits] + blocked((uint32_t)(item & (((size_t)1 << unit_bits) - 1)) << 12, rb);
        const uint32_t* tw = tw0 + cur * R32_C12_TW;
        const uint32_t* const tb_uni[5] = {tw + 1920 + 16 * warp, tw + 1984 + 8 * warp, tw + 2016 + 4 * warp, tw + 2032 + 2 * warp,
                                           tw + 2040 + warp};
        const uint32_t* const tb_lane[5] = {tw + 256 * warp + 8 * tm, tw + 256 * warp + 8 * tm, tw + 1024 + 128 * warp + 4 * tm,
                                            tw + 1536 + 64 * warp + 2 * tm, tw + 1792 + 32 * warp + tm};
        uint4* const row = reinterpret_cast<uint4*>(s + R32_PITCH * tm);
        uint32_t v[32];
        if (!INVERSE) {
            cross_blocks(sb, tw, nullptr, 0u);
            __syncthreads();
#pragma unroll
            for (int p = 0; p < 32; p++) v[p] = s[R32_PITCH * p + tm];
            radix32_stage<false, false, true>(v, tb_uni, 5, ps.act_lo, ps.act_hi);
#pragma unroll
            for (int p = 0; p < 32; p++) s[R32_PITCH * p + tm] = v[p];
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
                *reinterpret_cast<uint4*>(dst + (warp << 10) + 32 * r + 4 * c) = x;
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
            for (int p = 0; p < 32; p++) s[R32_PITCH * p + tm] = v[p];
            __syncthreads();
            cross_blocks(sb, tw, dst, scale);
        }
        cur ^= 1;
    }
    cp_async_wait<0>();
}

}  // namespace zk
