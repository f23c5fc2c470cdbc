// ColumnOps::bit_reverse_column: in-place permutation v[i] <-> v[bitrev(i)]
// (nitroo/crates/stwo/src/core/utils.rs:71-81).
//
// The index is split as [hi : mid : lo] with |hi| = |lo| = TB bits. Reversal maps
// (hi, mid, lo) -> (rev lo, rev mid, rev hi), so the 2^TB x 2^TB block of all (hi, lo) for a fixed
// `mid` lands, transposed and row/column-reversed, in the block of rev(mid). A CTA loads the two
// partner blocks (mid, rev mid) through shared memory so that both the loads and the stores are
// runs of 2^TB consecutive words.
#include "common.cuh"

namespace zk {

constexpr int TB = 5;  // 32 x 32 words per block

template <typename T>
__global__ void bit_reverse_small_kernel(T* __restrict__ v, int log_n) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (1u << log_n)) return;
    uint32_t j = __brev(i) >> (32 - log_n);
    if (j > i) {
        T a = v[i], b = v[j];
        v[i] = b;
        v[j] = a;
    }
}

template <typename T>
__global__ void __launch_bounds__(256) bit_reverse_tiled_kernel(T* __restrict__ v, int log_n) {
    __shared__ T sa[1 << TB][(1 << TB) + 1];
    __shared__ T sb[1 << TB][(1 << TB) + 1];
    const int mid_bits = log_n - 2 * TB;
    const uint32_t mid = blockIdx.x;
    const uint32_t rmid = mid_bits ? (__brev(mid) >> (32 - mid_bits)) : 0u;
    if (rmid < mid) return;  // the partner block does this pair
    const uint32_t lo = threadIdx.x & ((1u << TB) - 1u);
    const int shift_hi = TB + mid_bits;
    // load: sa[hi][lo] = v[hi : mid : lo], sb[hi][lo] = v[hi : rmid : lo]
    for (uint32_t hi = threadIdx.x >> TB; hi < (1u << TB); hi += blockDim.x >> TB) {
        sa[hi][lo] = v[(hi << shift_hi) | (mid << TB) | lo];
        if (rmid != mid) sb[hi][lo] = v[(hi << shift_hi) | (rmid << TB) | lo];
    }
    __syncthreads();
    // store: v[hi' : rmid : lo'] = old v[rev lo' : mid : rev hi'] = sa[rev lo'][rev hi']
    const uint32_t rlo = __brev(lo) >> (32 - TB);
    for (uint32_t hi = threadIdx.x >> TB; hi < (1u << TB); hi += blockDim.x >> TB) {
        uint32_t rhi = __brev(hi) >> (32 - TB);
        v[(hi << shift_hi) | (rmid << TB) | lo] = sa[rlo][rhi];
        if (rmid != mid) v[(hi << shift_hi) | (mid << TB) | lo] = sb[rlo][rhi];
    }
}

// 32-bit words, 2^12 elements and up: 64 x 64-word blocks, so that a block row is a 256-byte run, moved with 16-byte
// accesses. Rows are padded to 66 words: the transposed reads of a warp (sixteen rows two words apart, two adjacent
// columns) then fall into 32 different banks.
constexpr int TB6 = 6;
__device__ __forceinline__ uint32_t rev6(uint32_t x) { return __brev(x) >> 26; }
__global__ void __launch_bounds__(256) bit_reverse_tiled64_kernel(uint32_t* __restrict__ v, int log_n) {
    __shared__ uint32_t sa[64][66];
    __shared__ uint32_t sb[64][66];
    const int mid_bits = log_n - 2 * TB6;
    const uint32_t mid = blockIdx.x;
    const uint32_t rmid = mid_bits ? (__brev(mid) >> (32 - mid_bits)) : 0u;
    if (rmid < mid) return;  // the partner block does this pair
    const int shift_hi = TB6 + mid_bits;
    const bool two = rmid != mid;
    // load: a thread brings four consecutive words of a row
#pragma unroll
    for (int r = 0; r < 4; r++) {
        const uint32_t idx = threadIdx.x + 256u * r, hi = idx >> 4, q = idx & 15u;
        const uint4 x = *reinterpret_cast<const uint4*>(v + (((size_t)hi << shift_hi) | (mid << TB6) | (4u * q)));
        *reinterpret_cast<uint2*>(&sa[hi][4 * q]) = make_uint2(x.x, x.y);
        *reinterpret_cast<uint2*>(&sa[hi][4 * q + 2]) = make_uint2(x.z, x.w);
        if (two) {
            const uint4 y = *reinterpret_cast<const uint4*>(v + (((size_t)hi << shift_hi) | (rmid << TB6) | (4u * q)));
            *reinterpret_cast<uint2*>(&sb[hi][4 * q]) = make_uint2(y.x, y.y);
            *reinterpret_cast<uint2*>(&sb[hi][4 * q + 2]) = make_uint2(y.z, y.w);
        }
    }
    __syncthreads();
    // store: v[hi' : rmid : lo'] = old v[rev lo' : mid : rev hi'] = sa[rev lo'][rev hi']; the two half-warps take rows hi'
    // and hi' + 32, whose reversed indices are adjacent columns
    const uint32_t lane = threadIdx.x & 31u, w = threadIdx.x >> 5, q = lane & 15u;
#pragma unroll
    for (int r = 0; r < 4; r++) {
        const uint32_t hi = w + 8u * r + 32u * (lane >> 4), col = rev6(hi);
        const uint32_t r0 = rev6(4 * q), r1 = r0 | 32u, r2 = r0 | 16u, r3 = r0 | 48u;  // rev6(4q + k) for k = 0..3
        *reinterpret_cast<uint4*>(v + (((size_t)hi << shift_hi) | (rmid << TB6) | (4u * q))) = make_uint4(sa[r0][col], sa[r1][col], sa[r2][col], sa[r3][col]);
        if (two)
            *reinterpret_cast<uint4*>(v + (((size_t)hi << shift_hi) | (mid << TB6) | (4u * q))) = make_uint4(sb[r0][col], sb[r1][col], sb[r2][col], sb[r3][col]);
    }
}

template <typename T>
static int bit_reverse_impl(zkb_ctx* ctx, T* col, int log_n) {
    if (log_n < 2 * TB) {
        unsigned n = 1u << log_n;
        bit_reverse_small_kernel<T><<<(n + 255) / 256, 256, 0, ctx->stream>>>(col, log_n);
    } else if (sizeof(T) == 4 && log_n >= 2 * TB6 && ((uintptr_t)col & 15) == 0) {
        bit_reverse_tiled64_kernel<<<1u << (log_n - 2 * TB6), 256, 0, ctx->stream>>>(reinterpret_cast<uint32_t*>(col), log_n);
    } else {
        bit_reverse_tiled_kernel<T><<<1u << (log_n - 2 * TB), 256, 0, ctx->stream>>>(col, log_n);
    }
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

}  // namespace zk

using namespace zk;

extern "C" {

int zkb_bit_reverse_m31(zkb_ctx* ctx, uint32_t* col, int log_n) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, log_n >= 0 && log_n <= 30);
    if (log_n == 0) return ZKB_OK;
    ZKB_CHECK_ARG(ctx, col != nullptr);
    DeviceGuard g(ctx);
    return bit_reverse_impl<uint32_t>(ctx, col, log_n);
}

int zkb_bit_reverse_qm31(zkb_ctx* ctx, uint32_t* col, int log_n) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, log_n >= 0 && log_n <= 28);
    if (log_n == 0) return ZKB_OK;
    ZKB_CHECK_ARG(ctx, col != nullptr && ((uintptr_t)col & 15) == 0);
    DeviceGuard g(ctx);
    return bit_reverse_impl<uint4>(ctx, reinterpret_cast<uint4*>(col), log_n);
}

}  // extern "C"
