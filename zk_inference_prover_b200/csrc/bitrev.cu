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

template <typename T>
static int bit_reverse_impl(zkb_ctx* ctx, T* col, int log_n) {
    if (log_n < 2 * TB) {
        unsigned n = 1u << log_n;
        bit_reverse_small_kernel<T><<<(n + 255) / 256, 256, 0, ctx->stream>>>(col, log_n);
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
