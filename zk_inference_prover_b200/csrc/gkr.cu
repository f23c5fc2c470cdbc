// GkrOps / MleOps: eq evaluations, layer halving, sum-check round sums, fixing the first variable.
// Multilinear columns are arrays of QM31 (16 bytes, one 128-bit access each); the numerators of a
// LogUpMultiplicities layer are M31 words.
//   nitroo/crates/stwo/src/prover/backend/cpu/lookups/gkr.rs:17-263
//   nitroo/crates/stwo/src/prover/backend/cpu/lookups/mle.rs:13-46
#include "common.cuh"

namespace zk {

__device__ __forceinline__ qm31 ldq(const uint32_t* __restrict__ p, size_t i) {
    uint4 v = reinterpret_cast<const uint4*>(p)[i];
    return {{v.x, v.y, v.z, v.w}};
}
__device__ __forceinline__ void stq(uint32_t* __restrict__ p, size_t i, qm31 v) {
    reinterpret_cast<uint4*>(p)[i] = make_uint4(v.c[0], v.c[1], v.c[2], v.c[3]);
}

template <int KIND>
__global__ void __launch_bounds__(256) next_layer_kernel(const uint32_t* __restrict__ num, const uint32_t* __restrict__ den,
                                                         size_t half, uint32_t* __restrict__ num_out,
                                                         uint32_t* __restrict__ den_out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= half) return;
    qm31 d0 = ldq(den, 2 * i), d1 = ldq(den, 2 * i + 1);
    if (KIND == ZKB_GKR_GRAND_PRODUCT) {
        stq(den_out, i, qm31_mul(d0, d1));
        return;
    }
    qm31 n;
    if (KIND == ZKB_GKR_LOGUP_SINGLES) {
        n = qm31_add(d0, d1);
    } else if (KIND == ZKB_GKR_LOGUP_MULTIPLICITIES) {
        uint2 m = reinterpret_cast<const uint2*>(num)[i];
        n = qm31_add(qm31_mul_m31(d1, m.x), qm31_mul_m31(d0, m.y));
    } else {
        qm31 n0 = ldq(num, 2 * i), n1 = ldq(num, 2 * i + 1);
        n = qm31_add(qm31_mul(d1, n0), qm31_mul(d0, n1));
    }
    stq(num_out, i, n);
    stq(den_out, i, qm31_mul(d0, d1));
}

__device__ __forceinline__ qm31 warp_sum(qm31 v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        qm31 o;
#pragma unroll
        for (int k = 0; k < 4; k++) o.c[k] = __shfl_down_sync(0xffffffffu, v.c[k], off);
        v = qm31_add(v, o);
    }
    return v;
}

// Per-block partial sums land in `partials` (8 words per block); the block that takes the last
// ticket adds them up and writes the 8 result words. Addition mod p is exact, so the order of
// the reduction does not change the result.
template <int KIND>
__global__ void __launch_bounds__(256) gkr_sum_kernel(const uint32_t* __restrict__ num, const uint32_t* __restrict__ den,
                                                      size_t n_terms, const uint32_t* __restrict__ eq_evals, qm31 lambda,
                                                      uint32_t* __restrict__ partials, unsigned int* __restrict__ ticket,
                                                      uint32_t* __restrict__ result, const uint32_t* __restrict__ d_lambda = nullptr) {
    if (d_lambda) lambda = ldq(d_lambda, 0);  // the challenge of a device-resident transcript
    qm31 s0 = qm31_zero(), s2 = qm31_zero();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_terms; i += (size_t)gridDim.x * blockDim.x) {
        qm31 d00 = ldq(den, 2 * i), d01 = ldq(den, 2 * i + 1);
        qm31 d10 = ldq(den, 2 * (n_terms + i)), d11 = ldq(den, 2 * (n_terms + i) + 1);
        qm31 d20 = qm31_sub(qm31_dbl(d10), d00), d21 = qm31_sub(qm31_dbl(d11), d01);
        qm31 t0, t2;
        if (KIND == ZKB_GKR_GRAND_PRODUCT) {
            t0 = qm31_mul(d00, d01);
            t2 = qm31_mul(d20, d21);
        } else {
            qm31 n0, n2;
            if (KIND == ZKB_GKR_LOGUP_SINGLES) {
                n0 = qm31_add(d00, d01);
                n2 = qm31_add(d20, d21);
            } else if (KIND == ZKB_GKR_LOGUP_MULTIPLICITIES) {
                uint2 a = reinterpret_cast<const uint2*>(num)[i];
                uint2 b = reinterpret_cast<const uint2*>(num)[n_terms + i];
                uint32_t n20 = m31_sub(m31_dbl(b.x), a.x), n21 = m31_sub(m31_dbl(b.y), a.y);
                n0 = qm31_add(qm31_mul_m31(d01, a.x), qm31_mul_m31(d00, a.y));
                n2 = qm31_add(qm31_mul_m31(d21, n20), qm31_mul_m31(d20, n21));
            } else {
                qm31 n00 = ldq(num, 2 * i), n01 = ldq(num, 2 * i + 1);
                qm31 n10 = ldq(num, 2 * (n_terms + i)), n11 = ldq(num, 2 * (n_terms + i) + 1);
                qm31 n20 = qm31_sub(qm31_dbl(n10), n00), n21 = qm31_sub(qm31_dbl(n11), n01);
                n0 = qm31_add(qm31_mul(d01, n00), qm31_mul(d00, n01));
                n2 = qm31_add(qm31_mul(d21, n20), qm31_mul(d20, n21));
            }
            t0 = qm31_add(n0, qm31_mul(lambda, qm31_mul(d00, d01)));
            t2 = qm31_add(n2, qm31_mul(lambda, qm31_mul(d20, d21)));
        }
        qm31 e = ldq(eq_evals, i);
        s0 = qm31_add(s0, qm31_mul(e, t0));
        s2 = qm31_add(s2, qm31_mul(e, t2));
    }
    __shared__ uint32_t sh[8][8];
    __shared__ bool is_last;
    s0 = warp_sum(s0);
    s2 = warp_sum(s2);
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
    if (threadIdx.x == 0) {
        unsigned int t = atomicAdd(ticket, 1u);
        is_last = (t == gridDim.x - 1);
    }
    __syncthreads();
    if (is_last) {
        __threadfence();
        if (threadIdx.x < 8) {
            uint32_t acc = 0;
            for (unsigned b = 0; b < gridDim.x; b++) acc = m31_add(acc, __ldcg(&partials[8 * b + threadIdx.x]));
            result[threadIdx.x] = acc;
        }
        if (threadIdx.x == 0) *ticket = 0u;  // ready for the next launch
    }
}

// out[i] = in[i] + r * (in[i + half] - in[i])
__global__ void __launch_bounds__(256) mle_fix_qm31_kernel(const uint32_t* __restrict__ in, size_t half, qm31 r,
                                                           uint32_t* __restrict__ out, const uint32_t* __restrict__ d_r = nullptr) {
    if (d_r) r = ldq(d_r, 0);
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= half) return;
    qm31 a = ldq(in, i), b = ldq(in, i + half);
    stq(out, i, qm31_add(qm31_mul(r, qm31_sub(b, a)), a));
}
__global__ void __launch_bounds__(256) mle_fix_m31_kernel(const uint32_t* __restrict__ in, size_t half, qm31 r,
                                                          uint32_t* __restrict__ out, const uint32_t* __restrict__ d_r = nullptr) {
    if (d_r) r = ldq(d_r, 0);
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= half) return;
    uint32_t a = in[i], b = in[i + half];
    qm31 v = qm31_mul_m31(r, m31_sub(b, a));
    v.c[0] = m31_add(v.c[0], a);
    stq(out, i, v);
}

// Launchers for the device-resident transcript (gkr_resident.cu): challenges come from device memory and the
// sums stay on the device.
int gkr_sum_launch(zkb_ctx* ctx, int kind, const uint32_t* num, const uint32_t* den, size_t n, const uint32_t* eq_evals,
                   const uint32_t* d_lambda, uint32_t* d_result) {
    size_t n_terms = n / 4;
    unsigned blocks = (unsigned)((n_terms + 255) / 256);
    if (blocks > 148u * 8u) blocks = 148u * 8u;
    uint32_t* partials = ctx->scratch;
    qm31 z = qm31_zero();
    ProfScope* prof = new ProfScope(ctx, "gkr_sum_kernel");
    switch (kind) {
        case ZKB_GKR_GRAND_PRODUCT: gkr_sum_kernel<0><<<blocks, 256, 0, ctx->stream>>>(num, den, n_terms, eq_evals, z, partials, ctx->ticket, d_result, d_lambda); break;
        case ZKB_GKR_LOGUP_GENERIC: gkr_sum_kernel<1><<<blocks, 256, 0, ctx->stream>>>(num, den, n_terms, eq_evals, z, partials, ctx->ticket, d_result, d_lambda); break;
        case ZKB_GKR_LOGUP_MULTIPLICITIES: gkr_sum_kernel<2><<<blocks, 256, 0, ctx->stream>>>(num, den, n_terms, eq_evals, z, partials, ctx->ticket, d_result, d_lambda); break;
        default: gkr_sum_kernel<3><<<blocks, 256, 0, ctx->stream>>>(num, den, n_terms, eq_evals, z, partials, ctx->ticket, d_result, d_lambda); break;
    }
    delete prof;
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

int gkr_mle_fix_launch(zkb_ctx* ctx, bool base, const uint32_t* in, size_t n, const uint32_t* d_r, uint32_t* out) {
    size_t half = n / 2;
    unsigned blocks = (unsigned)((half + 255) / 256);
    ProfScope prof(ctx, base ? "mle_fix_m31_kernel" : "mle_fix_qm31_kernel");
    if (base) mle_fix_m31_kernel<<<blocks, 256, 0, ctx->stream>>>(in, half, qm31_zero(), out, d_r);
    else mle_fix_qm31_kernel<<<blocks, 256, 0, ctx->stream>>>(in, half, qm31_zero(), out, d_r);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

}  // namespace zk

using namespace zk;

static inline qm31 q4(const uint32_t* p) { return qm31{{p[0], p[1], p[2], p[3]}}; }

extern "C" {

int zkb_gkr_next_layer(zkb_ctx* ctx, int kind, const uint32_t* num, const uint32_t* den, size_t n, uint32_t* num_out,
                       uint32_t* den_out) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, kind >= 0 && kind <= 3 && den && den_out && n >= 2 && (n & (n - 1)) == 0);
    ZKB_CHECK_ARG(ctx, kind == ZKB_GKR_GRAND_PRODUCT || num_out != nullptr);
    ZKB_CHECK_ARG(ctx, (kind != ZKB_GKR_LOGUP_GENERIC && kind != ZKB_GKR_LOGUP_MULTIPLICITIES) || num != nullptr);
    ZKB_CHECK_ARG(ctx, ((uintptr_t)den & 15) == 0 && ((uintptr_t)den_out & 15) == 0 && ((uintptr_t)num_out & 15) == 0);
    DeviceGuard g(ctx);
    size_t half = n / 2;
    unsigned blocks = (unsigned)((half + 255) / 256);
    ProfScope prof(ctx, "next_layer_kernel");
    switch (kind) {
        case ZKB_GKR_GRAND_PRODUCT: next_layer_kernel<0><<<blocks, 256, 0, ctx->stream>>>(num, den, half, num_out, den_out); break;
        case ZKB_GKR_LOGUP_GENERIC: next_layer_kernel<1><<<blocks, 256, 0, ctx->stream>>>(num, den, half, num_out, den_out); break;
        case ZKB_GKR_LOGUP_MULTIPLICITIES: next_layer_kernel<2><<<blocks, 256, 0, ctx->stream>>>(num, den, half, num_out, den_out); break;
        default: next_layer_kernel<3><<<blocks, 256, 0, ctx->stream>>>(num, den, half, num_out, den_out); break;
    }
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

int zkb_gkr_sum(zkb_ctx* ctx, int kind, const uint32_t* num, const uint32_t* den, size_t n, const uint32_t* eq_evals,
                const uint32_t h_lambda[4], uint32_t h_out[8]) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, kind >= 0 && kind <= 3 && den && eq_evals && h_lambda && h_out && n >= 2 && (n & (n - 1)) == 0);
    ZKB_CHECK_ARG(ctx, (kind != ZKB_GKR_LOGUP_GENERIC && kind != ZKB_GKR_LOGUP_MULTIPLICITIES) || num != nullptr);
    // the kernel reads QM31 entries with 16-byte loads and M31 numerators in pairs (8-byte loads)
    ZKB_CHECK_ARG(ctx, (((uintptr_t)den | (uintptr_t)eq_evals) & 15) == 0);
    ZKB_CHECK_ARG(ctx, kind != ZKB_GKR_LOGUP_GENERIC || ((uintptr_t)num & 15) == 0);
    ZKB_CHECK_ARG(ctx, kind != ZKB_GKR_LOGUP_MULTIPLICITIES || ((uintptr_t)num & 7) == 0);
    DeviceGuard g(ctx);
    size_t n_terms = n / 4;
    if (n_terms == 0) {
        // A one-variable layer: sum_as_poly_in_first_variable is never asked for it by the
        // protocol (n_variables of the oracle would be 0); keep the call well defined.
        memset(h_out, 0, 32);
        return ZKB_OK;
    }
    unsigned blocks = (unsigned)((n_terms + 255) / 256);
    if (blocks > 148u * 8u) blocks = 148u * 8u;
    uint32_t* partials = ctx->scratch;
    uint32_t* result = ctx->scratch + 8 * (size_t)blocks;
    qm31 lam = q4(h_lambda);
    ProfScope* prof = new ProfScope(ctx, "gkr_sum_kernel");
    switch (kind) {
        case ZKB_GKR_GRAND_PRODUCT: gkr_sum_kernel<0><<<blocks, 256, 0, ctx->stream>>>(num, den, n_terms, eq_evals, lam, partials, ctx->ticket, result); break;
        case ZKB_GKR_LOGUP_GENERIC: gkr_sum_kernel<1><<<blocks, 256, 0, ctx->stream>>>(num, den, n_terms, eq_evals, lam, partials, ctx->ticket, result); break;
        case ZKB_GKR_LOGUP_MULTIPLICITIES: gkr_sum_kernel<2><<<blocks, 256, 0, ctx->stream>>>(num, den, n_terms, eq_evals, lam, partials, ctx->ticket, result); break;
        default: gkr_sum_kernel<3><<<blocks, 256, 0, ctx->stream>>>(num, den, n_terms, eq_evals, lam, partials, ctx->ticket, result); break;
    }
    delete prof;
    ZKB_LAUNCH_CHECK(ctx);
    ZKB_CUDA(ctx, cudaMemcpyAsync(ctx->h_small, result, 32, cudaMemcpyDeviceToHost, ctx->stream));
    ZKB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    memcpy(h_out, ctx->h_small, 32);
    return ZKB_OK;
}

int zkb_mle_fix_qm31(zkb_ctx* ctx, const uint32_t* in, size_t n, const uint32_t h_r[4], uint32_t* out) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, in && out && h_r && n >= 2 && (n & (n - 1)) == 0);
    ZKB_CHECK_ARG(ctx, ((uintptr_t)in & 15) == 0 && ((uintptr_t)out & 15) == 0);
    DeviceGuard g(ctx);
    size_t half = n / 2;
    ProfScope prof(ctx, "mle_fix_qm31_kernel");
    mle_fix_qm31_kernel<<<(unsigned)((half + 255) / 256), 256, 0, ctx->stream>>>(in, half, q4(h_r), out);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

int zkb_mle_fix_m31(zkb_ctx* ctx, const uint32_t* in, size_t n, const uint32_t h_r[4], uint32_t* out) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, in && out && h_r && n >= 2 && (n & (n - 1)) == 0 && ((uintptr_t)out & 15) == 0);
    DeviceGuard g(ctx);
    size_t half = n / 2;
    ProfScope prof(ctx, "mle_fix_m31_kernel");
    mle_fix_m31_kernel<<<(unsigned)((half + 255) / 256), 256, 0, ctx->stream>>>(in, half, q4(h_r), out);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Round sums without any allocation.
//
// Some callers may not allocate device memory at the point where they need a sum-check round sum:
// a prover that has handed the whole card to a fixed arena and runs with the allocator locked, a
// host thread inside a region where cudaMalloc/cudaFree would synchronise the device and stall other
// streams, or a plugin loaded into a process that forbids allocation after start-up. zkb_gkr_sum
// needs a context, and creating a context allocates (twiddles, scratch, pinned buffers).
// zkb_gkr_sum_noalloc needs none: its only scratch, the per-block partial sums and the ticket that
// elects the last block, lives in the fixed array below, which every GPU that loads this library
// holds from load until exit.
namespace zk {

constexpr int NOALLOC_MAX_BLOCKS = 2048;
constexpr size_t NOALLOC_MAX_ENTRIES = (size_t)1 << 28;  // largest layer (n) accepted
// 8 words per block of partial sums, then 64 words whose first is the ticket: 64.25 KiB.
static __device__ __align__(256) uint32_t g_noalloc_scratch[8 * NOALLOC_MAX_BLOCKS + 64];

constexpr int NOALLOC_MAX_DEVICES = 64;
static uint32_t* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {nullptr};  // device address of the array, per device
static thread_local char g_noalloc_err[256] = "";  // per host thread: concurrent failing calls do not garble it

}  // namespace zk

extern "C" {

const char* zkb_gkr_sum_noalloc_error(void) { return zk::g_noalloc_err; }

int zkb_gkr_sum_noalloc(int device, void* stream, int kind, const uint32_t* num, const uint32_t* den, size_t n,
                        const uint32_t* eq_evals, const uint32_t h_lambda[4], uint32_t* d_out) {
    auto fail = [](int code, const char* msg) { snprintf(zk::g_noalloc_err, sizeof(zk::g_noalloc_err), "zkb_gkr_sum_noalloc: %s", msg); return code; };
    if (device < 0 || device >= NOALLOC_MAX_DEVICES) return fail(ZKB_EINVAL, "device index out of range");
    if (kind < 0 || kind > 3 || !den || !eq_evals || !h_lambda || !d_out) return fail(ZKB_EINVAL, "null pointer or unknown layer kind");
    if ((kind == ZKB_GKR_LOGUP_GENERIC || kind == ZKB_GKR_LOGUP_MULTIPLICITIES) && !num) return fail(ZKB_EINVAL, "this layer kind needs numerators");
    if (n < 4 || (n & (n - 1))) return fail(ZKB_EINVAL, "n must be a power of two, at least 4");
    if (n > NOALLOC_MAX_ENTRIES) return fail(ZKB_EINVAL, "layer larger than this entry point's stated limit (2^28 entries at most)");
    // misaligned pointers would fault on the device (16-byte loads of QM31 entries, 8-byte loads of M31 pairs)
    if ((((uintptr_t)den | (uintptr_t)eq_evals) & 15) != 0) return fail(ZKB_EINVAL, "den and eq_evals must be 16-byte aligned");
    if (kind == ZKB_GKR_LOGUP_GENERIC && ((uintptr_t)num & 15) != 0) return fail(ZKB_EINVAL, "QM31 numerators must be 16-byte aligned");
    if (kind == ZKB_GKR_LOGUP_MULTIPLICITIES && ((uintptr_t)num & 7) != 0) return fail(ZKB_EINVAL, "M31 numerators must be 8-byte aligned");
    if (((uintptr_t)d_out & 3) != 0) return fail(ZKB_EINVAL, "d_out must be 4-byte aligned");
    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess) return fail(ZKB_ECUDA, "cudaGetDevice failed");
    if (prev != device && cudaSetDevice(device) != cudaSuccess) return fail(ZKB_ECUDA, "cudaSetDevice failed");
    int rc = ZKB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    // Set-up, once per device and with that device current: the array's name is only a host-side
    // handle, the kernel needs its address on this device.
    if (!zk::g_noalloc_ptr[device]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, zk::g_noalloc_scratch);
        if (e != cudaSuccess || !p) rc = fail(ZKB_ECUDA, cudaGetErrorString(e));
        else zk::g_noalloc_ptr[device] = (uint32_t*)p;
    }
    if (rc == ZKB_OK) {
        uint32_t* partials = zk::g_noalloc_ptr[device];
        unsigned int* ticket = (unsigned int*)(partials + 8 * NOALLOC_MAX_BLOCKS);
        size_t n_terms = n / 4;
        unsigned blocks = (unsigned)((n_terms + 255) / 256);
        if (blocks > (unsigned)NOALLOC_MAX_BLOCKS) blocks = NOALLOC_MAX_BLOCKS;
        qm31 lam = q4(h_lambda);
        // the ticket must start at zero whatever an earlier call left behind
        cudaError_t e = cudaMemsetAsync(ticket, 0, sizeof(unsigned int), st);
        if (e == cudaSuccess) {
            switch (kind) {
                case ZKB_GKR_GRAND_PRODUCT: gkr_sum_kernel<0><<<blocks, 256, 0, st>>>(num, den, n_terms, eq_evals, lam, partials, ticket, d_out); break;
                case ZKB_GKR_LOGUP_GENERIC: gkr_sum_kernel<1><<<blocks, 256, 0, st>>>(num, den, n_terms, eq_evals, lam, partials, ticket, d_out); break;
                case ZKB_GKR_LOGUP_MULTIPLICITIES: gkr_sum_kernel<2><<<blocks, 256, 0, st>>>(num, den, n_terms, eq_evals, lam, partials, ticket, d_out); break;
                default: gkr_sum_kernel<3><<<blocks, 256, 0, st>>>(num, den, n_terms, eq_evals, lam, partials, ticket, d_out); break;
            }
            e = cudaGetLastError();
        }
        if (e != cudaSuccess) rc = fail(ZKB_ECUDA, cudaGetErrorString(e));
    }
    if (prev >= 0 && prev != device) cudaSetDevice(prev);
    return rc;
}

}  // extern "C"
