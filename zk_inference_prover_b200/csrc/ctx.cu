// Context lifetime, device memory helpers, the twiddle tower and small utilities.
#include <cstdarg>
#include <vector>

#include "common.cuh"
#include "gather_blocks.hpp"

namespace zk {

int set_error(zkb_ctx* ctx, int code, const char* fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
        va_end(ap);
    }
    return code;
}

int stage_ptrs(zkb_ctx* ctx, const void* const* h_ptrs, int n, void*** out) {
    if (n < 0 || (size_t)n > ctx->ring_cap) return set_error(ctx, ZKB_EINVAL, "stage_ptrs: %d pointers exceed the staging ring", n);
    if (n == 0) { *out = ctx->d_ring; return ZKB_OK; }
    if (ctx->ring_pos + (size_t)n > ctx->ring_cap) {
        // Wrap: earlier slots may still be in flight, so drain the stream first.
        ZKB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        ctx->ring_pos = 0;
    }
    void** h = ctx->h_ring + ctx->ring_pos;
    void** d = ctx->d_ring + ctx->ring_pos;
    memcpy(h, h_ptrs, (size_t)n * sizeof(void*));
    ZKB_CUDA(ctx, cudaMemcpyAsync(d, h, (size_t)n * sizeof(void*), cudaMemcpyHostToDevice, ctx->stream));
    ctx->ring_pos += (size_t)n;
    *out = d;
    return ZKB_OK;
}

int stage_blob(zkb_ctx* ctx, const void* h_data, size_t bytes, void** out) {
    const size_t slots = (bytes + sizeof(void*) - 1) / sizeof(void*);
    if (slots + 1 > ctx->ring_cap) return set_error(ctx, ZKB_EINVAL, "stage_blob: %zu bytes exceed the staging ring", bytes);
    size_t pos = (ctx->ring_pos + 1) & ~(size_t)1;  // slots are 8 bytes and the ring's base is aligned: even slots are 16-byte aligned
    if (pos + slots > ctx->ring_cap) {
        ZKB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // earlier slots may still be in flight
        pos = 0;
    }
    memcpy(ctx->h_ring + pos, h_data, bytes);
    ZKB_CUDA(ctx, cudaMemcpyAsync(ctx->d_ring + pos, ctx->h_ring + pos, bytes, cudaMemcpyHostToDevice, ctx->stream));
    ctx->ring_pos = pos + slots;
    *out = ctx->d_ring + pos;
    return ZKB_OK;
}

// G * 2^b for the generator G of the order-2^31 circle group over M31
// (nitroo/crates/stwo/src/core/circle.rs:202-205).
__constant__ cpoint c_gen_pow2[31];

__device__ __forceinline__ cpoint circle_point_from_index(uint32_t idx) {
    cpoint r{1u, 0u};
#pragma unroll 1
    for (int b = 0; b < 31; b++)
        if ((idx >> b) & 1u) r = cpoint_add(r, c_gen_pow2[b]);
    return r;
}

// tw[t], t in [1, len): k = floor(log2 t) + 1, h = t - 2^(k-1);
// value = x( half_odds(k).at(bitrev_{k-1}(h)) ), index 2^(29-k) + j * 2^(31-k).
__global__ void twiddle_tower_kernel(uint32_t* __restrict__ tw, uint32_t* __restrict__ itw, size_t len) {
    size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= len) return;
    if (t == 0) { tw[0] = 1u; itw[0] = 1u; return; }
    int k = 32 - __clz((uint32_t)t);
    uint32_t h = (uint32_t)t - (1u << (k - 1));
    uint32_t j = (k > 1) ? (__brev(h) >> (32 - (k - 1))) : 0u;
    uint32_t index = (1u << (29 - k)) + (j << (31 - k));
    cpoint p = circle_point_from_index(index & 0x7fffffffu);
    tw[t] = p.x;
    itw[t] = m31_inv(p.x);
}

__global__ void double_words_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out, size_t len) {
    size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t < len) out[t] = in[t] << 1;
}

__global__ void gather_multi_kernel(const uint32_t* const* __restrict__ cols, int ncols, const uint32_t* __restrict__ idx,
                                    int nidx, uint32_t* __restrict__ out) {
    size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (size_t)ncols * nidx) return;
    int i = (int)(t / ncols), c = (int)(t % ncols);
    out[t] = cols[c][idx[i]];
}

__global__ void gather_hashes_kernel(const uint4* __restrict__ hashes, const uint32_t* __restrict__ idx, int nidx,
                                     uint4* __restrict__ out) {
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= 2 * nidx) return;
    out[t] = hashes[2 * (size_t)idx[t >> 1] + (t & 1)];
}

__global__ void gather_words_kernel(const uint32_t* const* __restrict__ addrs, size_t n, uint32_t* __restrict__ out) {
    size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n) out[t] = *addrs[t];
}

}  // namespace zk

using namespace zk;

extern "C" int zk_set_error_public(zkb_ctx* ctx, int code, const char* msg) { return set_error(ctx, code, "%s", msg); }

extern "C" {

int zkb_init(int device, int max_log_size, zkb_ctx** out) {
    if (!out) return ZKB_EINVAL;
    *out = nullptr;
    if (max_log_size < 3 || max_log_size > 28) return ZKB_EINVAL;
    zkb_ctx* ctx = new (std::nothrow) zkb_ctx();
    if (!ctx) return ZKB_ENOMEM;
    ctx->device = device;
    ctx->max_log = max_log_size;
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) { delete ctx; return ZKB_ECUDA; }
    auto fail = [&](int code) { zkb_destroy(ctx); return code; };
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) return fail(ZKB_ECUDA);
    ctx->tw_len = (size_t)1 << (max_log_size - 1);
    if (cudaMalloc(&ctx->tw, ctx->tw_len * 4) != cudaSuccess) return fail(ZKB_ENOMEM);
    if (cudaMalloc(&ctx->itw, ctx->tw_len * 4) != cudaSuccess) return fail(ZKB_ENOMEM);
    if (cudaMalloc(&ctx->tw2, ctx->tw_len * 4) != cudaSuccess) return fail(ZKB_ENOMEM);
    if (cudaMalloc(&ctx->itw2, ctx->tw_len * 4) != cudaSuccess) return fail(ZKB_ENOMEM);
    if (cudaMalloc(&ctx->dev_err, 64) != cudaSuccess) return fail(ZKB_ENOMEM);
    if (cudaMemsetAsync(ctx->dev_err, 0, 64, ctx->stream) != cudaSuccess) return fail(ZKB_ECUDA);
    ctx->ring_cap = RING_SLOTS;
    if (cudaMallocHost(&ctx->h_ring, ctx->ring_cap * sizeof(void*)) != cudaSuccess) return fail(ZKB_ENOMEM);
    if (cudaMalloc(&ctx->d_ring, ctx->ring_cap * sizeof(void*)) != cudaSuccess) return fail(ZKB_ENOMEM);
    ctx->scratch_words = SCRATCH_WORDS;
    if (cudaMalloc(&ctx->scratch, ctx->scratch_words * 4) != cudaSuccess) return fail(ZKB_ENOMEM);
    if (cudaMalloc(&ctx->ticket, 64) != cudaSuccess) return fail(ZKB_ENOMEM);
    if (cudaMemsetAsync(ctx->ticket, 0, 64, ctx->stream) != cudaSuccess) return fail(ZKB_ECUDA);
    if (cudaMallocHost(&ctx->h_small, (SMALL_WORDS + 16) * 4) != cudaSuccess) return fail(ZKB_ENOMEM);

    {
        cudaMemPool_t pool;
        if (cudaDeviceGetDefaultMemPool(&pool, device) != cudaSuccess) return fail(ZKB_ECUDA);
        unsigned long long keep = ~0ull;
        if (cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep) != cudaSuccess) return fail(ZKB_ECUDA);
    }
    // Generator doublings on the host, then the tower on the device.
    cpoint g[31];
    g[0] = {2u, 1268011823u};
    for (int b = 1; b < 31; b++) g[b] = cpoint_add(g[b - 1], g[b - 1]);
    if (cudaMemcpyToSymbolAsync(c_gen_pow2, g, sizeof(g), 0, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess) return fail(ZKB_ECUDA);
    unsigned blocks = (unsigned)((ctx->tw_len + 255) / 256);
    twiddle_tower_kernel<<<blocks, 256, 0, ctx->stream>>>(ctx->tw, ctx->itw, ctx->tw_len);
    double_words_kernel<<<blocks, 256, 0, ctx->stream>>>(ctx->tw, ctx->tw2, ctx->tw_len);
    double_words_kernel<<<blocks, 256, 0, ctx->stream>>>(ctx->itw, ctx->itw2, ctx->tw_len);
    if (cudaGetLastError() != cudaSuccess) return fail(ZKB_ECUDA);
    if (cudaStreamSynchronize(ctx->stream) != cudaSuccess) return fail(ZKB_ECUDA);
    *out = ctx;
    return ZKB_OK;
}

int zkb_destroy(zkb_ctx* ctx) {
    if (!ctx) return ZKB_EINVAL;
    cudaSetDevice(ctx->device);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    if (ctx->tw) cudaFree(ctx->tw);
    if (ctx->itw) cudaFree(ctx->itw);
    if (ctx->tw2) cudaFree(ctx->tw2);
    if (ctx->itw2) cudaFree(ctx->itw2);
    if (ctx->dev_err) cudaFree(ctx->dev_err);
    if (ctx->h_ring) cudaFreeHost(ctx->h_ring);
    if (ctx->d_ring) cudaFree(ctx->d_ring);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->ticket) cudaFree(ctx->ticket);
    if (ctx->h_small) cudaFreeHost(ctx->h_small);
    if (ctx->h_batch) cudaFreeHost(ctx->h_batch);
    if (ctx->batch_tickets) cudaFree(ctx->batch_tickets);
    for (int i = 0; i < 64; i++)
        if (ctx->events[i]) cudaEventDestroy(ctx->events[i]);
    if (ctx->prof) {
        for (int i = 0; i < ctx->prof_cap; i++)
            if (ctx->prof[i].a) { cudaEventDestroy(ctx->prof[i].a); cudaEventDestroy(ctx->prof[i].b); }
        delete[] ctx->prof;
    }
    for (int i = 0; i < 64; i++)
        if (ctx->fences[i]) cudaEventDestroy(ctx->fences[i]);
    if (ctx->copy_gate) cudaEventDestroy(ctx->copy_gate);
    if (ctx->copy_stream) cudaStreamDestroy(ctx->copy_stream);
    for (auto st : ctx->peer_streams)
        if (st) cudaStreamDestroy(st);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return ZKB_OK;
}

const char* zkb_last_error(zkb_ctx* ctx) { return ctx ? ctx->err : "null context"; }

int zkb_sync(zkb_ctx* ctx) {
    if (!ctx) return ZKB_EINVAL;
    DeviceGuard g(ctx);
    if (ctx->copy_stream) ZKB_CUDA(ctx, cudaStreamSynchronize(ctx->copy_stream));
    // a kernel whose bounded wait ran out has set the error word; report it here, where the host waits anyway
    ZKB_CUDA(ctx, cudaMemcpyAsync(ctx->h_small + SMALL_WORDS, ctx->dev_err, 4, cudaMemcpyDeviceToHost, ctx->stream));
    ZKB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->h_small[SMALL_WORDS] != 0) {
        unsigned code = ctx->h_small[SMALL_WORDS];
        cudaMemsetAsync(ctx->dev_err, 0, 4, ctx->stream);
        return set_error(ctx, ZKB_ETIMEOUT, "zkb_sync: a device-side wait ran out of its iteration limit (code 0x%x); results of the calls since the last sync are not valid", code);
    }
    return ZKB_OK;
}

int zkb_get_stream(zkb_ctx* ctx, void** stream) {
    if (!ctx || !stream) return ZKB_EINVAL;
    *stream = (void*)ctx->stream;
    return ZKB_OK;
}

int zkb_event_record(zkb_ctx* ctx, int slot) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, slot >= 0 && slot < 64);
    DeviceGuard g(ctx);
    if (!ctx->events[slot]) ZKB_CUDA(ctx, cudaEventCreate(&ctx->events[slot]));
    ZKB_CUDA(ctx, cudaEventRecord(ctx->events[slot], ctx->stream));
    return ZKB_OK;
}

int zkb_event_elapsed_ms(zkb_ctx* ctx, int a, int b, float* h_ms) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, a >= 0 && a < 64 && b >= 0 && b < 64 && h_ms && ctx->events[a] && ctx->events[b]);
    DeviceGuard g(ctx);
    ZKB_CUDA(ctx, cudaEventSynchronize(ctx->events[b]));
    ZKB_CUDA(ctx, cudaEventElapsedTime(h_ms, ctx->events[a], ctx->events[b]));
    return ZKB_OK;
}

int zkb_profile_begin(zkb_ctx* ctx) {
    if (!ctx) return ZKB_EINVAL;
    DeviceGuard g(ctx);
    if (!ctx->prof) {
        ctx->prof_cap = 8192;
        ctx->prof = new (std::nothrow) zkb_ctx::ProfRec[ctx->prof_cap]();
        if (!ctx->prof) { ctx->prof_cap = 0; return set_error(ctx, ZKB_ENOMEM, "zkb_profile_begin: out of host memory"); }
    }
    ctx->prof_n = 0;
    ctx->prof_on = true;
    return ZKB_OK;
}

int zkb_profile_end(zkb_ctx* ctx, const char** h_names, float* h_ms, int* h_count, int cap, int* n) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, h_names && h_ms && h_count && n && cap > 0);
    DeviceGuard g(ctx);
    ctx->prof_on = false;
    ZKB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    int k = 0;
    for (int i = 0; i < ctx->prof_n; i++) {
        float ms = 0.f;
        ZKB_CUDA(ctx, cudaEventElapsedTime(&ms, ctx->prof[i].a, ctx->prof[i].b));
        int j = 0;
        while (j < k && h_names[j] != ctx->prof[i].name) j++;
        if (j == k) {
            if (k == cap) continue;
            h_names[k] = ctx->prof[i].name; h_ms[k] = 0.f; h_count[k] = 0; k++;
        }
        h_ms[j] += ms;
        h_count[j] += 1;
    }
    *n = k;
    return ZKB_OK;
}

int zkb_max_log_size(zkb_ctx* ctx) { return ctx ? ctx->max_log : ZKB_EINVAL; }

int zkb_malloc(zkb_ctx* ctx, size_t bytes, void** dptr) {
    if (!ctx || !dptr) return ZKB_EINVAL;
    DeviceGuard g(ctx);
    *dptr = nullptr;
    if (bytes == 0) return ZKB_OK;
    // Stream-ordered allocation from the device's default pool (kept warm: the release threshold
    // is raised in zkb_init), so neither allocation nor release synchronises the device.
    ZKB_CUDA(ctx, cudaMallocAsync(dptr, bytes, ctx->stream));
    return ZKB_OK;
}

int zkb_free(zkb_ctx* ctx, void* dptr) {
    if (!ctx) return ZKB_EINVAL;
    if (!dptr) return ZKB_OK;
    DeviceGuard g(ctx);
    ZKB_CUDA(ctx, cudaFreeAsync(dptr, ctx->stream));
    return ZKB_OK;
}

int zkb_memset_zero(zkb_ctx* ctx, void* dptr, size_t bytes) {
    if (!ctx) return ZKB_EINVAL;
    if (bytes == 0) return ZKB_OK;
    ZKB_CHECK_ARG(ctx, dptr != nullptr);
    DeviceGuard g(ctx);
    ZKB_CUDA(ctx, cudaMemsetAsync(dptr, 0, bytes, ctx->stream));
    return ZKB_OK;
}

int zkb_h2d(zkb_ctx* ctx, void* dptr, const void* h_src, size_t bytes) {
    if (!ctx) return ZKB_EINVAL;
    if (bytes == 0) return ZKB_OK;
    ZKB_CHECK_ARG(ctx, dptr != nullptr && h_src != nullptr);
    DeviceGuard g(ctx);
    ZKB_CUDA(ctx, cudaMemcpyAsync(dptr, h_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    ZKB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return ZKB_OK;
}

int zkb_d2h(zkb_ctx* ctx, void* h_dst, const void* dptr, size_t bytes) {
    if (!ctx) return ZKB_EINVAL;
    if (bytes == 0) return ZKB_OK;
    ZKB_CHECK_ARG(ctx, dptr != nullptr && h_dst != nullptr);
    DeviceGuard g(ctx);
    ZKB_CUDA(ctx, cudaMemcpyAsync(h_dst, dptr, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    ZKB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return ZKB_OK;
}

int zkb_h2d_async(zkb_ctx* ctx, void* dptr, const void* h_pinned_src, size_t bytes) {
    if (!ctx) return ZKB_EINVAL;
    if (bytes == 0) return ZKB_OK;
    ZKB_CHECK_ARG(ctx, dptr != nullptr && h_pinned_src != nullptr);
    DeviceGuard g(ctx);
    ZKB_CUDA(ctx, cudaMemcpyAsync(dptr, h_pinned_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return ZKB_OK;
}

int zkb_h2d_overlapped(zkb_ctx* ctx, void* dptr, const void* h_pinned_src, size_t bytes, int fence) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, fence >= -1 && fence < 64 && (bytes == 0 || (dptr != nullptr && h_pinned_src != nullptr)));
    DeviceGuard g(ctx);
    if (!ctx->copy_stream) ZKB_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking));
    if (!ctx->copy_gate) ZKB_CUDA(ctx, cudaEventCreateWithFlags(&ctx->copy_gate, cudaEventDisableTiming));
    // the destination may have been allocated (stream-ordered) on the compute stream just now
    ZKB_CUDA(ctx, cudaEventRecord(ctx->copy_gate, ctx->stream));
    ZKB_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_stream, ctx->copy_gate, 0));
    if (bytes) ZKB_CUDA(ctx, cudaMemcpyAsync(dptr, h_pinned_src, bytes, cudaMemcpyHostToDevice, ctx->copy_stream));
    if (fence >= 0) {
        if (!ctx->fences[fence]) ZKB_CUDA(ctx, cudaEventCreateWithFlags(&ctx->fences[fence], cudaEventDisableTiming));
        ZKB_CUDA(ctx, cudaEventRecord(ctx->fences[fence], ctx->copy_stream));
    }
    return ZKB_OK;
}

int zkb_wait_fence(zkb_ctx* ctx, int fence) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, fence >= 0 && fence < 64 && ctx->fences[fence] != nullptr);
    DeviceGuard g(ctx);
    ZKB_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->fences[fence], 0));
    return ZKB_OK;
}

// ---- buffers another process's GPU can write into (one process per GPU on one host) -----------------------------
// The stream-ordered pool's memory can not be shared between processes, so these come from cudaMalloc. A peer opens the
// handle and copies into the buffer with the copy engines (zkb_copy_to_peer): no SM is used, which is what lets the
// exchange of a sharded commitment run under the transform kernels (a collective's copy kernels wait for SMs the
// persistent transform passes hold).
int zkb_peer_buffer_alloc(zkb_ctx* ctx, size_t bytes, void** dptr, unsigned char handle[64]) {
    if (!ctx || !dptr || !handle || bytes == 0) return ZKB_EINVAL;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    DeviceGuard g(ctx);
    *dptr = nullptr;
    ZKB_CUDA(ctx, cudaMalloc(dptr, bytes));
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, *dptr);
    if (e != cudaSuccess) {
        cudaFree(*dptr);
        *dptr = nullptr;
        return set_error(ctx, ZKB_ECUDA, "zkb_peer_buffer_alloc: %s", cudaGetErrorString(e));
    }
    memcpy(handle, &h, 64);
    return ZKB_OK;
}
int zkb_peer_buffer_free(zkb_ctx* ctx, void* dptr) {
    if (!ctx) return ZKB_EINVAL;
    if (!dptr) return ZKB_OK;
    DeviceGuard g(ctx);
    ZKB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    ZKB_CUDA(ctx, cudaFree(dptr));
    return ZKB_OK;
}
int zkb_peer_buffer_open(zkb_ctx* ctx, const unsigned char handle[64], void** peer_ptr) {
    if (!ctx || !handle || !peer_ptr) return ZKB_EINVAL;
    DeviceGuard g(ctx);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    *peer_ptr = nullptr;
    ZKB_CUDA(ctx, cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return ZKB_OK;
}
int zkb_peer_buffer_close(zkb_ctx* ctx, void* peer_ptr) {
    if (!ctx) return ZKB_EINVAL;
    if (!peer_ptr) return ZKB_OK;
    DeviceGuard g(ctx);
    for (auto st : ctx->peer_streams)
        if (st) ZKB_CUDA(ctx, cudaStreamSynchronize(st));
    ZKB_CUDA(ctx, cudaIpcCloseMemHandle(peer_ptr));
    return ZKB_OK;
}
int zkb_copy_to_peer(zkb_ctx* ctx, void* dst, const void* src, size_t bytes, int lane) {
    if (!ctx || !dst || !src || lane < 0) return ZKB_EINVAL;
    DeviceGuard g(ctx);
    cudaStream_t& st = ctx->peer_streams[lane & 3];
    if (!st) ZKB_CUDA(ctx, cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    if (!ctx->copy_gate) ZKB_CUDA(ctx, cudaEventCreateWithFlags(&ctx->copy_gate, cudaEventDisableTiming));
    // after everything enqueued on the compute stream so far (the source has just been written there)
    ZKB_CUDA(ctx, cudaEventRecord(ctx->copy_gate, ctx->stream));
    ZKB_CUDA(ctx, cudaStreamWaitEvent(st, ctx->copy_gate, 0));
    if (bytes) ZKB_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, st));
    return ZKB_OK;
}
int zkb_peer_copies_wait(zkb_ctx* ctx) {
    if (!ctx) return ZKB_EINVAL;
    DeviceGuard g(ctx);
    for (auto st : ctx->peer_streams)
        if (st) ZKB_CUDA(ctx, cudaStreamSynchronize(st));
    return ZKB_OK;
}

int zkb_d2h_async(zkb_ctx* ctx, void* h_pinned_dst, const void* dptr, size_t bytes) {
    if (!ctx) return ZKB_EINVAL;
    if (bytes == 0) return ZKB_OK;
    ZKB_CHECK_ARG(ctx, dptr != nullptr && h_pinned_dst != nullptr);
    DeviceGuard g(ctx);
    ZKB_CUDA(ctx, cudaMemcpyAsync(h_pinned_dst, dptr, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return ZKB_OK;
}

int zkb_d2d(zkb_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx) return ZKB_EINVAL;
    if (bytes == 0) return ZKB_OK;
    ZKB_CHECK_ARG(ctx, dst != nullptr && src != nullptr);
    DeviceGuard g(ctx);
    ZKB_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return ZKB_OK;
}

int zkb_host_alloc_pinned(zkb_ctx* ctx, size_t bytes, void** h_ptr) {
    if (!ctx || !h_ptr) return ZKB_EINVAL;
    DeviceGuard g(ctx);
    ZKB_CUDA(ctx, cudaMallocHost(h_ptr, bytes ? bytes : 1));
    return ZKB_OK;
}

int zkb_host_free_pinned(zkb_ctx* ctx, void* h_ptr) {
    if (!ctx) return ZKB_EINVAL;
    if (!h_ptr) return ZKB_OK;
    DeviceGuard g(ctx);
    ZKB_CUDA(ctx, cudaFreeHost(h_ptr));
    return ZKB_OK;
}

int zkb_gather_multi(zkb_ctx* ctx, const uint32_t* const* cols, int ncols, const uint32_t* h_idx, int nidx,
                     uint32_t* h_out) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, ncols >= 0 && nidx >= 0);
    if (ncols == 0 || nidx == 0) return ZKB_OK;
    ZKB_CHECK_ARG(ctx, cols != nullptr && h_idx != nullptr && h_out != nullptr);
    size_t total = (size_t)ncols * nidx;
    ZKB_CHECK_ARG(ctx, total + (size_t)nidx <= ctx->scratch_words);
    DeviceGuard g(ctx);
    void** d_cols;
    int rc = stage_ptrs(ctx, (const void* const*)cols, ncols, &d_cols);
    if (rc) return rc;
    uint32_t* d_idx = ctx->scratch;
    uint32_t* d_out = ctx->scratch + nidx;
    ZKB_CUDA(ctx, cudaMemcpyAsync(d_idx, h_idx, (size_t)nidx * 4, cudaMemcpyHostToDevice, ctx->stream));
    gather_multi_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>((const uint32_t* const*)d_cols, ncols,
                                                                                  d_idx, nidx, d_out);
    ZKB_LAUNCH_CHECK(ctx);
    ZKB_CUDA(ctx, cudaMemcpyAsync(h_out, d_out, total * 4, cudaMemcpyDeviceToHost, ctx->stream));
    ZKB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return ZKB_OK;
}

int zkb_gather_words(zkb_ctx* ctx, const uint32_t* const* h_addrs, size_t n, uint32_t* h_out) {
    if (!ctx) return ZKB_EINVAL;
    if (n == 0) return ZKB_OK;
    ZKB_CHECK_ARG(ctx, h_addrs != nullptr && h_out != nullptr);
    DeviceGuard g(ctx);
    // addresses (2 words each) and results share the scratch buffer; large requests go in slices
    const size_t slice = ctx->scratch_words / 3;
    for (size_t off = 0; off < n; off += slice) {
        size_t m = n - off < slice ? n - off : slice;
        const uint32_t** d_addrs = reinterpret_cast<const uint32_t**>(ctx->scratch);
        uint32_t* d_out = ctx->scratch + 2 * slice;
        ZKB_CUDA(ctx, cudaMemcpyAsync(d_addrs, h_addrs + off, m * sizeof(void*), cudaMemcpyHostToDevice, ctx->stream));
        gather_words_kernel<<<(unsigned)((m + 255) / 256), 256, 0, ctx->stream>>>(d_addrs, m, d_out);
        ZKB_LAUNCH_CHECK(ctx);
        ZKB_CUDA(ctx, cudaMemcpyAsync(h_out + off, d_out, m * 4, cudaMemcpyDeviceToHost, ctx->stream));
        ZKB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
    return ZKB_OK;
}

int zkb_gather_hashes(zkb_ctx* ctx, const uint32_t* hashes, const uint32_t* h_idx, int nidx, uint32_t* h_out) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, nidx >= 0);
    if (nidx == 0) return ZKB_OK;
    ZKB_CHECK_ARG(ctx, hashes != nullptr && h_idx != nullptr && h_out != nullptr && ((uintptr_t)hashes & 15) == 0);
    ZKB_CHECK_ARG(ctx, (size_t)nidx * 9 + 4 <= ctx->scratch_words);
    DeviceGuard g(ctx);
    uint32_t* d_out = ctx->scratch;  // 8 words per hash, 16-byte aligned
    uint32_t* d_idx = ctx->scratch + 8 * (size_t)nidx;
    ZKB_CUDA(ctx, cudaMemcpyAsync(d_idx, h_idx, (size_t)nidx * 4, cudaMemcpyHostToDevice, ctx->stream));
    gather_hashes_kernel<<<(2 * nidx + 127) / 128, 128, 0, ctx->stream>>>(reinterpret_cast<const uint4*>(hashes), d_idx, nidx,
                                                                        reinterpret_cast<uint4*>(d_out));
    ZKB_LAUNCH_CHECK(ctx);
    ZKB_CUDA(ctx, cudaMemcpyAsync(h_out, d_out, (size_t)nidx * 32, cudaMemcpyDeviceToHost, ctx->stream));
    ZKB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return ZKB_OK;
}

int zkb_twiddles_d2h(zkb_ctx* ctx, int log_size, uint32_t* h_tw, uint32_t* h_itw) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, h_tw != nullptr && log_size >= 0 && log_size <= ctx->max_log - 1);
    DeviceGuard g(ctx);
    // Level j of the reference layout is T_{log_size - j}: 2^(log_size-j-1) words at offset
    // 2^log_size - 2^(log_size-j); the last word is the padding value 1.
    size_t n = (size_t)1 << log_size;
    for (int j = 0; j < log_size; j++) {
        int k = log_size - j;
        size_t len = (size_t)1 << (k - 1), off = n - ((size_t)1 << k);
        ZKB_CUDA(ctx, cudaMemcpyAsync(h_tw + off, ctx->tw + len, len * 4, cudaMemcpyDeviceToHost, ctx->stream));
        if (h_itw) ZKB_CUDA(ctx, cudaMemcpyAsync(h_itw + off, ctx->itw + len, len * 4, cudaMemcpyDeviceToHost, ctx->stream));
    }
    ZKB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    h_tw[n - 1] = 1u;
    if (h_itw) h_itw[n - 1] = 1u;
    return ZKB_OK;
}

int zkb_secure_powers(zkb_ctx* ctx, const uint32_t h_felt[4], size_t n, uint32_t* h_out) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, h_felt != nullptr && (n == 0 || h_out != nullptr));
    qm31 f{{h_felt[0], h_felt[1], h_felt[2], h_felt[3]}}, acc = qm31_one();
    for (size_t i = 0; i < n; i++) {
        for (int k = 0; k < 4; k++) h_out[4 * i + k] = acc.c[k];
        acc = qm31_mul(acc, f);
    }
    return ZKB_OK;
}

}  // extern "C"

namespace zk {

int gather_blocks(zkb_ctx* ctx, const GatherBlock* blocks, int n_blocks, size_t total_words, uint32_t* h_out) {
    if (n_blocks <= 0 || total_words == 0) return ZKB_OK;
    DeviceGuard g(ctx);
    std::vector<uint32_t> idx;
    for (int b = 0; b < n_blocks; b++) idx.insert(idx.end(), blocks[b].idx, blocks[b].idx + blocks[b].nidx);
    uint32_t* d_buf = nullptr;  // [indices | results]
    ZKB_CUDA(ctx, cudaMallocAsync((void**)&d_buf, (idx.size() + total_words) * 4, ctx->stream));
    cudaError_t e = cudaMemcpyAsync(d_buf, idx.data(), idx.size() * 4, cudaMemcpyHostToDevice, ctx->stream);
    uint32_t* d_out = d_buf + idx.size();
    size_t ioff = 0;
    int rc = ZKB_OK;
    for (int b = 0; b < n_blocks && e == cudaSuccess && rc == ZKB_OK; b++) {
        const GatherBlock& blk = blocks[b];
        size_t total = (size_t)blk.ncols * blk.nidx;
        if (total) {
            void** d_cols;
            rc = stage_ptrs(ctx, (const void* const*)blk.cols, blk.ncols, &d_cols);
            if (rc == ZKB_OK) {
                gather_multi_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>((const uint32_t* const*)d_cols, blk.ncols,
                                                                                              d_buf + ioff, blk.nidx, d_out + blk.out_off);
                e = cudaGetLastError();
            }
        }
        ioff += blk.nidx;
    }
    if (e == cudaSuccess && rc == ZKB_OK) e = cudaMemcpyAsync(h_out, d_out, total_words * 4, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess && rc == ZKB_OK) e = cudaStreamSynchronize(ctx->stream);
    cudaFreeAsync(d_buf, ctx->stream);
    if (rc != ZKB_OK) return rc;
    if (e != cudaSuccess) return set_error(ctx, ZKB_ECUDA, "gather_blocks: %s", cudaGetErrorString(e));
    return ZKB_OK;
}

}  // namespace zk
