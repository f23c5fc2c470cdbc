// Shared declarations of the zkb200 library: the context, error handling, pointer-table staging.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "../../include/zkb200.h"
#include "m31.cuh"

struct zkb_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    int max_log = 0;
    // Twiddle tower. T_k = x-coordinates of the first half of Coset::half_odds(k), bit-reversed,
    // 2^(k-1) words at offset 2^(k-1), for k = 1 .. max_log-1. Word 0 is 1. itw holds the inverses.
    uint32_t* tw = nullptr;
    uint32_t* itw = nullptr;
    size_t tw_len = 0;
    // The same two towers with every word doubled (2t < 2^32): what the radix-32 butterflies multiply by.
    uint32_t* tw2 = nullptr;
    uint32_t* itw2 = nullptr;
    // One word the kernels with bounded waits set when a wait ran out (0 = none); read by zkb_sync.
    unsigned int* dev_err = nullptr;
    // Staging ring for tables of column pointers (pinned host mirror + device copy).
    void** h_ring = nullptr;
    void** d_ring = nullptr;
    size_t ring_cap = 0, ring_pos = 0;
    // Scratch for per-block partial results (round sums, point evaluations) and a ticket counter.
    uint32_t* scratch = nullptr;
    size_t scratch_words = 0;
    unsigned int* ticket = nullptr;
    uint32_t* h_small = nullptr;  // pinned, for small results read back by the host
    // Batched GKR rounds (gkr_batch.cu): per-item tickets (zero between launches: the last CTA of an item clears its own)
    // and a pinned landing buffer for the per-item results; both allocated on first use.
    unsigned int* batch_tickets = nullptr;
    uint32_t* h_batch = nullptr;
    unsigned int batch_round = 0;  // sequence number of the last batched round launched
    cudaEvent_t events[64] = {nullptr};
    // A second stream for host-to-device copies that overlap compute, and the fences between the two.
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t fences[64] = {nullptr};
    cudaEvent_t copy_gate = nullptr;  // orders the copy stream after allocations made on `stream`
    cudaStream_t peer_streams[4] = {nullptr, nullptr, nullptr, nullptr};  // device-to-device copies to other GPUs, side by side
    // Optional per-kernel timeline (zkb_profile_*): pairs of events around selected launches.
    bool prof_on = false;
    struct ProfRec { const char* name; cudaEvent_t a, b; };
    ProfRec* prof = nullptr;
    int prof_n = 0, prof_cap = 0;
    char err[512] = {0};
};

namespace zk {

constexpr int RING_SLOTS = 1 << 18;        // pointer-table staging capacity (2 MiB of pointers)
constexpr size_t SCRATCH_WORDS = 1 << 22;  // 16 MiB of scratch words
constexpr int SMALL_WORDS = 4096;

int set_error(zkb_ctx* ctx, int code, const char* fmt, ...);

#define ZKB_CHECK_ARG(ctx, cond)                                                        \
    do {                                                                                \
        if (!(cond)) return zk::set_error(ctx, ZKB_EINVAL, "%s: invalid argument: %s", __func__, #cond); \
    } while (0)

#define ZKB_CUDA(ctx, call)                                                             \
    do {                                                                                \
        cudaError_t e__ = (call);                                                       \
        if (e__ != cudaSuccess)                                                         \
            return zk::set_error(ctx, e__ == cudaErrorMemoryAllocation ? ZKB_ENOMEM : ZKB_ECUDA, \
                                 "%s: %s: %s", __func__, #call, cudaGetErrorString(e__)); \
    } while (0)

#define ZKB_LAUNCH_CHECK(ctx) ZKB_CUDA(ctx, cudaGetLastError())

// RAII guard making the context's device current for the duration of a call.
struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(const zkb_ctx* ctx) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != ctx->device) ok = cudaSetDevice(ctx->device) == cudaSuccess;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

// Copies `n` host-resident device pointers into the staging ring and returns their device
// address through *out. Ordered on the context's stream.
int stage_ptrs(zkb_ctx* ctx, const void* const* h_ptrs, int n, void*** out);
// The same ring for a block of bytes that the device reads as 16-byte vectors: starts on a 16-byte boundary.
int stage_blob(zkb_ctx* ctx, const void* h_data, size_t bytes, void** out);

// Brackets a kernel launch with events when the timeline is on (see zkb_profile_begin).
struct ProfScope {
    zkb_ctx* ctx;
    int slot = -1;
    ProfScope(zkb_ctx* c, const char* name) : ctx(c) {
        if (!c->prof_on || c->prof_n >= c->prof_cap) return;
        slot = c->prof_n++;
        c->prof[slot].name = name;
        if (!c->prof[slot].a) { cudaEventCreate(&c->prof[slot].a); cudaEventCreate(&c->prof[slot].b); }
        cudaEventRecord(c->prof[slot].a, c->stream);
    }
    ~ProfScope() {
        if (slot >= 0) cudaEventRecord(ctx->prof[slot].b, ctx->stream);
    }
};

// Reserves `words` of scratch (whole buffer is shared; one user per enqueued op sequence).
inline uint32_t* scratch_ptr(zkb_ctx* ctx) { return ctx->scratch; }

// Domain point helpers on the device, from the twiddle tower (tw or itw).
// For the canonic circle domain of log size L >= 3 in bit-reversed order, rows 2i and 2i+1 are
// p_i and its conjugate, with p_i the i-th point of Coset::half_odds(L-1) in bit-reversed order.
// Four consecutive half-coset points are (x,y), (-x,-y), (y,-x), (-y,x) with x = T[2q], y = T[2q+1]
// (nitroo/crates/stwo/src/prover/backend/cpu/circle.rs:312-332).
__device__ __forceinline__ void half_coset_point(const uint32_t* __restrict__ tower, int L, uint32_t i, uint32_t& px,
                                                 uint32_t& py) {
    const uint32_t* T = tower + (1u << (L - 2));
    uint32_t q = i >> 2, r = i & 3;
    uint32_t x = T[2 * q], y = T[2 * q + 1];
    uint32_t ax = (r & 2) ? y : x;   // r=0,1: x ; r=2,3: y
    uint32_t ay = (r & 2) ? x : y;   // r=0,1: y ; r=2,3: x
    // signs: r=0 (+,+), r=1 (-,-), r=2 (+,-), r=3 (-,+)
    px = (r & 1) ? m31_neg(ax) : ax;
    py = (r == 1 || r == 2) ? m31_neg(ay) : ay;
}

}  // namespace zk
