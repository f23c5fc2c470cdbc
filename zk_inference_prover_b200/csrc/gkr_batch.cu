// GKR batches of many instances (the prover's reductions hold hundreds: one instance per component and
// power-of-two share of its lookups, prover/src/gkr_key_tile.rs:34-55). prove_batch
// (nitroo/crates/stwo/src/prover/lookups/gkr_prover.rs:657-882) runs ONE sum-check per layer over all
// instances, so what every instance needs in a round is known together. Here a round of the whole batch is
// one launch and one read-back, whatever the number of instances: a table of work items (one per instance)
// says what to do with which arrays, a flat grid of CTAs is split over the items in proportion to their
// size, and every item's eight result words (and, at the end of a layer, its two-entry mask) land in one
// result array.
//
//   mode 0  sum_as_poly_in_first_variable sums of the item's layer (first round of a layer's sum-check)
//   mode 1  fix_first_variable with the round's challenge on every column, and the sums of the fixed layer
//   mode 2  fix_first_variable of a 4-entry layer; the 2 fixed entries are also copied to the results (the mask)
//   mode 3  next_layer (generation of the towers)
//
// Arithmetic as in gkr.cu / gkr_fused.cu (cpu/lookups/gkr.rs:17-263, cpu/lookups/mle.rs:13-46).
#include "common.cuh"
#include "gkr_batch.hpp"

namespace zk {

namespace {

__device__ __forceinline__ qm31 ldqb(const uint32_t* __restrict__ p, size_t i) {
    uint4 v = reinterpret_cast<const uint4*>(p)[i];
    return {{v.x, v.y, v.z, v.w}};
}
__device__ __forceinline__ void stqb(uint32_t* __restrict__ p, size_t i, qm31 v) {
    reinterpret_cast<uint4*>(p)[i] = make_uint4(v.c[0], v.c[1], v.c[2], v.c[3]);
}
__device__ __forceinline__ qm31 foldb(qm31 r, qm31 a, qm31 b) { return qm31_add(qm31_mul(r, qm31_sub(b, a)), a); }
__device__ __forceinline__ qm31 fold_m31(qm31 r, uint32_t a, uint32_t b) {
    qm31 v = qm31_mul_m31(r, m31_sub(b, a));
    v.c[0] = m31_add(v.c[0], a);
    return v;
}
__device__ __forceinline__ qm31 warp_sumb(qm31 v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        qm31 o;
#pragma unroll
        for (int k = 0; k < 4; k++) o.c[k] = __shfl_down_sync(0xffffffffu, v.c[k], off);
        v = qm31_add(v, o);
    }
    return v;
}

// The item a CTA of the flat grid works for: the last item whose first CTA is not after this one.
__device__ __forceinline__ int find_item(const GkrBatchItem* __restrict__ items, int n_items, uint32_t block) {
    int lo = 0, hi = n_items - 1;
    while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if (items[mid].first_block <= block) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// One term of the round sums from the four denominators (and numerators) at (0, i, {0,1}) and (1, i, {0,1}).
template <int KIND>
__device__ __forceinline__ void term(const qm31 d[4], const qm31 nu[4], qm31 lambda, qm31& t0, qm31& t2) {
    qm31 d20 = qm31_sub(qm31_dbl(d[2]), d[0]), d21 = qm31_sub(qm31_dbl(d[3]), d[1]);
    if (KIND == ZKB_GKR_GRAND_PRODUCT) {
        t0 = qm31_mul(d[0], d[1]);
        t2 = qm31_mul(d20, d21);
        return;
    }
    qm31 n0, n2;
    if (KIND == ZKB_GKR_LOGUP_SINGLES) {
        n0 = qm31_add(d[0], d[1]);
        n2 = qm31_add(d20, d21);
    } else {
        qm31 n20 = qm31_sub(qm31_dbl(nu[2]), nu[0]), n21 = qm31_sub(qm31_dbl(nu[3]), nu[1]);
        n0 = qm31_add(qm31_mul(d[1], nu[0]), qm31_mul(d[0], nu[1]));
        n2 = qm31_add(qm31_mul(d21, n20), qm31_mul(d20, n21));
    }
    t0 = qm31_add(n0, qm31_mul(lambda, qm31_mul(d[0], d[1])));
    t2 = qm31_add(n2, qm31_mul(lambda, qm31_mul(d20, d21)));
}

template <int KIND>
__device__ __forceinline__ void item_sums(const GkrBatchItem& it, uint32_t bx, qm31 r, const uint32_t* __restrict__ eq, qm31 lambda, qm31& s0,
                                          qm31& s2) {
    const size_t stride = (size_t)it.blocks * blockDim.x;
    if (it.mode == 0) {
        const size_t nt = it.n / 4;  // entries (0, i, b) at 2i + b, (1, i, b) at 2(nt + i) + b
        for (size_t i = (size_t)bx * blockDim.x + threadIdx.x; i < nt; i += stride) {
            const size_t o[4] = {2 * i, 2 * i + 1, 2 * (nt + i), 2 * (nt + i) + 1};
            qm31 d[4], nu[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                d[q] = ldqb(it.den, o[q]);
                if (KIND == ZKB_GKR_LOGUP_GENERIC) nu[q] = ldqb(it.num, o[q]);
                else if (KIND == ZKB_GKR_LOGUP_MULTIPLICITIES) nu[q] = qm31_from_m31(it.num[o[q]]);
            }
            qm31 t0, t2;
            term<KIND>(d, nu, lambda, t0, t2);
            qm31 e = ldqb(eq, i);
            s0 = qm31_add(s0, qm31_mul(e, t0));
            s2 = qm31_add(s2, qm31_mul(e, t2));
        }
    } else {
        const size_t half = it.n / 2, nt = half / 4;
        for (size_t i = (size_t)bx * blockDim.x + threadIdx.x; i < nt; i += stride) {
            const size_t o[4] = {2 * i, 2 * i + 1, 2 * (nt + i), 2 * (nt + i) + 1};
            qm31 d[4], nu[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                d[q] = foldb(r, ldqb(it.den, o[q]), ldqb(it.den, o[q] + half));
                stqb(it.den_out, o[q], d[q]);
                if (KIND == ZKB_GKR_LOGUP_GENERIC) {
                    nu[q] = foldb(r, ldqb(it.num, o[q]), ldqb(it.num, o[q] + half));
                    stqb(it.num_out, o[q], nu[q]);
                } else if (KIND == ZKB_GKR_LOGUP_MULTIPLICITIES) {
                    nu[q] = fold_m31(r, it.num[o[q]], it.num[o[q] + half]);
                    stqb(it.num_out, o[q], nu[q]);
                }
            }
            qm31 t0, t2;
            term<KIND>(d, nu, lambda, t0, t2);
            qm31 e = ldqb(eq, i);
            s0 = qm31_add(s0, qm31_mul(e, t0));
            s2 = qm31_add(s2, qm31_mul(e, t2));
        }
    }
}

// The CTA that completes an item reports it: when every item of the launch has reported, the round's sequence number is
// written after the results. `results` and `flag` are page-locked host memory the device writes directly, so the host sees
// a round's results a PCIe write after the last CTA ends, without a copy and a stream synchronisation of its own (a round of
// a small batch is a 5-10 us kernel; the copy and the wake-up cost as much again).
__device__ __forceinline__ void item_done(unsigned int* done, int n_items, volatile unsigned int* flag, unsigned int round_id) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        if (atomicAdd(done, 1u) == (unsigned int)n_items - 1u) {
            *done = 0u;  // every item has counted: ready for the next launch
            __threadfence_system();
            *flag = round_id;
        }
    }
}

__global__ void __launch_bounds__(256) gkr_batch_round_kernel(const GkrBatchItem* __restrict__ items, int n_items, qm31 r,
                                                              const uint32_t* __restrict__ eq, qm31 lambda, uint32_t* __restrict__ partials,
                                                              unsigned int* __restrict__ tickets, uint32_t* __restrict__ results,
                                                              unsigned int* __restrict__ done, volatile unsigned int* flag, unsigned int round_id) {
    const int idx = find_item(items, n_items, blockIdx.x);
    const GkrBatchItem it = items[idx];
    const uint32_t bx = blockIdx.x - it.first_block;
    uint32_t* res = results + (size_t)GKR_BATCH_RESULT_WORDS * idx;
    if (it.mode == 2) {
        // four entries -> two; one thread per (column, entry)
        if (threadIdx.x < 2) {
            qm31 dv = foldb(r, ldqb(it.den, threadIdx.x), ldqb(it.den, threadIdx.x + 2));
            stqb(it.den_out, threadIdx.x, dv);
            stqb(res + 8, threadIdx.x, dv);
            if (it.kind == ZKB_GKR_LOGUP_GENERIC || it.kind == ZKB_GKR_LOGUP_MULTIPLICITIES) {
                qm31 nv = it.kind == ZKB_GKR_LOGUP_GENERIC ? foldb(r, ldqb(it.num, threadIdx.x), ldqb(it.num, threadIdx.x + 2))
                                                           : fold_m31(r, it.num[threadIdx.x], it.num[threadIdx.x + 2]);
                stqb(it.num_out, threadIdx.x, nv);
                stqb(res + 16, threadIdx.x, nv);
            }
        }
        item_done(done, n_items, flag, round_id);
        return;
    }
    qm31 s0 = qm31_zero(), s2 = qm31_zero();
    switch (it.kind) {
        case ZKB_GKR_GRAND_PRODUCT: item_sums<ZKB_GKR_GRAND_PRODUCT>(it, bx, r, eq, lambda, s0, s2); break;
        case ZKB_GKR_LOGUP_GENERIC: item_sums<ZKB_GKR_LOGUP_GENERIC>(it, bx, r, eq, lambda, s0, s2); break;
        case ZKB_GKR_LOGUP_MULTIPLICITIES: item_sums<ZKB_GKR_LOGUP_MULTIPLICITIES>(it, bx, r, eq, lambda, s0, s2); break;
        default: item_sums<ZKB_GKR_LOGUP_SINGLES>(it, bx, r, eq, lambda, s0, s2); break;
    }
    __shared__ uint32_t sh[8][8];
    __shared__ bool is_last;
    s0 = warp_sumb(s0);
    s2 = warp_sumb(s2);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < 4; k++) { sh[warp][k] = s0.c[k]; sh[warp][4 + k] = s2.c[k]; }
    }
    __syncthreads();
    uint32_t* part = partials + 8 * (size_t)it.first_block;
    if (threadIdx.x < 8) {
        uint32_t acc = 0;
        for (int w = 0; w < 8; w++) acc = m31_add(acc, sh[w][threadIdx.x]);
        if (it.blocks == 1) res[threadIdx.x] = acc;
        else { part[8 * bx + threadIdx.x] = acc; __threadfence(); }
    }
    if (it.blocks == 1) {
        item_done(done, n_items, flag, round_id);
        return;
    }
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(tickets + idx, 1u) == it.blocks - 1;
    __syncthreads();
    if (is_last) {
        __threadfence();
        if (threadIdx.x < 8) {
            uint32_t acc = 0;
            for (uint32_t b = 0; b < it.blocks; b++) acc = m31_add(acc, __ldcg(&part[8 * b + threadIdx.x]));
            res[threadIdx.x] = acc;
        }
        if (threadIdx.x == 0) tickets[idx] = 0u;
        item_done(done, n_items, flag, round_id);
    }
}

template <int KIND>
__device__ __forceinline__ void item_next_layer(const GkrBatchItem& it, uint32_t bx) {
    const size_t half = it.n / 2, stride = (size_t)it.blocks * blockDim.x;
    for (size_t i = (size_t)bx * blockDim.x + threadIdx.x; i < half; i += stride) {
        qm31 d0 = ldqb(it.den, 2 * i), d1 = ldqb(it.den, 2 * i + 1);
        if (KIND != ZKB_GKR_GRAND_PRODUCT) {
            qm31 n;
            if (KIND == ZKB_GKR_LOGUP_SINGLES) n = qm31_add(d0, d1);
            else if (KIND == ZKB_GKR_LOGUP_MULTIPLICITIES) n = qm31_add(qm31_mul_m31(d1, it.num[2 * i]), qm31_mul_m31(d0, it.num[2 * i + 1]));
            else n = qm31_add(qm31_mul(d1, ldqb(it.num, 2 * i)), qm31_mul(d0, ldqb(it.num, 2 * i + 1)));
            stqb(it.num_out, i, n);
        }
        stqb(it.den_out, i, qm31_mul(d0, d1));
    }
}

__global__ void __launch_bounds__(256) gkr_batch_next_layer_kernel(const GkrBatchItem* __restrict__ items, int n_items) {
    const int idx = find_item(items, n_items, blockIdx.x);
    const GkrBatchItem it = items[idx];
    const uint32_t bx = blockIdx.x - it.first_block;
    switch (it.kind) {
        case ZKB_GKR_GRAND_PRODUCT: item_next_layer<ZKB_GKR_GRAND_PRODUCT>(it, bx); break;
        case ZKB_GKR_LOGUP_GENERIC: item_next_layer<ZKB_GKR_LOGUP_GENERIC>(it, bx); break;
        case ZKB_GKR_LOGUP_MULTIPLICITIES: item_next_layer<ZKB_GKR_LOGUP_MULTIPLICITIES>(it, bx); break;
        default: item_next_layer<ZKB_GKR_LOGUP_SINGLES>(it, bx); break;
    }
}

// Splits the flat grid over the items (first_block, blocks) by the work each has; returns the number of CTAs.
uint32_t plan_blocks(GkrBatchItem* items, int n_items, uint32_t threads_per_unit_shift) {
    uint32_t total = 0;
    for (int k = 0; k < n_items; k++) {
        GkrBatchItem& it = items[k];
        size_t units = it.mode == 3 ? it.n / 2 : it.mode == 0 ? it.n / 4 : it.mode == 1 ? it.n / 8 : 1;
        size_t blocks = (units + 255) / 256;
        blocks = (blocks + threads_per_unit_shift) >> threads_per_unit_shift;  // a few units per thread on large items
        if (blocks < 1) blocks = 1;
        if (blocks > 148u * 4u) blocks = 148u * 4u;
        it.first_block = total;
        it.blocks = (uint32_t)blocks;
        total += it.blocks;
    }
    return total;
}

int stage_items(zkb_ctx* ctx, const GkrBatchItem* items, int n_items, const GkrBatchItem** d_items) {
    static_assert(sizeof(GkrBatchItem) % sizeof(void*) == 0, "items are staged through the pointer ring");
    void** d = nullptr;
    int rc = stage_ptrs(ctx, reinterpret_cast<const void* const*>(items), (int)(n_items * (sizeof(GkrBatchItem) / sizeof(void*))), &d);
    if (rc) return rc;
    *d_items = reinterpret_cast<const GkrBatchItem*>(d);
    return ZKB_OK;
}

}  // namespace

int gkr_batch_next_layer(zkb_ctx* ctx, GkrBatchItem* items, int n_items) {
    if (n_items <= 0) return ZKB_OK;
    if ((size_t)n_items > GKR_BATCH_MAX_ITEMS) return set_error(ctx, ZKB_EINVAL, "gkr batch: more than %d instances", (int)GKR_BATCH_MAX_ITEMS);
    DeviceGuard g(ctx);
    for (int k = 0; k < n_items; k++) items[k].mode = 3;
    uint32_t total = plan_blocks(items, n_items, 1);
    const GkrBatchItem* d_items;
    int rc = stage_items(ctx, items, n_items, &d_items);
    if (rc) return rc;
    ProfScope prof(ctx, "gkr_batch_next_layer_kernel");
    gkr_batch_next_layer_kernel<<<total, 256, 0, ctx->stream>>>(d_items, n_items);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

int gkr_batch_round(zkb_ctx* ctx, GkrBatchItem* items, int n_items, const uint32_t h_r[4], const uint32_t* eq_evals, const uint32_t h_lambda[4],
                    uint32_t* h_results) {
    if (n_items <= 0) return ZKB_OK;
    if ((size_t)n_items > GKR_BATCH_MAX_ITEMS) return set_error(ctx, ZKB_EINVAL, "gkr batch: more than %d instances", (int)GKR_BATCH_MAX_ITEMS);
    DeviceGuard g(ctx);
    uint32_t total = plan_blocks(items, n_items, 0);
    if (!ctx->batch_tickets) {
        // tickets per item, then the launch's count of completed items
        ZKB_CUDA(ctx, cudaMalloc(&ctx->batch_tickets, (GKR_BATCH_MAX_ITEMS + 1) * sizeof(unsigned int)));
        ZKB_CUDA(ctx, cudaMemsetAsync(ctx->batch_tickets, 0, (GKR_BATCH_MAX_ITEMS + 1) * sizeof(unsigned int), ctx->stream));
        // results per item, then the sequence number of the last completed round
        ZKB_CUDA(ctx, cudaMallocHost(&ctx->h_batch, (GKR_BATCH_RESULT_WORDS * GKR_BATCH_MAX_ITEMS + 1) * 4));
        ctx->h_batch[GKR_BATCH_RESULT_WORDS * GKR_BATCH_MAX_ITEMS] = 0;
        ctx->batch_round = 0;
    }
    // The device writes the results straight into the page-locked host buffer (unified addressing: the host pointer is valid
    // on the device). scratch: [(unused) | partials]
    uint32_t* results = ctx->h_batch;
    unsigned int* tickets = ctx->batch_tickets;
    uint32_t* partials = ctx->scratch + (size_t)(GKR_BATCH_RESULT_WORDS + 1) * GKR_BATCH_MAX_ITEMS;
    if ((size_t)(GKR_BATCH_RESULT_WORDS + 1) * GKR_BATCH_MAX_ITEMS + 8 * (size_t)total > ctx->scratch_words)
        return set_error(ctx, ZKB_EINVAL, "gkr batch: %u CTAs exceed the scratch buffer", total);
    const GkrBatchItem* d_items;
    int rc = stage_items(ctx, items, n_items, &d_items);
    if (rc) return rc;
    volatile unsigned int* flag = reinterpret_cast<volatile unsigned int*>(ctx->h_batch + GKR_BATCH_RESULT_WORDS * GKR_BATCH_MAX_ITEMS);
    const unsigned int round_id = ++ctx->batch_round;
    qm31 r{{h_r[0], h_r[1], h_r[2], h_r[3]}}, lam{{h_lambda[0], h_lambda[1], h_lambda[2], h_lambda[3]}};
    {
        ProfScope prof(ctx, "gkr_batch_round_kernel");
        gkr_batch_round_kernel<<<total, 256, 0, ctx->stream>>>(d_items, n_items, r, eq_evals, lam, partials, tickets, results,
                                                               ctx->batch_tickets + GKR_BATCH_MAX_ITEMS, flag, round_id);
    }
    const size_t bytes = (size_t)n_items * GKR_BATCH_RESULT_WORDS * 4;
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess && !ctx->prof_on) {
        // wait on the host for the round's sequence number: a bounded spin (about 20 ms), then the stream
        for (long spin = 0; spin < 20000000L && *flag != round_id; spin++) {
#if defined(__x86_64__)
            __builtin_ia32_pause();
#endif
        }
    }
    if (e == cudaSuccess && *flag != round_id) e = cudaStreamSynchronize(ctx->stream);
    if (e == cudaSuccess && *flag != round_id) e = cudaErrorUnknown;  // the launch ended without completing every item
    if (e != cudaSuccess) {
        // a launch that did not run to its end may have left tickets counted up
        cudaMemsetAsync(ctx->batch_tickets, 0, (GKR_BATCH_MAX_ITEMS + 1) * sizeof(unsigned int), ctx->stream);
        return set_error(ctx, ZKB_ECUDA, "gkr batch round: %s", cudaGetErrorString(e));
    }
    memcpy(h_results, ctx->h_batch, bytes);
    return ZKB_OK;
}

}  // namespace zk
