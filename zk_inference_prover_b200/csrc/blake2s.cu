// MerkleOps::commit_on_layer with the Blake2s hasher, and the proof-of-work grind.
//
// A node's message is [left child hash | right child hash |] col_0[i] | col_1[i] | ... with every
// column value as one little-endian word (nitroo/crates/stwo/src/core/vcs/blake2_merkle.rs:18-39),
// hashed with Blake2s-256 (RFC 7693) and, for the M31 hasher, each digest word reduced mod 2^31-1
// (core/vcs/blake2_hash.rs:111-118). One thread hashes one node: the column words ARE the message
// words, so a 64-byte block is 16 coalesced loads (one per column) straight into registers.
#include "blake2s.cuh"
#include "common.cuh"

namespace zk {

__device__ __forceinline__ void store_hash(uint32_t* __restrict__ out, size_t i, const uint32_t h[8], bool m31_out) {
    uint32_t r[8];
#pragma unroll
    for (int k = 0; k < 8; k++) r[k] = m31_out ? reduce_word_m31(h[k]) : h[k];
    uint4* o = reinterpret_cast<uint4*>(out + 8 * i);
    o[0] = make_uint4(r[0], r[1], r[2], r[3]);
    o[1] = make_uint4(r[4], r[5], r[6], r[7]);
}

__global__ void __launch_bounds__(256) merkle_layer_kernel(int log_size, const uint32_t* __restrict__ prev,
                                                           const uint32_t* const* __restrict__ cols, int ncols,
                                                           int m31_out, uint32_t* __restrict__ out) {
    const size_t n = (size_t)1 << log_size;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    uint32_t h[8], m[16];
    blake2s_init(h);
    const uint32_t total = (prev ? 64u : 0u) + 4u * (uint32_t)ncols;
    uint32_t t = 0;
    int c = 0;
    if (prev) {
        const uint4* p = reinterpret_cast<const uint4*>(prev + 16 * i);
        uint4 a = p[0], b = p[1], cc = p[2], d = p[3];
        m[0] = a.x; m[1] = a.y; m[2] = a.z; m[3] = a.w; m[4] = b.x; m[5] = b.y; m[6] = b.z; m[7] = b.w;
        m[8] = cc.x; m[9] = cc.y; m[10] = cc.z; m[11] = cc.w; m[12] = d.x; m[13] = d.y; m[14] = d.z; m[15] = d.w;
        t = 64;
        blake2s_compress(h, m, t, total == 64u);
    }
    // full blocks of 16 columns that are not the last block
    while (ncols - c > 16) {
#pragma unroll
        for (int k = 0; k < 16; k++) m[k] = cols[c + k][i];
        c += 16;
        t += 64;
        blake2s_compress(h, m, t, false);
    }
    // last block: 1..16 remaining columns, or the empty message when nothing was hashed yet
    if (ncols - c > 0 || total == 0u) {
        int rem = ncols - c;
#pragma unroll
        for (int k = 0; k < 16; k++) m[k] = (k < rem) ? cols[c + k][i] : 0u;
        t += 4u * (uint32_t)rem;
        blake2s_compress(h, m, t, true);
    }
    store_hash(out, i, h, m31_out != 0);
}

// The same node hash for layers of few rows and many columns (a segment's trees hold tens of thousands of columns of
// 2^8 ... 2^11 rows: a leaf is then a chain of up to 2,000 compressions on a few hundred threads, and what a thread waits for
// is the memory latency of its next sixteen column words, not the arithmetic). A warp issues in order, so a word whose column
// pointer has not arrived holds up the compression behind it: the loads therefore run two blocks deep. During the compression
// of block b the sixteen words of block b + 1 are in flight (their pointers arrived during block b - 1) and so are the sixteen
// pointers of block b + 2. (Spreading a compression over four lanes was tried for these layers and is slower: the four column
// steps of a round are already independent instructions of one thread, and the lane exchanges add latency.)
__global__ void __launch_bounds__(256) merkle_layer_prefetch_kernel(int log_size, const uint32_t* __restrict__ prev,
                                                                    const uint32_t* const* __restrict__ cols, int ncols, int m31_out,
                                                                    uint32_t* __restrict__ out) {
    const size_t n = (size_t)1 << log_size;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    uint32_t h[8], m[16], nx[16];
    const uint32_t* pp[16];
    blake2s_init(h);
    const uint32_t total = (prev ? 64u : 0u) + 4u * (uint32_t)ncols;
    uint32_t t = 0;
    const int full = ncols > 0 ? (ncols - 1) / 16 : 0;  // blocks of sixteen columns that are not the last block
    if (full > 0) {
#pragma unroll
        for (int k = 0; k < 16; k++) pp[k] = cols[k];
#pragma unroll
        for (int k = 0; k < 16; k++) nx[k] = __ldg(pp[k] + i);
    }
    if (full > 1) {
#pragma unroll
        for (int k = 0; k < 16; k++) pp[k] = cols[16 + k];
    }
    if (prev) {
        const uint4* p = reinterpret_cast<const uint4*>(prev + 16 * i);
        uint4 a = p[0], b = p[1], cc = p[2], d = p[3];
        m[0] = a.x; m[1] = a.y; m[2] = a.z; m[3] = a.w; m[4] = b.x; m[5] = b.y; m[6] = b.z; m[7] = b.w;
        m[8] = cc.x; m[9] = cc.y; m[10] = cc.z; m[11] = cc.w; m[12] = d.x; m[13] = d.y; m[14] = d.z; m[15] = d.w;
        t = 64;
        blake2s_compress(h, m, t, total == 64u);
    }
    for (int b = 0; b < full; b++) {
#pragma unroll
        for (int k = 0; k < 16; k++) m[k] = nx[k];
        if (b + 1 < full) {
#pragma unroll
            for (int k = 0; k < 16; k++) nx[k] = __ldg(pp[k] + i);
        }
        if (b + 2 < full) {
            const uint32_t* const* cp = cols + 16 * (b + 2);
#pragma unroll
            for (int k = 0; k < 16; k++) pp[k] = cp[k];
        }
        t += 64;
        blake2s_compress(h, m, t, false);
    }
    const int c = 16 * full;
    if (ncols - c > 0 || total == 0u) {
        int rem = ncols - c;
#pragma unroll
        for (int k = 0; k < 16; k++) m[k] = (k < rem) ? cols[c + k][i] : 0u;
        t += 4u * (uint32_t)rem;
        blake2s_compress(h, m, t, true);
    }
    store_hash(out, i, h, m31_out != 0);
}

// A leaf layer (no children) hashed in several calls, a run of columns at a time, so that hashing can
// start while later columns are still being produced. `out` carries the chaining value between calls
// (8 words per leaf, exactly the space of the final hash). A call that is not the last one absorbs
// whole 64-byte blocks only (ncols a multiple of 16); the last call pads and finalises.
__global__ void __launch_bounds__(256) merkle_leaves_partial_kernel(int log_size, const uint32_t* const* __restrict__ cols,
                                                                    int ncols, uint32_t cols_before, int is_last, int m31_out,
                                                                    uint32_t* __restrict__ out) {
    const size_t n = (size_t)1 << log_size;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    uint32_t h[8], m[16];
    uint4* o = reinterpret_cast<uint4*>(out + 8 * i);
    if (cols_before == 0) {
        blake2s_init(h);
    } else {
        uint4 a = o[0], b = o[1];
        h[0] = a.x; h[1] = a.y; h[2] = a.z; h[3] = a.w; h[4] = b.x; h[5] = b.y; h[6] = b.z; h[7] = b.w;
    }
    uint32_t t = 4u * cols_before;
    int c = 0;
    while (ncols - c > 16 || (!is_last && ncols - c == 16)) {
#pragma unroll
        for (int k = 0; k < 16; k++) m[k] = cols[c + k][i];
        c += 16;
        t += 64;
        blake2s_compress(h, m, t, false);
    }
    if (is_last) {
        int rem = ncols - c;
#pragma unroll
        for (int k = 0; k < 16; k++) m[k] = (k < rem) ? cols[c + k][i] : 0u;
        t += 4u * (uint32_t)rem;
        blake2s_compress(h, m, t, true);
        store_hash(out, i, h, m31_out != 0);
    } else {
        o[0] = make_uint4(h[0], h[1], h[2], h[3]);
        o[1] = make_uint4(h[4], h[5], h[6], h[7]);
    }
}

// The top of a tree in one launch: layers 2^(top_log-1) ... 2^0 from layer 2^top_log, nodes only
// (no columns are injected). One CTA; a barrier separates the levels.
constexpr int MERKLE_TOP_MAX_LOG = 10;
struct MerkleTopArgs { uint32_t* layer[MERKLE_TOP_MAX_LOG + 1]; };  // layer[k]: 2^k hashes


// Several consecutive layers of nodes (no columns) in one launch: a CTA takes 512 child hashes and builds up to nine levels
// above them, every level written to its own layer array and kept in shared memory for the next one. A layer of a tree is
// one compression per node whatever the launch shape; what this saves is a launch (and its drain and refill of the whole
// GPU) per layer, for the layers between the leaves and the last ten, which merkle_top_kernel builds.
constexpr int MERKLE_LEVELS_MAX = 9;
struct MerkleLevelsArgs {
    const uint32_t* children;             // 2^child_log hashes
    uint32_t* out[MERKLE_LEVELS_MAX + 1];  // out[j]: the layer j levels above the children (2^(child_log - j) hashes), j = 1..levels
};
__global__ void __launch_bounds__(256) merkle_levels_kernel(MerkleLevelsArgs a, int levels, int m31_out) {
    __shared__ uint32_t sh[2][256][8];
    const size_t cta = blockIdx.x;
    uint32_t h[8], m[16];
    {
        blake2s_init(h);
        const uint4* p = reinterpret_cast<const uint4*>(a.children + 16 * (cta * 256 + threadIdx.x));
        uint4 x0 = p[0], x1 = p[1], x2 = p[2], x3 = p[3];
        m[0] = x0.x; m[1] = x0.y; m[2] = x0.z; m[3] = x0.w; m[4] = x1.x; m[5] = x1.y; m[6] = x1.z; m[7] = x1.w;
        m[8] = x2.x; m[9] = x2.y; m[10] = x2.z; m[11] = x2.w; m[12] = x3.x; m[13] = x3.y; m[14] = x3.z; m[15] = x3.w;
        blake2s_compress(h, m, 64u, true);
#pragma unroll
        for (int k = 0; k < 8; k++) { h[k] = m31_out ? reduce_word_m31(h[k]) : h[k]; sh[1][threadIdx.x][k] = h[k]; }
        store_hash(a.out[1], cta * 256 + threadIdx.x, h, false);
    }
    for (int j = 2; j <= levels; j++) {
        __syncthreads();
        const uint32_t n = 512u >> j;  // nodes of this level in the CTA
        if (threadIdx.x < n) {
            const uint32_t(*src)[8] = sh[(j - 1) & 1];
            blake2s_init(h);
#pragma unroll
            for (int k = 0; k < 8; k++) { m[k] = src[2 * threadIdx.x][k]; m[8 + k] = src[2 * threadIdx.x + 1][k]; }
            blake2s_compress(h, m, 64u, true);
#pragma unroll
            for (int k = 0; k < 8; k++) { h[k] = m31_out ? reduce_word_m31(h[k]) : h[k]; sh[j & 1][threadIdx.x][k] = h[k]; }
            store_hash(a.out[j], cta * n + threadIdx.x, h, false);
        }
    }
}

// Blake2sM31Channel on the device, for protocol loops whose next launch only needs a challenge
// (FRI: mix the layer's root, draw the folding challenge). State: chan[0..8) = digest, chan[8] = n_draws.
// mix_root is H(digest || root) (core/vcs/blake2_merkle.rs:53-58); draw_secure_felt hashes
// digest || n_draws (LE) || 0x00 and retries while a word is >= 2p (core/channel/blake2s.rs:34-52,
// 95-120); every digest word is reduced mod p.
__device__ __forceinline__ void channel_mix_root_draw(uint32_t* __restrict__ chan, const uint32_t* root,
                                                      uint32_t* __restrict__ alpha_out, uint32_t* __restrict__ root_copy) {
    uint32_t h[8], m[16];
    blake2s_init(h);
#pragma unroll
    for (int k = 0; k < 8; k++) { m[k] = chan[k]; m[8 + k] = root[k]; }
    blake2s_compress(h, m, 64u, true);
    uint32_t digest[8];
#pragma unroll
    for (int k = 0; k < 8; k++) digest[k] = reduce_word_m31(h[k]);
    uint32_t n_draws = 0, u[8];
    for (int attempt = 0; attempt < 64; attempt++) {  // the words are already below p: one pass in practice
        blake2s_init(h);
#pragma unroll
        for (int k = 0; k < 8; k++) m[k] = digest[k];
        m[8] = n_draws;
#pragma unroll
        for (int k = 9; k < 16; k++) m[k] = 0u;
        blake2s_compress(h, m, 37u, true);
        n_draws++;
        bool ok = true;
#pragma unroll
        for (int k = 0; k < 8; k++) { u[k] = reduce_word_m31(h[k]); ok = ok && u[k] < 2u * P; }
        if (ok) break;
    }
    if (root_copy) {
#pragma unroll
        for (int k = 0; k < 8; k++) root_copy[k] = root[k];
    }
#pragma unroll
    for (int k = 0; k < 8; k++) chan[k] = digest[k];
    chan[8] = n_draws;
#pragma unroll
    for (int k = 0; k < 4; k++) alpha_out[k] = u[k] >= P ? u[k] - P : u[k];
}
__global__ void channel_mix_root_draw_kernel(uint32_t* __restrict__ chan, const uint32_t* __restrict__ root,
                                             uint32_t* __restrict__ alpha_out, uint32_t* __restrict__ root_copy) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    channel_mix_root_draw(chan, root, alpha_out, root_copy);
}

// The last (at most ten) layers of a tree in one CTA. Every level is written to its layer array and kept in shared memory
// for the next one (a level read back from global memory costs an L2 round trip on top of the compression; ten levels are a
// chain of ten dependent hashes either way). When `chan` is given, the thread that wrote the root goes on with the channel
// step of a FRI layer (mix the root, draw the folding challenge), which would otherwise be a launch of its own.
// (Spreading a compression of the upper levels over four lanes, one G function each, was tried here and is slower: 35 us per
// tree top against 20: the per-lane message schedule becomes divergent constant-memory reads and the state rotation shuffles
// cost more than the shorter dependency chain saves.)
__global__ void __launch_bounds__(512) merkle_top_kernel(MerkleTopArgs a, int top_log, int m31_out, uint32_t* __restrict__ chan,
                                                         uint32_t* __restrict__ alpha_out, uint32_t* __restrict__ root_copy) {
    __shared__ uint32_t sh[2][512][8];
    for (int lg = top_log - 1; lg >= 0; lg--) {
        const bool from_global = lg == top_log - 1;
        const uint32_t(*src)[8] = sh[(lg + 1) & 1];
        for (uint32_t i = threadIdx.x; i < (1u << lg); i += blockDim.x) {
            uint32_t h[8], m[16];
            blake2s_init(h);
            if (from_global) {
                const uint4* p = reinterpret_cast<const uint4*>(a.layer[lg + 1] + 16 * (size_t)i);
                uint4 x0 = p[0], x1 = p[1], x2 = p[2], x3 = p[3];
                m[0] = x0.x; m[1] = x0.y; m[2] = x0.z; m[3] = x0.w; m[4] = x1.x; m[5] = x1.y; m[6] = x1.z; m[7] = x1.w;
                m[8] = x2.x; m[9] = x2.y; m[10] = x2.z; m[11] = x2.w; m[12] = x3.x; m[13] = x3.y; m[14] = x3.z; m[15] = x3.w;
            } else {
#pragma unroll
                for (int k = 0; k < 8; k++) { m[k] = src[2 * i][k]; m[8 + k] = src[2 * i + 1][k]; }
            }
            blake2s_compress(h, m, 64u, true);
#pragma unroll
            for (int k = 0; k < 8; k++) { h[k] = m31_out ? reduce_word_m31(h[k]) : h[k]; sh[lg & 1][i][k] = h[k]; }
            store_hash(a.layer[lg], i, h, false);
        }
        __syncthreads();
    }
    if (chan && threadIdx.x == 0) channel_mix_root_draw(chan, sh[0][0], alpha_out, root_copy);
}

// Grind: thread `lo` tests nonce (hi << 32) | lo; the minimum passing lo is kept.
__global__ void grind_kernel(uint32_t d0, uint32_t d1, uint32_t d2, uint32_t d3, uint32_t d4, uint32_t d5, uint32_t d6,
                             uint32_t d7, uint32_t hi, int pow_bits, int m31_out, unsigned int* __restrict__ best) {
    uint32_t lo = blockIdx.x * blockDim.x + threadIdx.x;
    uint32_t h[8], m[16] = {d0, d1, d2, d3, d4, d5, d6, d7, lo, hi, 0, 0, 0, 0, 0, 0};
    blake2s_init(h);
    blake2s_compress(h, m, 40u, true);
    uint32_t w = m31_out ? reduce_word_m31(h[0]) : h[0];
    int tz = w ? __ffs(w) - 1 : 32;
    if (tz >= pow_bits) atomicMin(best, lo);
}

}  // namespace zk

using namespace zk;

extern "C" {

int zkb_merkle_layer(zkb_ctx* ctx, int log_size, const uint32_t* prev, const uint32_t* const* cols, int ncols,
                     int m31_out, uint32_t* out) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, log_size >= 0 && log_size <= 30 && ncols >= 0 && out != nullptr);
    ZKB_CHECK_ARG(ctx, ncols == 0 || cols != nullptr);
    ZKB_CHECK_ARG(ctx, ((uintptr_t)out & 15) == 0 && ((uintptr_t)prev & 15) == 0);
    DeviceGuard g(ctx);
    void** d_cols = nullptr;
    if (ncols) {
        int rc = stage_ptrs(ctx, (const void* const*)cols, ncols, &d_cols);
        if (rc) return rc;
    }
    size_t n = (size_t)1 << log_size;
    unsigned threads = n < 256 ? 32 : 256;
    unsigned blocks = (unsigned)((n + threads - 1) / threads);
    if (ncols >= 64 && n <= ((size_t)1 << 17)) {
        // few rows (at 2^17 there are still only seven warps per scheduler), a long chain of compressions each: the next
        // block's loads are in flight during a compression; small CTAs so that the few rows spread over all SMs
        ProfScope prof(ctx, "merkle_layer_prefetch_kernel");
        merkle_layer_prefetch_kernel<<<(unsigned)((n + 31) / 32), 32, 0, ctx->stream>>>(log_size, prev, (const uint32_t* const*)d_cols, ncols, m31_out, out);
        ZKB_LAUNCH_CHECK(ctx);
        return ZKB_OK;
    }
    ProfScope prof(ctx, !ncols ? "merkle_layer_kernel(nodes only)" : (!prev && ncols > 16 ? "merkle_layer_kernel(leaves)" : "merkle_layer_kernel(columns)"));
    merkle_layer_kernel<<<blocks, threads, 0, ctx->stream>>>(log_size, prev, (const uint32_t* const*)d_cols, ncols, m31_out,
                                                             out);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

int zkb_merkle_leaves_partial(zkb_ctx* ctx, int log_size, const uint32_t* const* cols, int ncols, int cols_before, int total_cols,
                              int m31_out, uint32_t* out) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, log_size >= 0 && log_size <= 30 && cols != nullptr && out != nullptr && ((uintptr_t)out & 15) == 0);
    ZKB_CHECK_ARG(ctx, ncols >= 1 && cols_before >= 0 && cols_before % 16 == 0 && cols_before + ncols <= total_cols);
    const bool is_last = cols_before + ncols == total_cols;
    ZKB_CHECK_ARG(ctx, is_last || ncols % 16 == 0);
    DeviceGuard g(ctx);
    void** d_cols = nullptr;
    int rc = stage_ptrs(ctx, (const void* const*)cols, ncols, &d_cols);
    if (rc) return rc;
    size_t n = (size_t)1 << log_size;
    unsigned threads = n < 256 ? 32 : 256;
    ProfScope prof(ctx, "merkle_leaves_partial_kernel");
    merkle_leaves_partial_kernel<<<(unsigned)((n + threads - 1) / threads), threads, 0, ctx->stream>>>(
        log_size, (const uint32_t* const*)d_cols, ncols, (uint32_t)cols_before, is_last ? 1 : 0, m31_out, out);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

int zkb_merkle_levels(zkb_ctx* ctx, int child_log, const uint32_t* children, int levels, uint32_t* const* out_layers, int m31_out) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, children != nullptr && out_layers != nullptr && ((uintptr_t)children & 15) == 0);
    ZKB_CHECK_ARG(ctx, levels >= 1 && levels <= MERKLE_LEVELS_MAX && child_log >= 9 && child_log <= 31 && child_log - levels >= 0);
    MerkleLevelsArgs a{};
    a.children = children;
    for (int j = 1; j <= levels; j++) {
        ZKB_CHECK_ARG(ctx, out_layers[j - 1] != nullptr && ((uintptr_t)out_layers[j - 1] & 15) == 0);
        a.out[j] = out_layers[j - 1];
    }
    DeviceGuard g(ctx);
    ProfScope prof(ctx, "merkle_levels_kernel");
    merkle_levels_kernel<<<1u << (child_log - 9), 256, 0, ctx->stream>>>(a, levels, m31_out);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

static int merkle_top_impl(zkb_ctx* ctx, int top_log, const uint32_t* top_layer, uint32_t* const* lower_layers, int m31_out, uint32_t* d_chan,
                           uint32_t* d_alpha, uint32_t* d_root_copy);
int zkb_merkle_top(zkb_ctx* ctx, int top_log, const uint32_t* top_layer, uint32_t* const* lower_layers, int m31_out) {
    return merkle_top_impl(ctx, top_log, top_layer, lower_layers, m31_out, nullptr, nullptr, nullptr);
}
int zkb_merkle_top_channel(zkb_ctx* ctx, int top_log, const uint32_t* top_layer, uint32_t* const* lower_layers, int m31_out, uint32_t* d_chan,
                           uint32_t* d_alpha, uint32_t* d_root_copy) {
    if (ctx && (!d_chan || !d_alpha || top_log < 1)) return zk::set_error(ctx, ZKB_EINVAL, "zkb_merkle_top_channel: needs a channel, a challenge slot and at least one layer to build");
    return merkle_top_impl(ctx, top_log, top_layer, lower_layers, m31_out, d_chan, d_alpha, d_root_copy);
}
static int merkle_top_impl(zkb_ctx* ctx, int top_log, const uint32_t* top_layer, uint32_t* const* lower_layers, int m31_out, uint32_t* d_chan,
                           uint32_t* d_alpha, uint32_t* d_root_copy) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, top_log >= 0 && top_log <= MERKLE_TOP_MAX_LOG && top_layer != nullptr && ((uintptr_t)top_layer & 15) == 0);
    if (top_log == 0) return ZKB_OK;
    ZKB_CHECK_ARG(ctx, lower_layers != nullptr);
    MerkleTopArgs a;
    a.layer[top_log] = const_cast<uint32_t*>(top_layer);
    for (int k = 0; k < top_log; k++) {
        ZKB_CHECK_ARG(ctx, lower_layers[k] != nullptr && ((uintptr_t)lower_layers[k] & 15) == 0);
        a.layer[k] = lower_layers[k];
    }
    DeviceGuard g(ctx);
    ProfScope prof(ctx, "merkle_top_kernel");
    merkle_top_kernel<<<1, top_log >= 10 ? 512 : (top_log >= 6 ? 1 << (top_log - 1) : 32), 0, ctx->stream>>>(a, top_log, m31_out, d_chan, d_alpha,
                                                                                                              d_root_copy);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

int zkb_channel_mix_root_draw(zkb_ctx* ctx, uint32_t* d_chan, const uint32_t* d_root, uint32_t* d_alpha, uint32_t* d_root_copy) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, d_chan != nullptr && d_root != nullptr && d_alpha != nullptr);
    DeviceGuard g(ctx);
    ProfScope prof(ctx, "channel_mix_root_draw_kernel");
    channel_mix_root_draw_kernel<<<1, 32, 0, ctx->stream>>>(d_chan, d_root, d_alpha, d_root_copy);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

int zkb_grind(zkb_ctx* ctx, const uint32_t h_prefixed_digest[8], int pow_bits, int m31_out, uint64_t* h_nonce) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, h_prefixed_digest != nullptr && h_nonce != nullptr && pow_bits >= 0 && pow_bits <= 32);
    DeviceGuard g(ctx);
    const uint32_t* d = h_prefixed_digest;
    const unsigned LOW = 1u << 20;
    // Bounded search: hi values are tried in order; a miss over 2^20 nonces has probability
    // (1 - 2^-pow_bits)^(2^20), so the bound of 2^12 rounds is never reached for pow_bits <= 32
    // in practice and keeps the loop finite.
    for (uint32_t hi = 0; hi < (1u << 12); hi++) {
        unsigned int init = 0xffffffffu;
        ZKB_CUDA(ctx, cudaMemcpyAsync(ctx->ticket + 8, &init, 4, cudaMemcpyHostToDevice, ctx->stream));
        grind_kernel<<<LOW / 256, 256, 0, ctx->stream>>>(d[0], d[1], d[2], d[3], d[4], d[5], d[6], d[7], hi, pow_bits,
                                                         m31_out, ctx->ticket + 8);
        ZKB_LAUNCH_CHECK(ctx);
        unsigned int best = 0;
        ZKB_CUDA(ctx, cudaMemcpyAsync(&best, ctx->ticket + 8, 4, cudaMemcpyDeviceToHost, ctx->stream));
        ZKB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (best != 0xffffffffu) {
            *h_nonce = ((uint64_t)hi << 32) | best;
            return ZKB_OK;
        }
    }
    return set_error(ctx, ZKB_ETIMEOUT, "zkb_grind: no nonce found in 2^32 attempts");
}

}  // extern "C"
