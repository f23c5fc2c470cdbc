// GKR batches of many instances (the prover's reductions hold hundreds: one instance per component and
// power-of-two share of its lookups, prover/src/gkr_key_tile.rs:34-55). prove_batch
// (nitroo/crates/stwo/src/prover/lookups/gkr_prover.rs:657-882) runs ONE sum-check per layer over all
// instances, so what every instance needs in a round is known together. Here a round of the whole batch is
// one launch and one read-back, whatever the number of instances: a table of work items (one per instance)
// says what to do with which arrays, a flat grid of CTAs is split over the items in proportion to their
// size, and every item's eight result words (and, at the end of a layer, its two-entry mask) land in one
// result array.
//
// A whole layer's sum-check is enqueued at once (gkr_batch_layer): the CTA that completes a round's launch goes on with the
// transcript step (the batch's round polynomial, the channel, the challenge, the claims), the next launch reads the
// challenge from device memory, and the small rounds at the end of a layer run in one single-CTA launch.
//
//   mode 0  sum_as_poly_in_first_variable sums of the item's layer (first round of a layer's sum-check)
//   mode 1  fix_first_variable with the round's challenge on every column, and the sums of the fixed layer
//   mode 2  fix_first_variable of a 4-entry layer; the 2 fixed entries are also copied to the results (the mask)
//   mode 3  next_layer (generation of the towers)
//
// Arithmetic as in gkr.cu / gkr_fused.cu (cpu/lookups/gkr.rs:17-263, cpu/lookups/mle.rs:13-46).
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "blake2s.cuh"
#include "common.cuh"
#include "gkr_batch.hpp"

namespace zk {

namespace {

// (no __restrict__: the kernel of the small rounds reads in one round what it wrote in the round before)
__device__ __forceinline__ qm31 ldqb(const uint32_t* p, size_t i) {
    uint4 v = reinterpret_cast<const uint4*>(p)[i];
    return {{v.x, v.y, v.z, v.w}};
}
__device__ __forceinline__ void stqb(uint32_t* p, size_t i, qm31 v) {
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
__device__ __forceinline__ void item_sums(const GkrBatchItem& it, size_t first, size_t stride, qm31 r, const uint32_t* __restrict__ eq, qm31 lambda,
                                          qm31& s0, qm31& s2) {
    if (it.mode == 0) {
        const size_t nt = it.n / 4;  // entries (0, i, b) at 2i + b, (1, i, b) at 2(nt + i) + b
        for (size_t i = first; i < nt; i += stride) {
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
        for (size_t i = first; i < nt; i += stride) {
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

// ---- the transcript step of a round, for a layer enqueued at once
//
// State of a layer on the device. chan: digest (8 words), n_draws, error. Per oracle: its claim, the correction
// eq(assignment so far, point so far), its record in `res` (sums of the round at [0,8), mask at [8,24)), the round values
// rv (r0, r1, r2 of an active oracle; the constant of a waiting one in rv[0]).
constexpr int GKR_TAIL_THREADS = 512;

struct GkrLayerDev {
    uint32_t* chan;
    uint32_t* challenge;
    const uint32_t* n_vars;
    const uint32_t* alpha_pow;
    uint32_t* claim;
    uint32_t* corr;
    const uint32_t* res;
    uint32_t* rv;
    const GkrRoundConst* rounds;
    uint32_t* out;
    int n_oracles;
};

__device__ __forceinline__ qm31 ldc(const uint32_t* w) { return {{w[0], w[1], w[2], w[3]}}; }

// The transcript step runs once per launch, on instruction memory that the launch has not touched before: what it costs is
// mostly the fetching of its code, so it is written for size. The field multiplication is a call, and the hash is the
// ten-round loop over the message schedule with the block read from shared memory, not the unrolled compression the
// Merkle kernels use (three unrolled compressions in a row took 10 us here on first execution, 32 us in a launch's very
// first pass, 6.2 us when repeated; this loop takes 5.5 us either way. Laying the message schedule out in shared memory
// first, by the lanes of a warp, so that the loop reads it at fixed offsets, took 7.4 us).
__device__ __noinline__ qm31 qmul(qm31 a, qm31 b) { return qm31_mul(a, b); }

__constant__ uint8_t c_sigma_b[10][16] = {
    {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15}, {14, 10, 4, 8, 9, 15, 13, 6, 1, 12, 0, 2, 11, 7, 5, 3},
    {11, 8, 12, 0, 5, 2, 15, 13, 10, 14, 3, 6, 7, 1, 9, 4}, {7, 9, 3, 1, 13, 12, 11, 14, 2, 6, 5, 10, 4, 0, 15, 8},
    {9, 0, 5, 7, 2, 4, 10, 15, 14, 1, 11, 12, 6, 8, 3, 13}, {2, 12, 6, 10, 0, 11, 8, 3, 4, 13, 7, 5, 15, 14, 1, 9},
    {12, 5, 1, 15, 14, 13, 4, 10, 0, 7, 6, 3, 9, 2, 8, 11}, {13, 11, 7, 14, 12, 1, 3, 9, 5, 0, 15, 4, 8, 6, 2, 10},
    {6, 15, 14, 9, 11, 3, 0, 8, 12, 2, 13, 7, 1, 4, 10, 5}, {10, 2, 8, 4, 7, 6, 1, 5, 15, 11, 9, 14, 3, 12, 13, 0}};

#define B2S_GC(a, b, c, d, x, y) \
    do {                         \
        a = a + b + (x);         \
        d = rotr16(d ^ a);       \
        c = c + d;               \
        b = rotr12(b ^ c);       \
        a = a + b + (y);         \
        d = rotr8(d ^ a);        \
        c = c + d;               \
        b = rotr7(b ^ c);        \
    } while (0)

// RFC 7693 section 3.2; m: the 16 message words in shared memory; t: bytes hashed including this block.
__device__ __noinline__ void b2s_compress_small(uint32_t h[8], const uint32_t* m, uint32_t t, bool last) {
    uint32_t v0 = h[0], v1 = h[1], v2 = h[2], v3 = h[3], v4 = h[4], v5 = h[5], v6 = h[6], v7 = h[7];
    uint32_t v8 = B2S_IV0, v9 = B2S_IV1, v10 = B2S_IV2, v11 = B2S_IV3, v12 = B2S_IV4 ^ t, v13 = B2S_IV5, v14 = last ? ~B2S_IV6 : B2S_IV6, v15 = B2S_IV7;
#pragma unroll 1
    for (int r = 0; r < 10; r++) {
        const uint8_t* sg = c_sigma_b[r];
        B2S_GC(v0, v4, v8, v12, m[sg[0]], m[sg[1]]);
        B2S_GC(v1, v5, v9, v13, m[sg[2]], m[sg[3]]);
        B2S_GC(v2, v6, v10, v14, m[sg[4]], m[sg[5]]);
        B2S_GC(v3, v7, v11, v15, m[sg[6]], m[sg[7]]);
        B2S_GC(v0, v5, v10, v15, m[sg[8]], m[sg[9]]);
        B2S_GC(v1, v6, v11, v12, m[sg[10]], m[sg[11]]);
        B2S_GC(v2, v7, v8, v13, m[sg[12]], m[sg[13]]);
        B2S_GC(v3, v4, v9, v14, m[sg[14]], m[sg[15]]);
    }
    h[0] ^= v0 ^ v8; h[1] ^= v1 ^ v9; h[2] ^= v2 ^ v10; h[3] ^= v3 ^ v11;
    h[4] ^= v4 ^ v12; h[5] ^= v5 ^ v13; h[6] ^= v6 ^ v14; h[7] ^= v7 ^ v15;
}

// The channel step of a round by one thread, on a message laid out in shared memory: msg[0,8) the digest, msg[8, 8 + n) the
// words mixed in, zeros up to msg[32). digest <- H(digest || words) with every word reduced (core/channel/blake2s.rs:58-93),
// then draw_secure_felt (:34-52, :95-120): H(digest || n_draws || 0x00), again while a word is >= 2p. Leaves the new digest
// and n_draws in chan[0,9) and returns the challenge. msg is overwritten.
__device__ qm31 chan_mix_draw_1t(uint32_t* msg, int n, uint32_t* chan) {
    uint32_t h[8];
    blake2s_init(h);
    const int total = 8 + n;  // 8 ... 24 words: one or two blocks
    if (total > 16) b2s_compress_small(h, msg, 64u, false);
    b2s_compress_small(h, total > 16 ? msg + 16 : msg, 4u * (uint32_t)total, true);
    for (int k = 0; k < 8; k++) msg[k] = reduce_word_m31(h[k]);
    for (int k = 9; k < 16; k++) msg[k] = 0u;
    uint32_t n_draws = 0, u[8];
    for (int attempt = 0; attempt < 64; attempt++) {  // the words are already below p: one pass in practice
        blake2s_init(h);
        msg[8] = n_draws;
        b2s_compress_small(h, msg, 37u, true);
        n_draws++;
        bool ok = true;
        for (int k = 0; k < 8; k++) { u[k] = reduce_word_m31(h[k]); ok = ok && u[k] < 2u * P; }
        if (ok) break;
    }
    for (int k = 0; k < 8; k++) chan[k] = msg[k];
    chan[8] = n_draws;
    qm31 r;
    for (int k = 0; k < 4; k++) r.c[k] = u[k] >= P ? u[k] - P : u[k];
    return r;
}

// One CTA (256 threads as the tail of a launch, GKR_TAIL_THREADS in the kernel of the small rounds): the one that completes a launch (every other CTA has published its results and counted itself
// before). Restates the host's round (sumcheck.rs:115-171 over the batch): the round values of every oracle, their random
// linear combination in alpha as three sums over the shared basis plus the constants of the waiting oracles, the channel
// step, the claims at the challenge, the corrections. The step is a chain of small dependent pieces, so each piece is spread
// over as many threads as it has independent parts and only the three hash compressions run on one thread.
__device__ void transcript_step(const GkrLayerDev& s, int round) {
    __shared__ uint32_t red[GKR_TAIL_THREADS / 32][16];
    __shared__ uint32_t sh_rc[sizeof(GkrRoundConst) / 4];
    __shared__ uint32_t sh_S[4][4];   // S0, S1, S2 and the constants
    __shared__ uint32_t sh_msg[32];   // digest, the polynomial's words, zeros
    __shared__ uint32_t sh_q[5][4];   // L0(c), L1(c), L2(c), eq(c, y), the challenge
    __shared__ int sh_need_len, sh_len;
    if (threadIdx.x < sizeof(GkrRoundConst) / 4) sh_rc[threadIdx.x] = reinterpret_cast<const uint32_t*>(s.rounds + round)[threadIdx.x];
    if (threadIdx.x >= 64 && threadIdx.x < 72) sh_msg[threadIdx.x - 64] = s.chan[threadIdx.x - 64];
    if (threadIdx.x >= 72 && threadIdx.x < 96) sh_msg[threadIdx.x - 64] = 0u;
    if (threadIdx.x == 0) sh_len = 0;
    __syncthreads();
    const GkrRoundConst& rc = *reinterpret_cast<const GkrRoundConst*>(sh_rc);
    const uint32_t n_rem = rc.n_rem;
    const qm31 e0a = ldc(rc.e0a), e2a = ldc(rc.e2a);
    const uint32_t half = 1u << 30;  // 1 / 2
    const int K = s.n_oracles;
    qm31 S[4] = {qm31_zero(), qm31_zero(), qm31_zero(), qm31_zero()};
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
        const qm31 a = ldqb(s.alpha_pow, k), claim = ldqb(s.claim, k);
        if (n_rem <= s.n_vars[k]) {
            const qm31 corr = ldqb(s.corr, k);
            // the sums were written by other CTAs of this launch: read past the L1
            const uint4* r = reinterpret_cast<const uint4*>(s.res + (size_t)GKR_BATCH_RESULT_WORDS * k);
            const uint4 w0 = __ldcg(r), w2 = __ldcg(r + 1);
            const qm31 r0 = qmul(qmul(qm31{{w0.x, w0.y, w0.z, w0.w}}, corr), e0a);
            const qm31 r2 = qmul(qmul(qm31{{w2.x, w2.y, w2.z, w2.w}}, corr), e2a);
            const qm31 r1 = qm31_sub(claim, r0);
            stqb(s.rv, 3 * (size_t)k, r0);
            stqb(s.rv, 3 * (size_t)k + 1, r1);
            stqb(s.rv, 3 * (size_t)k + 2, r2);
            S[0] = qm31_add(S[0], qmul(a, r0));
            S[1] = qm31_add(S[1], qmul(a, r1));
            S[2] = qm31_add(S[2], qmul(a, r2));
        } else {
            const qm31 c = qm31_mul_m31(claim, half);
            stqb(s.rv, 3 * (size_t)k, c);
            S[3] = qm31_add(S[3], qmul(a, c));
        }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int t = 0; t < 4; t++) {
        S[t] = warp_sumb(S[t]);
        if (lane == 0) {
#pragma unroll
            for (int c = 0; c < 4; c++) red[warp][4 * t + c] = S[t].c[c];
        }
    }
    __syncthreads();
    if (threadIdx.x < 16) {
        uint32_t acc = 0;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) acc = m31_add(acc, red[w][threadIdx.x]);
        sh_S[threadIdx.x >> 2][threadIdx.x & 3] = acc;
    }
    __syncthreads();
    if (threadIdx.x < 4) {  // coefficient t of the combination
        const int t = threadIdx.x;
        qm31 c = qm31_add(qm31_add(qmul(ldc(sh_S[0]), ldc(rc.L[0][t])), qmul(ldc(sh_S[1]), ldc(rc.L[1][t]))), qmul(ldc(sh_S[2]), ldc(rc.L[2][t])));
        if (t == 0) c = qm31_add(c, ldc(sh_S[3]));
        if (t == 3) sh_need_len = qm31_is_zero(c) ? 1 : 0;
#pragma unroll
        for (int w = 0; w < 4; w++) sh_msg[8 + 4 * t + w] = c.c[w];
    }
    __syncthreads();
    if (sh_need_len) {
        // The combination keeps the length of its longest term (each term trimmed, sums not): a vanishing leading
        // coefficient does not say which case this is, so the terms' own lengths decide.
        int mine = 0;
        for (int k = threadIdx.x; k < K; k += blockDim.x) {
            int len = 0;
            if (n_rem <= s.n_vars[k]) {
                const qm31 r0 = ldqb(s.rv, 3 * (size_t)k), r1 = ldqb(s.rv, 3 * (size_t)k + 1), r2 = ldqb(s.rv, 3 * (size_t)k + 2);
                for (int t = 0; t < 4; t++) {
                    const qm31 c = qm31_add(qm31_add(qmul(r0, ldc(rc.L[0][t])), qmul(r1, ldc(rc.L[1][t]))), qmul(r2, ldc(rc.L[2][t])));
                    if (!qm31_is_zero(c)) len = t + 1;
                }
            } else if (!qm31_is_zero(ldqb(s.rv, 3 * (size_t)k))) {
                len = 1;
            }
            mine = max(mine, len);
        }
        atomicMax(&sh_len, mine);
        __syncthreads();
    }
    const int len = sh_need_len ? sh_len : 4;
    uint32_t* o = s.out + GKR_LAYER_OUT_WORDS * (size_t)round;
    if (threadIdx.x >= 32 && threadIdx.x < 48) o[threadIdx.x - 32] = sh_msg[8 + threadIdx.x - 32];  // the record keeps all four
    if (threadIdx.x == 48) o[16] = (uint32_t)len;
    __syncthreads();  // the channel step overwrites the message
    if (threadIdx.x == 0) {
        for (int w = 8 + 4 * len; w < 24; w++) sh_msg[w] = 0u;  // only the first `len` coefficients are mixed
        const qm31 ch = chan_mix_draw_1t(sh_msg, 4 * len, s.chan);
#pragma unroll
        for (int c = 0; c < 4; c++) { o[20 + c] = ch.c[c]; s.challenge[c] = ch.c[c]; sh_q[4][c] = ch.c[c]; }
    }
    __syncthreads();
    if (threadIdx.x < 4) {
        const qm31 ch = ldc(sh_q[4]);
        qm31 v;
        if (threadIdx.x < 3) {
            const int t = threadIdx.x;  // the basis polynomial of node t at the challenge
            v = qm31_add(qmul(qm31_add(qmul(qm31_add(qmul(ldc(rc.L[t][3]), ch), ldc(rc.L[t][2])), ch), ldc(rc.L[t][1])), ch), ldc(rc.L[t][0]));
        } else {
            const qm31 y = ldc(rc.y), one = qm31_one();
            v = qm31_add(qmul(ch, y), qmul(qm31_sub(one, ch), qm31_sub(one, y)));  // eq(challenge, y)
        }
#pragma unroll
        for (int c = 0; c < 4; c++) sh_q[threadIdx.x][c] = v.c[c];
    }
    __syncthreads();
    const qm31 L0 = ldc(sh_q[0]), L1 = ldc(sh_q[1]), L2 = ldc(sh_q[2]), eq_step = ldc(sh_q[3]);
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
        const qm31 r0 = ldqb(s.rv, 3 * (size_t)k);
        if (n_rem <= s.n_vars[k]) {
            const qm31 r1 = ldqb(s.rv, 3 * (size_t)k + 1), r2 = ldqb(s.rv, 3 * (size_t)k + 2);
            stqb(s.claim, k, qm31_add(qm31_add(qmul(r0, L0), qmul(r1, L1)), qmul(r2, L2)));
            if (s.n_vars[k] != 0) stqb(s.corr, k, qmul(ldqb(s.corr, k), eq_step));
        } else {
            stqb(s.claim, k, r0);
        }
    }
}

// The transcript step as the tail of a launch: every other CTA has ended, so the next launch of the layer may be scheduled
// now and run up to its wait while this one CTA finishes the round.
__device__ __forceinline__ void transcript_tail(const GkrLayerDev& s, int round) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    transcript_step(s, round);
}

// The CTA that completes an item reports it. A single round (flag given): when every item of the launch has reported, the
// round's sequence number is written after the results. `results` and `flag` are then page-locked host memory the device
// writes directly, so the host sees a round's results a PCIe write after the last CTA ends, without a copy and a stream
// synchronisation of its own (a round of a small batch is a 5-10 us kernel; the copy and the wake-up cost as much again).
// A layer enqueued at once (no flag): returns, to every thread of the CTA, whether this CTA completed the launch.
__device__ __forceinline__ bool item_done(unsigned int* done, int n_items, volatile unsigned int* flag, unsigned int round_id) {
    __shared__ int completes;
    __syncthreads();
    if (threadIdx.x == 0) {
        if (flag) __threadfence_system(); else __threadfence();
        const bool last = atomicAdd(done, 1u) == (unsigned int)n_items - 1u;
        completes = last && !flag;
        if (last) {
            *done = 0u;  // every item has counted: ready for the next launch
            if (flag) {
                __threadfence_system();
                *flag = round_id;
            } else {
                __threadfence();
            }
        }
    }
    __syncthreads();
    return completes != 0;
}

// d_r: the challenge in device memory (a layer enqueued at once), else `r`. by_slot: an item's results go to the record
// of its oracle (it.slot) instead of the record of its position in the table. tr_round >= 0: the CTA that completes the
// launch goes on with the transcript step of that round of `layer`.
__global__ void __launch_bounds__(256) gkr_batch_round_kernel(const GkrBatchItem* __restrict__ items, int n_items, qm31 r,
                                                              const uint32_t* __restrict__ d_r, int by_slot,
                                                              const uint32_t* __restrict__ eq, qm31 lambda, uint32_t* __restrict__ partials,
                                                              unsigned int* __restrict__ tickets, uint32_t* __restrict__ results,
                                                              unsigned int* __restrict__ done, volatile unsigned int* flag, unsigned int round_id,
                                                              GkrLayerDev layer, int tr_round) {
    const int idx = find_item(items, n_items, blockIdx.x);
    const GkrBatchItem it = items[idx];
    const uint32_t bx = blockIdx.x - it.first_block;
    // A launch of a layer enqueued at once may start while the launch before it is still in its transcript step (programmatic
    // dependent launch): its CTAs get here, with their items looked up, and wait for that grid to end before they touch
    // anything it writes. (No effect on a launch made without the attribute.)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (d_r) r = ldqb(d_r, 0);
    uint32_t* res = results + (size_t)GKR_BATCH_RESULT_WORDS * (by_slot ? (size_t)it.slot : (size_t)idx);
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
        if (item_done(done, n_items, flag, round_id) && tr_round >= 0) transcript_tail(layer, tr_round);
        return;
    }
    qm31 s0 = qm31_zero(), s2 = qm31_zero();
    {
        const size_t first = (size_t)bx * blockDim.x + threadIdx.x, stride = (size_t)it.blocks * blockDim.x;
        switch (it.kind) {
            case ZKB_GKR_GRAND_PRODUCT: item_sums<ZKB_GKR_GRAND_PRODUCT>(it, first, stride, r, eq, lambda, s0, s2); break;
            case ZKB_GKR_LOGUP_GENERIC: item_sums<ZKB_GKR_LOGUP_GENERIC>(it, first, stride, r, eq, lambda, s0, s2); break;
            case ZKB_GKR_LOGUP_MULTIPLICITIES: item_sums<ZKB_GKR_LOGUP_MULTIPLICITIES>(it, first, stride, r, eq, lambda, s0, s2); break;
            default: item_sums<ZKB_GKR_LOGUP_SINGLES>(it, first, stride, r, eq, lambda, s0, s2); break;
        }
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
        if (item_done(done, n_items, flag, round_id) && tr_round >= 0) transcript_tail(layer, tr_round);
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
        if (item_done(done, n_items, flag, round_id) && tr_round >= 0) transcript_tail(layer, tr_round);
    }
}

// The small rounds of a layer in ONE launch. All active oracles of a round have the same number of variables left, so late
// in a layer's sum-check (and in the layers near the outputs throughout) a round is a few thousand entries: a launch per
// round then costs its launch, its first pass through cold instruction memory and its drain, some 30 us for a microsecond
// of work. Here one CTA runs table after table (the fixes of a round and the first sums of the oracles that enter the next,
// then the transcript step, as the launches of gkr_batch_layer do), a barrier between them. An item is worked on by a group of
// `g` lanes (a power of two, 2 ... 32, chosen per table from the items' sizes), so a warp takes 32 / g items at a time.
// tables[t] = (first item, items, g, round of the transcript step + 1 or 0).
__global__ void __launch_bounds__(GKR_TAIL_THREADS) gkr_batch_tail_kernel(const GkrBatchItem* __restrict__ items_base, const uint4* __restrict__ tables,
                                                                          int n_tables, const uint32_t* __restrict__ eq, qm31 lambda, GkrLayerDev layer,
                                                                          uint32_t* __restrict__ results) {
    asm volatile("griddepcontrol.wait;" ::: "memory");  // see gkr_batch_round_kernel
    for (int t = 0; t < n_tables; t++) {
        const uint4 tb = tables[t];
        const GkrBatchItem* items = items_base + tb.x;
        const int n_items = (int)tb.y, g = (int)tb.z, per_pass = GKR_TAIL_THREADS / g;
        const qm31 r = ldqb(layer.challenge, 0);
        const int sub = threadIdx.x % g;
        for (int base = 0; base < n_items; base += per_pass) {
            const int idx = base + threadIdx.x / g;
            const bool live = idx < n_items;
            qm31 s0 = qm31_zero(), s2 = qm31_zero();
            GkrBatchItem it{};
            if (live) {
                it = items[idx];
                uint32_t* res = results + (size_t)GKR_BATCH_RESULT_WORDS * (size_t)it.slot;
                if (it.mode == 2) {
                    if (sub < 2) {
                        qm31 dv = foldb(r, ldqb(it.den, sub), ldqb(it.den, sub + 2));
                        stqb(it.den_out, sub, dv);
                        stqb(res + 8, sub, dv);
                        if (it.kind == ZKB_GKR_LOGUP_GENERIC || it.kind == ZKB_GKR_LOGUP_MULTIPLICITIES) {
                            qm31 nv = it.kind == ZKB_GKR_LOGUP_GENERIC ? foldb(r, ldqb(it.num, sub), ldqb(it.num, sub + 2))
                                                                       : fold_m31(r, it.num[sub], it.num[sub + 2]);
                            stqb(it.num_out, sub, nv);
                            stqb(res + 16, sub, nv);
                        }
                    }
                } else {
                    switch (it.kind) {
                        case ZKB_GKR_GRAND_PRODUCT: item_sums<ZKB_GKR_GRAND_PRODUCT>(it, sub, g, r, eq, lambda, s0, s2); break;
                        case ZKB_GKR_LOGUP_GENERIC: item_sums<ZKB_GKR_LOGUP_GENERIC>(it, sub, g, r, eq, lambda, s0, s2); break;
                        case ZKB_GKR_LOGUP_MULTIPLICITIES: item_sums<ZKB_GKR_LOGUP_MULTIPLICITIES>(it, sub, g, r, eq, lambda, s0, s2); break;
                        default: item_sums<ZKB_GKR_LOGUP_SINGLES>(it, sub, g, r, eq, lambda, s0, s2); break;
                    }
                }
            }
            for (int off = g >> 1; off > 0; off >>= 1) {
                qm31 o0, o2;
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    o0.c[k] = __shfl_down_sync(0xffffffffu, s0.c[k], off, g);
                    o2.c[k] = __shfl_down_sync(0xffffffffu, s2.c[k], off, g);
                }
                s0 = qm31_add(s0, o0);
                s2 = qm31_add(s2, o2);
            }
            if (live && sub == 0 && it.mode != 2) {
                uint32_t* res = results + (size_t)GKR_BATCH_RESULT_WORDS * (size_t)it.slot;
                stqb(res, 0, s0);
                stqb(res, 1, s2);
            }
        }
        __syncthreads();
        if (tb.w) {
            transcript_step(layer, (int)tb.w - 1);
            __syncthreads();
        }
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

// Page-locked words after the per-item results: the sequence number of the last completed round, then what a layer enqueued
// at once brings back beside the per-oracle records (its rounds' records, the channel, the error word).
constexpr size_t H_BATCH_FLAG = GKR_BATCH_RESULT_WORDS * GKR_BATCH_MAX_ITEMS;
constexpr size_t H_BATCH_LAYER_OUT = H_BATCH_FLAG + 4;
constexpr size_t H_BATCH_CHAN = H_BATCH_LAYER_OUT + GKR_LAYER_OUT_WORDS * GKR_LAYER_MAX_ROUNDS;
constexpr size_t H_BATCH_WORDS = H_BATCH_CHAN + 12;

static int batch_buffers(zkb_ctx* ctx) {
    if (ctx->batch_tickets) return ZKB_OK;
    // tickets per item, then the launch's count of completed items
    ZKB_CUDA(ctx, cudaMalloc(&ctx->batch_tickets, (GKR_BATCH_MAX_ITEMS + 1) * sizeof(unsigned int)));
    ZKB_CUDA(ctx, cudaMemsetAsync(ctx->batch_tickets, 0, (GKR_BATCH_MAX_ITEMS + 1) * sizeof(unsigned int), ctx->stream));
    ZKB_CUDA(ctx, cudaMallocHost(&ctx->h_batch, H_BATCH_WORDS * 4));
    ctx->h_batch[H_BATCH_FLAG] = 0;
    ctx->batch_round = 0;
    return ZKB_OK;
}

int gkr_batch_round(zkb_ctx* ctx, GkrBatchItem* items, int n_items, const uint32_t h_r[4], const uint32_t* eq_evals, const uint32_t h_lambda[4],
                    uint32_t* h_results) {
    if (n_items <= 0) return ZKB_OK;
    if ((size_t)n_items > GKR_BATCH_MAX_ITEMS) return set_error(ctx, ZKB_EINVAL, "gkr batch: more than %d instances", (int)GKR_BATCH_MAX_ITEMS);
    DeviceGuard g(ctx);
    uint32_t total = plan_blocks(items, n_items, 0);
    if (int rc = batch_buffers(ctx)) return rc;
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
    volatile unsigned int* flag = reinterpret_cast<volatile unsigned int*>(ctx->h_batch + H_BATCH_FLAG);
    const unsigned int round_id = ++ctx->batch_round;
    qm31 r{{h_r[0], h_r[1], h_r[2], h_r[3]}}, lam{{h_lambda[0], h_lambda[1], h_lambda[2], h_lambda[3]}};
    {
        ProfScope prof(ctx, "gkr_batch_round_kernel");
        gkr_batch_round_kernel<<<total, 256, 0, ctx->stream>>>(d_items, n_items, r, nullptr, 0, eq_evals, lam, partials, tickets, results,
                                                               ctx->batch_tickets + GKR_BATCH_MAX_ITEMS, flag, round_id, GkrLayerDev{}, -1);
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

int gkr_batch_layer(zkb_ctx* ctx, int n_oracles, const uint32_t* n_vars, const uint32_t* alpha_pow, const uint32_t* claims,
                    GkrLayerRound* rounds, int n_rounds, const uint32_t* eq_evals, const uint32_t h_lambda[4], uint32_t chan[9],
                    uint32_t* h_out, uint32_t* h_res) {
    if (n_oracles <= 0 || n_rounds <= 0) return ZKB_OK;
    if ((size_t)n_oracles > GKR_BATCH_MAX_ITEMS) return set_error(ctx, ZKB_EINVAL, "gkr batch: more than %d instances", (int)GKR_BATCH_MAX_ITEMS);
    if (n_rounds > GKR_LAYER_MAX_ROUNDS) return set_error(ctx, ZKB_EINVAL, "gkr batch: %d rounds in a layer", n_rounds);
    DeviceGuard g(ctx);
    if (int rc = batch_buffers(ctx)) return rc;
    const size_t K = (size_t)n_oracles, Kp = (K + 3) & ~(size_t)3;
    // The staged block (every part a multiple of four words): channel and error word, challenge, variables per oracle,
    // powers of alpha, claims, corrections (one), the rounds' constants, the rounds' item tables.
    const size_t o_chan = 0, o_challenge = 12, o_nvars = 16, o_alpha = o_nvars + Kp, o_claim = o_alpha + 4 * K, o_corr = o_claim + 4 * K,
                 o_rounds = o_corr + 4 * K, o_items = o_rounds + (sizeof(GkrRoundConst) / 4) * (size_t)n_rounds;
    // Launch j (0 <= j <= n_rounds) carries the fixes of round j - 1 (challenge of that round) and the first sums of the oracles
    // that enter in round j, and its completing CTA runs the transcript step of round j: one launch per round and one more.
    std::vector<std::vector<GkrBatchItem>> tables((size_t)n_rounds + 1);
    std::vector<uint32_t> totals((size_t)n_rounds + 1, 0u);
    size_t n_items = 0;
    uint32_t max_blocks = 0;
    for (int j = 0; j <= n_rounds; j++) {
        std::vector<GkrBatchItem>& t = tables[j];
        if (j > 0) t.insert(t.end(), rounds[j - 1].fix, rounds[j - 1].fix + rounds[j - 1].n_fix);
        if (j < n_rounds) t.insert(t.end(), rounds[j].first, rounds[j].first + rounds[j].n_first);
        if (t.empty()) {
            if (j < n_rounds) return set_error(ctx, ZKB_EINVAL, "gkr batch: round %d of the layer has no work", j);
            continue;
        }
        totals[j] = plan_blocks(t.data(), (int)t.size(), 0);
        max_blocks = std::max(max_blocks, totals[j]);
        n_items += t.size();
    }
    if ((size_t)(GKR_BATCH_RESULT_WORDS + 1) * GKR_BATCH_MAX_ITEMS + 8 * (size_t)max_blocks > ctx->scratch_words)
        return set_error(ctx, ZKB_EINVAL, "gkr batch: %u CTAs exceed the scratch buffer", max_blocks);
    // The small rounds at the end of the layer go to one single-CTA launch: from the first table on after which every table
    // is at most GKR_TAIL_MAX_UNITS units of work (a unit = what one thread does in a pass: eight entries of a fix): one unit
    // per thread of the CTA. Measured: a round of 128 units takes 4.5 us there, of 512 units 13 us, of 4096 units 120 us, against
    // some 25 us for a launch of its own.
    constexpr size_t GKR_TAIL_MAX_UNITS = 512;
    std::vector<uint32_t> group((size_t)n_rounds + 1, 2u);
    int j_tail = n_rounds + 1;
    for (int j = n_rounds; j >= 0; j--) {
        size_t units = 0, widest = 1;
        for (const GkrBatchItem& it : tables[j]) {
            const size_t u = it.mode == 0 ? it.n / 4 : it.mode == 1 ? it.n / 8 : 2;
            units += u;
            widest = std::max(widest, u);
        }
        if (units > GKR_TAIL_MAX_UNITS) break;
        uint32_t gsz = 2;
        while (gsz < 32 && gsz < widest) gsz *= 2;
        group[j] = gsz;
        j_tail = j;
    }
    if (const char* e = getenv("ZKB_GKR_ROUNDS"))
        if (!strcmp(e, "launches")) j_tail = n_rounds + 1;
    const size_t n_tail_tables = (size_t)(n_rounds + 1 - j_tail);
    const size_t o_tables = o_items + (sizeof(GkrBatchItem) / 4) * n_items;
    std::vector<uint32_t> blob(o_tables + 4 * n_tail_tables, 0u);
    memcpy(&blob[o_chan], chan, 9 * 4);
    memcpy(&blob[o_nvars], n_vars, K * 4);
    memcpy(&blob[o_alpha], alpha_pow, 4 * K * 4);
    memcpy(&blob[o_claim], claims, 4 * K * 4);
    for (size_t k = 0; k < K; k++) blob[o_corr + 4 * k] = 1u;
    for (int r = 0; r < n_rounds; r++) memcpy(&blob[o_rounds + (sizeof(GkrRoundConst) / 4) * (size_t)r], &rounds[r].rc, sizeof(GkrRoundConst));
    std::vector<size_t> table_at((size_t)n_rounds + 1);
    size_t at = o_items;
    for (int j = 0; j <= n_rounds; j++) {
        table_at[j] = at;
        if (!tables[j].empty()) memcpy(&blob[at], tables[j].data(), sizeof(GkrBatchItem) * tables[j].size());
        at += (sizeof(GkrBatchItem) / 4) * tables[j].size();
    }
    for (int j = j_tail; j <= n_rounds; j++) {
        uint32_t* tb = &blob[o_tables + 4 * (size_t)(j - j_tail)];
        tb[0] = (uint32_t)((table_at[j] - o_items) / (sizeof(GkrBatchItem) / 4));
        tb[1] = (uint32_t)tables[j].size();
        tb[2] = group[j];
        tb[3] = j < n_rounds ? (uint32_t)j + 1u : 0u;
    }
    void* d_blob_v = nullptr;
    if (int rc = stage_blob(ctx, blob.data(), blob.size() * 4, &d_blob_v)) return rc;
    uint32_t* d_blob = static_cast<uint32_t*>(d_blob_v);
    // device-only: the round values of every oracle, the rounds' records
    void* d_work_v = nullptr;
    const size_t work_words = 12 * K + GKR_LAYER_OUT_WORDS * (size_t)n_rounds;
    if (int rc = zkb_malloc(ctx, work_words * 4, &d_work_v)) return rc;
    uint32_t* d_work = static_cast<uint32_t*>(d_work_v);
    GkrLayerDev s{};
    s.chan = d_blob + o_chan;
    s.challenge = d_blob + o_challenge;
    s.n_vars = d_blob + o_nvars;
    s.alpha_pow = d_blob + o_alpha;
    s.claim = d_blob + o_claim;
    s.corr = d_blob + o_corr;
    s.res = ctx->scratch;  // one record per oracle; the partial sums of the launches follow
    s.rv = d_work;
    s.rounds = reinterpret_cast<const GkrRoundConst*>(d_blob + o_rounds);
    s.out = d_work + 12 * K;
    s.n_oracles = n_oracles;
    uint32_t* partials = ctx->scratch + (size_t)(GKR_BATCH_RESULT_WORDS + 1) * GKR_BATCH_MAX_ITEMS;
    const qm31 zero = qm31_zero(), lam{{h_lambda[0], h_lambda[1], h_lambda[2], h_lambda[3]}};
    cudaError_t e = cudaSuccess;
    // Each launch but the first is a programmatic dependent of the one before it (ZKB_GKR_PDL=0: plain stream order).
    const char* pdl_env = getenv("ZKB_GKR_PDL");
    const bool pdl = !(pdl_env && pdl_env[0] == '0') && !ctx->prof_on;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.dynamicSmemBytes = 0;
    cfg.stream = ctx->stream;
    cfg.attrs = attr;
    bool launched = false;
    for (int j = 0; j < j_tail && j <= n_rounds && e == cudaSuccess; j++) {
        if (tables[j].empty()) continue;
        ProfScope prof(ctx, totals[j] <= 8 ? "gkr_batch_round_kernel(<=8 CTAs)" : totals[j] <= 128 ? "gkr_batch_round_kernel(<=128 CTAs)"
                                 : totals[j] <= 2048 ? "gkr_batch_round_kernel(<=2048 CTAs)" : "gkr_batch_round_kernel(>2048 CTAs)");
        cfg.gridDim = dim3(totals[j]);
        cfg.blockDim = dim3(256);
        cfg.numAttrs = pdl && launched ? 1 : 0;  // the first launch follows a copy, not a kernel of this chain
        e = cudaLaunchKernelEx(&cfg, gkr_batch_round_kernel, reinterpret_cast<const GkrBatchItem*>(d_blob + table_at[j]), (int)tables[j].size(), zero,
                               (const uint32_t*)s.challenge, 1, eq_evals, lam, partials, ctx->batch_tickets, ctx->scratch,
                               ctx->batch_tickets + GKR_BATCH_MAX_ITEMS, (volatile unsigned int*)nullptr, 0u, s, j < n_rounds ? j : -1);
        launched = true;
    }
    if (n_tail_tables && e == cudaSuccess) {
        ProfScope prof(ctx, "gkr_batch_tail_kernel");
        cfg.gridDim = dim3(1);
        cfg.blockDim = dim3(GKR_TAIL_THREADS);
        cfg.numAttrs = pdl && launched ? 1 : 0;
        e = cudaLaunchKernelEx(&cfg, gkr_batch_tail_kernel, reinterpret_cast<const GkrBatchItem*>(d_blob + o_items),
                               reinterpret_cast<const uint4*>(d_blob + o_tables), (int)n_tail_tables, eq_evals, lam, s, ctx->scratch);
    }
    uint32_t* h = ctx->h_batch;
    if (e == cudaSuccess) e = cudaMemcpyAsync(h, ctx->scratch, K * GKR_BATCH_RESULT_WORDS * 4, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(h + H_BATCH_LAYER_OUT, s.out, GKR_LAYER_OUT_WORDS * (size_t)n_rounds * 4, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(h + H_BATCH_CHAN, s.chan, 12 * 4, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    zkb_free(ctx, d_work_v);
    if (e != cudaSuccess) {
        cudaMemsetAsync(ctx->batch_tickets, 0, (GKR_BATCH_MAX_ITEMS + 1) * sizeof(unsigned int), ctx->stream);
        return set_error(ctx, ZKB_ECUDA, "gkr batch layer: %s", cudaGetErrorString(e));
    }
    memcpy(h_res, h, K * GKR_BATCH_RESULT_WORDS * 4);
    memcpy(h_out, h + H_BATCH_LAYER_OUT, GKR_LAYER_OUT_WORDS * (size_t)n_rounds * 4);
    memcpy(chan, h + H_BATCH_CHAN, 9 * 4);
    return ZKB_OK;
}

}  // namespace zk
