// GKR prove_batch with the Fiat-Shamir transcript resident on the device.
//
// The reference's prover (nitroo/crates/stwo/src/prover/lookups/gkr_prover.rs:657-882 with
// sumcheck.rs:96-176) returns to the host channel after every sum-check round: 276 round trips for one
// instance of 2^24 fractions, each a launch, a 32-byte copy and a synchronisation. Which kernels run, on
// which sizes, in which order depends only on the instances' sizes, never on the transcript. So the host
// enqueues the whole proof without waiting: small single-thread kernels keep the channel, the claims and the
// round polynomials in device memory (layer_begin, round_step, layer_end below restate the host code of
// prover.cpp line for line), and the data-parallel kernels read their challenges from that state. One copy
// brings the proof back.
#include <vector>

#include "blake2s.cuh"
#include "common.cuh"
#include "gkr_internal.cuh"
#include "gkr_resident.hpp"
#include "host/b200_backend.hpp"

namespace zk {

constexpr int RES_MAX_INST = 16;
constexpr int RES_MAX_VARS = 32;
constexpr int RES_MAX_ROUNDS = RES_MAX_VARS * (RES_MAX_VARS + 1) / 2;

struct Poly4 { qm31 c[4]; int n; };

struct ResState {
    uint32_t digest[8];
    uint32_t n_draws, error, ood_len, pad;
    qm31 alpha, lambda, challenge, eq_v;
    qm31 ood[RES_MAX_VARS + 1];
    qm31 ood_prefix[RES_MAX_VARS + 2];  // ood_prefix[j] = prod_{i < j} (1 - ood[i])
    qm31 assignment[RES_MAX_VARS + 1];
    qm31 claims[RES_MAX_INST][2];
    uint32_t n_claims[RES_MAX_INST];
    qm31 sc_claim[RES_MAX_INST];
    qm31 eq_corr[RES_MAX_INST];
    uint32_t sums[RES_MAX_INST][8];
    // proof pieces
    qm31 output_claims[RES_MAX_INST][2];
    uint32_t n_output_claims[RES_MAX_INST];
    Poly4 round_polys[RES_MAX_ROUNDS];
    qm31 masks[RES_MAX_VARS][RES_MAX_INST][4];  // [layer][oracle][column 0: (v0, v1), column 1: (v0, v1)]
};

// ---- channel (core/channel/blake2s.rs:58-120 with the M31 reduction of every digest word)
// The transcript steps are executed by one whole warp. Scalar work is done redundantly by every lane (free
// under SIMT); the Blake2s compression is spread over four lanes, one column / diagonal G function each
// (RFC 7693 section 3.2), which shortens its dependency chain fourfold. The message block sits in shared
// memory so that a lane can pick the two words its G function needs in a round.
__constant__ uint8_t c_sigma[10][16] = {
    {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15}, {14, 10, 4, 8, 9, 15, 13, 6, 1, 12, 0, 2, 11, 7, 5, 3},
    {11, 8, 12, 0, 5, 2, 15, 13, 10, 14, 3, 6, 7, 1, 9, 4}, {7, 9, 3, 1, 13, 12, 11, 14, 2, 6, 5, 10, 4, 0, 15, 8},
    {9, 0, 5, 7, 2, 4, 10, 15, 14, 1, 11, 12, 6, 8, 3, 13}, {2, 12, 6, 10, 0, 11, 8, 3, 4, 13, 7, 5, 15, 14, 1, 9},
    {12, 5, 1, 15, 14, 13, 4, 10, 0, 7, 6, 3, 9, 2, 8, 11}, {13, 11, 7, 14, 12, 1, 3, 9, 5, 0, 15, 4, 8, 6, 2, 10},
    {6, 15, 14, 9, 11, 3, 0, 8, 12, 2, 13, 7, 1, 4, 10, 5}, {10, 2, 8, 4, 7, 6, 1, 5, 15, 11, 9, 14, 3, 12, 13, 0}};

struct Chan { uint32_t digest[8]; uint32_t n_draws; };

// Warp-collective. h: chaining value (same in every lane); m: 16 message words in shared memory.
__device__ void b2s_compress_warp(uint32_t h[8], const uint32_t* m, uint32_t t, bool last) {
    const int l = threadIdx.x & 3;
    const uint32_t iv[8] = {B2S_IV0, B2S_IV1, B2S_IV2, B2S_IV3, B2S_IV4, B2S_IV5, B2S_IV6, B2S_IV7};
    uint32_t a = h[l], b = h[4 + l], c = iv[l], d = iv[4 + l];
    if (l == 0) d ^= t;
    if (l == 2 && last) d = ~d;
    for (int r = 0; r < 10; r++) {
        uint32_t x = m[c_sigma[r][2 * l]], y = m[c_sigma[r][2 * l + 1]];
        B2S_G(a, b, c, d, x, y);
        b = __shfl_sync(0xffffffffu, b, (l + 1) & 3, 4);
        c = __shfl_sync(0xffffffffu, c, (l + 2) & 3, 4);
        d = __shfl_sync(0xffffffffu, d, (l + 3) & 3, 4);
        x = m[c_sigma[r][8 + 2 * l]];
        y = m[c_sigma[r][8 + 2 * l + 1]];
        B2S_G(a, b, c, d, x, y);
        b = __shfl_sync(0xffffffffu, b, (l + 3) & 3, 4);
        c = __shfl_sync(0xffffffffu, c, (l + 2) & 3, 4);
        d = __shfl_sync(0xffffffffu, d, (l + 1) & 3, 4);
    }
    const uint32_t lo = a ^ c, hi = b ^ d;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        h[i] ^= __shfl_sync(0xffffffffu, lo, i, 4);
        h[4 + i] ^= __shfl_sync(0xffffffffu, hi, i, 4);
    }
}

__shared__ uint32_t s_block[16];  // the message block of the compression in flight (one transcript warp per CTA)

// Warp-collective: digest <- H(digest || w[0..n)), every word reduced mod p.
__device__ void chan_mix_words(Chan& ch, const uint32_t* w, int n) {
    const int lane = threadIdx.x & 31;
    uint32_t h[8];
    blake2s_init(h);
    const int total = 8 + n;
    uint32_t t = 0;
    int pos = 0;
    for (;;) {
        const int rem = total - pos;
        const bool last = rem <= 16;
        __syncwarp();
        if (lane < 16) {
            const int i = pos + lane;
            s_block[lane] = lane < rem ? (i < 8 ? ch.digest[i & 7] : w[i - 8]) : 0u;
        }
        __syncwarp();
        t += last ? 4u * (uint32_t)rem : 64u;
        b2s_compress_warp(h, s_block, t, last);
        if (last) break;
        pos += 16;
    }
    for (int k = 0; k < 8; k++) ch.digest[k] = reduce_word_m31(h[k]);
    ch.n_draws = 0;
}
__device__ void chan_mix_felts(Chan& ch, const qm31* f, int n) { chan_mix_words(ch, (const uint32_t*)f, 4 * n); }
__device__ qm31 chan_draw_felt(Chan& ch) {
    const int lane = threadIdx.x & 31;
    uint32_t u[8];
    for (int attempt = 0; attempt < 64; attempt++) {
        uint32_t h[8];
        blake2s_init(h);
        __syncwarp();
        if (lane < 16) s_block[lane] = lane < 8 ? ch.digest[lane] : (lane == 8 ? ch.n_draws : 0u);
        __syncwarp();
        b2s_compress_warp(h, s_block, 37u, true);
        ch.n_draws++;
        bool ok = true;
        for (int k = 0; k < 8; k++) { u[k] = reduce_word_m31(h[k]); ok = ok && u[k] < 2u * P; }
        if (ok) break;
    }
    qm31 r;
    for (int k = 0; k < 4; k++) r.c[k] = u[k] >= P ? u[k] - P : u[k];
    return r;
}
__device__ Chan chan_load(const ResState* st) {
    Chan ch;
    for (int k = 0; k < 8; k++) ch.digest[k] = st->digest[k];
    ch.n_draws = st->n_draws;
    return ch;
}
__device__ void chan_store(ResState* st, const Chan& ch) {
    for (int k = 0; k < 8; k++) st->digest[k] = ch.digest[k];
    st->n_draws = ch.n_draws;
}

// ---- univariate polynomials of degree <= 3 (lookups/utils.rs:26-54, 165-170)
__device__ void p_trim(Poly4& p) { while (p.n > 0 && qm31_is_zero(p.c[p.n - 1])) p.n--; }
__device__ qm31 p_eval(const Poly4& p, qm31 x) {
    qm31 acc = qm31_zero();
    for (int i = p.n; i-- > 0;) acc = qm31_add(qm31_mul(acc, x), p.c[i]);
    return acc;
}
__device__ Poly4 p_add(const Poly4& a, const Poly4& b) {
    Poly4 r;
    r.n = a.n > b.n ? a.n : b.n;
    for (int i = 0; i < 4; i++) r.c[i] = qm31_add(i < a.n ? a.c[i] : qm31_zero(), i < b.n ? b.c[i] : qm31_zero());
    return r;
}
__device__ qm31 eq1(qm31 x, qm31 y) {
    return qm31_add(qm31_mul(x, y), qm31_mul(qm31_sub(qm31_one(), x), qm31_sub(qm31_one(), y)));
}
// gkr_prover.rs:884-923: the degree-3 polynomial through (0, r0), (1, r1), (2, r2), (b, 0) with
// b = (1 - y) / (1 - 2y), by Lagrange interpolation (lookups/utils.rs:26-54). Field inverses are unique, so
// the five inversions the formula needs (of prod_i eq(0, y_i), 1 - 2y, and of b, 1 - b, 2 - b, which are
// (1 - y), -y, (1 - 3y) over (1 - 2y)) are taken with ONE inversion of their product (Montgomery's trick);
// the fourth Lagrange term has value 0 and vanishes, exactly as its trimmed polynomial does on the host.
// Warp-collective helpers: lane l computes its own product (or inverse), then every lane reads the results it
// needs. The independent multiplications of a level run side by side instead of one after the other.
__device__ __forceinline__ qm31 bcast(qm31 v, int src) {
    qm31 r;
#pragma unroll
    for (int c = 0; c < 4; c++) r.c[c] = __shfl_sync(0xffffffffu, v.c[c], src);
    return r;
}
template <int N>
__device__ __forceinline__ void par_mul(const qm31 (&x)[N], const qm31 (&y)[N], qm31 (&out)[N]) {
    const int lane = threadIdx.x & 31;
    qm31 mx = x[0], my = y[0];
#pragma unroll
    for (int i = 1; i < N; i++)
        if (lane == i) { mx = x[i]; my = y[i]; }
    const qm31 p = qm31_mul(mx, my);
#pragma unroll
    for (int i = 0; i < N; i++) out[i] = bcast(p, i);
}
__device__ Poly4 correct_sum(qm31 f0, qm31 f2, qm31 claim, const qm31* y, const qm31* one_minus_y_prefix, int n, int k) {
    const int lane = threadIdx.x & 31;
    // a = prod_{i < n-k+1} eq(0, y_i) = prod (1 - y_i): kept as prefix products by layer_end
    const qm31 a = one_minus_y_prefix[n - k + 1];
    const qm31 one = qm31_one(), yk = y[n - k];
    const qm31 d = qm31_sub(one, qm31_dbl(yk));                       // 1 - 2y
    const qm31 omy = qm31_sub(one, yk);                                // 1 - y = eq(0, y)
    const qm31 m3y = qm31_sub(omy, qm31_dbl(yk));                      // 1 - 3y = -eq(2, y)
    // level 1: the five inversions (of a, 1-2y, 1-y, y, 1-3y), one per lane
    qm31 mine = a;
    if (lane == 1) mine = d;
    if (lane == 2) mine = omy;
    if (lane == 3) mine = yk;
    if (lane == 4) mine = m3y;
    const qm31 minv = qm31_inv(mine);
    const qm31 a_inv = bcast(minv, 0), d_inv = bcast(minv, 1), omy_inv = bcast(minv, 2), y_inv = bcast(minv, 3), m3y_inv = bcast(minv, 4);
    // level 2
    qm31 l2[6];
    {
        const qm31 x[6] = {omy, d, d, d, f0, f2}, z[6] = {d_inv, omy_inv, y_inv, m3y_inv, omy, qm31_neg(m3y)};
        par_mul<6>(x, z, l2);
    }
    const qm31 b = l2[0], inv_b = l2[1], inv_1mb = qm31_neg(l2[2]), inv_2mb = l2[3];   // b, 1/b, 1/(1-b), 1/(2-b)
    // level 3: r0 = f0 eq(0, y) / a, r2 = f2 eq(2, y) / a
    qm31 l3[2];
    {
        const qm31 x[2] = {l2[4], l2[5]}, z[2] = {a_inv, a_inv};
        par_mul<2>(x, z, l3);
    }
    const qm31 r0 = l3[0], r2 = l3[1], r1 = qm31_sub(claim, r0);
    // level 4: Lagrange weights p_i = ys[i] * prod_{j != i} 1 / (xs[i] - xs[j]) over xs = {0, 1, 2, b}; ys[3] = 0
    const uint32_t half = 1u << 30;  // 1 / 2
    qm31 l4[3];
    {
        const qm31 x[3] = {qm31_mul_m31(r0, half), r1, qm31_mul_m31(r2, half)}, z[3] = {inv_b, inv_1mb, inv_2mb};
        par_mul<3>(x, z, l4);
    }
    const qm31 p0 = qm31_neg(l4[0]), p1 = qm31_neg(l4[1]), p2 = l4[2];
    // level 5: sum_i p_i prod_{j != i} (t - xs[j]), expanded:
    //   (t-1)(t-2)(t-b) = t^3 - (3+b) t^2 + (2+3b) t - 2b;  t(t-2)(t-b) = t^3 - (2+b) t^2 + 2b t;  t(t-1)(t-b) = t^3 - (1+b) t^2 + b t
    const qm31 b2 = qm31_dbl(b), b3 = qm31_add(b2, b);
    qm31 l5[7];
    {
        const qm31 x[7] = {qm31_add(qm31_from_m31(3), b), qm31_add(qm31_from_m31(2), b), qm31_add(one, b), qm31_add(qm31_from_m31(2), b3), b2, b, b2};
        const qm31 z[7] = {p0, p1, p2, p0, p1, p2, p0};
        par_mul<7>(x, z, l5);
    }
    Poly4 c;
    c.n = 4;
    c.c[3] = qm31_add(qm31_add(p0, p1), p2);
    c.c[2] = qm31_neg(qm31_add(qm31_add(l5[0], l5[1]), l5[2]));
    c.c[1] = qm31_add(qm31_add(l5[3], l5[4]), l5[5]);
    c.c[0] = qm31_neg(l5[6]);
    p_trim(c);
    return c;
}

// ---- the three transcript steps
struct BeginArgs {
    int n_inst, n_oracles, nv;
    int activate[RES_MAX_INST], active[RES_MAX_INST], kind[RES_MAX_INST];
    const uint32_t* out_num[RES_MAX_INST];  // output layer (one entry per column)
    const uint32_t* out_den[RES_MAX_INST];
    int oracle_inst[RES_MAX_INST], oracle_nvars[RES_MAX_INST];
};
// Every lane of the warp runs the step and writes the same values; see the channel above.
__global__ void res_layer_begin_kernel(ResState* st, BeginArgs a) {
    if (threadIdx.x >= 32 || blockIdx.x != 0) return;
    Chan ch = chan_load(st);
    for (int i = 0; i < a.n_inst; i++)
        if (a.activate[i]) {
            const uint32_t* d = a.out_den[i];
            qm31 den0{{d[0], d[1], d[2], d[3]}};
            int n = 2;
            if (a.kind[i] == ZKB_GKR_GRAND_PRODUCT) { st->claims[i][0] = den0; n = 1; }
            else if (a.kind[i] == ZKB_GKR_LOGUP_GENERIC) { const uint32_t* q = a.out_num[i]; st->claims[i][0] = qm31{{q[0], q[1], q[2], q[3]}}; st->claims[i][1] = den0; }
            else if (a.kind[i] == ZKB_GKR_LOGUP_MULTIPLICITIES) { st->claims[i][0] = qm31_from_m31(a.out_num[i][0]); st->claims[i][1] = den0; }
            else { st->claims[i][0] = qm31_one(); st->claims[i][1] = den0; }
            st->n_claims[i] = n;
            for (int k = 0; k < n; k++) st->output_claims[i][k] = st->claims[i][k];
            st->n_output_claims[i] = n;
        }
    __syncwarp();
    for (int i = 0; i < a.n_inst; i++)
        if (a.active[i]) chan_mix_felts(ch, st->claims[i], (int)st->n_claims[i]);
    st->eq_v = st->ood_len == 0 ? qm31_one() : eq1(qm31_zero(), st->ood[0]);
    const qm31 alpha = chan_draw_felt(ch), lambda = chan_draw_felt(ch);
    st->alpha = alpha;
    st->lambda = lambda;
    chan_store(st, ch);
    for (int k = 0; k < a.n_oracles; k++) {
        int i = a.oracle_inst[k];
        qm31 acc = qm31_zero();
        for (int j = (int)st->n_claims[i]; j-- > 0;) acc = qm31_add(qm31_mul(acc, lambda), st->claims[i][j]);
        st->sc_claim[k] = qm31_mul_m31(acc, 1u << (a.nv - a.oracle_nvars[k]));
        st->eq_corr[k] = qm31_one();
    }
}

struct RoundArgs {
    int n_oracles, n_rem, round, poly_slot;
    int nvars[RES_MAX_INST];
};
// Warp-collective.
__device__ void round_step(ResState* st, const RoundArgs& a) {
    Chan ch = chan_load(st);
    const qm31 alpha = st->alpha;
    Poly4 rp[RES_MAX_INST];
    const uint32_t half = m31_inv(2);
    for (int k = 0; k < a.n_oracles; k++) {
        if (a.n_rem == a.nvars[k]) {
            const uint32_t* s = st->sums[k];
            qm31 s0 = qm31_mul(qm31{{s[0], s[1], s[2], s[3]}}, st->eq_corr[k]);
            qm31 s2 = qm31_mul(qm31{{s[4], s[5], s[6], s[7]}}, st->eq_corr[k]);
            rp[k] = correct_sum(s0, s2, st->sc_claim[k], st->ood, st->ood_prefix, (int)st->ood_len, a.nvars[k]);
        } else {
            rp[k].n = 1;
            rp[k].c[0] = qm31_mul_m31(st->sc_claim[k], half);
            for (int j = 1; j < 4; j++) rp[k].c[j] = qm31_zero();
            p_trim(rp[k]);
        }
        qm31 e = rp[k].n ? rp[k].c[0] : qm31_zero();  // r(0) + r(1) = c0 + (c0 + c1 + c2 + c3)
        for (int j = 0; j < rp[k].n; j++) e = qm31_add(e, rp[k].c[j]);
        if (!qm31_eq(e, st->sc_claim[k])) st->error = 1u;  // the round polynomial does not match the claim
    }
    Poly4 combined;
    combined.n = 0;
    for (int j = 0; j < 4; j++) combined.c[j] = qm31_zero();
    for (int k = a.n_oracles; k-- > 0;) {
        for (int j = 0; j < combined.n; j++) combined.c[j] = qm31_mul(combined.c[j], alpha);
        combined = p_add(combined, rp[k]);
    }
    chan_mix_felts(ch, combined.c, combined.n);
    qm31 challenge = chan_draw_felt(ch);
    chan_store(st, ch);
    for (int k = 0; k < a.n_oracles; k++) st->sc_claim[k] = p_eval(rp[k], challenge);
    for (int k = 0; k < a.n_oracles; k++)
        if (a.n_rem == a.nvars[k] && a.nvars[k] != 0) {
            const qm31 z0 = st->ood[st->ood_len - a.nvars[k]], old = st->eq_corr[k];
            const qm31 upd = qm31_mul(old, eq1(challenge, z0));
            __syncwarp();  // every lane has read the old value before any lane replaces it
            st->eq_corr[k] = upd;
        }
    st->round_polys[a.poly_slot] = combined;
    st->assignment[a.round] = challenge;
    st->challenge = challenge;
}
__global__ void res_round_kernel(ResState* st, RoundArgs a) {
    if (threadIdx.x >= 32 || blockIdx.x != 0) return;
    round_step(st, a);
}

// The last rounds of a layer's sum-check in ONE launch: once every live oracle has at most 2^14 entries, a
// single CTA runs round after round (sums over the layer, the transcript step on thread 0, fix_first_variable),
// so a round costs its own latency and no launch. The first fold goes from the oracle's layer into work buffers
// (the layer may be the caller's input, which is never modified), later folds are in place there.
constexpr int TAIL_MAX_LOG = 14;
constexpr int TAIL_THREADS = 512;
struct TailArgs {
    int n_oracles, nv, round_start, first_poly_slot;
    int kind[RES_MAX_INST], nvars[RES_MAX_INST];
    const uint32_t* num[RES_MAX_INST];
    const uint32_t* den[RES_MAX_INST];
    uint32_t* num_w[RES_MAX_INST];  // n/2 QM31 each (unused for kinds without numerators)
    uint32_t* den_w[RES_MAX_INST];
    const uint32_t* eq_evals;
};
__device__ __forceinline__ qm31 ldq_r(const uint32_t* p, size_t i) {
    uint4 v = reinterpret_cast<const uint4*>(p)[i];
    return {{v.x, v.y, v.z, v.w}};
}
__device__ __forceinline__ void stq_r(uint32_t* p, size_t i, qm31 v) {
    reinterpret_cast<uint4*>(p)[i] = make_uint4(v.c[0], v.c[1], v.c[2], v.c[3]);
}
// The summand of sum_as_poly_in_first_variable at t = 0 and t = 2 for term i (cpu/lookups/gkr.rs:39-211).
__device__ void sum_term(int kind, const uint32_t* num, const uint32_t* den, size_t nt, size_t i, qm31 lambda, qm31& t0, qm31& t2) {
    qm31 d00 = ldq_r(den, 2 * i), d01 = ldq_r(den, 2 * i + 1), d10 = ldq_r(den, 2 * (nt + i)), d11 = ldq_r(den, 2 * (nt + i) + 1);
    qm31 d20 = qm31_sub(qm31_dbl(d10), d00), d21 = qm31_sub(qm31_dbl(d11), d01);
    if (kind == ZKB_GKR_GRAND_PRODUCT) {
        t0 = qm31_mul(d00, d01);
        t2 = qm31_mul(d20, d21);
        return;
    }
    qm31 n0, n2;
    if (kind == ZKB_GKR_LOGUP_SINGLES) {
        n0 = qm31_add(d00, d01);
        n2 = qm31_add(d20, d21);
    } else if (kind == ZKB_GKR_LOGUP_MULTIPLICITIES) {
        uint32_t a0 = num[2 * i], a1 = num[2 * i + 1], b0 = num[2 * (nt + i)], b1 = num[2 * (nt + i) + 1];
        uint32_t n20 = m31_sub(m31_dbl(b0), a0), n21 = m31_sub(m31_dbl(b1), a1);
        n0 = qm31_add(qm31_mul_m31(d01, a0), qm31_mul_m31(d00, a1));
        n2 = qm31_add(qm31_mul_m31(d21, n20), qm31_mul_m31(d20, n21));
    } else {
        qm31 n00 = ldq_r(num, 2 * i), n01 = ldq_r(num, 2 * i + 1), n10 = ldq_r(num, 2 * (nt + i)), n11 = ldq_r(num, 2 * (nt + i) + 1);
        qm31 n20 = qm31_sub(qm31_dbl(n10), n00), n21 = qm31_sub(qm31_dbl(n11), n01);
        n0 = qm31_add(qm31_mul(d01, n00), qm31_mul(d00, n01));
        n2 = qm31_add(qm31_mul(d21, n20), qm31_mul(d20, n21));
    }
    t0 = qm31_add(n0, qm31_mul(lambda, qm31_mul(d00, d01)));
    t2 = qm31_add(n2, qm31_mul(lambda, qm31_mul(d20, d21)));
}
__global__ void __launch_bounds__(TAIL_THREADS) res_tail_kernel(ResState* st, TailArgs a) {
    __shared__ uint32_t red[TAIL_THREADS / 32][8];
    __shared__ qm31 sh_challenge;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // every thread tracks the oracles' current layers identically
    int kind[RES_MAX_INST], nvars[RES_MAX_INST];
    const uint32_t* num[RES_MAX_INST];
    const uint32_t* den[RES_MAX_INST];
    bool folded[RES_MAX_INST];
    for (int k = 0; k < a.n_oracles; k++) { kind[k] = a.kind[k]; nvars[k] = a.nvars[k]; num[k] = a.num[k]; den[k] = a.den[k]; folded[k] = false; }
    const qm31 lambda = st->lambda;
    for (int round = a.round_start; round < a.nv; round++) {
        const int n_rem = a.nv - round;
        for (int k = 0; k < a.n_oracles; k++) {
            if (n_rem != nvars[k]) continue;
            const size_t nt = ((size_t)2 << nvars[k]) / 4;  // the layer has 2^(nvars + 1) entries
            qm31 s0 = qm31_zero(), s2 = qm31_zero();
            for (size_t i = tid; i < nt; i += TAIL_THREADS) {
                qm31 t0, t2;
                sum_term(kind[k], num[k], den[k], nt, i, lambda, t0, t2);
                qm31 e = ldq_r(a.eq_evals, i);
                s0 = qm31_add(s0, qm31_mul(e, t0));
                s2 = qm31_add(s2, qm31_mul(e, t2));
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1)
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    s0.c[c] = m31_add(s0.c[c], __shfl_down_sync(0xffffffffu, s0.c[c], off));
                    s2.c[c] = m31_add(s2.c[c], __shfl_down_sync(0xffffffffu, s2.c[c], off));
                }
            if (lane == 0)
                for (int c = 0; c < 4; c++) { red[warp][c] = s0.c[c]; red[warp][4 + c] = s2.c[c]; }
            __syncthreads();
            if (tid < 8) {
                uint32_t acc = 0;
                for (int w = 0; w < TAIL_THREADS / 32; w++) acc = m31_add(acc, red[w][tid]);
                st->sums[k][tid] = acc;
            }
            __syncthreads();
        }
        if (warp == 0) {
            RoundArgs ra;
            ra.n_oracles = a.n_oracles;
            ra.n_rem = n_rem;
            ra.round = round;
            ra.poly_slot = a.first_poly_slot + (round - a.round_start);
            for (int k = 0; k < a.n_oracles; k++) ra.nvars[k] = nvars[k];
            round_step(st, ra);
            __syncwarp();
            if (lane == 0) sh_challenge = st->challenge;
        }
        __syncthreads();
        const qm31 r = sh_challenge;
        for (int k = 0; k < a.n_oracles; k++) {
            if (n_rem != nvars[k] || nvars[k] == 0) continue;
            const size_t half = (size_t)1 << nvars[k];  // entries after the fold
            const bool has_num = kind[k] == ZKB_GKR_LOGUP_GENERIC || kind[k] == ZKB_GKR_LOGUP_MULTIPLICITIES;
            for (size_t i = tid; i < half; i += TAIL_THREADS) {
                qm31 x = ldq_r(den[k], i), y = ldq_r(den[k], i + half);
                stq_r(a.den_w[k], i, qm31_add(qm31_mul(r, qm31_sub(y, x)), x));
                if (kind[k] == ZKB_GKR_LOGUP_MULTIPLICITIES) {
                    uint32_t p = num[k][i], q = num[k][i + half];
                    qm31 v = qm31_mul_m31(r, m31_sub(q, p));
                    v.c[0] = m31_add(v.c[0], p);
                    stq_r(a.num_w[k], i, v);
                } else if (has_num) {
                    qm31 p = ldq_r(num[k], i), q = ldq_r(num[k], i + half);
                    stq_r(a.num_w[k], i, qm31_add(qm31_mul(r, qm31_sub(q, p)), p));
                }
            }
            den[k] = a.den_w[k];
            if (has_num) { num[k] = a.num_w[k]; kind[k] = ZKB_GKR_LOGUP_GENERIC; }
            folded[k] = true;
            nvars[k]--;
        }
        __syncthreads();  // the folded layers are complete (and visible) before the next round reads them
    }
}

struct EndArgs {
    int n_oracles, nv, layer;
    int kind[RES_MAX_INST], inst[RES_MAX_INST];
    const uint32_t* num[RES_MAX_INST];  // the constant oracle's columns: two entries each
    const uint32_t* den[RES_MAX_INST];
};
__global__ void res_layer_end_kernel(ResState* st, EndArgs a) {
    if (threadIdx.x >= 32 || blockIdx.x != 0) return;
    Chan ch = chan_load(st);
    int ncols[RES_MAX_INST];
    for (int k = 0; k < a.n_oracles; k++) {  // try_into_mask, gkr_prover.rs:572-597
        qm31* m = st->masks[a.layer][k];
        const uint32_t* d = a.den[k];
        qm31 d0{{d[0], d[1], d[2], d[3]}}, d1{{d[4], d[5], d[6], d[7]}};
        if (a.kind[k] == ZKB_GKR_GRAND_PRODUCT) { m[0] = d0; m[1] = d1; ncols[k] = 1; }
        else if (a.kind[k] == ZKB_GKR_LOGUP_GENERIC) {
            const uint32_t* q = a.num[k];
            m[0] = qm31{{q[0], q[1], q[2], q[3]}}; m[1] = qm31{{q[4], q[5], q[6], q[7]}}; m[2] = d0; m[3] = d1; ncols[k] = 2;
        } else { m[0] = qm31_one(); m[1] = qm31_one(); m[2] = d0; m[3] = d1; ncols[k] = 2; }
    }
    __syncwarp();
    for (int k = 0; k < a.n_oracles; k++) chan_mix_felts(ch, st->masks[a.layer][k], 2 * ncols[k]);
    qm31 challenge = chan_draw_felt(ch);
    chan_store(st, ch);
    for (int j = 0; j < a.nv; j++) st->ood[j] = st->assignment[j];
    st->ood[a.nv] = challenge;
    st->ood_len = (uint32_t)a.nv + 1u;
    st->ood_prefix[0] = qm31_one();
    for (int j = 0; j <= a.nv; j++) st->ood_prefix[j + 1] = qm31_mul(st->ood_prefix[j], qm31_sub(qm31_one(), st->ood[j]));
    for (int k = 0; k < a.n_oracles; k++) {
        const qm31* m = st->masks[a.layer][k];
        int i = a.inst[k];
        for (int c = 0; c < ncols[k]; c++)
            st->claims[i][c] = qm31_add(qm31_mul(challenge, qm31_sub(m[2 * c + 1], m[2 * c])), m[2 * c]);
        st->n_claims[i] = (uint32_t)ncols[k];
    }
}

}  // namespace zk

using namespace zk;
using b200::B200Backend;
using b200::BaseColumn;
using b200::Device;
using b200::Layer;
using b200::SecureMle;

namespace b200 {

bool gkr_resident_supported(int n_inst, const uint64_t* ns) {
    if (n_inst < 1 || n_inst > RES_MAX_INST) return false;
    for (int i = 0; i < n_inst; i++)
        if (ns[i] < 2 || ns[i] > ((uint64_t)1 << 30)) return false;
    return true;
}

int gkr_prove_resident(zkb_ctx* ctx, std::vector<Layer> input_layers, uint32_t digest[8], uint32_t* n_draws,
                       std::vector<uint32_t>& o) {
    Device d(ctx);
    const size_t n_inst = input_layers.size();
    std::vector<size_t> n_layers_by_inst;
    for (auto& l : input_layers) n_layers_by_inst.push_back(l.n_variables());
    size_t n_layers = 0;
    for (auto v : n_layers_by_inst) n_layers = std::max(n_layers, v);
    std::vector<std::vector<Layer>> towers(n_inst);  // gen_layers, gkr_prover.rs:847-852
    for (size_t i = 0; i < n_inst; i++) {
        towers[i].push_back(std::move(input_layers[i]));
        while (towers[i].back().n_variables() > 0) towers[i].push_back(B200Backend::next_layer(d, towers[i].back()));
    }
    BaseColumn state_buf(d, (sizeof(ResState) + 3) / 4, true);
    ResState* st = reinterpret_cast<ResState*>(state_buf.ptr());
    {
        uint32_t head[12] = {0};
        for (int k = 0; k < 8; k++) head[k] = digest[k];
        head[8] = *n_draws;
        d.check(zkb_h2d(ctx, st, head, sizeof(head)));
    }
    cudaStream_t stream = ctx->stream;
    DeviceGuard guard(ctx);
    std::vector<bool> active(n_inst, false);
    std::vector<std::vector<int>> layer_oracle_inst(n_layers);   // per layer: instance of each oracle
    std::vector<std::vector<int>> layer_oracle_cols(n_layers);   // per layer: columns of each oracle's mask
    std::vector<int> layer_first_poly(n_layers), layer_nv(n_layers);
    int poly_slot = 0;
    auto take = [&](size_t i) { Layer l = std::move(towers[i].back()); towers[i].pop_back(); return l; };
    size_t ood_len = 0;
    for (size_t layer = 0; layer < n_layers; layer++) {
        const size_t n_remaining = n_layers - layer;
        BeginArgs ba;
        memset(&ba, 0, sizeof(ba));
        ba.n_inst = (int)n_inst;
        std::vector<Layer> out_layers;  // kept alive until the kernel has read them (stream-ordered frees)
        for (size_t i = 0; i < n_inst; i++)
            if (n_layers_by_inst[i] == n_remaining) {
                out_layers.push_back(take(i));
                const Layer& out = out_layers.back();
                ba.activate[i] = 1;
                ba.kind[i] = out.kind;
                ba.out_den[i] = out.den.words.ptr();
                ba.out_num[i] = out.kind == ZKB_GKR_LOGUP_MULTIPLICITIES ? out.num_base.ptr() : out.num_ptr();
                active[i] = true;
            }
        std::vector<Layer> oracle_layers;
        std::vector<int> nvars;
        for (size_t i = 0; i < n_inst; i++) {
            ba.active[i] = active[i] ? 1 : 0;
            if (active[i]) {
                ba.oracle_inst[oracle_layers.size()] = (int)i;
                oracle_layers.push_back(take(i));
                nvars.push_back((int)oracle_layers.back().n_variables() - 1);
            }
        }
        const int n_or = (int)oracle_layers.size();
        int nv = 0;
        for (int v : nvars) nv = std::max(nv, v);
        for (int k = 0; k < n_or; k++) ba.oracle_nvars[k] = nvars[k];
        ba.n_oracles = n_or;
        ba.nv = nv;
        { ProfScope prof(ctx, "res_layer_begin_kernel"); res_layer_begin_kernel<<<1, 32, 0, stream>>>(st, ba); }
        ZKB_LAUNCH_CHECK(ctx);
        out_layers.clear();
        // EqEvals::generate (gkr_prover.rs:235-247): eq(., ood[1..]) scaled by eq(0, ood[0]); nv - ... entries
        const int ny = ood_len == 0 ? 0 : (int)ood_len - 1;
        SecureMle eq_evals(d, (size_t)1 << ny);
        {
            const uint32_t* d_y = ood_len == 0 ? nullptr : reinterpret_cast<const uint32_t*>(&st->ood[1]);
            int rc = gkr_eq_evals_launch(ctx, d_y, ny, reinterpret_cast<const uint32_t*>(&st->eq_v), eq_evals.words.ptr());
            if (rc) return rc;
        }
        const uint32_t* d_lambda = reinterpret_cast<const uint32_t*>(&st->lambda);
        const uint32_t* d_r = reinterpret_cast<const uint32_t*>(&st->challenge);
        std::vector<bool> have_sums(n_or, false);
        layer_first_poly[layer] = poly_slot;
        layer_nv[layer] = nv;
        // rounds in which some layer still has more than 2^TAIL_MAX_LOG entries run as separate launches
        const int round_start = nv > TAIL_MAX_LOG - 1 ? nv - (TAIL_MAX_LOG - 1) : 0;
        for (int round = 0; round < round_start; round++) {
            const int n_rem = nv - round;
            for (int k = 0; k < n_or; k++)
                if (n_rem == nvars[k] && !have_sums[k]) {
                    const Layer& l = oracle_layers[k];
                    const uint32_t* num = l.kind == ZKB_GKR_LOGUP_MULTIPLICITIES ? l.num_base.ptr() : l.num_ptr();
                    int rc = gkr_sum_launch(ctx, l.kind, num, l.den.words.ptr(), l.len(), eq_evals.words.ptr(), d_lambda, st->sums[k]);
                    if (rc) return rc;
                }
            RoundArgs ra;
            memset(&ra, 0, sizeof(ra));
            ra.n_oracles = n_or;
            ra.n_rem = n_rem;
            ra.round = round;
            ra.poly_slot = poly_slot++;
            for (int k = 0; k < n_or; k++) ra.nvars[k] = nvars[k];
            { ProfScope prof(ctx, "res_round_kernel"); res_round_kernel<<<1, 32, 0, stream>>>(st, ra); }
            ZKB_LAUNCH_CHECK(ctx);
            for (int k = 0; k < n_or; k++)
                if (n_rem == nvars[k] && nvars[k] != 0) {
                    Layer& l = oracle_layers[k];
                    const size_t n = l.len();
                    Layer out;
                    out.kind = l.kind == ZKB_GKR_LOGUP_MULTIPLICITIES ? ZKB_GKR_LOGUP_GENERIC : l.kind;
                    out.den = SecureMle(d, n / 2);
                    if (out.kind == ZKB_GKR_LOGUP_GENERIC) out.num = SecureMle(d, n / 2);
                    const uint32_t* num = l.kind == ZKB_GKR_LOGUP_MULTIPLICITIES ? l.num_base.ptr() : l.num_ptr();
                    int rc;
                    if (n >= 8) {
                        rc = gkr_fold_sum_launch(ctx, l.kind, num, l.den.words.ptr(), n, d_r, eq_evals.words.ptr(), d_lambda,
                                                 out.kind == ZKB_GKR_LOGUP_GENERIC ? out.num.words.ptr() : nullptr, out.den.words.ptr(),
                                                 st->sums[k]);
                        have_sums[k] = true;
                    } else {
                        rc = gkr_mle_fix_launch(ctx, false, l.den.words.ptr(), n, d_r, out.den.words.ptr());
                        if (!rc && l.kind == ZKB_GKR_LOGUP_GENERIC) rc = gkr_mle_fix_launch(ctx, false, l.num.words.ptr(), n, d_r, out.num.words.ptr());
                        if (!rc && l.kind == ZKB_GKR_LOGUP_MULTIPLICITIES) rc = gkr_mle_fix_launch(ctx, true, l.num_base.ptr(), n, d_r, out.num.words.ptr());
                        have_sums[k] = false;
                    }
                    if (rc) return rc;
                    l = std::move(out);
                    nvars[k]--;  // the oracle's n_variables() follows its layer
                }
        }
        // the remaining rounds: one launch
        std::vector<SecureMle> work;  // alive until layer_end has been enqueued (stream-ordered frees)
        std::vector<int> fin_kind(n_or);
        std::vector<const uint32_t*> fin_num(n_or), fin_den(n_or);
        TailArgs ta;
        memset(&ta, 0, sizeof(ta));
        ta.n_oracles = n_or;
        ta.nv = nv;
        ta.round_start = round_start;
        ta.first_poly_slot = poly_slot;
        ta.eq_evals = eq_evals.words.ptr();
        for (int k = 0; k < n_or; k++) {
            const Layer& l = oracle_layers[k];
            ta.kind[k] = l.kind;
            ta.nvars[k] = nvars[k];
            ta.num[k] = l.num_ptr();
            ta.den[k] = l.den.words.ptr();
            fin_kind[k] = l.kind;
            fin_num[k] = l.num_ptr();
            fin_den[k] = l.den.words.ptr();
            if (l.len() > ((size_t)1 << TAIL_MAX_LOG) && round_start < nv) return set_error(ctx, ZKB_EINVAL, "gkr: tail layer too large");
            if (nvars[k] >= 1 && round_start < nv) {  // folded at least once by the tail kernel
                const bool has_num = l.kind == ZKB_GKR_LOGUP_GENERIC || l.kind == ZKB_GKR_LOGUP_MULTIPLICITIES;
                work.emplace_back(d, l.len() / 2);
                ta.den_w[k] = work.back().words.ptr();
                fin_den[k] = ta.den_w[k];
                if (has_num) {
                    work.emplace_back(d, l.len() / 2);
                    ta.num_w[k] = work.back().words.ptr();
                    fin_num[k] = ta.num_w[k];
                    fin_kind[k] = ZKB_GKR_LOGUP_GENERIC;
                }
            } else if (l.len() != 2) {
                return set_error(ctx, ZKB_EINVAL, "gkr: oracle is not constant after sumcheck");
            }
        }
        if (round_start < nv) {
            ProfScope prof(ctx, "res_tail_kernel");
            res_tail_kernel<<<1, TAIL_THREADS, 0, stream>>>(st, ta);
            ZKB_LAUNCH_CHECK(ctx);
            poly_slot += nv - round_start;
        }
        EndArgs ea;
        memset(&ea, 0, sizeof(ea));
        ea.n_oracles = n_or;
        ea.nv = nv;
        ea.layer = (int)layer;
        for (int k = 0; k < n_or; k++) {
            if (fin_kind[k] == ZKB_GKR_LOGUP_MULTIPLICITIES) return set_error(ctx, ZKB_EINVAL, "gkr: a multiplicities layer cannot be a mask");
            ea.kind[k] = fin_kind[k];
            ea.inst[k] = ba.oracle_inst[k];
            ea.den[k] = fin_den[k];
            ea.num[k] = fin_num[k];
            layer_oracle_inst[layer].push_back(ba.oracle_inst[k]);
            layer_oracle_cols[layer].push_back(fin_kind[k] == ZKB_GKR_GRAND_PRODUCT ? 1 : 2);
        }
        { ProfScope prof(ctx, "res_layer_end_kernel"); res_layer_end_kernel<<<1, 32, 0, stream>>>(st, ea); }
        ZKB_LAUNCH_CHECK(ctx);
        ood_len = (size_t)nv + 1;
    }
    // one copy, one synchronisation
    std::vector<uint32_t> raw = state_buf.to_cpu();
    const ResState* h = reinterpret_cast<const ResState*>(raw.data());
    if (h->error) return set_error(ctx, ZKB_EINVAL, "sumcheck: round polynomial does not match the claim");
    for (int k = 0; k < 8; k++) digest[k] = h->digest[k];
    *n_draws = h->n_draws;
    auto put = [&](const qm31& q) { o.insert(o.end(), q.c, q.c + 4); };
    o.push_back((uint32_t)n_layers);
    for (size_t layer = 0; layer < n_layers; layer++) {
        o.push_back((uint32_t)layer_nv[layer]);
        for (int r = 0; r < layer_nv[layer]; r++) {
            const Poly4& p = h->round_polys[layer_first_poly[layer] + r];
            o.push_back((uint32_t)p.n);
            for (int j = 0; j < p.n; j++) put(p.c[j]);
        }
    }
    for (size_t i = 0; i < n_inst; i++) {
        std::vector<std::pair<size_t, int>> where;  // (layer, oracle index) of every mask of this instance
        for (size_t layer = 0; layer < n_layers; layer++)
            for (size_t k = 0; k < layer_oracle_inst[layer].size(); k++)
                if (layer_oracle_inst[layer][k] == (int)i) where.push_back({layer, (int)k});
        o.push_back((uint32_t)where.size());
        for (auto& w : where) {
            int cols = layer_oracle_cols[w.first][w.second];
            o.push_back((uint32_t)cols);
            for (int c = 0; c < 2 * cols; c++) put(h->masks[w.first][w.second][c]);
        }
    }
    for (size_t i = 0; i < n_inst; i++) {
        o.push_back(h->n_output_claims[i]);
        for (uint32_t c = 0; c < h->n_output_claims[i]; c++) put(h->output_claims[i][c]);
    }
    o.push_back(h->ood_len);
    for (uint32_t j = 0; j < h->ood_len; j++) put(h->ood[j]);
    for (size_t i = 0; i < n_inst; i++) {
        o.push_back(h->n_claims[i]);
        for (uint32_t c = 0; c < h->n_claims[i]; c++) put(h->claims[i][c]);
    }
    return ZKB_OK;
}

}  // namespace b200
