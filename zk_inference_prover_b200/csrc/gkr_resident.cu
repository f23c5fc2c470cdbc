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
__device__ void chan_mix_words(ResState* st, const uint32_t* w, int n) {
    uint32_t h[8], m[16];
    blake2s_init(h);
    const int total = 8 + n;
    uint32_t t = 0;
    int pos = 0;
    while (total - pos > 16) {
        for (int k = 0; k < 16; k++) { int i = pos + k; m[k] = i < 8 ? st->digest[i] : w[i - 8]; }
        pos += 16;
        t += 64;
        blake2s_compress(h, m, t, false);
    }
    int rem = total - pos;
    for (int k = 0; k < 16; k++) { int i = pos + k; m[k] = k < rem ? (i < 8 ? st->digest[i] : w[i - 8]) : 0u; }
    t += 4u * (uint32_t)rem;
    blake2s_compress(h, m, t, true);
    for (int k = 0; k < 8; k++) st->digest[k] = reduce_word_m31(h[k]);
    st->n_draws = 0;
}
__device__ void chan_mix_felts(ResState* st, const qm31* f, int n) { chan_mix_words(st, (const uint32_t*)f, 4 * n); }
__device__ qm31 chan_draw_felt(ResState* st) {
    uint32_t u[8];
    for (int attempt = 0; attempt < 64; attempt++) {
        uint32_t h[8], m[16];
        blake2s_init(h);
        for (int k = 0; k < 8; k++) m[k] = st->digest[k];
        m[8] = st->n_draws;
        for (int k = 9; k < 16; k++) m[k] = 0u;
        blake2s_compress(h, m, 37u, true);
        st->n_draws++;
        bool ok = true;
        for (int k = 0; k < 8; k++) { u[k] = reduce_word_m31(h[k]); ok = ok && u[k] < 2u * P; }
        if (ok) break;
    }
    qm31 r;
    for (int k = 0; k < 4; k++) r.c[k] = u[k] >= P ? u[k] - P : u[k];
    return r;
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
__device__ Poly4 correct_sum(qm31 f0, qm31 f2, qm31 claim, const qm31* y, const qm31* one_minus_y_prefix, int n, int k) {
    // a = prod_{i < n-k+1} eq(0, y_i) = prod (1 - y_i): kept as prefix products by layer_end
    const qm31 a = one_minus_y_prefix[n - k + 1];
    const qm31 one = qm31_one(), yk = y[n - k];
    const qm31 d = qm31_sub(one, qm31_dbl(yk));                       // 1 - 2y
    const qm31 omy = qm31_sub(one, yk);                                // 1 - y = eq(0, y)
    const qm31 v[5] = {a, d, omy, yk, qm31_sub(omy, qm31_dbl(yk))};   // a, 1-2y, 1-y, y, 1-3y
    qm31 pre[5], inv[5];
    qm31 run = one;
    for (int i = 0; i < 5; i++) { pre[i] = run; run = qm31_mul(run, v[i]); }
    qm31 r = qm31_inv(run);
    for (int i = 5; i-- > 0;) { inv[i] = qm31_mul(r, pre[i]); r = qm31_mul(r, v[i]); }
    const qm31 a_inv = inv[0];
    const qm31 b = qm31_mul(omy, inv[1]);
    const qm31 inv_b = qm31_mul(d, inv[2]);               // 1 / b
    const qm31 inv_1mb = qm31_neg(qm31_mul(d, inv[3]));   // 1 / (1 - b) = (1 - 2y) / (-y)
    const qm31 inv_2mb = qm31_mul(d, inv[4]);             // 1 / (2 - b)
    const uint32_t half = 1u << 30;                        // 1 / 2
    // eq(0, y) = 1 - y; eq(2, y) = 2y + (1 - 2)(1 - y) = 3y - 1
    qm31 r0 = qm31_mul(qm31_mul(f0, omy), a_inv);
    qm31 r1 = qm31_sub(claim, r0);
    qm31 r2 = qm31_mul(qm31_mul(f2, qm31_neg(v[4])), a_inv);
    // Lagrange weights p_i = ys[i] * prod_{j != i} 1 / (xs[i] - xs[j]) over xs = {0, 1, 2, b}; ys[3] = 0
    qm31 p0 = qm31_neg(qm31_mul(qm31_mul_m31(r0, half), inv_b));      // 1/(0-1) * 1/(0-2) * 1/(0-b) = -1/(2b)
    qm31 p1 = qm31_neg(qm31_mul(r1, inv_1mb));                         // 1/(1-0) * 1/(1-2) * 1/(1-b)
    qm31 p2 = qm31_mul(qm31_mul_m31(r2, half), inv_2mb);               // 1/(2-0) * 1/(2-1) * 1/(2-b)
    // sum_i p_i prod_{j != i} (t - xs[j]), expanded:
    //   (t-1)(t-2)(t-b) = t^3 - (3+b) t^2 + (2+3b) t - 2b;  t(t-2)(t-b) = t^3 - (2+b) t^2 + 2b t;  t(t-1)(t-b) = t^3 - (1+b) t^2 + b t
    const qm31 b2 = qm31_dbl(b), b3 = qm31_add(b2, b);
    Poly4 c;
    c.n = 4;
    c.c[3] = qm31_add(qm31_add(p0, p1), p2);
    c.c[2] = qm31_neg(qm31_add(qm31_add(qm31_mul(qm31_add(qm31_from_m31(3), b), p0), qm31_mul(qm31_add(qm31_from_m31(2), b), p1)),
                               qm31_mul(qm31_add(one, b), p2)));
    c.c[1] = qm31_add(qm31_add(qm31_mul(qm31_add(qm31_from_m31(2), b3), p0), qm31_mul(b2, p1)), qm31_mul(b, p2));
    c.c[0] = qm31_neg(qm31_mul(b2, p0));
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
__global__ void res_layer_begin_kernel(ResState* st, BeginArgs a) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
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
    for (int i = 0; i < a.n_inst; i++)
        if (a.active[i]) chan_mix_felts(st, st->claims[i], (int)st->n_claims[i]);
    st->eq_v = st->ood_len == 0 ? qm31_one() : eq1(qm31_zero(), st->ood[0]);
    st->alpha = chan_draw_felt(st);
    st->lambda = chan_draw_felt(st);
    for (int k = 0; k < a.n_oracles; k++) {
        int i = a.oracle_inst[k];
        qm31 acc = qm31_zero();
        for (int j = (int)st->n_claims[i]; j-- > 0;) acc = qm31_add(qm31_mul(acc, st->lambda), st->claims[i][j]);
        st->sc_claim[k] = qm31_mul_m31(acc, 1u << (a.nv - a.oracle_nvars[k]));
        st->eq_corr[k] = qm31_one();
    }
}

struct RoundArgs {
    int n_oracles, n_rem, round, poly_slot;
    int nvars[RES_MAX_INST];
};
__global__ void res_round_kernel(ResState* st, RoundArgs a) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
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
        for (int j = 0; j < combined.n; j++) combined.c[j] = qm31_mul(combined.c[j], st->alpha);
        combined = p_add(combined, rp[k]);
    }
    chan_mix_felts(st, combined.c, combined.n);
    qm31 challenge = chan_draw_felt(st);
    for (int k = 0; k < a.n_oracles; k++) st->sc_claim[k] = p_eval(rp[k], challenge);
    for (int k = 0; k < a.n_oracles; k++)
        if (a.n_rem == a.nvars[k] && a.nvars[k] != 0) {
            qm31 z0 = st->ood[st->ood_len - a.nvars[k]];
            st->eq_corr[k] = qm31_mul(st->eq_corr[k], eq1(challenge, z0));
        }
    st->round_polys[a.poly_slot] = combined;
    st->assignment[a.round] = challenge;
    st->challenge = challenge;
}

struct EndArgs {
    int n_oracles, nv, layer;
    int kind[RES_MAX_INST], inst[RES_MAX_INST];
    const uint32_t* num[RES_MAX_INST];  // the constant oracle's columns: two entries each
    const uint32_t* den[RES_MAX_INST];
};
__global__ void res_layer_end_kernel(ResState* st, EndArgs a) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
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
    for (int k = 0; k < a.n_oracles; k++) chan_mix_felts(st, st->masks[a.layer][k], 2 * ncols[k]);
    qm31 challenge = chan_draw_felt(st);
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
        for (int round = 0; round < nv; round++) {
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
        EndArgs ea;
        memset(&ea, 0, sizeof(ea));
        ea.n_oracles = n_or;
        ea.nv = nv;
        ea.layer = (int)layer;
        for (int k = 0; k < n_or; k++) {
            const Layer& l = oracle_layers[k];
            if (l.len() != 2) return set_error(ctx, ZKB_EINVAL, "gkr: oracle is not constant after sumcheck");
            if (l.kind == ZKB_GKR_LOGUP_MULTIPLICITIES) return set_error(ctx, ZKB_EINVAL, "gkr: a multiplicities layer cannot be a mask");
            ea.kind[k] = l.kind;
            ea.inst[k] = ba.oracle_inst[k];
            ea.den[k] = l.den.words.ptr();
            ea.num[k] = l.num_ptr();
            layer_oracle_inst[layer].push_back(ba.oracle_inst[k]);
            layer_oracle_cols[layer].push_back(l.kind == ZKB_GKR_GRAND_PRODUCT ? 1 : 2);
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
