// One launch per sum-check round for a GKR batch of any number of instances (gkr_batch.cu); internal to the library.
#pragma once
#include <cstddef>
#include <cstdint>

struct zkb_ctx;

namespace zk {

// What to do for one instance in a batched launch. kind: ZKB_GKR_* of the INPUT arrays; n: entries of the input layer.
// mode 0: round sums of the layer; 1: fix the first variable into num_out/den_out (n >= 8) and round sums of the result;
// 2: fix the first variable of a 4-entry layer, the result also copied to the result words; 3: next_layer.
// first_block / blocks are filled by the launcher.
struct GkrBatchItem {
    const uint32_t* num;
    const uint32_t* den;
    uint32_t* num_out;
    uint32_t* den_out;
    unsigned long long n;
    uint32_t kind, mode, first_block, blocks;
    unsigned long long slot;  // gkr_batch_layer: the oracle the item belongs to (its results go to that oracle's record)
};
static_assert(sizeof(GkrBatchItem) == 64, "GkrBatchItem layout");

constexpr size_t GKR_BATCH_MAX_ITEMS = 8192;
// Per item: [0,8) the two sums (t = 0, t = 2); mode 2 only: [8,16) the two fixed denominators, [16,24) the two fixed numerators.
constexpr size_t GKR_BATCH_RESULT_WORDS = 24;

// next_layer of every item, one launch, stream-ordered.
int gkr_batch_next_layer(zkb_ctx* ctx, GkrBatchItem* items, int n_items);
// One round for every item with the transcript on the host: one launch that writes n_items * GKR_BATCH_RESULT_WORDS words and
// a completion word into page-locked host memory; returns when the host has seen the completion word (h_results filled).
int gkr_batch_round(zkb_ctx* ctx, GkrBatchItem* items, int n_items, const uint32_t h_r[4], const uint32_t* eq_evals, const uint32_t h_lambda[4],
                    uint32_t* h_results);


// ---- a layer's whole sum-check enqueued at once (no host round trip per round)
//
// What runs in a round depends on the oracles' sizes only, never on the transcript, so the host describes every round of a
// layer's sum-check up front and the device keeps the transcript between the launches. Launch j (0 <= j <= rounds) carries the
// fixes of round j - 1 (mode 1 / 2 items, the challenge read from device memory) and the first sums of the oracles that
// enter in round j (mode 0 items); the CTA that completes the launch goes on with the transcript step of round j: the
// batch's round polynomial from all oracles' sums, mixed into the channel, the challenge drawn, every oracle's claim and
// correction updated. The launches of the small rounds at the end of the layer are replaced by one single-CTA launch that
// runs the same tables one after the other. One copy brings back the round polynomials, the challenges, the masks and the
// channel (sumcheck.rs:96-176 inside gkr_prover.rs:669-844).
struct GkrRoundConst {
    // The basis of the round's polynomials (all active oracles have n_rem variables left, so their round polynomials are
    // r0 L0 + r1 L1 + r2 L2 over one basis): e0a = eq(0, y) / prod, e2a = eq(2, y) / prod, L[i] the coefficients (low first)
    // of the basis polynomial of node i; y = the coordinate of the layer's point this round fixes.
    uint32_t e0a[4], e2a[4], L[3][4][4], y[4];
    uint32_t n_rem, pad[3];
};
static_assert(sizeof(GkrRoundConst) == 256, "GkrRoundConst layout");

struct GkrLayerRound {
    GkrRoundConst rc;
    GkrBatchItem* first;  // mode 0 items of the oracles that enter in this round (slot = oracle)
    int n_first;
    GkrBatchItem* fix;    // mode 1 / 2 items of every active oracle (slot = oracle)
    int n_fix;
};

constexpr int GKR_LAYER_MAX_ROUNDS = 60;
constexpr size_t GKR_LAYER_OUT_WORDS = 24;  // per round: [0,16) coefficients, [16] length, [20,24) challenge

// n_vars[k]: variables of oracle k's sum-check (it is active in the rounds with n_rem <= n_vars[k]); alpha_pow[k] = alpha^k;
// claims[k]: its claim before the first round (4 words each). chan: digest (8 words) and n_draws, in and out.
// h_out: n_rounds x GKR_LAYER_OUT_WORDS; h_res: n_oracles x GKR_BATCH_RESULT_WORDS (the last sums and, for every oracle that
// had a round, its mask).
int gkr_batch_layer(zkb_ctx* ctx, int n_oracles, const uint32_t* n_vars, const uint32_t* alpha_pow, const uint32_t* claims,
                    GkrLayerRound* rounds, int n_rounds, const uint32_t* eq_evals, const uint32_t h_lambda[4], uint32_t chan[9],
                    uint32_t* h_out, uint32_t* h_res);

}  // namespace zk
