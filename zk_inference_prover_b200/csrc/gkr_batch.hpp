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
    unsigned long long pad;
};
static_assert(sizeof(GkrBatchItem) == 64, "GkrBatchItem layout");

constexpr size_t GKR_BATCH_MAX_ITEMS = 8192;
// Per item: [0,8) the two sums (t = 0, t = 2); mode 2 only: [8,16) the two fixed denominators, [16,24) the two fixed numerators.
constexpr size_t GKR_BATCH_RESULT_WORDS = 24;

// next_layer of every item, one launch, stream-ordered.
int gkr_batch_next_layer(zkb_ctx* ctx, GkrBatchItem* items, int n_items);
// One round for every item: one launch, one copy of n_items * GKR_BATCH_RESULT_WORDS words to h_results, one synchronisation.
int gkr_batch_round(zkb_ctx* ctx, GkrBatchItem* items, int n_items, const uint32_t h_r[4], const uint32_t* eq_evals, const uint32_t h_lambda[4],
                    uint32_t* h_results);

}  // namespace zk
