// Reads of many (column, row) cells in one round trip (ctx.cu); internal to the library.
#pragma once
#include <cstddef>
#include <cstdint>

struct zkb_ctx;

namespace zk {

// out[out_off + i * ncols + c] = cols[c][idx[i]]: the rows idx[0..nidx) of ncols device columns, row-major.
// cols and idx are host arrays (cols holds device pointers).
struct GatherBlock {
    const uint32_t* const* cols;
    int ncols;
    const uint32_t* idx;
    int nidx;
    size_t out_off;
};

// Runs every block (one small launch each) and brings all total_words results to h_out with one copy and one
// synchronisation. Column::batch_at_multi (nitroo/crates/stwo/src/prover/backend/mod.rs:74-89) for all the layers of
// all the trees of a decommitment at once.
int gather_blocks(zkb_ctx* ctx, const GatherBlock* blocks, int n_blocks, size_t total_words, uint32_t* h_out);

}  // namespace zk
