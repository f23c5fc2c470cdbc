// GKR prove_batch with the transcript resident on the device (gkr_resident.cu); internal to the library.
#pragma once
#include <cstdint>
#include <vector>

struct zkb_ctx;

namespace b200 {

struct Layer;

// Up to 16 instances of 2..2^30 entries each.
bool gkr_resident_supported(int n_inst, const uint64_t* ns);
// `digest`/`n_draws`: the channel before the proof on entry, after it on return. Appends the proof words to `o`.
int gkr_prove_resident(zkb_ctx* ctx, std::vector<Layer> input_layers, uint32_t digest[8], uint32_t* n_draws, std::vector<uint32_t>& o);

}  // namespace b200
