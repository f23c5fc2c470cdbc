// Entry points of fft.cu that other parts of the library use (not part of the C ABI).
#pragma once
#include <cstdint>

struct zkb_ctx;

namespace zk {

// zkb_lde_cols with every output column laid out in row blocks: word idx of column c lies at
// out[c] + (idx >> blk_log) * blk_stride + (idx mod 2^blk_log). A sharded commitment uses it to write the extended
// columns directly in the order the exchange sends them ([destination rank][column][rows]). blk_log = 31: plain columns.
bool lde_blocked_supported(int log_n, int log_out, int blk_log);
int lde_cols_blocked(zkb_ctx* ctx, const uint32_t* const* coeffs, int ncols, int log_n, uint32_t* const* out, int log_out, int blk_log,
                     uint32_t blk_stride);
// out[(b * ncols + c) << blk_log + i] = in[c << log_out + (b << blk_log) + i]: the same layout from plain columns, for the
// sizes the blocked transform does not cover.
int repack_row_blocks(zkb_ctx* ctx, const uint32_t* in, uint32_t* out, int ncols, int log_out, int blk_log);

}  // namespace zk
