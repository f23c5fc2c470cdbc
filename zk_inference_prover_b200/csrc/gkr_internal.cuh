// Launchers shared inside the library (not part of the C ABI): the GKR kernels with their challenges read from
// device memory and their sums left on the device, for the device-resident transcript of gkr_resident.cu.
#pragma once
#include "common.cuh"

namespace zk {

int gkr_sum_launch(zkb_ctx* ctx, int kind, const uint32_t* num, const uint32_t* den, size_t n, const uint32_t* eq_evals,
                   const uint32_t* d_lambda, uint32_t* d_result);
int gkr_mle_fix_launch(zkb_ctx* ctx, bool base, const uint32_t* in, size_t n, const uint32_t* d_r, uint32_t* out);
int gkr_eq_evals_launch(zkb_ctx* ctx, const uint32_t* d_y, int ny, const uint32_t* d_v, uint32_t* out);
int gkr_fold_sum_launch(zkb_ctx* ctx, int kind, const uint32_t* num, const uint32_t* den, size_t n, const uint32_t* d_r,
                        const uint32_t* eq_evals, const uint32_t* d_lambda, uint32_t* num_out, uint32_t* den_out, uint32_t* d_result);

}  // namespace zk
