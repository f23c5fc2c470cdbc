// TEST INFRASTRUCTURE - switchboard between the scalar oracle and its packed (16-lane) restatement of the reference's SIMD
// backend (simd.hpp). With no entry set (the default, and what every parity test uses as its checker) the oracle is the
// plain scalar restatement of CpuBackend; zko_set_simd(1) fills the entries, after which the operators below run packed
// and give the same words (tests/test_oracle_simd.py compares the two on every operator and on whole proofs).
#pragma once
#include <cstddef>
#include <cstdint>

#include "fields.hpp"

namespace zko {

struct Accel {
    int lanes = 0;  // 16 with AVX-512, 8 with AVX2 (a 16-lane vector is two registers), 0: scalar
    void (*interpolate)(uint32_t* v, unsigned log, const uint32_t* const* line_tw, const uint32_t* circle_tw, uint32_t n_inv) = nullptr;
    void (*evaluate)(uint32_t* v, unsigned log, const uint32_t* const* line_tw, const uint32_t* circle_tw) = nullptr;
    void (*leaf_hashes)(uint32_t* out, const uint32_t* const* cols, size_t ncols, size_t n, bool m31) = nullptr;
    void (*node_hashes)(uint32_t* out, const uint32_t* prev, size_t n, bool m31) = nullptr;
    QM31 (*eval_by_folding)(const uint32_t* coeffs, size_t n, const QM31* factors) = nullptr;
    void (*numerators)(uint32_t* acc, const uint32_t* const* cols, const size_t* idx, const QM31* c, size_t k, QM31 b_sum, size_t n) = nullptr;
};
inline Accel& accel() {
    static Accel a;
    return a;
}

}  // namespace zko
