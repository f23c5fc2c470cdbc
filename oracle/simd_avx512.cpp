// The packed restatement compiled for AVX-512 (one 64-byte register per 16-lane vector). Test infrastructure.
#define ZKO_SIMD_NS simd_avx512
#include "simd.hpp"
#include "accel.hpp"
namespace zko {
void fill_accel_avx512(Accel& a) {
    a.lanes = 16;
    a.interpolate = simd_avx512::interpolate;
    a.evaluate = simd_avx512::evaluate;
    a.leaf_hashes = simd_avx512::leaf_hashes;
    a.node_hashes = simd_avx512::node_hashes;
    a.eval_by_folding = simd_avx512::eval_by_folding;
    a.numerators = simd_avx512::numerators;
}
}  // namespace zko
