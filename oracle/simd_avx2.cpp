// The packed restatement compiled for AVX2 (a 16-lane vector is two 32-byte registers). Test infrastructure.
#define ZKO_SIMD_NS simd_avx2
#include "simd.hpp"
#include "accel.hpp"
namespace zko {
void fill_accel_avx2(Accel& a) {
    a.lanes = 8;
    a.interpolate = simd_avx2::interpolate;
    a.evaluate = simd_avx2::evaluate;
    a.leaf_hashes = simd_avx2::leaf_hashes;
    a.node_hashes = simd_avx2::node_hashes;
    a.eval_by_folding = simd_avx2::eval_by_folding;
    a.numerators = simd_avx2::numerators;
}
}  // namespace zko
