// TEST INFRASTRUCTURE ONLY (CPU oracle; see fields.hpp).
//
// Circle FFT (interpolate / evaluate / extend), twiddle tower, point evaluation. Follows
//   nitroo/crates/stwo/src/core/fft.rs:5-21                       (butterfly, ibutterfly)
//   nitroo/crates/stwo/src/prover/backend/cpu/circle.rs:28-80     (interpolate)
//   nitroo/crates/stwo/src/prover/backend/cpu/circle.rs:82-100    (eval_at_point)
//   nitroo/crates/stwo/src/prover/backend/cpu/circle.rs:182-228   (extend, evaluate)
//   nitroo/crates/stwo/src/prover/backend/cpu/circle.rs:230-332   (precompute_twiddles,
//        slow_precompute_twiddles, fft_layer_loop, circle_twiddles_from_line_twiddles)
//   nitroo/crates/stwo/src/core/poly/utils.rs:11-23, 98-114       (fold, domain_line_twiddles_from_tree)
#pragma once
#include "accel.hpp"
#include "circle.hpp"

namespace zko {

// fft.rs:5-12
template <class F> inline void butterfly(F& v0, F& v1, M31 twid) {
    F tmp = v1 * twid;
    v1 = v0 - tmp;
    v0 = v0 + tmp;
}
// fft.rs:14-21
template <class F> inline void ibutterfly(F& v0, F& v1, M31 itwid) {
    F tmp = v0;
    v0 = tmp + v1;
    v1 = (tmp - v1) * itwid;
}

// cpu/circle.rs:274-291
inline std::vector<M31> slow_precompute_twiddles(Coset coset) {
    std::vector<M31> tw;
    tw.reserve(coset.size());
    uint32_t log = coset.log_size;
    for (uint32_t k = 0; k < log; k++) {
        size_t i0 = tw.size();
        size_t half = coset.size() / 2;
        CirclePoint<M31> cur = coset.initial;
        for (size_t j = 0; j < half; j++) {
            tw.push_back(cur.x);
            cur = cur + coset.step;
        }
        bit_reverse(tw.data() + i0, half);
        coset = coset.dbl();
    }
    tw.push_back(M31(1));
    return tw;
}

struct TwiddleTree {
    Coset root_coset;
    std::vector<M31> twiddles, itwiddles;
};
// cpu/circle.rs:230-261 (inverses are unique, so the chunked batch inversion is restated as
// a per-element inversion)
inline TwiddleTree precompute_twiddles(Coset coset) {
    TwiddleTree t{coset, slow_precompute_twiddles(coset), {}};
    t.itwiddles.resize(t.twiddles.size());
    for (size_t i = 0; i < t.twiddles.size(); i++) t.itwiddles[i] = t.twiddles[i].inverse();
    return t;
}

// poly/utils.rs:98-114 — per line layer, a (pointer, length) slice of the tower.
struct TwSlice { const M31* p; size_t n; };
inline std::vector<TwSlice> domain_line_twiddles_from_tree(const Coset& half_coset, const std::vector<M31>& buf) {
    assert(half_coset.size() <= buf.size());
    std::vector<TwSlice> out;
    for (uint32_t i = 0; i < half_coset.log_size; i++) {
        size_t len = (size_t)1 << i;
        out.push_back({buf.data() + buf.size() - len * 2, len});
    }
    std::vector<TwSlice> rev(out.rbegin(), out.rend());
    return rev;
}

// cpu/circle.rs:312-332 — layer-0 twiddles [y, -y, -x, x] from each pair (x, y) of layer 1.
inline std::vector<M31> circle_twiddles_from_line_twiddles(TwSlice first) {
    std::vector<M31> out;
    out.reserve(first.n * 2);
    for (size_t k = 0; k + 2 <= first.n; k += 2) {
        M31 x = first.p[k], y = first.p[k + 1];
        out.push_back(y); out.push_back(-y); out.push_back(-x); out.push_back(x);
    }
    return out;
}

// cpu/circle.rs:293-307
template <class BF> inline void fft_layer_loop(M31* values, size_t i, size_t h, M31 t, BF bf) {
    for (size_t l = 0; l < ((size_t)1 << i); l++) {
        size_t idx0 = (h << (i + 1)) + l;
        size_t idx1 = idx0 + ((size_t)1 << i);
        bf(values[idx0], values[idx1], t);
    }
}

// cpu/circle.rs:28-80 — evaluations (bit-reversed, on `domain`) -> coefficients, in place.
inline void interpolate(std::vector<M31>& values, const CircleDomain& domain, const TwiddleTree& tw) {
    assert(values.size() == domain.size());
    assert(domain.log_size() <= tw.root_coset.log_size + 1);
    auto ibf = [](M31& a, M31& b, M31 t) { ibutterfly(a, b, t); };
    if (domain.log_size() == 1) {
        M31 y = domain.half_coset.initial.y;
        M31 n = M31(2);
        M31 yn_inv = (y * n).inverse();
        M31 y_inv = yn_inv * n;
        M31 n_inv = yn_inv * y;
        M31 v0 = values[0], v1 = values[1];
        ibutterfly(v0, v1, y_inv);
        values[0] = v0 * n_inv; values[1] = v1 * n_inv;
        return;
    }
    if (domain.log_size() == 2) {
        M31 x = domain.half_coset.initial.x, y = domain.half_coset.initial.y;
        M31 n = M31(4);
        M31 xyn_inv = (x * y * n).inverse();
        M31 x_inv = xyn_inv * y * n;
        M31 y_inv = xyn_inv * x * n;
        M31 n_inv = xyn_inv * x * y;
        M31 v0 = values[0], v1 = values[1], v2 = values[2], v3 = values[3];
        ibutterfly(v0, v1, y_inv);
        ibutterfly(v2, v3, -y_inv);
        ibutterfly(v0, v2, x_inv);
        ibutterfly(v1, v3, x_inv);
        values[0] = v0 * n_inv; values[1] = v1 * n_inv; values[2] = v2 * n_inv; values[3] = v3 * n_inv;
        return;
    }
    auto line_tw = domain_line_twiddles_from_tree(domain.half_coset, tw.itwiddles);
    auto circle_tw = circle_twiddles_from_line_twiddles(line_tw[0]);
    if (accel().interpolate && domain.log_size() >= 5) {  // the packed restatement of the SIMD backend (simd.hpp)
        std::vector<const uint32_t*> lt;
        for (auto& s : line_tw) lt.push_back(&s.p->v);
        accel().interpolate(&values[0].v, domain.log_size(), lt.data(), &circle_tw[0].v, M31((uint32_t)domain.size()).inverse().v);
        return;
    }
    for (size_t h = 0; h < circle_tw.size(); h++) fft_layer_loop(values.data(), 0, h, circle_tw[h], ibf);
    for (size_t layer = 0; layer < line_tw.size(); layer++)
        for (size_t h = 0; h < line_tw[layer].n; h++)
            fft_layer_loop(values.data(), layer + 1, h, line_tw[layer].p[h], ibf);
    M31 inv = M31((uint32_t)domain.size()).inverse();
    for (auto& v : values) v = v * inv;
}

// cpu/circle.rs:182-228 — coefficients (zero-extended to `domain`) -> bit-reversed evaluations.
inline std::vector<M31> evaluate(const std::vector<M31>& coeffs, const CircleDomain& domain, const TwiddleTree& tw) {
    assert(domain.half_coset.is_doubling_of(tw.root_coset));
    assert(domain.size() >= coeffs.size());
    std::vector<M31> values(coeffs);
    values.resize(domain.size(), M31(0));  // extend, :190-197
    auto bf = [](M31& a, M31& b, M31 t) { butterfly(a, b, t); };
    if (domain.log_size() == 1) {
        butterfly(values[0], values[1], domain.half_coset.initial.y);
        return values;
    }
    if (domain.log_size() == 2) {
        M31 x = domain.half_coset.initial.x, y = domain.half_coset.initial.y;
        butterfly(values[0], values[2], x);
        butterfly(values[1], values[3], x);
        butterfly(values[0], values[1], y);
        butterfly(values[2], values[3], -y);
        return values;
    }
    auto line_tw = domain_line_twiddles_from_tree(domain.half_coset, tw.twiddles);
    auto circle_tw = circle_twiddles_from_line_twiddles(line_tw[0]);
    if (accel().evaluate && domain.log_size() >= 5) {
        std::vector<const uint32_t*> lt;
        for (auto& s : line_tw) lt.push_back(&s.p->v);
        accel().evaluate(&values[0].v, domain.log_size(), lt.data(), &circle_tw[0].v);
        return values;
    }
    for (size_t layer = line_tw.size(); layer-- > 0;)
        for (size_t h = 0; h < line_tw[layer].n; h++)
            fft_layer_loop(values.data(), layer + 1, h, line_tw[layer].p[h], bf);
    for (size_t h = 0; h < circle_tw.size(); h++) fft_layer_loop(values.data(), 0, h, circle_tw[h], bf);
    return values;
}

// poly/utils.rs:11-23
template <class F> inline QM31 to_qm31(F v);
template <> inline QM31 to_qm31<M31>(M31 v) { return QM31(v); }
template <> inline QM31 to_qm31<QM31>(QM31 v) { return v; }
template <class F> inline QM31 fold(const F* values, size_t n, const QM31* factors) {
    if (n == 1) return to_qm31(values[0]);
    QM31 l = fold(values, n / 2, factors + 1);
    QM31 r = fold(values + n / 2, n / 2, factors + 1);
    return l + r * factors[0];
}

// cpu/circle.rs:82-100
inline QM31 eval_at_point(const std::vector<M31>& coeffs, CirclePoint<QM31> point) {
    uint32_t log_size = ilog2(coeffs.size());
    if (log_size == 0) return QM31(coeffs[0]);
    std::vector<QM31> mappings;
    mappings.push_back(point.y);
    QM31 x = point.x;
    for (uint32_t i = 1; i < log_size; i++) {
        mappings.push_back(x);
        x = double_x(x);
    }
    std::vector<QM31> rev(mappings.rbegin(), mappings.rend());
    if (accel().eval_by_folding && coeffs.size() >= 64) return accel().eval_by_folding(&coeffs[0].v, coeffs.size(), rev.data());
    return fold(coeffs.data(), coeffs.size(), rev.data());
}

}  // namespace zko
