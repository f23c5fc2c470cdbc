// TEST INFRASTRUCTURE ONLY (CPU oracle; see fields.hpp). The three PolyOps methods that evaluate a polynomial from its
// EVALUATIONS rather than from its coefficients:
//   nitroo/crates/stwo/src/prover/backend/cpu/circle.rs:101-132   barycentric_weights
//   nitroo/crates/stwo/src/prover/backend/cpu/circle.rs:134-141   barycentric_eval_at_point
//   nitroo/crates/stwo/src/prover/backend/cpu/circle.rs:143-180   eval_at_point_by_folding
//   nitroo/crates/stwo/src/core/constraints.rs:12-55, 87-93       coset_vanishing, coset_vanishing_derivative, point_vanishing
//   nitroo/crates/stwo/src/core/poly/utils.rs:45-70               get_folding_alphas
#pragma once
#include "stark.hpp"

namespace zko {

// constraints.rs:38-55 at a secure-field point (only the coset's log size enters)
inline QM31 coset_vanishing_derivative(uint32_t log_size, CirclePoint<QM31> p) {
    QM31 exp = QM31::one(), four = QM31(M31(4));
    for (uint32_t i = 1; i < log_size; i++) exp = exp * four;
    QM31 vanishing = QM31::one();
    for (uint32_t i = 1; i < log_size; i++) vanishing = vanishing * coset_vanishing(CanonicCoset(i).coset, p);
    return exp * vanishing;
}
// constraints.rs:87-93
inline QM31 point_vanishing(CirclePoint<M31> vanish_point, CirclePoint<QM31> p) {
    CirclePoint<QM31> h = p + into_ef(vanish_point.conjugate());
    return h.y / (QM31::one() + h.x);
}
// cpu/circle.rs:101-132
inline std::vector<QM31> barycentric_weights(uint32_t log_size, CirclePoint<QM31> p) {
    CircleDomain domain = CanonicCoset(log_size).circle_domain();
    size_t n = domain.size();
    std::vector<QM31> w(n);
    QM31 vn_p = coset_vanishing(CanonicCoset(log_size).coset, p);
#pragma omp parallel for schedule(static) if (n >= 256)
    for (size_t i = 0; i < n; i++) {
        CirclePoint<QM31> cp = into_ef(domain.at(bit_reverse_index(i, log_size)));
        QM31 minus_two_y = cp.y * QM31(M31(P - 2));
        QM31 si = minus_two_y * coset_vanishing_derivative(log_size, cp);
        QM31 vi = point_vanishing(domain.at(bit_reverse_index(i, log_size)), p);
        w[i] = vn_p / (si * vi);
    }
    return w;
}
// cpu/circle.rs:134-141
inline QM31 barycentric_eval_at_point(const std::vector<M31>& evals, const std::vector<QM31>& weights) {
    QM31 acc = QM31::zero();
    for (size_t i = 0; i < evals.size(); i++) acc = acc + weights[i] * evals[i];
    return acc;
}
// cpu/circle.rs:143-180
inline QM31 eval_at_point_by_folding(const std::vector<M31>& evals, CirclePoint<QM31> point) {
    uint32_t log_size = ilog2(evals.size());
    std::vector<QM31> alphas(log_size);  // poly/utils.rs:45-70
    alphas[log_size - 1] = point.y;
    QM31 x = point.x;
    for (uint32_t i = log_size - 1; i-- > 0;) { alphas[i] = x; x = double_x(x); }
    SecureColumn src(evals.size());
    for (size_t i = 0; i < evals.size(); i++) src[i] = QM31(evals[i]);
    SecureColumn layer(evals.size() / 2, QM31::zero());
    fold_circle_into_line(layer, src, CanonicCoset(log_size).circle_domain(), alphas.back());
    alphas.pop_back();
    LineDomain dom{Coset::half_odds(log_size - 1)};
    while (layer.size() > 1) {
        layer = fold_line(layer, dom, alphas.back());
        alphas.pop_back();
        dom = dom.dbl();
    }
    return layer[0] / QM31(M31(1u << log_size));
}

}  // namespace zko
