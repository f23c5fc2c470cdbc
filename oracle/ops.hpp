// TEST INFRASTRUCTURE ONLY (CPU oracle; see fields.hpp).
//
// The per-operator statements of the reference's CpuBackend that the CUDA kernels are checked
// against: FRI folds, quotient numerators / combine, secure-column accumulation, GKR layer ops.
// Secure columns are held here as vectors of QM31; the C API converts to the 4-coordinate layout.
//   nitroo/crates/stwo/src/prover/backend/cpu/fri.rs:67-123          (fold_line_cpu, fold_circle_into_line_cpu)
//   nitroo/crates/stwo/src/core/pcs/quotients.rs:217-304             (partial numerators, line coeffs, denominators)
//   nitroo/crates/stwo/src/core/constraints.rs:119-134               (complex_conjugate_line_coeffs)
//   nitroo/crates/stwo/src/prover/backend/cpu/quotients.rs:22-75     (accumulate_numerators, compute_quotients_and_combine)
//   nitroo/crates/stwo/src/prover/backend/cpu/accumulation.rs:9-48   (accumulate, powers, lift_and_accumulate)
//   nitroo/crates/stwo/src/prover/backend/cpu/lookups/gkr.rs:17-263  (gen_eq_evals, next_layer, round sums)
//   nitroo/crates/stwo/src/prover/backend/cpu/lookups/mle.rs:13-46   (fix_first_variable)
//   nitroo/crates/stwo/src/prover/lookups/utils.rs:26-54, 165-186    (Lagrange interpolation, horner, eq, fold_mle_evals)
//   nitroo/crates/stwo/src/prover/lookups/gkr_prover.rs:884-923      (correct_sum_as_poly_in_first_variable)
#pragma once
#include "accel.hpp"
#include "poly.hpp"

namespace zko {

using SecureColumn = std::vector<QM31>;

// ---------------------------------------------------------------- domain tables for the timed baseline
// The scalar statements below take every domain point by a scalar multiplication on the circle (Coset::at), as
// CpuBackend does. The reference's SIMD backend walks domains incrementally instead (simd/domain.rs:14-60,
// simd/fri.rs:27-116, simd/quotients.rs:73-164); when the packed restatement is switched on, the three functions that
// need a point per row take it from these tables: the coset's points by repeated addition of its step, inverted in
// one batch (core/fields/mod.rs batch_inverse). Same values, same results.
inline std::vector<CirclePoint<M31>> coset_points_natural(const Coset& c) {
    size_t n = c.size();
    std::vector<CirclePoint<M31>> pts(n);
    size_t chunk = n < 4096 ? n : 4096;
#pragma omp parallel for schedule(static)
    for (size_t a = 0; a < n; a += chunk) {
        CirclePoint<M31> p = c.at(a);
        for (size_t k = a; k < a + chunk && k < n; k++) { pts[k] = p; p = p + c.step; }
    }
    return pts;
}
inline void batch_inverse_in_place(std::vector<M31>& v) {
    size_t n = v.size(), chunk = 1024;
#pragma omp parallel for schedule(static)
    for (size_t a = 0; a < n; a += chunk) {
        size_t b = a + chunk < n ? a + chunk : n;
        std::vector<M31> pre(b - a);
        M31 run(1);
        for (size_t k = a; k < b; k++) { pre[k - a] = run; run = run * v[k]; }
        M31 inv = run.inverse();
        for (size_t k = b; k-- > a;) { M31 x = v[k]; v[k] = inv * pre[k - a]; inv = inv * x; }
    }
}
inline size_t fast_bit_reverse(size_t i, uint32_t log_size) {
    if (!log_size) return i;
    uint32_t x = (uint32_t)i;
    x = ((x >> 1) & 0x55555555u) | ((x & 0x55555555u) << 1);
    x = ((x >> 2) & 0x33333333u) | ((x & 0x33333333u) << 2);
    x = ((x >> 4) & 0x0f0f0f0fu) | ((x & 0x0f0f0f0fu) << 4);
    x = __builtin_bswap32(x);
    return (size_t)(x >> (32 - log_size));
}

// ---------------------------------------------------------------- FRI folds
// cpu/fri.rs:67-92. `eval` lives on `domain` (bit-reversed); the result lives on domain.dbl().
inline SecureColumn fold_line(const SecureColumn& eval, const LineDomain& domain, QM31 alpha) {
    size_t n = eval.size();
    assert(n >= 2);
    SecureColumn out(n / 2);
    if (accel().lanes && n >= 64) {
        auto pts = coset_points_natural(domain.coset);
        std::vector<M31> xi(n / 2);
        for (size_t i = 0; i < n / 2; i++) xi[i] = pts[fast_bit_reverse(i << 1, domain.log_size())].x;
        batch_inverse_in_place(xi);
#pragma omp parallel for schedule(static)
        for (size_t i = 0; i < n / 2; i++) {
            QM31 f0 = eval[2 * i], f1 = eval[2 * i + 1];
            ibutterfly(f0, f1, xi[i]);
            out[i] = f0 + alpha * f1;
        }
        return out;
    }
#pragma omp parallel for schedule(static) if (n >= 4096)
    for (size_t i = 0; i < n / 2; i++) {
        M31 x = domain.at(bit_reverse_index(i << 1, domain.log_size()));
        QM31 f0 = eval[2 * i], f1 = eval[2 * i + 1];
        ibutterfly(f0, f1, x.inverse());
        out[i] = f0 + alpha * f1;
    }
    return out;
}
// cpu/fri.rs:95-123
inline void fold_circle_into_line(SecureColumn& dst, const SecureColumn& src, const CircleDomain& domain, QM31 alpha) {
    assert(src.size() >> 1 == dst.size());
    QM31 alpha_sq = alpha * alpha;
    if (accel().lanes && dst.size() >= 64) {
        // rows 2i of the bit-reversed circle domain are the half coset's points in bit-reversed order
        auto pts = coset_points_natural(domain.half_coset);
        std::vector<M31> yi(dst.size());
        for (size_t i = 0; i < dst.size(); i++) {
            size_t j = fast_bit_reverse(i << 1, domain.log_size());
            yi[i] = j < pts.size() ? pts[j].y : -pts[j - pts.size()].y;
        }
        batch_inverse_in_place(yi);
#pragma omp parallel for schedule(static)
        for (size_t i = 0; i < dst.size(); i++) {
            QM31 f0 = src[2 * i], f1 = src[2 * i + 1];
            ibutterfly(f0, f1, yi[i]);
            dst[i] = dst[i] * alpha_sq + (alpha * f1 + f0);
        }
        return;
    }
#pragma omp parallel for schedule(static) if (dst.size() >= 4096)
    for (size_t i = 0; i < dst.size(); i++) {
        CirclePoint<M31> p = domain.at(bit_reverse_index(i << 1, domain.log_size()));
        QM31 f0 = src[2 * i], f1 = src[2 * i + 1];
        ibutterfly(f0, f1, p.y.inverse());
        QM31 f_prime = alpha * f1 + f0;
        dst[i] = dst[i] * alpha_sq + f_prime;
    }
}

// ---------------------------------------------------------------- quotients
struct PointSample { CirclePoint<QM31> point; QM31 value; };
struct NumeratorData { size_t column_index; QM31 sample_value; QM31 random_coeff; };
struct ColumnSampleBatch { CirclePoint<QM31> point; std::vector<NumeratorData> cols_vals_randpows; };
struct LineCoeffs { QM31 a, b, c; };

// constraints.rs:119-134
inline LineCoeffs complex_conjugate_line_coeffs(const PointSample& s, QM31 alpha) {
    assert(!(s.point.y == s.point.y.conj()));
    QM31 a = s.value.conj() - s.value;
    QM31 c = s.point.y.conj() - s.point.y;
    QM31 b = s.value * c - a * s.point.y;
    return {alpha * a, alpha * b, alpha * c};
}
// quotients.rs:229-258
inline std::vector<std::vector<LineCoeffs>> column_line_coeffs(const std::vector<ColumnSampleBatch>& batches) {
    std::vector<std::vector<LineCoeffs>> out;
    for (auto& b : batches) {
        std::vector<LineCoeffs> v;
        for (auto& d : b.cols_vals_randpows)
            v.push_back(complex_conjugate_line_coeffs(PointSample{b.point, d.sample_value}, d.random_coeff));
        out.push_back(v);
    }
    return out;
}
// quotients.rs:263-291 — CM31 line equation through (z, conj z) at the domain point, inverted.
inline std::vector<CM31> denominator_inverses(const std::vector<CirclePoint<QM31>>& pts, CirclePoint<M31> dp) {
    std::vector<CM31> out;
    for (auto& sp : pts) {
        CM31 prx = sp.x.a, pry = sp.y.a, pix = sp.x.b, piy = sp.y.b;
        CM31 den = (prx - CM31(dp.x)) * piy - (pry - CM31(dp.y)) * pix;
        out.push_back(den.inverse());
    }
    return out;
}

struct AccumulatedNumerators {
    CirclePoint<QM31> sample_point;
    SecureColumn partial_numerators_acc;
    QM31 first_linear_term_acc;
};

// cpu/quotients.rs:22-45 with quotients.rs:217-229
inline void accumulate_numerators(const std::vector<const M31*>& columns, size_t size,
                                  const std::vector<ColumnSampleBatch>& batches,
                                  std::vector<AccumulatedNumerators>& out) {
    auto coeffs = column_line_coeffs(batches);
    for (size_t bi = 0; bi < batches.size(); bi++) {
        SecureColumn acc(size);
        if (accel().numerators && size >= 16) {  // 16 rows per step (simd.hpp); sum_j (c_j v_j - b_j) = sum_j c_j v_j - sum_j b_j
            std::vector<const uint32_t*> cp;
            for (auto c : columns) cp.push_back(&c->v);
            std::vector<size_t> idx;
            std::vector<QM31> cs;
            QM31 b_sum = QM31::zero();
            for (size_t j = 0; j < batches[bi].cols_vals_randpows.size(); j++) {
                idx.push_back(batches[bi].cols_vals_randpows[j].column_index);
                cs.push_back(coeffs[bi][j].c);
                b_sum = b_sum + coeffs[bi][j].b;
            }
            accel().numerators(reinterpret_cast<uint32_t*>(acc.data()), cp.data(), idx.data(), cs.data(), idx.size(), b_sum, size);
            QM31 first = QM31::zero();
            for (auto& lc : coeffs[bi]) first = first + lc.a;
            out.push_back({batches[bi].point, acc, first});
            continue;
        }
#pragma omp parallel for schedule(static) if (size >= 4096)
        for (size_t row = 0; row < size; row++) {
            QM31 numerator = QM31::zero();
            for (size_t j = 0; j < batches[bi].cols_vals_randpows.size(); j++) {
                QM31 value = coeffs[bi][j].c * columns[batches[bi].cols_vals_randpows[j].column_index][row];
                numerator = numerator + (value - coeffs[bi][j].b);
            }
            acc[row] = numerator;
        }
        QM31 first = QM31::zero();
        for (auto& lc : coeffs[bi]) first = first + lc.a;
        out.push_back({batches[bi].point, acc, first});
    }
}

// cpu/quotients.rs:47-75
inline SecureColumn compute_quotients_and_combine(const std::vector<AccumulatedNumerators>& accs, uint32_t lifting_log_size) {
    CircleDomain domain = CanonicCoset(lifting_log_size).circle_domain();
    size_t n = (size_t)1 << lifting_log_size;
    SecureColumn q(n);
    std::vector<CirclePoint<QM31>> pts;
    for (auto& a : accs) pts.push_back(a.sample_point);
    std::vector<CirclePoint<M31>> table;
    if (accel().lanes && n >= 64) table = coset_points_natural(domain.half_coset);
#pragma omp parallel for schedule(static) if (n >= 4096)
    for (size_t row = 0; row < n; row++) {
        CirclePoint<M31> dp;
        if (!table.empty()) {
            size_t j = fast_bit_reverse(row, lifting_log_size);
            dp = j < table.size() ? table[j] : table[j - table.size()].conjugate();
        } else {
            dp = domain.at(bit_reverse_index(row, lifting_log_size));
        }
        auto inv = denominator_inverses(pts, dp);
        QM31 quotient = QM31::zero();
        for (size_t k = 0; k < accs.size(); k++) {
            uint32_t log_ratio = lifting_log_size - ilog2(accs[k].partial_numerators_acc.size());
            size_t lifted = ((row >> (log_ratio + 1)) << 1) + (row & 1);
            QM31 full = accs[k].partial_numerators_acc[lifted] - accs[k].first_linear_term_acc * dp.y;
            quotient = quotient + full.mul_cm31(inv[k]);
        }
        q[row] = quotient;
    }
    return q;
}

// ---------------------------------------------------------------- accumulation
// cpu/accumulation.rs:9-15
inline void accumulate(SecureColumn& col, const SecureColumn& other) {
    for (size_t i = 0; i < col.size(); i++) col[i] = col[i] + other[i];
}
// cpu/accumulation.rs:17-25
inline std::vector<QM31> generate_secure_powers(QM31 felt, size_t n) {
    std::vector<QM31> out;
    QM31 acc = QM31::one();
    for (size_t i = 0; i < n; i++) { out.push_back(acc); acc = acc * felt; }
    return out;
}
// cpu/accumulation.rs:27-48 — columns ascending in size; each is added the lift of the running sum.
inline SecureColumn lift_and_accumulate(std::vector<SecureColumn> cols) {
    assert(!cols.empty() && cols[0].size() >= 2);
    SecureColumn curr(2, QM31::zero());
    for (auto& col : cols) {
        uint32_t log_ratio = ilog2(col.size()) - ilog2(curr.size());
        for (size_t i = 0; i < col.size(); i++) col[i] = col[i] + curr[((i >> (log_ratio + 1)) << 1) + (i & 1)];
        curr = col;
    }
    return curr;
}

// ---------------------------------------------------------------- GKR / MLE
// lookups/utils.rs:165-186
inline QM31 eq1(QM31 x, QM31 y) { return x * y + (QM31::one() - x) * (QM31::one() - y); }
inline QM31 eq(const QM31* x, const QM31* y, size_t n) {
    QM31 r = QM31::one();
    for (size_t i = 0; i < n; i++) r = r * eq1(x[i], y[i]);
    return r;
}
inline QM31 horner_eval(const std::vector<QM31>& c, QM31 x) {
    QM31 acc = QM31::zero();
    for (size_t i = c.size(); i-- > 0;) acc = acc * x + c[i];
    return acc;
}
inline QM31 fold_mle_evals(QM31 r, QM31 e0, QM31 e1) { return r * (e1 - e0) + e0; }

// cpu/lookups/gkr.rs:216-231
inline std::vector<QM31> gen_eq_evals(const QM31* y, size_t ny, QM31 v) {
    std::vector<QM31> evals;
    evals.reserve((size_t)1 << ny);
    evals.push_back(v);
    for (size_t k = ny; k-- > 0;) {
        size_t len = evals.size();
        for (size_t j = 0; j < len; j++) {
            QM31 tmp = evals[j] * y[k];
            evals.push_back(tmp);
            evals[j] = evals[j] - tmp;
        }
    }
    return evals;
}

enum LayerKind { GRAND_PRODUCT = 0, LOGUP_GENERIC = 1, LOGUP_MULTIPLICITIES = 2, LOGUP_SINGLES = 3 };
struct Layer {
    LayerKind kind;
    std::vector<QM31> num;      // LOGUP_GENERIC numerators
    std::vector<M31> num_base;  // LOGUP_MULTIPLICITIES numerators
    std::vector<QM31> den;      // denominators, or the GRAND_PRODUCT column
    size_t len() const { return den.size(); }
    size_t n_variables() const { return ilog2(den.size()); }
    QM31 numerator_at(size_t i) const {
        switch (kind) {
            case LOGUP_GENERIC: return num[i];
            case LOGUP_MULTIPLICITIES: return QM31(num_base[i]);
            default: return QM31::one();
        }
    }
};

// cpu/lookups/gkr.rs:22-37, 233-263; fraction add core/fraction.rs:24-33
inline Layer next_layer(const Layer& l) {
    size_t half = l.len() / 2;
    Layer out;
    if (l.kind == GRAND_PRODUCT) {
        out.kind = GRAND_PRODUCT;
        out.den.resize(half);
        for (size_t i = 0; i < half; i++) out.den[i] = l.den[2 * i] * l.den[2 * i + 1];
        return out;
    }
    out.kind = LOGUP_GENERIC;
    out.num.resize(half);
    out.den.resize(half);
    for (size_t i = 0; i < half; i++) {
        QM31 d0 = l.den[2 * i], d1 = l.den[2 * i + 1];
        QM31 n;
        if (l.kind == LOGUP_MULTIPLICITIES) n = d1 * l.num_base[2 * i] + d0 * l.num_base[2 * i + 1];
        else n = d1 * l.numerator_at(2 * i) + d0 * l.numerator_at(2 * i + 1);
        out.num[i] = n;
        out.den[i] = d0 * d1;
    }
    return out;
}

// cpu/lookups/mle.rs:13-46
inline std::vector<QM31> fix_first_variable(const std::vector<QM31>& mle, QM31 r) {
    size_t mid = mle.size() / 2;
    std::vector<QM31> out(mid);
    for (size_t i = 0; i < mid; i++) out[i] = fold_mle_evals(r, mle[i], mle[i + mid]);
    return out;
}
inline std::vector<QM31> fix_first_variable(const std::vector<M31>& mle, QM31 r) {
    size_t mid = mle.size() / 2;
    std::vector<QM31> out(mid);
    for (size_t i = 0; i < mid; i++) out[i] = r * (mle[i + mid] - mle[i]) + mle[i];
    return out;
}
// gkr_prover.rs:354-381 — LogUpMultiplicities becomes LogUpGeneric once a variable is fixed.
inline Layer layer_fix_first_variable(const Layer& l, QM31 x0) {
    if (l.n_variables() == 0) return l;
    Layer out;
    out.den = fix_first_variable(l.den, x0);
    switch (l.kind) {
        case GRAND_PRODUCT: out.kind = GRAND_PRODUCT; break;
        case LOGUP_GENERIC: out.kind = LOGUP_GENERIC; out.num = fix_first_variable(l.num, x0); break;
        case LOGUP_MULTIPLICITIES: out.kind = LOGUP_GENERIC; out.num = fix_first_variable(l.num_base, x0); break;
        case LOGUP_SINGLES: out.kind = LOGUP_SINGLES; break;
    }
    return out;
}

// cpu/lookups/gkr.rs:73-213 — (eval at t=0, eval at t=2) of sum_x eq * (numerator + lambda * denominator),
// before the eq correction.
inline void round_sums(const Layer& l, const QM31* eq_evals, size_t n_terms, QM31 lambda, QM31& at0, QM31& at2) {
    at0 = QM31::zero();
    at2 = QM31::zero();
    for (size_t i = 0; i < n_terms; i++) {
        if (l.kind == GRAND_PRODUCT) {
            QM31 a00 = l.den[i * 2], a01 = l.den[i * 2 + 1];
            QM31 a10 = l.den[(n_terms + i) * 2], a11 = l.den[(n_terms + i) * 2 + 1];
            QM31 a20 = a10.dbl() - a00, a21 = a11.dbl() - a01;
            at0 = at0 + eq_evals[i] * (a00 * a01);
            at2 = at2 + eq_evals[i] * (a20 * a21);
            continue;
        }
        QM31 d00 = l.den[i * 2], d01 = l.den[i * 2 + 1];
        QM31 d10 = l.den[(n_terms + i) * 2], d11 = l.den[(n_terms + i) * 2 + 1];
        QM31 d20 = d10.dbl() - d00, d21 = d11.dbl() - d01;
        QM31 num0, num2;
        if (l.kind == LOGUP_SINGLES) {
            num0 = d00 + d01;
            num2 = d20 + d21;
        } else if (l.kind == LOGUP_MULTIPLICITIES) {
            M31 n00 = l.num_base[i * 2], n01 = l.num_base[i * 2 + 1];
            M31 n10 = l.num_base[(n_terms + i) * 2], n11 = l.num_base[(n_terms + i) * 2 + 1];
            M31 n20 = n10.dbl() - n00, n21 = n11.dbl() - n01;
            num0 = d01 * n00 + d00 * n01;
            num2 = d21 * n20 + d20 * n21;
        } else {
            QM31 n00 = l.num[i * 2], n01 = l.num[i * 2 + 1];
            QM31 n10 = l.num[(n_terms + i) * 2], n11 = l.num[(n_terms + i) * 2 + 1];
            QM31 n20 = n10.dbl() - n00, n21 = n11.dbl() - n01;
            num0 = d01 * n00 + d00 * n01;
            num2 = d21 * n20 + d20 * n21;
        }
        at0 = at0 + eq_evals[i] * (num0 + lambda * (d00 * d01));
        at2 = at2 + eq_evals[i] * (num2 + lambda * (d20 * d21));
    }
}

// lookups/utils.rs:12-146 — dense univariate polynomial, low coefficient first, leading zeros dropped.
struct UnivariatePoly {
    std::vector<QM31> c;
    void trim() { while (!c.empty() && c.back().is_zero()) c.pop_back(); }
    QM31 eval(QM31 x) const { return horner_eval(c, x); }
    size_t degree() const { size_t n = c.size(); while (n && c[n - 1].is_zero()) n--; return n ? n - 1 : 0; }
    static UnivariatePoly mul(UnivariatePoly a, UnivariatePoly b) {
        a.trim(); b.trim();
        if (a.c.empty() || b.c.empty()) return {};
        UnivariatePoly r;
        r.c.assign(a.c.size() + b.c.size() - 1, QM31::zero());
        for (size_t i = 0; i < a.c.size(); i++)
            for (size_t j = 0; j < b.c.size(); j++) r.c[i + j] = r.c[i + j] + a.c[i] * b.c[j];
        r.trim();
        return r;
    }
    static UnivariatePoly add(const UnivariatePoly& a, const UnivariatePoly& b) {
        UnivariatePoly r;
        size_t n = std::max(a.c.size(), b.c.size());
        for (size_t i = 0; i < n; i++) {
            QM31 x = i < a.c.size() ? a.c[i] : QM31::zero();
            QM31 y = i < b.c.size() ? b.c[i] : QM31::zero();
            r.c.push_back(x + y);
        }
        return r;
    }
    // lookups/utils.rs:26-54
    static UnivariatePoly interpolate_lagrange(const std::vector<QM31>& xs, const std::vector<QM31>& ys) {
        UnivariatePoly coeffs;
        for (size_t i = 0; i < xs.size(); i++) {
            QM31 prod = ys[i];
            for (size_t j = 0; j < xs.size(); j++)
                if (i != j) prod = prod / (xs[i] - xs[j]);
            UnivariatePoly term;
            term.c = {prod};
            term.trim();
            for (size_t j = 0; j < xs.size(); j++)
                if (i != j) {
                    UnivariatePoly lin;
                    lin.c = {-xs[j], QM31::one()};
                    term = mul(term, lin);
                }
            coeffs = add(coeffs, term);
        }
        coeffs.trim();
        return coeffs;
    }
};

// gkr_prover.rs:884-923
inline UnivariatePoly correct_sum_as_poly_in_first_variable(QM31 f_at_0, QM31 f_at_2, QM31 claim,
                                                            const std::vector<QM31>& y, size_t k) {
    size_t n = y.size();
    assert(k != 0 && k <= n);
    std::vector<QM31> zeros(n - k + 1, QM31::zero());
    QM31 a_const = eq(zeros.data(), y.data(), n - k + 1).inverse();
    QM31 b_const = (QM31::one() - y[n - k]) / (QM31::one() - y[n - k].dbl());
    QM31 two = QM31(M31(2));
    QM31 r_at_0 = f_at_0 * eq1(QM31::zero(), y[n - k]) * a_const;
    QM31 r_at_1 = claim - r_at_0;
    QM31 r_at_2 = f_at_2 * eq1(two, y[n - k]) * a_const;
    return UnivariatePoly::interpolate_lagrange({QM31::zero(), QM31::one(), two, b_const},
                                                {r_at_0, r_at_1, r_at_2, QM31::zero()});
}

}  // namespace zko
