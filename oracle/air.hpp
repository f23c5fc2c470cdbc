// TEST INFRASTRUCTURE ONLY (CPU oracle; see fields.hpp).
//
// Constraint-quotient evaluation on the evaluation domain, as the reference's CPU backend states it:
//   nitroo/crates/constraint-framework/src/prover/component_prover.rs:206-294  (ComponentProver<CpuBackend>)
//   nitroo/crates/constraint-framework/src/prover/component_prover.rs:603-633  (accumulate_pointwise_cpu)
//   nitroo/crates/constraint-framework/src/prover/cpu_domain.rs:17-98          (CpuDomainEvaluator)
//   nitroo/crates/constraint-framework/src/lib.rs:70-199, 214-290              (EvalAtRow, the LogUp proxy)
//   nitroo/crates/constraint-framework/src/logup.rs:15-104                     (LogupAtRow, LookupElements::combine)
//   nitroo/crates/stwo/src/core/utils.rs:97-113                                (mask offset in bit-reversed order)
//   nitroo/crates/stwo/src/core/constraints.rs:12-35                           (coset_vanishing)
//   nitroo/crates/stwo/src/core/fraction.rs:20-60                              (Fraction add / sum)
// Two independent routes to the same numbers:
//   (1) AIRs written directly against CpuDomainEvaluator, as their `evaluate` functions are in the reference:
//       wide Fibonacci (nitroo/crates/examples/src/wide_fibonacci/mod.rs:47-57), Plonk
//       (nitroo/crates/examples/src/plonk/mod.rs:51-88), the Freivalds component
//       (prover/src/gadgets/freivalds/mod.rs:114-186);
//   (2) an interpreter of the single-assignment lowering, as prover/src/cudagen.rs:1217-1262 interprets its `Ir`.
#pragma once
#include <cstring>
#include <vector>

#include "circle.hpp"

namespace zko {

constexpr int PREPROCESSED_TRACE_IDX = 0, MODEL_TRACE_IDX = 1, ORIGINAL_TRACE_IDX = 2, INTERACTION_TRACE_IDX = 3;  // lib.rs:40-58

// core/utils.rs:97-113
inline size_t offset_bit_reversed_circle_domain_index(size_t i, uint32_t domain_log_size, uint32_t eval_log_size, int64_t offset) {
    int64_t prev_index = (int64_t)bit_reverse_index(i, eval_log_size);
    const int64_t half_size = (int64_t)1 << (eval_log_size - 1);
    const int64_t step_size = offset * ((int64_t)1 << (eval_log_size - domain_log_size - 1));
    auto rem_euclid = [](int64_t a, int64_t m) { int64_t r = a % m; return r < 0 ? r + m : r; };
    if (prev_index < half_size) prev_index = rem_euclid(prev_index + step_size, half_size);
    else prev_index = rem_euclid(prev_index - step_size, half_size) + half_size;
    return bit_reverse_index((size_t)prev_index, eval_log_size);
}

// core/constraints.rs:12-35
inline M31 coset_vanishing(const Coset& coset, CirclePoint<M31> p) {
    CirclePointIndex half_step{coset.step_size.i >> 1};
    p = p + coset.initial.conjugate() + half_step.to_point();  // p - initial + step/2
    M31 x = p.x;
    for (uint32_t k = 1; k < coset.log_size; k++) x = double_x(x);
    return x;
}

// component_prover.rs:262-266
inline std::vector<M31> constraint_denom_inv(uint32_t trace_log, uint32_t eval_log) {
    CircleDomain eval_domain = CanonicCoset(eval_log).circle_domain();
    Coset trace_coset = CanonicCoset(trace_log).coset;
    const uint32_t log_expand = eval_log - trace_log;
    std::vector<M31> d((size_t)1 << log_expand);
    for (size_t i = 0; i < d.size(); i++) d[i] = coset_vanishing(trace_coset, eval_domain.at(i)).inverse();
    bit_reverse(d.data(), d.size());
    return d;
}

using TraceView = std::vector<std::vector<const uint32_t*>>;  // [interaction][column] -> 2^eval_log words

// What lifts a base-field value or a secure-field constant into an evaluator's fields.
inline QM31 to_ef(M31 x) { return QM31(x); }
inline QM31 to_ef(QM31 x) { return x; }
template <class F> inline F from_m31(M31 x);
template <> inline M31 from_m31<M31>(M31 x) { return x; }
template <> inline QM31 from_m31<QM31>(M31 x) { return QM31(x); }
inline M31 square(M31 x) { return x.square(); }
inline QM31 square(QM31 x) { return x.square(); }

template <class EF> struct FractionT {
    EF numerator, denominator;
    FractionT operator+(const FractionT& r) const {  // fraction.rs:27-33
        return {r.denominator * numerator + denominator * r.numerator, denominator * r.denominator};
    }
};

// logup.rs:62-104
struct LookupElements {
    QM31 z;
    std::vector<QM31> alpha_powers;
    template <class F> QM31 combine(const std::vector<F>& values) const {
        assert(alpha_powers.size() >= values.size());
        QM31 acc = QM31::zero();
        for (size_t i = 0; i < values.size(); i++) acc = acc + alpha_powers[i] * values[i];
        return acc - z;
    }
};

// The part of EvalAtRow every evaluator shares (lib.rs:70-199) with the LogUp proxy (lib.rs:214-290). Derived supplies
//   std::vector<F> mask(interaction, column, offsets), void add_constraint(EF) (and add_constraint(F) where F != EF),
//   static EF combine_ef(F, F, F, F).
template <class Derived, class F_, class EF_> struct EvalAtRowBase {
    using F = F_;
    using EF = EF_;
    std::vector<size_t> column_index_per_interaction;
    int logup_interaction = INTERACTION_TRACE_IDX;
    QM31 cumsum_shift;  // LogupAtRow::new, logup.rs:33-41
    std::vector<FractionT<EF>> fracs;

    EvalAtRowBase(size_t n_interactions, QM31 claimed_sum, uint32_t log_size)
        : column_index_per_interaction(n_interactions, 0), cumsum_shift(claimed_sum * QM31(M31((uint32_t)1 << log_size)).inverse()) {}
    Derived& self() { return static_cast<Derived&>(*this); }

    std::vector<F> next_interaction_mask(int interaction, const std::vector<int>& offsets) {
        size_t col = column_index_per_interaction[interaction]++;
        return self().mask(interaction, col, offsets);
    }
    F next_trace_mask() { return next_interaction_mask(ORIGINAL_TRACE_IDX, {0})[0]; }
    F get_preprocessed_column() { return next_interaction_mask(PREPROCESSED_TRACE_IDX, {0})[0]; }
    // lib.rs:127-137: four consecutive columns, combined per offset
    std::vector<EF> next_extension_interaction_mask(int interaction, const std::vector<int>& offsets) {
        std::vector<F> c[4];
        for (int k = 0; k < 4; k++) c[k] = next_interaction_mask(interaction, offsets);
        std::vector<EF> out;
        for (size_t j = 0; j < offsets.size(); j++) out.push_back(Derived::combine_ef(c[0][j], c[1][j], c[2][j], c[3][j]));
        return out;
    }
    // lib.rs:169-180
    void add_to_relation(const LookupElements& rel, EF multiplicity, const std::vector<F>& values) {
        fracs.push_back({multiplicity, rel.combine(values)});
    }
    // lib.rs:226-275
    void finalize_logup_batched(const std::vector<size_t>& batching) {
        assert(batching.size() == fracs.size());
        size_t last_batch = 0;
        for (size_t b : batching) last_batch = b > last_batch ? b : last_batch;
        std::vector<std::vector<FractionT<EF>>> by_batch(last_batch + 1);
        for (size_t i = 0; i < batching.size(); i++) by_batch[batching[i]].push_back(fracs[i]);
        auto sum = [](const std::vector<FractionT<EF>>& v) {  // fraction.rs:56-59
            FractionT<EF> acc = v[0];
            for (size_t i = 1; i < v.size(); i++) acc = acc + v[i];
            return acc;
        };
        EF prev_col_cumsum = QM31::zero();
        for (size_t b = 0; b < last_batch; b++) {
            FractionT<EF> cur = sum(by_batch[b]);
            EF cur_cumsum = next_extension_interaction_mask(logup_interaction, {0})[0];
            EF diff = cur_cumsum - prev_col_cumsum;
            prev_col_cumsum = cur_cumsum;
            self().add_constraint(diff * cur.denominator - cur.numerator);
        }
        FractionT<EF> frac = sum(by_batch[last_batch]);
        std::vector<EF> m = next_extension_interaction_mask(logup_interaction, {-1, 0});
        EF diff = m[1] - m[0] - prev_col_cumsum;
        EF shifted = diff + cumsum_shift;
        self().add_constraint(shifted * frac.denominator - frac.numerator);
        fracs.clear();
    }
    void finalize_logup() {
        std::vector<size_t> b(fracs.size());
        for (size_t i = 0; i < b.size(); i++) b[i] = i;
        finalize_logup_batched(b);
    }
    void finalize_logup_in_pairs() {
        std::vector<size_t> b(fracs.size());
        for (size_t i = 0; i < b.size(); i++) b[i] = i / 2;
        finalize_logup_batched(b);
    }
};

// cpu_domain.rs:17-98
struct CpuDomainEvaluator : EvalAtRowBase<CpuDomainEvaluator, M31, QM31> {
    const TraceView& trace_eval;
    size_t row;
    const QM31* random_coeff_powers;
    QM31 row_res = QM31::zero();
    size_t constraint_index = 0;
    uint32_t domain_log_size, eval_domain_log_size;

    CpuDomainEvaluator(const TraceView& t, size_t row_, const QM31* rcp, uint32_t domain_log, uint32_t eval_log, uint32_t log_size,
                       QM31 claimed_sum)
        : EvalAtRowBase(t.size(), claimed_sum, log_size), trace_eval(t), row(row_), random_coeff_powers(rcp), domain_log_size(domain_log),
          eval_domain_log_size(eval_log) {}
    std::vector<M31> mask(int interaction, size_t col_index, const std::vector<int>& offsets) {
        const uint32_t* col = trace_eval[interaction][col_index];
        std::vector<M31> out;
        for (int off : offsets) {
            if (off == 0) { out.push_back(M31(col[row])); continue; }
            size_t r = offset_bit_reversed_circle_domain_index(row, domain_log_size, eval_domain_log_size, off);
            out.push_back(M31(col[r]));
        }
        return out;
    }
    void add_constraint(QM31 c) { row_res = row_res + random_coeff_powers[constraint_index++] * c; }
    void add_constraint(M31 c) { row_res = row_res + random_coeff_powers[constraint_index++] * c; }
    static QM31 combine_ef(M31 a, M31 b, M31 c, M31 d) { return QM31::from_m31s(a, b, c, d); }
};

// qm31.rs:51-57
inline QM31 from_partial_evals(QM31 e0, QM31 e1, QM31 e2, QM31 e3) {
    return e0 + e1 * QM31::from_u32(0, 1, 0, 0) + e2 * QM31::from_u32(0, 0, 1, 0) + e3 * QM31::from_u32(0, 0, 0, 1);
}

// point.rs:14-80 with PointEvaluationAccumulator (core/air/accumulation.rs:12-36)
struct PointEvaluator : EvalAtRowBase<PointEvaluator, QM31, QM31> {
    const std::vector<std::vector<std::vector<QM31>>>& mask_values;  // [interaction][column][k]
    QM31 random_coeff, denom_inverse;
    QM31 accumulation = QM31::zero();
    size_t n_constraints = 0;
    PointEvaluator(const std::vector<std::vector<std::vector<QM31>>>& m, QM31 random_coeff_, QM31 denom_inverse_, uint32_t log_size,
                   QM31 claimed_sum)
        : EvalAtRowBase(m.size(), claimed_sum, log_size), mask_values(m), random_coeff(random_coeff_), denom_inverse(denom_inverse_) {}
    std::vector<QM31> mask(int interaction, size_t col_index, const std::vector<int>& offsets) {
        const std::vector<QM31>& v = mask_values[interaction][col_index];
        assert(v.size() == offsets.size());
        return v;
    }
    void add_constraint(QM31 c) {
        accumulation = accumulation * random_coeff + denom_inverse * c;
        n_constraints++;
    }
    static QM31 combine_ef(QM31 a, QM31 b, QM31 c, QM31 d) { return from_partial_evals(a, b, c, d); }
};

// info.rs: which mask offsets each column is asked for, and how many constraints there are
struct InfoEvaluator : EvalAtRowBase<InfoEvaluator, QM31, QM31> {
    std::vector<std::vector<std::vector<int>>> mask_offsets;  // [interaction][column] -> offsets
    size_t n_constraints = 0;
    explicit InfoEvaluator(size_t n_interactions) : EvalAtRowBase(n_interactions, QM31::zero(), 1), mask_offsets(n_interactions) {}
    std::vector<QM31> mask(int interaction, size_t col_index, const std::vector<int>& offsets) {
        if (mask_offsets[interaction].size() <= col_index) mask_offsets[interaction].resize(col_index + 1);
        mask_offsets[interaction][col_index] = offsets;
        return std::vector<QM31>(offsets.size(), QM31::one());
    }
    void add_constraint(QM31) { n_constraints++; }
    static QM31 combine_ef(QM31 a, QM31, QM31, QM31) { return a; }
};

// ---------------------------------------------------------------------------------------------- AIRs, written as in the reference

// nitroo/crates/examples/src/wide_fibonacci/mod.rs:47-57
template <class E> inline void wide_fibonacci_evaluate(E& eval, size_t n_cols) {
    auto a = eval.next_trace_mask(), b = eval.next_trace_mask();
    for (size_t k = 2; k < n_cols; k++) {
        auto c = eval.next_trace_mask();
        eval.add_constraint(c - (square(a) + square(b)));
        a = b;
        b = c;
    }
}

// nitroo/crates/examples/src/plonk/mod.rs:51-88
template <class E> inline void plonk_evaluate(E& eval, const LookupElements& lookup) {
    using F = typename E::F;
    F a_wire = eval.get_preprocessed_column(), b_wire = eval.get_preprocessed_column();
    F c_wire = eval.get_preprocessed_column(), op = eval.get_preprocessed_column();
    F mult = eval.next_trace_mask(), a_val = eval.next_trace_mask(), b_val = eval.next_trace_mask(), c_val = eval.next_trace_mask();
    eval.add_constraint(c_val - op * (a_val + b_val) + (from_m31<F>(M31(1)) - op) * a_val * b_val);
    eval.add_to_relation(lookup, QM31::one(), {a_wire, a_val});
    eval.add_to_relation(lookup, QM31::one(), {b_wire, b_val});
    eval.add_to_relation(lookup, to_ef(-mult), {c_wire, c_val});
    eval.finalize_logup_in_pairs();
}

// prover/src/gadgets/freivalds/mod.rs:62-96 (the fields `evaluate` reads; the optional activation claim is absent)
struct FreivaldsEval {
    size_t pk, pq, n_mats;
    std::vector<QM31> rv_pow;
    QM31 rv_step;
    std::vector<QM31> s_pow;
    QM31 s_step;
    std::vector<QM31> claimed;
    LookupElements rel_act;
    uint32_t act_off;
    bool range_check;
};
// prover/src/gadgets/freivalds/mod.rs:114-186
template <class E> inline void freivalds_evaluate(E& eval, const FreivaldsEval& e) {
    using F = typename E::F;
    F nofirst = eval.get_preprocessed_column(), last = eval.get_preprocessed_column();
    F notzero = eval.get_preprocessed_column(), end = eval.get_preprocessed_column();
    std::vector<std::vector<F>> ws(e.n_mats);
    for (size_t m = 0; m < e.n_mats; m++)
        for (size_t p = 0; p < e.pk; p++) ws[m].push_back(eval.get_preprocessed_column());
    std::vector<F> acts;
    for (size_t p = 0; p < e.pq; p++) acts.push_back(eval.next_trace_mask());
    std::vector<QM31> vv = eval.next_extension_interaction_mask(INTERACTION_TRACE_IDX, {-1, 0});
    QM31 v_prev = vv[0], v = vv[1];
    QM31 vf = QM31::zero();
    for (size_t p = 0; p < e.pq; p++) vf = vf + e.s_pow[p] * acts[p];
    QM31 off_sum = QM31::zero();
    for (const QM31& s : e.s_pow) off_sum = off_sum + s;
    off_sum = off_sum * QM31::from_u32(e.act_off, 0, 0, 0);
    vf = vf - off_sum;
    eval.add_constraint(v - (v_prev * e.s_step) * nofirst - vf);
    for (size_t m = 0; m < e.n_mats; m++) {
        std::vector<QM31> uu = eval.next_extension_interaction_mask(INTERACTION_TRACE_IDX, {-1, 0});
        std::vector<QM31> aa = eval.next_extension_interaction_mask(INTERACTION_TRACE_IDX, {-1, 0});
        QM31 uf = QM31::zero();
        for (size_t p = 0; p < e.pk; p++) uf = uf + e.rv_pow[p] * ws[m][p];
        eval.add_constraint(uu[1] - (uu[0] * e.rv_step) * nofirst - uf);
        eval.add_constraint(aa[1] - aa[0] * notzero - (uu[1] * v) * last);
        eval.add_constraint((aa[1] - e.claimed[m]) * end);
    }
    if (e.range_check) {
        for (F a : acts) eval.add_to_relation(e.rel_act, QM31::one(), {a});
        eval.finalize_logup_in_pairs();
    }
}

// The three AIRs above behind one description (what the C entry points take).
struct AirSpec {
    int air = 0;  // 0 wide Fibonacci, 1 Plonk, 2 Freivalds
    size_t n_cols = 0;
    LookupElements plonk_rel;
    FreivaldsEval fe{};
    template <class E> void evaluate(E& eval) const {
        if (air == 0) wide_fibonacci_evaluate(eval, n_cols);
        else if (air == 1) plonk_evaluate(eval, plonk_rel);
        else freivalds_evaluate(eval, fe);
    }
};

// component_prover.rs:603-633 around a row evaluator
template <class RowFn>
inline void accumulate_pointwise_cpu(RowFn&& row_fn, uint32_t eval_log, uint32_t trace_log, uint32_t* const accum[4], bool accumulate) {
    std::vector<M31> denom_inv = constraint_denom_inv(trace_log, eval_log);
    const size_t n = (size_t)1 << eval_log;
#pragma omp parallel for schedule(static)
    for (size_t row = 0; row < n; row++) {
        QM31 row_res = row_fn(row);
        QM31 prev = accumulate ? QM31::from_u32(accum[0][row], accum[1][row], accum[2][row], accum[3][row]) : QM31::zero();
        QM31 r = prev + row_res * denom_inv[row >> trace_log];
        uint32_t w[4];
        r.to_u32(w);
        for (int k = 0; k < 4; k++) accum[k][row] = w[k];
    }
}

// ---------------------------------------------------------------------------------------------- the single-assignment form

struct AirOp {
    uint32_t op, a, b, c, d;
};
enum : uint32_t { AIR_LOAD = 0, AIR_CONST_M31, AIR_SCALAR, AIR_CUMSUM_SHIFT, AIR_ADD_B, AIR_SUB_B, AIR_MUL_B, AIR_NEG_B,
                  AIR_ADD_E, AIR_SUB_E, AIR_MUL_E, AIR_NEG_E, AIR_PACK, AIR_INV_B };

// prover/src/cudagen.rs:1217-1262: every instruction in order, base values promoted where a secure value is asked for
inline QM31 air_interpret_row(const AirOp* ops, size_t n_ops, const uint32_t* constraints, size_t n_constraints,
                              const std::vector<std::vector<const uint32_t*>>& cols, const QM31* scalars, QM31 cumsum_shift,
                              const QM31* rcp, size_t row, uint32_t trace_log, uint32_t eval_log) {
    std::vector<QM31> v(n_ops);
    auto b = [&](uint32_t i) { return v[i].a.a; };
    for (size_t i = 0; i < n_ops; i++) {
        const AirOp& o = ops[i];
        switch (o.op) {
            case AIR_LOAD: {
                int32_t off = (int32_t)o.c;
                size_t r = off == 0 ? row : offset_bit_reversed_circle_domain_index(row, trace_log, eval_log, off);
                v[i] = QM31(M31(cols[o.a][o.b][r]));
                break;
            }
            case AIR_CONST_M31: v[i] = QM31(M31(o.a)); break;
            case AIR_SCALAR: v[i] = scalars[o.a]; break;
            case AIR_CUMSUM_SHIFT: v[i] = cumsum_shift; break;
            case AIR_ADD_B: v[i] = QM31(b(o.a) + b(o.b)); break;
            case AIR_SUB_B: v[i] = QM31(b(o.a) - b(o.b)); break;
            case AIR_MUL_B: v[i] = QM31(b(o.a) * b(o.b)); break;
            case AIR_NEG_B: v[i] = QM31(-b(o.a)); break;
            case AIR_INV_B: v[i] = QM31(b(o.a).is_zero() ? M31(0) : b(o.a).inverse()); break;
            case AIR_ADD_E: v[i] = v[o.a] + v[o.b]; break;
            case AIR_SUB_E: v[i] = v[o.a] - v[o.b]; break;
            case AIR_MUL_E: v[i] = v[o.a] * v[o.b]; break;
            case AIR_NEG_E: v[i] = -v[o.a]; break;
            case AIR_PACK: v[i] = QM31::from_m31s(b(o.a), b(o.b), b(o.c), b(o.d)); break;
            default: assert(false);
        }
    }
    QM31 res = QM31::zero();
    for (size_t k = 0; k < n_constraints; k++) res = res + rcp[k] * v[constraints[k]];
    return res;
}

}  // namespace zko
