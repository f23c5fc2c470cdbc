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

struct Fraction {
    QM31 numerator, denominator;
    Fraction operator+(const Fraction& r) const {  // fraction.rs:27-33
        return {r.denominator * numerator + denominator * r.numerator, denominator * r.denominator};
    }
};
inline Fraction fraction_sum(const std::vector<Fraction>& v) {  // fraction.rs:56-59
    if (v.empty()) return {QM31::zero(), QM31::one()};
    Fraction acc = v[0];
    for (size_t i = 1; i < v.size(); i++) acc = acc + v[i];
    return acc;
}

// logup.rs:62-104
struct LookupElements {
    QM31 z;
    std::vector<QM31> alpha_powers;
    QM31 combine(const std::vector<M31>& values) const {
        assert(alpha_powers.size() >= values.size());
        QM31 acc = QM31::zero();
        for (size_t i = 0; i < values.size(); i++) acc = acc + alpha_powers[i] * values[i];
        return acc - z;
    }
};

using TraceView = std::vector<std::vector<const uint32_t*>>;  // [interaction][column] -> 2^eval_log words

// cpu_domain.rs:17-98 with the LogUp proxy of lib.rs:214-290
struct CpuDomainEvaluator {
    const TraceView& trace_eval;
    std::vector<size_t> column_index_per_interaction;
    size_t row;
    const QM31* random_coeff_powers;
    QM31 row_res = QM31::zero();
    size_t constraint_index = 0;
    uint32_t domain_log_size, eval_domain_log_size;
    // LogupAtRow (logup.rs:15-41)
    int logup_interaction = INTERACTION_TRACE_IDX;
    QM31 cumsum_shift;
    std::vector<Fraction> fracs;

    CpuDomainEvaluator(const TraceView& t, size_t row_, const QM31* rcp, uint32_t domain_log, uint32_t eval_log, uint32_t log_size,
                       QM31 claimed_sum)
        : trace_eval(t), column_index_per_interaction(t.size(), 0), row(row_), random_coeff_powers(rcp), domain_log_size(domain_log),
          eval_domain_log_size(eval_log) {
        cumsum_shift = claimed_sum * QM31(M31((uint32_t)1 << log_size)).inverse();
    }

    std::vector<M31> next_interaction_mask(int interaction, const std::vector<int>& offsets) {
        size_t col_index = column_index_per_interaction[interaction]++;
        const uint32_t* col = trace_eval[interaction][col_index];
        std::vector<M31> out;
        for (int off : offsets) {
            if (off == 0) { out.push_back(M31(col[row])); continue; }
            size_t r = offset_bit_reversed_circle_domain_index(row, domain_log_size, eval_domain_log_size, off);
            out.push_back(M31(col[r]));
        }
        return out;
    }
    M31 next_trace_mask() { return next_interaction_mask(ORIGINAL_TRACE_IDX, {0})[0]; }
    M31 get_preprocessed_column() { return next_interaction_mask(PREPROCESSED_TRACE_IDX, {0})[0]; }
    // lib.rs:127-137: four consecutive columns, combined per offset
    std::vector<QM31> next_extension_interaction_mask(int interaction, const std::vector<int>& offsets) {
        std::vector<M31> c[4];
        for (int k = 0; k < 4; k++) c[k] = next_interaction_mask(interaction, offsets);
        std::vector<QM31> out;
        for (size_t j = 0; j < offsets.size(); j++) out.push_back(QM31::from_m31s(c[0][j], c[1][j], c[2][j], c[3][j]));
        return out;
    }
    void add_constraint(QM31 c) { row_res = row_res + random_coeff_powers[constraint_index++] * c; }
    void add_constraint(M31 c) { row_res = row_res + random_coeff_powers[constraint_index++] * c; }
    // lib.rs:169-180
    void add_to_relation(const LookupElements& rel, QM31 multiplicity, const std::vector<M31>& values) {
        fracs.push_back({multiplicity, rel.combine(values)});
    }
    // lib.rs:226-275
    void finalize_logup_batched(const std::vector<size_t>& batching) {
        assert(batching.size() == fracs.size());
        size_t last_batch = 0;
        for (size_t b : batching) last_batch = b > last_batch ? b : last_batch;
        std::vector<std::vector<Fraction>> by_batch(last_batch + 1);
        for (size_t i = 0; i < batching.size(); i++) by_batch[batching[i]].push_back(fracs[i]);
        QM31 prev_col_cumsum = QM31::zero();
        for (size_t b = 0; b < last_batch; b++) {
            Fraction cur = fraction_sum(by_batch[b]);
            QM31 cur_cumsum = next_extension_interaction_mask(logup_interaction, {0})[0];
            QM31 diff = cur_cumsum - prev_col_cumsum;
            prev_col_cumsum = cur_cumsum;
            add_constraint(diff * cur.denominator - cur.numerator);
        }
        Fraction frac = fraction_sum(by_batch[last_batch]);
        std::vector<QM31> m = next_extension_interaction_mask(logup_interaction, {-1, 0});
        QM31 diff = m[1] - m[0] - prev_col_cumsum;
        QM31 shifted = diff + cumsum_shift;
        add_constraint(shifted * frac.denominator - frac.numerator);
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

// ---------------------------------------------------------------------------------------------- AIRs, written as in the reference

// nitroo/crates/examples/src/wide_fibonacci/mod.rs:47-57
inline void wide_fibonacci_evaluate(CpuDomainEvaluator& eval, size_t n_cols) {
    M31 a = eval.next_trace_mask(), b = eval.next_trace_mask();
    for (size_t k = 2; k < n_cols; k++) {
        M31 c = eval.next_trace_mask();
        eval.add_constraint(c - (a.square() + b.square()));
        a = b;
        b = c;
    }
}

// nitroo/crates/examples/src/plonk/mod.rs:51-88
inline void plonk_evaluate(CpuDomainEvaluator& eval, const LookupElements& lookup) {
    M31 a_wire = eval.get_preprocessed_column(), b_wire = eval.get_preprocessed_column();
    M31 c_wire = eval.get_preprocessed_column(), op = eval.get_preprocessed_column();
    M31 mult = eval.next_trace_mask(), a_val = eval.next_trace_mask(), b_val = eval.next_trace_mask(), c_val = eval.next_trace_mask();
    eval.add_constraint(c_val - op * (a_val + b_val) + (M31(1) - op) * a_val * b_val);
    eval.add_to_relation(lookup, QM31::one(), {a_wire, a_val});
    eval.add_to_relation(lookup, QM31::one(), {b_wire, b_val});
    eval.add_to_relation(lookup, QM31(-mult), {c_wire, c_val});
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
inline void freivalds_evaluate(CpuDomainEvaluator& eval, const FreivaldsEval& e) {
    M31 nofirst = eval.get_preprocessed_column(), last = eval.get_preprocessed_column();
    M31 notzero = eval.get_preprocessed_column(), end = eval.get_preprocessed_column();
    std::vector<std::vector<M31>> ws(e.n_mats);
    for (size_t m = 0; m < e.n_mats; m++)
        for (size_t p = 0; p < e.pk; p++) ws[m].push_back(eval.get_preprocessed_column());
    std::vector<M31> acts;
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
        for (M31 a : acts) eval.add_to_relation(e.rel_act, QM31::one(), {a});
        eval.finalize_logup_in_pairs();
    }
}

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
