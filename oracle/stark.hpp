// TEST INFRASTRUCTURE ONLY (CPU oracle; see fields.hpp).
//
// A whole STARK proof of one component, as the reference's generic prover runs it:
//   nitroo/crates/stwo/src/prover/mod.rs:41-173                      (prove_ex)
//   nitroo/crates/stwo/src/prover/air/component_prover.rs / accumulation.rs:20-125   (DomainEvaluationAccumulator)
//   nitroo/crates/stwo/src/prover/poly/circle/secure_poly.rs:54-65, backend/cpu/circle.rs:263-271  (split_at_mid)
//   nitroo/crates/constraint-framework/src/component.rs:356-413      (mask_points, evaluate_constraint_quotients_at_point)
//   nitroo/crates/stwo/src/core/proof.rs:27-57                       (extract_composition_oods_eval)
//   nitroo/crates/stwo/src/core/air/accumulation.rs:12-36            (PointEvaluationAccumulator)
// The trees are committed in the fork's order: preprocessed, model, base trace, interaction (some may be empty), then
// the composition tree. The AIR is one of the three of air.hpp, evaluated on the domain with CpuDomainEvaluator and at
// the out-of-domain point with PointEvaluator; the proof is accepted by the prover's own sanity check iff both agree.
#pragma once
#include "air.hpp"
#include "protocol.hpp"

namespace zko {

// core/constraints.rs:12-35 at a secure-field point
inline QM31 coset_vanishing(const Coset& coset, CirclePoint<QM31> p) {
    CirclePointIndex half_step{coset.step_size.i >> 1};
    p = p + into_ef(coset.initial.conjugate()) + into_ef(half_step.to_point());
    QM31 x = p.x;
    for (uint32_t k = 1; k < coset.log_size; k++) x = double_x(x);
    return x;
}

// circle.rs:113-119
inline CirclePoint<M31> mul_signed(CirclePoint<M31> p, int off) { return off > 0 ? p.mul((uint64_t)off) : p.conjugate().mul((uint64_t)(-off)); }

struct StarkResult {
    PcsProof proof;
    Hash digest;
    QM31 committed_eval, point_eval;
};

inline StarkResult stark_prove(const AirSpec& air, const std::vector<std::vector<std::vector<M31>>>& trees, QM31 claimed_sum,
                               uint32_t trace_log, uint32_t composition_log, PcsConfig cfg) {
    const uint32_t blowup = cfg.fri.log_blowup_factor;
    Channel ch(true);
    cfg.mix_into(ch);
    CommitmentSchemeProver prover(cfg, std::max(trace_log, composition_log - 1) + blowup);
    for (auto& t : trees) prover.commit_evals(t, ch);

    // the AIR's shape: mask offsets per column, number of constraints (info.rs)
    InfoEvaluator info(trees.size());
    air.evaluate(info);
    const size_t n_constraints = info.n_constraints;

    // ---- composition polynomial (prover/mod.rs:70-85; accumulation.rs:33-68, 89-124)
    const QM31 random_coeff = ch.draw_secure_felt();
    std::vector<QM31> powers = generate_secure_powers(random_coeff, n_constraints);
    std::reverse(powers.begin(), powers.end());  // component_prover.rs:271: the first constraint takes the highest power
    CircleDomain eval_domain = CanonicCoset(composition_log).circle_domain();
    std::vector<std::vector<std::vector<M31>>> ext(trees.size());
    TraceView view(trees.size());
    for (size_t t = 0; t < trees.size(); t++) {
        ext[t].resize(trees[t].size());
#pragma omp parallel for schedule(dynamic)
        for (size_t c = 0; c < trees[t].size(); c++) ext[t][c] = evaluate(prover.trees[t].coeffs[c], eval_domain, prover.twiddles);
        for (auto& col : ext[t]) view[t].push_back(reinterpret_cast<const uint32_t*>(col.data()));
    }
    const size_t N = (size_t)1 << composition_log;
    std::vector<std::vector<uint32_t>> acc(4, std::vector<uint32_t>(N, 0));
    uint32_t* accp[4] = {acc[0].data(), acc[1].data(), acc[2].data(), acc[3].data()};
    accumulate_pointwise_cpu([&](size_t row) {
        CpuDomainEvaluator eval(view, row, powers.data(), trace_log, composition_log, trace_log, claimed_sum);
        air.evaluate(eval);
        return eval.row_res;
    }, composition_log, trace_log, accp, false);
    // finalize: interpolate the four coordinate columns; split_at_mid; commit left halves then right halves
    std::vector<std::vector<M31>> halves(8);
    const uint32_t half_log = composition_log - 1;
    CircleDomain half_domain = CanonicCoset(half_log).circle_domain();
    for (int k = 0; k < 4; k++) {
        std::vector<M31> c(N);
        for (size_t i = 0; i < N; i++) c[i] = M31(acc[k][i]);
        interpolate(c, eval_domain, prover.twiddles);
        std::vector<M31> left(c.begin(), c.begin() + N / 2), right(c.begin() + N / 2, c.end());
        // commit_evals takes evaluations on the polynomial's own domain and interpolates them back to these coefficients
        halves[k] = evaluate(left, half_domain, prover.twiddles);
        halves[4 + k] = evaluate(right, half_domain, prover.twiddles);
    }
    prover.commit_evals(halves, ch);

    // ---- out-of-domain sampling (prover/mod.rs:98-139)
    CirclePoint<QM31> oods = get_random_point(ch);
    const uint32_t lifting_log = prover.trees.back().max_log();
    const uint32_t max_log_degree_bound = lifting_log - blowup;
    CirclePoint<M31> trace_step = CanonicCoset(max_log_degree_bound).step();
    std::vector<std::vector<std::vector<CirclePoint<QM31>>>> points(trees.size() + 1);
    for (size_t t = 0; t < trees.size(); t++) {
        points[t].resize(trees[t].size());
        for (size_t c = 0; c < trees[t].size(); c++)
            if (c < info.mask_offsets[t].size())
                for (int off : info.mask_offsets[t][c]) points[t][c].push_back(oods + into_ef(mul_signed(trace_step, off)));
    }
    points.back().assign(8, {oods});
    StarkResult r;
    r.proof = prover.prove_values(points, ch);
    r.digest = ch.digest;

    // ---- the prover's sanity check (prover/mod.rs:141-166; core/proof.rs:27-57; component.rs:374-413)
    const auto& comp = r.proof.sampled_values.back();
    QM31 left_eval = from_partial_evals(comp[0][0], comp[1][0], comp[2][0], comp[3][0]);
    QM31 right_eval = from_partial_evals(comp[4][0], comp[5][0], comp[6][0], comp[7][0]);
    r.committed_eval = left_eval + oods.repeated_double(max_log_degree_bound - 1).x * right_eval;
    std::vector<std::vector<std::vector<QM31>>> mask(trees.size());
    for (size_t t = 0; t < trees.size(); t++) mask[t] = r.proof.sampled_values[t];
    QM31 denom_inverse = coset_vanishing(CanonicCoset(max_log_degree_bound).coset, oods).inverse();
    PointEvaluator pe(mask, random_coeff, denom_inverse, trace_log, claimed_sum);
    air.evaluate(pe);
    r.point_eval = pe.accumulation;
    return r;
}

}  // namespace zko
