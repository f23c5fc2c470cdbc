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
#include <map>

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

// One component of the statement: its AIR, the size of its trace and its LogUp claimed sum. In every tree the columns
// of component k follow those of components 0..k-1 (TraceLocationAllocator, constraint-framework/src/component.rs).
struct StarkComponent {
    AirSpec air;
    uint32_t trace_log;
    QM31 claimed_sum;
};

inline StarkResult stark_prove_multi(const std::vector<StarkComponent>& comps, const std::vector<std::vector<std::vector<M31>>>& trees,
                                     PcsConfig cfg) {
    const uint32_t blowup = cfg.fri.log_blowup_factor;
    const size_t n_trees = trees.size();
    uint32_t max_trace_log = 0;
    for (auto& c : comps) max_trace_log = std::max(max_trace_log, c.trace_log);
    const uint32_t composition_log = max_trace_log + 1;  // Components::composition_log_degree_bound (core/air/components.rs:24-30)
    Channel ch(true);
    cfg.mix_into(ch);
    CommitmentSchemeProver prover(cfg, max_trace_log + blowup);
    for (auto& t : trees) prover.commit_evals(t, ch);

    // the shape of every AIR (info.rs) and where its columns start in each tree
    std::vector<InfoEvaluator> infos;
    std::vector<std::vector<size_t>> first(comps.size(), std::vector<size_t>(n_trees, 0));
    std::vector<size_t> next(n_trees, 0);
    size_t total_constraints = 0;
    for (size_t k = 0; k < comps.size(); k++) {
        infos.emplace_back(n_trees);
        comps[k].air.evaluate(infos.back());
        total_constraints += infos.back().n_constraints;
        for (size_t t = 0; t < n_trees; t++) {
            first[k][t] = next[t];
            next[t] += infos.back().mask_offsets[t].size();
        }
    }
    for (size_t t = 0; t < n_trees; t++) assert(next[t] == trees[t].size());

    // ---- composition polynomial (prover/air/component_prover.rs:161-176; accumulation.rs:33-68, 89-124)
    const QM31 random_coeff = ch.draw_secure_felt();
    std::vector<QM31> remaining = generate_secure_powers(random_coeff, total_constraints);
    std::map<uint32_t, SecureColumn> sub;  // sub_accumulations by log size
    for (size_t k = 0; k < comps.size(); k++) {
        const size_t n_k = infos[k].n_constraints;
        std::vector<QM31> powers(remaining.end() - n_k, remaining.end());  // columns(): the last n_k powers
        remaining.resize(remaining.size() - n_k);
        std::reverse(powers.begin(), powers.end());  // component_prover.rs:271
        const uint32_t trace_log = comps[k].trace_log, eval_log = trace_log + 1;
        CircleDomain eval_domain = CanonicCoset(eval_log).circle_domain();
        std::vector<std::vector<std::vector<M31>>> ext(n_trees);
        TraceView view(n_trees);
        for (size_t t = 0; t < n_trees; t++) {
            const size_t cnt = infos[k].mask_offsets[t].size();
            ext[t].resize(cnt);
#pragma omp parallel for schedule(dynamic)
            for (size_t c = 0; c < cnt; c++) ext[t][c] = evaluate(prover.trees[t].coeffs[first[k][t] + c], eval_domain, prover.twiddles);
            for (auto& col : ext[t]) view[t].push_back(reinterpret_cast<const uint32_t*>(col.data()));
        }
        const size_t N = (size_t)1 << eval_log;
        std::vector<std::vector<uint32_t>> acc(4, std::vector<uint32_t>(N, 0));
        SecureColumn& dst = sub[eval_log];
        if (!dst.empty())
            for (size_t i = 0; i < N; i++) { uint32_t w[4]; dst[i].to_u32(w); for (int q = 0; q < 4; q++) acc[q][i] = w[q]; }
        uint32_t* accp[4] = {acc[0].data(), acc[1].data(), acc[2].data(), acc[3].data()};
        accumulate_pointwise_cpu([&](size_t row) {
            CpuDomainEvaluator eval(view, row, powers.data(), trace_log, eval_log, trace_log, comps[k].claimed_sum);
            comps[k].air.evaluate(eval);
            return eval.row_res;
        }, eval_log, trace_log, accp, !dst.empty());
        dst.resize(N);
        for (size_t i = 0; i < N; i++) dst[i] = QM31::from_u32(acc[0][i], acc[1][i], acc[2][i], acc[3][i]);
    }
    assert(remaining.empty());
    std::vector<SecureColumn> ascending;
    for (auto& kv : sub) ascending.push_back(std::move(kv.second));
    SecureColumn composition = lift_and_accumulate(std::move(ascending));
    assert(composition.size() == ((size_t)1 << composition_log));
    // finalize: interpolate the four coordinate columns; split_at_mid; commit left halves then right halves
    const size_t N = (size_t)1 << composition_log;
    CircleDomain comp_domain = CanonicCoset(composition_log).circle_domain();
    CircleDomain half_domain = CanonicCoset(composition_log - 1).circle_domain();
    std::vector<std::vector<M31>> halves(8);
    for (int q = 0; q < 4; q++) {
        std::vector<M31> c(N);
        for (size_t i = 0; i < N; i++) { uint32_t w[4]; composition[i].to_u32(w); c[i] = M31(w[q]); }
        interpolate(c, comp_domain, prover.twiddles);
        std::vector<M31> left(c.begin(), c.begin() + N / 2), right(c.begin() + N / 2, c.end());
        // commit_evals takes evaluations on the polynomial's own domain and interpolates them back to these coefficients
        halves[q] = evaluate(left, half_domain, prover.twiddles);
        halves[4 + q] = evaluate(right, half_domain, prover.twiddles);
    }
    prover.commit_evals(halves, ch);

    // ---- out-of-domain sampling (prover/mod.rs:98-139; core/air/components.rs:32-74)
    CirclePoint<QM31> oods = get_random_point(ch);
    const uint32_t lifting_log = prover.trees.back().max_log();
    const uint32_t max_log_degree_bound = lifting_log - blowup;
    CirclePoint<M31> trace_step = CanonicCoset(max_log_degree_bound).step();
    std::vector<std::vector<std::vector<CirclePoint<QM31>>>> points(n_trees + 1);
    for (size_t t = 0; t < n_trees; t++) points[t].resize(trees[t].size());
    for (size_t k = 0; k < comps.size(); k++)
        for (size_t t = 0; t < n_trees; t++)
            for (size_t c = 0; c < infos[k].mask_offsets[t].size(); c++)
                for (int off : infos[k].mask_offsets[t][c]) points[t][first[k][t] + c].push_back(oods + into_ef(mul_signed(trace_step, off)));
    points.back().assign(8, {oods});
    StarkResult r;
    r.proof = prover.prove_values(points, ch);
    r.digest = ch.digest;

    // ---- the prover's sanity check (prover/mod.rs:141-166; core/proof.rs:27-57; core/air/components.rs:76-94)
    const auto& comp = r.proof.sampled_values.back();
    QM31 left_eval = from_partial_evals(comp[0][0], comp[1][0], comp[2][0], comp[3][0]);
    QM31 right_eval = from_partial_evals(comp[4][0], comp[5][0], comp[6][0], comp[7][0]);
    r.committed_eval = left_eval + oods.repeated_double(max_log_degree_bound - 1).x * right_eval;
    QM31 denom_inverse = coset_vanishing(CanonicCoset(max_log_degree_bound).coset, oods).inverse();
    QM31 accumulation = QM31::zero();
    for (size_t k = 0; k < comps.size(); k++) {
        std::vector<std::vector<std::vector<QM31>>> mask(n_trees);
        for (size_t t = 0; t < n_trees; t++)
            for (size_t c = 0; c < infos[k].mask_offsets[t].size(); c++) mask[t].push_back(r.proof.sampled_values[t][first[k][t] + c]);
        PointEvaluator pe(mask, random_coeff, denom_inverse, comps[k].trace_log, comps[k].claimed_sum);
        pe.accumulation = accumulation;  // one PointEvaluationAccumulator runs through all components
        comps[k].air.evaluate(pe);
        accumulation = pe.accumulation;
    }
    r.point_eval = accumulation;
    return r;
}

inline StarkResult stark_prove(const AirSpec& air, const std::vector<std::vector<std::vector<M31>>>& trees, QM31 claimed_sum,
                               uint32_t trace_log, PcsConfig cfg) {
    return stark_prove_multi({StarkComponent{air, trace_log, claimed_sum}}, trees, cfg);
}

}  // namespace zko
