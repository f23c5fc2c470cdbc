// TEST INFRASTRUCTURE - CPU restatement of the reference's VERIFIER for the commitment-and-proving path. Only
// tests/, __graft_entry__.smoke() and bench.py's checking legs may use it; the product never does.
//
// Follows, function by function:
//   nitroo/crates/stwo/src/core/vcs/verifier.rs:85-211        MerkleVerifier::verify
//   nitroo/crates/stwo/src/core/fri.rs:108-193                FriVerifier::commit
//   nitroo/crates/stwo/src/core/fri.rs:201-295                decommit, decommit_first_layer / inner_layers / last_layer
//   nitroo/crates/stwo/src/core/fri.rs:297-306                sample_query_positions
//   nitroo/crates/stwo/src/core/fri.rs:424-577                FriFirstLayerVerifier::verify, FriInnerLayerVerifier::verify_and_fold
//   nitroo/crates/stwo/src/core/fri.rs:579-625                compute_decommitment_positions_and_rebuild_evals
//   nitroo/crates/stwo/src/core/fri.rs:632-690                SparseEvaluation::fold_line / fold_circle
//   nitroo/crates/stwo/src/core/fri.rs:692-778                fold_line, fold_coset, fold_circle_into_line
//   nitroo/crates/stwo/src/core/poly/line.rs:137-145, core/poly/utils.rs:27-38   LinePoly::eval_at_point, fold
//   nitroo/crates/stwo/src/core/pcs/verifier.rs:45-178        CommitmentSchemeVerifier::commit / verify_values, build_queries_per_log_size
//   nitroo/crates/stwo/src/core/pcs/quotients.rs:127-213      fri_answers, accumulate_row_quotients
//   nitroo/crates/stwo/src/core/pcs/quotients.rs:316-351      build_samples_with_randomness_and_periodicity
//   nitroo/crates/stwo/src/core/pcs/quotients.rs:353-439      reshape_flat_to_per_column
//   nitroo/crates/stwo/src/core/pcs/utils.rs:200-218          prepare_preprocessed_query_positions
// The reference's errors (MerkleVerificationError, FriVerificationError, VerificationError::ProofOfWork) are the values of
// VerifyError; `Malformed` is the word-stream parser's (a proof whose counts run past its end).
//
// Pinned by the reference's own relational tests for this level, restated in tests/test_oracle_verifier.py: valid proofs
// are accepted, and each of the tamper cases of core/fri.rs:815-1150 and core/vcs/verifier.rs's tests is rejected with
// the error the reference names.
#pragma once
#include <map>
#include <vector>

#include "protocol.hpp"

namespace zko {

enum class VerifyError : int {
    Ok = 0,
    MerkleWitnessTooShort = 1,
    MerkleWitnessTooLong = 2,
    MerkleTooManyQueriedValues = 3,
    MerkleTooFewQueriedValues = 4,
    MerkleRootMismatch = 5,
    FriInvalidNumFriLayers = 10,
    FriFirstLayerEvaluationsInvalid = 11,
    FriFirstLayerCommitmentInvalid = 12,   // + the Merkle error in `detail`
    FriInnerLayerCommitmentInvalid = 13,   // + the Merkle error in `detail`, the layer in `layer`
    FriInnerLayerEvaluationsInvalid = 14,
    FriLastLayerDegreeInvalid = 15,
    FriLastLayerEvaluationsInvalid = 16,
    ProofOfWork = 20,
    TraceDecommitmentInvalid = 21,         // VerificationError::Merkle: + the Merkle error in `detail`, the tree in `layer`
    Malformed = 30,
};
struct VerifyResult {
    VerifyError error = VerifyError::Ok;
    VerifyError detail = VerifyError::Ok;
    int layer = -1;
    bool ok() const { return error == VerifyError::Ok; }
};

// ------------------------------------------------------------------ Merkle (core/vcs/verifier.rs:85-211)
struct MerkleVerifier {
    Hash root;
    std::vector<uint32_t> column_log_sizes;
    bool m31 = true;

    VerifyError verify(const std::map<uint32_t, std::vector<size_t>>& queries_per_log_size, const std::vector<M31>& queried_values,
                       const MerkleDecommitment& dec) const {
        if (column_log_sizes.empty()) return VerifyError::Ok;
        uint32_t max_log = 0;
        std::map<uint32_t, size_t> n_columns_per_log_size;
        for (auto l : column_log_sizes) { max_log = std::max(max_log, l); n_columns_per_log_size[l]++; }
        size_t qv = 0, hw = 0, cw = 0;
        std::vector<std::pair<size_t, Hash>> last;
        bool have_last = false;
        for (uint32_t layer = max_log + 1; layer-- > 0;) {
            size_t n_cols = n_columns_per_log_size.count(layer) ? n_columns_per_log_size[layer] : 0;
            std::vector<std::pair<size_t, Hash>> total;
            std::vector<size_t> prev_q;
            for (auto& e : last) prev_q.push_back(e.first);
            static const std::vector<size_t> none;
            auto cq_it = queries_per_log_size.find(layer);
            const std::vector<size_t>& colq = cq_it == queries_per_log_size.end() ? none : cq_it->second;
            size_t pi = 0, ci = 0, hi = 0;  // cursors: previous-layer queries, column queries, previous-layer hashes
            for (;;) {
                // next_decommitment_node: the smaller of the next column query and the parent of the next previous-layer query
                bool hp = pi < prev_q.size(), hc = ci < colq.size();
                if (!hp && !hc) break;
                size_t node;
                if (hp && hc) node = std::min(prev_q[pi] / 2, colq[ci]);
                else node = hp ? prev_q[pi] / 2 : colq[ci];
                while (pi < prev_q.size() && prev_q[pi] / 2 == node) pi++;
                Hash left{}, right{};
                if (have_last) {
                    if (hi < last.size() && last[hi].first == 2 * node) left = last[hi++].second;
                    else { if (hw >= dec.hash_witness.size()) return VerifyError::MerkleWitnessTooShort; left = dec.hash_witness[hw++]; }
                    if (hi < last.size() && last[hi].first == 2 * node + 1) right = last[hi++].second;
                    else { if (hw >= dec.hash_witness.size()) return VerifyError::MerkleWitnessTooShort; right = dec.hash_witness[hw++]; }
                }
                std::vector<M31> vals;
                if (ci < colq.size() && colq[ci] == node) {
                    ci++;
                    if (qv + n_cols > queried_values.size()) return VerifyError::MerkleTooFewQueriedValues;
                    vals.assign(queried_values.begin() + qv, queried_values.begin() + qv + n_cols);
                    qv += n_cols;
                } else {
                    if (cw + n_cols > dec.column_witness.size()) return VerifyError::MerkleWitnessTooShort;
                    vals.assign(dec.column_witness.begin() + cw, dec.column_witness.begin() + cw + n_cols);
                    cw += n_cols;
                }
                total.push_back({node, hash_node(have_last ? &left : nullptr, have_last ? &right : nullptr, vals.data(), vals.size(), m31)});
            }
            last = std::move(total);
            have_last = true;
        }
        if (hw != dec.hash_witness.size()) return VerifyError::MerkleWitnessTooLong;
        if (qv != queried_values.size()) return VerifyError::MerkleTooManyQueriedValues;
        if (cw != dec.column_witness.size()) return VerifyError::MerkleWitnessTooLong;
        if (last.size() != 1 || last[0].second != root) return VerifyError::MerkleRootMismatch;
        return VerifyError::Ok;
    }
};

// ------------------------------------------------------------------ FRI folds on sparse evaluations
// core/fri.rs:692-716
inline QM31 fold_coset(std::vector<QM31> eval, LineDomain domain, QM31 alpha) {
    uint32_t n = domain.log_size();
    QM31 folding_alpha = alpha;
    for (uint32_t i = 0; i < n; i++) {
        for (size_t j = 0; j < ((size_t)1 << (n - i)); j += 2) {
            M31 x = domain.at(bit_reverse_index(j, domain.log_size()));
            QM31 f0 = eval[j], f1 = eval[j + 1];
            QM31 t = f0;  // ibutterfly (core/fft.rs:31-41): (f0 + f1, (f0 - f1) * twiddle)
            f0 = t + f1;
            f1 = (t - f1) * QM31(x.inverse());
            eval[j >> 1] = f0 + folding_alpha * f1;
        }
        folding_alpha = folding_alpha * folding_alpha;
        domain = domain.dbl();
    }
    return eval[0];
}
// core/poly/line.rs:137-145 with core/poly/utils.rs:27-38
inline QM31 fold_values(const QM31* values, size_t n, const QM31* factors) {
    if (n == 1) return values[0];
    QM31 lhs = fold_values(values, n / 2, factors + 1), rhs = fold_values(values + n / 2, n / 2, factors + 1);
    return lhs + rhs * factors[0];
}
inline QM31 line_poly_eval_at_point(const std::vector<QM31>& coeffs, QM31 x) {
    uint32_t log_size = ilog2(coeffs.size());
    std::vector<QM31> doublings;
    for (uint32_t i = 0; i < log_size; i++) { doublings.push_back(x); x = double_x(x); }
    return fold_values(coeffs.data(), coeffs.size(), doublings.data());
}

struct SparseEvaluation {
    std::vector<std::vector<QM31>> subset_evals;
    std::vector<size_t> subset_domain_initial_indexes;
    // core/fri.rs:660-672
    std::vector<QM31> fold_line(QM31 alpha, LineDomain source, uint32_t fold_step) const {
        std::vector<QM31> out;
        for (size_t k = 0; k < subset_evals.size(); k++) {
            CirclePointIndex init = source.coset.index_at(subset_domain_initial_indexes[k]);
            out.push_back(fold_coset(subset_evals[k], LineDomain{Coset::make(init, fold_step)}, alpha));
        }
        return out;
    }
    // core/fri.rs:674-689: a circle fold of one pair
    std::vector<QM31> fold_circle(QM31 alpha, CircleDomain source) const {
        std::vector<QM31> out;
        for (size_t k = 0; k < subset_evals.size(); k++) {
            CirclePoint<M31> p = source.index_at(subset_domain_initial_indexes[k]).to_point();
            QM31 f0 = subset_evals[k][0], f1 = subset_evals[k][1];
            QM31 t = f0;
            f0 = t + f1;
            f1 = (t - f1) * QM31(p.y.inverse());
            out.push_back(alpha * f1 + f0);  // dst starts at zero: dst * alpha^2 + f'
        }
        return out;
    }
};

// core/fri.rs:579-625. Returns false when the witness runs out.
inline bool decommitment_positions_and_rebuild(const std::vector<size_t>& queries, uint32_t log_domain_size, const std::vector<QM31>& query_evals,
                                               const std::vector<QM31>& witness, size_t& wpos, uint32_t fold_step,
                                               std::vector<size_t>& positions, SparseEvaluation& sparse) {
    size_t qe = 0, i = 0;
    while (i < queries.size()) {
        size_t j = i;
        while (j < queries.size() && (queries[j] >> fold_step) == (queries[i] >> fold_step)) j++;
        size_t start = (queries[i] >> fold_step) << fold_step;
        std::vector<QM31> evals;
        size_t k = i;
        for (size_t pos = start; pos < start + ((size_t)1 << fold_step); pos++) {
            positions.push_back(pos);
            if (k < j && queries[k] == pos) { evals.push_back(query_evals[qe++]); k++; }
            else { if (wpos >= witness.size()) return false; evals.push_back(witness[wpos++]); }
        }
        sparse.subset_evals.push_back(evals);
        sparse.subset_domain_initial_indexes.push_back(bit_reverse_index(start, log_domain_size));
        i = j;
    }
    return true;
}

inline std::vector<M31> flatten_coords(const SparseEvaluation& s) {
    std::vector<M31> flat;
    for (auto& sub : s.subset_evals)
        for (auto q : sub) { uint32_t w[4]; q.to_u32(w); for (int k = 0; k < 4; k++) flat.push_back(M31(w[k])); }
    return flat;
}

// ------------------------------------------------------------------ FriVerifier (core/fri.rs:83-306)
struct FriVerifier {
    FriConfig config;
    CircleDomain column_commitment_domain;
    FriLayerProof first_proof;
    QM31 first_alpha;
    struct Inner { LineDomain domain; QM31 alpha; size_t index; FriLayerProof proof; uint32_t fold_step; };
    std::vector<Inner> inner;
    LineDomain last_domain;
    std::vector<QM31> last_poly;
    std::vector<size_t> queries;
    uint32_t queries_log = 0;
    bool m31 = true;

    // :108-193. log_degree_bound is the committed circle polynomial's.
    static VerifyResult commit(Channel& ch, FriConfig config, const FriProof& proof, uint32_t log_degree_bound, FriVerifier& out) {
        out.config = config;
        out.m31 = ch.m31;
        ch.mix_root(proof.first_layer.commitment);
        out.column_commitment_domain = CanonicCoset(log_degree_bound + config.log_blowup_factor).circle_domain();
        out.first_proof = proof.first_layer;
        out.first_alpha = ch.draw_secure_felt();
        if (log_degree_bound < 1) return {VerifyError::FriInvalidNumFriLayers};
        uint32_t layer_bound = log_degree_bound - 1;  // fold_to_line
        LineDomain layer_domain{Coset::half_odds(layer_bound + config.log_blowup_factor)};
        size_t n_inner = proof.inner_layers.size();
        for (size_t k = 0; k < n_inner; k++) {
            ch.mix_root(proof.inner_layers[k].commitment);
            uint32_t fold_step;
            if (k + 1 != n_inner) fold_step = config.line_fold_step;
            else {
                if (layer_bound < config.log_last_layer_degree_bound) return {VerifyError::FriInvalidNumFriLayers};
                uint32_t res = layer_bound - config.log_last_layer_degree_bound;
                if (res < 1 || res > config.line_fold_step) return {VerifyError::FriInvalidNumFriLayers};
                fold_step = res;
            }
            out.inner.push_back({layer_domain, ch.draw_secure_felt(), k, proof.inner_layers[k], fold_step});
            if (layer_bound < fold_step) return {VerifyError::FriInvalidNumFriLayers};
            layer_bound -= fold_step;
            layer_domain = LineDomain{layer_domain.coset.repeated_double(fold_step)};
        }
        if (layer_bound != config.log_last_layer_degree_bound) return {VerifyError::FriInvalidNumFriLayers};
        out.last_domain = layer_domain;
        out.last_poly = proof.last_layer_poly;
        if (out.last_poly.size() > ((size_t)1 << config.log_last_layer_degree_bound)) return {VerifyError::FriLastLayerDegreeInvalid};
        ch.mix_felts(out.last_poly);
        return {};
    }

    // :297-306
    std::vector<size_t> sample_query_positions(Channel& ch) {
        queries_log = column_commitment_domain.log_size();
        queries = sorted_dedup(draw_queries(ch, queries_log, config.n_queries));
        return queries;
    }

    // :201-295 with the two layer verifiers (:424-577)
    VerifyResult decommit(const std::vector<QM31>& first_layer_query_evals) const {
        // first layer
        size_t wpos = 0;
        std::vector<size_t> positions;
        SparseEvaluation sparse;
        if (!decommitment_positions_and_rebuild(queries, queries_log, first_layer_query_evals, first_proof.fri_witness, wpos, 1, positions, sparse))
            return {VerifyError::FriFirstLayerEvaluationsInvalid};
        if (wpos != first_proof.fri_witness.size()) return {VerifyError::FriFirstLayerEvaluationsInvalid};
        {
            uint32_t log = column_commitment_domain.log_size();
            MerkleVerifier mv{first_proof.commitment, std::vector<uint32_t>(4, log), m31};
            VerifyError e = mv.verify({{log, positions}}, flatten_coords(sparse), first_proof.decommitment);
            if (e != VerifyError::Ok) return {VerifyError::FriFirstLayerCommitmentInvalid, e};
        }
        std::vector<size_t> layer_queries = fold_queries(queries, 1);
        std::vector<QM31> layer_evals = sparse.fold_circle(first_alpha, column_commitment_domain);
        // inner layers
        for (auto& layer : inner) {
            size_t w = 0;
            std::vector<size_t> pos;
            SparseEvaluation sp;
            if (!decommitment_positions_and_rebuild(layer_queries, layer.domain.log_size(), layer_evals, layer.proof.fri_witness, w, layer.fold_step, pos, sp))
                return {VerifyError::FriInnerLayerEvaluationsInvalid, VerifyError::Ok, (int)layer.index};
            if (w != layer.proof.fri_witness.size()) return {VerifyError::FriInnerLayerEvaluationsInvalid, VerifyError::Ok, (int)layer.index};
            uint32_t log = layer.domain.log_size();
            MerkleVerifier mv{layer.proof.commitment, std::vector<uint32_t>(4, log), m31};
            VerifyError e = mv.verify({{log, pos}}, flatten_coords(sp), layer.proof.decommitment);
            if (e != VerifyError::Ok) return {VerifyError::FriInnerLayerCommitmentInvalid, e, (int)layer.index};
            layer_queries = fold_queries(layer_queries, layer.fold_step);
            layer_evals = sp.fold_line(layer.alpha, layer.domain, layer.fold_step);
        }
        // last layer
        for (size_t k = 0; k < layer_queries.size(); k++) {
            M31 x = last_domain.at(bit_reverse_index(layer_queries[k], last_domain.log_size()));
            if (!(layer_evals[k] == line_poly_eval_at_point(last_poly, QM31(x)))) return {VerifyError::FriLastLayerEvaluationsInvalid};
        }
        return {};
    }
};

// ------------------------------------------------------------------ commitment scheme (core/pcs/verifier.rs, core/pcs/quotients.rs)
// core/pcs/utils.rs:200-218
inline std::vector<size_t> prepare_preprocessed_query_positions(const std::vector<size_t>& q, uint32_t max_log, uint32_t pp_max_log) {
    std::vector<size_t> out;
    if (pp_max_log == 0) return out;
    for (auto pos : q)
        out.push_back(max_log < pp_max_log ? ((pos >> 1) << (pp_max_log - max_log + 1)) + (pos & 1)
                                           : ((pos >> (max_log - pp_max_log + 1)) << 1) + (pos & 1));
    return out;
}
// core/pcs/verifier.rs:158-178
inline std::map<uint32_t, std::vector<size_t>> build_queries_per_log_size(const std::vector<uint32_t>& column_log_sizes,
                                                                           const std::vector<size_t>& query_positions) {
    uint32_t max_log = 0;
    for (auto l : column_log_sizes) max_log = std::max(max_log, l);
    std::map<uint32_t, std::vector<size_t>> out;
    for (auto l : column_log_sizes) {
        if (out.count(l)) continue;
        std::vector<size_t> p;
        for (auto pos : query_positions) p.push_back(((pos >> (max_log - l + 1)) << 1) + (pos & 1));
        out[l] = sorted_dedup(p);
    }
    return out;
}
// core/pcs/quotients.rs:353-439
inline std::vector<std::vector<M31>> reshape_flat_to_per_column(const std::vector<M31>& flat, const std::vector<uint32_t>& column_log_sizes,
                                                                const std::vector<size_t>& query_positions, uint32_t max_log, bool& ok) {
    uint32_t tree_max = 0;
    for (auto l : column_log_sizes) tree_max = std::max(tree_max, l);
    std::vector<size_t> tq = prepare_preprocessed_query_positions(query_positions, max_log, tree_max);
    std::map<uint32_t, std::vector<size_t>> cols_by_log;
    for (size_t c = 0; c < column_log_sizes.size(); c++) cols_by_log[column_log_sizes[c]].push_back(c);
    std::map<uint32_t, std::vector<size_t>> qpl;
    for (auto& e : cols_by_log) {
        std::vector<size_t> p;
        for (auto pos : tq) p.push_back(((pos >> (tree_max - e.first + 1)) << 1) + (pos & 1));
        qpl[e.first] = sorted_dedup(p);
    }
    std::vector<std::vector<M31>> natural(column_log_sizes.size());
    size_t at = 0;
    for (auto it = cols_by_log.rbegin(); it != cols_by_log.rend(); ++it)
        for (size_t k = 0; k < qpl[it->first].size(); k++)
            for (auto c : it->second) {
                if (at >= flat.size()) { ok = false; return {}; }
                natural[c].push_back(flat[at++]);
            }
    if (at != flat.size()) { ok = false; return {}; }
    std::vector<std::vector<M31>> result(column_log_sizes.size());
    for (size_t c = 0; c < column_log_sizes.size(); c++) {
        auto& positions = qpl[column_log_sizes[c]];
        for (auto p : tq) {
            size_t lifted = ((p >> (tree_max - column_log_sizes[c] + 1)) << 1) + (p & 1);
            size_t idx = std::lower_bound(positions.begin(), positions.end(), lifted) - positions.begin();
            result[c].push_back(natural[c][idx]);
        }
    }
    return result;
}

struct CommitmentSchemeVerifier {
    PcsConfig config;
    std::vector<MerkleVerifier> trees;
    bool m31 = true;

    // :45-61: log_sizes are the TRACE columns' log sizes
    void commit(const Hash& commitment, const std::vector<uint32_t>& log_sizes, Channel& ch) {
        ch.mix_root(commitment);
        std::vector<uint32_t> ext;
        for (auto l : log_sizes) ext.push_back(l + config.fri.log_blowup_factor);
        trees.push_back({commitment, ext, m31});
    }

    // :63-155
    VerifyResult verify_values(const std::vector<std::vector<std::vector<CirclePoint<QM31>>>>& sampled_points, const PcsProof& proof,
                               Channel& ch) const {
        std::vector<QM31> flat;
        for (auto& t : proof.sampled_values) for (auto& c : t) for (auto v : c) flat.push_back(v);
        ch.mix_felts(flat);
        QM31 random_coeff = ch.draw_secure_felt();
        uint32_t lifting_log = 0;
        for (size_t t = 0; t < trees.size(); t++)
            for (size_t c = 0; c < trees[t].column_log_sizes.size(); c++)
                if (!sampled_points[t][c].empty()) lifting_log = std::max(lifting_log, trees[t].column_log_sizes[c]);
        FriVerifier fri;
        VerifyResult r = FriVerifier::commit(ch, config.fri, proof.fri, lifting_log - config.fri.log_blowup_factor, fri);
        if (!r.ok()) return r;
        if (!ch.verify_pow_nonce(config.pow_bits, proof.proof_of_work)) return {VerifyError::ProofOfWork};
        ch.mix_u64(proof.proof_of_work);
        std::vector<size_t> query_positions = fri.sample_query_positions(ch);
        for (size_t t = 0; t < trees.size(); t++) {
            uint32_t tree_max = 0;
            for (auto l : trees[t].column_log_sizes) tree_max = std::max(tree_max, l);
            auto tq = prepare_preprocessed_query_positions(query_positions, lifting_log, tree_max);
            VerifyError e = trees[t].verify(build_queries_per_log_size(trees[t].column_log_sizes, tq), proof.queried_values[t], proof.decommitments[t]);
            if (e != VerifyError::Ok) return {VerifyError::TraceDecommitmentInvalid, e, (int)t};
        }
        // fri_answers, core/pcs/quotients.rs:127-178
        std::vector<std::vector<M31>> per_col;
        for (size_t t = 0; t < trees.size(); t++) {
            bool ok = true;
            auto cols = reshape_flat_to_per_column(proof.queried_values[t], trees[t].column_log_sizes, query_positions, lifting_log, ok);
            if (!ok) return {VerifyError::Malformed};
            for (auto& c : cols) per_col.push_back(std::move(c));
        }
        // build_samples_with_randomness_and_periodicity, :316-351, then ColumnSampleBatch::new_vec (stable grouping by point)
        std::vector<ColumnSampleBatch> batches;
        QM31 pow = QM31::one();
        CirclePoint<M31> gen = CanonicCoset(lifting_log).step();
        size_t flat_col = 0;
        for (size_t t = 0; t < trees.size(); t++)
            for (size_t c = 0; c < trees[t].column_log_sizes.size(); c++, flat_col++) {
                const auto& pts = sampled_points[t][c];
                const auto& vals = proof.sampled_values[t][c];
                if (pts.size() != vals.size()) return {VerifyError::Malformed};
                if (pts.empty()) continue;
                std::vector<std::pair<PointSample, QM31>> with_rand;
                if (pts.size() == 2) {
                    CirclePoint<M31> per = gen.repeated_double(trees[t].column_log_sizes[c]);
                    with_rand.push_back({PointSample{pts[1] + into_ef(per), vals[1]}, pow});
                    pow = pow * random_coeff;
                }
                for (size_t k = 0; k < pts.size(); k++) { with_rand.push_back({PointSample{pts[k], vals[k]}, pow}); pow = pow * random_coeff; }
                for (auto& sp : with_rand) {
                    ColumnSampleBatch* b = nullptr;
                    for (auto& x : batches) if (x.point == sp.first.point) { b = &x; break; }
                    if (!b) { batches.push_back({sp.first.point, {}}); b = &batches.back(); }
                    b->cols_vals_randpows.push_back({flat_col, sp.first.value, sp.second});
                }
            }
        auto line_coeffs = column_line_coeffs(batches);
        CircleDomain lifting_domain = CanonicCoset(lifting_log).circle_domain();
        std::vector<CirclePoint<QM31>> sample_points;
        for (auto& b : batches) sample_points.push_back(b.point);
        std::vector<QM31> answers;
        for (size_t qi = 0; qi < query_positions.size(); qi++) {
            CirclePoint<M31> dp = lifting_domain.at(bit_reverse_index(query_positions[qi], lifting_log));
            auto dinv = denominator_inverses(sample_points, dp);
            QM31 acc = QM31::zero();
            for (size_t b = 0; b < batches.size(); b++) {  // accumulate_row_quotients, :180-213
                QM31 numerator = QM31::zero();
                for (size_t k = 0; k < batches[b].cols_vals_randpows.size(); k++) {
                    const LineCoeffs& lc = line_coeffs[b][k];
                    QM31 value = lc.c * QM31(per_col[batches[b].cols_vals_randpows[k].column_index][qi]);
                    numerator = numerator + (value - (lc.a * QM31(dp.y) + lc.b));
                }
                acc = acc + numerator.mul_cm31(dinv[b]);
            }
            answers.push_back(acc);
        }
        return fri.decommit(answers);
    }
};

// ------------------------------------------------------------------ the word stream of PcsProof::to_words, read back
struct WordReader {
    const uint32_t* p;
    size_t n, at = 0;
    bool bad = false;
    uint32_t u32() { if (at >= n) { bad = true; return 0; } return p[at++]; }
    Hash hash() { Hash h{}; for (int i = 0; i < 8; i++) store_le32(&h[4 * i], u32()); return h; }
    QM31 q() { uint32_t a = u32(), b = u32(), c = u32(), d = u32(); return QM31::from_u32(a % P, b % P, c % P, d % P); }
    bool count(uint32_t& c, size_t words_each) { c = u32(); if (bad || (size_t)c * words_each > n - at) { bad = true; return false; } return true; }
    MerkleDecommitment dec() {
        MerkleDecommitment d;
        uint32_t c;
        if (!count(c, 8)) return d;
        for (uint32_t i = 0; i < c; i++) d.hash_witness.push_back(hash());
        if (!count(c, 1)) return d;
        for (uint32_t i = 0; i < c; i++) d.column_witness.push_back(M31(u32() % P));
        return d;
    }
    FriLayerProof layer() {
        FriLayerProof l;
        uint32_t c;
        if (!count(c, 4)) return l;
        for (uint32_t i = 0; i < c; i++) l.fri_witness.push_back(q());
        l.decommitment = dec();
        l.commitment = hash();
        return l;
    }
};
inline bool parse_pcs_proof(const uint32_t* words, size_t n, const std::vector<size_t>& tree_ncols, PcsProof& proof, size_t& consumed) {
    WordReader r{words, n};
    uint32_t c;
    if (!r.count(c, 8) || c != tree_ncols.size()) return false;
    for (uint32_t i = 0; i < c; i++) proof.commitments.push_back(r.hash());
    for (size_t t = 0; t < tree_ncols.size(); t++) {
        uint32_t nc;
        if (!r.count(nc, 1) || nc != tree_ncols[t]) return false;
        proof.sampled_values.emplace_back();
        for (uint32_t k = 0; k < nc; k++) {
            uint32_t ns;
            if (!r.count(ns, 4)) return false;
            std::vector<QM31> v;
            for (uint32_t s = 0; s < ns; s++) v.push_back(r.q());
            proof.sampled_values[t].push_back(v);
        }
    }
    for (size_t t = 0; t < tree_ncols.size(); t++) proof.decommitments.push_back(r.dec());
    for (size_t t = 0; t < tree_ncols.size(); t++) {
        uint32_t nv;
        if (!r.count(nv, 1)) return false;
        std::vector<M31> v;
        for (uint32_t k = 0; k < nv; k++) v.push_back(M31(r.u32() % P));
        proof.queried_values.push_back(v);
    }
    uint64_t lo = r.u32(), hi = r.u32();
    proof.proof_of_work = lo | (hi << 32);
    proof.fri.first_layer = r.layer();
    if (!r.count(c, 1)) return false;
    for (uint32_t i = 0; i < c && !r.bad; i++) proof.fri.inner_layers.push_back(r.layer());
    if (!r.count(c, 4)) return false;
    for (uint32_t i = 0; i < c; i++) proof.fri.last_layer_poly.push_back(r.q());
    consumed = r.at;
    return !r.bad;
}

}  // namespace zko
