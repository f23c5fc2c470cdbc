// TEST INFRASTRUCTURE ONLY (CPU oracle; see fields.hpp).
//
// The backend-generic protocol code of the reference that CALLS the operators, restated over the
// oracle's own operators so that whole commitments, FRI proofs and GKR proofs can be compared with
// the CUDA path word for word. Follows
//   nitroo/crates/stwo/src/prover/vcs/prover.rs:39-217        (MerkleProver::commit / decommit)
//   nitroo/crates/stwo/src/prover/fri.rs:109-467              (FriProver commit / decommit)
//   nitroo/crates/stwo/src/prover/line.rs:41-66               (LineEvaluation::interpolate, line_ifft)
//   nitroo/crates/stwo/src/prover/pcs/mod.rs:168-419, 481-630 (prove_values, CommitmentTreeProver)
//   nitroo/crates/stwo/src/prover/pcs/quotient_ops.rs:73-194  (compute_fri_quotients)
//   nitroo/crates/stwo/src/core/pcs/quotients.rs:306-345      (samples with randomness and periodicity)
//   nitroo/crates/stwo/src/core/pcs/mod.rs:47-69              (PcsConfig::mix_into)
//   nitroo/crates/stwo/src/core/circle.rs:147-163             (get_random_point)
//   nitroo/crates/stwo/src/prover/lookups/gkr_prover.rs:657-882 (prove_batch)
//   nitroo/crates/stwo/src/prover/lookups/sumcheck.rs:96-176  (sumcheck prove_batch)
//   nitroo/crates/stwo/src/prover/lookups/gkr_verifier.rs:17-149 (partially_verify_batch)
#pragma once
#include <omp.h>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <numeric>

#include "hash.hpp"
#include "ops.hpp"

namespace zko {

// ------------------------------------------------------------------ configuration
struct FriConfig {
    uint32_t log_blowup_factor = 1, log_last_layer_degree_bound = 0, n_queries = 3, line_fold_step = 1;
    size_t last_layer_domain_size() const { return (size_t)1 << (log_last_layer_degree_bound + log_blowup_factor); }
};
struct PcsConfig {
    uint32_t pow_bits = 10;
    FriConfig fri;
    uint32_t lifting_log_size = 0;  // 0 stands for None
    // core/pcs/mod.rs:47-69
    void mix_into(Channel& ch) const {
        QM31 f[2] = {QM31::from_u32(pow_bits, fri.log_blowup_factor, fri.n_queries, fri.log_last_layer_degree_bound),
                     QM31::from_u32(fri.line_fold_step, lifting_log_size, 0, 0)};
        ch.mix_felts(f, 2);
    }
};

// core/circle.rs:147-163
inline CirclePoint<QM31> get_random_point(Channel& ch) {
    QM31 t = ch.draw_secure_felt();
    QM31 t2 = t.square();
    QM31 inv = (t2 + QM31::one()).inverse();
    return {(QM31::one() - t2) * inv, t.dbl() * inv};
}

// ------------------------------------------------------------------ Merkle prover
struct MerkleDecommitment { std::vector<Hash> hash_witness; std::vector<M31> column_witness; };
struct ColumnRef { const M31* data; size_t len; };

struct MerkleProver {
    std::vector<std::vector<Hash>> layers;  // layers[log_size]; layers[0] is the root layer
    bool m31;
    // vcs/prover.rs:39-64
    static MerkleProver commit(const std::vector<ColumnRef>& columns, bool m31 = true) {
        MerkleProver mp;
        mp.m31 = m31;
        if (columns.empty()) {
            mp.layers.push_back(commit_on_layer(0, nullptr, {}, m31));
            return mp;
        }
        std::vector<ColumnRef> sorted(columns);
        std::stable_sort(sorted.begin(), sorted.end(), [](const ColumnRef& a, const ColumnRef& b) { return a.len > b.len; });
        uint32_t max_log = ilog2(sorted[0].len);
        mp.layers.resize(max_log + 1);
        size_t pos = 0;
        for (uint32_t log = max_log + 1; log-- > 0;) {
            std::vector<const M31*> layer_cols;
            while (pos < sorted.size() && ilog2(sorted[pos].len) == log) layer_cols.push_back(sorted[pos++].data);
            double t0 = omp_get_wtime();
            mp.layers[log] = commit_on_layer(log, log == max_log ? nullptr : &mp.layers[log + 1], layer_cols, m31);
            if (getenv("ZKO_TIMING") && log + 3 > max_log) fprintf(stderr, "[zko]   layer %u: %.3f s (%zu cols)\n", log, omp_get_wtime() - t0, layer_cols.size());
        }
        return mp;
    }
    Hash root() const { return layers[0][0]; }

    // vcs/prover.rs:84-217. Returns the queried values (largest layer first) and the decommitment.
    std::pair<std::vector<M31>, MerkleDecommitment> decommit(const std::map<uint32_t, std::vector<size_t>>& queries_per_log_size,
                                                             const std::vector<ColumnRef>& columns) const {
        std::vector<M31> queried_values;
        MerkleDecommitment dec;
        std::vector<ColumnRef> sorted(columns);
        std::stable_sort(sorted.begin(), sorted.end(), [](const ColumnRef& a, const ColumnRef& b) { return a.len > b.len; });
        size_t pos = 0;
        std::vector<size_t> last_layer_queries;
        for (uint32_t log = (uint32_t)layers.size(); log-- > 0;) {
            bool has_prev = (size_t)log + 1 < layers.size();
            std::set<size_t> prev_set(last_layer_queries.begin(), last_layer_queries.end());
            std::set<size_t> merged;
            for (auto q : last_layer_queries) merged.insert(q / 2);
            std::set<size_t> col_queries;
            auto it = queries_per_log_size.find(log);
            if (it != queries_per_log_size.end()) col_queries.insert(it->second.begin(), it->second.end());
            merged.insert(col_queries.begin(), col_queries.end());
            std::vector<size_t> merged_nodes(merged.begin(), merged.end());

            std::vector<const M31*> layer_cols;
            while (pos < sorted.size() && ilog2(sorted[pos].len) == log) layer_cols.push_back(sorted[pos++].data);

            std::vector<size_t> queried_nodes, witness_nodes;
            for (size_t node : merged_nodes) {
                if (has_prev) {
                    if (!prev_set.count(2 * node)) dec.hash_witness.push_back(layers[log + 1][2 * node]);
                    if (!prev_set.count(2 * node + 1)) dec.hash_witness.push_back(layers[log + 1][2 * node + 1]);
                }
                if (col_queries.count(node)) queried_nodes.push_back(node);
                else witness_nodes.push_back(node);
            }
            for (size_t node : queried_nodes)
                for (auto c : layer_cols) queried_values.push_back(c[node]);
            for (size_t node : witness_nodes)
                for (auto c : layer_cols) dec.column_witness.push_back(c[node]);
            last_layer_queries = merged_nodes;
        }
        return {queried_values, dec};
    }
};

// Coordinate columns of a secure column, for Merkle commitment.
struct CoordColumns {
    std::vector<M31> c[4];
    explicit CoordColumns(const SecureColumn& v) {
        for (int k = 0; k < 4; k++) c[k].resize(v.size());
        for (size_t i = 0; i < v.size(); i++) {
            uint32_t w[4]; v[i].to_u32(w);
            for (int k = 0; k < 4; k++) c[k][i] = M31(w[k]);
        }
    }
    std::vector<ColumnRef> refs() const {
        return {{c[0].data(), c[0].size()}, {c[1].data(), c[1].size()}, {c[2].data(), c[2].size()}, {c[3].data(), c[3].size()}};
    }
};

// ------------------------------------------------------------------ FRI prover
struct FriLayerProof { std::vector<QM31> fri_witness; MerkleDecommitment decommitment; Hash commitment; };
struct FriProof { FriLayerProof first_layer; std::vector<FriLayerProof> inner_layers; std::vector<QM31> last_layer_poly; };

// prover/line.rs:41-66 — bit-reversed evaluations on `domain` -> coefficients (LinePoly order).
inline std::vector<QM31> line_interpolate(std::vector<QM31> values, LineDomain domain) {
    bit_reverse(values.data(), values.size());
    LineDomain d = domain;
    while (d.size() > 1) {
        for (size_t off = 0; off < values.size(); off += d.size()) {
            size_t half = d.size() / 2;
            CirclePoint<M31> cur = d.coset.initial;
            for (size_t i = 0; i < half; i++) {
                ibutterfly(values[off + i], values[off + half + i], cur.x.inverse());
                cur = cur + d.coset.step;
            }
        }
        d = d.dbl();
    }
    M31 len_inv = M31::from_u32((uint32_t)values.size()).inverse();
    for (auto& v : values) v = v * len_inv;
    return values;
}

// prover/fri.rs:392-436
inline void decommitment_positions_and_witness(const SecureColumn& column, const std::vector<size_t>& queries, uint32_t fold_step,
                                               std::vector<size_t>& positions, std::vector<QM31>& witness) {
    size_t i = 0;
    while (i < queries.size()) {
        size_t j = i;
        while (j < queries.size() && (queries[j] >> fold_step) == (queries[i] >> fold_step)) j++;
        size_t start = (queries[i] >> fold_step) << fold_step;
        size_t qi = i;
        for (size_t p = start; p < start + ((size_t)1 << fold_step); p++) {
            positions.push_back(p);
            if (qi < j && queries[qi] == p) qi++;
            else witness.push_back(column[p]);
        }
        i = j;
    }
}

struct FriProver {
    FriConfig config;
    const SecureColumn* first_column;
    uint32_t first_log;
    MerkleProver first_tree;
    struct Inner { SecureColumn eval; MerkleProver tree; uint32_t fold_step; };
    std::vector<Inner> inner;
    std::vector<QM31> last_layer_poly;

    // prover/fri.rs:109-221
    static FriProver commit(Channel& ch, FriConfig config, const SecureColumn& column) {
        FriProver fp;
        fp.config = config;
        fp.first_column = &column;
        fp.first_log = ilog2(column.size());
        {
            CoordColumns cc(column);
            fp.first_tree = MerkleProver::commit(cc.refs(), ch.m31);
        }
        ch.mix_root(fp.first_tree.root());
        uint32_t inner_log = fp.first_log - 1;
        LineDomain dom{Coset::half_odds(inner_log)};
        SecureColumn layer((size_t)1 << inner_log, QM31::zero());
        QM31 alpha = ch.draw_secure_felt();
        fold_circle_into_line(layer, column, CanonicCoset(fp.first_log).circle_domain(), alpha);
        uint32_t last_log = ilog2(config.last_layer_domain_size());
        if (inner_log != last_log) {
            while (ilog2(layer.size()) > last_log + config.line_fold_step) {
                Inner in{layer, {}, config.line_fold_step};
                CoordColumns cc(in.eval);
                in.tree = MerkleProver::commit(cc.refs(), ch.m31);
                ch.mix_root(in.tree.root());
                QM31 a = ch.draw_secure_felt();
                layer = fold_line(in.eval, dom, a);
                dom = dom.dbl();
                fp.inner.push_back(std::move(in));
            }
            uint32_t last_step = ilog2(layer.size()) - last_log;
            Inner in{layer, {}, last_step};
            CoordColumns cc(in.eval);
            in.tree = MerkleProver::commit(cc.refs(), ch.m31);
            ch.mix_root(in.tree.root());
            QM31 a = ch.draw_secure_felt();
            for (uint32_t s = 0; s < last_step; s++) {  // cpu/fri.rs:15-30
                layer = fold_line(s == 0 ? in.eval : layer, dom, a);
                dom = dom.dbl();
                a = a * a;
            }
            fp.inner.push_back(std::move(in));
        }
        // commit_last_layer, prover/fri.rs:193-221
        assert(layer.size() == config.last_layer_domain_size());
        std::vector<QM31> coeffs = line_interpolate(layer, dom);
        bit_reverse(coeffs.data(), coeffs.size());  // into_ordered_coefficients
        size_t bound = (size_t)1 << config.log_last_layer_degree_bound;
        for (size_t i = bound; i < coeffs.size(); i++) assert(coeffs[i].is_zero() && "invalid degree");
        coeffs.resize(bound);
        bit_reverse(coeffs.data(), coeffs.size());  // from_ordered_coefficients
        fp.last_layer_poly = coeffs;
        ch.mix_felts(fp.last_layer_poly);
        return fp;
    }

    static FriLayerProof decommit_layer(const SecureColumn& col, const MerkleProver& tree, const std::vector<size_t>& queries,
                                        uint32_t fold_step) {
        FriLayerProof lp;
        std::vector<size_t> positions;
        decommitment_positions_and_witness(col, queries, fold_step, positions, lp.fri_witness);
        CoordColumns cc(col);
        std::map<uint32_t, std::vector<size_t>> q{{ilog2(col.size()), positions}};
        lp.decommitment = tree.decommit(q, cc.refs()).second;
        lp.commitment = tree.root();
        return lp;
    }

    // prover/fri.rs:223-281. Returns the proof, the sorted query positions and the unsorted draws.
    FriProof decommit(Channel& ch, std::vector<size_t>& query_positions, std::vector<size_t>& unsorted) const {
        unsorted = draw_queries(ch, first_log, config.n_queries);
        query_positions = sorted_dedup(unsorted);
        FriProof proof;
        proof.first_layer = decommit_layer(*first_column, first_tree, query_positions, 1);
        std::vector<size_t> q = fold_queries(query_positions, 1);
        for (auto& in : inner) {
            proof.inner_layers.push_back(decommit_layer(in.eval, in.tree, q, in.fold_step));
            q = fold_queries(q, in.fold_step);
        }
        proof.last_layer_poly = last_layer_poly;
        return proof;
    }
};

// ------------------------------------------------------------------ commitment scheme prover
struct CommitmentTree {
    std::vector<std::vector<M31>> coeffs;  // per column
    std::vector<std::vector<M31>> evals;   // per column, on the blown-up canonic domain
    MerkleProver tree;
    uint32_t max_log() const { return (uint32_t)tree.layers.size() - 1; }
};

struct PcsProof {
    std::vector<Hash> commitments;
    std::vector<std::vector<std::vector<QM31>>> sampled_values;  // tree, column, sample
    std::vector<MerkleDecommitment> decommitments;
    std::vector<std::vector<M31>> queried_values;
    uint64_t proof_of_work = 0;
    FriProof fri;
    // Flat word stream, the order the fields are listed in
    // nitroo/crates/stwo/src/core/pcs/quotients.rs:28-38 and core/fri.rs (FriProof, FriLayerProof).
    static void put_hash(std::vector<uint32_t>& o, const Hash& h) { for (int i = 0; i < 8; i++) o.push_back(load_le32(&h[4 * i])); }
    static void put_q(std::vector<uint32_t>& o, QM31 q) { uint32_t w[4]; q.to_u32(w); o.insert(o.end(), w, w + 4); }
    static void put_dec(std::vector<uint32_t>& o, const MerkleDecommitment& d) {
        o.push_back((uint32_t)d.hash_witness.size());
        for (auto& h : d.hash_witness) put_hash(o, h);
        o.push_back((uint32_t)d.column_witness.size());
        for (auto v : d.column_witness) o.push_back(v.v);
    }
    static void put_layer(std::vector<uint32_t>& o, const FriLayerProof& l) {
        o.push_back((uint32_t)l.fri_witness.size());
        for (auto q : l.fri_witness) put_q(o, q);
        put_dec(o, l.decommitment);
        put_hash(o, l.commitment);
    }
    std::vector<uint32_t> to_words() const {
        std::vector<uint32_t> o;
        o.push_back((uint32_t)commitments.size());
        for (auto& h : commitments) put_hash(o, h);
        for (auto& t : sampled_values) {
            o.push_back((uint32_t)t.size());
            for (auto& c : t) { o.push_back((uint32_t)c.size()); for (auto q : c) put_q(o, q); }
        }
        for (auto& d : decommitments) put_dec(o, d);
        for (auto& t : queried_values) { o.push_back((uint32_t)t.size()); for (auto v : t) o.push_back(v.v); }
        o.push_back((uint32_t)proof_of_work);
        o.push_back((uint32_t)(proof_of_work >> 32));
        put_layer(o, fri.first_layer);
        o.push_back((uint32_t)fri.inner_layers.size());
        for (auto& l : fri.inner_layers) put_layer(o, l);
        o.push_back((uint32_t)fri.last_layer_poly.size());
        for (auto q : fri.last_layer_poly) put_q(o, q);
        return o;
    }
};

// Phase times on stderr when ZKO_TIMING is set (a diagnostic for the timed CPU baseline).
struct PhaseClock {
    bool on = getenv("ZKO_TIMING") != nullptr;
    double t0 = on ? omp_get_wtime() : 0.0;
    void lap(const char* name) {
        if (!on) return;
        double t1 = omp_get_wtime();
        fprintf(stderr, "[zko] %-12s %.3f s\n", name, t1 - t0);
        t0 = t1;
    }
};

struct CommitmentSchemeProver {
    PcsConfig config;
    std::vector<CommitmentTree> trees;
    TwiddleTree twiddles;  // rooted at the half coset of the largest blown-up domain

    CommitmentSchemeProver(PcsConfig cfg, uint32_t max_lde_log) : config(cfg), twiddles(precompute_twiddles(Coset::half_odds(max_lde_log - 1))) {}

    // TreeBuilder::extend_evals + commit (pcs/mod.rs:429-464, 481-537): interpolate each column,
    // extend by the blow-up factor, build the Merkle tree, mix the root.
    void commit_evals(const std::vector<std::vector<M31>>& columns, Channel& ch) {
        CommitmentTree t;
        t.evals.resize(columns.size());
        t.coeffs.resize(columns.size());
        PhaseClock clock;
#pragma omp parallel for schedule(dynamic)
        for (size_t k = 0; k < columns.size(); k++) {
            const auto& col = columns[k];
            uint32_t log = ilog2(col.size());
            std::vector<M31> c(col);
            interpolate(c, CanonicCoset(log).circle_domain(), twiddles);
            t.evals[k] = evaluate(c, CanonicCoset(log + config.fri.log_blowup_factor).circle_domain(), twiddles);
            t.coeffs[k] = std::move(c);
        }
        clock.lap("fft");
        std::vector<ColumnRef> refs;
        for (auto& e : t.evals) refs.push_back({e.data(), e.size()});
        t.tree = MerkleProver::commit(refs, ch.m31);
        ch.mix_root(t.tree.root());
        clock.lap("merkle");
        trees.push_back(std::move(t));
    }

    // pcs/quotient_ops.rs:73-194 with core/pcs/quotients.rs:306-345 and :75-104
    SecureColumn compute_fri_quotients(const std::vector<std::vector<std::vector<PointSample>>>& samples, QM31 random_coeff,
                                       uint32_t lifting_log) const {
        // flat columns, log sizes and samples with their random powers (and the periodicity sample)
        std::vector<const std::vector<M31>*> flat_cols;
        std::vector<uint32_t> flat_logs;
        std::vector<std::vector<std::pair<PointSample, QM31>>> flat_samples;
        QM31 pow = QM31::one();
        CirclePoint<M31> lifting_gen = CanonicCoset(lifting_log).step();
        for (size_t t = 0; t < trees.size(); t++)
            for (size_t c = 0; c < trees[t].evals.size(); c++) {
                uint32_t log_size = ilog2(trees[t].evals[c].size());
                flat_cols.push_back(&trees[t].evals[c]);
                flat_logs.push_back(log_size);
                std::vector<std::pair<PointSample, QM31>> v;
                const auto& sc = samples[t][c];
                if (!sc.empty()) {
                    if (sc.size() == 2) {
                        CirclePoint<M31> period = lifting_gen.repeated_double(log_size);
                        v.push_back({PointSample{sc[1].point + into_ef(period), sc[1].value}, pow});
                        pow = pow * random_coeff;
                    }
                    for (auto& s : sc) { v.push_back({s, pow}); pow = pow * random_coeff; }
                }
                flat_samples.push_back(v);
            }
        // group by log size (ascending, stable)
        std::vector<size_t> order(flat_cols.size());
        std::iota(order.begin(), order.end(), 0);
        std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) { return flat_logs[a] < flat_logs[b]; });
        std::vector<AccumulatedNumerators> accs;
        for (size_t i = 0; i < order.size();) {
            size_t j = i;
            while (j < order.size() && flat_logs[order[j]] == flat_logs[order[i]]) j++;
            std::vector<const M31*> group_cols;
            std::vector<ColumnSampleBatch> batches;  // insertion-ordered by point
            for (size_t k = i; k < j; k++) {
                size_t ci = k - i;
                group_cols.push_back(flat_cols[order[k]]->data());
                for (auto& sp : flat_samples[order[k]]) {
                    ColumnSampleBatch* b = nullptr;
                    for (auto& x : batches) if (x.point == sp.first.point) { b = &x; break; }
                    if (!b) { batches.push_back({sp.first.point, {}}); b = &batches.back(); }
                    b->cols_vals_randpows.push_back({ci, sp.first.value, sp.second});
                }
            }
            accumulate_numerators(group_cols, (size_t)1 << flat_logs[order[i]], batches, accs);
            i = j;
        }
        // one accumulation per sample point: sort by (point.x, point.y), lift and accumulate ascending sizes
        auto key = [](const QM31& q) { uint32_t w[4]; q.to_u32(w); return std::array<uint32_t, 4>{w[0], w[1], w[2], w[3]}; };
        std::stable_sort(accs.begin(), accs.end(), [&](const AccumulatedNumerators& a, const AccumulatedNumerators& b) {
            auto ka = std::make_pair(key(a.sample_point.x), key(a.sample_point.y));
            auto kb = std::make_pair(key(b.sample_point.x), key(b.sample_point.y));
            return ka < kb;
        });
        std::vector<AccumulatedNumerators> per_point;
        for (size_t i = 0; i < accs.size();) {
            size_t j = i;
            while (j < accs.size() && accs[j].sample_point == accs[i].sample_point) j++;
            QM31 first = QM31::zero();
            std::vector<SecureColumn> cols;
            for (size_t k = i; k < j; k++) { first = first + accs[k].first_linear_term_acc; cols.push_back(accs[k].partial_numerators_acc); }
            per_point.push_back({accs[i].sample_point, lift_and_accumulate(cols), first});
            i = j;
        }
        return compute_quotients_and_combine(per_point, lifting_log);
    }

    // pcs/mod.rs:168-419
    PcsProof prove_values(const std::vector<std::vector<std::vector<CirclePoint<QM31>>>>& sampled_points, Channel& ch) {
        PcsProof proof;
        PhaseClock clock;
        uint32_t lifting_log = trees.back().max_log();
        std::vector<std::vector<std::vector<PointSample>>> samples(trees.size());
        std::vector<QM31> flat_values;
        for (size_t t = 0; t < trees.size(); t++) {
            samples[t].resize(trees[t].coeffs.size());
            proof.sampled_values.emplace_back();
#pragma omp parallel for schedule(dynamic)
            for (size_t c = 0; c < trees[t].coeffs.size(); c++) {
                uint32_t poly_log = ilog2(trees[t].evals[c].size());
                for (auto& p : sampled_points[t][c])
                    samples[t][c].push_back({p, eval_at_point(trees[t].coeffs[c], p.repeated_double(lifting_log - poly_log))});
            }
            for (size_t c = 0; c < trees[t].coeffs.size(); c++) {
                std::vector<QM31> vals;
                for (auto& smp : samples[t][c]) { vals.push_back(smp.value); flat_values.push_back(smp.value); }
                proof.sampled_values[t].push_back(vals);
            }
        }
        clock.lap("sample");
        ch.mix_felts(flat_values);
        QM31 random_coeff = ch.draw_secure_felt();
        SecureColumn quotients = compute_fri_quotients(samples, random_coeff, lifting_log);
        clock.lap("quotients");
        FriProver fri = FriProver::commit(ch, config.fri, quotients);
        clock.lap("fri_commit");
        proof.proof_of_work = ch.grind(config.pow_bits);
        ch.mix_u64(proof.proof_of_work);
        clock.lap("grind");
        std::vector<size_t> query_positions, unsorted;
        proof.fri = fri.decommit(ch, query_positions, unsorted);
        for (auto& t : trees) {
            // core/pcs/utils.rs:200-218 then pcs/mod.rs:575-630
            uint32_t tree_max = t.max_log();
            std::vector<size_t> q;
            for (auto pos : query_positions) q.push_back(((pos >> (lifting_log - tree_max + 1)) << 1) + (pos & 1));
            std::map<uint32_t, std::vector<size_t>> per_log;
            std::vector<ColumnRef> refs;
            for (auto& e : t.evals) {
                refs.push_back({e.data(), e.size()});
                uint32_t log = ilog2(e.size());
                if (per_log.count(log)) continue;
                uint32_t shift = tree_max - log;
                std::vector<size_t> positions;
                for (auto pos : q) positions.push_back(((pos >> (shift + 1)) << 1) + (pos & 1));
                per_log[log] = sorted_dedup(positions);
            }
            auto r = t.tree.decommit(per_log, refs);
            proof.queried_values.push_back(r.first);
            proof.decommitments.push_back(r.second);
            proof.commitments.push_back(t.tree.root());
        }
        return proof;
    }
};

// ------------------------------------------------------------------ GKR
struct GkrProof {
    std::vector<std::vector<UnivariatePoly>> sumcheck_round_polys;  // per layer
    std::vector<std::vector<std::vector<std::array<QM31, 2>>>> layer_masks_by_instance;  // instance, layer, column
    std::vector<std::vector<QM31>> output_claims_by_instance;
    std::vector<QM31> ood_point;
    std::vector<std::vector<QM31>> claims_to_verify_by_instance;
    std::vector<uint32_t> to_words() const {
        std::vector<uint32_t> o;
        auto put = [&](QM31 q) { uint32_t w[4]; q.to_u32(w); o.insert(o.end(), w, w + 4); };
        o.push_back((uint32_t)sumcheck_round_polys.size());
        for (auto& l : sumcheck_round_polys) {
            o.push_back((uint32_t)l.size());
            for (auto& p : l) { o.push_back((uint32_t)p.c.size()); for (auto q : p.c) put(q); }
        }
        for (auto& inst : layer_masks_by_instance) {
            o.push_back((uint32_t)inst.size());
            for (auto& m : inst) { o.push_back((uint32_t)m.size()); for (auto& col : m) { put(col[0]); put(col[1]); } }
        }
        for (auto& c : output_claims_by_instance) { o.push_back((uint32_t)c.size()); for (auto q : c) put(q); }
        o.push_back((uint32_t)ood_point.size());
        for (auto q : ood_point) put(q);
        for (auto& c : claims_to_verify_by_instance) { o.push_back((uint32_t)c.size()); for (auto q : c) put(q); }
        return o;
    }
};

// lookups/utils.rs:160-163
inline QM31 random_linear_combination(const std::vector<QM31>& v, QM31 alpha) { return horner_eval(v, alpha); }

struct GkrOracle {  // GkrMultivariatePolyOracle, gkr_prover.rs:473-556
    const std::vector<QM31>* eq_evals;
    const std::vector<QM31>* y;
    Layer input_layer;
    QM31 eq_fixed_var_correction;
    QM31 lambda;
    size_t n_variables() const { return input_layer.n_variables() - 1; }
};

// cpu/lookups/gkr.rs:39-71
inline UnivariatePoly sum_as_poly_in_first_variable(const GkrOracle& h, QM31 claim) {
    size_t nv = h.n_variables();
    size_t n_terms = (size_t)1 << (nv - 1);
    QM31 at0, at2;
    round_sums(h.input_layer, h.eq_evals->data(), n_terms, h.lambda, at0, at2);
    at0 = at0 * h.eq_fixed_var_correction;
    at2 = at2 * h.eq_fixed_var_correction;
    return correct_sum_as_poly_in_first_variable(at0, at2, claim, *h.y, nv);
}

// gkr_prover.rs:572-597
inline std::vector<std::array<QM31, 2>> oracle_into_mask(const GkrOracle& o) {
    const Layer& l = o.input_layer;
    assert(l.len() == 2);
    switch (l.kind) {
        case GRAND_PRODUCT: return {{l.den[0], l.den[1]}};
        case LOGUP_GENERIC: return {{l.num[0], l.num[1]}, {l.den[0], l.den[1]}};
        case LOGUP_SINGLES: return {{QM31::one(), QM31::one()}, {l.den[0], l.den[1]}};
        default: assert(false && "multiplicities layer cannot be a mask"); return {};
    }
}

// gkr_prover.rs:657-882 with sumcheck.rs:96-176
inline GkrProof gkr_prove_batch(Channel& ch, std::vector<Layer> input_layers) {
    size_t n_inst = input_layers.size();
    std::vector<size_t> n_layers_by_inst;
    for (auto& l : input_layers) n_layers_by_inst.push_back(l.n_variables());
    size_t n_layers = *std::max_element(n_layers_by_inst.begin(), n_layers_by_inst.end());
    // gen_layers: the whole tower per instance, consumed output layer first
    std::vector<std::vector<Layer>> towers(n_inst);
    for (size_t i = 0; i < n_inst; i++) {
        towers[i].push_back(std::move(input_layers[i]));
        while (towers[i].back().n_variables() > 0) towers[i].push_back(next_layer(towers[i].back()));
    }
    std::vector<size_t> cursor(n_inst);
    for (size_t i = 0; i < n_inst; i++) cursor[i] = towers[i].size();  // next to take is towers[i][cursor-1]

    GkrProof proof;
    proof.layer_masks_by_instance.resize(n_inst);
    proof.output_claims_by_instance.resize(n_inst);
    std::vector<std::vector<QM31>> claims(n_inst);
    std::vector<bool> active(n_inst, false);
    std::vector<QM31> ood_point;

    for (size_t layer = 0; layer < n_layers; layer++) {
        size_t n_remaining = n_layers - layer;
        for (size_t i = 0; i < n_inst; i++)
            if (n_layers_by_inst[i] == n_remaining) {
                const Layer& out = towers[i][--cursor[i]];
                std::vector<QM31> vals;
                if (out.kind == GRAND_PRODUCT) vals = {out.den[0]};
                else vals = {out.numerator_at(0), out.den[0]};
                claims[i] = vals;
                proof.output_claims_by_instance[i] = vals;
                active[i] = true;
            }
        for (size_t i = 0; i < n_inst; i++)
            if (active[i]) ch.mix_felts(claims[i]);
        // EqEvals::generate, gkr_prover.rs:235-247
        std::vector<QM31> eq_evals;
        if (ood_point.empty()) eq_evals = {QM31::one()};
        else eq_evals = gen_eq_evals(ood_point.data() + 1, ood_point.size() - 1, eq1(QM31::zero(), ood_point[0]));
        QM31 sumcheck_alpha = ch.draw_secure_felt();
        QM31 instance_lambda = ch.draw_secure_felt();
        std::vector<GkrOracle> oracles;
        std::vector<QM31> sc_claims;
        std::vector<size_t> sc_inst;
        for (size_t i = 0; i < n_inst; i++)
            if (active[i]) {
                oracles.push_back({&eq_evals, &ood_point, towers[i][--cursor[i]], QM31::one(), instance_lambda});
                sc_claims.push_back(random_linear_combination(claims[i], instance_lambda));
                sc_inst.push_back(i);
            }
        // sumcheck::prove_batch
        size_t nv = 0;
        for (auto& o : oracles) nv = std::max(nv, o.n_variables());
        for (size_t k = 0; k < oracles.size(); k++)
            sc_claims[k] = sc_claims[k] * M31::from_u32(1u << (nv - oracles[k].n_variables()));
        std::vector<UnivariatePoly> round_polys;
        std::vector<QM31> assignment;
        for (size_t round = 0; round < nv; round++) {
            size_t n_rem = nv - round;
            std::vector<UnivariatePoly> this_round;
            for (size_t k = 0; k < oracles.size(); k++) {
                UnivariatePoly rp;
                if (n_rem == oracles[k].n_variables()) rp = sum_as_poly_in_first_variable(oracles[k], sc_claims[k]);
                else { rp.c = {sc_claims[k] * M31(2).inverse()}; rp.trim(); }
                assert(rp.eval(QM31::zero()) + rp.eval(QM31::one()) == sc_claims[k]);
                assert(rp.degree() <= 3);
                this_round.push_back(rp);
            }
            UnivariatePoly combined;  // rfold(acc * alpha + poly)
            for (size_t k = this_round.size(); k-- > 0;) {
                for (auto& c : combined.c) c = c * sumcheck_alpha;
                combined = UnivariatePoly::add(combined, this_round[k]);
            }
            ch.mix_felts(combined.c);
            QM31 challenge = ch.draw_secure_felt();
            for (size_t k = 0; k < oracles.size(); k++) sc_claims[k] = this_round[k].eval(challenge);
            for (size_t k = 0; k < oracles.size(); k++)
                if (n_rem == oracles[k].n_variables() && oracles[k].n_variables() != 0) {
                    GkrOracle& o = oracles[k];
                    QM31 z0 = (*o.y)[o.y->size() - o.n_variables()];
                    o.eq_fixed_var_correction = o.eq_fixed_var_correction * eq1(challenge, z0);
                    o.input_layer = layer_fix_first_variable(o.input_layer, challenge);
                }
            round_polys.push_back(combined);
            assignment.push_back(challenge);
        }
        proof.sumcheck_round_polys.push_back(round_polys);
        std::vector<std::vector<std::array<QM31, 2>>> masks;
        for (auto& o : oracles) masks.push_back(oracle_into_mask(o));
        for (size_t k = 0; k < oracles.size(); k++) {
            std::vector<QM31> flat;
            for (auto& col : masks[k]) { flat.push_back(col[0]); flat.push_back(col[1]); }
            ch.mix_felts(flat);
            proof.layer_masks_by_instance[sc_inst[k]].push_back(masks[k]);
        }
        QM31 challenge = ch.draw_secure_felt();
        ood_point = assignment;
        ood_point.push_back(challenge);
        for (size_t k = 0; k < oracles.size(); k++) {
            std::vector<QM31> next;
            for (auto& col : masks[k]) next.push_back(fold_mle_evals(challenge, col[0], col[1]));
            claims[sc_inst[k]] = next;
        }
    }
    proof.ood_point = ood_point;
    proof.claims_to_verify_by_instance = claims;
    return proof;
}

// gkr_verifier.rs:17-149 (gates: GrandProduct multiplies the mask column, LogUp adds the two
// fractions, gkr_verifier.rs:180-215). Returns true when every layer's circuit check passes and
// fills the artifact (ood point, claims to verify).
inline bool gkr_partially_verify_batch(const std::vector<int>& gate_is_logup, const GkrProof& proof, Channel& ch,
                                       std::vector<QM31>& ood_out, std::vector<std::vector<QM31>>& claims_out) {
    size_t n_inst = proof.layer_masks_by_instance.size();
    if (n_inst != proof.output_claims_by_instance.size() || gate_is_logup.size() != n_inst) return false;
    auto inst_layers = [&](size_t i) { return proof.layer_masks_by_instance[i].size(); };
    size_t n_layers = 0;
    for (size_t i = 0; i < n_inst; i++) n_layers = std::max(n_layers, inst_layers(i));
    if (n_layers != proof.sumcheck_round_polys.size()) return false;
    std::vector<QM31> ood_point;
    std::vector<std::vector<QM31>> claims(n_inst);
    std::vector<bool> active(n_inst, false);
    for (size_t layer = 0; layer < n_layers; layer++) {
        size_t n_remaining = n_layers - layer;
        for (size_t i = 0; i < n_inst; i++)
            if (inst_layers(i) == n_remaining) { claims[i] = proof.output_claims_by_instance[i]; active[i] = true; }
        for (size_t i = 0; i < n_inst; i++)
            if (active[i]) ch.mix_felts(claims[i]);
        QM31 sumcheck_alpha = ch.draw_secure_felt();
        QM31 instance_lambda = ch.draw_secure_felt();
        std::vector<QM31> sc_claims;
        std::vector<size_t> sc_inst;
        for (size_t i = 0; i < n_inst; i++)
            if (active[i]) {
                size_t unused = n_layers - inst_layers(i);
                sc_claims.push_back(random_linear_combination(claims[i], instance_lambda) * M31::from_u32(1u << unused));
                sc_inst.push_back(i);
            }
        QM31 claim = random_linear_combination(sc_claims, sumcheck_alpha);
        // sumcheck::partially_verify, sumcheck.rs:190-230
        std::vector<QM31> assignment;
        for (auto& rp : proof.sumcheck_round_polys[layer]) {
            if (rp.degree() > 3) return false;
            if (!(rp.eval(QM31::zero()) + rp.eval(QM31::one()) == claim)) return false;
            ch.mix_felts(rp.c);
            QM31 challenge = ch.draw_secure_felt();
            claim = rp.eval(challenge);
            assignment.push_back(challenge);
        }
        std::vector<QM31> layer_evals;
        for (size_t i : sc_inst) {
            size_t unused = n_layers - inst_layers(i);
            auto& mask = proof.layer_masks_by_instance[i][layer - unused];
            std::vector<QM31> gate_out;
            if (gate_is_logup[i]) {
                if (mask.size() != 2) return false;
                QM31 n0 = mask[0][0], n1 = mask[0][1], d0 = mask[1][0], d1 = mask[1][1];
                gate_out = {d1 * n0 + d0 * n1, d0 * d1};
            } else {
                if (mask.size() != 1) return false;
                gate_out = {mask[0][0] * mask[0][1]};
            }
            QM31 eq_eval = eq(ood_point.data() + unused, assignment.data() + unused, ood_point.size() - unused);
            layer_evals.push_back(eq_eval * random_linear_combination(gate_out, instance_lambda));
        }
        if (!(claim == random_linear_combination(layer_evals, sumcheck_alpha))) return false;
        for (size_t i : sc_inst) {
            size_t unused = n_layers - inst_layers(i);
            auto& mask = proof.layer_masks_by_instance[i][layer - unused];
            std::vector<QM31> flat;
            for (auto& col : mask) { flat.push_back(col[0]); flat.push_back(col[1]); }
            ch.mix_felts(flat);
        }
        QM31 challenge = ch.draw_secure_felt();
        ood_point = assignment;
        ood_point.push_back(challenge);
        for (size_t i : sc_inst) {
            size_t unused = n_layers - inst_layers(i);
            auto& mask = proof.layer_masks_by_instance[i][layer - unused];
            std::vector<QM31> next;
            for (auto& col : mask) next.push_back(fold_mle_evals(challenge, col[0], col[1]));
            claims[i] = next;
        }
    }
    ood_out = ood_point;
    claims_out = claims;
    return true;
}

}  // namespace zko
