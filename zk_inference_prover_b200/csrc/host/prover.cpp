// Protocol drivers over B200Backend: Merkle prover, FRI prover, commitment-scheme prover and the
// GKR batch prover, with the call order of the reference's backend-generic code (cited per
// function; STWO = nitroo/crates/stwo/src). All field and hash work on columns happens on the
// device through the operator ABI; the host runs the Fiat-Shamir channel, the query bookkeeping
// and scalar QM31 arithmetic on a handful of values per round.
#include <algorithm>
#include <iterator>
#include <chrono>
#include <map>
#include <memory>
#include <numeric>
#include <set>
#include <string>
#include <thread>
#include <cstdio>
#include <cstdlib>

#include <cuda_runtime_api.h>

#include "../../../include/zkb200_prover.h"
#include "../air_program.hpp"
#include "b200_backend.hpp"
#include "../fft_internal.hpp"
#include "../gkr_resident.hpp"
#include "../gkr_batch.hpp"
#include "../gather_blocks.hpp"
#include "channel.hpp"

// Records a message on the context (defined with the context, ctx.cu).
extern "C" int zk_set_error_public(zkb_ctx* ctx, int code, const char* msg);

namespace b200 {

using namespace zk;

// Host-side timing of the protocol code's own steps (the device has per-kernel events; this is for the time the host
// spends between launches). Off unless ZKB_HOST_TIMING is set; totals per label go to stderr when a proof call returns.
struct HostClock {
    static bool on() { static const bool v = getenv("ZKB_HOST_TIMING") != nullptr; return v; }
    static std::map<std::string, std::pair<double, size_t>>& totals() { static std::map<std::string, std::pair<double, size_t>> m; return m; }
    const char* label;
    std::chrono::steady_clock::time_point t0;
    explicit HostClock(const char* l) : label(l) { if (on()) t0 = std::chrono::steady_clock::now(); }
    ~HostClock() {
        if (!on()) return;
        auto& e = totals()[label];
        e.first += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        e.second++;
    }
    static void dump(const char* what) {
        if (!on()) return;
        fprintf(stderr, "[host timing] %s\n", what);
        for (auto& kv : totals()) fprintf(stderr, "  %-34s %10.3f ms %8zu calls\n", kv.first.c_str(), kv.second.first, kv.second.second);
        totals().clear();
    }
};

static inline uint32_t ilog2(size_t n) { return n ? 63u - (uint32_t)__builtin_clzll((unsigned long long)n) : 0u; }
static inline qm31 operator+(qm31 a, qm31 b) { return qm31_add(a, b); }
static inline qm31 operator-(qm31 a, qm31 b) { return qm31_sub(a, b); }
static inline qm31 operator*(qm31 a, qm31 b) { return qm31_mul(a, b); }

static std::vector<size_t> sorted_dedup(std::vector<size_t> v) {
    std::sort(v.begin(), v.end());
    v.erase(std::unique(v.begin(), v.end()), v.end());
    return v;
}
static std::vector<size_t> fold_queries(const std::vector<size_t>& q, uint32_t n_folds) {  // core/queries.rs:55-62
    std::vector<size_t> out;
    for (auto x : q) { size_t y = x >> n_folds; if (out.empty() || out.back() != y) out.push_back(y); }
    return out;
}

// Every address a decommitment will read is known once the query positions are: collect them all,
// read them in one device round trip, then assemble the proof parts from the results.
struct GatherPlan {
    std::vector<const uint32_t*> addrs;
    std::vector<uint32_t> words;
    size_t add(const uint32_t* p) { addrs.push_back(p); return addrs.size() - 1; }
    size_t add_hash(const uint32_t* p) { size_t s = addrs.size(); for (int k = 0; k < 8; k++) addrs.push_back(p + k); return s; }
    // Rows of many columns at once (the queried and witness values of one tree layer): row-major [row][column] in
    // block_words from the returned offset. One pointer per column and one index per row travel, not one address per word.
    struct Block { std::vector<const uint32_t*> cols; std::vector<uint32_t> idx; size_t out_off; };
    std::vector<Block> blocks;
    // Tens of megabytes for trees of many columns. The buffer is kept per thread between proofs: a fresh allocation of
    // that size comes from mmap, and its first-touch page faults cost as much as the gather itself.
    uint32_t* block_words = nullptr;
    size_t block_total = 0;
    // Page-locked once it is large (from 4 MiB): the device-to-host copy of a wide tree's values then runs at the link's
    // speed instead of through the driver's bounce buffers (50 MB: 4 ms pageable). Small buffers stay ordinary memory:
    // pinning costs more than it saves there.
    struct Arena {
        uint32_t* p = nullptr;
        size_t words = 0;
        bool pinned = false;
        void release() {
            if (!p) return;
            if (pinned) cudaFreeHost(p); else free(p);
            p = nullptr; words = 0;
        }
        // Nothing is released when the thread ends: at process exit the CUDA runtime may already be gone.
    };
    static uint32_t* arena(size_t words) {
        thread_local Arena a;
        if (a.words < words) {
            a.release();
            size_t want = words + words / 4;
            void* q = nullptr;
            if (want * 4 >= ((size_t)4 << 20) && cudaMallocHost(&q, want * 4) == cudaSuccess && q) a.pinned = true;
            else { (void)cudaGetLastError(); q = malloc(want * 4); a.pinned = false; }
            if (!q) throw Error(ZKB_ENOMEM, "gather buffer");
            a.p = (uint32_t*)q;
            a.words = want;
        }
        return a.p;
    }
    size_t add_block(const std::vector<const uint32_t*>& cols, const std::vector<size_t>& rows) {
        Block b;
        b.cols = cols;
        for (auto r : rows) b.idx.push_back((uint32_t)r);
        b.out_off = block_total;
        block_total += cols.size() * rows.size();
        blocks.push_back(std::move(b));
        return blocks.back().out_off;
    }
    void execute(const Device& d) {
        words.resize(addrs.size());
        d.check(zkb_gather_words(d.ctx(), addrs.data(), addrs.size(), words.data()));
        if (block_total) {
            block_words = arena(block_total);
            std::vector<zk::GatherBlock> gb;
            for (auto& b : blocks) gb.push_back({b.cols.data(), (int)b.cols.size(), b.idx.data(), (int)b.idx.size(), b.out_off});
            d.check(zk::gather_blocks(d.ctx(), gb.data(), (int)gb.size(), block_total, block_words));
        }
    }
    Hash hash_at(size_t slot) const { Hash h; for (int k = 0; k < 8; k++) h[k] = words[slot + k]; return h; }
};

// ------------------------------------------------------------------ MerkleProver (STWO/prover/vcs/prover.rs:17-217)
// A word sequence of a proof: its own vector, or runs inside the gather buffer of the plan that read them (the buffer is
// kept per thread until the next proof on that thread, so a proof can be serialised straight out of it: a tree of tens of
// thousands of columns has tens of megabytes of queried values, and every copy of them costs milliseconds).
struct Words {
    std::vector<uint32_t> own;
    std::vector<std::pair<const uint32_t*, size_t>> runs;
    size_t size() const { size_t n = own.size(); for (auto& r : runs) n += r.second; return n; }
    template <class O> void append_to(O& o) const {
        o.insert(o.end(), own.begin(), own.end());
        for (auto& r : runs) o.insert(o.end(), r.first, r.first + r.second);
    }
};
struct MerkleDecommitment { std::vector<Hash> hash_witness; Words column_witness; };
struct PendingMerkle {  // slots of a planned decommitment
    std::vector<size_t> hash_slots;
    struct Run { size_t off, count; bool queried; };  // `count` words of plan.block_words, in proof order
    std::vector<Run> runs;
    std::pair<Words, MerkleDecommitment> finish(const GatherPlan& plan) const {
        std::pair<Words, MerkleDecommitment> r;
        r.second.hash_witness.reserve(hash_slots.size());
        for (auto s : hash_slots) r.second.hash_witness.push_back(plan.hash_at(s));
        for (auto& run : runs) (run.queried ? r.first : r.second.column_witness).runs.push_back({plan.block_words + run.off, run.count});
        return r;
    }
};

struct MerkleProver {
    std::vector<HashColumn> layers;  // layers[log_size]; layers[0] holds the root
    // the committed columns of each layer (device addresses, in commitment order), kept for the decommitment: sorting tens
    // of thousands of columns by size a second time costs milliseconds
    std::vector<std::vector<const uint32_t*>> layer_col_ptrs;
    size_t n_columns = 0;

    // `leaves`, when given, is the already hashed largest layer (see zkb_merkle_leaves_partial).
    // `chan_step`, when given, is a FRI layer's channel step (channel state, challenge slot, root copy; device addresses) to run
    // in the launch that builds the root; *chan_done says whether it ran (a tree of one node has no such launch).
    struct ChanStep { uint32_t *chan, *alpha, *root_copy; };
    static MerkleProver commit(const Device& d, const std::vector<const BaseColumn*>& columns, HashColumn* leaves = nullptr,
                               const ChanStep* chan_step = nullptr, bool* chan_done = nullptr) {  // :39-64
        if (chan_done) *chan_done = false;
        auto top = [&](uint32_t log, uint32_t* top_layer, uint32_t** lower) {
            if (chan_step && log >= 1) {
                d.check(zkb_merkle_top_channel(d.ctx(), (int)log, top_layer, lower, 1, chan_step->chan, chan_step->alpha, chan_step->root_copy));
                if (chan_done) *chan_done = true;
            } else d.check(zkb_merkle_top(d.ctx(), (int)log, top_layer, lower, 1));
        };
        MerkleProver mp;
        if (columns.empty()) {
            mp.layers.push_back(B200Backend::commit_on_layer(d, 0, nullptr, {}));
            return mp;
        }
        std::vector<const BaseColumn*> sorted(columns);
        std::stable_sort(sorted.begin(), sorted.end(), [](const BaseColumn* a, const BaseColumn* b) { return a->len() > b->len(); });
        uint32_t max_log = sorted[0]->log_size();
        mp.layers.resize(max_log + 1);
        mp.layer_col_ptrs.resize(max_log + 1);
        mp.n_columns = sorted.size();
        size_t pos = 0;
        for (uint32_t log = max_log + 1; log-- > 0;) {
            std::vector<const BaseColumn*> layer_cols;
            while (pos < sorted.size() && sorted[pos]->log_size() == log) layer_cols.push_back(sorted[pos++]);
            for (auto c : layer_cols) mp.layer_col_ptrs[log].push_back(c->ptr());
            if (log == max_log && leaves) mp.layers[log] = std::move(*leaves);
            else mp.layers[log] = B200Backend::commit_on_layer(d, log, log == max_log ? nullptr : &mp.layers[log + 1], layer_cols);
            if (log > 0 && log <= 10 && pos == sorted.size()) {
                // no columns left below: the rest of the tree is nodes only, built in one launch
                std::vector<uint32_t*> lower;
                for (uint32_t k = 0; k < log; k++) { mp.layers[k] = HashColumn(d, (size_t)8 << k); lower.push_back(mp.layers[k].ptr()); }
                top(log, mp.layers[log].ptr(), lower.data());
                break;
            }
            // The layers below this one that hold no column (down to the next layer that has one, or to the last ten, which
            // the launch above builds): up to nine of them per launch.
            const uint32_t floor_log = pos == sorted.size() ? 10u : sorted[pos]->log_size() + 1;
            while (log > floor_log && log >= 9) {
                const uint32_t levels = std::min<uint32_t>(9, log - floor_log);
                std::vector<uint32_t*> outs;
                for (uint32_t j = 1; j <= levels; j++) { mp.layers[log - j] = HashColumn(d, (size_t)8 << (log - j)); outs.push_back(mp.layers[log - j].ptr()); }
                d.check(zkb_merkle_levels(d.ctx(), (int)log, mp.layers[log].ptr(), (int)levels, outs.data(), 1));
                log -= levels;
            }
            if (log > 0 && log <= 10 && pos == sorted.size() && mp.layers[log - 1].len() == 0) {
                std::vector<uint32_t*> lower;
                for (uint32_t k = 0; k < log; k++) { mp.layers[k] = HashColumn(d, (size_t)8 << k); lower.push_back(mp.layers[k].ptr()); }
                top(log, mp.layers[log].ptr(), lower.data());
                break;
            }
        }
        return mp;
    }
    Hash root(const Device& d) const {
        if (!have_root) { root_cache = B200Backend::batch_at(d, layers[0], {0})[0]; have_root = true; }
        return root_cache;
    }
    mutable Hash root_cache{};
    mutable bool have_root = false;

    // :84-217 — the reference plans the indices of all layers on the host first (its phase 1) and then
    // reads layer by layer; here the reads of all layers join one GatherPlan.
    // `hashes_per_layer`, when given, receives the number of witness hashes each layer contributed (largest layer first).
    PendingMerkle plan_decommit(GatherPlan& plan, const std::map<uint32_t, std::vector<size_t>>& queries_per_log_size,
                                const std::vector<const BaseColumn*>& columns, std::vector<size_t>* hashes_per_layer = nullptr) const {
        PendingMerkle pm;
        // the layers' column lists as recorded by commit(); sorted again only for a tree that was not built there
        const bool recorded = layer_col_ptrs.size() == layers.size() && n_columns == columns.size();
        std::vector<const BaseColumn*> sorted;
        if (!recorded) {
            sorted = columns;
            std::stable_sort(sorted.begin(), sorted.end(), [](const BaseColumn* a, const BaseColumn* b) { return a->len() > b->len(); });
        }
        size_t pos = 0;
        std::vector<size_t> last;
        for (uint32_t log = (uint32_t)layers.size(); log-- > 0;) {
            bool has_prev = (size_t)log + 1 < layers.size();
            // Sorted vectors, not sets: `last` (the nodes of the layer below) is ascending, so are its halves and the layer's
            // own queries; a FRI proof plans some twenty trees of some twenty layers each.
            const std::vector<size_t>& prev_nodes = last;
            std::vector<size_t> parents, col_queries, merged_nodes;
            parents.reserve(last.size());
            for (auto q : last)
                if (parents.empty() || parents.back() != q / 2) parents.push_back(q / 2);
            auto it = queries_per_log_size.find(log);
            if (it != queries_per_log_size.end()) {
                col_queries = it->second;
                if (!std::is_sorted(col_queries.begin(), col_queries.end())) std::sort(col_queries.begin(), col_queries.end());
                col_queries.erase(std::unique(col_queries.begin(), col_queries.end()), col_queries.end());
            }
            merged_nodes.reserve(parents.size() + col_queries.size());
            std::set_union(parents.begin(), parents.end(), col_queries.begin(), col_queries.end(), std::back_inserter(merged_nodes));
            auto in_prev = [&](size_t node) { return std::binary_search(prev_nodes.begin(), prev_nodes.end(), node); };
            auto is_query = [&](size_t node) { return std::binary_search(col_queries.begin(), col_queries.end(), node); };
            std::vector<const uint32_t*> layer_ptrs_own;
            if (!recorded)
                while (pos < sorted.size() && sorted[pos]->log_size() == log) layer_ptrs_own.push_back(sorted[pos++]->ptr());
            const std::vector<const uint32_t*>& ptrs = recorded ? layer_col_ptrs[log] : layer_ptrs_own;
            std::vector<size_t> witness_children, queried_nodes, witness_nodes;
            for (size_t node : merged_nodes) {
                if (has_prev) {
                    if (!in_prev(2 * node)) witness_children.push_back(2 * node);
                    if (!in_prev(2 * node + 1)) witness_children.push_back(2 * node + 1);
                }
                (is_query(node) ? queried_nodes : witness_nodes).push_back(node);
            }
            for (size_t child : witness_children) pm.hash_slots.push_back(plan.add_hash(layers[log + 1].ptr() + 8 * child));
            if (hashes_per_layer) hashes_per_layer->push_back(witness_children.size());
            if (!ptrs.empty() && !merged_nodes.empty()) {
                // every node of the layer is read once; the proof lists the queried nodes' values first, then the witnesses'
                std::vector<size_t> order(queried_nodes);
                order.insert(order.end(), witness_nodes.begin(), witness_nodes.end());
                size_t off = plan.add_block(ptrs, order);
                if (!queried_nodes.empty()) pm.runs.push_back({off, queried_nodes.size() * ptrs.size(), true});
                if (!witness_nodes.empty()) pm.runs.push_back({off + queried_nodes.size() * ptrs.size(), witness_nodes.size() * ptrs.size(), false});
            }
            last = merged_nodes;
        }
        return pm;
    }
};

// ------------------------------------------------------------------ FRI (STWO/prover/fri.rs:87-467)
struct FriConfig {
    uint32_t log_blowup_factor, log_last_layer_degree_bound, n_queries, line_fold_step;
    size_t last_layer_domain_size() const { return (size_t)1 << (log_last_layer_degree_bound + log_blowup_factor); }
};
struct FriLayerProof { std::vector<qm31> fri_witness; MerkleDecommitment decommitment; Hash commitment; };
struct FriProof { FriLayerProof first_layer; std::vector<FriLayerProof> inner_layers; std::vector<qm31> last_layer_poly; };

static cpoint host_circle_point(uint32_t index) {
    cpoint g{2u, 1268011823u}, r{1u, 0u};
    for (int b = 0; b < 31; b++) {
        if ((index >> b) & 1u) r = cpoint_add(r, g);
        g = cpoint_add(g, g);
    }
    return r;
}
template <class T> static void bit_reverse_vec(std::vector<T>& v) {
    uint32_t log = ilog2(v.size());
    for (size_t i = 0; i < v.size(); i++) {
        size_t j = 0;
        for (uint32_t b = 0; b < log; b++) j |= ((i >> b) & 1) << (log - 1 - b);
        if (j > i) std::swap(v[i], v[j]);
    }
}
// LineEvaluation::interpolate on the host (STWO/prover/line.rs:41-66) for the last FRI layer, whose
// domain is Coset::half_odds(log): initial index 2^(29-log), step 2^(31-log).
static std::vector<qm31> line_interpolate(std::vector<qm31> values) {
    uint32_t log = ilog2(values.size());
    bit_reverse_vec(values);
    for (uint32_t k = log; k > 0; k--) {  // domain of the current chunk size 2^k: half_odds(k)
        size_t size = (size_t)1 << k, half = size / 2;
        for (size_t off = 0; off < values.size(); off += size)
            for (size_t i = 0; i < half; i++) {
                uint32_t idx = ((1u << (29 - k)) + ((uint32_t)i << (31 - k))) & 0x7fffffffu;
                uint32_t xinv = m31_inv(host_circle_point(idx).x);
                qm31 a = values[off + i], b = values[off + half + i];
                values[off + i] = a + b;
                values[off + half + i] = qm31_mul_m31(a - b, xinv);
            }
    }
    uint32_t len_inv = m31_inv((uint32_t)values.size());
    for (auto& v : values) v = qm31_mul_m31(v, len_inv);
    return values;
}

static std::vector<qm31> secure_at_batch(const Device& d, const SecureColumnByCoords& col, const std::vector<size_t>& positions) {
    auto flat = B200Backend::batch_at_multi(d, col.refs(), positions);  // secure_column.rs:33-44
    std::vector<qm31> out(positions.size());
    for (size_t j = 0; j < positions.size(); j++) out[j] = {{flat[4 * j], flat[4 * j + 1], flat[4 * j + 2], flat[4 * j + 3]}};
    return out;
}

struct PendingFriLayer {
    std::vector<size_t> eval_slots;  // 4 per decommitment position
    std::vector<bool> is_witness;
    PendingMerkle merkle;
    Hash commitment;
};

// fri.rs:392-436 — positions first, then one gather for all of them (here: joined to the plan).
static PendingFriLayer plan_fri_layer(GatherPlan& plan, const Device& d, const SecureColumnByCoords& column, const MerkleProver& tree,
                                      const std::vector<size_t>& queries, uint32_t fold_step) {
    PendingFriLayer pl;
    std::vector<size_t> positions;
    size_t i = 0;
    while (i < queries.size()) {
        size_t j = i;
        while (j < queries.size() && (queries[j] >> fold_step) == (queries[i] >> fold_step)) j++;
        size_t start = (queries[i] >> fold_step) << fold_step, qi = i;
        for (size_t p = start; p < start + ((size_t)1 << fold_step); p++) {
            positions.push_back(p);
            if (qi < j && queries[qi] == p) { qi++; pl.is_witness.push_back(false); }
            else pl.is_witness.push_back(true);
        }
        i = j;
    }
    for (size_t p : positions)
        for (int k = 0; k < 4; k++) pl.eval_slots.push_back(plan.add(column.columns[k].ptr() + p));
    std::map<uint32_t, std::vector<size_t>> q{{column.columns[0].log_size(), positions}};
    pl.merkle = tree.plan_decommit(plan, q, column.refs());
    pl.commitment = tree.root(d);
    return pl;
}

struct FriProver {
    FriConfig config;
    const SecureColumnByCoords* first_column = nullptr;
    MerkleProver first_tree;
    struct Inner { SecureColumnByCoords eval; MerkleProver tree; uint32_t fold_step; };
    std::vector<Inner> inner;
    std::vector<qm31> last_layer_poly;

    // fri.rs:109-221
    static FriProver commit(const Device& d, Channel& ch, FriConfig config, const SecureColumnByCoords& column) {
        FriProver fp;
        fp.config = config;
        fp.first_column = &column;
        uint32_t first_log = column.columns[0].log_size(), inner_log = first_log - 1;
        uint32_t last_log = ilog2(config.last_layer_domain_size());
        SecureColumnByCoords layer(d, (size_t)1 << inner_log, true);
        if (config.line_fold_step == 1) {
            // Device-resident commit phase: every layer's tree, the channel step (mix the root, draw the
            // folding challenge) and the fold are enqueued back to back; the host reads all roots and the
            // channel state once, after the last fold.
            size_t n_layers = 1 + (inner_log > last_log ? inner_log - last_log : 0);
            BaseColumn fs(d, 16 + 12 * n_layers);  // [channel 16 | challenges 4 each (16-byte aligned) | roots 8 each]
            uint32_t* chan = fs.ptr();
            uint32_t* alphas = fs.ptr() + 16;
            uint32_t* roots = fs.ptr() + 16 + 4 * n_layers;
            uint32_t st[16] = {0};
            for (int k = 0; k < 8; k++) st[k] = ch.digest()[k];
            st[8] = ch.n_draws();
            d.check(zkb_h2d(d.ctx(), chan, st, sizeof(st)));
            bool stepped = false;
            MerkleProver::ChanStep step0{chan, alphas, roots};
            fp.first_tree = MerkleProver::commit(d, column.refs(), nullptr, &step0, &stepped);
            if (!stepped) d.check(zkb_channel_mix_root_draw(d.ctx(), chan, fp.first_tree.layers[0].ptr(), alphas, roots));
            // every fold but the last also hashes the leaves of the layer it produces: that layer is committed next
            HashColumn leaves;
            bool have_leaves = n_layers > 1 && first_log >= 3;
            B200Backend::fold_circle_into_line(d, layer, column, alphas, have_leaves ? &leaves : nullptr);
            for (size_t k = 1; k < n_layers; k++) {
                Inner in{std::move(layer), {}, 1};
                std::vector<const BaseColumn*> refs = in.eval.refs();
                MerkleProver::ChanStep step{chan, alphas + 4 * k, roots + 8 * k};
                in.tree = MerkleProver::commit(d, refs, have_leaves ? &leaves : nullptr, &step, &stepped);
                if (!stepped) d.check(zkb_channel_mix_root_draw(d.ctx(), chan, in.tree.layers[0].ptr(), alphas + 4 * k, roots + 8 * k));
                have_leaves = k + 1 < n_layers;
                if (have_leaves) layer = B200Backend::fold_line(d, in.eval, alphas + 4 * k, leaves);
                else layer = B200Backend::fold_line(d, in.eval, alphas + 4 * k);
                fp.inner.push_back(std::move(in));
            }
            std::vector<uint32_t> h = fs.to_cpu();  // one copy, one synchronisation
            HashWords dg;
            for (int k = 0; k < 8; k++) dg[k] = h[k];
            ch.set_state(dg, h[8]);
            auto root_at = [&](size_t k) { Hash r; for (int w = 0; w < 8; w++) r[w] = h[16 + 4 * n_layers + 8 * k + w]; return r; };
            fp.first_tree.root_cache = root_at(0);
            fp.first_tree.have_root = true;
            for (size_t k = 1; k < n_layers; k++) { fp.inner[k - 1].tree.root_cache = root_at(k); fp.inner[k - 1].tree.have_root = true; }
        } else {
            fp.first_tree = MerkleProver::commit(d, column.refs());
            ch.mix_root(fp.first_tree.root(d));
            qm31 alpha = ch.draw_secure_felt();
            B200Backend::fold_circle_into_line(d, layer, column, alpha);
            if (inner_log != last_log) {
                for (;;) {
                    uint32_t cur_log = layer.columns[0].log_size();
                    bool last_fold = !(cur_log > last_log + config.line_fold_step);
                    uint32_t step = last_fold ? cur_log - last_log : config.line_fold_step;
                    Inner in{std::move(layer), {}, step};
                    in.tree = MerkleProver::commit(d, in.eval.refs());
                    ch.mix_root(in.tree.root(d));
                    qm31 a = ch.draw_secure_felt();
                    layer = B200Backend::fold_line(d, in.eval, a);
                    for (uint32_t s2 = 1; s2 < step; s2++) {  // backend/cpu/fri.rs:15-30
                        a = a * a;
                        layer = B200Backend::fold_line(d, layer, a);
                    }
                    fp.inner.push_back(std::move(in));
                    if (last_fold) break;
                }
            }
        }
        // commit_last_layer, fri.rs:193-221
        if (layer.len() != config.last_layer_domain_size()) throw Error(ZKB_EINVAL, "FRI: unexpected last layer size");
        std::vector<size_t> all(layer.len());
        std::iota(all.begin(), all.end(), 0);
        std::vector<qm31> coeffs = line_interpolate(secure_at_batch(d, layer, all));
        bit_reverse_vec(coeffs);
        size_t bound = (size_t)1 << config.log_last_layer_degree_bound;
        for (size_t i = bound; i < coeffs.size(); i++)
            if (!qm31_is_zero(coeffs[i])) throw Error(ZKB_EINVAL, "FRI: invalid degree");
        coeffs.resize(bound);
        bit_reverse_vec(coeffs);
        fp.last_layer_poly = coeffs;
        ch.mix_felts(fp.last_layer_poly);
        return fp;
    }

    // fri.rs:223-281, planned: `finish` is called after the plan has been executed.
    std::vector<PendingFriLayer> plan_decommit(GatherPlan& plan, const Device& d, Channel& ch, std::vector<size_t>& query_positions) const {
        uint32_t first_log = first_column->columns[0].log_size();
        query_positions = sorted_dedup(draw_queries(ch, first_log, config.n_queries));
        std::vector<PendingFriLayer> pending;
        pending.push_back(plan_fri_layer(plan, d, *first_column, first_tree, query_positions, 1));
        std::vector<size_t> q = fold_queries(query_positions, 1);
        for (auto& in : inner) {
            pending.push_back(plan_fri_layer(plan, d, in.eval, in.tree, q, in.fold_step));
            q = fold_queries(q, in.fold_step);
        }
        return pending;
    }
    FriProof finish_decommit(const GatherPlan& plan, const std::vector<PendingFriLayer>& pending) const {
        FriProof proof;
        auto layer = [&](const PendingFriLayer& pl) {
            FriLayerProof lp;
            for (size_t k = 0; k < pl.is_witness.size(); k++)
                if (pl.is_witness[k])
                    lp.fri_witness.push_back({{plan.words[pl.eval_slots[4 * k]], plan.words[pl.eval_slots[4 * k + 1]],
                                               plan.words[pl.eval_slots[4 * k + 2]], plan.words[pl.eval_slots[4 * k + 3]]}});
            lp.decommitment = pl.merkle.finish(plan).second;
            lp.commitment = pl.commitment;
            return lp;
        };
        proof.first_layer = layer(pending[0]);
        for (size_t k = 1; k < pending.size(); k++) proof.inner_layers.push_back(layer(pending[k]));
        proof.last_layer_poly = last_layer_poly;
        return proof;
    }
};

}  // namespace b200

namespace b200 {

// ------------------------------------------------------------------ commitment scheme (STWO/prover/pcs/mod.rs)
struct PcsConfig {
    uint32_t pow_bits;
    FriConfig fri;
    void mix_into(Channel& ch) const {  // STWO/core/pcs/mod.rs:47-69 (lifting_log_size None -> 0)
        qm31 f[2] = {{{pow_bits, fri.log_blowup_factor, fri.n_queries, fri.log_last_layer_degree_bound}}, {{fri.line_fold_step, 0, 0, 0}}};
        ch.mix_felts(f, 2);
    }
};

struct CommitmentTreeProver {  // pcs/mod.rs:466-630
    std::vector<BaseColumn> coeffs;  // views of the caller's columns after interpolation
    BaseColumn coeff_slab;           // host path: the one allocation the coefficient columns are views of
    std::vector<BaseColumn> evals;
    std::vector<BaseColumn> eval_slabs;  // device path: one allocation per column size, which the evals are views of
    MerkleProver commitment;
    uint32_t max_log() const { return (uint32_t)commitment.layers.size() - 1; }
};

static CirclePointQ point_add(CirclePointQ p, CirclePointQ q) {  // STWO/core/circle.rs:103-113
    return {p.x * q.x - p.y * q.y, p.x * q.y + p.y * q.x};
}
static CirclePointQ point_repeated_double(CirclePointQ p, uint32_t n) {
    for (uint32_t i = 0; i < n; i++) p = point_add(p, p);
    return p;
}
static CirclePointQ get_random_point(Channel& ch) {  // circle.rs:147-163
    qm31 t = ch.draw_secure_felt();
    qm31 t2 = t * t;
    qm31 inv = qm31_inv(t2 + qm31_one());
    return {(qm31_one() - t2) * inv, qm31_dbl(t) * inv};
}
static bool point_less(const CirclePointQ& a, const CirclePointQ& b) {
    for (int k = 0; k < 4; k++) if (a.x.c[k] != b.x.c[k]) return a.x.c[k] < b.x.c[k];
    for (int k = 0; k < 4; k++) if (a.y.c[k] != b.y.c[k]) return a.y.c[k] < b.y.c[k];
    return false;
}

struct PcsProof {
    std::vector<Hash> commitments;
    std::vector<std::vector<std::vector<qm31>>> sampled_values;
    std::vector<MerkleDecommitment> decommitments;
    std::vector<Words> queried_values;
    uint64_t proof_of_work = 0;
    FriProof fri;
    // A sink with the two vector operations the writers use, over a caller's buffer: words past the capacity are counted, not
    // written (the caller compares size() with the capacity afterwards).
    struct RawSink {
        uint32_t* out;
        size_t cap, n = 0;
        int end() const { return 0; }
        void reserve(size_t) {}
        void push_back(uint32_t v) { if (n < cap) out[n] = v; n++; }
        template <class It> void insert(int, It b, It e) {
            size_t k = (size_t)(e - b);
            if (n + k <= cap && k) copy_words(out + n, &*b, k);
            n += k;
        }
        // A run of many megabytes (the queried values of a wide tree) is copied by four threads: one core moves about
        // 10 GB/s, and the proof of a composed segment is 50 MB.
        static void copy_words(uint32_t* dst, const uint32_t* src, size_t k) {
            if (k < ((size_t)2 << 20)) { memcpy(dst, src, k * 4); return; }
            const size_t part = (k + 3) / 4;
            std::thread th[3];
            for (int t = 0; t < 3; t++) {
                size_t lo = (size_t)(t + 1) * part, hi = std::min(k, lo + part);
                th[t] = std::thread([=] { if (lo < hi) memcpy(dst + lo, src + lo, (hi - lo) * 4); });
            }
            memcpy(dst, src, std::min(k, part) * 4);
            for (auto& t : th) t.join();
        }
        size_t size() const { return n; }
    };
    template <class O> static void put_q(O& o, qm31 q) { o.insert(o.end(), q.c, q.c + 4); }
    template <class O> static void put_hash(O& o, const Hash& h) { o.insert(o.end(), h.begin(), h.end()); }
    template <class O> static void put_dec(O& o, const MerkleDecommitment& d) {
        o.push_back((uint32_t)d.hash_witness.size());
        for (auto& h : d.hash_witness) put_hash(o, h);
        o.push_back((uint32_t)d.column_witness.size());
        d.column_witness.append_to(o);
    }
    template <class O> static void put_layer(O& o, const FriLayerProof& l) {
        o.push_back((uint32_t)l.fri_witness.size());
        for (auto q : l.fri_witness) put_q(o, q);
        put_dec(o, l.decommitment);
        put_hash(o, l.commitment);
    }
    std::vector<uint32_t> to_words() const {
        std::vector<uint32_t> o;
        write(o);
        return o;
    }
    template <class O> void write(O& o) const {
        size_t expect = 1 << 16;
        for (auto& t : sampled_values) expect += 6 * t.size();
        for (auto& d : decommitments) expect += 8 * d.hash_witness.size() + d.column_witness.size();
        for (auto& t : queried_values) expect += t.size();
        o.reserve(expect);
        o.push_back((uint32_t)commitments.size());
        for (auto& h : commitments) put_hash(o, h);
        for (auto& t : sampled_values) {
            o.push_back((uint32_t)t.size());
            for (auto& c : t) { o.push_back((uint32_t)c.size()); for (auto q : c) put_q(o, q); }
        }
        for (auto& d : decommitments) put_dec(o, d);
        for (auto& t : queried_values) { o.push_back((uint32_t)t.size()); t.append_to(o); }
        o.push_back((uint32_t)proof_of_work);
        o.push_back((uint32_t)(proof_of_work >> 32));
        put_layer(o, fri.first_layer);
        o.push_back((uint32_t)fri.inner_layers.size());
        for (auto& l : fri.inner_layers) put_layer(o, l);
        o.push_back((uint32_t)fri.last_layer_poly.size());
        for (auto q : fri.last_layer_poly) put_q(o, q);
    }
};

struct CommitmentSchemeProver {
    const Device& d;
    PcsConfig config;
    std::vector<CommitmentTreeProver> trees;
    float* phase_ms;
    int ev = 32;  // event slots 32.. mark phase boundaries
    std::vector<std::pair<int, int>> marks;  // (phase, slot after it)

    CommitmentSchemeProver(const Device& dev, PcsConfig cfg, float* phases) : d(dev), config(cfg), phase_ms(phases) {
        if (phase_ms) { for (int i = 0; i < ZKB_PCS_N_PHASES; i++) phase_ms[i] = 0.f; mark(-1); }
    }
    void mark(int phase) {
        if (!phase_ms || ev >= 63) return;
        d.check(zkb_event_record(d.ctx(), ev));
        marks.push_back({phase, ev++});
    }
    void finish_timing() {
        if (!phase_ms) return;
        for (size_t i = 1; i < marks.size(); i++) {
            float ms = 0.f;
            d.check(zkb_event_elapsed_ms(d.ctx(), marks[i - 1].second, marks[i].second, &ms));
            if (marks[i].first >= 0) phase_ms[marks[i].first] += ms;
        }
    }

    // TreeBuilder::extend_evals + commit (pcs/mod.rs:429-464) -> CommitmentTreeProver::new (:481-537).
    // `columns` are consumed: interpolated in place, per size group.
    // `fence_of` (optional, one entry per column) names the copy fence after which a column's values have
    // arrived from the host; columns are then interpolated and extended fence by fence, while later
    // columns are still in flight.
    void commit_evals(std::vector<BaseColumn> columns, Channel& ch, const std::vector<int>* fence_of = nullptr,
                      BaseColumn* slab = nullptr, bool are_coeffs = false) {
        CommitmentTreeProver t;
        if (slab) t.coeff_slab = std::move(*slab);
        std::map<uint32_t, std::vector<size_t>> by_log;
        for (size_t i = 0; i < columns.size(); i++) by_log[columns[i].log_size()].push_back(i);
        t.evals.resize(columns.size());
        HashColumn leaves;
        bool have_leaves = false;
        if (fence_of && !columns.empty()) {
            mark(0);
            // One column size: the leaf layer is hashed run by run (whole Blake2s blocks of 16 columns) as the
            // extended columns appear, instead of after the last one.
            const bool incremental = by_log.size() == 1 && columns.size() > 16;
            const uint32_t leaf_log = columns[0].log_size() + config.fri.log_blowup_factor;
            size_t hashed = 0, extended = 0;
            if (incremental) leaves = HashColumn(d, (size_t)8 << leaf_log);
            auto hash_ready = [&](bool final) {
                size_t avail = extended - hashed;
                size_t take = final ? avail : (avail > 16 ? (avail - 1) / 16 * 16 : 0);  // keep at least one column for the final call
                if (!take) return;
                std::vector<const uint32_t*> p;
                for (size_t c = hashed; c < hashed + take; c++) p.push_back(t.evals[c].ptr());
                d.check(zkb_merkle_leaves_partial(d.ctx(), (int)leaf_log, p.data(), (int)take, (int)hashed, (int)columns.size(), 1, leaves.ptr()));
                hashed += take;
            };
            std::map<int, std::map<uint32_t, std::vector<size_t>>> by_fence;  // fences in the order they complete
            for (size_t i = 0; i < columns.size(); i++) by_fence[(*fence_of)[i]][columns[i].log_size()].push_back(i);
            for (auto& f : by_fence) {
                d.check(zkb_wait_fence(d.ctx(), f.first));
                for (auto& g : f.second) {
                    std::vector<BaseColumn*> cols;
                    std::vector<const BaseColumn*> ccols;
                    for (auto i : g.second) { cols.push_back(&columns[i]); ccols.push_back(&columns[i]); }
                    B200Backend::interpolate_columns(d, cols);
                    auto ev_cols = B200Backend::evaluate_polynomials(d, ccols, config.fri.log_blowup_factor);
                    for (size_t k = 0; k < g.second.size(); k++) t.evals[g.second[k]] = std::move(ev_cols[k]);
                    if (incremental) { extended = g.second.back() + 1; hash_ready(false); }
                }
            }
            if (incremental) { hash_ready(true); have_leaves = true; }
        } else {
            for (auto& g : by_log) {
                if (are_coeffs) break;  // TreeBuilder::extend_polys (pcs/mod.rs:437-452): the columns are coefficients already
                std::vector<BaseColumn*> cols;
                for (auto i : g.second) cols.push_back(&columns[i]);
                B200Backend::interpolate_columns(d, cols);
            }
            mark(0);
            for (auto& g : by_log) {
                std::vector<const BaseColumn*> cols;
                for (auto i : g.second) cols.push_back(&columns[i]);
                t.eval_slabs.emplace_back();
                auto ev_cols = B200Backend::evaluate_polynomials(d, cols, config.fri.log_blowup_factor, &t.eval_slabs.back());
                for (size_t k = 0; k < g.second.size(); k++) t.evals[g.second[k]] = std::move(ev_cols[k]);
            }
        }
        mark(1);
        t.coeffs = std::move(columns);
        std::vector<const BaseColumn*> refs;
        for (auto& e : t.evals) refs.push_back(&e);
        t.commitment = MerkleProver::commit(d, refs, have_leaves ? &leaves : nullptr);
        ch.mix_root(t.commitment.root(d));
        mark(2);
        trees.push_back(std::move(t));
    }

    // pcs/quotient_ops.rs:73-194 with STWO/core/pcs/quotients.rs:306-345 and :75-104
    SecureColumnByCoords compute_fri_quotients(const std::vector<std::vector<std::vector<PointSample>>>& samples, qm31 random_coeff,
                                               uint32_t lifting_log) {
        std::unique_ptr<HostClock> hc(new HostClock("pcs.quot.flatten"));
        std::vector<const BaseColumn*> flat_cols;
        std::vector<uint32_t> flat_logs;
        size_t n_flat = 0;
        for (auto& t : trees) n_flat += t.evals.size();
        flat_cols.reserve(n_flat); flat_logs.reserve(n_flat);
        // step of CanonicCoset(lifting_log): the point of index 2^(31 - lifting_log)
        cpoint gen = host_circle_point(1u << (31 - lifting_log));
        // Sample j of the flattened list takes random_coeff^j (quotients.rs:306-345 multiplies as it goes): the powers are
        // filled in chunks on several threads, each starting from its own power.
        std::vector<size_t> first_pow;
        first_pow.reserve(n_flat + 1);
        size_t n_pows = 0;
        for (size_t t = 0; t < trees.size(); t++)
            for (size_t c = 0; c < trees[t].evals.size(); c++) {
                first_pow.push_back(n_pows);
                const size_t ns = samples[t][c].size();
                n_pows += ns + (ns == 2 ? 1 : 0);
            }
        first_pow.push_back(n_pows);
        // column i's samples with their powers: flat_samples[first_pow[i] .. first_pow[i + 1]) (one array: a vector per column
        // is an allocation per column)
        std::vector<std::pair<PointSample, qm31>> flat_samples(n_pows);
        parallel_chunks(n_pows, 8192, [&](size_t lo, size_t hi, size_t) {
            qm31 p = qm31_one(), sq = random_coeff;
            for (size_t e = lo; e; e >>= 1) { if (e & 1) p = p * sq; sq = sq * sq; }
            for (size_t i = lo; i < hi; i++) { flat_samples[i].second = p; p = p * random_coeff; }
        });
        // the periodicity sample's point depends on the column's height and the sampled point only: a handful of distinct ones
        struct Shifted { uint32_t log_size; CirclePointQ from, to; };
        std::vector<Shifted> shifted;
        for (size_t t = 0; t < trees.size(); t++)
            for (size_t c = 0; c < trees[t].evals.size(); c++) {
                uint32_t log_size = trees[t].evals[c].log_size();
                flat_cols.push_back(&trees[t].evals[c]);
                flat_logs.push_back(log_size);
                const auto& sc = samples[t][c];
                std::pair<PointSample, qm31>* v = flat_samples.data() + first_pow[flat_cols.size() - 1];
                if (!sc.empty()) {
                    if (sc.size() == 2) {
                        const Shifted* hit = nullptr;
                        for (auto& sh : shifted) if (sh.log_size == log_size && sh.from == sc[1].point) { hit = &sh; break; }
                        if (!hit) {
                            cpoint per = gen;
                            for (uint32_t k = 0; k < log_size; k++) per = cpoint_add(per, per);
                            CirclePointQ pq{qm31_from_m31(per.x), qm31_from_m31(per.y)};
                            shifted.push_back({log_size, sc[1].point, point_add(sc[1].point, pq)});
                            hit = &shifted.back();
                        }
                        (v++)->first = PointSample{hit->to, sc[1].value};
                    }
                    for (auto& smp : sc) (v++)->first = smp;
                }
            }
        hc.reset(new HostClock("pcs.quot.groups"));
        // the columns by ascending size, in their own order within a size: a counting sort (sizes are below 2^32)
        std::vector<size_t> order(flat_cols.size());
        {
            size_t first_of[34] = {0};
            for (uint32_t lg : flat_logs) first_of[std::min<uint32_t>(lg, 32) + 1]++;
            for (int k = 1; k < 34; k++) first_of[k] += first_of[k - 1];
            for (size_t i = 0; i < flat_logs.size(); i++) order[first_of[std::min<uint32_t>(flat_logs[i], 32)]++] = i;
        }
        std::vector<AccumulatedNumerators> accs;
        for (size_t i = 0; i < order.size();) {
            size_t j = i;
            while (j < order.size() && flat_logs[order[j]] == flat_logs[order[i]]) j++;
            std::vector<const BaseColumn*> group_cols;
            std::vector<ColumnSampleBatch> batches;
            for (size_t k = i; k < j; k++) {
                group_cols.push_back(flat_cols[order[k]]);
                for (size_t q = first_pow[order[k]]; q < first_pow[order[k] + 1]; q++) {
                    const std::pair<PointSample, qm31>& sp = flat_samples[q];
                    ColumnSampleBatch* b = nullptr;
                    for (auto& x : batches) if (x.point == sp.first.point) { b = &x; break; }
                    if (!b) { batches.push_back({sp.first.point, {}}); b = &batches.back(); }
                    b->cols_vals_randpows.push_back({k - i, sp.first.value, sp.second});
                }
            }
            {
                HostClock hn("pcs.quot.numerators");
                B200Backend::accumulate_numerators(d, group_cols, batches, accs);
            }
            i = j;
        }
        hc.reset(new HostClock("pcs.quot.combine"));
        std::stable_sort(accs.begin(), accs.end(),
                         [](const AccumulatedNumerators& a, const AccumulatedNumerators& b) { return point_less(a.sample_point, b.sample_point); });
        std::vector<AccumulatedNumerators> per_point;
        for (size_t i = 0; i < accs.size();) {
            size_t j = i;
            while (j < accs.size() && accs[j].sample_point == accs[i].sample_point) j++;
            qm31 first = qm31_zero();
            std::vector<SecureColumnByCoords> cols;
            for (size_t k = i; k < j; k++) {
                first = first + accs[k].first_linear_term_acc;
                cols.push_back(std::move(accs[k].partial_numerators_acc));
            }
            CirclePointQ pt = accs[i].sample_point;
            per_point.push_back({pt, B200Backend::lift_and_accumulate(d, std::move(cols)), first});
            i = j;
        }
        return B200Backend::compute_quotients_and_combine(d, per_point, lifting_log);
    }

    // pcs/mod.rs:168-419
    PcsProof prove_values(const std::vector<std::vector<std::vector<CirclePointQ>>>& sampled_points, Channel& ch) {
        PcsProof proof;
        uint32_t lifting_log = trees.back().max_log();
        // Every column is lifted to the height of the LAST tree (pcs/mod.rs:180: in a proof it is the composition tree, which
        // is the tallest); a taller column in an earlier tree has no lift.
        for (auto& t : trees)
            if (!t.evals.empty() && t.max_log() > lifting_log)
                throw Error(ZKB_EINVAL, "pcs: the last tree must hold the tallest column (every column is lifted to its height)");
        // batch out-of-domain evaluation: one call per (coefficient size, transformed point) group (:187-265)
        std::unique_ptr<HostClock> hc(new HostClock("pcs.sample.group"));
        std::vector<std::vector<std::vector<PointSample>>> samples(trees.size());
        struct Group { uint32_t log; CirclePointQ pt; std::vector<std::array<size_t, 3>> where; std::vector<const BaseColumn*> cols; };
        std::vector<Group> groups;
        struct Doubled { CirclePointQ p; uint32_t shift; CirclePointQ tp; };
        std::vector<Doubled> doubled;
        for (size_t t = 0; t < trees.size(); t++) {
            samples[t].resize(trees[t].coeffs.size());
            for (size_t c = 0; c < trees[t].coeffs.size(); c++) {
                uint32_t poly_log = trees[t].evals[c].log_size(), coeff_log = trees[t].coeffs[c].log_size();
                samples[t][c].reserve(sampled_points[t][c].size());
                for (size_t k = 0; k < sampled_points[t][c].size(); k++) {
                    CirclePointQ p = sampled_points[t][c][k];
                    samples[t][c].push_back({p, qm31_zero()});
                    // most columns share the point and the shift: double once per distinct (point, shift)
                    CirclePointQ tp;
                    bool seen = false;
                    for (auto& m : doubled) if (m.shift == lifting_log - poly_log && m.p == p) { tp = m.tp; seen = true; break; }
                    if (!seen) { tp = point_repeated_double(p, lifting_log - poly_log); doubled.push_back({p, lifting_log - poly_log, tp}); }
                    Group* g = nullptr;
                    for (auto& x : groups) if (x.log == coeff_log && x.pt == tp) { g = &x; break; }
                    if (!g) { groups.push_back({coeff_log, tp, {}, {}}); g = &groups.back(); }
                    g->where.push_back({t, c, k});
                    g->cols.push_back(&trees[t].coeffs[c]);
                }
            }
        }
        hc.reset(new HostClock("pcs.sample.eval"));
        for (auto& g : groups) {
            auto vals = B200Backend::batch_eval_at_point(d, g.cols, g.pt);
            for (size_t i = 0; i < vals.size(); i++) samples[g.where[i][0]][g.where[i][1]][g.where[i][2]].value = vals[i];
        }
        hc.reset(new HostClock("pcs.sample.flatten"));
        std::vector<qm31> flat_values;
        size_t n_values = 0;
        for (auto& t : samples) for (auto& col : t) n_values += col.size();
        flat_values.reserve(n_values);
        for (size_t t = 0; t < trees.size(); t++) {
            proof.sampled_values.emplace_back();
            proof.sampled_values[t].resize(samples[t].size());
            for (size_t c = 0; c < samples[t].size(); c++) {
                std::vector<qm31>& v = proof.sampled_values[t][c];
                v.reserve(samples[t][c].size());
                for (auto& smp : samples[t][c]) { v.push_back(smp.value); flat_values.push_back(smp.value); }
            }
        }
        mark(3);
        hc.reset(new HostClock("pcs.quot.mix"));
        ch.mix_felts(flat_values);
        qm31 random_coeff = ch.draw_secure_felt();
        hc.reset(new HostClock("pcs.quot.compute"));
        SecureColumnByCoords quotients = compute_fri_quotients(samples, random_coeff, lifting_log);
        hc.reset();
        mark(4);
        FriProver fri = FriProver::commit(d, ch, config.fri, quotients);
        mark(5);
        proof.proof_of_work = B200Backend::grind(d, ch.pow_prefixed_digest(config.pow_bits), config.pow_bits);
        ch.mix_u64(proof.proof_of_work);
        mark(6);
        hc.reset(new HostClock("pcs.decommit.plan"));
        std::vector<size_t> query_positions;
        GatherPlan plan;
        std::unique_ptr<HostClock> hc2(new HostClock("pcs.decommit.plan.fri"));
        auto fri_pending = fri.plan_decommit(plan, d, ch, query_positions);
        hc2.reset(new HostClock("pcs.decommit.plan.trees"));
        std::vector<PendingMerkle> tree_pending;
        for (auto& t : trees) {  // STWO/core/pcs/utils.rs:200-218, then pcs/mod.rs:575-630
            uint32_t tree_max = t.max_log();
            std::vector<size_t> q;
            for (auto pos : query_positions) q.push_back(((pos >> (lifting_log - tree_max + 1)) << 1) + (pos & 1));
            std::map<uint32_t, std::vector<size_t>> per_log;
            std::vector<const BaseColumn*> refs;
            refs.reserve(t.evals.size());
            uint64_t seen_logs = 0;  // a tree has tens of thousands of columns and a handful of heights
            for (auto& e : t.evals) {
                refs.push_back(&e);
                uint32_t log = e.log_size();
                if ((seen_logs >> log) & 1) continue;
                seen_logs |= (uint64_t)1 << log;
                std::vector<size_t> positions;
                for (auto pos : q) positions.push_back(((pos >> (tree_max - log + 1)) << 1) + (pos & 1));
                per_log[log] = sorted_dedup(positions);
            }
            tree_pending.push_back(t.commitment.plan_decommit(plan, per_log, refs));
        }
        hc2.reset();
        hc.reset(new HostClock("pcs.decommit.gather"));
        plan.execute(d);
        hc.reset(new HostClock("pcs.decommit.finish"));
        proof.fri = fri.finish_decommit(plan, fri_pending);
        for (size_t k = 0; k < trees.size(); k++) {
            auto r = tree_pending[k].finish(plan);
            proof.queried_values.push_back(std::move(r.first));
            proof.decommitments.push_back(std::move(r.second));
            proof.commitments.push_back(trees[k].commitment.root(d));
        }
        hc.reset();
        mark(7);
        return proof;
    }
};

// ------------------------------------------------------------------ GKR (STWO/prover/lookups)
// Dense univariate polynomial over QM31, low coefficient first (lookups/utils.rs:12-146).
struct UniPoly {
    std::vector<qm31> c;
    void trim() { while (!c.empty() && qm31_is_zero(c.back())) c.pop_back(); }
    qm31 eval(qm31 x) const {
        qm31 acc = qm31_zero();
        for (size_t i = c.size(); i-- > 0;) acc = acc * x + c[i];
        return acc;
    }
    static UniPoly mul(UniPoly a, UniPoly b) {
        a.trim(); b.trim();
        if (a.c.empty() || b.c.empty()) return {};
        UniPoly r;
        r.c.assign(a.c.size() + b.c.size() - 1, qm31_zero());
        for (size_t i = 0; i < a.c.size(); i++)
            for (size_t j = 0; j < b.c.size(); j++) r.c[i + j] = r.c[i + j] + a.c[i] * b.c[j];
        r.trim();
        return r;
    }
    static UniPoly add(const UniPoly& a, const UniPoly& b) {
        UniPoly r;
        for (size_t i = 0; i < std::max(a.c.size(), b.c.size()); i++)
            r.c.push_back((i < a.c.size() ? a.c[i] : qm31_zero()) + (i < b.c.size() ? b.c[i] : qm31_zero()));
        return r;
    }
    static UniPoly interpolate_lagrange(const std::vector<qm31>& xs, const std::vector<qm31>& ys) {  // utils.rs:26-54
        UniPoly coeffs;
        for (size_t i = 0; i < xs.size(); i++) {
            qm31 prod = ys[i];
            for (size_t j = 0; j < xs.size(); j++)
                if (i != j) prod = prod * qm31_inv(xs[i] - xs[j]);
            UniPoly term;
            term.c = {prod};
            term.trim();
            for (size_t j = 0; j < xs.size(); j++)
                if (i != j) { UniPoly lin; lin.c = {qm31_neg(xs[j]), qm31_one()}; term = mul(term, lin); }
            coeffs = add(coeffs, term);
        }
        coeffs.trim();
        return coeffs;
    }
};

static qm31 eq1(qm31 x, qm31 y) { return x * y + (qm31_one() - x) * (qm31_one() - y); }  // utils.rs:165-170
static qm31 horner(const std::vector<qm31>& v, qm31 x) {
    qm31 acc = qm31_zero();
    for (size_t i = v.size(); i-- > 0;) acc = acc * x + v[i];
    return acc;
}

// correct_sum_as_poly_in_first_variable (gkr_prover.rs:884-923), split in two.
// The part that depends only on the out-of-domain point y and on the number of
// variables k: every oracle that is active in a round shares it, so it is worked out once per round (two inversions and
// the Lagrange basis on {0, 1, 2, b}) instead of once per instance (a batch has hundreds). The round polynomial of an
// oracle is then r0 L0 + r1 L1 + r2 L2 (the value at b is zero), the same field elements as the interpolation gives.
struct RoundBasis {
    qm31 e0a, e2a;   // eq(0, y[n-k]) / prod_{i <= n-k} eq(0, y_i) and eq(2, y[n-k]) / the same product
    qm31 L[3][4];    // coefficients (low first) of the basis polynomials of the nodes 0, 1, 2
    RoundBasis(const std::vector<qm31>& y, size_t k) {
        size_t n = y.size();
        qm31 a = qm31_one();
        for (size_t i = 0; i < n - k + 1; i++) a = a * eq1(qm31_zero(), y[i]);
        a = qm31_inv(a);
        qm31 two = qm31_from_m31(2);
        qm31 b = (qm31_one() - y[n - k]) * qm31_inv(qm31_one() - qm31_dbl(y[n - k]));
        e0a = eq1(qm31_zero(), y[n - k]) * a;
        e2a = eq1(two, y[n - k]) * a;
        const qm31 xs[4] = {qm31_zero(), qm31_one(), two, b};
        for (int i = 0; i < 3; i++) {
            qm31 denom = qm31_one();
            qm31 poly[4] = {qm31_one(), qm31_zero(), qm31_zero(), qm31_zero()};
            int deg = 0;
            for (int j = 0; j < 4; j++) {
                if (j == i) continue;
                denom = denom * (xs[i] - xs[j]);
                for (int t = ++deg; t > 0; t--) poly[t] = poly[t - 1] - xs[j] * poly[t];  // times (x - xs[j])
                poly[0] = qm31_neg(xs[j] * poly[0]);
            }
            qm31 inv = qm31_inv(denom);
            for (int t = 0; t < 4; t++) L[i][t] = poly[t] * inv;
        }
    }
    // the polynomial with the values r0, r1, r2 at 0, 1, 2 and zero at b
    UniPoly round_poly(qm31 r0, qm31 r1, qm31 r2) const {
        UniPoly p;
        p.c.resize(4);
        for (int t = 0; t < 4; t++) p.c[t] = r0 * L[0][t] + r1 * L[1][t] + r2 * L[2][t];
        p.trim();
        return p;
    }
};

struct GkrOracle {  // GkrMultivariatePolyOracle, gkr_prover.rs:473-556
    Layer input_layer;
    qm31 eq_fixed_var_correction;
    bool have_sums = false;  // the next round's sums, produced together with the last fix
    std::pair<qm31, qm31> sums;
    bool have_mask = false;  // the two entries of every column after the last fix, read back with that round's results
    qm31 mask_den[2], mask_num[2];
    size_t n_variables() const { return input_layer.n_variables() - 1; }
};

static std::vector<qm31> mle_to_cpu(const Device& d, const SecureMle& m) {
    auto w = m.words.to_cpu();
    std::vector<qm31> out(m.len());
    for (size_t i = 0; i < out.size(); i++) out[i] = {{w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]}};
    return out;
}

static Layer layer_view(const Device& d, int kind, const uint32_t* num, const uint32_t* den, size_t n) {
    Layer l;
    l.kind = kind;
    l.den.words = BaseColumn::view(d, const_cast<uint32_t*>(den), 4 * n);
    if (kind == ZKB_GKR_LOGUP_GENERIC) l.num.words = BaseColumn::view(d, const_cast<uint32_t*>(num), 4 * n);
    if (kind == ZKB_GKR_LOGUP_MULTIPLICITIES) l.num_base = BaseColumn::view(d, const_cast<uint32_t*>(num), n);
    return l;
}

// gkr_prover.rs:657-882 with sumcheck.rs:96-176. Returns the proof word stream.
static std::vector<uint32_t> gkr_prove_batch(const Device& d, Channel& ch, std::vector<Layer> input_layers) {
    size_t n_inst = input_layers.size();
    std::vector<size_t> n_layers_by_inst;
    for (auto& l : input_layers) n_layers_by_inst.push_back(l.n_variables());
    size_t n_layers = *std::max_element(n_layers_by_inst.begin(), n_layers_by_inst.end());
    std::vector<std::vector<Layer>> towers(n_inst);  // gen_layers, :847-852; one launch per level for the whole batch
    for (size_t i = 0; i < n_inst; i++) towers[i].push_back(std::move(input_layers[i]));
    std::vector<zk::GkrBatchItem> items;
    auto item_of = [](const Layer& in, Layer& out, uint32_t mode) {
        zk::GkrBatchItem it{};
        it.num = in.num_ptr();
        it.den = in.den.words.ptr();
        it.num_out = out.kind == ZKB_GKR_LOGUP_GENERIC ? out.num.words.ptr() : nullptr;
        it.den_out = out.den.words.ptr();
        it.n = in.len();
        it.kind = (uint32_t)in.kind;
        it.mode = mode;
        return it;
    };
    std::vector<BaseColumn> slabs;  // one allocation per tower level; the layers of that level are views of it
    std::unique_ptr<HostClock> hc_towers(new HostClock("gkr.towers"));
    for (;;) {
        items.clear();
        size_t words = 0;
        for (size_t i = 0; i < n_inst; i++) {
            const Layer& in = towers[i].back();
            if (in.n_variables() == 0) continue;
            words += (in.kind == ZKB_GKR_GRAND_PRODUCT ? 1 : 2) * 4 * (in.len() / 2);
        }
        if (!words) break;
        slabs.emplace_back(d, words);
        uint32_t* cur = slabs.back().ptr();
        for (size_t i = 0; i < n_inst; i++) {
            const Layer& in = towers[i].back();
            if (in.n_variables() == 0) continue;
            const size_t half_words = 4 * (in.len() / 2);
            Layer out;
            out.writable = true;
            out.kind = in.kind == ZKB_GKR_GRAND_PRODUCT ? ZKB_GKR_GRAND_PRODUCT : ZKB_GKR_LOGUP_GENERIC;
            out.den.words = BaseColumn::view(d, cur, half_words);
            cur += half_words;
            if (out.kind == ZKB_GKR_LOGUP_GENERIC) { out.num.words = BaseColumn::view(d, cur, half_words); cur += half_words; }
            items.push_back(item_of(in, out, 3));
            towers[i].push_back(std::move(out));
        }
        d.check(zk::gkr_batch_next_layer(d.ctx(), items.data(), (int)items.size()));
    }
    hc_towers.reset();
    std::vector<uint32_t> results;
    // the output layers (one entry per column) of all instances, read in one gather
    GatherPlan top_plan;
    std::vector<size_t> top_slot(n_inst, SIZE_MAX);
    for (size_t i = 0; i < n_inst; i++) {
        const Layer& t = towers[i].back();
        if (t.len() != 1 || (t.kind != ZKB_GKR_GRAND_PRODUCT && t.kind != ZKB_GKR_LOGUP_GENERIC)) continue;
        top_slot[i] = top_plan.addrs.size();
        for (int w = 0; w < 4; w++) top_plan.add(t.den.words.ptr() + w);
        if (t.kind == ZKB_GKR_LOGUP_GENERIC)
            for (int w = 0; w < 4; w++) top_plan.add(t.num.words.ptr() + w);
    }
    if (!top_plan.addrs.empty()) top_plan.execute(d);
    auto top_q = [&](size_t slot) { return qm31{{top_plan.words[slot], top_plan.words[slot + 1], top_plan.words[slot + 2], top_plan.words[slot + 3]}}; };
    std::vector<std::vector<UniPoly>> sumcheck_round_polys;
    struct MaskRec { uint32_t n_cols; qm31 v[4]; };  // column c is (v[2c], v[2c+1])
    std::vector<std::vector<MaskRec>> masks_by_inst(n_inst);
    for (size_t i = 0; i < n_inst; i++) masks_by_inst[i].reserve(n_layers_by_inst[i]);
    std::vector<std::vector<qm31>> output_claims(n_inst), claims(n_inst);
    std::vector<bool> active(n_inst, false);
    std::vector<qm31> ood_point;

    auto take = [&](size_t i) { Layer l = std::move(towers[i].back()); towers[i].pop_back(); return l; };
    for (size_t layer = 0; layer < n_layers; layer++) {
        size_t n_remaining = n_layers - layer;
        for (size_t i = 0; i < n_inst; i++)
            if (n_layers_by_inst[i] == n_remaining) {
                Layer out = take(i);  // output layer: one entry per column
                std::vector<qm31> vals;
                const bool planned = top_slot[i] != SIZE_MAX;
                qm31 den0 = planned ? top_q(top_slot[i]) : mle_to_cpu(d, out.den)[0];
                if (out.kind == ZKB_GKR_GRAND_PRODUCT) vals = {den0};
                else if (out.kind == ZKB_GKR_LOGUP_GENERIC) vals = {planned ? top_q(top_slot[i] + 4) : mle_to_cpu(d, out.num)[0], den0};
                else if (out.kind == ZKB_GKR_LOGUP_MULTIPLICITIES) vals = {qm31_from_m31(out.num_base.to_cpu()[0]), den0};
                else vals = {qm31_one(), den0};
                claims[i] = vals;
                output_claims[i] = vals;
                active[i] = true;
            }
        for (size_t i = 0; i < n_inst; i++)
            if (active[i]) ch.mix_felts(claims[i]);
        // EqEvals::generate, :235-247
        std::unique_ptr<HostClock> hc_eq(new HostClock("gkr.layer.eq_evals"));
        SecureMle eq_evals;
        if (ood_point.empty()) eq_evals = B200Backend::gen_eq_evals(d, {}, qm31_one());
        else eq_evals = B200Backend::gen_eq_evals(d, std::vector<qm31>(ood_point.begin() + 1, ood_point.end()), eq1(qm31_zero(), ood_point[0]));
        hc_eq.reset();
        qm31 sumcheck_alpha = ch.draw_secure_felt();
        qm31 lambda = ch.draw_secure_felt();
        std::vector<GkrOracle> oracles;
        std::vector<qm31> sc_claims;
        std::vector<size_t> sc_inst;
        for (size_t i = 0; i < n_inst; i++)
            if (active[i]) {
                oracles.push_back({take(i), qm31_one(), false, {}});
                sc_claims.push_back(horner(claims[i], lambda));
                sc_inst.push_back(i);
            }
        size_t nv = 0;
        for (auto& o : oracles) nv = std::max(nv, o.n_variables());
        for (size_t k = 0; k < oracles.size(); k++) sc_claims[k] = qm31_mul_m31(sc_claims[k], 1u << (nv - oracles[k].n_variables()));
        std::vector<UniPoly> round_polys;
        std::vector<qm31> assignment;
        const uint32_t half = m31_inv(2);
        // By default the whole sum-check of the layer is enqueued at once and the transcript of its rounds stays on the
        // device (gkr_batch_layer); ZKB_GKR_ROUNDS=host keeps the channel on the host and returns to it every round, and
        // ZKB_GKR_ROUNDS=launches keeps a launch per round also for the small rounds (both for comparison and tests).
        const char* rounds_env = getenv("ZKB_GKR_ROUNDS");
        bool host_rounds = rounds_env && !strcmp(rounds_env, "host");
        {
            // The layer's description is staged as one block (an item per oracle and active round, 64 bytes each, and some
            // 52 bytes per oracle): a batch of thousands of tall instances would not fit the staging ring (2 MiB) and takes
            // the round-by-round path, which stages one round's items at a time.
            size_t items = 0;
            for (auto& o : oracles) items += o.n_variables() + 1;
            if (64 * items + 64 * oracles.size() + 256 * nv + 4096 > ((size_t)1 << 20)) host_rounds = true;
        }
        if (nv > 0 && !host_rounds) {
            std::unique_ptr<HostClock> hc(new HostClock("gkr.layer.plan"));
            const size_t K = oracles.size();
            std::vector<uint32_t> n_vars(K);
            std::vector<qm31> alpha_pow(K);
            for (size_t k = 0; k < K; k++) {
                n_vars[k] = (uint32_t)oracles[k].n_variables();
                alpha_pow[k] = k ? alpha_pow[k - 1] * sumcheck_alpha : qm31_one();
            }
            std::vector<std::vector<zk::GkrBatchItem>> first(nv), fix(nv);
            std::vector<zk::GkrLayerRound> plan(nv);
            std::vector<Layer> retired;  // layers replaced by their fixed copies: alive until the enqueued launches have read them
            for (size_t round = 0; round < nv; round++) {
                const size_t n_rem = nv - round;
                const RoundBasis basis(ood_point, n_rem);
                zk::GkrRoundConst& rc = plan[round].rc;
                memset(&rc, 0, sizeof(rc));
                memcpy(rc.e0a, basis.e0a.c, 16);
                memcpy(rc.e2a, basis.e2a.c, 16);
                for (int i = 0; i < 3; i++)
                    for (int t = 0; t < 4; t++) memcpy(rc.L[i][t], basis.L[i][t].c, 16);
                memcpy(rc.y, ood_point[ood_point.size() - n_rem].c, 16);
                rc.n_rem = (uint32_t)n_rem;
                for (size_t k = 0; k < K; k++) {
                    GkrOracle& o = oracles[k];
                    if (n_rem != o.n_variables() || o.n_variables() == 0) continue;
                    Layer& in = o.input_layer;
                    if (n_vars[k] == n_rem) {  // enters in this round: its first sums
                        zk::GkrBatchItem it{};
                        it.num = in.num_ptr();
                        it.den = in.den.words.ptr();
                        it.n = in.len();
                        it.kind = (uint32_t)in.kind;
                        it.mode = 0;
                        it.slot = k;
                        first[round].push_back(it);
                    }
                    Layer out;  // Layer::fix_first_variable, gkr_prover.rs:354-381
                    out.writable = true;
                    out.kind = in.kind == ZKB_GKR_LOGUP_MULTIPLICITIES ? ZKB_GKR_LOGUP_GENERIC : in.kind;
                    const uint32_t mode = in.len() >= 8 ? 1 : 2;
                    if (in.writable && in.kind != ZKB_GKR_LOGUP_MULTIPLICITIES) {
                        // in place: the result is the first half of the layer (see the host-round path below)
                        out.den.words = BaseColumn::view(d, in.den.words.ptr(), in.den.words.len() / 2);
                        if (out.kind == ZKB_GKR_LOGUP_GENERIC) out.num.words = BaseColumn::view(d, in.num.words.ptr(), in.num.words.len() / 2);
                        zk::GkrBatchItem it = item_of(in, out, mode);
                        it.slot = k;
                        fix[round].push_back(it);
                        in.den.words.shrink(in.den.words.len() / 2);
                        if (out.kind == ZKB_GKR_LOGUP_GENERIC) in.num.words.shrink(in.num.words.len() / 2);
                    } else {
                        out.den = SecureMle(d, in.len() / 2);
                        if (out.kind == ZKB_GKR_LOGUP_GENERIC) out.num = SecureMle(d, in.len() / 2);
                        zk::GkrBatchItem it = item_of(in, out, mode);
                        it.slot = k;
                        fix[round].push_back(it);
                        retired.push_back(std::move(in));
                        in = std::move(out);
                    }
                }
                plan[round].first = first[round].data();
                plan[round].n_first = (int)first[round].size();
                plan[round].fix = fix[round].data();
                plan[round].n_fix = (int)fix[round].size();
            }
            hc.reset(new HostClock("gkr.layer.rounds"));
            uint32_t chan[9];
            memcpy(chan, ch.digest().data(), 32);
            chan[8] = ch.n_draws();
            std::vector<uint32_t> out_words(zk::GKR_LAYER_OUT_WORDS * nv), res(zk::GKR_BATCH_RESULT_WORDS * K);
            d.check(zk::gkr_batch_layer(d.ctx(), (int)K, n_vars.data(), alpha_pow[0].c, sc_claims[0].c, plan.data(), (int)nv, eq_evals.words.ptr(),
                                        lambda.c, chan, out_words.data(), res.data()));
            retired.clear();
            HashWords digest;
            memcpy(digest.data(), chan, 32);
            ch.set_state(digest, chan[8]);
            for (size_t round = 0; round < nv; round++) {
                const uint32_t* w = out_words.data() + zk::GKR_LAYER_OUT_WORDS * round;
                UniPoly rp;
                for (uint32_t t = 0; t < w[16] && t < 4; t++) rp.c.push_back(qm31{{w[4 * t], w[4 * t + 1], w[4 * t + 2], w[4 * t + 3]}});
                round_polys.push_back(std::move(rp));
                assignment.push_back(qm31{{w[20], w[21], w[22], w[23]}});
            }
            for (size_t k = 0; k < K; k++) {
                if (n_vars[k] == 0) continue;  // no round, no mask from a launch: read with the others below
                GkrOracle& o = oracles[k];
                const uint32_t* w = res.data() + zk::GKR_BATCH_RESULT_WORDS * k;
                for (int e = 0; e < 2; e++) {
                    o.mask_den[e] = qm31{{w[8 + 4 * e], w[9 + 4 * e], w[10 + 4 * e], w[11 + 4 * e]}};
                    o.mask_num[e] = qm31{{w[16 + 4 * e], w[17 + 4 * e], w[18 + 4 * e], w[19 + 4 * e]}};
                }
                o.have_mask = true;
            }
        }
        for (size_t round = 0; host_rounds && round < nv; round++) {
            size_t n_rem = nv - round;
            // the oracles that enter the sum-check in this round have no sums yet: one launch for all of them
            std::unique_ptr<HostClock> hc(new HostClock("gkr.round.first_sums"));
            items.clear();
            std::vector<size_t> who;
            for (size_t k = 0; k < oracles.size(); k++)
                if (n_rem == oracles[k].n_variables() && !oracles[k].have_sums) {
                    zk::GkrBatchItem it{};
                    it.num = oracles[k].input_layer.num_ptr();
                    it.den = oracles[k].input_layer.den.words.ptr();
                    it.n = oracles[k].input_layer.len();
                    it.kind = (uint32_t)oracles[k].input_layer.kind;
                    it.mode = 0;
                    items.push_back(it);
                    who.push_back(k);
                }
            if (!items.empty()) {
                results.resize(items.size() * zk::GKR_BATCH_RESULT_WORDS);
                qm31 zero = qm31_zero();
                d.check(zk::gkr_batch_round(d.ctx(), items.data(), (int)items.size(), zero.c, eq_evals.words.ptr(), lambda.c, results.data()));
                for (size_t j = 0; j < who.size(); j++) {
                    const uint32_t* w = results.data() + j * zk::GKR_BATCH_RESULT_WORDS;
                    oracles[who[j]].sums = {qm31{{w[0], w[1], w[2], w[3]}}, qm31{{w[4], w[5], w[6], w[7]}}};
                    oracles[who[j]].have_sums = true;
                }
            }
            // Every active oracle has n_rem variables left, so all their round polynomials are r0 L0 + r1 L1 + r2 L2 over the
            // same basis, and the random linear combination over the batch (sumcheck.rs:139-149, Horner in alpha from the
            // last oracle down) is (sum alpha^k r0_k) L0 + (sum alpha^k r1_k) L1 + (sum alpha^k r2_k) L2 plus the constants of
            // the oracles that wait: eleven multiplications per oracle and round instead of a Lagrange interpolation each.
            // r0 + r1 is the claim by construction, which is the check sumcheck.rs:128-130 makes.
            hc.reset(new HostClock("gkr.round.algebra"));
            const RoundBasis basis(ood_point, n_rem);
            const size_t K = oracles.size();
            std::vector<qm31> rv(3 * K);
            std::vector<char> act(K);
            qm31 S[3] = {qm31_zero(), qm31_zero(), qm31_zero()}, Sc = qm31_zero();
            for (size_t k = K; k-- > 0;) {
                for (int t = 0; t < 3; t++) S[t] = S[t] * sumcheck_alpha;
                Sc = Sc * sumcheck_alpha;
                act[k] = n_rem == oracles[k].n_variables();
                if (act[k]) {
                    const qm31 corr = oracles[k].eq_fixed_var_correction;
                    rv[3 * k] = oracles[k].sums.first * corr * basis.e0a;
                    rv[3 * k + 1] = sc_claims[k] - rv[3 * k];
                    rv[3 * k + 2] = oracles[k].sums.second * corr * basis.e2a;
                    oracles[k].have_sums = false;
                    for (int t = 0; t < 3; t++) S[t] = S[t] + rv[3 * k + t];
                } else {
                    rv[3 * k] = qm31_mul_m31(sc_claims[k], half);
                    Sc = Sc + rv[3 * k];
                }
            }
            UniPoly combined;
            combined.c.resize(4);
            for (int t = 0; t < 4; t++) combined.c[t] = S[0] * basis.L[0][t] + S[1] * basis.L[1][t] + S[2] * basis.L[2][t];
            combined.c[0] = combined.c[0] + Sc;
            if (qm31_is_zero(combined.c[3])) {
                // The combination keeps the length of its longest term. A vanishing leading coefficient does not say which
                // case this is (every term short, or a cancellation), so this round goes term by term.
                combined = UniPoly();
                for (size_t k = K; k-- > 0;) {
                    UniPoly rp;
                    if (act[k]) rp = basis.round_poly(rv[3 * k], rv[3 * k + 1], rv[3 * k + 2]);
                    else { rp.c = {rv[3 * k]}; rp.trim(); }
                    for (auto& c : combined.c) c = c * sumcheck_alpha;
                    combined = UniPoly::add(combined, rp);
                }
            }
            hc.reset(new HostClock("gkr.round.channel"));
            ch.mix_felts(combined.c);
            qm31 challenge = ch.draw_secure_felt();
            hc.reset(new HostClock("gkr.round.claims"));
            qm31 Lc[3];
            for (int t = 0; t < 3; t++) Lc[t] = ((basis.L[t][3] * challenge + basis.L[t][2]) * challenge + basis.L[t][1]) * challenge + basis.L[t][0];
            for (size_t k = 0; k < K; k++)
                sc_claims[k] = act[k] ? rv[3 * k] * Lc[0] + rv[3 * k + 1] * Lc[1] + rv[3 * k + 2] * Lc[2] : rv[3 * k];
            const qm31 eq_step = eq1(challenge, ood_point[ood_point.size() - n_rem]);  // the same for every active oracle
            // fix the first variable of every active oracle (and take the next round's sums in the same pass): one launch
            hc.reset(new HostClock("gkr.round.fix_prepare"));
            items.clear();
            who.clear();
            std::vector<Layer> fixed;
            for (size_t k = 0; k < oracles.size(); k++)
                if (n_rem == oracles[k].n_variables() && oracles[k].n_variables() != 0) {
                    oracles[k].eq_fixed_var_correction = oracles[k].eq_fixed_var_correction * eq_step;
                    Layer& in = oracles[k].input_layer;
                    Layer out;  // Layer::fix_first_variable, gkr_prover.rs:354-381
                    out.writable = true;
                    out.kind = in.kind == ZKB_GKR_LOGUP_MULTIPLICITIES ? ZKB_GKR_LOGUP_GENERIC : in.kind;
                    if (in.writable && in.kind != ZKB_GKR_LOGUP_MULTIPLICITIES) {
                        // A thread of the fixing kernel reads entries i and i + n/2 and writes entry i, and no other thread
                        // touches either: the prover's own layers are fixed in place, the result being their first half.
                        out.den.words = BaseColumn::view(d, in.den.words.ptr(), in.den.words.len() / 2);
                        if (out.kind == ZKB_GKR_LOGUP_GENERIC) out.num.words = BaseColumn::view(d, in.num.words.ptr(), in.num.words.len() / 2);
                        items.push_back(item_of(in, out, in.len() >= 8 ? 1 : 2));
                        // keep the allocation alive under its new, shorter shape
                        in.den.words.shrink(in.den.words.len() / 2);
                        if (out.kind == ZKB_GKR_LOGUP_GENERIC) in.num.words.shrink(in.num.words.len() / 2);
                        out = std::move(in);
                        out.writable = true;
                    } else {
                        out.den = SecureMle(d, in.len() / 2);
                        if (out.kind == ZKB_GKR_LOGUP_GENERIC) out.num = SecureMle(d, in.len() / 2);
                        items.push_back(item_of(in, out, in.len() >= 8 ? 1 : 2));
                    }
                    fixed.push_back(std::move(out));
                    who.push_back(k);
                }
            if (!items.empty()) {
                hc.reset(new HostClock("gkr.round.fix_launch_wait"));
                results.resize(items.size() * zk::GKR_BATCH_RESULT_WORDS);
                d.check(zk::gkr_batch_round(d.ctx(), items.data(), (int)items.size(), challenge.c, eq_evals.words.ptr(), lambda.c, results.data()));
                hc.reset(new HostClock("gkr.round.fix_results"));
                for (size_t j = 0; j < who.size(); j++) {
                    GkrOracle& o = oracles[who[j]];
                    const uint32_t* w = results.data() + j * zk::GKR_BATCH_RESULT_WORDS;
                    if (items[j].mode == 1) {
                        o.sums = {qm31{{w[0], w[1], w[2], w[3]}}, qm31{{w[4], w[5], w[6], w[7]}}};
                        o.have_sums = true;
                    } else {
                        for (int e = 0; e < 2; e++) {
                            o.mask_den[e] = qm31{{w[8 + 4 * e], w[9 + 4 * e], w[10 + 4 * e], w[11 + 4 * e]}};
                            o.mask_num[e] = qm31{{w[16 + 4 * e], w[17 + 4 * e], w[18 + 4 * e], w[19 + 4 * e]}};
                        }
                        o.have_mask = true;
                    }
                    o.input_layer = std::move(fixed[j]);
                }
            }
            hc.reset();
            round_polys.push_back(combined);
            assignment.push_back(challenge);
        }
        HostClock hc_masks("gkr.layer.masks");
        sumcheck_round_polys.push_back(round_polys);
        // try_into_mask, :572-597. A mask is one column pair (grand product) or two (numerators, denominators): kept as flat
        // records; a batch has hundreds of oracles per layer, and a vector of vectors per oracle cost more than the hashing.
        std::vector<MaskRec> masks(oracles.size());
        // An oracle that entered this layer with two entries had no sum-check round, so no launch has returned its mask:
        // those (every instance once, in the layer above its output) are read in one gather, not one copy per column.
        GatherPlan mask_plan;
        std::vector<size_t> mask_slot(oracles.size(), SIZE_MAX);
        for (size_t k = 0; k < oracles.size(); k++) {
            const GkrOracle& o = oracles[k];
            if (o.have_mask || o.input_layer.len() != 2) continue;
            mask_slot[k] = mask_plan.addrs.size();
            for (int w = 0; w < 8; w++) mask_plan.add(o.input_layer.den.words.ptr() + w);
            if (o.input_layer.kind == ZKB_GKR_LOGUP_GENERIC)
                for (int w = 0; w < 8; w++) mask_plan.add(o.input_layer.num.words.ptr() + w);
        }
        if (!mask_plan.addrs.empty()) mask_plan.execute(d);
        auto gathered = [&](size_t slot) { return qm31{{mask_plan.words[slot], mask_plan.words[slot + 1], mask_plan.words[slot + 2], mask_plan.words[slot + 3]}}; };
        for (size_t k = 0; k < oracles.size(); k++) {
            const GkrOracle& o = oracles[k];
            const Layer& l = o.input_layer;
            if (l.len() != 2) throw Error(ZKB_EINVAL, "gkr: oracle is not constant after sumcheck");
            MaskRec& m = masks[k];
            qm31 den[2], num[2];
            if (o.have_mask) { den[0] = o.mask_den[0]; den[1] = o.mask_den[1]; }
            else { den[0] = gathered(mask_slot[k]); den[1] = gathered(mask_slot[k] + 4); }
            if (l.kind == ZKB_GKR_GRAND_PRODUCT) { m.n_cols = 1; m.v[0] = den[0]; m.v[1] = den[1]; continue; }
            if (l.kind == ZKB_GKR_LOGUP_GENERIC) {
                if (o.have_mask) { num[0] = o.mask_num[0]; num[1] = o.mask_num[1]; }
                else { num[0] = gathered(mask_slot[k] + 8); num[1] = gathered(mask_slot[k] + 12); }
            } else if (l.kind == ZKB_GKR_LOGUP_SINGLES) num[0] = num[1] = qm31_one();
            else throw Error(ZKB_EINVAL, "gkr: a multiplicities layer cannot be a mask");
            m.n_cols = 2; m.v[0] = num[0]; m.v[1] = num[1]; m.v[2] = den[0]; m.v[3] = den[1];
        }
        for (size_t k = 0; k < oracles.size(); k++) {
            ch.mix_felts(masks[k].v, 2 * masks[k].n_cols);
            masks_by_inst[sc_inst[k]].push_back(masks[k]);
        }
        qm31 challenge = ch.draw_secure_felt();
        ood_point = assignment;
        ood_point.push_back(challenge);
        for (size_t k = 0; k < oracles.size(); k++) {
            std::vector<qm31>& next = claims[sc_inst[k]];
            next.resize(masks[k].n_cols);
            for (uint32_t c = 0; c < masks[k].n_cols; c++) next[c] = challenge * (masks[k].v[2 * c + 1] - masks[k].v[2 * c]) + masks[k].v[2 * c];
        }
    }
    std::vector<uint32_t> o;
    auto put = [&](qm31 q) { o.insert(o.end(), q.c, q.c + 4); };
    o.push_back((uint32_t)sumcheck_round_polys.size());
    for (auto& l : sumcheck_round_polys) {
        o.push_back((uint32_t)l.size());
        for (auto& p : l) { o.push_back((uint32_t)p.c.size()); for (auto q : p.c) put(q); }
    }
    for (auto& inst : masks_by_inst) {
        o.push_back((uint32_t)inst.size());
        for (auto& m : inst) { o.push_back(m.n_cols); for (uint32_t c = 0; c < 2 * m.n_cols; c++) put(m.v[c]); }
    }
    for (auto& c : output_claims) { o.push_back((uint32_t)c.size()); for (auto q : c) put(q); }
    o.push_back((uint32_t)ood_point.size());
    for (auto q : ood_point) put(q);
    for (auto& c : claims) { o.push_back((uint32_t)c.size()); for (auto q : c) put(q); }
    return o;
}

// ------------------------------------------------------------------ one PCS proof over G ranks
// The reference has no multi-device code; this is the proof of pcs_prove_impl (one tree of equally sized columns, one
// out-of-domain sample per column) with the data-parallel phases sharded: rank r interpolates and extends ncols / G
// columns; an exchange (the caller's: the library moves no data between devices) turns the column shards into row
// shards [ncols][N / G]; every rank hashes the Merkle subtree over its rows, evaluates its own polynomials at the
// out-of-domain point and computes the quotients of its rows. The Fiat-Shamir channel is replicated: every rank mixes
// the same values in the same order. The quotient column (4 x N words, 1 / (ncols / 4) of the evaluations) is gathered
// by the caller and every rank runs the same FRI commitment, grind and query draw on it; a rank then decommits the
// queried rows it owns, and any rank merges the parts, layer by layer in rank order, into the single-device proof's words.
struct ShardSession {
    zkb_ctx* ctx;
    Device dev;
    int rank, world, log_g, ncols, ncl, n_chunks = 1;
    uint32_t* ext_rows = nullptr;
    std::vector<uint32_t*> peer_rows;  // every rank's receive buffer as this process sees it (own buffer at [rank]); empty: the caller exchanges
    uint32_t log_n, log_out, log_local;
    size_t N, R;
    PcsConfig config;
    Channel ch;
    std::vector<BaseColumn> coeffs;    // views of the caller's local columns, interpolated in place
    BaseColumn evals;                  // [ncl][N]
    BaseColumn rows;                   // [ncols][R]; global column c = source rank * ncl + j
    std::vector<BaseColumn> row_cols;  // views of `rows`
    MerkleProver subtree, top;
    BaseColumn roots;                  // [world][8]
    Hash root{};
    CirclePointQ oods{};
    std::vector<qm31> samples;
    SecureColumnByCoords quot_local, quot_full;
    FriProver fri;
    uint64_t nonce = 0;
    std::vector<size_t> query_positions;
    FriProof fri_proof;
    MerkleDecommitment top_dec;
    ShardSession(zkb_ctx* c) : ctx(c), dev(c) {}
};

}  // namespace b200

struct zkb_shard_pcs { b200::ShardSession s; zkb_shard_pcs(zkb_ctx* c) : s(c) {} };

namespace b200 {

template <class F> static int shard_guard(zkb_ctx* ctx, F&& f) {
    try {
        f();
        return ZKB_OK;
    } catch (const Error& e) {
        return zk_set_error_public(ctx, e.code, e.what());
    } catch (const std::exception& e) {
        return zk_set_error_public(ctx, ZKB_ENOMEM, e.what());
    }
}

}  // namespace b200

using namespace b200;

extern "C" {

int zkb_shard_pcs_begin(zkb_ctx* ctx, int rank, int world, int ncols_total, int log_n, const zkb_pcs_config* cfg, zkb_shard_pcs** out) {
    if (!ctx || !cfg || !out) return ZKB_EINVAL;
    *out = nullptr;
    if (world < 1 || (world & (world - 1)) || rank < 0 || rank >= world || ncols_total < world || ncols_total % world || log_n < 1)
        return zk_set_error_public(ctx, ZKB_EINVAL, "zkb_shard_pcs_begin: the rank count must be a power of two that divides the column count");
    int log_g = 0;
    while ((1 << log_g) < world) log_g++;
    int log_out = log_n + (int)cfg->log_blowup_factor;
    if (log_out > zkb_max_log_size(ctx) || log_out - log_g < 3)
        return zk_set_error_public(ctx, ZKB_EINVAL, "zkb_shard_pcs_begin: every rank needs at least 8 rows and the context must cover the evaluation domain");
    return shard_guard(ctx, [&] {
        auto* h = new zkb_shard_pcs(ctx);
        ShardSession& s = h->s;
        s.rank = rank; s.world = world; s.log_g = log_g; s.ncols = ncols_total; s.ncl = ncols_total / world;
        s.log_n = (uint32_t)log_n; s.log_out = (uint32_t)log_out; s.log_local = (uint32_t)(log_out - log_g);
        s.N = (size_t)1 << log_out; s.R = s.N >> log_g;
        s.config = PcsConfig{cfg->pow_bits, {cfg->log_blowup_factor, cfg->log_last_layer_degree_bound, cfg->n_queries, 1}};
        s.config.mix_into(s.ch);
        *out = h;
    });
}

int zkb_shard_pcs_end(zkb_shard_pcs* h) {
    if (!h) return ZKB_EINVAL;
    zkb_ctx* ctx = h->s.ctx;
    zkb_sync(ctx);
    delete h;
    return ZKB_OK;
}

int zkb_shard_pcs_set_rows(zkb_shard_pcs* h, uint32_t* d_rows) {
    if (!h) return ZKB_EINVAL;
    h->s.ext_rows = d_rows;
    return ZKB_OK;
}

int zkb_shard_pcs_set_peer_rows(zkb_shard_pcs* h, uint32_t* const* peer_rows) {
    if (!h) return ZKB_EINVAL;
    ShardSession& s = h->s;
    s.peer_rows.clear();
    if (!peer_rows) return ZKB_OK;
    for (int r = 0; r < s.world; r++) {
        if (!peer_rows[r]) return zk_set_error_public(s.ctx, ZKB_EINVAL, "zkb_shard_pcs_set_peer_rows: null buffer");
        s.peer_rows.push_back(peer_rows[r]);
    }
    s.ext_rows = s.peer_rows[s.rank];
    return ZKB_OK;
}

int zkb_shard_pcs_extend_begin(zkb_shard_pcs* h, uint32_t* const* d_cols, int n_chunks) {
    if (!h || !d_cols) return ZKB_EINVAL;
    ShardSession& s = h->s;
    if (n_chunks < 1 || s.ncl % n_chunks) return zk_set_error_public(s.ctx, ZKB_EINVAL, "zkb_shard_pcs_extend_begin: the chunk count must divide the local column count");
    return shard_guard(s.ctx, [&] {
        std::vector<BaseColumn*> cols;
        s.coeffs.clear();
        for (int c = 0; c < s.ncl; c++) s.coeffs.push_back(BaseColumn::view(s.dev, d_cols[c], (size_t)1 << s.log_n));
        for (auto& c : s.coeffs) cols.push_back(&c);
        B200Backend::interpolate_columns(s.dev, cols);
        s.n_chunks = n_chunks;
        s.evals = BaseColumn(s.dev, (size_t)s.ncl * s.N);  // [chunk][world][ncl / chunks][R]: block d of a chunk is what rank d receives
        // [chunk][source rank][ncl / chunks][R]; the caller's own buffer when it has given one (a buffer its peers can write)
        s.rows = s.ext_rows ? BaseColumn::view(s.dev, s.ext_rows, (size_t)s.ncols * s.R) : BaseColumn(s.dev, (size_t)s.ncols * s.R);
    });
}

int zkb_shard_pcs_extend_chunk(zkb_shard_pcs* h, int k, uint32_t** d_send, uint32_t** d_recv, size_t* words_per_peer) {
    if (!h || !d_send || !d_recv || !words_per_peer) return ZKB_EINVAL;
    ShardSession& s = h->s;
    if (k < 0 || k >= s.n_chunks || s.coeffs.empty()) return zk_set_error_public(s.ctx, ZKB_EINVAL, "zkb_shard_pcs_extend_chunk: no such chunk");
    return shard_guard(s.ctx, [&] {
        const int cc = s.ncl / s.n_chunks;
        std::vector<const uint32_t*> src;
        std::vector<uint32_t*> dst;
        uint32_t* send = s.evals.ptr() + (size_t)k * s.world * cc * s.R;
        for (int j = 0; j < cc; j++) src.push_back(s.coeffs[k * cc + j].ptr());
        if (zk::lde_blocked_supported((int)s.log_n, (int)s.log_out, (int)s.log_local)) {
            // the transform's last pass writes every row block where the exchange sends it from: no repack
            for (int j = 0; j < cc; j++) dst.push_back(send + (size_t)j * s.R);
            s.dev.check(zk::lde_cols_blocked(s.ctx, src.data(), cc, (int)s.log_n, dst.data(), (int)s.log_out, (int)s.log_local,
                                             (uint32_t)((size_t)cc * s.R)));
        } else {
            BaseColumn plain(s.dev, (size_t)cc * s.N);
            for (int j = 0; j < cc; j++) dst.push_back(plain.ptr() + (size_t)j * s.N);
            s.dev.check(zkb_lde_cols(s.ctx, src.data(), cc, (int)s.log_n, dst.data(), (int)s.log_out));
            s.dev.check(zk::repack_row_blocks(s.ctx, plain.ptr(), send, cc, (int)s.log_out, (int)s.log_local));
        }
        *d_send = send;
        *d_recv = s.rows.ptr() + (size_t)k * s.world * cc * s.R;
        *words_per_peer = (size_t)cc * s.R;
        if (!s.peer_rows.empty()) {
            // block d of the chunk goes to rank d's buffer, into the place of this rank's block there: copy engines, after the
            // transform just enqueued, four copies side by side; every rank starts with a different peer
            const size_t words = (size_t)cc * s.R, at = ((size_t)k * s.world + s.rank) * words;
            for (int j = 0; j < s.world; j++) {
                const int dst = (s.rank + j) % s.world;
                s.dev.check(zkb_copy_to_peer(s.ctx, s.peer_rows[dst] + at, send + (size_t)dst * words, words * 4, j));
            }
        }
    });
}

int zkb_shard_pcs_extend(zkb_shard_pcs* h, uint32_t* const* d_cols, uint32_t** d_send, uint32_t** d_rows) {
    if (!h || !d_cols || !d_send || !d_rows) return ZKB_EINVAL;
    int rc = zkb_shard_pcs_extend_begin(h, d_cols, 1);
    if (rc) return rc;
    size_t words = 0;
    return zkb_shard_pcs_extend_chunk(h, 0, d_send, d_rows, &words);
}

int zkb_shard_pcs_subtree(zkb_shard_pcs* h, uint32_t** d_root, uint32_t** d_roots) {
    if (!h || !d_root || !d_roots) return ZKB_EINVAL;
    ShardSession& s = h->s;
    return shard_guard(s.ctx, [&] {
        s.evals = BaseColumn();  // the column shards have been sent
        s.row_cols.clear();
        // global column c = source rank * ncl + chunk * cc + j lies in block [chunk][source rank] of the received rows
        const int cc = s.ncl / s.n_chunks;
        for (int c = 0; c < s.ncols; c++) {
            const int src = c / s.ncl, k = (c % s.ncl) / cc, j = c % cc;
            s.row_cols.push_back(BaseColumn::view(s.dev, s.rows.ptr() + ((size_t)(k * s.world + src) * cc + j) * s.R, s.R));
        }
        std::vector<const BaseColumn*> refs;
        for (auto& c : s.row_cols) refs.push_back(&c);
        s.subtree = MerkleProver::commit(s.dev, refs);
        s.roots = BaseColumn(s.dev, (size_t)8 * s.world);
        *d_root = s.subtree.layers[0].ptr();
        *d_roots = s.roots.ptr();
    });
}

int zkb_shard_pcs_sample(zkb_shard_pcs* h, uint32_t* h_samples) {
    if (!h || !h_samples) return ZKB_EINVAL;
    ShardSession& s = h->s;
    return shard_guard(s.ctx, [&] {
        // the top log2(G) layers over the gathered subtree roots: the same nodes the single-device tree has there
        s.top = MerkleProver();
        s.top.layers.resize(s.log_g + 1);
        s.top.layers[s.log_g] = BaseColumn::view(s.dev, s.roots.ptr(), (size_t)8 * s.world);
        for (int lg = s.log_g - 1; lg >= 0; lg--) s.top.layers[lg] = B200Backend::commit_on_layer(s.dev, (uint32_t)lg, &s.top.layers[lg + 1], {});
        s.root = s.top.root(s.dev);
        s.ch.mix_root(s.root);
        s.oods = get_random_point(s.ch);
        std::vector<const BaseColumn*> polys;
        for (auto& c : s.coeffs) polys.push_back(&c);
        auto vals = B200Backend::batch_eval_at_point(s.dev, polys, s.oods);
        for (int c = 0; c < s.ncl; c++) memcpy(h_samples + 4 * c, vals[c].c, 16);
    });
}

int zkb_shard_pcs_quotients(zkb_shard_pcs* h, const uint32_t* h_all_samples, uint32_t* d_quot_local[4], uint32_t* d_quot_full[4]) {
    if (!h || !h_all_samples || !d_quot_local || !d_quot_full) return ZKB_EINVAL;
    ShardSession& s = h->s;
    return shard_guard(s.ctx, [&] {
        s.samples.resize(s.ncols);
        for (int c = 0; c < s.ncols; c++) memcpy(s.samples[c].c, h_all_samples + 4 * c, 16);
        s.ch.mix_felts(s.samples);
        qm31 random_coeff = s.ch.draw_secure_felt();
        // compute_fri_quotients for one size group and one sample point, on this rank's rows: the numerators are
        // row-local; the denominators need the rows' domain points (zkb_quot_combine_rows)
        std::vector<const BaseColumn*> refs;
        for (auto& c : s.row_cols) refs.push_back(&c);
        ColumnSampleBatch batch{s.oods, {}};
        qm31 pow = qm31_one();
        for (int c = 0; c < s.ncols; c++) { batch.cols_vals_randpows.push_back({(size_t)c, s.samples[c], pow}); pow = pow * random_coeff; }
        std::vector<AccumulatedNumerators> accs;
        B200Backend::accumulate_numerators(s.dev, refs, {batch}, accs);
        s.quot_local = SecureColumnByCoords(s.dev, s.R);
        s.quot_full = SecureColumnByCoords(s.dev, s.N);
        std::vector<const uint32_t*> cols;
        for (auto p : accs[0].partial_numerators_acc.cptrs()) cols.push_back(p);
        int acc_log = (int)s.log_out;
        uint32_t pts[8];
        memcpy(pts, s.oods.x.c, 16);
        memcpy(pts + 4, s.oods.y.c, 16);
        auto o = s.quot_local.ptrs();
        s.dev.check(zkb_quot_combine_rows(s.ctx, 1, cols.data(), &acc_log, accs[0].first_linear_term_acc.c, pts, (int)s.log_out,
                                          (size_t)s.rank * s.R, s.R, o.data()));
        s.dev.check(zkb_sync(s.ctx));  // the accumulation is freed when this returns; the caller's gather may run on another stream
        auto f = s.quot_full.ptrs();
        for (int k = 0; k < 4; k++) { d_quot_local[k] = o[k]; d_quot_full[k] = f[k]; }
    });
}

// Serialised part of one rank: [layers L][per layer: count, count x 8 words][n value words][values].
int zkb_shard_pcs_fri_and_decommit(zkb_shard_pcs* h, uint32_t* h_part, size_t cap, size_t* n_words) {
    if (!h || !h_part || !n_words) return ZKB_EINVAL;
    ShardSession& s = h->s;
    return shard_guard(s.ctx, [&] {
        s.fri = FriProver::commit(s.dev, s.ch, s.config.fri, s.quot_full);
        s.nonce = B200Backend::grind(s.dev, s.ch.pow_prefixed_digest(s.config.pow_bits), s.config.pow_bits);
        s.ch.mix_u64(s.nonce);
        GatherPlan plan;
        auto fri_pending = s.fri.plan_decommit(plan, s.dev, s.ch, s.query_positions);
        // this rank's rows among the queried ones, and the ranks that own any
        std::vector<size_t> local, owners;
        for (auto q : s.query_positions) {
            if ((q >> s.log_local) == (size_t)s.rank) local.push_back(q - ((size_t)s.rank << s.log_local));
            owners.push_back(q >> s.log_local);
        }
        std::vector<const BaseColumn*> refs;
        for (auto& c : s.row_cols) refs.push_back(&c);
        std::vector<size_t> per_layer, top_per_layer;
        PendingMerkle pm = s.subtree.plan_decommit(plan, {{s.log_local, sorted_dedup(local)}}, refs, &per_layer);
        PendingMerkle pt = s.top.plan_decommit(plan, {{(uint32_t)s.log_g, sorted_dedup(owners)}}, {}, &top_per_layer);
        plan.execute(s.dev);
        s.fri_proof = s.fri.finish_decommit(plan, fri_pending);
        s.top_dec = pt.finish(plan).second;
        auto mine = pm.finish(plan);
        std::vector<uint32_t> o;
        o.push_back((uint32_t)per_layer.size());
        size_t at = 0;
        for (size_t cnt : per_layer) {
            o.push_back((uint32_t)cnt);
            for (size_t k = 0; k < cnt; k++, at++) o.insert(o.end(), mine.second.hash_witness[at].begin(), mine.second.hash_witness[at].end());
        }
        o.push_back((uint32_t)mine.first.size());
        mine.first.append_to(o);
        *n_words = o.size();
        if (o.size() > cap) throw Error(ZKB_EINVAL, "zkb_shard_pcs_fri_and_decommit: output buffer too small");
        memcpy(h_part, o.data(), o.size() * 4);
    });
}

int zkb_shard_pcs_finish(zkb_shard_pcs* h, const uint32_t* const* h_parts, const size_t* part_words, uint32_t* h_out, size_t cap,
                         size_t* n_words) {
    if (!h || !h_parts || !part_words || !h_out || !n_words) return ZKB_EINVAL;
    ShardSession& s = h->s;
    return shard_guard(s.ctx, [&] {
        PcsProof proof;
        proof.commitments.push_back(s.root);
        proof.sampled_values.emplace_back();
        for (auto v : s.samples) proof.sampled_values[0].push_back({v});
        MerkleDecommitment dec;
        std::vector<uint32_t> values;
        std::vector<size_t> cursor(s.world, 1);
        size_t n_layers = 0;
        for (int r = 0; r < s.world; r++) {
            if (part_words[r] < 2) throw Error(ZKB_EINVAL, "zkb_shard_pcs_finish: truncated part");
            if (r == 0) n_layers = h_parts[0][0];
            else if (h_parts[r][0] != n_layers) throw Error(ZKB_EINVAL, "zkb_shard_pcs_finish: the parts disagree on the layer count");
        }
        // the single-device decommitment lists a layer's witness hashes in node order: rank order within each layer
        for (size_t l = 0; l < n_layers; l++)
            for (int r = 0; r < s.world; r++) {
                const uint32_t* p = h_parts[r];
                size_t& c = cursor[r];
                if (c >= part_words[r]) throw Error(ZKB_EINVAL, "zkb_shard_pcs_finish: truncated part");
                size_t cnt = p[c++];
                if (c + 8 * cnt > part_words[r]) throw Error(ZKB_EINVAL, "zkb_shard_pcs_finish: truncated part");
                for (size_t k = 0; k < cnt; k++, c += 8) { Hash hh; memcpy(hh.data(), p + c, 32); dec.hash_witness.push_back(hh); }
            }
        dec.hash_witness.insert(dec.hash_witness.end(), s.top_dec.hash_witness.begin(), s.top_dec.hash_witness.end());
        for (int r = 0; r < s.world; r++) {
            const uint32_t* p = h_parts[r];
            size_t c = cursor[r];
            if (c >= part_words[r]) throw Error(ZKB_EINVAL, "zkb_shard_pcs_finish: truncated part");
            size_t cnt = p[c++];
            if (c + cnt > part_words[r]) throw Error(ZKB_EINVAL, "zkb_shard_pcs_finish: truncated part");
            values.insert(values.end(), p + c, p + c + cnt);
        }
        proof.decommitments.push_back(std::move(dec));
        proof.queried_values.push_back(Words{std::move(values), {}});
        proof.proof_of_work = s.nonce;
        proof.fri = s.fri_proof;
        PcsProof::RawSink w{h_out, cap};
        proof.write(w);
        w.insert(w.end(), s.ch.digest().begin(), s.ch.digest().end());
        *n_words = w.size();
        if (w.size() > cap) throw Error(ZKB_EINVAL, "zkb_shard_pcs_finish: output buffer too small");
    });
}

}  // extern "C"


// Commits the caller's trees in order (TreeBuilder::extend_evals + commit per tree), from device columns or from host
// columns with the upload overlapped.
static void commit_input_trees(Device& dev, zkb_ctx* ctx, CommitmentSchemeProver& prover, Channel& ch, int n_trees, const int* tree_ncols,
                               uint32_t* const* d_cols, const uint32_t* const* h_cols, const uint32_t* col_logs, int total) {
        int flat = 0;
        if (d_cols) {
            for (int t = 0; t < n_trees; t++) {
                std::vector<BaseColumn> columns;
                for (int c = 0; c < tree_ncols[t]; c++, flat++)
                    columns.push_back(BaseColumn::view(dev, d_cols[flat], (size_t)1 << col_logs[flat]));
                prover.commit_evals(std::move(columns), ch);
            }
        } else {
            // Host columns: every copy of every tree is enqueued on the copy stream first, with a fence
            // after each ~1/32 of the bytes, so that the transfer runs at link speed from start to end
            // while the compute stream interpolates and extends what has already arrived.
            size_t total_bytes = 0;
            for (int i = 0; i < total; i++) total_bytes += (size_t)4 << col_logs[i];
            const size_t per_fence = std::max<size_t>(total_bytes / 32, 1);
            // The columns of a tree live in one allocation (each padded to 64 words), so that columns that
            // are adjacent in host memory, as a row-major trace is, go up in one copy per fence.
            std::vector<std::vector<BaseColumn>> tree_cols(n_trees);
            std::vector<std::vector<int>> tree_fences(n_trees);
            std::vector<BaseColumn> slabs;
            for (int t = 0; t < n_trees; t++) {
                size_t words = 0;
                for (int c = 0; c < tree_ncols[t]; c++) words += std::max<size_t>((size_t)1 << col_logs[flat + c], 64);
                if (words) slabs.emplace_back(dev, words);
                else slabs.emplace_back();  // a tree without columns (it is still committed: its root is the hash of nothing)
                size_t off = 0;
                for (int c = 0; c < tree_ncols[t]; c++, flat++) {
                    size_t n = (size_t)1 << col_logs[flat];
                    tree_cols[t].push_back(BaseColumn::view(dev, slabs.back().ptr() + off, n));
                    off += std::max<size_t>(n, 64);
                }
            }
            flat = 0;
            int fence = 0;
            size_t since = 0;
            // a pending run of copies that are contiguous on both sides
            uint32_t* run_dst = nullptr;
            const uint32_t* run_src = nullptr;
            size_t run_bytes = 0;
            auto flush = [&](int fence_id) {
                if (run_bytes) dev.check(zkb_h2d_overlapped(ctx, run_dst, run_src, run_bytes, fence_id));
                else if (fence_id >= 0) dev.check(zkb_h2d_overlapped(ctx, nullptr, nullptr, 0, fence_id));
                run_bytes = 0;
            };
            try {  // from the first enqueued copy on, no column may be freed while the copy stream still writes into it
            for (int t = 0; t < n_trees; t++)
                for (int c = 0; c < tree_ncols[t]; c++, flat++) {
                    size_t bytes = (size_t)4 << col_logs[flat];
                    uint32_t* dst = tree_cols[t][c].ptr();
                    if (run_bytes && (const uint8_t*)run_src + run_bytes == (const uint8_t*)h_cols[flat] &&
                        (uint8_t*)run_dst + run_bytes == (uint8_t*)dst) {
                        run_bytes += bytes;
                    } else {
                        flush(-1);
                        run_dst = dst; run_src = h_cols[flat]; run_bytes = bytes;
                    }
                    since += bytes;
                    bool close = since >= per_fence || flat == total - 1;
                    tree_fences[t].push_back(fence);
                    if (close) { flush(fence); since = 0; if (fence < 63) fence++; }
                }
                for (int t = 0; t < n_trees; t++) prover.commit_evals(std::move(tree_cols[t]), ch, &tree_fences[t], &slabs[t]);
            } catch (...) {
                zkb_sync(ctx);
                throw;
            }
        }
}

static int pcs_prove_impl(zkb_ctx* ctx, int n_trees, const int* tree_ncols, uint32_t* const* d_cols, const uint32_t* const* h_cols,
                          const uint32_t* col_logs, const zkb_pcs_config* cfg, int two_sample_every, uint32_t* h_out, size_t cap,
                          size_t* n_words, float* h_phase_ms) {
    if (!ctx) return ZKB_EINVAL;
    if (!tree_ncols || !col_logs || !cfg || !h_out || !n_words || n_trees <= 0 || (!d_cols && !h_cols)) return ZKB_EINVAL;
    try {
        Device dev(ctx);
        PcsConfig config{cfg->pow_bits, {cfg->log_blowup_factor, cfg->log_last_layer_degree_bound, cfg->n_queries, 1}};
        int total = 0;
        uint32_t max_log = 0;
        for (int t = 0; t < n_trees; t++) total += tree_ncols[t];
        for (int i = 0; i < total; i++) max_log = std::max(max_log, col_logs[i]);
        if ((int)(max_log + config.fri.log_blowup_factor) > zkb_max_log_size(ctx)) return ZKB_EINVAL;
        Channel ch;
        config.mix_into(ch);
        CommitmentSchemeProver prover(dev, config, h_phase_ms);
        {
            HostClock hcc("pcs.commit_trees");
            commit_input_trees(dev, ctx, prover, ch, n_trees, tree_ncols, d_cols, h_cols, col_logs, total);
        }
        int flat = 0;
        CirclePointQ oods = get_random_point(ch);
        std::vector<std::vector<std::vector<CirclePointQ>>> points(n_trees);
        flat = 0;
        for (int t = 0; t < n_trees; t++)
            for (int c = 0; c < tree_ncols[t]; c++, flat++) {
                std::vector<CirclePointQ> p;
                if (two_sample_every && flat % two_sample_every == 0) {
                    // one trace step back: the conjugate of the step of CanonicCoset(col_log)
                    cpoint st = host_circle_point(1u << (31 - col_logs[flat]));
                    p.push_back(point_add(oods, {qm31_from_m31(st.x), qm31_from_m31(m31_neg(st.y))}));
                }
                p.push_back(oods);
                points[t].push_back(p);
            }
        std::unique_ptr<HostClock> hc(new HostClock("pcs.prove_values"));
        PcsProof proof = prover.prove_values(points, ch);
        prover.finish_timing();
        hc.reset(new HostClock("pcs.write"));
        PcsProof::RawSink w{h_out, cap};  // straight into the caller's buffer: a proof of many columns is tens of megabytes
        proof.write(w);
        w.insert(w.end(), ch.digest().begin(), ch.digest().end());
        *n_words = w.size();
        hc.reset();
        HostClock::dump("zkb_pcs_prove");
        if (w.size() > cap) return zk_set_error_public(ctx, ZKB_EINVAL, "zkb_pcs_prove: output buffer too small");
        return ZKB_OK;
    } catch (const Error& e) {
        return zk_set_error_public(ctx, e.code, e.what());
    } catch (const std::exception& e) {
        return zk_set_error_public(ctx, ZKB_ENOMEM, e.what());
    }
}

// prove() (STWO/prover/mod.rs:41-173) for a statement of one or more components: commit the trees, draw the random
// coefficient, evaluate every component's constraint quotients on the evaluation domain of twice its trace size
// (zkb_constraint_quotients) into the accumulation of that size, lift and add the accumulations
// (DomainEvaluationAccumulator, prover/air/accumulation.rs), interpolate and split the composition polynomial, commit its
// eight coordinate halves, sample every column at its mask points around a drawn out-of-domain point, and prove the
// samples. The prover's own sanity check - the composition polynomial's value at the point, once from the committed
// halves (core/proof.rs:27-57) and once from the constraints at the sampled mask values (core/air/components.rs:76-94,
// constraint-framework/src/component.rs:374-413, point.rs) - is returned in oods_evals for the caller to compare.
static int stark_prove_impl(zkb_ctx* ctx, int n_trees, const int* tree_ncols, uint32_t* const* d_cols, const uint32_t* const* h_cols,
                            int n_components, const zkb_stark_component* comps, const zkb_pcs_config* cfg, uint32_t* h_out, size_t cap,
                            size_t* n_words, uint32_t* oods_evals, float* h_phase_ms, float* composition_ms) {
    if (!ctx) return ZKB_EINVAL;
    if (!tree_ncols || !cfg || !h_out || !n_words || !comps || !oods_evals || n_trees <= 0 || n_components <= 0 || (!d_cols && !h_cols))
        return ZKB_EINVAL;
    try {
        Device dev(ctx);
        PcsConfig config{cfg->pow_bits, {cfg->log_blowup_factor, cfg->log_last_layer_degree_bound, cfg->n_queries, 1}};
        const uint32_t blowup = config.fri.log_blowup_factor;
        uint32_t max_trace_log = 0;
        size_t n_constraints = 0;
        for (int k = 0; k < n_components; k++) {
            const zkb_stark_component& c = comps[k];
            if (!c.prog || c.trace_log < 1 || (size_t)n_trees != c.prog->tree_base.size() || (c.prog->n_scalars && !c.scalars))
                return zk_set_error_public(ctx, ZKB_EINVAL, "zkb_stark_prove: a component has no program, no scalars, or a program compiled for other trees");
            max_trace_log = std::max(max_trace_log, c.trace_log);
            n_constraints += c.prog->constraints.size();
        }
        if (blowup < 1 || (int)(max_trace_log + blowup) > zkb_max_log_size(ctx)) return ZKB_EINVAL;
        // where each component's columns start in each tree (they follow those of the components before it), column sizes
        auto cols_of = [&](int k, int t) {
            const auto& tb = comps[k].prog->tree_base;
            return (t + 1 < n_trees ? tb[t + 1] : comps[k].prog->n_cols) - tb[t];
        };
        std::vector<std::vector<uint32_t>> first((size_t)n_components, std::vector<uint32_t>((size_t)n_trees, 0));
        std::vector<uint32_t> tree_start((size_t)n_trees, 0), col_logs;
        int total = 0;
        for (int t = 0; t < n_trees; t++) {
            tree_start[t] = (uint32_t)total;
            uint32_t at = 0;
            for (int k = 0; k < n_components; k++) {
                first[k][t] = at;
                at += cols_of(k, t);
                col_logs.insert(col_logs.end(), cols_of(k, t), comps[k].trace_log);
            }
            if ((int)at != tree_ncols[t])
                return zk_set_error_public(ctx, ZKB_EINVAL, "zkb_stark_prove: the trees do not have the columns the programs were compiled for");
            total += tree_ncols[t];
        }
        Channel ch;
        config.mix_into(ch);
        CommitmentSchemeProver prover(dev, config, h_phase_ms);
        commit_input_trees(dev, ctx, prover, ch, n_trees, tree_ncols, d_cols, h_cols, col_logs.data(), total);

        // ---- composition polynomial
        const qm31 random_coeff = ch.draw_secure_felt();
        dev.check(zkb_event_record(ctx, 28));
        std::vector<qm31> ascending_powers(n_constraints);
        {
            qm31 pw = qm31_one();
            for (size_t i = 0; i < n_constraints; i++) { ascending_powers[i] = pw; pw = pw * random_coeff; }
        }
        size_t remaining = n_constraints;
        std::map<uint32_t, SecureColumnByCoords> sub;  // sub_accumulations by log size
        std::vector<qm31> shifts((size_t)n_components, qm31_zero());
        for (int k = 0; k < n_components; k++) {
            const zkb_stark_component& c = comps[k];
            const size_t n_k = c.prog->constraints.size();
            // columns(): the last n_k powers, reversed so that the component's first constraint takes the highest (component_prover.rs:271)
            std::vector<qm31> powers(n_k);
            for (size_t i = 0; i < n_k; i++) powers[i] = ascending_powers[remaining - 1 - i];
            remaining -= n_k;
            const uint32_t eval_log = c.trace_log + 1;
            // the component's columns on its evaluation domain: the committed evaluations themselves when the blow-up is 2
            std::vector<BaseColumn> extended;
            std::vector<const uint32_t*> col_ptrs;
            for (int t = 0; t < n_trees; t++) {
                const uint32_t cnt = cols_of(k, t);
                if (blowup == 1) {
                    for (uint32_t q = 0; q < cnt; q++) col_ptrs.push_back(prover.trees[t].evals[first[k][t] + q].ptr());
                } else if (cnt) {
                    std::vector<const BaseColumn*> cc;
                    for (uint32_t q = 0; q < cnt; q++) cc.push_back(&prover.trees[t].coeffs[first[k][t] + q]);
                    auto ev = B200Backend::evaluate_polynomials(dev, cc, 1);
                    for (auto& e : ev) { col_ptrs.push_back(e.ptr()); extended.push_back(std::move(e)); }
                }
            }
            if (c.claimed_sum) {
                qm31 claimed;
                for (int q = 0; q < 4; q++) claimed.c[q] = c.claimed_sum[q];
                shifts[k] = claimed * qm31_inv(qm31_from_m31(1u << c.trace_log));  // LogupAtRow::new, logup.rs:33-41
            }
            uint32_t denom_inv[2];
            if (zkb_constraint_denom_inv((int)c.trace_log, (int)eval_log, denom_inv) != ZKB_OK) return ZKB_EINVAL;
            auto it = sub.find(eval_log);
            const bool fresh = it == sub.end();
            if (fresh) it = sub.emplace(eval_log, SecureColumnByCoords(dev, (size_t)1 << eval_log)).first;
            auto accp = it->second.ptrs();
            dev.check(zkb_constraint_quotients(ctx, c.prog, col_ptrs.data(), c.scalars, shifts[k].c, reinterpret_cast<const uint32_t*>(powers.data()),
                                               denom_inv, (int)c.trace_log, (int)eval_log, accp.data(), fresh ? 0 : 1));
        }
        // DomainEvaluationAccumulator::finalize (air/accumulation.rs:89-124): lift and add ascending sizes, interpolate;
        // then split_at_mid and extend_polys + commit
        std::vector<SecureColumnByCoords> ascending;
        for (auto& kv : sub) ascending.push_back(std::move(kv.second));
        sub.clear();
        SecureColumnByCoords acc = B200Backend::lift_and_accumulate(dev, std::move(ascending));
        const uint32_t comp_log = max_trace_log + 1;
        const size_t N = (size_t)1 << comp_log;
        if (acc.len() != N) return zk_set_error_public(ctx, ZKB_EINVAL, "zkb_stark_prove: no component of the largest size");
        {
            std::vector<BaseColumn*> ap = {&acc.columns[0], &acc.columns[1], &acc.columns[2], &acc.columns[3]};
            B200Backend::interpolate_columns(dev, ap);
            std::vector<BaseColumn> halves;
            for (int q = 0; q < 4; q++) halves.push_back(BaseColumn::view(dev, acc.columns[q].ptr(), N / 2));
            for (int q = 0; q < 4; q++) halves.push_back(BaseColumn::view(dev, acc.columns[q].ptr() + N / 2, N / 2));
            dev.check(zkb_event_record(ctx, 29));
            prover.mark(-1);  // the composition is timed on its own, not as part of the next tree's first phase
            prover.commit_evals(std::move(halves), ch, nullptr, nullptr, true);
        }

        // ---- mask points (component.rs:356-368, core/air/components.rs:32-74) and the samples' proof
        CirclePointQ oods = get_random_point(ch);
        const uint32_t lifting_log = prover.trees.back().max_log();
        const uint32_t max_log_degree_bound = lifting_log - blowup;
        // per component: the mask offsets of each of its columns, in the order the program asks for them
        std::vector<std::vector<std::vector<int32_t>>> offsets((size_t)n_components);
        std::vector<std::vector<std::vector<CirclePointQ>>> points((size_t)n_trees + 1);
        for (int t = 0; t < n_trees; t++) points[t].resize((size_t)tree_ncols[t]);
        for (int k = 0; k < n_components; k++) {
            const zkb_air_program* prog = comps[k].prog;
            offsets[k].resize(prog->n_cols);
            for (const zkb_air_op& o : prog->ops)
                if (o.op == ZKB_AIR_LOAD) {
                    auto& v = offsets[k][prog->tree_base[o.a] + o.b];
                    if (std::find(v.begin(), v.end(), (int32_t)o.c) == v.end()) v.push_back((int32_t)o.c);
                }
            for (int t = 0; t < n_trees; t++)
                for (uint32_t q = 0; q < cols_of(k, t); q++)
                    for (int32_t off : offsets[k][prog->tree_base[t] + q]) {
                        // trace_step.mul_signed(off): the point of index off * 2^(31 - max_log_degree_bound) in the circle group
                        cpoint st = host_circle_point(((uint32_t)off << (31 - max_log_degree_bound)) & 0x7fffffffu);
                        points[t][first[k][t] + q].push_back(point_add(oods, {qm31_from_m31(st.x), qm31_from_m31(st.y)}));
                    }
        }
        points.back().assign(8, {oods});
        PcsProof proof = prover.prove_values(points, ch);
        prover.finish_timing();
        if (composition_ms) dev.check(zkb_event_elapsed_ms(ctx, 28, 29, composition_ms));

        // ---- the sanity check of prove_ex
        auto from_partial_evals = [](qm31 e0, qm31 e1, qm31 e2, qm31 e3) {  // qm31.rs:51-57
            const qm31 i{{0, 1, 0, 0}}, u{{0, 0, 1, 0}}, iu{{0, 0, 0, 1}};
            return e0 + e1 * i + e2 * u + e3 * iu;
        };
        const auto& comp = proof.sampled_values.back();
        const qm31 left = from_partial_evals(comp[0][0], comp[1][0], comp[2][0], comp[3][0]);
        const qm31 right = from_partial_evals(comp[4][0], comp[5][0], comp[6][0], comp[7][0]);
        const qm31 committed = left + point_repeated_double(oods, max_log_degree_bound - 1).x * right;
        // coset_vanishing(CanonicCoset(max_log_degree_bound).coset, oods): the shift -initial + step/2 is zero for a canonic coset
        qm31 vanish = oods.x;
        for (uint32_t q = 1; q < max_log_degree_bound; q++) vanish = qm31_double_x(vanish);
        const qm31 denom_inverse = qm31_inv(vanish);
        qm31 at_point = qm31_zero();  // one PointEvaluationAccumulator (core/air/accumulation.rs:12-36) through all components
        for (int k = 0; k < n_components; k++) {
            const zkb_air_program* prog = comps[k].prog;
            // the program at the point: every value is a secure-field element, a LOAD is the sampled mask value
            std::vector<qm31> v(prog->ops.size(), qm31_zero());
            std::vector<std::pair<int, uint32_t>> where(prog->n_cols);
            for (int t = 0; t < n_trees; t++)
                for (uint32_t q = 0; q < cols_of(k, t); q++) where[prog->tree_base[t] + q] = {t, first[k][t] + q};
            for (size_t i = 0; i < prog->ops.size(); i++) {
                const zkb_air_op& o = prog->ops[i];
                switch (o.op) {
                    case ZKB_AIR_LOAD: {
                        const uint32_t col = prog->tree_base[o.a] + o.b;
                        const auto& offs = offsets[k][col];
                        const size_t j = std::find(offs.begin(), offs.end(), (int32_t)o.c) - offs.begin();
                        v[i] = proof.sampled_values[where[col].first][where[col].second][j];
                        break;
                    }
                    case ZKB_AIR_CONST_M31: v[i] = qm31_from_m31(o.a); break;
                    case ZKB_AIR_SCALAR: for (int q = 0; q < 4; q++) v[i].c[q] = comps[k].scalars[4 * (size_t)o.a + q]; break;
                    case ZKB_AIR_CUMSUM_SHIFT: v[i] = shifts[k]; break;
                    case ZKB_AIR_ADD_B: case ZKB_AIR_ADD_E: v[i] = v[o.a] + v[o.b]; break;
                    case ZKB_AIR_SUB_B: case ZKB_AIR_SUB_E: v[i] = v[o.a] - v[o.b]; break;
                    case ZKB_AIR_MUL_B: case ZKB_AIR_MUL_E: v[i] = v[o.a] * v[o.b]; break;
                    case ZKB_AIR_NEG_B: case ZKB_AIR_NEG_E: v[i] = qm31_neg(v[o.a]); break;
                    case ZKB_AIR_INV_B: v[i] = qm31_is_zero(v[o.a]) ? qm31_zero() : qm31_inv(v[o.a]); break;
                    case ZKB_AIR_PACK: v[i] = from_partial_evals(v[o.a], v[o.b], v[o.c], v[o.d]); break;
                    default: break;
                }
            }
            for (uint32_t cn : prog->constraints) at_point = at_point * random_coeff + denom_inverse * v[cn];
        }
        for (int q = 0; q < 4; q++) { oods_evals[q] = committed.c[q]; oods_evals[4 + q] = at_point.c[q]; }

        std::vector<uint32_t> w = proof.to_words();
        w.insert(w.end(), ch.digest().begin(), ch.digest().end());
        *n_words = w.size();
        if (w.size() > cap) return zk_set_error_public(ctx, ZKB_EINVAL, "zkb_stark_prove: output buffer too small");
        memcpy(h_out, w.data(), w.size() * 4);
        return ZKB_OK;
    } catch (const Error& e) {
        return zk_set_error_public(ctx, e.code, e.what());
    } catch (const std::exception& e) {
        return zk_set_error_public(ctx, ZKB_ENOMEM, e.what());
    }
}

extern "C" {

int zkb_pcs_prove_device(zkb_ctx* ctx, int n_trees, const int* tree_ncols, uint32_t* const* d_cols, const uint32_t* col_logs,
                         const zkb_pcs_config* config, int two_sample_every, uint32_t* h_out, size_t cap, size_t* n_words,
                         float* h_phase_ms) {
    return pcs_prove_impl(ctx, n_trees, tree_ncols, d_cols, nullptr, col_logs, config, two_sample_every, h_out, cap, n_words, h_phase_ms);
}

int zkb_stark_prove_multi_device(zkb_ctx* ctx, int n_trees, const int* tree_ncols, uint32_t* const* d_cols, int n_components,
                                 const zkb_stark_component* components, const zkb_pcs_config* config, uint32_t* h_out, size_t cap,
                                 size_t* n_words, uint32_t* oods_evals, float* h_phase_ms, float* composition_ms) {
    return stark_prove_impl(ctx, n_trees, tree_ncols, d_cols, nullptr, n_components, components, config, h_out, cap, n_words, oods_evals,
                            h_phase_ms, composition_ms);
}

int zkb_stark_prove_multi_host(zkb_ctx* ctx, int n_trees, const int* tree_ncols, const uint32_t* const* h_cols, int n_components,
                               const zkb_stark_component* components, const zkb_pcs_config* config, uint32_t* h_out, size_t cap,
                               size_t* n_words, uint32_t* oods_evals, float* h_phase_ms, float* composition_ms) {
    return stark_prove_impl(ctx, n_trees, tree_ncols, nullptr, h_cols, n_components, components, config, h_out, cap, n_words, oods_evals,
                            h_phase_ms, composition_ms);
}

int zkb_stark_prove_device(zkb_ctx* ctx, int n_trees, const int* tree_ncols, uint32_t* const* d_cols, uint32_t trace_log,
                           zkb_air_program* prog, const uint32_t* scalars, const uint32_t* claimed_sum, const zkb_pcs_config* config,
                           uint32_t* h_out, size_t cap, size_t* n_words, uint32_t* oods_evals, float* h_phase_ms, float* composition_ms) {
    zkb_stark_component c{prog, trace_log, scalars, claimed_sum};
    return stark_prove_impl(ctx, n_trees, tree_ncols, d_cols, nullptr, 1, &c, config, h_out, cap, n_words, oods_evals, h_phase_ms, composition_ms);
}

int zkb_stark_prove_host(zkb_ctx* ctx, int n_trees, const int* tree_ncols, const uint32_t* const* h_cols, uint32_t trace_log,
                         zkb_air_program* prog, const uint32_t* scalars, const uint32_t* claimed_sum, const zkb_pcs_config* config,
                         uint32_t* h_out, size_t cap, size_t* n_words, uint32_t* oods_evals, float* h_phase_ms, float* composition_ms) {
    zkb_stark_component c{prog, trace_log, scalars, claimed_sum};
    return stark_prove_impl(ctx, n_trees, tree_ncols, nullptr, h_cols, 1, &c, config, h_out, cap, n_words, oods_evals, h_phase_ms, composition_ms);
}

int zkb_pcs_prove_host(zkb_ctx* ctx, int n_trees, const int* tree_ncols, const uint32_t* const* h_cols, const uint32_t* col_logs,
                       const zkb_pcs_config* config, int two_sample_every, uint32_t* h_out, size_t cap, size_t* n_words,
                       float* h_phase_ms) {
    return pcs_prove_impl(ctx, n_trees, tree_ncols, nullptr, h_cols, col_logs, config, two_sample_every, h_out, cap, n_words, h_phase_ms);
}

int zkb_gkr_prove_device(zkb_ctx* ctx, int n_inst, const int* kinds, const uint32_t* const* d_nums, const uint32_t* const* d_dens,
                         const uint64_t* ns, uint64_t seed, uint32_t* h_out, size_t cap, size_t* n_words) {
    if (!ctx) return ZKB_EINVAL;
    if (n_inst <= 0 || !kinds || !d_nums || !d_dens || !ns || !h_out || !n_words) return ZKB_EINVAL;
    try {
        Device dev(ctx);
        std::vector<Layer> layers;
        for (int i = 0; i < n_inst; i++) {
            if (kinds[i] < 0 || kinds[i] > 3 || ns[i] < 1 || (ns[i] & (ns[i] - 1))) return ZKB_EINVAL;
            layers.push_back(layer_view(dev, kinds[i], d_nums[i], d_dens[i], ns[i]));
        }
        Channel ch;
        ch.mix_u64(seed);
        std::vector<uint32_t> w;
        // Two drivers give the same proof. With the transcript on the device a round costs no host round trip but runs its
        // Fiat-Shamir step on one warp, which pays for ONE large instance; a batch of several instances is cheaper with one
        // launch and one read-back per round for all of them. ZKB_GKR_DRIVER=resident|batch overrides the choice.
        bool resident = gkr_resident_supported(n_inst, ns) && n_inst <= 2;
        if (const char* pick = getenv("ZKB_GKR_DRIVER")) {
            if (!strcmp(pick, "resident")) resident = gkr_resident_supported(n_inst, ns);
            else if (!strcmp(pick, "batch")) resident = false;
        }
        if (resident) {
            // the transcript stays on the device: no host round trip per sum-check round
            uint32_t dg[8], nd = ch.n_draws();
            for (int k = 0; k < 8; k++) dg[k] = ch.digest()[k];
            int rc = gkr_prove_resident(ctx, std::move(layers), dg, &nd, w);
            if (rc) return rc;
            HashWords hw;
            for (int k = 0; k < 8; k++) hw[k] = dg[k];
            ch.set_state(hw, nd);
        } else {
            w = gkr_prove_batch(dev, ch, std::move(layers));
        }
        w.insert(w.end(), ch.digest().begin(), ch.digest().end());
        *n_words = w.size();
        if (w.size() > cap) return zk_set_error_public(ctx, ZKB_EINVAL, "zkb_gkr_prove: output buffer too small");
        memcpy(h_out, w.data(), w.size() * 4);
        HostClock::dump("zkb_gkr_prove_device");
        return ZKB_OK;
    } catch (const Error& e) {
        return zk_set_error_public(ctx, e.code, e.what());
    } catch (const std::exception& e) {
        return zk_set_error_public(ctx, ZKB_ENOMEM, e.what());
    }
}

}  // extern "C"
