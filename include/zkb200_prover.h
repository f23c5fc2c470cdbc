/*
 * zkb200_prover — whole-protocol drivers over the operator ABI of zkb200.h.
 *
 * The reference's protocol code is generic Rust that calls the backend's operators
 * (STWO = nitroo/crates/stwo/src): CommitmentSchemeProver (STWO/prover/pcs/mod.rs:34-419),
 * CommitmentTreeProver (:466-630), compute_fri_quotients (STWO/prover/pcs/quotient_ops.rs:73-194),
 * FriProver (STWO/prover/fri.rs:87-467), MerkleProver (STWO/prover/vcs/prover.rs:17-217) and the GKR
 * batch prover (STWO/prover/lookups/gkr_prover.rs:657-882, sumcheck.rs:96-176). A Rust build keeps
 * using that code with the new backend type. These entry points are its C++ counterpart for
 * programs without a Rust toolchain: the benchmark and the parity tests drive whole commitments
 * and proofs through them. The Fiat-Shamir channel is Blake2sM31Channel, run on the host.
 *
 * Proof word streams (uint32, all field elements canonical):
 *   PCS: n_trees, roots (8 words each); per tree: n_cols, per column n_samples and the sampled
 *        values; per tree the Merkle decommitment (n_hashes, hashes, n_values, values); per tree
 *        n_queried, queried values; proof-of-work nonce (lo, hi); FRI first layer, n_inner, inner
 *        layers (each: n_witness, witness values, decommitment, commitment); n_coeffs, last-layer
 *        polynomial; then the 8 words of the channel digest after the proof.
 *   GKR: n_layers, per layer n_rounds and each round polynomial (n_coeffs, coeffs); per instance
 *        n_masks and each mask (n_columns, two values per column); per instance the output claims;
 *        the out-of-domain point; per instance the claims to verify; the final channel digest.
 */
#ifndef ZKB200_PROVER_H
#define ZKB200_PROVER_H

#include "zkb200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct zkb_pcs_config {
    uint32_t pow_bits;
    uint32_t log_blowup_factor;
    uint32_t log_last_layer_degree_bound;
    uint32_t n_queries;
} zkb_pcs_config;

#define ZKB_PCS_N_PHASES 8
/* phase times in h_phase_ms: 0 interpolate, 1 extend (LDE), 2 Merkle commit, 3 out-of-domain
 * sampling, 4 quotients, 5 FRI commit, 6 grind, 7 decommit. */

/* Commits n_trees trees of trace columns and proves one opening per column at a channel-drawn point
 * (columns whose flat index is a multiple of two_sample_every, when that is non-zero, are also opened
 * one trace step before it). d_cols: device columns of 2^col_logs[i] evaluations on the canonic
 * domain, bit-reversed; they are consumed (interpolated in place). The context's max_log_size must
 * cover the largest column plus the blow-up. h_phase_ms may be NULL. */
int zkb_pcs_prove_device(zkb_ctx* ctx, int n_trees, const int* tree_ncols, uint32_t* const* d_cols, const uint32_t* col_logs,
                         const zkb_pcs_config* config, int two_sample_every, uint32_t* h_out, size_t cap, size_t* n_words,
                         float* h_phase_ms);
/* Same with host columns (each is copied to the device first; h_cols are left untouched). The copies
 * run on a second stream under the interpolation, extension and leaf hashing of what has already
 * arrived; that overlap only happens when the host columns are page-locked (zkb_host_alloc_pinned,
 * or memory registered with cudaHostRegister). Pageable columns are accepted and give the same
 * proof, but the driver stages them and the copy no longer overlaps compute. */
int zkb_pcs_prove_host(zkb_ctx* ctx, int n_trees, const int* tree_ncols, const uint32_t* const* h_cols, const uint32_t* col_logs,
                       const zkb_pcs_config* config, int two_sample_every, uint32_t* h_out, size_t cap, size_t* n_words,
                       float* h_phase_ms);

/* A whole STARK proof of one component: prove() of nitroo/crates/stwo/src/prover/mod.rs:41-173 with the component's
 * constraints given as a compiled AIR program (zkb200_air.h). The trees are the fork's: preprocessed, model, base
 * trace, interaction (a tree may have no columns); every column has 2^trace_log evaluations on the canonic domain,
 * bit-reversed, and d_cols are consumed. The flow: commit the trees; draw the random coefficient; constraint quotients
 * on the domain of size 2^(trace_log+1) (zkb_constraint_quotients; the committed evaluations are used as they are when
 * the blow-up is 2); interpolate, split in halves, commit the composition tree (8 columns); draw the out-of-domain
 * point; sample every column at its mask points (point + offset * trace step, constraint-framework/src/component.rs:
 * 356-368) and the composition halves at the point; prove the samples. Output: the proof words as zkb_pcs_prove gives
 * them (5 trees) followed by the channel digest. oods_evals[0..4) is the composition polynomial at the point from the
 * committed halves, oods_evals[4..8) the same value from the constraints at the sampled mask values: the reference's
 * prover refuses (ProvingError::ConstraintsNotSatisfied) when they differ, here the caller compares them.
 * claimed_sum (4 words or NULL) is the LogUp claimed sum of the component; scalars the program's run-time scalars.
 * composition_ms (may be NULL) receives the device time from the draw of the random coefficient to the interpolated
 * composition polynomial. The context's max_log_size must cover trace_log + log_blowup_factor (at least 1). */
typedef struct zkb_air_program zkb_air_program;
int zkb_stark_prove_device(zkb_ctx* ctx, int n_trees, const int* tree_ncols, uint32_t* const* d_cols, uint32_t trace_log,
                           zkb_air_program* prog, const uint32_t* scalars, const uint32_t* claimed_sum, const zkb_pcs_config* config,
                           uint32_t* h_out, size_t cap, size_t* n_words, uint32_t* oods_evals, float* h_phase_ms, float* composition_ms);
int zkb_stark_prove_host(zkb_ctx* ctx, int n_trees, const int* tree_ncols, const uint32_t* const* h_cols, uint32_t trace_log,
                         zkb_air_program* prog, const uint32_t* scalars, const uint32_t* claimed_sum, const zkb_pcs_config* config,
                         uint32_t* h_out, size_t cap, size_t* n_words, uint32_t* oods_evals, float* h_phase_ms, float* composition_ms);

/* The same for a statement of several components of different sizes (ComponentProvers, prover/air/component_prover.rs:
 * 161-176): in every tree the columns of component k follow those of components 0..k-1 and have 2^trace_log_k rows.
 * Each component's constraint quotients go to the accumulation of its own evaluation-domain size with its share of the
 * random-coefficient powers (DomainEvaluationAccumulator::columns hands them out from the end); the accumulations are
 * lifted and added in ascending size; every mask point is point + offset * step of the largest trace; one
 * PointEvaluationAccumulator runs through all components for the out-of-domain check. At least one component must have
 * the largest size on which the composition polynomial lives. */
typedef struct zkb_stark_component {
    zkb_air_program* prog;
    uint32_t trace_log;
    const uint32_t* scalars;     /* the program's run-time scalars (may be NULL if it has none) */
    const uint32_t* claimed_sum; /* 4 words or NULL */
} zkb_stark_component;
int zkb_stark_prove_multi_device(zkb_ctx* ctx, int n_trees, const int* tree_ncols, uint32_t* const* d_cols, int n_components,
                                 const zkb_stark_component* components, const zkb_pcs_config* config, uint32_t* h_out, size_t cap,
                                 size_t* n_words, uint32_t* oods_evals, float* h_phase_ms, float* composition_ms);
int zkb_stark_prove_multi_host(zkb_ctx* ctx, int n_trees, const int* tree_ncols, const uint32_t* const* h_cols, int n_components,
                               const zkb_stark_component* components, const zkb_pcs_config* config, uint32_t* h_out, size_t cap,
                               size_t* n_words, uint32_t* oods_evals, float* h_phase_ms, float* composition_ms);

/* GKR batch proof of n_inst instances. kinds: ZKB_GKR_*; d_nums[i] (NULL where the kind has no
 * numerators) and d_dens[i] are device arrays of ns[i] entries laid out as zkb_gkr_next_layer takes
 * them; they are not modified. The channel starts from Blake2sM31Channel::default() after
 * mix_u64(seed). One or two instances are proved with the Fiat-Shamir transcript resident on the device (no host
 * round trip per sum-check round); larger batches (up to 8,192 instances) with one launch and one read-back per
 * round for all instances. Both give the same words; the environment variable ZKB_GKR_DRIVER=resident|batch
 * forces one of them (resident: at most 16 instances). */
int zkb_gkr_prove_device(zkb_ctx* ctx, int n_inst, const int* kinds, const uint32_t* const* d_nums, const uint32_t* const* d_dens,
                         const uint64_t* ns, uint64_t seed, uint32_t* h_out, size_t cap, size_t* n_words);

/* ---- One PCS proof over G devices (no counterpart in the reference, which has no multi-device code) ----------
 * The proof zkb_pcs_prove_device gives for ONE tree of ncols_total columns of 2^log_n rows with one out-of-domain
 * sample per column, word for word, computed by `world` ranks (a power of two that divides ncols_total), one
 * context per rank. The library moves nothing between devices: between the calls below the caller performs the
 * exchanges (NCCL, MPI, peer copies ...), in this order:
 *   begin    every rank, same arguments except `rank`
 *   extend   d_cols: this rank's ncl = ncols_total / world columns (evaluations, bit-reversed; consumed). Returns
 *            *d_send = [world][ncl][R] (R = N / world): block d holds rows [d R, (d+1) R) of the extended local columns (the
 *            transform's last pass writes them there directly), and *d_rows = [world][ncl][R] to receive into.
 *            EXCHANGE: one all-to-all: block d of d_send goes to rank d, which stores it as block `rank` of its d_rows
 *   subtree  hashes the Merkle subtree over the rank's rows. *d_root: its root (8 words, device);
 *            EXCHANGE: all-gather the roots into *d_roots ([world][8], device), rank order
 *   sample   top layers of the tree, channel, out-of-domain point; h_samples receives this rank's ncl x 4 words
 *            EXCHANGE: all-gather the samples (host), rank order = global column order
 *   quotients  mixes all samples, draws the coefficient, computes the quotients of the rank's rows:
 *            d_quot_local[k] (R words) is coordinate k;
 *            EXCHANGE: all-gather coordinate k into d_quot_full[k] (N words), for k = 0..3
 *   fri_and_decommit  every rank runs the same FRI commitment, grind and query draw on the gathered column (it is
 *            4 / ncols of the evaluations: sharding it would cost a collective per layer for less than 2 ms of work),
 *            then serialises the decommitment of the queried rows it owns into h_part
 *            EXCHANGE: gather the parts (host) on the rank that calls finish
 *   finish   merges the parts into the proof words (plus the 8 words of the channel digest, as zkb_pcs_prove_device)
 *   end      frees the session
 * Errors: ZKB_EINVAL for shapes that do not shard (world not a power of two, fewer than 8 rows per rank). */
typedef struct zkb_shard_pcs zkb_shard_pcs;
int zkb_shard_pcs_begin(zkb_ctx* ctx, int rank, int world, int ncols_total, int log_n, const zkb_pcs_config* config, zkb_shard_pcs** out);
int zkb_shard_pcs_extend(zkb_shard_pcs* s, uint32_t* const* d_cols, uint32_t** d_send, uint32_t** d_rows);
/* The same stage by chunks of columns, so that a chunk's exchange runs while the next chunk is extended: begin interpolates all
 * local columns and fixes the chunk count (it must divide ncl); chunk k extends columns [k ncl / n_chunks, (k + 1) ncl / n_chunks)
 * and returns that chunk's send block ([world][ncl / n_chunks][R]), where to receive it ([world][ncl / n_chunks][R]: block s
 * from rank s) and the words per peer. Every launch is stream-ordered: the caller starts chunk k's all-to-all after what has
 * been enqueued so far and only has to order the subtree stage after the last one. zkb_shard_pcs_extend is begin with one
 * chunk followed by chunk 0. */
/* Optional, before extend_begin: the buffer the row shards are received into (ncols_total x N / world words), e.g. one from
 * zkb_peer_buffer_alloc that the other ranks copy into directly; NULL (the default) lets the session allocate it. The
 * caller keeps the buffer alive until zkb_shard_pcs_end. */
int zkb_shard_pcs_set_rows(zkb_shard_pcs* s, uint32_t* d_rows);
/* Optional, instead of set_rows: every rank's receive buffer as THIS process sees it (peer_rows[r] for rank r, opened with
 * zkb_peer_buffer_open; peer_rows[rank] is this rank's own). Every chunk's blocks are then copied into the peers' buffers by
 * the library right after the chunk's transform is enqueued (zkb_copy_to_peer), and the caller's part of the exchange is
 * zkb_peer_copies_wait followed by a barrier between the ranks. NULL returns to a caller-side exchange. */
int zkb_shard_pcs_set_peer_rows(zkb_shard_pcs* s, uint32_t* const* peer_rows);
int zkb_shard_pcs_extend_begin(zkb_shard_pcs* s, uint32_t* const* d_cols, int n_chunks);
int zkb_shard_pcs_extend_chunk(zkb_shard_pcs* s, int k, uint32_t** d_send, uint32_t** d_recv, size_t* words_per_peer);
int zkb_shard_pcs_subtree(zkb_shard_pcs* s, uint32_t** d_root, uint32_t** d_roots);
int zkb_shard_pcs_sample(zkb_shard_pcs* s, uint32_t* h_samples);
int zkb_shard_pcs_quotients(zkb_shard_pcs* s, const uint32_t* h_all_samples, uint32_t* d_quot_local[4], uint32_t* d_quot_full[4]);
int zkb_shard_pcs_fri_and_decommit(zkb_shard_pcs* s, uint32_t* h_part, size_t cap, size_t* n_words);
int zkb_shard_pcs_finish(zkb_shard_pcs* s, const uint32_t* const* h_parts, const size_t* part_words, uint32_t* h_out, size_t cap,
                         size_t* n_words);
int zkb_shard_pcs_end(zkb_shard_pcs* s);

#ifdef __cplusplus
}
#endif
#endif /* ZKB200_PROVER_H */
