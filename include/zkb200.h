/*
 * zkb200 — C ABI of the B200 (sm_100a) proving backend for the Circle-STARK operator traits.
 *
 * One entry point per backend operator of the reference's vendored STARK library. Each comment
 * names the reference interface the function stands in for, by path inside the reference project
 * (STWO = nitroo/crates/stwo/src). A Rust `Backend` type binds these with `extern "C"`.
 *
 * Conventions
 *  - Every function returns a status: ZKB_OK (0) or a negative ZKB_E* code. Nothing aborts or
 *    exits the process. zkb_last_error() gives the message of the last failure on a context.
 *  - M31 values are uint32_t in [0, 2^31 - 1). A "secure column" is four device arrays, one per
 *    QM31 coordinate (STWO/prover/secure_column.rs:13-15). GKR multilinear columns are device
 *    arrays of QM31 stored as 4 consecutive uint32_t (as the reference's SecureFieldVec).
 *    A hash column is 8 uint32_t (32 little-endian bytes) per node.
 *  - Pointers are DEVICE pointers unless the parameter name starts with h_. Arrays of column
 *    pointers (`cols`, `coeffs`, `out` of the batched calls, the `[4]` coordinate arrays) are host
 *    arrays whose entries are device pointers.
 *  - Work is enqueued on the context's stream and the call returns; calls that write to h_
 *    outputs synchronise that stream before returning.
 *  - Buffers are owned by whoever allocated them. The library frees only what zkb_malloc gave out
 *    and only in zkb_free / zkb_destroy.
 *  - A context serves one host thread at a time (its stream, scratch and staging ring are not
 *    locked). Several contexts, on one device or on several, may be used from different threads
 *    concurrently; the traits' per-column default methods that the reference runs on rayon workers
 *    (STWO/prover/poly/circle/ops.rs:28-39, 98-120) are replaced by the batched calls below.
 */
#ifndef ZKB200_H
#define ZKB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ZKB_OK 0
#define ZKB_EINVAL (-1)   /* bad argument (null pointer, size out of range, ...) */
#define ZKB_ENOMEM (-2)   /* device or host allocation failed */
#define ZKB_ECUDA (-3)    /* a CUDA call failed; see zkb_last_error */
#define ZKB_ETIMEOUT (-4) /* a bounded device-side wait ran out */
#define ZKB_ENCCL (-5)    /* a collective failed */

typedef struct zkb_ctx zkb_ctx;

/* ---- context ------------------------------------------------------------------------------
 * The reference keeps CUDA state process-global (STWO/stwo_cuda/mod.rs:25-43); here it is an
 * explicit handle. `max_log_size` is the largest circle-domain log size any later call will use
 * (the twiddle tower is built once, for Coset::half_odds(max_log_size - 1), replacing
 * PolyOps::precompute_twiddles, STWO/prover/poly/circle/ops.rs:123 and
 * STWO/prover/backend/cpu/circle.rs:230-291). */
int zkb_init(int device, int max_log_size, zkb_ctx** out);
int zkb_destroy(zkb_ctx* ctx);
const char* zkb_last_error(zkb_ctx* ctx);
int zkb_sync(zkb_ctx* ctx);
/* The CUDA stream (cudaStream_t) all work of this context is ordered on. */
int zkb_get_stream(zkb_ctx* ctx, void** stream);
int zkb_max_log_size(zkb_ctx* ctx);

/* Timing helpers for benchmarks (no counterpart in the reference, which times with host clocks
 * around synchronised calls, STWO/prover/lookups/gkr_prover.rs:81-150): CUDA events recorded on
 * the context's stream. `slot` < 64. zkb_event_elapsed_ms synchronises on event `b`. */
int zkb_event_record(zkb_ctx* ctx, int slot);
int zkb_event_elapsed_ms(zkb_ctx* ctx, int a, int b, float* h_ms);

/* Per-kernel timeline: between zkb_profile_begin and zkb_profile_end the large kernels (FFT passes,
 * Merkle layers, quotient kernels, FRI folds) are bracketed by CUDA events. zkb_profile_end
 * synchronises and writes up to `cap` aggregated records: h_names[i] (a static string), h_ms[i]
 * (total milliseconds) and h_count[i] (launches); *n receives the number of distinct kernels. */
int zkb_profile_begin(zkb_ctx* ctx);
int zkb_profile_end(zkb_ctx* ctx, const char** h_names, float* h_ms, int* h_count, int cap, int* n);

/* The arithmetic ceiling of the circle-FFT butterfly on this device (no counterpart in the reference): runs the
 * radix-32 butterfly stages the FFT passes use on registers only, with no global traffic, at the passes' own
 * occupancy, and returns butterflies per second. An FFT pass cannot run faster than its butterfly count divided
 * by this figure; the benchmark reports the passes against it beside the HBM figure. Takes about a millisecond. */
int zkb_fft_arith_ceiling(zkb_ctx* ctx, double* h_butterflies_per_s);

/* ---- device columns (STWO/stwo_cuda/base_field_vec.rs:7-60, bindings.rs:84-103) ------------ */
int zkb_malloc(zkb_ctx* ctx, size_t bytes, void** dptr);
int zkb_free(zkb_ctx* ctx, void* dptr);
int zkb_memset_zero(zkb_ctx* ctx, void* dptr, size_t bytes);
int zkb_h2d(zkb_ctx* ctx, void* dptr, const void* h_src, size_t bytes); /* returns after the copy */
int zkb_d2h(zkb_ctx* ctx, void* h_dst, const void* dptr, size_t bytes); /* returns after the copy */
int zkb_h2d_async(zkb_ctx* ctx, void* dptr, const void* h_pinned_src, size_t bytes);
int zkb_d2h_async(zkb_ctx* ctx, void* h_pinned_dst, const void* dptr, size_t bytes);
/* Host-to-device copy on the context's second (copy) stream, so that it overlaps kernels on the compute stream.
 * The copy starts after everything enqueued on the compute stream so far (the destination may just have been
 * allocated there). fence >= 0 records fence slot `fence` (0..63) after the copy; zkb_wait_fence makes the compute
 * stream wait for that slot. Neither call blocks the host. fence = -1 records nothing. */
int zkb_h2d_overlapped(zkb_ctx* ctx, void* dptr, const void* h_pinned_src, size_t bytes, int fence);
int zkb_wait_fence(zkb_ctx* ctx, int fence);
/* Buffers that another process's GPU on the same host can copy into (one process per GPU): alloc returns device
 * memory of this context's GPU (plain cudaMalloc: pool memory can not be shared) and a 64-byte handle to send to the
 * peers; a peer opens the handle (peer access is enabled on first use) and gets an address valid in ITS process.
 * zkb_copy_to_peer copies `bytes` from this GPU's `src` to `dst` (a peer address, or a local one) with the copy engines,
 * after everything enqueued on the compute stream so far, on one of four copy streams (`lane` mod 4: copies on different
 * lanes run side by side); it does not block the host and uses no SM, so it runs under kernels. zkb_peer_copies_wait blocks the host until this context's copies have landed; the
 * RECEIVER learns that its data is there from the caller (a barrier between the processes after every sender has waited).
 * close before the owner frees; free synchronises the compute stream. ZKB_ECUDA when the GPUs can not reach each other. */
int zkb_peer_buffer_alloc(zkb_ctx* ctx, size_t bytes, void** dptr, unsigned char handle[64]);
int zkb_peer_buffer_free(zkb_ctx* ctx, void* dptr);
int zkb_peer_buffer_open(zkb_ctx* ctx, const unsigned char handle[64], void** peer_ptr);
int zkb_peer_buffer_close(zkb_ctx* ctx, void* peer_ptr);
int zkb_copy_to_peer(zkb_ctx* ctx, void* dst, const void* src, size_t bytes, int lane);
int zkb_peer_copies_wait(zkb_ctx* ctx);
int zkb_d2d(zkb_ctx* ctx, void* dst, const void* src, size_t bytes);
int zkb_host_alloc_pinned(zkb_ctx* ctx, size_t bytes, void** h_ptr);
int zkb_host_free_pinned(zkb_ctx* ctx, void* h_ptr);
/* Column::batch_at_multi (STWO/prover/backend/mod.rs:70-89; bindings.rs:340-346):
 * h_out[i * ncols + c] = cols[c][h_idx[i]]. */
int zkb_gather_multi(zkb_ctx* ctx, const uint32_t* const* cols, int ncols, const uint32_t* h_idx, int nidx,
                     uint32_t* h_out);

/* Column<Blake2sHash>::batch_at (STWO/prover/backend/mod.rs:68-72): h_out[8*i..] = hashes[h_idx[i]]. */
int zkb_gather_hashes(zkb_ctx* ctx, const uint32_t* hashes, const uint32_t* h_idx, int nidx, uint32_t* h_out);

/* One round trip for many small reads: h_out[i] = *h_addrs[i], each a device address of a word.
 * It serves the decommitment phase, where the reference issues one batch_at / batch_at_multi per tree
 * layer (STWO/prover/vcs/prover.rs:160-207): the positions of ALL layers are known before any value is
 * read, so a caller can collect every address first and read them together. */
int zkb_gather_words(zkb_ctx* ctx, const uint32_t* const* h_addrs, size_t n, uint32_t* h_out);

/* ---- twiddles ------------------------------------------------------------------------------
 * Copies out the tower of Coset::half_odds(log_size) in the reference's layout
 * (slow_precompute_twiddles, STWO/prover/backend/cpu/circle.rs:274-291): 2^log_size words each,
 * last word 1. h_itw may be NULL. log_size <= max_log_size - 1. */
int zkb_twiddles_d2h(zkb_ctx* ctx, int log_size, uint32_t* h_tw, uint32_t* h_itw);

/* ---- PolyOps (STWO/prover/poly/circle/ops.rs:16-145) --------------------------------------- */
/* interpolate / interpolate_columns (ops.rs:23-39; cpu/circle.rs:28-80): evaluations on the
 * canonic circle domain of log_n, bit-reversed, to FFT-basis coefficients; in place. */
int zkb_ifft_cols(zkb_ctx* ctx, uint32_t* const* cols, int ncols, int log_n);
/* evaluate / evaluate_polynomials / extend (ops.rs:88-120; cpu/circle.rs:182-228): 2^log_n
 * coefficients to evaluations on the canonic domain of log_out >= log_n, bit-reversed.
 * out[c] must not alias coeffs[c]. */
int zkb_lde_cols(zkb_ctx* ctx, const uint32_t* const* coeffs, int ncols, int log_n, uint32_t* const* out,
                 int log_out);
/* eval_at_point / batch_eval_at_point (ops.rs:46-63; cpu/circle.rs:82-100): h_out[4*c..] is the
 * value of column c's polynomial at the QM31 circle point h_point = (x[4], y[4]). */
int zkb_eval_at_point_cols(zkb_ctx* ctx, const uint32_t* const* coeffs, int ncols, int log_n,
                           const uint32_t* h_point, uint32_t* h_out);
/* The PolyOps methods that evaluate from EVALUATIONS (STWO/prover/poly/circle/ops.rs:59-86; CPU statements
 * backend/cpu/circle.rs:101-180). Off the prover's path (it keeps coefficients), provided in simplest correct form.
 * barycentric_weights: 2^log_size weights (QM31, 4 consecutive words each, 16-byte aligned) for the canonic domain of
 * that size and the point h_point (x[4], y[4]); log_size >= 3. */
int zkb_barycentric_weights(zkb_ctx* ctx, int log_size, const uint32_t h_point[8], uint32_t* d_weights);
/* barycentric_eval_at_point: sum_i evals[i] * weights[i] (evals bit-reversed on the canonic domain). */
int zkb_barycentric_eval_at_point(zkb_ctx* ctx, const uint32_t* d_evals, const uint32_t* d_weights, int log_size, uint32_t h_out[4]);
/* eval_at_point_by_folding: one circle fold and log_size - 1 line folds with the point's folding factors
 * (core/poly/utils.rs:45-70), then division by 2^log_size; log_size >= 2. The evaluations are not modified. */
int zkb_eval_at_point_by_folding(zkb_ctx* ctx, const uint32_t* d_evals, int log_size, const uint32_t h_point[8], uint32_t h_out[4]);
/* FriOps::decompose (STWO/prover/fri.rs:82): not used by the prover and `todo!()` in the reference's own device
 * backend (backend/cuda/fri.rs:71-77). Always returns ZKB_EINVAL with a message saying so. */
int zkb_fri_decompose(zkb_ctx* ctx, const uint32_t* const d_eval[4], int log_size, uint32_t* const d_out[4], uint32_t h_lambda[4]);


/* ---- ColumnOps::bit_reverse_column (STWO/prover/backend/mod.rs:39-42; core/utils.rs:71-81) -- */
int zkb_bit_reverse_m31(zkb_ctx* ctx, uint32_t* col, int log_n);
int zkb_bit_reverse_qm31(zkb_ctx* ctx, uint32_t* col, int log_n); /* 4-word elements */

/* ---- MerkleOps::commit_on_layer (STWO/prover/vcs/ops.rs:24-29; cpu/blake2s.rs:13-26;
 * hasher core/vcs/blake2_merkle.rs:18-39). prev: 2^(log_size+1) hashes or NULL. cols: ncols
 * columns of 2^log_size values (ncols may be 0). m31_out != 0 selects the hasher whose digest
 * words are reduced mod 2^31-1. out: 2^log_size hashes. */
int zkb_merkle_layer(zkb_ctx* ctx, int log_size, const uint32_t* prev, const uint32_t* const* cols, int ncols,
                     int m31_out, uint32_t* out);

/* The leaf layer of a tree (no children) in several calls, a run of columns at a time, so that hashing overlaps
 * the production of later columns. Call with consecutive runs in column order: cols_before = columns absorbed by
 * earlier calls (a multiple of 16), total_cols = columns of the layer. Every call but the last must bring a
 * multiple of 16 columns (whole Blake2s blocks); the call with cols_before + ncols == total_cols finalises. `out`
 * (2^log_size x 8 words) carries the chaining values between calls and holds the hashes zkb_merkle_layer(log_size,
 * NULL, all columns) would produce after the last one. */
int zkb_merkle_leaves_partial(zkb_ctx* ctx, int log_size, const uint32_t* const* cols, int ncols, int cols_before, int total_cols,
                              int m31_out, uint32_t* out);
/* `levels` (1..9) consecutive layers of nodes without columns in one launch (MerkleProver::commit's loop,
 * STWO/prover/vcs/prover.rs:39-64, for the layers that hold no column): children = the 2^child_log hashes of a layer
 * (child_log >= 9), out_layers[j] = the layer j + 1 levels above it (2^(child_log - j - 1) hashes). Same node hash as
 * zkb_merkle_layer with no columns. */
int zkb_merkle_levels(zkb_ctx* ctx, int child_log, const uint32_t* children, int levels, uint32_t* const* out_layers, int m31_out);
/* The upper part of a tree in one launch, for trees whose small layers take no columns (every FRI
 * layer tree; a trace tree without tiny columns): given the layer of 2^top_log hashes
 * (top_log <= 10), writes lower_layers[k] (2^k hashes) for k = top_log-1 .. 0, each node being
 * commit_on_layer(k, prev = layer k+1, no columns). Equivalent to top_log calls of zkb_merkle_layer. */
int zkb_merkle_top(zkb_ctx* ctx, int top_log, const uint32_t* top_layer, uint32_t* const* lower_layers, int m31_out);
/* The same, followed in the same launch by a FRI layer's channel step on the root it has just built: as
 * zkb_channel_mix_root_draw(d_chan, root, d_alpha, d_root_copy) right after zkb_merkle_top (top_log >= 1). */
int zkb_merkle_top_channel(zkb_ctx* ctx, int top_log, const uint32_t* top_layer, uint32_t* const* lower_layers, int m31_out, uint32_t* d_chan,
                           uint32_t* d_alpha, uint32_t* d_root_copy);

/* ---- FriOps (STWO/prover/fri.rs:37-85; cpu/fri.rs:67-123) ---------------------------------- */
/* fold_circle_into_line: src on the canonic circle domain of log_n_src; dst (2^(log_n_src-1)
 * entries) is updated as dst*alpha^2 + f0 + alpha*f1. */
int zkb_fold_circle_into_line(zkb_ctx* ctx, uint32_t* const dst[4], const uint32_t* const src[4], int log_n_src,
                              const uint32_t h_alpha[4]);
/* The same folds with the challenge read from device memory (4 words, 16-byte aligned), and the channel step that
 * produces it: d_chan = {digest[8], n_draws} of a Blake2sM31Channel (core/channel/blake2s.rs:20-141); the kernel does
 * mix_root(root) then draw_secure_felt(), leaves the new state in d_chan, the challenge in d_alpha and, if d_root_copy
 * is not NULL, a copy of the root there. With these, FriProver::commit (prover/fri.rs:109-221) enqueues every layer's
 * commit, channel step and fold without returning to the host; the host reads the roots and the channel once at the end. */
int zkb_fold_line_dalpha(zkb_ctx* ctx, uint32_t* const out[4], const uint32_t* const in[4], int log_n, const uint32_t* d_alpha);
int zkb_fold_circle_into_line_dalpha(zkb_ctx* ctx, uint32_t* const dst[4], const uint32_t* const src[4], int log_n_src,
                                     const uint32_t* d_alpha);
int zkb_channel_mix_root_draw(zkb_ctx* ctx, uint32_t* d_chan, const uint32_t* d_root, uint32_t* d_alpha, uint32_t* d_root_copy);
/* The same, and `leaves` (2^(log_n - 1) x 8 words) receives the Blake2s-M31 leaf hashes of the folded layer
 * (what zkb_merkle_layer(log_n - 1, NULL, the four output columns) would write): the next FRI tree starts from
 * them. log_n >= 2 for the line fold (at least two leaves), log_n_src >= 3 for the circle fold. */
int zkb_fold_line_dalpha_leaves(zkb_ctx* ctx, uint32_t* const out[4], const uint32_t* const in[4], int log_n, const uint32_t* d_alpha,
                                uint32_t* leaves);
int zkb_fold_circle_into_line_dalpha_leaves(zkb_ctx* ctx, uint32_t* const dst[4], const uint32_t* const src[4], int log_n_src,
                                            const uint32_t* d_alpha, uint32_t* leaves);
/* fold_line with fold_step 1: in on the line domain Coset::half_odds(log_n); out has 2^(log_n-1). */
int zkb_fold_line(zkb_ctx* ctx, uint32_t* const out[4], const uint32_t* const in[4], int log_n,
                  const uint32_t h_alpha[4]);

/* ---- QuotientOps (STWO/prover/pcs/quotient_ops.rs:19-43; cpu/quotients.rs:22-75) ------------ */
/* accumulate_numerators for ONE sample batch: out[row] = sum_j (c_j * cols[col_idx[j]][row] - b_j),
 * j < k, with the line coefficients (b_j, c_j) of core/pcs/quotients.rs:229-258 as k x 4 words. */
int zkb_quot_numerators(zkb_ctx* ctx, const uint32_t* const* cols, int ncols, int log_n, const uint32_t* h_col_idx,
                        const uint32_t* h_b, const uint32_t* h_c, int k, uint32_t* const out[4]);
/* compute_quotients_and_combine: n_acc accumulations; acc_cols[4*a + i] is coordinate i of
 * accumulation a with 2^h_acc_log[a] rows; h_first_lin (n_acc x 4) the summed `a` coefficients;
 * h_points (n_acc x 8) the sample points (x[4], y[4]). out has 2^lifting_log rows. */
int zkb_quot_combine(zkb_ctx* ctx, int n_acc, const uint32_t* const* acc_cols, const int* h_acc_log,
                     const uint32_t* h_first_lin, const uint32_t* h_points, int lifting_log, uint32_t* const out[4]);
/* The same for the rows [row_begin, row_begin + n_rows) of the lifting domain only: what one rank of a row-sharded
 * commitment computes (no counterpart in the reference, which has no multi-device code). The accumulations and
 * `out` hold only those rows (index 0 = row_begin); row_begin must be a multiple of 2^(lifting_log - acc_log + 1)
 * for every accumulation, so that lifted pairs do not straddle the shard. */
int zkb_quot_combine_rows(zkb_ctx* ctx, int n_acc, const uint32_t* const* acc_cols, const int* h_acc_log, const uint32_t* h_first_lin,
                          const uint32_t* h_points, int lifting_log, size_t row_begin, size_t n_rows, uint32_t* const out[4]);

/* ---- AccumulationOps (STWO/prover/air/accumulation.rs:127-145; cpu/accumulation.rs:9-48) --- */
int zkb_accumulate(zkb_ctx* ctx, uint32_t* const col[4], const uint32_t* const other[4], size_t n);
/* dst (2^log_dst rows) += lift of src (2^log_src rows, log_src <= log_dst):
 * dst[i] += src[(i >> (log_dst-log_src+1) << 1) + (i & 1)]. lift_and_accumulate over ascending
 * columns is a chain of these. */
int zkb_lift_accumulate(zkb_ctx* ctx, uint32_t* const dst[4], int log_dst, const uint32_t* const src[4], int log_src);
/* generate_secure_powers: h_out[4*i..] = felt^i. Host-side (n is small). */
int zkb_secure_powers(zkb_ctx* ctx, const uint32_t h_felt[4], size_t n, uint32_t* h_out);

/* ---- GkrOps / MleOps (STWO/prover/lookups/gkr_prover.rs:172-220, mle.rs:9-14;
 * cpu/lookups/gkr.rs:17-263, cpu/lookups/mle.rs:13-46) ------------------------------------- */
#define ZKB_GKR_GRAND_PRODUCT 0
#define ZKB_GKR_LOGUP_GENERIC 1        /* num: QM31 */
#define ZKB_GKR_LOGUP_MULTIPLICITIES 2 /* num: M31 (1 word per entry) */
#define ZKB_GKR_LOGUP_SINGLES 3        /* num: NULL, implicitly 1 */
/* gen_eq_evals: out[x] = v * eq(x, y) for x in {0,1}^ny, bit-reversed; h_y is ny x 4 words. */
int zkb_gkr_eq_evals(zkb_ctx* ctx, const uint32_t* h_y, int ny, const uint32_t h_v[4], uint32_t* out);
/* next_layer: n input entries -> n/2. For the three LogUp kinds the result is LOGUP_GENERIC
 * (num_out, den_out); for GRAND_PRODUCT den/den_out hold the single column. */
int zkb_gkr_next_layer(zkb_ctx* ctx, int kind, const uint32_t* num, const uint32_t* den, size_t n, uint32_t* num_out,
                       uint32_t* den_out);
/* sum_as_poly_in_first_variable, device part: h_out[0..4] = sum at t=0, h_out[4..8] = sum at t=2
 * of eq_evals[i] * (numerator + lambda * denominator) over i < n/4, before the eq correction
 * (the caller applies eq_fixed_var_correction and gkr_prover.rs:884-923). n = layer entries.
 * Alignment (checked, ZKB_EINVAL otherwise): den and eq_evals 16 bytes, QM31 numerators 16 bytes,
 * M31 numerators 8 bytes. */
int zkb_gkr_sum(zkb_ctx* ctx, int kind, const uint32_t* num, const uint32_t* den, size_t n, const uint32_t* eq_evals,
                const uint32_t h_lambda[4], uint32_t h_out[8]);
/* One sum-check round in one launch: fix_first_variable with challenge r on every column of the layer
 * (n entries -> n/2, written to num_out / den_out; a LOGUP_MULTIPLICITIES layer becomes LOGUP_GENERIC,
 * Layer::fix_first_variable, gkr_prover.rs:354-381) AND the sums zkb_gkr_sum would return for the fixed
 * layer (h_out as there). n >= 8. The outputs must not alias the inputs. */
int zkb_gkr_fix_and_sum(zkb_ctx* ctx, int kind, const uint32_t* num, const uint32_t* den, size_t n, const uint32_t h_r[4],
                        const uint32_t* eq_evals, const uint32_t h_lambda[4], uint32_t* num_out, uint32_t* den_out, uint32_t h_out[8]);
/* fix_first_variable: out[i] = in[i] + r * (in[i + n/2] - in[i]); out may alias in for QM31. */
int zkb_mle_fix_qm31(zkb_ctx* ctx, const uint32_t* in, size_t n, const uint32_t h_r[4], uint32_t* out);
int zkb_mle_fix_m31(zkb_ctx* ctx, const uint32_t* in, size_t n, const uint32_t h_r[4], uint32_t* out);

/* Round sums with no allocation anywhere. This entry point has no counterpart in the reference. It
 * is for callers that cannot allocate device memory when they need the sums: a prover running with
 * its allocator locked after it has carved the card into a fixed arena, a thread that must not
 * trigger the device-wide synchronisation an allocation or free can cause, a host that forbids
 * allocation after start-up. It takes no context (creating one allocates); the per-block partial
 * sums and the ticket live in a 64.25 KiB array built into the library, held by every GPU that
 * loads it until the process exits. Same arithmetic and argument meaning as zkb_gkr_sum, except:
 * `device` and `stream` (a cudaStream_t, may be NULL for the default stream) say where to run,
 * d_out receives the 8 result words ON THE DEVICE (stream-ordered; nothing is copied or
 * synchronised), and n is limited to 2^28 entries. That limit is this entry point's stated contract
 * (the kernel walks the layer with a fixed grid of at most 2,048 blocks, so the array's size does
 * not depend on n); larger layers are refused with ZKB_EINVAL. Pointers must be aligned as for
 * zkb_gkr_sum (checked on the host before anything is launched; d_out 4 bytes).
 * The first call on a device looks up the array's device address; make that call before any
 * stream capture. All calls share the one array, so calls that overlap on the same GPU (two
 * streams, two threads) race; issue them on one stream or order them yourself. It calls neither
 * cudaMalloc nor cudaFree nor any allocating routine. zkb_gkr_sum_noalloc_error() returns the text
 * of the calling host thread's last failure. */
int zkb_gkr_sum_noalloc(int device, void* stream, int kind, const uint32_t* num, const uint32_t* den, size_t n,
                        const uint32_t* eq_evals, const uint32_t h_lambda[4], uint32_t* d_out);
const char* zkb_gkr_sum_noalloc_error(void);

/* ---- GrindOps::grind (STWO/core/proof_of_work.rs:3-7; simd/grind.rs:18-93) ------------------
 * Smallest nonce (hi << 32) | lo, lo < 2^20, whose Blake2s(prefixed_digest || nonce) has at least
 * pow_bits trailing zero bits in its first word. h_prefixed_digest: 8 words. */
int zkb_grind(zkb_ctx* ctx, const uint32_t h_prefixed_digest[8], int pow_bits, int m31_out, uint64_t* h_nonce);

/* ---- The Freivalds attention-witness component ------------------------------------------------
 * Rows are tiled by a grid over the input channels (prover/src/layout.rs:141-183, descending
 * groups): groups * chunks + lead = 2^log_rows. */
typedef struct zkb_grid {
    uint32_t log_rows, groups, chunks, lead;
} zkb_grid;
/* Witness scatter (prover/src/gadgets/freivalds/trace.rs:43-162; device original
 * zk_witness_gen_freivalds, prover/src/gadgets/freivalds/device.rs:26-38): from int8 activations
 * qx[tokens][n_in] and weights qw[m][n_in][n_out[m]] (device arrays; qw is a host array of device
 * pointers) writes the pq committed columns (activation + 128) and the n_mats*pk + 4 preprocessed
 * columns (weights, then the selectors chunk+1<chunks, chunk==0, j>0, j+1==rows), every column in
 * committed order (row j at index coset_perm(j), prover/src/common.rs:76-80), and adds the 8-bit
 * range multiplicities of every committed cell to m_r8[table_len] (device) and the count of cells
 * outside the table to *off_table (device). grid->groups must equal n_in. */
int zkb_freivalds_scatter(zkb_ctx* ctx, const int8_t* qx, const int8_t* const* qw, const uint32_t* h_n_out, const zkb_grid* grid,
                          uint32_t pq, uint32_t pk, uint32_t n_in, uint32_t tokens, uint32_t n_mats, uint32_t* const* base_cols,
                          uint32_t* const* pre_cols, uint32_t* m_r8, uint32_t table_len, unsigned long long* off_table);
/* Accumulators (prover/src/gadgets/freivalds/claims.rs:37-109; device original devacc::freivalds,
 * prover/src/devacc.rs:665-713 over zk_acc_freivalds / zk_acc_scan / zk_acc_stage2 / zk_acc_split):
 * from the committed columns (pq) and the weight columns (n_mats*pk) and the challenges s, rv,
 * writes v, then (u_m, acc_m) per matrix, each as 4 coordinate columns in committed order
 * (out_cols: (1 + 2 n_mats) * 4 device columns), and the claims acc_m[last row] (n_mats x 4 words). */
int zkb_freivalds_acc(zkb_ctx* ctx, const uint32_t* const* base_cols, const uint32_t* const* pre_cols, const zkb_grid* grid, uint32_t pq,
                      uint32_t pk, uint32_t n_mats, const uint32_t h_s[4], const uint32_t h_rv[4], uint32_t* const* out_cols,
                      uint32_t* h_claims);

/* ---- Witness generation of two more column families, in committed order --------------------------
 * Both write row j of the natural (coset) order at index coset_perm(j) (prover/src/common.rs:76-80), so no
 * trace column is shuffled, packed or uploaded by the host. All pointers are device pointers unless named h_*;
 * counters / base_cols / pre_cols are host arrays of device pointers. Nothing is synchronised: results are
 * ordered on the context's stream. */

/* The shared lookup tables' own columns (device original zk_witness_gen_tables, stwo_cuda/cuda/
 * zk_table_witness_gen.cu:124-146, called from prover/src/devtab.rs:267): for every committed row i with
 * d = coset_perm(i): x_col[i] = d; y_col[i] = expmap[pattern(d)] where pattern(d) is d itself when bf16x is
 * non-zero and otherwise the bf16 bits (round to nearest even) of -d / two_pow, which is exp_int_table
 * (prover/src/bf16.rs:374) read through the 2^16-entry map of bf16 patterns to numerators; m_col[i] (skipped when
 * m_col is NULL) = the sum over the n_counters counter arrays of counters[c][d]. Then natural row patch_idx[t] of
 * y takes patch_val[t] (the rows where a witness's own table differs from the closed form). 2^log_rows rows. */
int zkb_witness_tables(zkb_ctx* ctx, const uint32_t* expmap, const uint32_t* const* counters, uint32_t n_counters, const uint32_t* patch_idx,
                       const uint32_t* patch_val, uint32_t n_patch, uint32_t log_rows, int bf16x, double two_pow, uint32_t* x_col,
                       uint32_t* y_col, uint32_t* m_col);

/* Shape of one matmul dequantize component, as the prover's Map / MatLayout / Spec fix it (the reference passes
 * the same numbers in ZkDequantWitnessGenCfg, stwo_cuda/cuda/zk_dequant_witness_gen.cuh:38-60, filled at
 * prover/src/gadgets/dequant/device.rs:290-325). tokens * chunks = 2^log_rows and chunks * per_row = n_out. */
typedef struct zkb_dequant_cfg {
    uint32_t variant;   /* 0 = power-of-two scales (jx, jw), 1 = bf16 scale chain (sx, sw, mul2) */
    uint32_t sticky;    /* the rounding mode keeps a sticky bit (round to nearest even) */
    uint32_t kmax;      /* largest round-bit weight the normalisation table carries */
    uint32_t do_ref;    /* also run the double-precision cross-check and count its disagreements */
    uint32_t tokens, n_out, per_row, chunks, log_rows;
    uint32_t slot0, per_slot; /* column of slot s, field f: slot0 + s * per_slot + f */
    uint32_t chan_w;    /* preprocessed scale columns per slot: 1 (variant 0) or 2 (variant 1) */
    uint32_t f_acc, f_sg, f_m2, f_ph, f_st, f_r, f_m7, f_ef, f_nz, f_eo;
    uint32_t f_mul[6];  /* variant 1: (product mantissa, carry, exponent) of the two chain steps */
    uint32_t sh0, sh1;  /* the per-row shared columns (activation scale) */
    uint32_t n_norm, n_frac, n_mul, n_r8; /* table lengths (bounds of the multiplicity arrays) */
} zkb_dequant_cfg;

/* One dequantize component (device original zk_witness_gen_dequant, stwo_cuda/cuda/zk_dequant_witness_gen.cu:190-386;
 * the per-row arithmetic is witness_gen_mat_row, prover/src/gadgets/dequant/trace.rs:503-690): from the int32
 * accumulators acc[tokens][n_out], the scales (jx[tokens], jw[n_out] or (mantissa, exponent) pairs sx, sw), the
 * normalisation table norm3 (m7, exponent field, non-zero flag per row) and the mantissa product table mul2
 * (m7, carry per row) writes every committed column (base_cols, n_base) and every preprocessed column (pre_cols,
 * n_pre = chan_w * per_row + 5: the per-channel scales, then the selectors not-first, last, j>0 and not last,
 * j>0 and last, j+1 == rows), adds the table multiplicities to m_norm, m_frac, m_mul and m_r8 (zeroed by the
 * caller) and counts into counts[3]: range look-ups outside the 8-bit table, cross-check disagreements, and slots
 * the tables cannot describe (those slots' remaining columns are left unwritten, as in the reference). want_out
 * (NULL or rows * per_row words) receives the cross-check's bf16 pattern per (natural row, slot). */
int zkb_witness_dequant(zkb_ctx* ctx, const int32_t* acc, const int32_t* jx, const int32_t* jw, const uint32_t* sx, const uint32_t* sw,
                        const uint32_t* norm3, const uint32_t* mul2, uint32_t* const* base_cols, uint32_t n_base, uint32_t* const* pre_cols,
                        uint32_t n_pre, uint32_t* m_norm, uint32_t* m_frac, uint32_t* m_mul, uint32_t* m_r8, uint32_t* counts,
                        uint32_t* want_out, const zkb_dequant_cfg* cfg);

/* ---- Witness generation, three more families: shared bf16 tables, key tile selectors, residual stream ------
 * Same conventions as above: committed order, device pointers unless named h_ or said to be host arrays, nothing
 * synchronised. The reference kernels' `mutate` arguments (deliberate defects for negative controls) are not built. */

#define ZKB_PRE_NORM 0  /* 6 columns: m2, ph, st, m7, exponent field, non-zero flag (prover/src/bf16.rs:130-158) */
#define ZKB_PRE_FRAC 1  /* 3 columns: ph, r, st (prover/src/gadgets/residual_stream/mod.rs:1116-1122) */
#define ZKB_PRE_MUL 2   /* 4 columns: a, b, m7, carry (prover/src/bf16.rs:264-281) */
#define ZKB_PRE_QNZ 3   /* 2 columns: the row index and whether it is non-zero */
#define ZKB_PRE_RANGE 4 /* 1 column: the row index */
/* One shared table's preprocessed columns and its multiplicity column (device original zk_witness_gen_pre_table,
 * stwo_cuda/cuda/zk_pre_witness_gen.cu:150-270, called from prover/src/devpre.rs:482). Every row is computed from its
 * own index d = coset_perm(i): no table is uploaded. round: 0 nearest-even (the tables then carry a sticky bit),
 * 1 nearest-away, 2 truncate. The table's own length (256 + (kmax+1) * 256 * (1 + sticky) for NORM, 2^(kmax+1) for
 * FRAC, 2^14 for MUL, 2^log_rows otherwise) must fit 2^log_rows; rows past it commit zero. n_cols must be the
 * kind's column count; cols is a host array of n_cols device columns (8-byte aligned). m_col (may be NULL)
 * receives the sum over the n_counters counter arrays at the row. Then natural row patch_idx[t] takes the n_cols
 * values patch_val[t * n_cols ..] (the rows where a witness's own table is not the closed form). log_rows >= 1. */
int zkb_witness_pre_table(zkb_ctx* ctx, uint32_t kind, uint32_t log_rows, uint32_t kmax, uint32_t round, const uint32_t* const* counters,
                          uint32_t n_counters, const uint32_t* patch_idx, const uint32_t* patch_val, uint32_t n_patch, uint32_t* const* cols,
                          uint32_t n_cols, uint32_t* m_col);

#define ZKB_TILE_CHAN 0
#define ZKB_TILE_KEY 1
#define ZKB_TILE_TOK 2
#define ZKB_TILE_ACTIVE 1u  /* the row belongs to a group (not an inert lead row) */
#define ZKB_TILE_NOFIRST 2u /* not the first row of its group */
#define ZKB_TILE_LAST 4u    /* the last row of its group */
#define ZKB_TILE_ISTART 8u  /* the first row of an instance */
/* The per-row layout flags of one key tile sub-component, in NATURAL row order (device original zk_flags_key_tile,
 * stwo_cuda/cuda/zk_acc.cu:78-97 with zk_acc.cuh:116-180; host statement prover/src/gadgets/attention/trace.rs:742-790
 * over Grid::row, prover/src/layout.rs:141-183). CHAN and KEY rows are tiled groups * chunks + lead = 2^log_rows
 * (descending: groups run downwards); an instance starts at the first row of a group g with g mod modulus ==
 * modulus - 1 (modulus = head dimension for CHAN, context length for KEY). TOK has no groups: every row is active and
 * an instance starts where (rows - j) * rw is a multiple of modulus (the sequence length). */
int zkb_key_tile_flags(zkb_ctx* ctx, uint32_t shape, uint32_t log_rows, uint32_t groups, uint32_t chunks, uint32_t lead, uint32_t descending,
                       uint32_t modulus, uint32_t rw, uint32_t* flags);
/* The selector columns of that sub-component, committed order, from its flags (device original zk_witness_gen_sel,
 * stwo_cuda/cuda/zk_pre_witness_gen.cu:292-385, called from prover/src/devpre.rs:635). With pos = (j > 0) and
 * end = (j + 1 == rows): TOK (3 columns) pos, end, ISTART; CHAN (5) NOFIRST, LAST, pos, end, ISTART; KEY (8 or 9)
 * NOFIRST, LAST, pos, end, pos & !LAST, pos & LAST, ISTART, the key scale scale[group / ctx_len] of the row's
 * instance (1 on inert rows, and everywhere when with_scale is 0; scale holds n_insts inverted scales), and as a
 * ninth column ACTIVE. cols: host array of n_cols device columns. */
int zkb_witness_selectors(zkb_ctx* ctx, uint32_t shape, uint32_t log_rows, uint32_t groups, uint32_t chunks, uint32_t lead, uint32_t descending,
                          const uint32_t* flags, const uint32_t* scale, uint32_t ctx_len, uint32_t n_insts, int with_scale, uint32_t* const* cols,
                          uint32_t n_cols);

/* The residual-stream component's program, lowered to column indices (Prog, prover/src/gadgets/residual_stream/mod.rs:387-611;
 * the reference passes the same records, stwo_cuda/cuda/zk_residual_stream_witness_gen.cuh:70-115, filled at
 * prover/src/gadgets/residual_stream/device.rs:300-420). Values are bf16 numbers held as (sm, ef): signed significand
 * +-[128, 256) or 0, and exponent field. */
#define ZKB_RS_NONE 0xffffffffu /* an operand that is the constant zero */
typedef struct zkb_rs_group {
    uint32_t n;        /* leaves of this group per row */
    uint32_t leaf_col; /* column of leaf 0's sm; leaf k is at leaf_col + k * width: sm, ef[, unary sm, unary ef] */
    uint32_t width;    /* 2, or 4 when the group carries a unary image */
    uint32_t un;       /* 0: none; else 1 + index of the unary table */
    uint32_t flat;     /* index of the group's first leaf inside a row of `wit` (the sum of the earlier groups' n) */
} zkb_rs_group;
typedef struct zkb_rs_slot {
    uint32_t a_sm, a_ef, b_sm, b_ef; /* columns of the two operands (a_sm == ZKB_RS_NONE: the constant zero) */
    uint32_t base;                   /* first column of the slot's own cells */
    uint32_t o_sm, o_ef;             /* columns of the slot's output pair */
    uint32_t from_slot;              /* bit 0: operand a is a slot output (its exponent is clamped to 0xfe on reading); bit 1: b */
} zkb_rs_slot;
typedef struct zkb_rs_program {
    const zkb_rs_group* groups; /* host array */
    uint32_t n_groups;
    const zkb_rs_slot* slots;   /* host array, evaluation order */
    uint32_t n_slots;
    const uint32_t* out_slot;   /* host array: the slots whose outputs are reported, flattened */
    uint32_t out_w;
    uint32_t kind;              /* 0: every slot adds (13 cells, 14 with the sticky bit); 1: every slot multiplies (4 cells) */
    uint32_t sticky, kmax;      /* as for the tables above */
} zkb_rs_program;
typedef struct zkb_rs_tables {
    const uint32_t* norm3;     /* device: (m7, exponent field, non-zero flag) per normalisation row; adds only */
    uint32_t n_norm;
    const int32_t* smul3;      /* device: (signed significand, carry, non-zero flag) per signed-product row; multiplies only */
    uint32_t n_smul;
    const int32_t* const* un2; /* host array of n_un device tables: (sm, ef) of the unary image per value-table row, 8-byte aligned */
    uint32_t n_un, n_val;
} zkb_rs_tables;
typedef struct zkb_rs_mult {
    uint32_t* m; /* device multiplicity array, zeroed by the caller */
    uint32_t n;
} zkb_rs_mult;
typedef struct zkb_rs_mults {
    zkb_rs_mult pow, norm, val, frac, smul;
    const zkb_rs_mult* un; /* host array, one per unary table */
} zkb_rs_mults;
/* One residual-stream component (device original zk_witness_gen_residual_stream, stwo_cuda/cuda/
 * zk_residual_stream_witness_gen.cu:231-470; host statement residual_stream_component,
 * prover/src/gadgets/residual_stream/mod.rs:1418-1760). wit: live_rows x n_leaves bf16 patterns (one per word),
 * row-flat; rows from live_rows up to 2^log_rows are evaluated on zero leaves. Writes every committed cell (cols: host
 * array of n_cols device columns), adds every lookup to its multiplicity array, and writes in NATURAL row order
 * out_pat (rows x out_w bf16 patterns of the reported slots), out_nat (rows x out_w pairs: significand and unclamped
 * exponent) and in_nat (rows x n_leaves pairs); out_nat and in_nat 8-byte aligned. counts[0] += lookups that fall
 * outside their table, counts[1] += results whose exponent leaves bf16's normal range, counts[2] += leaves whose unary
 * image has no table row. Every column index of the program is checked against n_cols before the launch. */
int zkb_witness_residual_stream(zkb_ctx* ctx, const zkb_rs_program* prog, const zkb_rs_tables* tables, const uint32_t* wit, uint32_t live_rows,
                                uint32_t log_rows, uint32_t* const* cols, uint32_t n_cols, uint32_t* out_pat, int32_t* out_nat, int32_t* in_nat,
                                const zkb_rs_mults* mults, uint32_t* counts);

#ifdef __cplusplus
}
#endif
#endif /* ZKB200_H */
