// TEST INFRASTRUCTURE ONLY. C entry points over the CPU oracle so that tests (ctypes) and the
// bench's CPU-baseline leg can call it. The product library never links this file.
//
// Conventions: M31 values are uint32_t in [0, p). A "secure column" is four uint32_t arrays
// (coordinate layout, as SecureColumnByCoords, nitroo/crates/stwo/src/prover/secure_column.rs:13-15);
// GKR multilinear columns are arrays of QM31 as 4 consecutive uint32_t.
#include "protocol.hpp"
#include "verify.hpp"
#include "bary.hpp"
#include "accel.hpp"
namespace zko {
void fill_accel_avx512(Accel& a);
void fill_accel_avx2(Accel& a);
}
#include <cstdlib>
#ifdef _OPENMP
#include <omp.h>
#endif

using namespace zko;

static inline QM31 q_from(const uint32_t* p) { return QM31::from_u32(p[0], p[1], p[2], p[3]); }
static inline void q_to(QM31 q, uint32_t* p) { q.to_u32(p); }
static SecureColumn load_soa(const uint32_t* const c[4], size_t n) {
    SecureColumn v(n);
    for (size_t i = 0; i < n; i++) v[i] = QM31::from_u32(c[0][i], c[1][i], c[2][i], c[3][i]);
    return v;
}
static void store_soa(const SecureColumn& v, uint32_t* const c[4]) {
    for (size_t i = 0; i < v.size(); i++) {
        uint32_t w[4]; v[i].to_u32(w);
        for (int k = 0; k < 4; k++) c[k][i] = w[k];
    }
}

static const TwiddleTree& tower(uint32_t log_half_coset) {
    // one canonic twiddle tree per root size, built on demand
    static std::vector<TwiddleTree*> cache(32, nullptr);
    TwiddleTree*& t = cache[log_half_coset];
    if (!t) t = new TwiddleTree(precompute_twiddles(Coset::half_odds(log_half_coset)));
    return *t;
}

extern "C" {

int zko_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void zko_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

// ---- fields (for unit tests of the restatement itself)
uint32_t zko_m31_mul(uint32_t a, uint32_t b) { return (M31(a) * M31(b)).v; }
uint32_t zko_m31_inv(uint32_t a) { return M31(a).inverse().v; }
uint32_t zko_m31_reduce64(uint64_t a) { return M31::reduce(a).v; }
void zko_cm31_mul(const uint32_t* a, const uint32_t* b, uint32_t* out) {
    CM31 r = CM31(M31(a[0]), M31(a[1])) * CM31(M31(b[0]), M31(b[1]));
    out[0] = r.a.v; out[1] = r.b.v;
}
void zko_cm31_inv(const uint32_t* a, uint32_t* out) {
    CM31 r = CM31(M31(a[0]), M31(a[1])).inverse();
    out[0] = r.a.v; out[1] = r.b.v;
}
void zko_qm31_mul(const uint32_t* a, const uint32_t* b, uint32_t* out) { q_to(q_from(a) * q_from(b), out); }
void zko_qm31_inv(const uint32_t* a, uint32_t* out) { q_to(q_from(a).inverse(), out); }

// ---- circle
void zko_circle_point(uint64_t index, uint32_t* xy) {
    auto p = CirclePointIndex{index}.reduce().to_point();
    xy[0] = p.x.v; xy[1] = p.y.v;
}
void zko_secure_circle_mul(uint64_t lo, uint64_t hi, uint32_t* xy8) {
    auto p = secure_field_circle_gen().mul(lo, hi);
    q_to(p.x, xy8); q_to(p.y, xy8 + 4);
}
// domain point of row `i` (natural order) of the canonic circle domain of `log_size`
void zko_domain_at(uint32_t log_size, uint64_t i, uint32_t* xy) {
    auto p = CanonicCoset(log_size).circle_domain().at(i);
    xy[0] = p.x.v; xy[1] = p.y.v;
}

// ---- twiddles: the tower of Coset::half_odds(log_size), `2^log_size` entries each
void zko_twiddles(uint32_t log_size, uint32_t* tw, uint32_t* itw) {
    const TwiddleTree& t = tower(log_size);
    for (size_t i = 0; i < t.twiddles.size(); i++) { tw[i] = t.twiddles[i].v; if (itw) itw[i] = t.itwiddles[i].v; }
}
void zko_line_twiddles_slices(uint32_t domain_log_size, const uint32_t* buf, size_t buf_len, uint64_t* offs, uint64_t* lens) {
    std::vector<M31> b(buf_len);
    for (size_t i = 0; i < buf_len; i++) b[i] = M31(buf[i]);
    auto s = domain_line_twiddles_from_tree(CanonicCoset(domain_log_size).half_coset(), b);
    for (size_t i = 0; i < s.size(); i++) { offs[i] = s[i].p - b.data(); lens[i] = s[i].n; }
}

// ---- circle FFT on canonic domains, many columns (columns are independent; threads split them)
void zko_interpolate_cols(uint32_t* const* cols, int ncols, uint32_t log_n) {
    CircleDomain d = CanonicCoset(log_n).circle_domain();
    const TwiddleTree& t = tower(log_n >= 1 ? log_n - 1 : 0);
    size_t n = (size_t)1 << log_n;
#pragma omp parallel for schedule(dynamic)
    for (int c = 0; c < ncols; c++) {
        std::vector<M31> v(n);
        for (size_t i = 0; i < n; i++) v[i] = M31(cols[c][i]);
        interpolate(v, d, t);
        for (size_t i = 0; i < n; i++) cols[c][i] = v[i].v;
    }
}
void zko_evaluate_cols(const uint32_t* const* coeffs, int ncols, uint32_t log_n, uint32_t* const* out, uint32_t log_out) {
    CircleDomain d = CanonicCoset(log_out).circle_domain();
    const TwiddleTree& t = tower(log_out - 1);
    size_t n = (size_t)1 << log_n, N = (size_t)1 << log_out;
#pragma omp parallel for schedule(dynamic)
    for (int c = 0; c < ncols; c++) {
        std::vector<M31> v(n);
        for (size_t i = 0; i < n; i++) v[i] = M31(coeffs[c][i]);
        std::vector<M31> e = evaluate(v, d, t);
        for (size_t i = 0; i < N; i++) out[c][i] = e[i].v;
    }
}
void zko_eval_at_point(const uint32_t* coeffs, uint32_t log_n, const uint32_t* point8, uint32_t* out4) {
    std::vector<M31> v((size_t)1 << log_n);
    for (size_t i = 0; i < v.size(); i++) v[i] = M31(coeffs[i]);
    CirclePoint<QM31> p{q_from(point8), q_from(point8 + 4)};
    q_to(eval_at_point(v, p), out4);
}

// PolyOps from evaluations: weights (2^log x 4 words), the weighted sum, and evaluation by folding (cpu/circle.rs:101-180).
void zko_barycentric_weights(uint32_t log_n, const uint32_t* point8, uint32_t* out) {
    CirclePoint<QM31> p{q_from(point8), q_from(point8 + 4)};
    auto w = barycentric_weights(log_n, p);
    for (size_t i = 0; i < w.size(); i++) q_to(w[i], out + 4 * i);
}
void zko_barycentric_eval(const uint32_t* evals, const uint32_t* weights, uint32_t log_n, uint32_t* out4) {
    size_t n = (size_t)1 << log_n;
    std::vector<M31> e(n);
    std::vector<QM31> w(n);
    for (size_t i = 0; i < n; i++) { e[i] = M31(evals[i]); w[i] = q_from(weights + 4 * i); }
    q_to(barycentric_eval_at_point(e, w), out4);
}
void zko_eval_by_folding(const uint32_t* evals, uint32_t log_n, const uint32_t* point8, uint32_t* out4) {
    std::vector<M31> e((size_t)1 << log_n);
    for (size_t i = 0; i < e.size(); i++) e[i] = M31(evals[i]);
    CirclePoint<QM31> p{q_from(point8), q_from(point8 + 4)};
    q_to(eval_at_point_by_folding(e, p), out4);
}

void zko_bit_reverse_u32(uint32_t* v, uint32_t log_n) { bit_reverse(v, (size_t)1 << log_n); }

// ---- hashing
void zko_blake2s(const uint8_t* data, size_t len, int m31, uint8_t* out32) {
    Hash h = Hasher::hash(data, len, m31 != 0);
    memcpy(out32, h.data(), 32);
}
// prev: 2^(log_size+1) hashes of 32 bytes, or NULL. out: 2^log_size hashes.
void zko_commit_on_layer(uint32_t log_size, const uint8_t* prev, const uint32_t* const* cols, int ncols, int m31, uint8_t* out) {
    size_t n = (size_t)1 << log_size;
    std::vector<Hash> pv;
    if (prev) { pv.resize(2 * n); memcpy(pv.data(), prev, 64 * n); }
    std::vector<const M31*> cp;
    for (int c = 0; c < ncols; c++) cp.push_back(reinterpret_cast<const M31*>(cols[c]));
    std::vector<Hash> h = commit_on_layer(log_size, prev ? &pv : nullptr, cp, m31 != 0);  // scalar, or packed when zko_set_simd(1)
    memcpy(out, h.data(), 32 * n);
}

// ---- channel (opaque handle)
void* zko_channel_new(int m31) { return new Channel(m31 != 0); }
void zko_channel_free(void* c) { delete (Channel*)c; }
void zko_channel_digest(void* c, uint8_t* out32) { memcpy(out32, ((Channel*)c)->digest.data(), 32); }
void zko_channel_mix_u32s(void* c, const uint32_t* d, size_t n) { ((Channel*)c)->mix_u32s(d, n); }
void zko_channel_mix_u64(void* c, uint64_t v) { ((Channel*)c)->mix_u64(v); }
void zko_channel_mix_felts(void* c, const uint32_t* felts, size_t n) {
    std::vector<QM31> f(n);
    for (size_t i = 0; i < n; i++) f[i] = q_from(felts + 4 * i);
    ((Channel*)c)->mix_felts(f);
}
void zko_channel_mix_root(void* c, const uint8_t* root32) { Hash h; memcpy(h.data(), root32, 32); ((Channel*)c)->mix_root(h); }
void zko_channel_draw_u32s(void* c, uint32_t* out8) { auto u = ((Channel*)c)->draw_u32s(); for (int i = 0; i < 8; i++) out8[i] = u[i]; }
void zko_channel_draw_secure_felt(void* c, uint32_t* out4) { q_to(((Channel*)c)->draw_secure_felt(), out4); }
void zko_channel_draw_secure_felts(void* c, size_t n, uint32_t* out) {
    auto v = ((Channel*)c)->draw_secure_felts(n);
    for (size_t i = 0; i < n; i++) q_to(v[i], out + 4 * i);
}
uint64_t zko_channel_grind(void* c, uint32_t pow_bits) { return ((Channel*)c)->grind(pow_bits); }
int zko_channel_verify_pow(void* c, uint32_t pow_bits, uint64_t nonce) { return ((Channel*)c)->verify_pow_nonce(pow_bits, nonce); }
void zko_draw_queries(void* c, uint32_t log_domain_size, size_t n, uint64_t* out) {
    auto q = draw_queries(*(Channel*)c, log_domain_size, n);
    for (size_t i = 0; i < n; i++) out[i] = q[i];
}

// ---- FRI folds (secure columns in coordinate layout)
void zko_fold_line(const uint32_t* const in[4], uint32_t log_n, const uint32_t* alpha4, uint32_t* const out[4]) {
    SecureColumn e = load_soa(in, (size_t)1 << log_n);
    LineDomain d{Coset::half_odds(log_n)};
    store_soa(fold_line(e, d, q_from(alpha4)), out);
}
void zko_fold_circle_into_line(uint32_t* const dst[4], const uint32_t* const src[4], uint32_t log_n_src, const uint32_t* alpha4) {
    size_t n = (size_t)1 << log_n_src;
    SecureColumn s = load_soa(src, n);
    const uint32_t* const dc[4] = {dst[0], dst[1], dst[2], dst[3]};
    SecureColumn d = load_soa(dc, n / 2);
    fold_circle_into_line(d, s, CanonicCoset(log_n_src).circle_domain(), q_from(alpha4));
    store_soa(d, dst);
}

// ---- quotients
// One sample batch: k entries (col_idx[j], value[j] (QM31), rand[j] (QM31)) at `point8`.
// Writes the partial numerators (coordinate layout) and the first-linear-term sum.
void zko_quot_numerators(const uint32_t* const* cols, int /*ncols*/, uint32_t log_n, const uint32_t* point8, int k,
                         const uint32_t* col_idx, const uint32_t* values, const uint32_t* rands,
                         uint32_t* const out[4], uint32_t* first_lin4) {
    size_t n = (size_t)1 << log_n;
    ColumnSampleBatch b;
    b.point = {q_from(point8), q_from(point8 + 4)};
    for (int j = 0; j < k; j++) b.cols_vals_randpows.push_back({col_idx[j], q_from(values + 4 * j), q_from(rands + 4 * j)});
    auto coeffs = column_line_coeffs({b})[0];
    QM31 first = QM31::zero();
    for (auto& lc : coeffs) first = first + lc.a;
    q_to(first, first_lin4);
#pragma omp parallel for schedule(static)
    for (size_t row = 0; row < n; row++) {
        QM31 numerator = QM31::zero();
        for (int j = 0; j < k; j++) {
            QM31 value = coeffs[j].c * M31(cols[col_idx[j]][row]);
            numerator = numerator + (value - coeffs[j].b);
        }
        uint32_t w[4]; numerator.to_u32(w);
        for (int c = 0; c < 4; c++) out[c][row] = w[c];
    }
}
// Line coefficients (a, b, c) of one sample, as 12 uint32_t.
void zko_line_coeffs(const uint32_t* point8, const uint32_t* value4, const uint32_t* alpha4, uint32_t* out12) {
    LineCoeffs lc = complex_conjugate_line_coeffs({{q_from(point8), q_from(point8 + 4)}, q_from(value4)}, q_from(alpha4));
    q_to(lc.a, out12); q_to(lc.b, out12 + 4); q_to(lc.c, out12 + 8);
}
// accs: n_acc accumulations; acc_cols[4*a + c] is coordinate c of accumulation a, of length 2^acc_log[a].
void zko_quot_combine(int n_acc, const uint32_t* const* acc_cols, const uint32_t* acc_log, const uint32_t* first_lin,
                      const uint32_t* points, uint32_t lifting_log, uint32_t* const out[4]) {
    std::vector<AccumulatedNumerators> accs;
    for (int a = 0; a < n_acc; a++) {
        const uint32_t* const c[4] = {acc_cols[4 * a], acc_cols[4 * a + 1], acc_cols[4 * a + 2], acc_cols[4 * a + 3]};
        accs.push_back({{q_from(points + 8 * a), q_from(points + 8 * a + 4)}, load_soa(c, (size_t)1 << acc_log[a]), q_from(first_lin + 4 * a)});
    }
    store_soa(compute_quotients_and_combine(accs, lifting_log), out);
}
void zko_accumulate(uint32_t* const col[4], const uint32_t* const other[4], size_t n) {
    const uint32_t* const cc[4] = {col[0], col[1], col[2], col[3]};
    SecureColumn a = load_soa(cc, n), b = load_soa(other, n);
    accumulate(a, b);
    store_soa(a, col);
}
// cols[4*i + c], ascending sizes 2^logs[i]; result written into `out` (size of the last).
void zko_lift_and_accumulate(int ncols, const uint32_t* const* cols, const uint32_t* logs, uint32_t* const out[4]) {
    std::vector<SecureColumn> v;
    for (int i = 0; i < ncols; i++) {
        const uint32_t* const c[4] = {cols[4 * i], cols[4 * i + 1], cols[4 * i + 2], cols[4 * i + 3]};
        v.push_back(load_soa(c, (size_t)1 << logs[i]));
    }
    store_soa(lift_and_accumulate(v), out);
}
void zko_secure_powers(const uint32_t* felt4, size_t n, uint32_t* out) {
    auto v = generate_secure_powers(q_from(felt4), n);
    for (size_t i = 0; i < n; i++) q_to(v[i], out + 4 * i);
}

// ---- GKR (QM31 arrays as 4 consecutive words)
void zko_gkr_eq_evals(const uint32_t* y, size_t ny, const uint32_t* v4, uint32_t* out) {
    std::vector<QM31> yy(ny);
    for (size_t i = 0; i < ny; i++) yy[i] = q_from(y + 4 * i);
    auto e = gen_eq_evals(yy.data(), ny, q_from(v4));
    for (size_t i = 0; i < e.size(); i++) q_to(e[i], out + 4 * i);
}
static Layer load_layer(int kind, const uint32_t* num, const uint32_t* den, size_t n) {
    Layer l;
    l.kind = (LayerKind)kind;
    l.den.resize(n);
    for (size_t i = 0; i < n; i++) l.den[i] = q_from(den + 4 * i);
    if (kind == LOGUP_GENERIC) { l.num.resize(n); for (size_t i = 0; i < n; i++) l.num[i] = q_from(num + 4 * i); }
    if (kind == LOGUP_MULTIPLICITIES) { l.num_base.resize(n); for (size_t i = 0; i < n; i++) l.num_base[i] = M31(num[i]); }
    return l;
}
// n = input entries. Outputs n/2 QM31 each (num_out unused for GRAND_PRODUCT).
void zko_gkr_next_layer(int kind, const uint32_t* num, const uint32_t* den, size_t n, uint32_t* num_out, uint32_t* den_out) {
    Layer o = next_layer(load_layer(kind, num, den, n));
    for (size_t i = 0; i < n / 2; i++) {
        q_to(o.den[i], den_out + 4 * i);
        if (o.kind != GRAND_PRODUCT) q_to(o.num[i], num_out + 4 * i);
    }
}
void zko_gkr_round_sums(int kind, const uint32_t* num, const uint32_t* den, size_t n, const uint32_t* eq_evals,
                        const uint32_t* lambda4, uint32_t* out8) {
    Layer l = load_layer(kind, num, den, n);
    size_t n_terms = n / 4;
    std::vector<QM31> e(n_terms);
    for (size_t i = 0; i < n_terms; i++) e[i] = q_from(eq_evals + 4 * i);
    QM31 a0, a2;
    round_sums(l, e.data(), n_terms, q_from(lambda4), a0, a2);
    q_to(a0, out8); q_to(a2, out8 + 4);
}
void zko_mle_fix_first_qm31(const uint32_t* in, size_t n, const uint32_t* r4, uint32_t* out) {
    std::vector<QM31> v(n);
    for (size_t i = 0; i < n; i++) v[i] = q_from(in + 4 * i);
    auto o = fix_first_variable(v, q_from(r4));
    for (size_t i = 0; i < o.size(); i++) q_to(o[i], out + 4 * i);
}
void zko_mle_fix_first_m31(const uint32_t* in, size_t n, const uint32_t* r4, uint32_t* out) {
    std::vector<M31> v(n);
    for (size_t i = 0; i < n; i++) v[i] = M31(in[i]);
    auto o = fix_first_variable(v, q_from(r4));
    for (size_t i = 0; i < o.size(); i++) q_to(o[i], out + 4 * i);
}

}  // extern "C"

// ---------------------------------------------------------------- whole protocols
extern "C" {

void zko_channel_pow_prefixed_digest(void* c, uint32_t pow_bits, uint32_t* out8) {
    Hash h = ((Channel*)c)->pow_prefixed_digest(pow_bits);
    for (int i = 0; i < 8; i++) out8[i] = load_le32(&h[4 * i]);
}

// Commits `n_trees` trees of trace columns (evaluations on the canonic domain of their own size,
// bit-reversed), samples every column at one channel-drawn point (columns whose flat index is a
// multiple of `two_sample_every`, if non-zero, also at the point one trace step before it), and
// proves the values. Channel: Blake2sM31, default state, PcsConfig mixed in first.
// Writes the proof words to `out` (capacity `cap` words) and returns the word count, or -1.
long zko_pcs_prove(int n_trees, const int* tree_ncols, const uint32_t* const* cols, const uint32_t* col_logs,
                   uint32_t pow_bits, uint32_t log_blowup, uint32_t log_last_layer, uint32_t n_queries,
                   int two_sample_every, uint32_t* out, size_t cap) {
    PcsConfig cfg;
    cfg.pow_bits = pow_bits;
    cfg.fri = {log_blowup, log_last_layer, n_queries, 1};
    uint32_t max_log = 0;
    int total = 0;
    for (int t = 0; t < n_trees; t++) total += tree_ncols[t];
    for (int i = 0; i < total; i++) max_log = std::max(max_log, col_logs[i]);
    Channel ch(true);
    cfg.mix_into(ch);
    CommitmentSchemeProver prover(cfg, max_log + log_blowup);
    int flat = 0;
    for (int t = 0; t < n_trees; t++) {
        std::vector<std::vector<M31>> columns;
        columns.resize(tree_ncols[t]);
        const int flat0 = flat;
#pragma omp parallel for schedule(dynamic)
        for (int c = 0; c < tree_ncols[t]; c++) {
            size_t n = (size_t)1 << col_logs[flat0 + c];
            columns[c].resize(n);
            memcpy(static_cast<void*>(columns[c].data()), cols[flat0 + c], 4 * n);  // M31 is one canonical word
        }
        flat += tree_ncols[t];
        prover.commit_evals(columns, ch);
    }
    CirclePoint<QM31> oods = get_random_point(ch);
    std::vector<std::vector<std::vector<CirclePoint<QM31>>>> points(n_trees);
    flat = 0;
    for (int t = 0; t < n_trees; t++)
        for (int c = 0; c < tree_ncols[t]; c++, flat++) {
            std::vector<CirclePoint<QM31>> p;
            if (two_sample_every && flat % two_sample_every == 0)
                p.push_back(oods + into_ef(CanonicCoset(col_logs[flat]).step().conjugate()));
            p.push_back(oods);
            points[t].push_back(p);
        }
    PcsProof proof = prover.prove_values(points, ch);
    std::vector<uint32_t> w = proof.to_words();
    // the channel state after the proof pins every Fiat-Shamir step
    for (int i = 0; i < 8; i++) w.push_back(load_le32(&ch.digest[4 * i]));
    if (w.size() > cap) return -1;
    memcpy(out, w.data(), w.size() * 4);
    return (long)w.size();
}

// Verifies a proof made by zko_pcs_prove (or by the CUDA path's zkb_pcs_prove_*, same words) for trees of trace columns of
// the given log sizes: the verifier replays the channel (config, commitments from the proof, out-of-domain point, the same
// sampled points per column as the prover's rule) and runs CommitmentSchemeVerifier::verify_values. Returns 0 when the
// proof is accepted AND the channel digest after it equals the 8 words that follow the proof; otherwise the VerifyError
// code, with the nested Merkle error in info[0] and the layer / tree index in info[1] (info may be NULL). 31: the
// trailing digest differs although the proof verifies.
int zko_pcs_verify(const uint32_t* words, size_t n_words, int n_trees, const int* tree_ncols, const uint32_t* col_logs, uint32_t pow_bits,
                   uint32_t log_blowup, uint32_t log_last_layer, uint32_t n_queries, int two_sample_every, int* info) {
    PcsConfig cfg;
    cfg.pow_bits = pow_bits;
    cfg.fri = {log_blowup, log_last_layer, n_queries, 1};
    std::vector<size_t> ncols;
    for (int t = 0; t < n_trees; t++) ncols.push_back((size_t)tree_ncols[t]);
    PcsProof proof;
    size_t used = 0;
    if (info) { info[0] = 0; info[1] = -1; }
    if (!parse_pcs_proof(words, n_words, ncols, proof, used)) return (int)VerifyError::Malformed;
    Channel ch(true);
    cfg.mix_into(ch);
    CommitmentSchemeVerifier v;
    v.config = cfg;
    int flat = 0;
    for (int t = 0; t < n_trees; t++) {
        std::vector<uint32_t> logs;
        for (int c = 0; c < tree_ncols[t]; c++, flat++) logs.push_back(col_logs[flat]);
        v.commit(proof.commitments[t], logs, ch);
    }
    CirclePoint<QM31> oods = get_random_point(ch);
    std::vector<std::vector<std::vector<CirclePoint<QM31>>>> points(n_trees);
    flat = 0;
    for (int t = 0; t < n_trees; t++)
        for (int c = 0; c < tree_ncols[t]; c++, flat++) {
            std::vector<CirclePoint<QM31>> p;
            if (two_sample_every && flat % two_sample_every == 0)
                p.push_back(oods + into_ef(CanonicCoset(col_logs[flat]).step().conjugate()));
            p.push_back(oods);
            points[t].push_back(p);
        }
    VerifyResult r = v.verify_values(points, proof, ch);
    if (info) { info[0] = (int)r.detail; info[1] = r.layer; }
    if (!r.ok()) return (int)r.error;
    if (used + 8 <= n_words)
        for (int i = 0; i < 8; i++)
            if (words[used + i] != load_le32(&ch.digest[4 * i])) return 31;
    return 0;
}

// Switches the packed restatement of the SIMD backend on (1) or off (0) for every later call; returns the lanes in use:
// 16 (AVX-512), 8 (AVX2) or 0 (scalar: off, or the CPU has neither).
int zko_set_simd(int on) {
    Accel& a = accel();
    a = Accel();
    if (on) {
        __builtin_cpu_init();
        if (__builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw") && __builtin_cpu_supports("avx512dq") &&
            __builtin_cpu_supports("avx512vl"))
            fill_accel_avx512(a);
        else if (__builtin_cpu_supports("avx2"))
            fill_accel_avx2(a);
    }
    return a.lanes;
}

// GKR batch proof of `n_inst` instances (kinds as in ops.hpp; nums[i] may be NULL). The channel is
// Blake2sM31 default state after mix_u64(seed). If verify != 0 the proof is checked with
// partially_verify_batch and -2 is returned on rejection.
long zko_gkr_prove(int n_inst, const int* kinds, const uint32_t* const* nums, const uint32_t* const* dens, const uint64_t* ns,
                   uint64_t seed, int verify, uint32_t* out, size_t cap) {
    std::vector<Layer> layers;
    std::vector<int> is_logup;
    for (int i = 0; i < n_inst; i++) {
        layers.push_back(load_layer(kinds[i], nums[i], dens[i], ns[i]));
        is_logup.push_back(kinds[i] != GRAND_PRODUCT);
    }
    Channel ch(true);
    ch.mix_u64(seed);
    GkrProof proof = gkr_prove_batch(ch, layers);
    if (verify) {
        Channel vch(true);
        vch.mix_u64(seed);
        std::vector<QM31> ood;
        std::vector<std::vector<QM31>> claims;
        if (!gkr_partially_verify_batch(is_logup, proof, vch, ood, claims)) return -2;
        if (ood.size() != proof.ood_point.size()) return -2;
        for (size_t k = 0; k < ood.size(); k++) if (ood[k] != proof.ood_point[k]) return -2;
        if (vch.digest != ch.digest) return -2;
    }
    std::vector<uint32_t> w = proof.to_words();
    for (int i = 0; i < 8; i++) w.push_back(load_le32(&ch.digest[4 * i]));
    if (w.size() > cap) return -1;
    memcpy(out, w.data(), w.size() * 4);
    return (long)w.size();
}

}  // extern "C"

// ---------------------------------------------------------------- Freivalds component
#include "freivalds.hpp"
extern "C" {

uint64_t zko_coset_perm(uint64_t i, uint32_t log_n) { return coset_perm(i, log_n); }

// base_out: pq columns, pre_out: n_mats*pk+4 columns, each 2^log_rows words; m_r8: table_len counters.
void zko_freivalds_columns(const int8_t* qx, const int8_t* const* qw, const uint32_t* n_out, uint32_t n_mats, uint32_t log_rows,
                           uint32_t groups, uint32_t chunks, uint32_t lead, uint32_t pq, uint32_t pk, uint32_t n_in, uint32_t tokens,
                           uint32_t* const* base_out, uint32_t* const* pre_out, uint32_t* m_r8, uint32_t table_len, uint64_t* off_table) {
    std::vector<const int8_t*> w(qw, qw + n_mats);
    std::vector<uint32_t> no(n_out, n_out + n_mats);
    FreivaldsColumns fc = freivalds_columns(qx, w, no, Grid{log_rows, groups, chunks, lead}, pq, pk, n_in, tokens, table_len);
    size_t rows = (size_t)1 << log_rows;
    for (size_t c = 0; c < fc.base.size(); c++) for (size_t i = 0; i < rows; i++) base_out[c][i] = fc.base[c][i].v;
    for (size_t c = 0; c < fc.pre.size(); c++) for (size_t i = 0; i < rows; i++) pre_out[c][i] = fc.pre[c][i].v;
    for (size_t i = 0; i < table_len; i++) m_r8[i] = fc.m_r8[i];
    *off_table = fc.off_table;
}

// out: (1 + 2 n_mats) * 4 columns; claims: n_mats * 4 words.
void zko_freivalds_acc(const uint32_t* const* base, const uint32_t* const* pre, uint32_t n_mats, uint32_t log_rows, uint32_t groups,
                       uint32_t chunks, uint32_t lead, uint32_t pq, uint32_t pk, const uint32_t* s4, const uint32_t* rv4,
                       uint32_t* const* out, uint32_t* claims) {
    size_t rows = (size_t)1 << log_rows;
    std::vector<std::vector<M31>> b(pq, std::vector<M31>(rows)), p(n_mats * pk, std::vector<M31>(rows));
    for (uint32_t c = 0; c < pq; c++) for (size_t i = 0; i < rows; i++) b[c][i] = M31(base[c][i]);
    for (uint32_t c = 0; c < n_mats * pk; c++) for (size_t i = 0; i < rows; i++) p[c][i] = M31(pre[c][i]);
    std::vector<std::vector<M31>> cols;
    std::vector<QM31> cl;
    freivalds_accumulators(b, p, Grid{log_rows, groups, chunks, lead}, pq, pk, n_mats, q_from(s4), q_from(rv4), cols, cl);
    for (size_t c = 0; c < cols.size(); c++) for (size_t i = 0; i < rows; i++) out[c][i] = cols[c][i].v;
    for (size_t m = 0; m < cl.size(); m++) q_to(cl[m], claims + 4 * m);
}

}  // extern "C"

// ---------------------------------------------------------------- witness generation: tables, dequantize
#include "witness.hpp"
extern "C" {

void zko_witness_tables(const uint32_t* expmap, const uint32_t* const* counters, uint32_t n_counters, const uint32_t* patch_idx,
                        const uint32_t* patch_val, uint32_t n_patch, uint32_t log_rows, int bf16x, double two_pow, uint32_t* x, uint32_t* y,
                        uint32_t* m) {
    std::vector<const uint32_t*> cn(counters, counters + n_counters);
    TableColumns t = witness_tables(expmap, cn, patch_idx, patch_val, n_patch, log_rows, bf16x != 0, two_pow);
    size_t rows = (size_t)1 << log_rows;
    std::memcpy(x, t.x.data(), rows * 4);
    std::memcpy(y, t.y.data(), rows * 4);
    std::memcpy(m, t.m.data(), rows * 4);
}

// cfg34: the 34 words of DequantCfg in declaration order. want: rows * per_row words.
void zko_witness_dequant(const int32_t* acc, const int32_t* jx, const int32_t* jw, const uint32_t* sx, const uint32_t* sw, const uint32_t* norm3,
                         const uint32_t* mul2, uint32_t* const* base_out, uint32_t n_base, uint32_t* const* pre_out, uint32_t n_pre,
                         uint32_t* m_norm, uint32_t* m_frac, uint32_t* m_mul, uint32_t* m_r8, uint32_t* counts, uint32_t* want,
                         const uint32_t* cfg34) {
    static_assert(sizeof(DequantCfg) == 34 * 4, "DequantCfg layout");
    DequantCfg c;
    std::memcpy(&c, cfg34, sizeof c);
    DequantOut o = witness_dequant(acc, jx, jw, sx, sw, norm3, mul2, n_base, n_pre, c);
    size_t rows = (size_t)1 << c.log_rows;
    for (uint32_t k = 0; k < n_base; k++) std::memcpy(base_out[k], o.base[k].data(), rows * 4);
    for (uint32_t k = 0; k < n_pre; k++) std::memcpy(pre_out[k], o.pre[k].data(), rows * 4);
    std::memcpy(m_norm, o.m_norm.data(), o.m_norm.size() * 4);
    std::memcpy(m_frac, o.m_frac.data(), o.m_frac.size() * 4);
    if (m_mul) std::memcpy(m_mul, o.m_mul.data(), o.m_mul.size() * 4);
    std::memcpy(m_r8, o.m_r8.data(), o.m_r8.size() * 4);
    std::memcpy(counts, o.counts, 12);
    std::memcpy(want, o.want.data(), o.want.size() * 4);
}

}  // extern "C"

// ---------------------------------------------------------------- witness generation: shared tables, key tile selectors, residual stream
#include "witness_pre.hpp"
extern "C" {

// cols_out: n_cols columns of 2^log_rows words; m_out may be NULL.
void zko_witness_pre_table(uint32_t kind, uint32_t log_rows, uint32_t kmax, uint32_t round, const uint32_t* const* counters, uint32_t n_counters,
                           const uint32_t* patch_idx, const uint32_t* patch_val, uint32_t n_patch, uint32_t* const* cols_out, uint32_t* m_out) {
    std::vector<const uint32_t*> cn(counters, counters + n_counters);
    PreTableOut o = witness_pre_table(kind, log_rows, kmax, round, cn, m_out != nullptr, patch_idx, patch_val, n_patch);
    size_t rows = (size_t)1 << log_rows;
    for (size_t k = 0; k < o.cols.size(); k++) std::memcpy(cols_out[k], o.cols[k].data(), rows * 4);
    if (m_out) std::memcpy(m_out, o.m.data(), rows * 4);
}

void zko_key_tile_flags(uint32_t shape, uint32_t log_rows, uint32_t groups, uint32_t chunks, uint32_t lead, uint32_t descending, uint32_t modulus,
                        uint32_t rw, uint32_t* flags) {
    auto f = key_tile_flags(shape, KtGrid{log_rows, groups, chunks, lead, descending}, modulus, rw);
    std::memcpy(flags, f.data(), f.size() * 4);
}

void zko_witness_selectors(uint32_t shape, uint32_t log_rows, uint32_t groups, uint32_t chunks, uint32_t lead, uint32_t descending,
                           const uint32_t* flags, const uint32_t* scale, uint32_t ctx_len, int with_scale, uint32_t* const* cols_out, uint32_t n_cols) {
    size_t rows = (size_t)1 << log_rows;
    std::vector<uint32_t> f(flags, flags + rows);
    auto cols = witness_selectors(shape, KtGrid{log_rows, groups, chunks, lead, descending}, f, scale, ctx_len, with_scale != 0, n_cols);
    for (uint32_t k = 0; k < n_cols; k++) std::memcpy(cols_out[k], cols[k].data(), rows * 4);
}

// groups: n_groups x (n, un). slots: n_slots x (kind, g, i, kind, g, i) with kind 0 zero, 1 leaf (g, i), 2 unary image (g, i), 3 slot g.
// m_len: lengths of the multiplicity arrays pow, norm, val, frac, smul, un; m_out: pointers in the same order, the unary ones appended.
uint32_t zko_rs_n_cols(const uint32_t* groups, uint32_t n_groups, uint32_t n_slots, uint32_t kind, uint32_t sticky) {
    RsProg p;
    for (uint32_t g = 0; g < n_groups; g++) p.groups.push_back({groups[2 * g], groups[2 * g + 1]});
    p.kind = kind; p.sticky = sticky != 0; p.slots.resize(n_slots);
    return (uint32_t)p.n_cols();
}
void zko_witness_residual_stream(const uint32_t* groups, uint32_t n_groups, const uint32_t* slots, uint32_t n_slots, const uint32_t* out_slot,
                                 uint32_t out_w, uint32_t kind, uint32_t sticky, uint32_t kmax, const uint32_t* norm3, uint32_t n_norm,
                                 const int32_t* smul3, uint32_t n_smul, const int32_t* const* un2, uint32_t n_un, uint32_t n_val,
                                 const uint32_t* wit, uint32_t live_rows, uint32_t log_rows, const uint64_t* m_len, uint32_t* const* cols_out,
                                 uint32_t* out_pat, int32_t* out_nat, int32_t* in_nat, uint32_t* const* m_out, uint32_t* counts) {
    RsProg p;
    for (uint32_t g = 0; g < n_groups; g++) p.groups.push_back({groups[2 * g], groups[2 * g + 1]});
    p.kind = kind; p.sticky = sticky != 0; p.kmax = kmax;
    for (uint32_t s = 0; s < n_slots; s++) {
        const uint32_t* w = slots + 6 * s;
        p.slots.push_back({RsSrc{w[0], w[1], w[2]}, RsSrc{w[3], w[4], w[5]}});
    }
    p.out_slot.assign(out_slot, out_slot + out_w);
    RsTables t{norm3, n_norm, smul3, n_smul, std::vector<const int32_t*>(un2, un2 + n_un), n_val};
    size_t ml[6];
    for (int k = 0; k < 6; k++) ml[k] = (size_t)m_len[k];
    RsOut o = witness_residual_stream(p, t, wit, live_rows, log_rows, ml);
    size_t rows = (size_t)1 << log_rows;
    for (size_t k = 0; k < o.cols.size(); k++) std::memcpy(cols_out[k], o.cols[k].data(), rows * 4);
    std::memcpy(out_pat, o.out_pat.data(), o.out_pat.size() * 4);
    std::memcpy(out_nat, o.out_nat.data(), o.out_nat.size() * 4);
    std::memcpy(in_nat, o.in_nat.data(), o.in_nat.size() * 4);
    const std::vector<uint32_t>* ms[5] = {&o.m_pow, &o.m_norm, &o.m_val, &o.m_frac, &o.m_smul};
    for (int k = 0; k < 5; k++) std::memcpy(m_out[k], ms[k]->data(), ms[k]->size() * 4);
    for (uint32_t u = 0; u < n_un; u++) std::memcpy(m_out[5 + u], o.m_un[u].data(), o.m_un[u].size() * 4);
    std::memcpy(counts, o.counts, 12);
}

}  // extern "C"

// ---------------------------------------------------------------- constraint quotients of an AIR
#include "air.hpp"
extern "C" {

uint64_t zko_offset_bit_reversed_circle_domain_index(uint64_t i, uint32_t domain_log, uint32_t eval_log, int64_t offset) {
    return offset_bit_reversed_circle_domain_index((size_t)i, domain_log, eval_log, offset);
}

void zko_constraint_denom_inv(uint32_t trace_log, uint32_t eval_log, uint32_t* out) {
    std::vector<M31> d = constraint_denom_inv(trace_log, eval_log);
    for (size_t i = 0; i < d.size(); i++) out[i] = d[i].v;
}

static TraceView trace_view(const uint32_t* tree_cols, int n_trees, const uint32_t* const* cols) {
    TraceView t(n_trees);
    size_t at = 0;
    for (int k = 0; k < n_trees; k++)
        for (uint32_t c = 0; c < tree_cols[k]; c++) t[k].push_back(cols[at++]);
    return t;
}

// The lowered program, row by row (ops: n_ops x 5 words).
void zko_constraint_quotients_ssa(const uint32_t* ops, size_t n_ops, const uint32_t* constraints, size_t n_constraints,
                                  const uint32_t* tree_cols, int n_trees, const uint32_t* const* cols, const uint32_t* scalars,
                                  size_t n_scalars, const uint32_t* cumsum_shift, const uint32_t* rcp, uint32_t trace_log,
                                  uint32_t eval_log, uint32_t* const accum[4], int accumulate) {
    TraceView t = trace_view(tree_cols, n_trees, cols);
    std::vector<QM31> sc(n_scalars), coef(n_constraints);
    for (size_t i = 0; i < n_scalars; i++) sc[i] = q_from(scalars + 4 * i);
    for (size_t i = 0; i < n_constraints; i++) coef[i] = q_from(rcp + 4 * i);
    QM31 shift = cumsum_shift ? q_from(cumsum_shift) : QM31::zero();
    const AirOp* o = reinterpret_cast<const AirOp*>(ops);
    accumulate_pointwise_cpu([&](size_t row) {
        return air_interpret_row(o, n_ops, constraints, n_constraints, t, sc.data(), shift, coef.data(), row, trace_log, eval_log);
    }, eval_log, trace_log, accum, accumulate != 0);
}

// The AIRs written against the evaluators. air: 0 wide Fibonacci (ip = {n_cols}), 1 Plonk (qp = {z, alpha^0, alpha^1}),
// 2 Freivalds (ip = {pk, pq, n_mats, act_off, range_check}; qp = {rv_pow[pk], rv_step, s_pow[pq], s_step, claimed[n_mats], z, alpha^0}).
static AirSpec make_air_spec(int air, const uint32_t* ip, const uint32_t* qp) {
    AirSpec a;
    a.air = air;
    if (air == 0) {
        a.n_cols = ip[0];
    } else if (air == 1) {
        a.plonk_rel.z = q_from(qp);
        a.plonk_rel.alpha_powers = {q_from(qp + 4), q_from(qp + 8)};
    } else {
        FreivaldsEval& fe = a.fe;
        fe.pk = ip[0]; fe.pq = ip[1]; fe.n_mats = ip[2]; fe.act_off = ip[3]; fe.range_check = ip[4] != 0;
        const uint32_t* q = qp;
        for (size_t p = 0; p < fe.pk; p++, q += 4) fe.rv_pow.push_back(q_from(q));
        fe.rv_step = q_from(q); q += 4;
        for (size_t p = 0; p < fe.pq; p++, q += 4) fe.s_pow.push_back(q_from(q));
        fe.s_step = q_from(q); q += 4;
        for (size_t m = 0; m < fe.n_mats; m++, q += 4) fe.claimed.push_back(q_from(q));
        fe.rel_act.z = q_from(q); q += 4;
        fe.rel_act.alpha_powers = {q_from(q)};
    }
    return a;
}

void zko_constraint_quotients_air(int air, const uint32_t* ip, const uint32_t* qp, const uint32_t* tree_cols, int n_trees,
                                  const uint32_t* const* cols, const uint32_t* claimed_sum, const uint32_t* rcp, size_t n_constraints,
                                  uint32_t trace_log, uint32_t eval_log, uint32_t* const accum[4], int accumulate) {
    TraceView t = trace_view(tree_cols, n_trees, cols);
    std::vector<QM31> coef(n_constraints);
    for (size_t i = 0; i < n_constraints; i++) coef[i] = q_from(rcp + 4 * i);
    QM31 claimed = claimed_sum ? q_from(claimed_sum) : QM31::zero();
    AirSpec spec = make_air_spec(air, ip, qp);
    accumulate_pointwise_cpu([&](size_t row) {
        CpuDomainEvaluator eval(t, row, coef.data(), trace_log, eval_log, trace_log, claimed);
        spec.evaluate(eval);
        assert(eval.constraint_index == n_constraints);
        return eval.row_res;
    }, eval_log, trace_log, accum, accumulate != 0);
}

}  // extern "C"

// ---------------------------------------------------------------- a whole STARK proof of one component
#include "stark.hpp"
extern "C" {

// prove() of nitroo/crates/stwo/src/prover/mod.rs:41-173 for n_comp components whose AIRs are among the three above.
// Component k is described by air[k], trace_log[k], its parameter blocks ip + ip_off[k] and qp + 4 * qp_off[k], and
// claimed_sums + 4k. In every tree the columns of component k follow those of the components before it; cols holds the
// traces on their trace domains, trees concatenated. Output: the PCS proof words, the channel digest (8 words), the
// composition polynomial's out-of-domain value from the committed halves (4 words) and from the constraints at the sampled
// mask values (4 words). Returns the word count or -1.
long zko_stark_prove_multi(int n_comp, const int* air, const uint32_t* trace_log, const uint32_t* ip, const uint32_t* ip_off,
                           const uint32_t* qp, const uint32_t* qp_off, const uint32_t* claimed_sums, const uint32_t* tree_cols, int n_trees,
                           const uint32_t* const* cols, const uint32_t* col_logs, uint32_t pow_bits, uint32_t log_blowup,
                           uint32_t log_last_layer, uint32_t n_queries, uint32_t* out, size_t cap) {
    PcsConfig cfg;
    cfg.pow_bits = pow_bits;
    cfg.fri = {log_blowup, log_last_layer, n_queries, 1};
    std::vector<StarkComponent> comps;
    for (int k = 0; k < n_comp; k++)
        comps.push_back({make_air_spec(air[k], ip + ip_off[k], qp + 4 * (size_t)qp_off[k]), trace_log[k], q_from(claimed_sums + 4 * k)});
    std::vector<std::vector<std::vector<M31>>> trees(n_trees);
    size_t at = 0;
    for (int t = 0; t < n_trees; t++)
        for (uint32_t c = 0; c < tree_cols[t]; c++, at++) {
            std::vector<M31> v((size_t)1 << col_logs[at]);
            for (size_t i = 0; i < v.size(); i++) v[i] = M31(cols[at][i]);
            trees[t].push_back(std::move(v));
        }
    StarkResult r = stark_prove_multi(comps, trees, cfg);
    std::vector<uint32_t> w = r.proof.to_words();
    for (int i = 0; i < 8; i++) w.push_back(load_le32(&r.digest[4 * i]));
    uint32_t q[4];
    r.committed_eval.to_u32(q);
    w.insert(w.end(), q, q + 4);
    r.point_eval.to_u32(q);
    w.insert(w.end(), q, q + 4);
    if (w.size() > cap) return -1;
    memcpy(out, w.data(), w.size() * 4);
    return (long)w.size();
}

}  // extern "C"
