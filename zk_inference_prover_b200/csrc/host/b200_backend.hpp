// Host-side mirror of the reference's operator traits over the C ABI (include/zkb200.h).
//
// The reference selects a backend with a type (`PcsB`, prover/src/common.rs:163-166) whose
// associated functions implement the traits of nitroo/crates/stwo/src/prover/backend/mod.rs:20-92.
// `B200Backend` has one static function per trait method, with the trait's name and argument
// meaning; columns own their device buffers and free them on destruction, as the reference's
// device vectors do (stwo_cuda/base_field_vec.rs:7-60). Precondition failures throw (the
// reference's backends panic); nothing here falls back to host arithmetic.
#pragma once
#include <array>
#include <cstdint>
#include <cstring>
#include <exception>
#include <memory>
#include <stdexcept>
#include <string>
#include <thread>
#include <utility>
#include <vector>

#include "../../../include/zkb200.h"
#include "../m31.cuh"

namespace b200 {

using zk::cm31;
using zk::qm31;
using SecureField = zk::qm31;

struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};

struct CirclePointQ { qm31 x, y; };
inline bool operator==(const qm31& a, const qm31& b) { return zk::qm31_eq(a, b); }
inline bool operator==(const CirclePointQ& a, const CirclePointQ& b) { return a.x == b.x && a.y == b.y; }

// The context every column and operator call of one prover uses.
class Device {
  public:
    explicit Device(zkb_ctx* c) : ctx_(c) {}
    zkb_ctx* ctx() const { return ctx_; }
    void check(int rc) const {
        if (rc != ZKB_OK) throw Error(rc, std::string("zkb200: ") + zkb_last_error(ctx_));
    }
  private:
    zkb_ctx* ctx_;
};

// Col<B, BaseField>: `len` M31 words on the device.
class BaseColumn {
  public:
    BaseColumn() = default;
    BaseColumn(const Device& d, size_t len, bool zero = false) : dev_(&d), len_(len) {
        void* p = nullptr;
        d.check(zkb_malloc(d.ctx(), len * 4, &p));
        ptr_ = (uint32_t*)p;
        if (zero && len) d.check(zkb_memset_zero(d.ctx(), ptr_, len * 4));
    }
    BaseColumn(const Device& d, const uint32_t* host, size_t len) : BaseColumn(d, len) {
        d.check(zkb_h2d(d.ctx(), ptr_, host, len * 4));
    }
    // A column over memory the caller owns (never freed here).
    static BaseColumn view(const Device& d, uint32_t* ptr, size_t len) {
        BaseColumn c;
        c.dev_ = &d; c.ptr_ = ptr; c.len_ = len; c.owned_ = false;
        return c;
    }
    BaseColumn(BaseColumn&& o) noexcept { *this = std::move(o); }
    BaseColumn& operator=(BaseColumn&& o) noexcept {
        if (this != &o) {
            release();
            dev_ = o.dev_; ptr_ = o.ptr_; len_ = o.len_; owned_ = o.owned_;
            o.ptr_ = nullptr; o.len_ = 0;
        }
        return *this;
    }
    BaseColumn(const BaseColumn&) = delete;
    BaseColumn& operator=(const BaseColumn&) = delete;
    ~BaseColumn() { release(); }
    uint32_t* ptr() const { return ptr_; }
    size_t len() const { return len_; }
    void shrink(size_t len) { if (len < len_) len_ = len; }  // keeps the allocation, forgets the tail
    uint32_t log_size() const { return len_ ? 63u - (uint32_t)__builtin_clzll((unsigned long long)len_) : 0u; }
    std::vector<uint32_t> to_cpu() const {
        std::vector<uint32_t> v(len_);
        if (len_) dev_->check(zkb_d2h(dev_->ctx(), v.data(), ptr_, len_ * 4));
        return v;
    }
  private:
    void release() {
        if (ptr_ && owned_) zkb_free(dev_->ctx(), ptr_);
        ptr_ = nullptr;
    }
    const Device* dev_ = nullptr;
    uint32_t* ptr_ = nullptr;
    size_t len_ = 0;
    bool owned_ = true;
};

// SecureColumnByCoords<B> (prover/secure_column.rs:13-15).
struct SecureColumnByCoords {
    BaseColumn columns[4];
    SecureColumnByCoords() = default;
    SecureColumnByCoords(const Device& d, size_t len, bool zero = false) {
        for (auto& c : columns) c = BaseColumn(d, len, zero);
    }
    size_t len() const { return columns[0].len(); }
    std::array<uint32_t*, 4> ptrs() const { return {columns[0].ptr(), columns[1].ptr(), columns[2].ptr(), columns[3].ptr()}; }
    std::array<const uint32_t*, 4> cptrs() const { return {columns[0].ptr(), columns[1].ptr(), columns[2].ptr(), columns[3].ptr()}; }
    std::vector<const BaseColumn*> refs() const { return {&columns[0], &columns[1], &columns[2], &columns[3]}; }
};

// Col<B, Blake2sHash>: 8 words per node.
using HashColumn = BaseColumn;
using Hash = std::array<uint32_t, 8>;

// Mle<B, SecureField>: QM31 stored as 4 consecutive words. `len` counts field elements.
struct SecureMle {
    BaseColumn words;
    SecureMle() = default;
    SecureMle(const Device& d, size_t len) : words(d, 4 * len) {}
    size_t len() const { return words.len() / 4; }
};

// ---- quotient inputs (core/pcs/quotients.rs:58-104)
struct PointSample { CirclePointQ point; qm31 value; };
struct NumeratorData { size_t column_index; qm31 sample_value; qm31 random_coeff; };
struct ColumnSampleBatch { CirclePointQ point; std::vector<NumeratorData> cols_vals_randpows; };
struct AccumulatedNumerators {
    CirclePointQ sample_point;
    SecureColumnByCoords partial_numerators_acc;
    qm31 first_linear_term_acc;
};

// ---- GKR layer (prover/lookups/gkr_prover.rs:262-280)
struct Layer {
    int kind = ZKB_GKR_GRAND_PRODUCT;
    SecureMle num;      // LOGUP_GENERIC numerators
    BaseColumn num_base;  // LOGUP_MULTIPLICITIES numerators
    SecureMle den;      // denominators, or the grand-product column
    bool writable = false;  // the arrays are the prover's own scratch (a tower layer, a fixed layer): they may be overwritten
    size_t len() const { return den.len(); }
    size_t n_variables() const { size_t l = 0; while (((size_t)1 << (l + 1)) <= len()) l++; return l; }
    const uint32_t* num_ptr() const {
        return kind == ZKB_GKR_LOGUP_GENERIC ? num.words.ptr() : kind == ZKB_GKR_LOGUP_MULTIPLICITIES ? num_base.ptr() : nullptr;
    }
};

// f(begin, end, chunk) over [0, n) on up to four host threads (the caller's among them; chunk = 0 ... 3) when every thread
// gets at least `min_per_thread` items: the per-column arithmetic of a proof over tens of thousands of columns (powers of
// the random coefficient, line coefficients) is independent per item. An exception of any chunk is rethrown on the caller's
// thread after all chunks have ended.
template <class F>
inline void parallel_chunks(size_t n, size_t min_per_thread, F f) {
    size_t nt = min_per_thread ? n / min_per_thread : 1;
    if (nt > 4) nt = 4;
    if (nt <= 1) { f((size_t)0, n, (size_t)0); return; }
    const size_t per = (n + nt - 1) / nt;
    std::exception_ptr failed[4];
    auto run = [&](size_t t) {
        try { f(t * per < n ? t * per : n, (t + 1) * per < n ? (t + 1) * per : n, t); } catch (...) { failed[t] = std::current_exception(); }
    };
    std::thread th[3];
    for (size_t t = 1; t < nt; t++) th[t - 1] = std::thread(run, t);
    run(0);
    for (size_t t = 1; t < nt; t++) th[t - 1].join();
    for (size_t t = 0; t < nt; t++)
        if (failed[t]) std::rethrow_exception(failed[t]);
}

// complex_conjugate_line_coeffs (core/constraints.rs:119-134): (alpha a, alpha b, alpha c).
struct LineCoeffs { qm31 a, b, c; };
inline qm31 conj(qm31 v) { return {{v.c[0], v.c[1], zk::m31_neg(v.c[2]), zk::m31_neg(v.c[3])}}; }
inline LineCoeffs complex_conjugate_line_coeffs(const PointSample& s, qm31 alpha) {
    qm31 a = zk::qm31_sub(conj(s.value), s.value);
    qm31 c = zk::qm31_sub(conj(s.point.y), s.point.y);
    if (zk::qm31_is_zero(c)) throw Error(ZKB_EINVAL, "sample point lies on the base-field circle");
    qm31 b = zk::qm31_sub(zk::qm31_mul(s.value, c), zk::qm31_mul(a, s.point.y));
    return {zk::qm31_mul(alpha, a), zk::qm31_mul(alpha, b), zk::qm31_mul(alpha, c)};
}

struct B200Backend {
    // ---- ColumnOps (backend/mod.rs:39-42)
    static void bit_reverse_column(const Device& d, BaseColumn& col) {
        d.check(zkb_bit_reverse_m31(d.ctx(), col.ptr(), (int)col.log_size()));
    }
    // Column::batch_at_multi (backend/mod.rs:74-89): row-major [index][column].
    static std::vector<uint32_t> batch_at_multi(const Device& d, const std::vector<const BaseColumn*>& cols,
                                                const std::vector<size_t>& indices) {
        std::vector<uint32_t> out(cols.size() * indices.size());
        if (out.empty()) return out;
        std::vector<const uint32_t*> p;
        for (auto c : cols) p.push_back(c->ptr());
        std::vector<uint32_t> idx(indices.begin(), indices.end());
        d.check(zkb_gather_multi(d.ctx(), p.data(), (int)p.size(), idx.data(), (int)idx.size(), out.data()));
        return out;
    }
    static std::vector<Hash> batch_at(const Device& d, const HashColumn& hashes, const std::vector<size_t>& indices) {
        std::vector<Hash> out(indices.size());
        if (out.empty()) return out;
        std::vector<uint32_t> idx(indices.begin(), indices.end());
        d.check(zkb_gather_hashes(d.ctx(), hashes.ptr(), idx.data(), (int)idx.size(), (uint32_t*)out.data()));
        return out;
    }

    // ---- PolyOps (prover/poly/circle/ops.rs:16-145). Columns of one call share a size.
    static void interpolate_columns(const Device& d, const std::vector<BaseColumn*>& cols) {
        if (cols.empty()) return;
        std::vector<uint32_t*> p;
        for (auto c : cols) p.push_back(c->ptr());
        d.check(zkb_ifft_cols(d.ctx(), p.data(), (int)p.size(), (int)cols[0]->log_size()));
    }
    // With `slab`, the extended columns are views of ONE allocation that *slab then owns (a tree of tens of thousands of
    // short columns would otherwise spend its time in the allocator).
    static std::vector<BaseColumn> evaluate_polynomials(const Device& d, const std::vector<const BaseColumn*>& coeffs,
                                                        uint32_t log_blowup_factor, BaseColumn* slab = nullptr) {
        std::vector<BaseColumn> out;
        if (coeffs.empty()) return out;
        uint32_t log_n = coeffs[0]->log_size(), log_out = log_n + log_blowup_factor;
        std::vector<const uint32_t*> src;
        std::vector<uint32_t*> dst;
        if (slab && coeffs.size() > 1 && log_out >= 2) *slab = BaseColumn(d, coeffs.size() << log_out);
        else slab = nullptr;
        for (size_t i = 0; i < coeffs.size(); i++) {
            if (slab) out.push_back(BaseColumn::view(d, slab->ptr() + (i << log_out), (size_t)1 << log_out));
            else out.emplace_back(d, (size_t)1 << log_out);
            src.push_back(coeffs[i]->ptr());
        }
        for (auto& o : out) dst.push_back(o.ptr());
        d.check(zkb_lde_cols(d.ctx(), src.data(), (int)src.size(), (int)log_n, dst.data(), (int)log_out));
        return out;
    }
    static std::vector<qm31> batch_eval_at_point(const Device& d, const std::vector<const BaseColumn*>& coeffs, CirclePointQ point) {
        std::vector<qm31> out(coeffs.size());
        if (coeffs.empty()) return out;
        std::vector<const uint32_t*> src;
        for (auto c : coeffs) src.push_back(c->ptr());
        uint32_t pt[8];
        for (int k = 0; k < 4; k++) { pt[k] = point.x.c[k]; pt[4 + k] = point.y.c[k]; }
        d.check(zkb_eval_at_point_cols(d.ctx(), src.data(), (int)src.size(), (int)coeffs[0]->log_size(), pt, (uint32_t*)out.data()));
        return out;
    }

    // ---- MerkleOps::commit_on_layer (prover/vcs/ops.rs:24-29), Blake2sM31 hasher
    static HashColumn commit_on_layer(const Device& d, uint32_t log_size, const HashColumn* prev_layer,
                                      const std::vector<const BaseColumn*>& columns) {
        HashColumn out(d, (size_t)8 << log_size);
        std::vector<const uint32_t*> p;
        for (auto c : columns) p.push_back(c->ptr());
        d.check(zkb_merkle_layer(d.ctx(), (int)log_size, prev_layer ? prev_layer->ptr() : nullptr, p.data(), (int)p.size(), 1, out.ptr()));
        return out;
    }

    // ---- FriOps (prover/fri.rs:37-85)
    static SecureColumnByCoords fold_line(const Device& d, const SecureColumnByCoords& eval, qm31 alpha) {
        uint32_t log_n = eval.columns[0].log_size();
        SecureColumnByCoords out(d, eval.len() / 2);
        auto o = out.ptrs();
        auto i = eval.cptrs();
        d.check(zkb_fold_line(d.ctx(), o.data(), i.data(), (int)log_n, alpha.c));
        return out;
    }
    // The same folds with the challenge in device memory (see zkb_channel_mix_root_draw).
    static SecureColumnByCoords fold_line(const Device& d, const SecureColumnByCoords& eval, const uint32_t* d_alpha) {
        uint32_t log_n = eval.columns[0].log_size();
        SecureColumnByCoords out(d, eval.len() / 2);
        auto o = out.ptrs();
        auto i = eval.cptrs();
        d.check(zkb_fold_line_dalpha(d.ctx(), o.data(), i.data(), (int)log_n, d_alpha));
        return out;
    }
    static void fold_circle_into_line(const Device& d, SecureColumnByCoords& dst, const SecureColumnByCoords& src, const uint32_t* d_alpha,
                                      HashColumn* leaves = nullptr) {
        auto o = dst.ptrs();
        auto i = src.cptrs();
        if (leaves) {
            *leaves = HashColumn(d, 8 * dst.len());
            d.check(zkb_fold_circle_into_line_dalpha_leaves(d.ctx(), o.data(), i.data(), (int)src.columns[0].log_size(), d_alpha, leaves->ptr()));
        } else {
            d.check(zkb_fold_circle_into_line_dalpha(d.ctx(), o.data(), i.data(), (int)src.columns[0].log_size(), d_alpha));
        }
    }
    // fold_line that also hashes the folded layer's Merkle leaves (the layer's four columns are its coordinates)
    static SecureColumnByCoords fold_line(const Device& d, const SecureColumnByCoords& eval, const uint32_t* d_alpha, HashColumn& leaves) {
        uint32_t log_n = eval.columns[0].log_size();
        SecureColumnByCoords out(d, eval.len() / 2);
        leaves = HashColumn(d, 8 * (eval.len() / 2));
        auto o = out.ptrs();
        auto i = eval.cptrs();
        d.check(zkb_fold_line_dalpha_leaves(d.ctx(), o.data(), i.data(), (int)log_n, d_alpha, leaves.ptr()));
        return out;
    }
    static void fold_circle_into_line(const Device& d, SecureColumnByCoords& dst, const SecureColumnByCoords& src, qm31 alpha) {
        auto o = dst.ptrs();
        auto i = src.cptrs();
        d.check(zkb_fold_circle_into_line(d.ctx(), o.data(), i.data(), (int)src.columns[0].log_size(), alpha.c));
    }

    // ---- QuotientOps (prover/pcs/quotient_ops.rs:19-43)
    static void accumulate_numerators(const Device& d, const std::vector<const BaseColumn*>& columns,
                                      const std::vector<ColumnSampleBatch>& sample_batches,
                                      std::vector<AccumulatedNumerators>& accumulated_numerators_vec) {
        uint32_t log_n = columns[0]->log_size();
        std::vector<const uint32_t*> p;
        p.reserve(columns.size());
        for (auto c : columns) p.push_back(c->ptr());
        for (auto& batch : sample_batches) {
            const size_t ns = batch.cols_vals_randpows.size();
            std::vector<uint32_t> idx(ns), b(4 * ns), c(4 * ns);
            qm31 firsts[4] = {zk::qm31_zero(), zk::qm31_zero(), zk::qm31_zero(), zk::qm31_zero()};
            parallel_chunks(ns, 4096, [&](size_t lo, size_t hi, size_t chunk) {
                qm31 acc = zk::qm31_zero();
                for (size_t i = lo; i < hi; i++) {
                    const auto& nd = batch.cols_vals_randpows[i];
                    LineCoeffs lc = complex_conjugate_line_coeffs({batch.point, nd.sample_value}, nd.random_coeff);
                    idx[i] = (uint32_t)nd.column_index;
                    memcpy(&b[4 * i], lc.b.c, 16);
                    memcpy(&c[4 * i], lc.c.c, 16);
                    acc = zk::qm31_add(acc, lc.a);
                }
                firsts[chunk] = acc;
            });
            qm31 first = zk::qm31_add(zk::qm31_add(firsts[0], firsts[1]), zk::qm31_add(firsts[2], firsts[3]));
            SecureColumnByCoords acc(d, (size_t)1 << log_n);
            auto o = acc.ptrs();
            d.check(zkb_quot_numerators(d.ctx(), p.data(), (int)p.size(), (int)log_n, idx.data(), b.data(), c.data(), (int)idx.size(), o.data()));
            accumulated_numerators_vec.push_back({batch.point, std::move(acc), first});
        }
    }
    static SecureColumnByCoords compute_quotients_and_combine(const Device& d, const std::vector<AccumulatedNumerators>& accs,
                                                              uint32_t lifting_log_size) {
        std::vector<const uint32_t*> cols;
        std::vector<int> logs;
        std::vector<uint32_t> first, pts;
        for (auto& a : accs) {
            for (auto p : a.partial_numerators_acc.cptrs()) cols.push_back(p);
            logs.push_back((int)a.partial_numerators_acc.columns[0].log_size());
            first.insert(first.end(), a.first_linear_term_acc.c, a.first_linear_term_acc.c + 4);
            pts.insert(pts.end(), a.sample_point.x.c, a.sample_point.x.c + 4);
            pts.insert(pts.end(), a.sample_point.y.c, a.sample_point.y.c + 4);
        }
        SecureColumnByCoords out(d, (size_t)1 << lifting_log_size);
        auto o = out.ptrs();
        d.check(zkb_quot_combine(d.ctx(), (int)accs.size(), cols.data(), logs.data(), first.data(), pts.data(), (int)lifting_log_size, o.data()));
        return out;
    }

    // ---- AccumulationOps::lift_and_accumulate (prover/air/accumulation.rs:140-145): ascending sizes.
    static SecureColumnByCoords lift_and_accumulate(const Device& d, std::vector<SecureColumnByCoords> cols) {
        if (cols.empty()) throw Error(ZKB_EINVAL, "lift_and_accumulate: no columns");
        for (size_t i = 1; i < cols.size(); i++) {
            auto dst = cols[i].ptrs();
            auto src = cols[i - 1].cptrs();
            d.check(zkb_lift_accumulate(d.ctx(), dst.data(), (int)cols[i].columns[0].log_size(), src.data(), (int)cols[i - 1].columns[0].log_size()));
        }
        return std::move(cols.back());
    }

    // ---- GrindOps::grind (core/proof_of_work.rs:3-7)
    static uint64_t grind(const Device& d, const Hash& prefixed_digest, uint32_t pow_bits) {
        uint64_t nonce = 0;
        d.check(zkb_grind(d.ctx(), prefixed_digest.data(), (int)pow_bits, 1, &nonce));
        return nonce;
    }

    // ---- GkrOps / MleOps (prover/lookups/gkr_prover.rs:172-220, mle.rs:9-14)
    static SecureMle gen_eq_evals(const Device& d, const std::vector<qm31>& y, qm31 v) {
        SecureMle out(d, (size_t)1 << y.size());
        d.check(zkb_gkr_eq_evals(d.ctx(), y.empty() ? nullptr : (const uint32_t*)y.data(), (int)y.size(), v.c, out.words.ptr()));
        return out;
    }
    static Layer next_layer(const Device& d, const Layer& layer) {
        Layer out;
        size_t half = layer.len() / 2;
        out.kind = layer.kind == ZKB_GKR_GRAND_PRODUCT ? ZKB_GKR_GRAND_PRODUCT : ZKB_GKR_LOGUP_GENERIC;
        out.den = SecureMle(d, half);
        if (out.kind == ZKB_GKR_LOGUP_GENERIC) out.num = SecureMle(d, half);
        d.check(zkb_gkr_next_layer(d.ctx(), layer.kind, layer.num_ptr(), layer.den.words.ptr(), layer.len(),
                                   out.kind == ZKB_GKR_LOGUP_GENERIC ? out.num.words.ptr() : nullptr, out.den.words.ptr()));
        return out;
    }
    // The device part of sum_as_poly_in_first_variable: (sum at t=0, sum at t=2), uncorrected.
    static std::pair<qm31, qm31> round_sums(const Device& d, const Layer& layer, const SecureMle& eq_evals, qm31 lambda) {
        uint32_t out[8];
        d.check(zkb_gkr_sum(d.ctx(), layer.kind, layer.num_ptr(), layer.den.words.ptr(), layer.len(), eq_evals.words.ptr(), lambda.c, out));
        return {qm31{{out[0], out[1], out[2], out[3]}}, qm31{{out[4], out[5], out[6], out[7]}}};
    }
    // fix_first_variable fused with the next round's sums (one launch per sum-check round).
    static std::pair<Layer, std::pair<qm31, qm31>> fix_first_variable_and_sum(const Device& d, const Layer& layer, qm31 x0,
                                                                             const SecureMle& eq_evals, qm31 lambda) {
        size_t n = layer.len();
        Layer out;
        out.kind = layer.kind == ZKB_GKR_LOGUP_MULTIPLICITIES ? ZKB_GKR_LOGUP_GENERIC : layer.kind;
        out.den = SecureMle(d, n / 2);
        if (out.kind == ZKB_GKR_LOGUP_GENERIC) out.num = SecureMle(d, n / 2);
        uint32_t s[8];
        d.check(zkb_gkr_fix_and_sum(d.ctx(), layer.kind, layer.num_ptr(), layer.den.words.ptr(), n, x0.c, eq_evals.words.ptr(), lambda.c,
                                    out.kind == ZKB_GKR_LOGUP_GENERIC ? out.num.words.ptr() : nullptr, out.den.words.ptr(), s));
        std::pair<qm31, qm31> sums{qm31{{s[0], s[1], s[2], s[3]}}, qm31{{s[4], s[5], s[6], s[7]}}};
        return std::make_pair(std::move(out), sums);
    }
    // Layer::fix_first_variable (gkr_prover.rs:354-381) over MleOps::fix_first_variable.
    static Layer fix_first_variable(const Device& d, Layer layer, qm31 x0) {
        if (layer.n_variables() == 0) return layer;
        size_t n = layer.len();
        Layer out;
        out.den = SecureMle(d, n / 2);
        d.check(zkb_mle_fix_qm31(d.ctx(), layer.den.words.ptr(), n, x0.c, out.den.words.ptr()));
        switch (layer.kind) {
            case ZKB_GKR_GRAND_PRODUCT: out.kind = ZKB_GKR_GRAND_PRODUCT; break;
            case ZKB_GKR_LOGUP_SINGLES: out.kind = ZKB_GKR_LOGUP_SINGLES; break;
            case ZKB_GKR_LOGUP_GENERIC:
                out.kind = ZKB_GKR_LOGUP_GENERIC;
                out.num = SecureMle(d, n / 2);
                d.check(zkb_mle_fix_qm31(d.ctx(), layer.num.words.ptr(), n, x0.c, out.num.words.ptr()));
                break;
            default:
                out.kind = ZKB_GKR_LOGUP_GENERIC;
                out.num = SecureMle(d, n / 2);
                d.check(zkb_mle_fix_m31(d.ctx(), layer.num_base.ptr(), n, x0.c, out.num.words.ptr()));
        }
        return out;
    }
};

}  // namespace b200
