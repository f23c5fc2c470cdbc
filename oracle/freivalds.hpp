// TEST INFRASTRUCTURE ONLY (CPU oracle; see fields.hpp).
//
// The Freivalds attention-witness component: column construction and the Horner accumulators,
// restated from the reference's host code.
//   prover/src/layout.rs:141-183                         (Grid, Grid::row)
//   prover/src/common.rs:76-80, 100-139                  (coset_perm, eval_of)
//   prover/src/gadgets/freivalds/trace.rs:43-162         (base / pre columns, selectors, range bumps)
//   prover/src/gadgets/freivalds/claims.rs:37-109        (inner sums, v / us / accs, claims)
//   prover/src/encoding.rs:29-32, 86-91                  (m31_of, secure_cols)
//   prover/src/layer.rs:2071-2077                        (bump)
#pragma once
#include "fields.hpp"

namespace zko {

struct Grid {  // layout.rs:141-183, descending = true
    uint32_t log_rows, groups, chunks, lead;
    size_t rows() const { return (size_t)1 << log_rows; }
    // (group, chunk) of coset-order row j, or false for an inert row
    bool row(size_t j, size_t& g, size_t& chunk) const {
        if (j < lead) return false;
        size_t idx = j - lead;
        g = groups - 1 - idx / chunks;
        chunk = chunks - 1 - (idx % chunks);
        return true;
    }
};

// common.rs:76-80
inline size_t coset_perm(size_t i, uint32_t log_n) {
    size_t n = (size_t)1 << log_n;
    size_t c = (i % 2 == 0) ? i / 2 : (2 * n - i - 1) / 2;
    size_t r = 0;
    for (uint32_t b = 0; b < log_n; b++) r |= ((c >> b) & 1) << (log_n - 1 - b);
    return r;
}
// common.rs:100-139: committed[i] = coset_order[coset_perm(i)]
template <class T> inline std::vector<T> eval_of(uint32_t log_n, const std::vector<T>& coset_order) {
    std::vector<T> out(coset_order.size());
    for (size_t i = 0; i < out.size(); i++) out[i] = coset_order[coset_perm(i, log_n)];
    return out;
}
inline M31 m31_of(int64_t v) { int64_t p = P; return M31((uint32_t)(((v % p) + p) % p)); }  // encoding.rs:29-32

struct FreivaldsColumns {
    std::vector<std::vector<M31>> base, pre;  // committed order
    std::vector<uint32_t> m_r8;               // range multiplicities added by this component
    size_t off_table = 0;
};

// trace.rs:43-162 with act_bits = 8 (offset 128); qw[m] is [n_in][n_out[m]] row-major, qx is [tokens][n_in].
inline FreivaldsColumns freivalds_columns(const int8_t* qx, const std::vector<const int8_t*>& qw, const std::vector<uint32_t>& n_out,
                                          Grid g, uint32_t pq, uint32_t pk, uint32_t n_in, uint32_t tokens, size_t table_len) {
    FreivaldsColumns fc;
    fc.m_r8.assign(table_len, 0);
    size_t rows = g.rows();
    const int off = 128;
    for (uint32_t p = 0; p < pq; p++) {
        std::vector<M31> col(rows);
        for (size_t j = 0; j < rows; j++) {
            size_t k, chunk;
            int v = off;
            if (g.row(j, k, chunk)) {
                size_t t = chunk * pq + p;
                if (t < tokens) v = (int)qx[t * n_in + k] + off;
            }
            if (v >= 0 && (size_t)v < table_len) fc.m_r8[v]++; else fc.off_table++;
            col[j] = m31_of(v);
        }
        fc.base.push_back(eval_of(g.log_rows, col));
    }
    for (size_t m = 0; m < qw.size(); m++)
        for (uint32_t p = 0; p < pk; p++) {
            std::vector<M31> col(rows);
            for (size_t j = 0; j < rows; j++) {
                size_t k, chunk;
                if (g.row(j, k, chunk)) {
                    size_t i = chunk * pk + p;
                    if (i < n_out[m]) col[j] = m31_of(qw[m][k * n_out[m] + i]);
                }
            }
            fc.pre.push_back(eval_of(g.log_rows, col));
        }
    auto sel = [&](auto f) {
        std::vector<M31> col(rows);
        for (size_t j = 0; j < rows; j++) col[j] = M31(f(j) ? 1u : 0u);
        fc.pre.push_back(eval_of(g.log_rows, col));
    };
    auto chunk_of = [&](size_t j, size_t& c) { size_t k; return g.row(j, k, c); };
    sel([&](size_t j) { size_t c; return chunk_of(j, c) && c + 1 < g.chunks; });
    sel([&](size_t j) { size_t c; return chunk_of(j, c) && c == 0; });
    sel([&](size_t j) { return j > 0; });
    sel([&](size_t j) { return j + 1 == rows; });
    return fc;
}

// claims.rs:37-109 from the committed columns: v, then us[m] and accs[m] per matmul, each as four
// coordinate columns in committed order (secure_cols, encoding.rs:86-91); claims = accs[m][rows-1].
inline void freivalds_accumulators(const std::vector<std::vector<M31>>& base, const std::vector<std::vector<M31>>& pre, Grid g,
                                   uint32_t pq, uint32_t pk, uint32_t n_mats, QM31 s_ch, QM31 rv,
                                   std::vector<std::vector<M31>>& out_cols, std::vector<QM31>& claims) {
    size_t rows = g.rows();
    std::vector<QM31> s_pow, rv_pow;
    QM31 cur = QM31::one();
    for (uint32_t p = 0; p < pq; p++) { s_pow.push_back(cur); cur = cur * s_ch; }
    QM31 s_step = cur;
    cur = QM31::one();
    for (uint32_t p = 0; p < pk; p++) { rv_pow.push_back(cur); cur = cur * rv; }
    QM31 rv_step = cur;
    std::vector<QM31> v(rows);
    std::vector<std::vector<QM31>> us(n_mats, std::vector<QM31>(rows)), accs(n_mats, std::vector<QM31>(rows));
    const M31 off = m31_of(128);
    for (size_t j = 0; j < rows; j++) {
        size_t i = coset_perm(j, g.log_rows);  // an involution: row j sits at committed index coset_perm(j)
        size_t k, chunk;
        bool some = g.row(j, k, chunk);
        QM31 vf = QM31::zero();
        std::vector<QM31> ufs(n_mats, QM31::zero());
        if (some) {
            for (uint32_t p = 0; p < pq; p++) vf = vf + s_pow[p] * (base[p][i] - off);
            for (uint32_t m = 0; m < n_mats; m++)
                for (uint32_t p = 0; p < pk; p++) ufs[m] = ufs[m] + rv_pow[p] * pre[m * pk + p][i];
        }
        bool nofirst = some && chunk + 1 < g.chunks, last = some && chunk == 0;
        v[j] = (nofirst ? v[j - 1] * s_step : QM31::zero()) + vf;
        for (uint32_t m = 0; m < n_mats; m++) {
            us[m][j] = (nofirst ? us[m][j - 1] * rv_step : QM31::zero()) + ufs[m];
            accs[m][j] = j > 0 ? accs[m][j - 1] : QM31::zero();
            if (last) accs[m][j] = accs[m][j] + us[m][j] * v[j];
        }
    }
    auto push_secure = [&](const std::vector<QM31>& vals) {
        for (int c = 0; c < 4; c++) {
            std::vector<M31> col(rows);
            for (size_t j = 0; j < rows; j++) { uint32_t w[4]; vals[j].to_u32(w); col[j] = M31(w[c]); }
            out_cols.push_back(eval_of(g.log_rows, col));
        }
    };
    push_secure(v);
    for (uint32_t m = 0; m < n_mats; m++) { push_secure(us[m]); push_secure(accs[m]); }
    for (uint32_t m = 0; m < n_mats; m++) claims.push_back(accs[m][rows - 1]);
}

}  // namespace zko
