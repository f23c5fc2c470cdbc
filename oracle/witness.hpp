// TEST INFRASTRUCTURE ONLY (CPU oracle; see fields.hpp).
//
// Witness generation of the shared lookup tables' own columns and of the matmul dequantize component,
// restated from the reference's HOST code: columns are built in natural (coset) order, row by row, and
// then permuted into committed order by eval_of, exactly as the host path does. Plain loops.
//   prover/src/common.rs:76-80, 100-139                      (coset_perm, eval_of)
//   prover/src/bf16.rs:31-43, 161-163, 197-230, 300-316, 374 (to_f32, from_f32, pattern, from_f64_round, normalise, exp_int_table)
//   prover/src/layer.rs:2042-2068, 2071-2077                 (Tables::norm_at, frac_at, bump)
//   prover/src/gadgets/dequant/trace.rs:503-690              (witness_gen_mat_row, pow2 and chain arms)
//   prover/src/encoding.rs:29-32                             (m31_of)
//   prover/src/devtab.rs:200-290                             (what the tables' three columns hold)
// Pinned by the reference's own device kernels for the same columns (zk_witness_gen_tables,
// zk_witness_gen_dequant), compiled unmodified and run on the same inputs by the GPU tests.
#pragma once
#include <cmath>
#include <cstring>

#include "freivalds.hpp"

namespace zko {

inline uint32_t w_m31_of(int64_t v) {  // encoding.rs:29-32
    const int64_t p = 2147483647LL;
    int64_t x = v % p;
    return (uint32_t)(x < 0 ? x + p : x);
}
inline uint32_t w_bf16_pattern(uint32_t sg, uint32_t ef, uint32_t m7) { return ((sg << 15) | (ef << 7) | m7) & 0xffffu; }  // bf16.rs:161-163
inline double w_bf16_to_f64(uint32_t bits) {  // bf16.rs:31-33
    uint32_t u = bits << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return (double)f;
}
inline uint32_t w_bf16_from_f32(float x) {  // bf16.rs:36-43 (finite arguments)
    uint32_t u;
    std::memcpy(&u, &x, 4);
    uint32_t bias = 0x7fffu + ((u >> 16) & 1u);
    return ((u + bias) >> 16) & 0xffffu;
}
inline uint32_t w_bf16_from_f64(double x) {  // bf16.rs:197-230, Round::Even, normal range
    uint64_t u;
    std::memcpy(&u, &x, 8);
    uint32_t sign = (uint32_t)(u >> 63);
    if (x == 0.0) return w_bf16_pattern(sign, 0, 0);
    int e = (int)((u >> 52) & 0x7ff) - 1023;
    uint64_t man = u & ((1ull << 52) - 1);
    uint32_t keep = (uint32_t)(man >> 45), rb = (uint32_t)((man >> 44) & 1), st = (man & ((1ull << 44) - 1)) != 0;
    uint32_t m7 = keep + ((rb && (st || (keep & 1))) ? 1u : 0u);
    if (m7 == 128) { m7 = 0; e += 1; }
    return w_bf16_pattern(sign, (uint32_t)(e + 127), m7);
}

// ---- the tables' columns ------------------------------------------------------------------------
struct TableColumns { std::vector<uint32_t> x, y, m; };
inline TableColumns witness_tables(const uint32_t* expmap, const std::vector<const uint32_t*>& counters, const uint32_t* patch_idx,
                                   const uint32_t* patch_val, uint32_t n_patch, uint32_t log_rows, bool bf16x, double two_pow) {
    size_t rows = (size_t)1 << log_rows;
    std::vector<uint32_t> x(rows), y(rows), m(rows, 0);
    for (size_t d = 0; d < rows; d++) {  // natural order
        x[d] = (uint32_t)d;
        uint32_t pat = bf16x ? (uint32_t)(d & 0xffff) : w_bf16_from_f32((float)(-(double)d / two_pow));
        y[d] = expmap[pat];
        for (const uint32_t* c : counters) m[d] += c[d];
    }
    for (uint32_t t = 0; t < n_patch; t++) y[patch_idx[t]] = patch_val[t];
    return TableColumns{eval_of(log_rows, x), eval_of(log_rows, y), eval_of(log_rows, m)};
}

// ---- the dequantize component ---------------------------------------------------------------------
struct DequantCfg {
    uint32_t variant, sticky, kmax, do_ref, tokens, n_out, per_row, chunks, log_rows, slot0, per_slot, chan_w;
    uint32_t f_acc, f_sg, f_m2, f_ph, f_st, f_r, f_m7, f_ef, f_nz, f_eo, f_mul[6], sh0, sh1, n_norm, n_frac, n_mul, n_r8;
};
struct DequantOut {
    std::vector<std::vector<uint32_t>> base, pre;  // committed order
    std::vector<uint32_t> m_norm, m_frac, m_mul, m_r8, want;
    uint32_t counts[3] = {0, 0, 0};
};

inline bool w_normalise(uint64_t mag, uint32_t kmax, uint32_t& m2, uint32_t& ph, uint32_t& st, uint64_t& r) {  // bf16.rs:300-316
    if (mag == 0) { m2 = ph = st = 0; r = 0; return true; }
    uint32_t bits = 64 - (uint32_t)__builtin_clzll(mag);
    uint32_t k = bits > 9 ? bits - 9 : 0;
    if (k > kmax) return false;
    ph = 1u << k;
    m2 = (uint32_t)(mag >> k);
    r = mag & (((uint64_t)1 << k) - 1);
    st = r != 0;
    return true;
}
inline int64_t w_norm_at(uint32_t m2, uint32_t ph, uint32_t st, uint32_t kmax, bool sticky) {  // layer.rs:2042-2062
    if (m2 == 0 && ph == 0 && st == 0) return 0;
    if (m2 >= 1 && m2 < 256 && ph == 1 && st == 0) return m2;
    if (m2 >= 256 && m2 < 512 && ph && !(ph & (ph - 1))) {
        uint32_t k = 31 - (uint32_t)__builtin_clz(ph);
        if (k > kmax || (st == 1 && !sticky) || st > 1) return -1;
        return 256 + (int64_t)(k * 256 + (m2 - 256)) * (1 + (sticky ? 1 : 0)) + st;
    }
    return -1;
}
inline int64_t w_frac_at(uint32_t ph, uint64_t r) {  // layer.rs:2063-2068
    if (ph == 0) return r == 0 ? 0 : -1;
    return r < ph ? (int64_t)(ph + r) : -1;
}

inline DequantOut witness_dequant(const int32_t* acc, const int32_t* jx, const int32_t* jw, const uint32_t* sx, const uint32_t* sw,
                                  const uint32_t* norm3, const uint32_t* mul2, uint32_t n_base, uint32_t n_pre, const DequantCfg& c) {
    size_t rows = (size_t)1 << c.log_rows;
    DequantOut o;
    std::vector<std::vector<uint32_t>> base(n_base, std::vector<uint32_t>(rows, 0)), pre(n_pre, std::vector<uint32_t>(rows, 0));
    o.m_norm.assign(c.n_norm, 0); o.m_frac.assign(c.n_frac, 0); o.m_mul.assign(c.n_mul, 0); o.m_r8.assign(c.n_r8, 0);
    o.want.assign(rows * c.per_row, 0);
    auto bump = [&](std::vector<uint32_t>& m, int64_t v) {  // layer.rs:2071-2077
        if (v >= 0 && (size_t)v < m.size()) m[v]++; else o.counts[0]++;
    };
    bool chain = c.variant == 1;
    for (size_t j = 0; j < rows; j++) {  // natural order; the layout runs tokens and chunks downwards
        uint32_t t = c.tokens - 1 - (uint32_t)(j / c.chunks), jm = (uint32_t)(j % c.chunks), b = c.chunks - 1 - jm;
        if (chain) { base[c.sh0][j] = sx[2 * t]; base[c.sh1][j] = sx[2 * t + 1]; }
        else base[c.sh0][j] = w_m31_of(jx[t]);
        uint32_t last = jm == c.chunks - 1, sel0 = c.chan_w * c.per_row;
        pre[sel0 + 0][j] = jm != 0;
        pre[sel0 + 1][j] = last;
        pre[sel0 + 2][j] = j > 0 && !last;
        pre[sel0 + 3][j] = j > 0 && last;
        pre[sel0 + 4][j] = j + 1 == rows;
        for (uint32_t s = 0; s < c.per_row; s++) {
            uint32_t ch = b * c.per_row + s, col0 = c.slot0 + s * c.per_slot;
            if (chain) { pre[2 * s][j] = sw[2 * ch]; pre[2 * s + 1][j] = sw[2 * ch + 1]; }
            else pre[s][j] = w_m31_of(jw[ch]);
            int64_t a = acc[(size_t)t * c.n_out + ch];
            base[col0 + c.f_acc][j] = w_m31_of(a);
            uint32_t sg = a < 0;
            uint64_t mag = (uint64_t)(a < 0 ? -a : a);
            uint32_t m2, ph, st;
            uint64_t r;
            if (!w_normalise(mag, c.kmax, m2, ph, st, r)) { o.counts[2]++; continue; }
            if (!c.sticky) st = 0;
            int64_t ri = w_norm_at(m2, ph, st, c.kmax, c.sticky), fi = w_frac_at(ph, r);
            if (ri < 0 || fi < 0 || ri >= (int64_t)c.n_norm || fi >= (int64_t)c.n_frac) { o.counts[2]++; continue; }
            uint32_t n_m7 = norm3[3 * ri], n_ef = norm3[3 * ri + 1], n_nz = norm3[3 * ri + 2];
            o.m_norm[ri]++;
            o.m_frac[fi]++;
            base[col0 + c.f_sg][j] = sg;
            base[col0 + c.f_m2][j] = m2;
            base[col0 + c.f_ph][j] = ph;
            if (c.sticky) base[col0 + c.f_st][j] = st;
            base[col0 + c.f_r][j] = w_m31_of((int64_t)r);
            base[col0 + c.f_m7][j] = n_m7;
            base[col0 + c.f_ef][j] = n_ef;
            base[col0 + c.f_nz][j] = n_nz;
            if (!chain) {
                int64_t jjx = (int64_t)jx[t] + jw[ch];
                int64_t eo = n_nz == 1 ? (int64_t)n_ef + jjx : 0;
                base[col0 + c.f_eo][j] = w_m31_of(eo);
                bump(o.m_r8, eo);
                if (c.do_ref) {
                    uint32_t want = w_bf16_from_f64(std::ldexp((double)a, (int)jjx));  // a * 2^jjx, exact before the one rounding
                    uint32_t got = w_bf16_pattern(sg, (uint32_t)(eo > 0 ? eo : 0), n_m7);
                    if (want != got) o.counts[1]++;
                    o.want[j * c.per_row + s] = want;
                }
            } else {
                uint32_t m_in = n_m7;
                int64_t e_in = n_ef;
                for (int step = 0; step < 2; step++) {
                    uint32_t ms = step ? sw[2 * ch] : sx[2 * t];
                    int64_t es = step ? sw[2 * ch + 1] : sx[2 * t + 1];
                    uint32_t mi = m_in * 128 + ms;
                    if (mi >= c.n_mul) { o.counts[2]++; break; }
                    uint32_t po = 0, ca = 0;
                    if (n_nz == 1) { po = mul2[2 * mi]; ca = mul2[2 * mi + 1]; }
                    int64_t eo = n_nz == 1 ? e_in + es - 127 + ca : 0;
                    base[col0 + c.f_mul[3 * step + 0]][j] = po;
                    base[col0 + c.f_mul[3 * step + 1]][j] = ca;
                    base[col0 + c.f_mul[3 * step + 2]][j] = w_m31_of(eo);
                    if (n_nz == 1) o.m_mul[mi]++;
                    bump(o.m_r8, eo);
                    m_in = po;
                    e_in = eo;
                }
                if (c.do_ref) {
                    double y0 = w_bf16_to_f64(w_bf16_from_f64((double)(int64_t)mag));
                    double t1 = w_bf16_to_f64(w_bf16_from_f64(y0 * w_bf16_to_f64(w_bf16_pattern(0, sx[2 * t + 1], sx[2 * t]))));
                    uint32_t want = w_bf16_from_f64(t1 * w_bf16_to_f64(w_bf16_pattern(0, sw[2 * ch + 1], sw[2 * ch]))) | (sg << 15);
                    uint32_t got = w_bf16_pattern(sg, (uint32_t)(e_in > 0 ? e_in : 0), m_in);
                    if (want != got) o.counts[1]++;
                    o.want[j * c.per_row + s] = want;
                }
            }
        }
    }
    for (auto& col : base) o.base.push_back(eval_of(c.log_rows, col));
    for (auto& col : pre) o.pre.push_back(eval_of(c.log_rows, col));
    return o;
}

}  // namespace zko
