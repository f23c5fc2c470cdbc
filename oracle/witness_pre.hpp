// TEST INFRASTRUCTURE ONLY (CPU oracle; see fields.hpp).
//
// Witness generation of (1) the shared bf16 tables' preprocessed columns and multiplicities, (2) the key tile's
// layout flags and selector columns and (3) the residual-stream component, restated from the reference's HOST code:
// tables are built by the loops that define them (not by a closed form of the row index), rows are evaluated in
// natural (coset) order with per-row local values, and columns are permuted into committed order by eval_of.
//   prover/src/bf16.rs:36-43, 47-90, 92, 130-158, 264-281, 289-292      (from_f32, Round, EXP_BIAS, norm_table, mul_table, decode)
//   prover/src/layout.rs:141-183                                        (Grid::row)
//   prover/src/gadgets/attention/trace.rs:742-790                       (nofirst / last / istart of a grid row)
//   prover/src/gadgets/residual_stream/mod.rs:173-245                   (DMAX, UMIN, pow/val/smul tables)
//   prover/src/gadgets/residual_stream/mod.rs:548-611                   (Prog column layout)
//   prover/src/gadgets/residual_stream/mod.rs:1116-1122, 1168-1236      (frac table, pow_at, smul_at, norm_at, frac_at, val_at)
//   prover/src/gadgets/residual_stream/mod.rs:1476-1760                 (residual_stream_component, the honest path)
//   prover/src/gadgets/residual_stream/witness.rs                       (split, join, sgn_of)
// Pinned by the reference's own device kernels for the same columns (zk_witness_gen_pre_table, zk_flags_key_tile,
// zk_witness_gen_sel, zk_witness_gen_residual_stream), compiled unmodified and run on the same inputs by the GPU tests.
#pragma once
#include <array>

#include "witness.hpp"

namespace zko {

// ---- bf16 rounding (bf16.rs:47-90) --------------------------------------------------------------
enum PreRound : uint32_t { ROUND_EVEN = 0, ROUND_AWAY = 1, ROUND_ZERO = 2 };
inline bool round_needs_sticky(uint32_t round) { return round == ROUND_EVEN; }
inline uint32_t round_carry(uint32_t round, uint32_t m, uint32_t rb, uint32_t st) {
    if (round == ROUND_EVEN) return rb & (st | (m & 1));
    if (round == ROUND_AWAY) return rb;
    return 0;
}
constexpr uint32_t PRE_EXP_BIAS = 134;

// ---- the shared tables, row by row as the host builds them --------------------------------------
using PreRow = std::array<uint32_t, 6>;
inline std::vector<PreRow> pre_norm_table(uint32_t kmax, uint32_t round) {  // bf16.rs:130-158, as (m2, ph, st, m7, expfield, nz)
    std::vector<PreRow> rows{{0, 0, 0, 0, 0, 0}};
    for (uint32_t m2 = 1; m2 < 256; m2++) {
        uint32_t b = w_bf16_from_f32((float)m2);
        rows.push_back({m2, 1, 0, b & 0x7f, (b >> 7) & 0xff, 1});
    }
    for (uint32_t k = 0; k <= kmax; k++)
        for (uint32_t m2 = 256; m2 < 512; m2++)
            for (uint32_t st = 0; st <= (round_needs_sticky(round) ? 1u : 0u); st++) {
                uint32_t m = m2 >> 1, rb = m2 & 1, up = round_carry(round, m, rb, st);
                uint32_t msig = m + up, extra = 0;
                if (msig == 256) { msig = 128; extra = 1; }
                rows.push_back({m2, 1u << k, st, msig - 128, k + 1 + extra + PRE_EXP_BIAS, 1});
            }
    return rows;
}
inline std::vector<PreRow> pre_frac_table(uint32_t kmax, bool sticky) {  // residual_stream/mod.rs:1116-1122, as (ph, r, st)
    std::vector<PreRow> rows{{0, 0, 0, 0, 0, 0}};
    for (uint32_t k = 0; k <= kmax; k++)
        for (uint32_t r = 0; r < (1u << k); r++) rows.push_back({1u << k, r, (sticky && r != 0) ? 1u : 0u, 0, 0, 0});
    return rows;
}
inline std::vector<PreRow> pre_mul_table(uint32_t round) {  // bf16.rs:264-281, as (a, b, m7, carry)
    std::vector<PreRow> rows;
    for (uint32_t a = 0; a < 128; a++)
        for (uint32_t b = 0; b < 128; b++) {
            uint32_t p = (128 + a) * (128 + b), carry = (p >> 15) & 1, shift = 7 + carry, m = p >> shift;
            uint32_t rb = (p >> (shift - 1)) & 1, st = (p & ((1u << (shift - 1)) - 1)) != 0, up = round_carry(round, m, rb, st);
            uint32_t msig = m + up, extra = 0;
            if (msig == 256) { msig = 128; extra = 1; }
            rows.push_back({a, b, msig - 128, carry + extra, 0, 0});
        }
    return rows;
}

enum PreKind : uint32_t { PRE_NORM = 0, PRE_FRAC = 1, PRE_MUL = 2, PRE_QNZ = 3, PRE_RANGE = 4 };
inline uint32_t pre_kind_cols(uint32_t kind) { return kind == PRE_NORM ? 6 : kind == PRE_FRAC ? 3 : kind == PRE_MUL ? 4 : kind == PRE_QNZ ? 2 : 1; }
// The table's own length (the rows beyond it, up to 2^log_rows, commit zero).
inline size_t pre_real_rows(uint32_t kind, uint32_t log_rows, uint32_t kmax, uint32_t round) {
    if (kind == PRE_NORM) return 256 + (size_t)(kmax + 1) * 256 * (round_needs_sticky(round) ? 2 : 1);
    if (kind == PRE_FRAC) return (size_t)1 << (kmax + 1);
    if (kind == PRE_MUL) return (size_t)1 << 14;
    return (size_t)1 << log_rows;
}
struct PreTableOut { std::vector<std::vector<uint32_t>> cols; std::vector<uint32_t> m; };
inline PreTableOut witness_pre_table(uint32_t kind, uint32_t log_rows, uint32_t kmax, uint32_t round,
                                     const std::vector<const uint32_t*>& counters, bool with_m, const uint32_t* patch_idx,
                                     const uint32_t* patch_val, uint32_t n_patch) {
    size_t rows = (size_t)1 << log_rows;
    uint32_t n_cols = pre_kind_cols(kind);
    std::vector<PreRow> table;
    if (kind == PRE_NORM) table = pre_norm_table(kmax, round);
    else if (kind == PRE_FRAC) table = pre_frac_table(kmax, round_needs_sticky(round));
    else if (kind == PRE_MUL) table = pre_mul_table(round);
    else for (size_t d = 0; d < rows; d++) table.push_back({(uint32_t)d, d != 0 ? 1u : 0u, 0, 0, 0, 0});
    std::vector<std::vector<uint32_t>> nat(n_cols, std::vector<uint32_t>(rows, 0));
    for (size_t d = 0; d < rows && d < table.size(); d++)
        for (uint32_t c = 0; c < n_cols; c++) nat[c][d] = table[d][c];
    for (uint32_t t = 0; t < n_patch; t++)  // the rows where this run's table is not the closed form
        for (uint32_t c = 0; c < n_cols; c++) nat[c][patch_idx[t]] = patch_val[(size_t)t * n_cols + c];
    PreTableOut o;
    for (auto& col : nat) o.cols.push_back(eval_of(log_rows, col));
    if (with_m) {
        std::vector<uint32_t> m(rows, 0);
        for (size_t d = 0; d < rows; d++)
            for (const uint32_t* c : counters) m[d] += c[d];
        o.m = eval_of(log_rows, m);
    }
    return o;
}

// ---- key tile flags and selectors ------------------------------------------------------------------
constexpr uint32_t KT_ACTIVE = 1, KT_NOFIRST = 2, KT_LAST = 4, KT_ISTART = 8;
enum KtShape : uint32_t { KT_CHAN = 0, KT_KEY = 1, KT_TOK = 2 };
struct KtGrid { uint32_t log_rows, groups, chunks, lead, descending; };
inline bool kt_grid_row(const KtGrid& g, size_t j, uint32_t& grp, uint32_t& chunk) {  // layout.rs:141-183
    if (j < g.lead) return false;
    size_t idx = j - g.lead;
    uint32_t gi = (uint32_t)(idx / g.chunks);
    grp = g.descending ? g.groups - 1 - gi : gi;
    chunk = g.chunks - 1 - (uint32_t)(idx % g.chunks);
    return true;
}
// In natural (coset) row order. `modulus` is hd (chan), C (key) or S (tok); `rw` the per-token row width.
inline std::vector<uint32_t> key_tile_flags(uint32_t shape, const KtGrid& g, uint32_t modulus, uint32_t rw) {
    size_t rows = (size_t)1 << g.log_rows;
    std::vector<uint32_t> f(rows, 0);
    for (size_t j = 0; j < rows; j++) {
        if (shape == KT_TOK) {  // every row active, no chunks; an instance starts where the row's highest token is S-1 mod S
            uint64_t hi = (uint64_t)(rows - 1 - j) * rw + rw;
            f[j] = KT_ACTIVE | (j > 0 ? KT_NOFIRST : 0) | ((j > 0 && hi % modulus == 0) ? KT_ISTART : 0);
            continue;
        }
        uint32_t grp = 0, chunk = 0;
        if (!kt_grid_row(g, j, grp, chunk)) continue;
        f[j] = KT_ACTIVE | (chunk + 1 < g.chunks ? KT_NOFIRST : 0) | (chunk == 0 ? KT_LAST : 0);
        if (j > 0 && chunk + 1 == g.chunks && grp % modulus == modulus - 1) f[j] |= KT_ISTART;
    }
    return f;
}
// The selector columns of one sub-component, committed order. `scale`: 1/delta per instance (key shape, with_scale).
inline std::vector<std::vector<uint32_t>> witness_selectors(uint32_t shape, const KtGrid& g, const std::vector<uint32_t>& flags,
                                                            const uint32_t* scale, uint32_t ctx, bool with_scale, uint32_t n_cols) {
    size_t rows = (size_t)1 << g.log_rows;
    std::vector<std::vector<uint32_t>> nat(n_cols, std::vector<uint32_t>(rows, 0));
    for (size_t j = 0; j < rows; j++) {
        uint32_t f = flags[j];
        bool act = f & KT_ACTIVE, nofirst = f & KT_NOFIRST, last = f & KT_LAST, istart = f & KT_ISTART, pos = j > 0, end = j + 1 == rows;
        if (shape == KT_TOK) { nat[0][j] = pos; nat[1][j] = end; nat[2][j] = istart; continue; }
        nat[0][j] = nofirst; nat[1][j] = last; nat[2][j] = pos; nat[3][j] = end;
        if (shape == KT_CHAN) { nat[4][j] = istart; continue; }
        nat[4][j] = pos && !last; nat[5][j] = pos && last; nat[6][j] = istart;
        uint32_t sc = 1;
        if (with_scale) {
            uint32_t grp = 0, chunk = 0;
            if (kt_grid_row(g, j, grp, chunk)) sc = scale[grp / ctx];
        }
        nat[7][j] = sc;
        if (n_cols > 8) nat[8][j] = act;
    }
    std::vector<std::vector<uint32_t>> out;
    for (auto& col : nat) out.push_back(eval_of(g.log_rows, col));
    return out;
}

// ---- the residual-stream component ---------------------------------------------------------------
constexpr uint32_t RS_DMAX = 12, RS_EXP_BIAS = 134;
constexpr int64_t RS_UMIN = 260;
constexpr int64_t RS_NONE = -1;
inline void rs_split(uint32_t pat, int64_t& sm, uint32_t& ef) {  // witness.rs split: zeros, infinities and NaNs collapse to (0, 0)
    uint32_t sg = (pat >> 15) & 1, e = (pat >> 7) & 0xff, m7 = pat & 0x7f;
    if (e == 0 || e == 0xff) { sm = 0; ef = 0; return; }
    sm = sg ? -(int64_t)(128 + m7) : (int64_t)(128 + m7);
    ef = e;
}
inline uint32_t rs_join(int64_t sm, uint32_t ef) {
    if (sm == 0) return 0;
    uint32_t sg = sm < 0, m7 = (uint32_t)((sm < 0 ? -sm : sm) - 128);
    return ((sg << 15) | (ef << 7) | m7) & 0xffff;
}
inline int64_t rs_sgn_of(uint32_t v) { return v > 2147483647u / 2 ? (int64_t)v - 2147483647LL : (int64_t)v; }
inline int64_t rs_pow_at(int64_t u) {  // mod.rs:1168-1176
    if (u >= 0 && u <= (int64_t)RS_DMAX) return u;
    if (u >= -RS_UMIN && u < 0) return RS_DMAX + 1 + (-u - 1);
    return RS_NONE;
}
inline int64_t rs_val_at(int64_t sm, uint32_t ef) {  // mod.rs:1224-1236
    if (sm == 0 && ef == 0) return 0;
    uint64_t a = (uint64_t)(sm < 0 ? -sm : sm);
    if (ef == 0 || ef >= 0xff || a < 128 || a >= 256) return RS_NONE;
    return 1 + ((int64_t)(ef - 1) * 128 + (int64_t)(a - 128)) * 2 + (sm < 0 ? 1 : 0);
}
inline int64_t rs_smul_at(int64_t a, int64_t b) {  // mod.rs:1180-1191
    auto idx = [](int64_t v) -> int64_t {
        if (v == 0) return 0;
        uint64_t m = (uint64_t)(v < 0 ? -v : v);
        if (m < 128 || m >= 256) return RS_NONE;
        return 1 + (v < 0 ? 128 : 0) + (int64_t)(m - 128);
    };
    int64_t ia = idx(a), ib = idx(b);
    return (ia < 0 || ib < 0) ? RS_NONE : ia * 257 + ib;
}
inline int64_t rs_norm_at(uint32_t m2, uint32_t ph, uint32_t st, uint32_t kmax, bool sticky) {  // mod.rs:1194-1211
    if (m2 == 0 && ph == 0) return 0;
    if (ph == 1 && m2 >= 1 && m2 < 256) return m2;
    if (ph == 0 || (ph & (ph - 1)) || m2 < 256 || m2 >= 512) return RS_NONE;
    uint32_t k = (uint32_t)__builtin_ctz(ph);
    if (k > kmax) return RS_NONE;
    return 256 + ((int64_t)k * 256 + (m2 - 256)) * (sticky ? 2 : 1) + (sticky ? st : 0);
}
inline int64_t rs_frac_at(uint32_t ph, uint64_t r, uint32_t kmax) {  // mod.rs:1212-1220
    if (ph == 0) return r == 0 ? 0 : RS_NONE;
    if ((ph & (ph - 1)) || (uint32_t)__builtin_ctz(ph) > kmax || r >= ph) return RS_NONE;
    return (int64_t)ph + (int64_t)r;
}

struct RsSrc { uint32_t kind, g, i; };  // kind: 0 the constant zero, 1 a committed leaf, 2 its unary image, 3 an earlier slot's output
struct RsProg {
    std::vector<std::array<uint32_t, 2>> groups;  // (n, un): un = 0 for none, else 1 + the unary table's index
    uint32_t kind = 0;                            // 0 add, 1 multiply
    std::vector<std::array<RsSrc, 2>> slots;
    std::vector<uint32_t> out_slot;               // Prog::outs, flattened
    bool sticky = true;
    uint32_t kmax = 0;
    // Prog's column layout, mod.rs:548-590
    size_t leaf_width(size_t g) const { return groups[g][1] == 0 ? 2 : 4; }
    size_t n_leaves() const { size_t n = 0; for (auto& g : groups) n += g[0]; return n; }
    size_t group_base(size_t g) const { size_t b = 0; for (size_t k = 0; k < g; k++) b += groups[k][0] * leaf_width(k); return b; }
    size_t leaf_at(size_t g, size_t i) const { return group_base(g) + i * leaf_width(g); }
    size_t slot_width() const { return kind == 0 ? 13 + (sticky ? 1 : 0) : 4; }
    size_t slot_at(size_t s) const { return group_base(groups.size()) + s * slot_width(); }
    size_t n_cols() const { return slot_at(slots.size()); }
    std::pair<size_t, size_t> out_cols(size_t s) const {
        size_t b = slot_at(s);
        if (kind == 0) { size_t k = 11 + (sticky ? 1 : 0); return {b + k, b + k + 1}; }
        return {b, b + 3};
    }
};
struct RsTables {
    const uint32_t* norm3; size_t n_norm;           // (m7, expfield, nz) per norm_table row
    const int32_t* smul3; size_t n_smul;            // (signed significand, carry, nz) per smul_table row
    std::vector<const int32_t*> un2; size_t n_val;  // (osm, oef) per val_table row, per unary table
};
struct RsOut {
    std::vector<std::vector<uint32_t>> cols;  // committed order
    std::vector<uint32_t> out_pat;            // natural row order, rows x out_w
    std::vector<int32_t> out_nat, in_nat;     // natural row order, pairs
    std::vector<uint32_t> m_pow, m_norm, m_val, m_frac, m_smul;
    std::vector<std::vector<uint32_t>> m_un;
    uint32_t counts[3] = {0, 0, 0};           // lookups off their table, exponents out of range, unary images off the table
};
// wit: live_rows x n_leaves bf16 patterns, row-flat (group after group inside a row). m_len: lengths of the
// multiplicity arrays in the order pow, norm, val, frac, smul, un.
inline RsOut witness_residual_stream(const RsProg& p, const RsTables& t, const uint32_t* wit, size_t live_rows, uint32_t log_rows,
                                     const size_t m_len[6]) {
    size_t rows = (size_t)1 << log_rows, n_cols = p.n_cols(), n_leaves = p.n_leaves(), out_w = p.out_slot.size();
    RsOut o;
    std::vector<std::vector<uint32_t>> nat(n_cols, std::vector<uint32_t>(rows, 0));
    o.out_pat.assign(rows * out_w, 0); o.out_nat.assign(rows * out_w * 2, 0); o.in_nat.assign(rows * n_leaves * 2, 0);
    o.m_pow.assign(m_len[0], 0); o.m_norm.assign(m_len[1], 0); o.m_val.assign(m_len[2], 0); o.m_frac.assign(m_len[3], 0);
    o.m_smul.assign(m_len[4], 0); o.m_un.assign(t.un2.size(), std::vector<uint32_t>(m_len[5], 0));
    auto bump = [&](std::vector<uint32_t>& m, int64_t idx) { if (idx >= 0 && (size_t)idx < m.size()) m[idx]++; else o.counts[0]++; };
    for (size_t j = 0; j < rows; j++) {
        bool live = j < live_rows;
        std::vector<std::vector<std::pair<int64_t, uint32_t>>> lin(p.groups.size()), lun(p.groups.size());
        size_t flat = 0;
        for (size_t g = 0; g < p.groups.size(); g++)
            for (size_t i = 0; i < p.groups[g][0]; i++, flat++) {
                uint32_t pat = live ? wit[j * n_leaves + flat] : 0;
                int64_t sm; uint32_t ef;
                rs_split(pat, sm, ef);
                size_t b = p.leaf_at(g, i);
                nat[b][j] = w_m31_of(sm); nat[b + 1][j] = ef;
                o.in_nat[(j * n_leaves + flat) * 2] = (int32_t)sm; o.in_nat[(j * n_leaves + flat) * 2 + 1] = (int32_t)ef;
                int64_t v = rs_val_at(sm, ef);
                lin[g].push_back({sm, ef});
                if (p.groups[g][1] == 0) { bump(o.m_val, v); lun[g].push_back({0, 0}); continue; }
                size_t u = p.groups[g][1] - 1;
                bump(o.m_un[u], v);
                int64_t osm = 0; uint32_t oef = 0;
                if (v >= 0 && (size_t)v < t.n_val) { osm = t.un2[u][v * 2]; oef = (uint32_t)t.un2[u][v * 2 + 1]; }
                else o.counts[2]++;
                nat[b + 2][j] = w_m31_of(osm); nat[b + 3][j] = oef;
                lun[g].push_back({osm, oef});
            }
        std::vector<std::pair<int64_t, uint32_t>> outs;  // (c_sm, clamped c_ef) per slot
        std::vector<int64_t> raw_ef;                     // the unclamped exponent, as the cell holds it
        auto get = [&](const RsSrc& s) -> std::pair<int64_t, uint32_t> {
            if (s.kind == 1) return lin[s.g][s.i];
            if (s.kind == 2) return lun[s.g][s.i];
            if (s.kind == 3) return outs[s.g];
            return {0, 0};
        };
        for (size_t si = 0; si < p.slots.size(); si++) {
            auto [a_sm, a_ef] = get(p.slots[si][0]);
            auto [b_sm, b_ef] = get(p.slots[si][1]);
            size_t b = p.slot_at(si);
            int64_t c_sm = 0, c_ef = 0;
            if (p.kind == 0) {
                int64_t etop = std::max(a_ef, b_ef);
                auto pw = [&](int64_t u) -> int64_t {
                    int64_t i = rs_pow_at(u);
                    bump(o.m_pow, i);
                    return (i >= 0 && u >= 0) ? ((int64_t)1 << u) : 0;
                };
                int64_t fa = pw((int64_t)a_ef - etop + RS_DMAX), fb = pw((int64_t)b_ef - etop + RS_DMAX);
                nat[b][j] = w_m31_of(fa); nat[b + 1][j] = w_m31_of(fb);
                int64_t acc = a_sm * fa + b_sm * fb;
                uint32_t sg = acc < 0;
                uint64_t mag = (uint64_t)(acc < 0 ? -acc : acc), r = 0;
                uint32_t m2 = 0, ph = 0, st_raw = 0;
                if (!w_normalise(mag, p.kmax, m2, ph, st_raw, r)) { o.counts[0]++; m2 = ph = st_raw = 0; r = 0; }
                uint32_t st = p.sticky ? st_raw : 0;
                int64_t ni = rs_norm_at(m2, ph, st, p.kmax, p.sticky);
                uint32_t m7n = 0, efn = 0, nzn = 0;
                if (ni >= 0 && (size_t)ni < t.n_norm) { m7n = t.norm3[ni * 3]; efn = t.norm3[ni * 3 + 1]; nzn = t.norm3[ni * 3 + 2]; }
                else o.counts[0]++;
                bump(o.m_norm, ni);
                bump(o.m_frac, rs_frac_at(ph, r, p.kmax));
                c_sm = (int64_t)(128 * nzn + m7n) * (sg ? -1 : 1);
                c_ef = nzn == 1 ? (int64_t)efn + etop - RS_DMAX - RS_EXP_BIAS : 0;
                if (nzn == 1 && !(c_ef >= 1 && c_ef < 0xff)) o.counts[1]++;
                nat[b + 2][j] = w_m31_of(etop); nat[b + 3][j] = w_m31_of((int64_t)mag); nat[b + 4][j] = sg; nat[b + 5][j] = m2;
                nat[b + 6][j] = ph; nat[b + 7][j] = w_m31_of((int64_t)r);
                size_t k = 8;
                if (p.sticky) nat[b + k++][j] = st;
                nat[b + k][j] = m7n; nat[b + k + 1][j] = efn; nat[b + k + 2][j] = nzn;
                nat[b + k + 3][j] = w_m31_of(c_sm); nat[b + k + 4][j] = w_m31_of(c_ef);
            } else {
                int64_t si_ = rs_smul_at(a_sm, b_sm), c0 = 0;
                uint32_t cy = 0, nzc = 0;
                if (si_ >= 0 && (size_t)si_ < t.n_smul) { c0 = t.smul3[si_ * 3]; cy = (uint32_t)t.smul3[si_ * 3 + 1]; nzc = (uint32_t)t.smul3[si_ * 3 + 2]; }
                else o.counts[0]++;
                bump(o.m_smul, si_);
                c_ef = nzc == 1 ? (int64_t)a_ef + (int64_t)b_ef + cy - 127 : 0;
                if (nzc == 1 && !(c_ef >= 1 && c_ef < 0xff)) o.counts[1]++;
                c_sm = c0;
                nat[b][j] = w_m31_of(c_sm); nat[b + 1][j] = cy; nat[b + 2][j] = nzc; nat[b + 3][j] = w_m31_of(c_ef);
            }
            bump(o.m_val, (c_ef >= 0 && c_ef < 0xff) ? rs_val_at(c_sm, (uint32_t)c_ef) : RS_NONE);
            outs.push_back({c_sm, (uint32_t)std::min<int64_t>(std::max<int64_t>(c_ef, 0), 0xfe)});
            raw_ef.push_back(c_ef);
        }
        for (size_t k = 0; k < out_w; k++) {
            size_t s = p.out_slot[k];
            o.out_pat[j * out_w + k] = rs_join(outs[s].first, outs[s].second);
            o.out_nat[(j * out_w + k) * 2] = (int32_t)outs[s].first;
            o.out_nat[(j * out_w + k) * 2 + 1] = (int32_t)raw_ef[s];
        }
    }
    for (auto& col : nat) o.cols.push_back(eval_of(log_rows, col));
    return o;
}

}  // namespace zko
