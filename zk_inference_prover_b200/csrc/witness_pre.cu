// Witness generation on the device, three more families: the shared bf16 tables' preprocessed columns and their
// multiplicity columns, the key tile's layout flags and selector columns, and the residual-stream component.
// Everything is written in committed order (natural row j lands at index coset_perm(j), prover/src/common.rs:76-80).
//
// Host statements these replace: bf16::norm_table / mul_table (prover/src/bf16.rs:130-158, 264-281), the fraction table
// (prover/src/gadgets/residual_stream/mod.rs:1116-1122), the key tile's row predicates
// (prover/src/gadgets/attention/trace.rs:742-790) and residual_stream_component
// (prover/src/gadgets/residual_stream/mod.rs:1418-1760). The reference's device originals are zk_witness_gen_pre_table and
// zk_witness_gen_sel (stwo_cuda/cuda/zk_pre_witness_gen.cu), zk_flags_key_tile (stwo_cuda/cuda/zk_acc.cu:78-97) and
// zk_witness_gen_residual_stream (stwo_cuda/cuda/zk_residual_stream_witness_gen.cu). Their "mutate" arguments
// (deliberate defects for negative controls) are not part of the operators and are not built.
#include <algorithm>
#include <cstring>
#include <vector>

#include "common.cuh"

namespace zk {

namespace {

constexpr uint32_t OFF_TABLE = 0xffffffffu;

__device__ __forceinline__ uint32_t committed_to_natural(uint32_t i, uint32_t log_n) {
    uint32_t c = (i & 1u) ? (((2u << log_n) - i - 1u) >> 1) : (i >> 1);
    return __brev(c) >> (32u - log_n);
}
__device__ __forceinline__ uint32_t field_of(long long v) {  // ((v % p) + p) % p, encoding.rs:29-32
    // two folds of 31 bits bring any |v| < 2^62 below 2p (2^31 = 1 mod p); no 64-bit division
    unsigned long long u = (unsigned long long)(v < 0 ? -v : v);
    u = (u & P) + (u >> 31);
    u = (u & P) + (u >> 31);
    uint32_t r = (uint32_t)u;
    if (r >= P) r -= P;
    return (v < 0 && r) ? P - r : r;
}
__device__ __forceinline__ long long signed_of(uint32_t v) { return v > P / 2 ? (long long)v - (long long)P : (long long)v; }

// ---------------------------------------------------------------------------------------------------
// The shared tables. Every row is a function of its own index; no table is uploaded.
// ---------------------------------------------------------------------------------------------------
struct PreCfg {
    uint32_t kind, log_rows, real_rows, kmax, round, sticky, n_cols, n_counters;
};

// One rounding step of an 8-bit significand m in [128, 256) with round bit rb and sticky flag st: the significand
// field (m7) and whether the step carried into the next binade (bf16.rs:81-88 and the renormalisation at :146).
__device__ __forceinline__ void round_significand(uint32_t round, uint32_t m, uint32_t rb, uint32_t st, uint32_t& m7, uint32_t& binade_up) {
    uint32_t up = round == 0 ? (rb & (st | (m & 1u))) : round == 1 ? rb : 0u;
    uint32_t sig = m + up;
    binade_up = sig >> 8;              // 256 only from m = 255 with a carry
    m7 = binade_up ? 0u : sig - 128u;  // 256 renormalises to significand 128
}

template <uint32_t KIND>
__device__ __forceinline__ void table_row(const PreCfg& c, uint32_t d, uint32_t (&o)[6]) {
#pragma unroll
    for (int k = 0; k < 6; k++) o[k] = 0;
    if (KIND == 3) { o[0] = d; o[1] = d != 0; return; }  // q != 0 indicator
    if (KIND == 4) { o[0] = d; return; }                 // a range table is its own index
    if (d >= c.real_rows) return;                        // past the table's own length: zero rows
    if (KIND == 0) {                                     // normalisation: (m2, ph, st, m7, expfield, nz)
        if (d == 0) return;
        if (d < 256u) {  // an integer below 256 is exactly representable: its top bit gives the binade, the rest the fraction
            uint32_t t = 31u - __clz(d);
            o[0] = d; o[1] = 1; o[3] = (d << (7u - t)) - 128u; o[4] = 127u + t; o[5] = 1;
            return;
        }
        uint32_t per_k = 256u << c.sticky, idx = d - 256u, k = idx / per_k, rem = idx - k * per_k;
        uint32_t m2 = 256u + (rem >> c.sticky), st = c.sticky ? (rem & 1u) : 0u, m7, up;
        round_significand(c.round, m2 >> 1, m2 & 1u, st, m7, up);
        o[0] = m2; o[1] = 1u << k; o[2] = st; o[3] = m7; o[4] = k + 1u + up + 134u; o[5] = 1;
        return;
    }
    if (KIND == 1) {  // fraction: (2^k, r, sticky && r != 0) for 2^k <= d < 2^(k+1)
        if (d == 0) return;
        uint32_t k = 31u - __clz(d), r = d - (1u << k);
        o[0] = 1u << k; o[1] = r; o[2] = (c.sticky && r != 0) ? 1u : 0u;
        return;
    }
    // multiply: (a, b, m7, carry) of the significand product (128 + a)(128 + b), a 16-bit integer in [2^14, 2^16)
    uint32_t a = d >> 7, b = d & 127u, p = (128u + a) * (128u + b), carry = p >> 15, shift = 7u + carry, m7, up;
    round_significand(c.round, p >> shift, (p >> (shift - 1u)) & 1u, (p & ((1u << (shift - 1u)) - 1u)) != 0, m7, up);
    o[0] = a; o[1] = b; o[2] = m7; o[3] = carry + up;
}

// One thread per PAIR of committed rows 2q, 2q+1 (natural rows brev(q) and its complement): 8-byte stores per column.
template <uint32_t KIND>
__global__ void __launch_bounds__(256) pre_table_kernel(const uint32_t* const* __restrict__ counters, uint32_t* const* __restrict__ cols,
                                                        uint32_t* __restrict__ m_col, PreCfg c) {
    const uint32_t L = c.log_rows, q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q >> (L - 1)) return;
    const uint32_t j0 = __brev(q) >> (32u - L), j1 = (~j0) & ((1u << L) - 1u);
    uint32_t r0[6], r1[6];
    table_row<KIND>(c, j0, r0);
    table_row<KIND>(c, j1, r1);
#pragma unroll
    for (uint32_t k = 0; k < 6; k++)
        if (k < c.n_cols) reinterpret_cast<uint2*>(cols[k])[q] = make_uint2(r0[k], r1[k]);
    if (m_col) {  // the multiplicities: every component that bumped this table kept a counter of its own; the column is their sum
        uint32_t s0 = 0, s1 = 0;
        for (uint32_t k = 0; k < c.n_counters; k++) {
            const uint32_t* cnt = counters[k];
            s0 += __ldg(cnt + j0);
            s1 += __ldg(cnt + j1);
        }
        reinterpret_cast<uint2*>(m_col)[q] = make_uint2(s0, s1);
    }
}

// Rows where this run's own table is not the closed form (the reference's corrupted-table probe; empty otherwise).
__global__ void pre_patch_kernel(const uint32_t* __restrict__ idx, const uint32_t* __restrict__ val, uint32_t n, uint32_t* const* __restrict__ cols,
                                 uint32_t n_cols, uint32_t log_rows) {
    uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n) return;
    uint32_t i = committed_to_natural(idx[t], log_rows);  // the permutation is an involution
    for (uint32_t k = 0; k < n_cols; k++) cols[k][i] = val[(size_t)t * n_cols + k];
}

// ---------------------------------------------------------------------------------------------------
// Key tile: per-row layout flags (natural order) and the selector columns built from them (committed order).
// ---------------------------------------------------------------------------------------------------
constexpr uint32_t F_ACTIVE = 1, F_NOFIRST = 2, F_LAST = 4, F_ISTART = 8;
struct TileGrid {
    uint32_t log_rows, groups, chunks, lead, descending;
};
__device__ __forceinline__ bool tile_row(const TileGrid& g, uint32_t j, uint32_t& grp, uint32_t& chunk) {  // layout.rs:141-183
    if (j < g.lead) return false;
    uint32_t idx = j - g.lead, gi = idx / g.chunks;
    grp = g.descending ? g.groups - 1u - gi : gi;
    chunk = g.chunks - 1u - (idx - gi * g.chunks);
    return true;
}
__global__ void tile_flags_kernel(uint32_t* __restrict__ flags, uint32_t shape, TileGrid g, uint32_t modulus, uint32_t rw) {
    uint32_t j = blockIdx.x * blockDim.x + threadIdx.x, rows = 1u << g.log_rows;
    if (j >= rows) return;
    uint32_t f = 0;
    if (shape == 2) {  // per-token component: every row active, an instance starts where the row's highest token is S-1 mod S
        unsigned long long hi = (unsigned long long)(rows - 1u - j) * rw + rw;
        f = F_ACTIVE | (j > 0 ? F_NOFIRST : 0u) | ((j > 0 && hi % modulus == 0) ? F_ISTART : 0u);
    } else {
        uint32_t grp = 0, chunk = 0;
        if (tile_row(g, j, grp, chunk)) {
            f = F_ACTIVE | (chunk + 1u < g.chunks ? F_NOFIRST : 0u) | (chunk == 0 ? F_LAST : 0u);
            if (j > 0 && chunk + 1u == g.chunks && grp % modulus == modulus - 1u) f |= F_ISTART;
        }
    }
    flags[j] = f;
}

struct SelCfg {
    uint32_t shape;  // 0 channel, 1 key, 2 per-token
    TileGrid g;
    uint32_t ctx, with_scale, n_cols;
};
__global__ void selectors_kernel(const uint32_t* __restrict__ flags, const uint32_t* __restrict__ scale, uint32_t* const* __restrict__ cols, SelCfg c) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x, rows = 1u << c.g.log_rows;
    if (i >= rows) return;
    uint32_t j = committed_to_natural(i, c.g.log_rows), f = __ldg(flags + j);
    uint32_t act = f & F_ACTIVE ? 1u : 0u, nofirst = f & F_NOFIRST ? 1u : 0u, last = f & F_LAST ? 1u : 0u, istart = f & F_ISTART ? 1u : 0u;
    uint32_t pos = j > 0, end = j + 1u == rows;
    if (c.shape == 2) { cols[0][i] = pos; cols[1][i] = end; cols[2][i] = istart; return; }
    cols[0][i] = nofirst; cols[1][i] = last; cols[2][i] = pos; cols[3][i] = end;
    if (c.shape == 0) { cols[4][i] = istart; return; }
    cols[4][i] = pos & (last ^ 1u); cols[5][i] = pos & last; cols[6][i] = istart;
    uint32_t sc = 1;  // the master exp table's key scale, inverted, per instance; an inert row takes 1
    if (c.with_scale) {
        uint32_t grp = 0, chunk = 0;
        if (tile_row(c.g, j, grp, chunk)) sc = __ldg(scale + grp / c.ctx);
    }
    cols[7][i] = sc;
    if (c.n_cols > 8) cols[8][i] = act;
}


// ---------------------------------------------------------------------------------------------------
// The residual-stream component: a row is a small program over bf16 values held as (signed significand, exponent
// field) pairs: committed leaves (optionally with a tabulated unary image), then slots that each add or multiply two
// earlier values with one bf16 rounding, every intermediate being a committed cell and every table read a counted
// lookup. One thread owns one committed row. A slot's operands are cells the same thread wrote earlier, read back
// from the columns (plain loads, program order), so no per-row state is kept however long the program is.
// ---------------------------------------------------------------------------------------------------
struct RsGroup { uint32_t n, leaf_col, width, un, flat; };
struct RsSlot { uint32_t a_sm, a_ef, b_sm, b_ef, base, o_sm, o_ef, from_slot; };
struct RsMult { uint32_t* m; uint32_t n; };
struct RsArgs {
    const uint32_t* wit;
    const RsGroup* groups;
    const RsSlot* slots;
    const uint32_t* norm3;
    const int32_t* smul3;
    const int32_t* const* un2;
    const uint32_t* out_slot;
    const uint32_t* order;        // slot indices sorted by level
    const uint32_t* level_start;  // n_levels + 1 offsets into `order`
    uint32_t* const* cols;
    uint32_t* out_pat;
    int32_t* out_nat;
    int32_t* in_nat;
    RsMult m_pow, m_norm, m_val, m_frac, m_smul;
    const RsMult* m_un;
    uint32_t* counts;
    uint32_t n_norm, n_smul, n_val, log_rows, live, n_groups, n_leaves, n_slots, n_levels, kmax, out_w;
};
constexpr uint32_t RS_DMAX = 12, RS_UMIN = 260, RS_BIAS = 134, RS_POW_ROWS = RS_DMAX + 1 + RS_UMIN;

// One lookup: bump the table's multiplicity, or count the lookup as off the table. Lanes of a warp that hit the same
// entry (a padded row's leaves all hit entry 0) are merged into one atomic.
__device__ __forceinline__ void lookup(const RsMult& t, uint32_t idx, uint32_t& off) {
    if (idx >= t.n) { off++; return; }  // OFF_TABLE is larger than any table
    uint32_t peers = __match_any_sync(__activemask(), idx);
    if ((threadIdx.x & 31u) == (uint32_t)(__ffs(peers) - 1)) atomicAdd(t.m + idx, (uint32_t)__popc(peers));
}
__device__ __forceinline__ uint32_t value_index(long long sm, long long ef) {  // val_table's row order: zero, then (ef, m7, sign)
    if (sm == 0 && ef == 0) return 0;
    unsigned long long a = (unsigned long long)(sm < 0 ? -sm : sm);
    if (ef <= 0 || ef >= 0xff || a < 128 || a >= 256) return OFF_TABLE;
    return 1u + (((uint32_t)ef - 1u) * 128u + (uint32_t)(a - 128)) * 2u + (sm < 0 ? 1u : 0u);
}
__device__ __forceinline__ uint32_t pow_index(long long u) {  // [0, DMAX], then [-UMIN, -1]
    if (u >= 0 && u <= (long long)RS_DMAX) return (uint32_t)u;
    if (u < 0 && u >= -(long long)RS_UMIN) return RS_DMAX + (uint32_t)(-u);
    return OFF_TABLE;
}
__device__ __forceinline__ uint32_t signed_significand_index(long long v) {
    if (v == 0) return 0;
    unsigned long long a = (unsigned long long)(v < 0 ? -v : v);
    return (a < 128 || a >= 256) ? OFF_TABLE : 1u + (v < 0 ? 128u : 0u) + (uint32_t)(a - 128);
}
// The column table is never written by the kernel: its entries are fetched through the read-only path, so that the loads
// of a slot's fourteen column addresses are independent of the stores between them (a plain load would have to be
// ordered after every earlier store, one address at a time).
__device__ __forceinline__ uint32_t* column(uint32_t* const* cols, uint32_t c) {
    return reinterpret_cast<uint32_t*>(__ldg(reinterpret_cast<const unsigned long long*>(cols) + c));
}
// An operand as the (significand, exponent) it encodes. A slot's output exponent is clamped to [0, 0xfe] on the way
// out of the slot while its cell keeps the unclamped value, so the clamp applies to slot sources only.
__device__ __forceinline__ void operand(uint32_t* const* cols, uint32_t i, uint32_t c_sm, uint32_t c_ef, bool from_slot, long long& sm, long long& ef) {
    if (c_sm == OFF_TABLE) { sm = 0; ef = 0; return; }
    const uint32_t *p_sm = column(cols, c_sm), *p_ef = column(cols, c_ef);
    sm = signed_of(p_sm[i]);
    long long e = signed_of(p_ef[i]);
    ef = e < 0 ? 0 : (from_slot && e > 0xfe) ? 0xfe : e;
}

// A CTA owns 32 consecutive committed rows: lane = row, so that every column access of a warp is one 128-byte line.
// Its RS_LANES warps share the row's work: the leaves, then the slots level by level (a level holds the slots whose
// operands are leaves or outputs of earlier levels; `order` lists the slots by level, `level_start` where each begins),
// with a CTA barrier between levels, since a slot's operand may be a cell another warp of the CTA wrote.
constexpr uint32_t RS_LANES = 8;
template <bool MUL, bool STICKY>
__global__ void __launch_bounds__(32 * RS_LANES) residual_stream_kernel(RsArgs a) {
    // The power table has 273 rows and every addition hits row DMAX with its larger operand: counted per CTA in shared
    // memory and added to the global array once at the end (one hot address would serialise every warp of the grid).
    __shared__ uint32_t pow_hist[RS_POW_ROWS];
    if (!MUL) {
        for (uint32_t k = threadIdx.x; k < RS_POW_ROWS; k += blockDim.x) pow_hist[k] = 0;
        __syncthreads();
    }
    const uint32_t i = blockIdx.x * 32u + (threadIdx.x & 31u), t = threadIdx.x >> 5;
    const bool in_range = (i >> a.log_rows) == 0;
    const uint32_t j = in_range ? committed_to_natural(i, a.log_rows) : 0u;
    const bool live = j < a.live;
    uint32_t off = 0, bad_exp = 0, un_off = 0;
    uint32_t* const* cols = a.cols;
    const size_t leaf0 = (size_t)j * a.n_leaves;

    if (in_range)
    for (uint32_t g = 0; g < a.n_groups; g++) {
        const RsGroup gr = a.groups[g];
        for (uint32_t k = t; k < gr.n; k += RS_LANES) {
            const uint32_t pat = live ? __ldg(a.wit + leaf0 + gr.flat + k) : 0u;
            // a bf16 pattern as (sm, ef); both zeros, infinities and NaNs collapse to (0, 0)
            const uint32_t e = (pat >> 7) & 0xffu;
            const bool finite = e != 0 && e != 0xffu;
            const long long mag = 128 + (pat & 0x7fu);
            const long long sm = finite ? ((pat >> 15) & 1u ? -mag : mag) : 0;
            const uint32_t ef = finite ? e : 0u;
            const uint32_t b = gr.leaf_col + k * gr.width;
            uint32_t *c0 = column(cols, b), *c1 = column(cols, b + 1), *c2 = nullptr, *c3 = nullptr;
            if (gr.un) { c2 = column(cols, b + 2); c3 = column(cols, b + 3); }
            c0[i] = field_of(sm);
            c1[i] = ef;
            reinterpret_cast<int2*>(a.in_nat)[leaf0 + gr.flat + k] = make_int2((int)sm, (int)ef);  // natural row order
            const uint32_t v = value_index(sm, ef);
            if (gr.un == 0) { lookup(a.m_val, v, off); continue; }
            lookup(a.m_un[gr.un - 1], v, off);
            int2 img = make_int2(0, 0);  // the unary image, tabulated over the value table's rows
            if (v < a.n_val) img = __ldg(reinterpret_cast<const int2*>(a.un2[gr.un - 1]) + v);
            else un_off++;
            c2[i] = field_of(img.x);
            c3[i] = field_of(img.y);
        }
    }

    for (uint32_t level = 0; level < a.n_levels; level++) {
      __syncthreads();
      if (in_range)
      for (uint32_t at = a.level_start[level] + t; at < a.level_start[level + 1]; at += RS_LANES) {
        const RsSlot sl = a.slots[a.order[at]];
        long long a_sm, a_ef, b_sm, b_ef, c_sm, c_ef;
        operand(cols, i, sl.a_sm, sl.a_ef, sl.from_slot & 1u, a_sm, a_ef);
        operand(cols, i, sl.b_sm, sl.b_ef, sl.from_slot & 2u, b_sm, b_ef);
        const uint32_t b = sl.base;
        constexpr uint32_t W = MUL ? 4u : (STICKY ? 14u : 13u);
        uint32_t* cell[W];
#pragma unroll
        for (uint32_t k = 0; k < W; k++) cell[k] = column(cols, b + k);
        if (!MUL) {
            // align both operands to the larger exponent (a shift of up to DMAX bits is kept, a smaller operand is dropped),
            // add, normalise the magnitude to a 9-bit M2 with its round-bit weight ph, round through the table
            const long long etop = a_ef > b_ef ? a_ef : b_ef;
            const long long ua = a_ef - etop + RS_DMAX, ub = b_ef - etop + RS_DMAX;
            const uint32_t pa = pow_index(ua), pb = pow_index(ub);
            if (pa < a.m_pow.n) atomicAdd(pow_hist + pa, 1u); else off++;
            if (pb < a.m_pow.n) atomicAdd(pow_hist + pb, 1u); else off++;
            const long long fa = (pa != OFF_TABLE && ua >= 0) ? (1LL << ua) : 0, fb = (pb != OFF_TABLE && ub >= 0) ? (1LL << ub) : 0;
            const long long acc = a_sm * fa + b_sm * fb;
            const uint32_t sg = acc < 0;
            const unsigned long long mag = (unsigned long long)(acc < 0 ? -acc : acc);
            uint32_t m2 = 0, ph = 0, st = 0, k = 0;
            unsigned long long r = 0;
            if (mag) {
                const uint32_t bits = 64u - (uint32_t)__clzll((long long)mag);
                k = bits > 9u ? bits - 9u : 0u;
                if (k > a.kmax) off++;  // a round-bit weight the table does not carry
                else { ph = 1u << k; m2 = (uint32_t)(mag >> k); r = mag & ((1ull << k) - 1ull); st = STICKY && r != 0; }
            }
            uint32_t ni;  // the normalisation table's row: zero row, 255 exact small magnitudes, then (k, m2, st) ascending
            if (m2 == 0 && ph == 0) ni = 0;
            else if (ph == 1 && m2 < 256u) ni = m2;
            else if (m2 >= 256u && m2 < 512u) ni = 256u + (k * 256u + (m2 - 256u)) * (STICKY ? 2u : 1u) + st;
            else ni = OFF_TABLE;
            uint32_t m7n = 0, efn = 0, nzn = 0;
            if (ni < a.n_norm) { m7n = __ldg(a.norm3 + 3 * (size_t)ni); efn = __ldg(a.norm3 + 3 * (size_t)ni + 1); nzn = __ldg(a.norm3 + 3 * (size_t)ni + 2); }
            else off++;
            lookup(a.m_norm, ni, off);
            lookup(a.m_frac, ph == 0 ? (r == 0 ? 0u : OFF_TABLE) : ph + (uint32_t)r, off);
            c_sm = (long long)(128u * nzn + m7n) * (sg ? -1 : 1);
            c_ef = nzn == 1 ? (long long)efn + etop - RS_DMAX - RS_BIAS : 0;
            bad_exp += nzn == 1 && !(c_ef >= 1 && c_ef < 0xff);
            cell[0][i] = field_of(fa);
            cell[1][i] = field_of(fb);
            cell[2][i] = field_of(etop);
            cell[3][i] = field_of((long long)mag);
            cell[4][i] = sg;
            cell[5][i] = m2;
            cell[6][i] = ph;
            cell[7][i] = field_of((long long)r);
            if (STICKY) cell[8][i] = st;
            constexpr uint32_t kk = STICKY ? 9u : 8u;
            cell[kk][i] = m7n;
            cell[kk + 1][i] = efn;
            cell[kk + 2][i] = nzn;
            cell[kk + 3][i] = field_of(c_sm);
            cell[kk + 4][i] = field_of(c_ef);
        } else {
            // the signed significands' correctly rounded product and binade carry come from one table row
            const uint32_t ia = signed_significand_index(a_sm), ib = signed_significand_index(b_sm);
            const uint32_t si = (ia == OFF_TABLE || ib == OFF_TABLE) ? OFF_TABLE : ia * 257u + ib;
            int32_t prod = 0, cy = 0, nzc = 0;
            if (si < a.n_smul) { prod = __ldg(a.smul3 + 3 * (size_t)si); cy = __ldg(a.smul3 + 3 * (size_t)si + 1); nzc = __ldg(a.smul3 + 3 * (size_t)si + 2); }
            else off++;
            lookup(a.m_smul, si, off);
            c_sm = prod;
            c_ef = nzc == 1 ? a_ef + b_ef + cy - 127 : 0;
            bad_exp += nzc == 1 && !(c_ef >= 1 && c_ef < 0xff);
            cell[0][i] = field_of(c_sm);
            cell[1][i] = (uint32_t)cy;
            cell[2][i] = (uint32_t)nzc;
            cell[3][i] = field_of(c_ef);
        }
        lookup(a.m_val, (c_ef >= 0 && c_ef < 0xff) ? value_index(c_sm, c_ef) : OFF_TABLE, off);  // the slot's own output is a looked-up pair too
      }
    }
    __syncthreads();

    // what the bindings and the next component read, in natural row order
    if (in_range)
    for (uint32_t k = t; k < a.out_w; k += RS_LANES) {
        const RsSlot sl = a.slots[a.out_slot[k]];
        const long long sm = signed_of(column(cols, sl.o_sm)[i]), e = signed_of(column(cols, sl.o_ef)[i]);
        const uint32_t ef = (uint32_t)(e < 0 ? 0 : e > 0xfe ? 0xfe : e);
        uint32_t pat = 0;
        if (sm != 0) pat = ((sm < 0 ? 1u << 15 : 0u) | (ef << 7) | (uint32_t)((sm < 0 ? -sm : sm) - 128)) & 0xffffu;
        a.out_pat[(size_t)j * a.out_w + k] = pat;
        reinterpret_cast<int2*>(a.out_nat)[(size_t)j * a.out_w + k] = make_int2((int)sm, (int)e);
    }
    if (!MUL) {
        __syncthreads();
        for (uint32_t k = threadIdx.x; k < RS_POW_ROWS && k < a.m_pow.n; k += blockDim.x)
            if (pow_hist[k]) atomicAdd(a.m_pow.m + k, pow_hist[k]);
    }
    off = __reduce_add_sync(0xffffffffu, off);
    bad_exp = __reduce_add_sync(0xffffffffu, bad_exp);
    un_off = __reduce_add_sync(0xffffffffu, un_off);
    if ((threadIdx.x & 31u) == 0) {
        if (off) atomicAdd(a.counts, off);
        if (bad_exp) atomicAdd(a.counts + 1, bad_exp);
        if (un_off) atomicAdd(a.counts + 2, un_off);
    }
}

}  // namespace
}  // namespace zk

using namespace zk;

namespace {
// Host arrays the kernels index (groups, slots, pointer tables) go up through the context's staging ring, 8 bytes a word.
template <class T> int stage_array(zkb_ctx* ctx, const T* src, size_t n, const T** out) {
    std::vector<uint64_t> blob((n * sizeof(T) + 7) / 8 + 1, 0);
    if (n) memcpy(blob.data(), src, n * sizeof(T));
    void** d = nullptr;
    int rc = stage_ptrs(ctx, reinterpret_cast<const void* const*>(blob.data()), (int)blob.size(), &d);
    *out = reinterpret_cast<const T*>(d);
    return rc;
}
}  // namespace

extern "C" {

int zkb_witness_pre_table(zkb_ctx* ctx, uint32_t kind, uint32_t log_rows, uint32_t kmax, uint32_t round, const uint32_t* const* counters,
                          uint32_t n_counters, const uint32_t* patch_idx, const uint32_t* patch_val, uint32_t n_patch, uint32_t* const* cols,
                          uint32_t n_cols, uint32_t* m_col) {
    if (!ctx) return ZKB_EINVAL;
    static const uint32_t width[5] = {6, 3, 4, 2, 1};
    ZKB_CHECK_ARG(ctx, kind <= 4 && round <= 2 && cols && n_cols == width[kind] && log_rows >= 1 && log_rows <= 30 && kmax <= 21);
    ZKB_CHECK_ARG(ctx, (n_counters == 0 || counters) && n_counters <= 4096 && (n_patch == 0 || (patch_idx && patch_val)));
    ZKB_CHECK_ARG(ctx, m_col == nullptr || ((uintptr_t)m_col & 7) == 0);
    for (uint32_t k = 0; k < n_cols; k++) ZKB_CHECK_ARG(ctx, cols[k] != nullptr && ((uintptr_t)cols[k] & 7) == 0);
    for (uint32_t k = 0; k < n_counters; k++) ZKB_CHECK_ARG(ctx, counters[k] != nullptr);
    const uint32_t sticky = round == 0;
    uint64_t real = kind == 0 ? 256ull + (uint64_t)(kmax + 1) * (256u << sticky) : kind == 1 ? 1ull << (kmax + 1) : kind == 2 ? 1ull << 14 : 1ull << log_rows;
    // The table must fit the committed height (the rows above its own length commit zero).
    ZKB_CHECK_ARG(ctx, real <= (1ull << log_rows));
    DeviceGuard g(ctx);
    void **d_cnt = nullptr, **d_cols = nullptr;
    int rc = stage_ptrs(ctx, (const void* const*)cols, (int)n_cols, &d_cols);
    if (rc) return rc;
    if (n_counters && m_col) {
        rc = stage_ptrs(ctx, (const void* const*)counters, (int)n_counters, &d_cnt);
        if (rc) return rc;
    }
    PreCfg c{kind, log_rows, (uint32_t)real, kmax, round, sticky, n_cols, m_col ? n_counters : 0u};
    const uint32_t pairs = 1u << (log_rows - 1), grid = (pairs + 255) / 256;
    {
        ProfScope prof(ctx, "pre_table_kernel");
        auto cnt = (const uint32_t* const*)d_cnt;
        auto cl = (uint32_t* const*)d_cols;
        switch (kind) {
            case 0: pre_table_kernel<0><<<grid, 256, 0, ctx->stream>>>(cnt, cl, m_col, c); break;
            case 1: pre_table_kernel<1><<<grid, 256, 0, ctx->stream>>>(cnt, cl, m_col, c); break;
            case 2: pre_table_kernel<2><<<grid, 256, 0, ctx->stream>>>(cnt, cl, m_col, c); break;
            case 3: pre_table_kernel<3><<<grid, 256, 0, ctx->stream>>>(cnt, cl, m_col, c); break;
            default: pre_table_kernel<4><<<grid, 256, 0, ctx->stream>>>(cnt, cl, m_col, c); break;
        }
        ZKB_LAUNCH_CHECK(ctx);
    }
    if (n_patch) {
        pre_patch_kernel<<<(n_patch + 255) / 256, 256, 0, ctx->stream>>>(patch_idx, patch_val, n_patch, (uint32_t* const*)d_cols, n_cols, log_rows);
        ZKB_LAUNCH_CHECK(ctx);
    }
    return ZKB_OK;
}

static int check_tile(zkb_ctx* ctx, uint32_t shape, uint32_t log_rows, uint32_t groups, uint32_t chunks, uint32_t lead) {
    ZKB_CHECK_ARG(ctx, shape <= 2 && log_rows <= 30);
    if (shape != 2) ZKB_CHECK_ARG(ctx, groups >= 1 && chunks >= 1 && (uint64_t)groups * chunks + lead == (1ull << log_rows));
    return ZKB_OK;
}

int zkb_key_tile_flags(zkb_ctx* ctx, uint32_t shape, uint32_t log_rows, uint32_t groups, uint32_t chunks, uint32_t lead, uint32_t descending,
                       uint32_t modulus, uint32_t rw, uint32_t* flags) {
    if (!ctx) return ZKB_EINVAL;
    int rc = check_tile(ctx, shape, log_rows, groups, chunks, lead);
    if (rc) return rc;
    ZKB_CHECK_ARG(ctx, flags && modulus >= 1 && (shape != 2 || rw >= 1));
    DeviceGuard g(ctx);
    const uint32_t rows = 1u << log_rows;
    ProfScope prof(ctx, "tile_flags_kernel");
    tile_flags_kernel<<<(rows + 255) / 256, 256, 0, ctx->stream>>>(flags, shape, TileGrid{log_rows, groups, chunks, lead, descending ? 1u : 0u}, modulus, rw);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

int zkb_witness_selectors(zkb_ctx* ctx, uint32_t shape, uint32_t log_rows, uint32_t groups, uint32_t chunks, uint32_t lead, uint32_t descending,
                          const uint32_t* flags, const uint32_t* scale, uint32_t ctx_len, uint32_t n_insts, int with_scale, uint32_t* const* cols,
                          uint32_t n_cols) {
    if (!ctx) return ZKB_EINVAL;
    int rc = check_tile(ctx, shape, log_rows, groups, chunks, lead);
    if (rc) return rc;
    ZKB_CHECK_ARG(ctx, flags && cols && n_cols == (shape == 0 ? 5u : shape == 2 ? 3u : n_cols) && (shape != 1 || n_cols == 8 || n_cols == 9));
    // every group's instance must have a scale entry
    if (shape == 1 && with_scale) ZKB_CHECK_ARG(ctx, scale && ctx_len >= 1 && (groups - 1) / ctx_len < n_insts);
    for (uint32_t k = 0; k < n_cols; k++) ZKB_CHECK_ARG(ctx, cols[k] != nullptr);
    DeviceGuard g(ctx);
    void** d_cols = nullptr;
    rc = stage_ptrs(ctx, (const void* const*)cols, (int)n_cols, &d_cols);
    if (rc) return rc;
    const uint32_t rows = 1u << log_rows;
    SelCfg c{shape, TileGrid{log_rows, groups, chunks, lead, descending ? 1u : 0u}, ctx_len, (shape == 1 && with_scale) ? 1u : 0u, n_cols};
    ProfScope prof(ctx, "selectors_kernel");
    selectors_kernel<<<(rows + 255) / 256, 256, 0, ctx->stream>>>(flags, scale, (uint32_t* const*)d_cols, c);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

int zkb_witness_residual_stream(zkb_ctx* ctx, const zkb_rs_program* prog, const zkb_rs_tables* tables, const uint32_t* wit, uint32_t live_rows,
                                uint32_t log_rows, uint32_t* const* cols, uint32_t n_cols, uint32_t* out_pat, int32_t* out_nat, int32_t* in_nat,
                                const zkb_rs_mults* mults, uint32_t* counts) {
    if (!ctx) return ZKB_EINVAL;
    ZKB_CHECK_ARG(ctx, prog && tables && mults && wit && cols && out_pat && out_nat && in_nat && counts && log_rows <= 30);
    const zkb_rs_program& p = *prog;
    ZKB_CHECK_ARG(ctx, p.kind <= 1 && p.sticky <= 1 && p.kmax <= 21 && p.groups && p.n_groups >= 1 && (p.n_slots == 0 || p.slots) && (p.out_w == 0 || p.out_slot));
    ZKB_CHECK_ARG(ctx, live_rows <= (1u << log_rows) && n_cols >= 1 && n_cols <= 65536);
    ZKB_CHECK_ARG(ctx, ((uintptr_t)out_nat & 7) == 0 && ((uintptr_t)in_nat & 7) == 0);
    ZKB_CHECK_ARG(ctx, p.kind == 1 ? (tables->smul3 != nullptr && mults->smul.m != nullptr) : (tables->norm3 != nullptr && mults->pow.m && mults->norm.m && mults->frac.m));
    ZKB_CHECK_ARG(ctx, mults->val.m != nullptr && (tables->n_un == 0 || (tables->un2 && mults->un)));
    // every column index a row touches is checked here, so that the kernel needs no bounds tests
    const uint32_t slot_w = p.kind == 0 ? 13u + p.sticky : 4u;
    uint64_t n_leaves = 0;
    for (uint32_t g = 0; g < p.n_groups; g++) {
        const zkb_rs_group& gr = p.groups[g];
        ZKB_CHECK_ARG(ctx, gr.un <= tables->n_un && gr.width == (gr.un ? 4u : 2u) && gr.flat == n_leaves);
        ZKB_CHECK_ARG(ctx, (uint64_t)gr.leaf_col + (uint64_t)gr.n * gr.width <= n_cols);
        n_leaves += gr.n;
    }
    ZKB_CHECK_ARG(ctx, n_leaves >= 1 && n_leaves <= (1u << 20));
    auto col_ok = [&](uint32_t c) { return c == OFF_TABLE || c < n_cols; };
    for (uint32_t s = 0; s < p.n_slots; s++) {
        const zkb_rs_slot& sl = p.slots[s];
        ZKB_CHECK_ARG(ctx, (uint64_t)sl.base + slot_w <= n_cols && sl.o_sm < n_cols && sl.o_ef < n_cols && sl.from_slot <= 3);
        ZKB_CHECK_ARG(ctx, col_ok(sl.a_sm) && col_ok(sl.b_sm) && (sl.a_sm == OFF_TABLE || sl.a_ef < n_cols) && (sl.b_sm == OFF_TABLE || sl.b_ef < n_cols));
    }
    for (uint32_t k = 0; k < p.out_w; k++) ZKB_CHECK_ARG(ctx, p.out_slot[k] < p.n_slots);
    // Levels: a slot that reads a cell of another slot comes one level after it, and that slot must come earlier in
    // evaluation order (an operand inside a later slot's cells would be read before it is written).
    std::vector<uint32_t> level(p.n_slots, 0), owner(n_cols, OFF_TABLE);
    for (uint32_t s = 0; s < p.n_slots; s++)
        for (uint32_t c = 0; c < slot_w; c++) {
            ZKB_CHECK_ARG(ctx, owner[p.slots[s].base + c] == OFF_TABLE);  // two slots' cells overlap
            owner[p.slots[s].base + c] = s;
        }
    for (uint32_t g = 0; g < p.n_groups; g++)
        for (uint64_t c = p.groups[g].leaf_col; c < (uint64_t)p.groups[g].leaf_col + (uint64_t)p.groups[g].n * p.groups[g].width; c++)
            ZKB_CHECK_ARG(ctx, owner[c] == OFF_TABLE);  // a leaf inside a slot's cells
    uint32_t n_levels = 0;
    for (uint32_t s = 0; s < p.n_slots; s++) {
        const zkb_rs_slot& sl = p.slots[s];
        ZKB_CHECK_ARG(ctx, owner[sl.o_sm] == s && owner[sl.o_ef] == s);
        const uint32_t ops[4] = {sl.a_sm, sl.a_ef, sl.b_sm, sl.b_ef};
        for (int o = 0; o < 4; o++) {
            if (ops[o & 2] == OFF_TABLE || owner[ops[o]] == OFF_TABLE) continue;
            ZKB_CHECK_ARG(ctx, owner[ops[o]] < s);
            level[s] = std::max(level[s], level[owner[ops[o]]] + 1u);
        }
        n_levels = std::max(n_levels, level[s] + 1u);
    }
    std::vector<uint32_t> order, level_start(n_levels + 1, 0);
    for (uint32_t l = 0; l < n_levels; l++) {
        level_start[l] = (uint32_t)order.size();
        for (uint32_t s = 0; s < p.n_slots; s++)
            if (level[s] == l) order.push_back(s);
    }
    level_start[n_levels] = (uint32_t)order.size();
    for (uint32_t u = 0; u < tables->n_un; u++) ZKB_CHECK_ARG(ctx, tables->un2[u] && ((uintptr_t)tables->un2[u] & 7) == 0 && mults->un[u].m);
    for (uint32_t k = 0; k < n_cols; k++) ZKB_CHECK_ARG(ctx, cols[k] != nullptr);
    DeviceGuard g(ctx);
    RsArgs a{};
    void** d_cols = nullptr;
    int rc = stage_ptrs(ctx, (const void* const*)cols, (int)n_cols, &d_cols);
    if (rc) return rc;
    static_assert(sizeof(zkb_rs_group) == sizeof(RsGroup) && sizeof(zkb_rs_slot) == sizeof(RsSlot) && sizeof(zkb_rs_mult) == sizeof(RsMult), "layout");
    if ((rc = stage_array(ctx, reinterpret_cast<const RsGroup*>(p.groups), p.n_groups, &a.groups))) return rc;
    if ((rc = stage_array(ctx, reinterpret_cast<const RsSlot*>(p.slots), p.n_slots, &a.slots))) return rc;
    if ((rc = stage_array(ctx, p.out_slot, p.out_w, &a.out_slot))) return rc;
    if ((rc = stage_array(ctx, order.data(), order.size(), &a.order))) return rc;
    if ((rc = stage_array(ctx, level_start.data(), level_start.size(), &a.level_start))) return rc;
    if ((rc = stage_array(ctx, tables->un2, tables->n_un, &a.un2))) return rc;
    if ((rc = stage_array(ctx, reinterpret_cast<const RsMult*>(mults->un), tables->n_un, &a.m_un))) return rc;
    a.wit = wit; a.norm3 = tables->norm3; a.smul3 = tables->smul3; a.cols = (uint32_t* const*)d_cols;
    a.out_pat = out_pat; a.out_nat = out_nat; a.in_nat = in_nat; a.counts = counts;
    auto mult = [](const zkb_rs_mult& m) { return RsMult{m.m, m.m ? m.n : 0u}; };
    a.m_pow = mult(mults->pow); a.m_norm = mult(mults->norm); a.m_val = mult(mults->val); a.m_frac = mult(mults->frac); a.m_smul = mult(mults->smul);
    a.n_norm = tables->norm3 ? tables->n_norm : 0; a.n_smul = tables->smul3 ? tables->n_smul : 0; a.n_val = tables->n_val;
    a.log_rows = log_rows; a.live = live_rows; a.n_groups = p.n_groups; a.n_leaves = (uint32_t)n_leaves; a.n_slots = p.n_slots;
    a.kmax = p.kmax; a.out_w = p.out_w; a.n_levels = n_levels;
    const uint32_t rows = 1u << log_rows, grid = (rows + 31) / 32, threads = 32 * RS_LANES;
    ProfScope prof(ctx, "residual_stream_kernel");
    if (p.kind == 1) residual_stream_kernel<true, false><<<grid, threads, 0, ctx->stream>>>(a);
    else if (p.sticky) residual_stream_kernel<false, true><<<grid, threads, 0, ctx->stream>>>(a);
    else residual_stream_kernel<false, false><<<grid, threads, 0, ctx->stream>>>(a);
    ZKB_LAUNCH_CHECK(ctx);
    return ZKB_OK;
}

}  // extern "C"
