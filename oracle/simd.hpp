// TEST INFRASTRUCTURE - the timed CPU baseline's packed arithmetic: a 16-lane restatement of the reference's SIMD backend
// for the operators that carry the commitment-and-proving path's CPU time. Only bench.py's CPU legs and the tests that
// compare it with the scalar oracle use it; the product never does.
//
// What follows what:
//   PackedM31 (add, sub, mul with the even/odd 32x32->64 products and the shift-free reduction)
//       nitroo/crates/stwo/src/prover/backend/simd/m31.rs:30-330
//   circle FFT and inverse FFT on a column of packed lanes: layers whose butterfly distance is 16 lanes or more run on
//   whole vectors with a broadcast twiddle, the four lowest layers pair lanes of two neighbouring vectors with permutes
//   (the reference interleaves 16x16 transposes with three-layer loops instead; same butterflies, same twiddles,
//   same results)
//       nitroo/crates/stwo/src/prover/backend/simd/fft/rfft.rs:35, simd/fft/ifft.rs:33, simd/circle.rs:138-166, 377-443
//   Blake2s over 16 rows at once, a column's 16 consecutive rows being one message-word vector
//       nitroo/crates/stwo/src/prover/backend/simd/blake2s.rs:61-143 (compress16 :165-323)
//   out-of-domain evaluation by folding halves with packed secure-field arithmetic
//       nitroo/crates/stwo/src/prover/backend/simd/circle.rs:186-260
//   quotient numerators, 16 rows per step
//       nitroo/crates/stwo/src/prover/backend/simd/quotients.rs:34-70
// Everything else of the proof (upper Merkle layers, the combine step, FRI folds, channel, decommitment) stays on the
// scalar oracle with OpenMP: it is a few percent of the CPU time of the benchmark workload.
//
// The lanes are GCC vector extensions (64-byte vectors): compiled once with AVX-512 (one register per vector) and once
// with AVX2 (two), selected at run time. Results are identical to the scalar oracle's, word for word
// (tests/test_oracle_simd.py).
#pragma once
#include <cstdint>
#include <cstring>
#include <vector>

#include "fields.hpp"

#ifndef ZKO_SIMD_NS
#define ZKO_SIMD_NS simd_generic
#endif

namespace zko {
namespace ZKO_SIMD_NS {

typedef uint32_t v16 __attribute__((vector_size(64), aligned(4)));
typedef uint64_t v8q __attribute__((vector_size(64), aligned(4)));
typedef uint32_t v8 __attribute__((vector_size(32), aligned(4)));
typedef uint32_t v4 __attribute__((vector_size(16), aligned(4)));
typedef uint32_t v2 __attribute__((vector_size(8), aligned(4)));

static inline v16 splat(uint32_t x) { return v16{x, x, x, x, x, x, x, x, x, x, x, x, x, x, x, x}; }
static inline v16 load16(const uint32_t* p) { v16 r; memcpy(&r, p, 64); return r; }
static inline void store16(uint32_t* p, v16 v) { memcpy(p, &v, 64); }
static inline v16 vmin(v16 a, v16 b) { return a < b ? a : b; }
// simd/m31.rs: results canonical in [0, p)
static inline v16 padd(v16 a, v16 b) { v16 c = a + b; return vmin(c, c - P); }
static inline v16 psub(v16 a, v16 b) { v16 c = a - b; return vmin(c, c + P); }
static inline v16 pneg(v16 a) { return psub(splat(0), a); }
static inline v16 pmul(v16 a, v16 b) {
    const v8q lo32 = {0xffffffffull, 0xffffffffull, 0xffffffffull, 0xffffffffull, 0xffffffffull, 0xffffffffull, 0xffffffffull, 0xffffffffull};
    v8q ae = (v8q)a & lo32, ao = (v8q)a >> 32, be = (v8q)b & lo32, bo = (v8q)b >> 32;
    v8q pe = ae * be, po = ao * bo;  // 62-bit products of the even and of the odd lanes
    v8q re = (pe & (uint64_t)P) + (pe >> 31), ro = (po & (uint64_t)P) + (po >> 31);  // below 2^32
    v16 r = (v16)(re | (ro << 32));
    return vmin(r, r - P);
}

// ---- packed secure field (four coordinate vectors: a0 + a1 i + (a2 + a3 i) u)
struct PQ { v16 c[4]; };
static inline PQ pq_add(const PQ& x, const PQ& y) { return {{padd(x.c[0], y.c[0]), padd(x.c[1], y.c[1]), padd(x.c[2], y.c[2]), padd(x.c[3], y.c[3])}}; }
// CM31 product (cm31.rs:44-52)
static inline void cmul(v16 a, v16 b, v16 c, v16 d, v16& re, v16& im) {
    re = psub(pmul(a, c), pmul(b, d));
    im = padd(pmul(a, d), pmul(b, c));
}
// QM31 product (qm31.rs:80-88): (a + b u)(c + d u) = ac + R bd + (ad + bc) u, R = 2 + i
static inline PQ pq_mul(const PQ& x, const PQ& y) {
    v16 acr, aci, bdr, bdi, adr, adi, bcr, bci;
    cmul(x.c[0], x.c[1], y.c[0], y.c[1], acr, aci);
    cmul(x.c[2], x.c[3], y.c[2], y.c[3], bdr, bdi);
    cmul(x.c[0], x.c[1], y.c[2], y.c[3], adr, adi);
    cmul(x.c[2], x.c[3], y.c[0], y.c[1], bcr, bci);
    // R * bd = (2 + i)(bdr + bdi i) = (2 bdr - bdi) + (bdr + 2 bdi) i
    v16 rr = psub(padd(bdr, bdr), bdi), ri = padd(bdr, padd(bdi, bdi));
    return {{padd(acr, rr), padd(aci, ri), padd(adr, bcr), padd(adi, bci)}};
}
static inline PQ pq_splat(QM31 q) {
    uint32_t w[4];
    q.to_u32(w);
    return {{splat(w[0]), splat(w[1]), splat(w[2]), splat(w[3])}};
}

// ------------------------------------------------------------------ circle FFT on one column
template <bool INV> static inline void bfly(v16& a, v16& b, v16 t) {
    if (INV) { v16 s = padd(a, b); b = pmul(psub(a, b), t); a = s; }  // core/fft.rs:31-41
    else { v16 m = pmul(b, t); b = psub(a, m); a = padd(a, m); }      // core/fft.rs:17-27
}
// layer i >= 4 on the sub-array v[0, n) that starts at word `base` of the column: pairs are 2^i >= 16 apart; tw[h] for
// block h of the whole column (cpu/circle.rs:293-307 with 16 butterflies per step)
template <bool INV> static void layer_wide(uint32_t* v, size_t n, size_t base, unsigned i, const uint32_t* tw) {
    const size_t half = (size_t)1 << i;
    const uint32_t* tb = tw + (base >> (i + 1));
    for (size_t h = 0; h < (n >> (i + 1)); h++) {
        const v16 t = splat(tb[h]);
        uint32_t* p0 = v + (h << (i + 1));
        uint32_t* p1 = p0 + half;
        for (size_t l = 0; l < half; l += 16) {
            v16 a = load16(p0 + l), b = load16(p1 + l);
            bfly<INV>(a, b, t);
            store16(p0 + l, a);
            store16(p1 + l, b);
        }
    }
}
// layers 0..3: the partners sit inside a run of 32 values; tw has one entry per block of 2^(i+1) values
template <bool INV, int I> static void layer_narrow(uint32_t* v, size_t n, size_t base0, const uint32_t* tw) {
    for (size_t off = 0; off < n; off += 32) {
        const size_t base = base0 + off;
        v16 x = load16(v + off), y = load16(v + off + 16), a, b, t;
        const uint32_t* tp = tw + (base >> (I + 1));
        if (I == 0) {
            a = __builtin_shufflevector(x, y, 0, 2, 4, 6, 8, 10, 12, 14, 16, 18, 20, 22, 24, 26, 28, 30);
            b = __builtin_shufflevector(x, y, 1, 3, 5, 7, 9, 11, 13, 15, 17, 19, 21, 23, 25, 27, 29, 31);
            t = load16(tp);
        } else if (I == 1) {
            a = __builtin_shufflevector(x, y, 0, 1, 4, 5, 8, 9, 12, 13, 16, 17, 20, 21, 24, 25, 28, 29);
            b = __builtin_shufflevector(x, y, 2, 3, 6, 7, 10, 11, 14, 15, 18, 19, 22, 23, 26, 27, 30, 31);
            v8 t8; memcpy(&t8, tp, 32);
            t = __builtin_shufflevector(t8, t8, 0, 0, 1, 1, 2, 2, 3, 3, 4, 4, 5, 5, 6, 6, 7, 7);
        } else if (I == 2) {
            a = __builtin_shufflevector(x, y, 0, 1, 2, 3, 8, 9, 10, 11, 16, 17, 18, 19, 24, 25, 26, 27);
            b = __builtin_shufflevector(x, y, 4, 5, 6, 7, 12, 13, 14, 15, 20, 21, 22, 23, 28, 29, 30, 31);
            v4 t4; memcpy(&t4, tp, 16);
            t = __builtin_shufflevector(t4, t4, 0, 0, 0, 0, 1, 1, 1, 1, 2, 2, 2, 2, 3, 3, 3, 3);
        } else {
            a = __builtin_shufflevector(x, y, 0, 1, 2, 3, 4, 5, 6, 7, 16, 17, 18, 19, 20, 21, 22, 23);
            b = __builtin_shufflevector(x, y, 8, 9, 10, 11, 12, 13, 14, 15, 24, 25, 26, 27, 28, 29, 30, 31);
            v2 t2; memcpy(&t2, tp, 8);
            t = __builtin_shufflevector(t2, t2, 0, 0, 0, 0, 0, 0, 0, 0, 1, 1, 1, 1, 1, 1, 1, 1);
        }
        bfly<INV>(a, b, t);
        if (I == 0) {
            x = __builtin_shufflevector(a, b, 0, 16, 1, 17, 2, 18, 3, 19, 4, 20, 5, 21, 6, 22, 7, 23);
            y = __builtin_shufflevector(a, b, 8, 24, 9, 25, 10, 26, 11, 27, 12, 28, 13, 29, 14, 30, 15, 31);
        } else if (I == 1) {
            x = __builtin_shufflevector(a, b, 0, 1, 16, 17, 2, 3, 18, 19, 4, 5, 20, 21, 6, 7, 22, 23);
            y = __builtin_shufflevector(a, b, 8, 9, 24, 25, 10, 11, 26, 27, 12, 13, 28, 29, 14, 15, 30, 31);
        } else if (I == 2) {
            x = __builtin_shufflevector(a, b, 0, 1, 2, 3, 16, 17, 18, 19, 4, 5, 6, 7, 20, 21, 22, 23);
            y = __builtin_shufflevector(a, b, 8, 9, 10, 11, 24, 25, 26, 27, 12, 13, 14, 15, 28, 29, 30, 31);
        } else {
            x = __builtin_shufflevector(a, b, 0, 1, 2, 3, 4, 5, 6, 7, 16, 17, 18, 19, 20, 21, 22, 23);
            y = __builtin_shufflevector(a, b, 8, 9, 10, 11, 12, 13, 14, 15, 24, 25, 26, 27, 28, 29, 30, 31);
        }
        store16(v + off, x);
        store16(v + off + 16, y);
    }
}
template <bool INV> static void layer(uint32_t* v, size_t n, size_t base, unsigned i, const uint32_t* tw) {
    switch (i) {
        case 0: layer_narrow<INV, 0>(v, n, base, tw); break;
        case 1: layer_narrow<INV, 1>(v, n, base, tw); break;
        case 2: layer_narrow<INV, 2>(v, n, base, tw); break;
        case 3: layer_narrow<INV, 3>(v, n, base, tw); break;
        default: layer_wide<INV>(v, n, base, i, tw);
    }
}

// Layers below CACHED_LOG run block by block on 2^CACHED_LOG consecutive words (256 KiB: the block stays in the cache
// through all of them, as the reference's CACHED_FFT_LOG_SIZE = 16 does, simd/fft/mod.rs:14); the layers above it sweep
// the whole column once each.
constexpr unsigned CACHED_LOG = 16;
static inline const uint32_t* layer_tw(unsigned i, const uint32_t* const* line_tw, const uint32_t* circle_tw) { return i == 0 ? circle_tw : line_tw[i - 1]; }

// values: 2^log words (log >= 5). line_tw[k]: the twiddles of line layer k + 1 (2^(log-2-k) words), circle_tw: 2^(log-1)
// words (layer 0). Inverse: evaluations -> coefficients, scaled by 1 / n (cpu/circle.rs:28-80).
static void interpolate(uint32_t* v, unsigned log, const uint32_t* const* line_tw, const uint32_t* circle_tw, uint32_t n_inv) {
    const size_t n = (size_t)1 << log;
    const unsigned low = log < CACHED_LOG ? log : CACHED_LOG;
    for (size_t base = 0; base < n; base += (size_t)1 << low)
        for (unsigned i = 0; i < low; i++) layer<true>(v + base, (size_t)1 << low, base, i, layer_tw(i, line_tw, circle_tw));
    for (unsigned i = low; i < log; i++) layer<true>(v, n, 0, i, layer_tw(i, line_tw, circle_tw));
    const v16 s = splat(n_inv);
    for (size_t j = 0; j < n; j += 16) store16(v + j, pmul(load16(v + j), s));
}
// Forward on an array already zero-extended to 2^log words (cpu/circle.rs:182-228).
static void evaluate(uint32_t* v, unsigned log, const uint32_t* const* line_tw, const uint32_t* circle_tw) {
    const size_t n = (size_t)1 << log;
    const unsigned low = log < CACHED_LOG ? log : CACHED_LOG;
    for (unsigned i = log; i-- > low;) layer<false>(v, n, 0, i, layer_tw(i, line_tw, circle_tw));
    for (size_t base = 0; base < n; base += (size_t)1 << low)
        for (unsigned i = low; i-- > 0;) layer<false>(v + base, (size_t)1 << low, base, i, layer_tw(i, line_tw, circle_tw));
}

// ------------------------------------------------------------------ Blake2s over 16 rows (RFC 7693; simd/blake2s.rs)
static inline v16 rotr(v16 x, int r) { return (x >> r) | (x << (32 - r)); }
static const uint32_t IV[8] = {0x6A09E667u, 0xBB67AE85u, 0x3C6EF372u, 0xA54FF53Au, 0x510E527Fu, 0x9B05688Cu, 0x1F83D9ABu, 0x5BE0CD19u};
static constexpr uint8_t SIGMA[10][16] = {
    {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15}, {14, 10, 4, 8, 9, 15, 13, 6, 1, 12, 0, 2, 11, 7, 5, 3},
    {11, 8, 12, 0, 5, 2, 15, 13, 10, 14, 3, 6, 7, 1, 9, 4}, {7, 9, 3, 1, 13, 12, 11, 14, 2, 6, 5, 10, 4, 0, 15, 8},
    {9, 0, 5, 7, 2, 4, 10, 15, 14, 1, 11, 12, 6, 8, 3, 13}, {2, 12, 6, 10, 0, 11, 8, 3, 4, 13, 7, 5, 15, 14, 1, 9},
    {12, 5, 1, 15, 14, 13, 4, 10, 0, 7, 6, 3, 9, 2, 8, 11}, {13, 11, 7, 14, 12, 1, 3, 9, 5, 0, 15, 4, 8, 6, 2, 10},
    {6, 15, 14, 9, 11, 3, 0, 8, 12, 2, 13, 7, 1, 4, 10, 5}, {10, 2, 8, 4, 7, 6, 1, 5, 15, 11, 9, 14, 3, 12, 13, 0}};
template <int R> static inline void blake_round(v16 (&v)[16], const v16 (&m)[16]) {
    constexpr const uint8_t* s = SIGMA[R];
#define ZKO_G(a, b, c, d, x, y)                                    \
    v[a] = v[a] + v[b] + m[x]; v[d] = rotr(v[d] ^ v[a], 16);       \
    v[c] = v[c] + v[d];        v[b] = rotr(v[b] ^ v[c], 12);       \
    v[a] = v[a] + v[b] + m[y]; v[d] = rotr(v[d] ^ v[a], 8);        \
    v[c] = v[c] + v[d];        v[b] = rotr(v[b] ^ v[c], 7);
    ZKO_G(0, 4, 8, 12, s[0], s[1])   ZKO_G(1, 5, 9, 13, s[2], s[3])
    ZKO_G(2, 6, 10, 14, s[4], s[5])  ZKO_G(3, 7, 11, 15, s[6], s[7])
    ZKO_G(0, 5, 10, 15, s[8], s[9])  ZKO_G(1, 6, 11, 12, s[10], s[11])
    ZKO_G(2, 7, 8, 13, s[12], s[13]) ZKO_G(3, 4, 9, 14, s[14], s[15])
#undef ZKO_G
}
static inline void compress16(v16 (&h)[8], const v16 (&m)[16], uint64_t t, bool last) {
    v16 v[16];
    for (int i = 0; i < 8; i++) { v[i] = h[i]; v[8 + i] = splat(IV[i]); }
    v[12] ^= splat((uint32_t)t);
    v[13] ^= splat((uint32_t)(t >> 32));
    if (last) v[14] = ~v[14];
    blake_round<0>(v, m); blake_round<1>(v, m); blake_round<2>(v, m); blake_round<3>(v, m); blake_round<4>(v, m);
    blake_round<5>(v, m); blake_round<6>(v, m); blake_round<7>(v, m); blake_round<8>(v, m); blake_round<9>(v, m);
    for (int i = 0; i < 8; i++) h[i] ^= v[i] ^ v[8 + i];
}
// Leaf layer without children: out[row] (8 words) = Blake2s(col_0[row] || col_1[row] || ...), each digest word taken mod p
// when m31 is set (core/vcs/blake2_merkle.rs:18-39, cpu/blake2s.rs:13-26). n rows, a multiple of 16; ncols >= 1.
// Rows are taken in tiles of 1024 and, inside a tile, sixteen columns at a time: each column is then read in runs of
// 4 KiB instead of 64 bytes from hundreds of arrays in turn; the states of the tile's 64 row groups wait in the cache.
static void leaf_hashes(uint32_t* out, const uint32_t* const* cols, size_t ncols, size_t n, bool m31) {
    const size_t TILE = n < 1024 ? n : 1024;
#pragma omp parallel for schedule(static)
    for (size_t tile = 0; tile < n; tile += TILE) {
        const size_t groups = TILE / 16;
        std::vector<v16> st(groups * 8);
        for (size_t g = 0; g < groups; g++) {
            for (int i = 0; i < 8; i++) st[8 * g + i] = splat(IV[i]);
            st[8 * g] ^= splat(0x01010020u);  // digest length 32, no key, fanout 1, depth 1
        }
        const size_t total = 4 * ncols;
        for (size_t c0 = 0; c0 < ncols; c0 += 16) {
            const bool last = c0 + 16 >= ncols;
            for (size_t g = 0; g < groups; g++) {
                const size_t row = tile + 16 * g;
                v16 m[16], h[8];
                for (size_t j = 0; j < 16; j++) m[j] = c0 + j < ncols ? load16(cols[c0 + j] + row) : splat(0);
                for (int i = 0; i < 8; i++) h[i] = st[8 * g + i];
                compress16(h, m, last ? total : 4 * (c0 + 16), last);
                for (int i = 0; i < 8; i++) st[8 * g + i] = h[i];
            }
        }
        for (size_t g = 0; g < groups; g++) {
            uint32_t tmp[8][16];
            for (int i = 0; i < 8; i++) {
                v16 w = st[8 * g + i];
                if (m31) { v16 r = (w & P) + (w >> 31); w = vmin(r, r - P); }
                store16(tmp[i], w);
            }
            for (int l = 0; l < 16; l++)
                for (int i = 0; i < 8; i++) out[8 * (tile + 16 * g + l) + i] = tmp[i][l];
        }
    }
}

// Inner layer without columns: out[i] = Blake2s(prev[2i] || prev[2i+1]), one 64-byte block per node. n nodes, a multiple of 16.
static void node_hashes(uint32_t* out, const uint32_t* prev, size_t n, bool m31) {
#pragma omp parallel for schedule(static)
    for (size_t node = 0; node < n; node += 16) {
        uint32_t in[16][16];  // [word][lane]
        for (int l = 0; l < 16; l++)
            for (int j = 0; j < 16; j++) in[j][l] = prev[16 * (node + l) + j];
        v16 h[8], m[16];
        for (int i = 0; i < 8; i++) h[i] = splat(IV[i]);
        h[0] ^= splat(0x01010020u);
        for (int j = 0; j < 16; j++) m[j] = load16(in[j]);
        compress16(h, m, 64, true);
        uint32_t tmp[8][16];
        for (int i = 0; i < 8; i++) {
            v16 w = h[i];
            if (m31) { v16 r = (w & P) + (w >> 31); w = vmin(r, r - P); }
            store16(tmp[i], w);
        }
        for (int l = 0; l < 16; l++)
            for (int i = 0; i < 8; i++) out[8 * (node + l) + i] = tmp[i][l];
    }
}

// ------------------------------------------------------------------ out-of-domain evaluation (cpu/circle.rs:82-100 by halves)
// factors: the folding factors in the order poly.hpp's fold() takes them (factors[0] joins the two halves of the whole array).
static QM31 eval_by_folding(const uint32_t* coeffs, size_t n, const QM31* factors) {
    if (n < 64) return QM31();  // callers use the scalar path below 64 coefficients
    size_t half = n / 2;
    std::vector<uint32_t> buf(4 * half);
    uint32_t* c[4] = {buf.data(), buf.data() + half, buf.data() + 2 * half, buf.data() + 3 * half};
    {
        PQ f = pq_splat(factors[0]);
        for (size_t j = 0; j < half; j += 16) {
            v16 l = load16(coeffs + j), r = load16(coeffs + half + j);
            store16(c[0] + j, padd(l, pmul(r, f.c[0])));
            for (int k = 1; k < 4; k++) store16(c[k] + j, pmul(r, f.c[k]));
        }
    }
    size_t len = half;
    int fi = 1;
    while (len >= 32) {
        size_t h2 = len / 2;
        PQ f = pq_splat(factors[fi++]);
        for (size_t j = 0; j < h2; j += 16) {
            PQ l = {{load16(c[0] + j), load16(c[1] + j), load16(c[2] + j), load16(c[3] + j)}};
            PQ r = {{load16(c[0] + h2 + j), load16(c[1] + h2 + j), load16(c[2] + h2 + j), load16(c[3] + h2 + j)}};
            PQ o = pq_add(l, pq_mul(r, f));
            for (int k = 0; k < 4; k++) store16(c[k] + j, o.c[k]);
        }
        len = h2;
    }
    // the last 16 values with scalar secure-field arithmetic
    std::vector<QM31> tail(len);
    for (size_t j = 0; j < len; j++) tail[j] = QM31::from_u32(c[0][j], c[1][j], c[2][j], c[3][j]);
    while (len > 1) {
        size_t h2 = len / 2;
        for (size_t j = 0; j < h2; j++) tail[j] = tail[j] + tail[h2 + j] * factors[fi];
        fi++;
        len = h2;
    }
    return tail[0];
}

// ------------------------------------------------------------------ quotient numerators (cpu/quotients.rs:22-45)
// acc[row] = sum_j c_j * cols[idx_j][row] - sum_j b_j, QM31 array-of-structs output (4 words per row). n a multiple of 16.
static void numerators(uint32_t* acc, const uint32_t* const* cols, const size_t* idx, const QM31* c, size_t k, QM31 b_sum, size_t n) {
    std::vector<uint32_t> cw(4 * k);
    for (size_t j = 0; j < k; j++) c[j].to_u32(&cw[4 * j]);
    const PQ bs = pq_splat(b_sum);
    // tiles of 1024 rows: every column is read in runs of 4 KiB while the tile's sums stay in the cache
    const size_t TILE = n < 1024 ? n : 1024;
#pragma omp parallel for schedule(static)
    for (size_t tile = 0; tile < n; tile += TILE) {
        const size_t groups = TILE / 16;
        std::vector<v16> a(4 * groups, splat(0));
        for (size_t j = 0; j < k; j++) {
            const uint32_t* col = cols[idx[j]] + tile;
            const v16 c0 = splat(cw[4 * j]), c1 = splat(cw[4 * j + 1]), c2 = splat(cw[4 * j + 2]), c3 = splat(cw[4 * j + 3]);
            for (size_t g = 0; g < groups; g++) {
                v16 x = load16(col + 16 * g);
                a[4 * g] = padd(a[4 * g], pmul(x, c0));
                a[4 * g + 1] = padd(a[4 * g + 1], pmul(x, c1));
                a[4 * g + 2] = padd(a[4 * g + 2], pmul(x, c2));
                a[4 * g + 3] = padd(a[4 * g + 3], pmul(x, c3));
            }
        }
        for (size_t g = 0; g < groups; g++) {
            uint32_t t[4][16];
            for (int q = 0; q < 4; q++) store16(t[q], psub(a[4 * g + q], bs.c[q]));
            for (int l = 0; l < 16; l++)
                for (int q = 0; q < 4; q++) acc[4 * (tile + 16 * g + l) + q] = t[q][l];
        }
    }
}

}  // namespace ZKO_SIMD_NS
}  // namespace zko
