// Field arithmetic for the Circle-STARK operators: M31 (p = 2^31 - 1), CM31 = M31[i]/(i^2+1),
// QM31 = CM31[u]/(u^2 - 2 - i). Usable from device and host code.
//
// Every value stored to memory is canonical, i.e. in [0, p): the reference's backends compare and
// hash raw words (nitroo/crates/stwo/src/core/fields/m31.rs:58-60 gives the reduction,
// cm31.rs:44-52 and qm31.rs:80-88 the extension products). Products are accumulated unreduced in
// 64 bits and folded once per output coordinate, which is exact because 2^31 = 1 (mod p).
#pragma once
#include <cstdint>

#ifdef __CUDACC__
#define ZK_HD __host__ __device__ __forceinline__
#else
#define ZK_HD inline
#endif

namespace zk {

constexpr uint32_t P = 0x7fffffffu;
constexpr uint64_t P_SQ = (uint64_t)P * (uint64_t)P;

ZK_HD uint32_t umin32(uint32_t a, uint32_t b) { return a < b ? a : b; }

// a, b in [0, p) -> canonical.
ZK_HD uint32_t m31_add(uint32_t a, uint32_t b) { uint32_t s = a + b; return umin32(s, s - P); }
ZK_HD uint32_t m31_sub(uint32_t a, uint32_t b) { uint32_t d = a - b; return umin32(d, d + P); }
ZK_HD uint32_t m31_neg(uint32_t a) { return a ? P - a : 0u; }
ZK_HD uint32_t m31_dbl(uint32_t a) { return m31_add(a, a); }

// Any 64-bit value -> canonical residue.
ZK_HD uint32_t m31_reduce64(uint64_t v) {
    uint32_t lo = (uint32_t)v, hi = (uint32_t)(v >> 32);
    // v = hi * 2^32 + lo = 2*hi + lo (mod p); split so that the sum stays below 2^32.
    uint32_t s = (lo & P) + (lo >> 31) + ((hi << 1) & P) + (hi >> 30);
    s = (s & P) + (s >> 31);  // <= p + 1
    return umin32(s, s - P);
}
// Product of two canonical values.
ZK_HD uint32_t m31_mul(uint32_t a, uint32_t b) {
    uint64_t p = (uint64_t)a * b;  // < 2^62
    uint32_t s = ((uint32_t)p & P) + (uint32_t)(p >> 31);
    return umin32(s, s - P);
}
ZK_HD uint32_t m31_sqr(uint32_t a) { return m31_mul(a, a); }
ZK_HD uint32_t m31_sqn(uint32_t v, int n) { for (int i = 0; i < n; i++) v = m31_sqr(v); return v; }
// v^(p-2): 37 multiplications, the addition chain of m31.rs:192-200.
ZK_HD uint32_t m31_inv(uint32_t v) {
    uint32_t t0 = m31_mul(m31_sqn(v, 2), v);
    uint32_t t1 = m31_mul(m31_sqn(t0, 1), t0);
    uint32_t t2 = m31_mul(m31_sqn(t1, 3), t0);
    uint32_t t3 = m31_mul(m31_sqn(t2, 1), t0);
    uint32_t t4 = m31_mul(m31_sqn(t3, 8), t3);
    uint32_t t5 = m31_mul(m31_sqn(t4, 8), t3);
    return m31_mul(m31_sqn(t5, 7), t2);
}

struct cm31 { uint32_t a, b; };
ZK_HD cm31 cm31_add(cm31 x, cm31 y) { return {m31_add(x.a, y.a), m31_add(x.b, y.b)}; }
ZK_HD cm31 cm31_sub(cm31 x, cm31 y) { return {m31_sub(x.a, y.a), m31_sub(x.b, y.b)}; }
ZK_HD cm31 cm31_mul(cm31 x, cm31 y) {
    uint64_t re = (uint64_t)x.a * y.a + (P_SQ - (uint64_t)x.b * y.b);
    uint64_t im = (uint64_t)x.a * y.b + (uint64_t)x.b * y.a;
    return {m31_reduce64(re), m31_reduce64(im)};
}
ZK_HD cm31 cm31_mul_m31(cm31 x, uint32_t y) { return {m31_mul(x.a, y), m31_mul(x.b, y)}; }
// 1/(a+bi) = (a-bi)/(a^2+b^2), cm31.rs:66-72
ZK_HD cm31 cm31_inv(cm31 x) {
    uint32_t n = m31_reduce64((uint64_t)x.a * x.a + (uint64_t)x.b * x.b);
    uint32_t ni = m31_inv(n);
    return {m31_mul(x.a, ni), m31_mul(m31_neg(x.b), ni)};
}

// c[0] + c[1] i + (c[2] + c[3] i) u
struct qm31 { uint32_t c[4]; };
ZK_HD qm31 qm31_zero() { return {{0, 0, 0, 0}}; }
ZK_HD qm31 qm31_one() { return {{1, 0, 0, 0}}; }
ZK_HD qm31 qm31_from_m31(uint32_t v) { return {{v, 0, 0, 0}}; }
ZK_HD qm31 qm31_add(qm31 x, qm31 y) {
    return {{m31_add(x.c[0], y.c[0]), m31_add(x.c[1], y.c[1]), m31_add(x.c[2], y.c[2]), m31_add(x.c[3], y.c[3])}};
}
ZK_HD qm31 qm31_sub(qm31 x, qm31 y) {
    return {{m31_sub(x.c[0], y.c[0]), m31_sub(x.c[1], y.c[1]), m31_sub(x.c[2], y.c[2]), m31_sub(x.c[3], y.c[3])}};
}
ZK_HD qm31 qm31_neg(qm31 x) { return {{m31_neg(x.c[0]), m31_neg(x.c[1]), m31_neg(x.c[2]), m31_neg(x.c[3])}}; }
ZK_HD qm31 qm31_dbl(qm31 x) { return qm31_add(x, x); }
ZK_HD qm31 qm31_mul_m31(qm31 x, uint32_t y) {
    return {{m31_mul(x.c[0], y), m31_mul(x.c[1], y), m31_mul(x.c[2], y), m31_mul(x.c[3], y)}};
}
ZK_HD bool qm31_eq(qm31 x, qm31 y) {
    return x.c[0] == y.c[0] && x.c[1] == y.c[1] && x.c[2] == y.c[2] && x.c[3] == y.c[3];
}
ZK_HD bool qm31_is_zero(qm31 x) { return (x.c[0] | x.c[1] | x.c[2] | x.c[3]) == 0; }
// (A + B u)(C + D u) = (AC + (2+i) BD) + (AD + BC) u, qm31.rs:80-88.
// Sixteen 62-bit products; at most four are summed (plus p^2 offsets for the subtracted ones)
// before a fold, so nothing overflows 64 bits: 4 * p^2 < 2^64.
ZK_HD qm31 qm31_mul(qm31 x, qm31 y) {
    const uint32_t x0 = x.c[0], x1 = x.c[1], x2 = x.c[2], x3 = x.c[3];
    const uint32_t y0 = y.c[0], y1 = y.c[1], y2 = y.c[2], y3 = y.c[3];
    // BD = br + bi i
    uint32_t br = m31_reduce64((uint64_t)x2 * y2 + (P_SQ - (uint64_t)x3 * y3));
    uint32_t bi = m31_reduce64((uint64_t)x2 * y3 + (uint64_t)x3 * y2);
    // (2+i)(br + bi i) = (2 br - bi) + (br + 2 bi) i
    uint64_t r0 = (uint64_t)x0 * y0 + (P_SQ - (uint64_t)x1 * y1) + 2ull * br + (uint64_t)(P - bi);
    uint64_t r1 = (uint64_t)x0 * y1 + (uint64_t)x1 * y0 + (uint64_t)br + 2ull * bi;
    uint64_t r2 = (uint64_t)x0 * y2 + (uint64_t)x2 * y0 + (2 * P_SQ - (uint64_t)x1 * y3 - (uint64_t)x3 * y1);
    uint64_t r3 = (uint64_t)x0 * y3 + (uint64_t)x1 * y2 + (uint64_t)x2 * y1 + (uint64_t)x3 * y0;
    return {{m31_reduce64(r0), m31_reduce64(r1), m31_reduce64(r2), m31_reduce64(r3)}};
}
ZK_HD qm31 qm31_sqr(qm31 x) { return qm31_mul(x, x); }
ZK_HD qm31 qm31_mul_cm31(qm31 x, cm31 y) {
    cm31 a = cm31_mul({x.c[0], x.c[1]}, y), b = cm31_mul({x.c[2], x.c[3]}, y);
    return {{a.a, a.b, b.a, b.b}};
}
// (a + bu)^-1 = (a - bu) / (a^2 - (2+i) b^2), qm31.rs:118-127
ZK_HD qm31 qm31_inv(qm31 x) {
    cm31 a{x.c[0], x.c[1]}, b{x.c[2], x.c[3]};
    cm31 b2 = cm31_mul(b, b);
    cm31 ib2{m31_neg(b2.b), b2.a};
    cm31 denom = cm31_sub(cm31_mul(a, a), cm31_add(cm31_add(b2, b2), ib2));
    cm31 di = cm31_inv(denom);
    cm31 ra = cm31_mul(a, di), rb = cm31_mul({m31_neg(b.a), m31_neg(b.b)}, di);
    return {{ra.a, ra.b, rb.a, rb.b}};
}

// Circle group law over M31 (nitroo/crates/stwo/src/core/circle.rs:103-113).
struct cpoint { uint32_t x, y; };
ZK_HD cpoint cpoint_add(cpoint p, cpoint q) {
    uint64_t x = (uint64_t)p.x * q.x + (P_SQ - (uint64_t)p.y * q.y);
    uint64_t y = (uint64_t)p.x * q.y + (uint64_t)p.y * q.x;
    return {m31_reduce64(x), m31_reduce64(y)};
}
// pi(x) = 2x^2 - 1 (circle.rs:28-31)
ZK_HD uint32_t m31_double_x(uint32_t x) { uint32_t s = m31_sqr(x); return m31_sub(m31_add(s, s), 1u); }
ZK_HD qm31 qm31_double_x(qm31 x) { qm31 s = qm31_sqr(x); return qm31_sub(qm31_add(s, s), qm31_one()); }

}  // namespace zk
