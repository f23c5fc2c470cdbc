// TEST INFRASTRUCTURE ONLY. CPU oracle: a plain C++ restatement of the reference's scalar
// CpuBackend arithmetic. Nothing in the product library links, includes or calls this.
//
// Field tower over the Mersenne prime p = 2^31 - 1:
//   M31   follows nitroo/crates/stwo/src/core/fields/m31.rs:32-108 (reduce :58-60, inverse :192-200)
//   CM31  follows nitroo/crates/stwo/src/core/fields/cm31.rs:17-73  (M31[i]/(i^2+1))
//   QM31  follows nitroo/crates/stwo/src/core/fields/qm31.rs:14-128 (CM31[u]/(u^2-2-i))
#pragma once
#include <cstdint>
#include <cstddef>
#include <vector>
#include <cassert>

namespace zko {

constexpr uint32_t P = 2147483647u;

struct M31 {
    uint32_t v;
    constexpr M31() : v(0) {}
    constexpr explicit M31(uint32_t x) : v(x) {}
    // m31.rs:58-60 — valid for val in [0, P^2).
    static constexpr M31 reduce(uint64_t val) {
        return M31((uint32_t)((((((val >> 31) + val + 1) >> 31) + val)) & P));
    }
    // m31.rs:44-46 — val in [0, 2P).
    static constexpr M31 partial_reduce(uint32_t val) { return M31(val >= P ? val - P : val); }
    static constexpr M31 from_u32(uint32_t x) { return reduce((uint64_t)x); }
    static constexpr M31 from_i32(int32_t x) {
        if (x < 0) return reduce(2ull * P - (uint64_t)(-(int64_t)x));
        return reduce((uint64_t)x);
    }
    constexpr bool is_zero() const { return v == 0; }
    M31 square() const;
    M31 inverse() const;
    M31 dbl() const;
};
constexpr M31 operator+(M31 a, M31 b) { return M31::partial_reduce(a.v + b.v); }
constexpr M31 operator-(M31 a) { return M31::partial_reduce(P - a.v); }
constexpr M31 operator-(M31 a, M31 b) { return M31::partial_reduce(a.v + P - b.v); }
constexpr M31 operator*(M31 a, M31 b) { return M31::reduce((uint64_t)a.v * (uint64_t)b.v); }
constexpr bool operator==(M31 a, M31 b) { return a.v == b.v; }
constexpr bool operator!=(M31 a, M31 b) { return a.v != b.v; }
inline M31 M31::square() const { return *this * *this; }
inline M31 M31::dbl() const { return *this + *this; }

template <class T> inline T sqn(T v, int n) { for (int i = 0; i < n; i++) v = v * v; return v; }
// m31.rs:192-200 — v^(p-2) by the 37-multiplication addition chain.
inline M31 M31::inverse() const {
    assert(!is_zero());
    M31 v = *this;
    M31 t0 = sqn(v, 2) * v;
    M31 t1 = sqn(t0, 1) * t0;
    M31 t2 = sqn(t1, 3) * t0;
    M31 t3 = sqn(t2, 1) * t0;
    M31 t4 = sqn(t3, 8) * t3;
    M31 t5 = sqn(t4, 8) * t3;
    return sqn(t5, 7) * t2;
}

struct CM31 {
    M31 a, b;  // a + b i
    constexpr CM31() {}
    constexpr CM31(M31 a_, M31 b_) : a(a_), b(b_) {}
    constexpr explicit CM31(M31 a_) : a(a_), b() {}
    bool is_zero() const { return a.is_zero() && b.is_zero(); }
    CM31 square() const;
    CM31 inverse() const;
};
constexpr CM31 operator+(CM31 x, CM31 y) { return CM31(x.a + y.a, x.b + y.b); }
constexpr CM31 operator-(CM31 x, CM31 y) { return CM31(x.a - y.a, x.b - y.b); }
constexpr CM31 operator-(CM31 x) { return CM31(-x.a, -x.b); }
// cm31.rs:44-52
constexpr CM31 operator*(CM31 x, CM31 y) {
    return CM31(x.a * y.a - x.b * y.b, x.a * y.b + x.b * y.a);
}
constexpr CM31 operator*(CM31 x, M31 y) { return CM31(x.a * y, x.b * y); }
constexpr bool operator==(CM31 x, CM31 y) { return x.a == y.a && x.b == y.b; }
inline CM31 CM31::square() const { return *this * *this; }
// cm31.rs:66-72
inline CM31 CM31::inverse() const {
    assert(!is_zero());
    return CM31(a, -b) * (a.square() + b.square()).inverse();
}

struct QM31 {
    CM31 a, b;  // a + b u
    constexpr QM31() {}
    constexpr QM31(CM31 a_, CM31 b_) : a(a_), b(b_) {}
    constexpr explicit QM31(M31 x) : a(x), b() {}
    static constexpr QM31 from_u32(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3) {
        return QM31(CM31(M31(c0), M31(c1)), CM31(M31(c2), M31(c3)));
    }
    static constexpr QM31 from_m31s(M31 c0, M31 c1, M31 c2, M31 c3) {
        return QM31(CM31(c0, c1), CM31(c2, c3));
    }
    static constexpr QM31 zero() { return QM31(); }
    static constexpr QM31 one() { return QM31(M31(1)); }
    void to_u32(uint32_t out[4]) const { out[0] = a.a.v; out[1] = a.b.v; out[2] = b.a.v; out[3] = b.b.v; }
    bool is_zero() const { return a.is_zero() && b.is_zero(); }
    QM31 square() const;
    QM31 inverse() const;
    QM31 dbl() const;
    // qm31.rs:60-62
    QM31 mul_cm31(CM31 r) const { return QM31(a * r, b * r); }
    // complex conjugate with respect to CM31: a - b u
    QM31 conj() const { return QM31(a, -b); }
};
constexpr CM31 QM31_R(M31(2), M31(1));  // qm31.rs:14
constexpr QM31 operator+(QM31 x, QM31 y) { return QM31(x.a + y.a, x.b + y.b); }
constexpr QM31 operator-(QM31 x, QM31 y) { return QM31(x.a - y.a, x.b - y.b); }
constexpr QM31 operator-(QM31 x) { return QM31(-x.a, -x.b); }
// qm31.rs:80-88
constexpr QM31 operator*(QM31 x, QM31 y) {
    return QM31(x.a * y.a + QM31_R * x.b * y.b, x.a * y.b + x.b * y.a);
}
constexpr QM31 operator*(QM31 x, M31 y) { return QM31(x.a * y, x.b * y); }
constexpr QM31 operator+(QM31 x, M31 y) { return QM31(CM31(x.a.a + y, x.a.b), x.b); }
constexpr QM31 operator-(QM31 x, M31 y) { return QM31(CM31(x.a.a - y, x.a.b), x.b); }
constexpr bool operator==(QM31 x, QM31 y) { return x.a == y.a && x.b == y.b; }
constexpr bool operator!=(QM31 x, QM31 y) { return !(x == y); }
inline QM31 QM31::square() const { return *this * *this; }
inline QM31 QM31::dbl() const { return *this + *this; }
// qm31.rs:118-127
inline QM31 QM31::inverse() const {
    assert(!is_zero());
    CM31 b2 = b.square();
    CM31 ib2(-b2.b, b2.a);
    CM31 denom = a.square() - (b2 + b2 + ib2);
    CM31 dinv = denom.inverse();
    return QM31(a * dinv, -b * dinv);
}
inline QM31 operator/(QM31 x, QM31 y) { return x * y.inverse(); }

using SecureField = QM31;
using BaseField = M31;

}  // namespace zko
