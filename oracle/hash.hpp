// TEST INFRASTRUCTURE ONLY (CPU oracle; see fields.hpp).
//
// Blake2s-256 (RFC 7693; the reference takes it from the `blake2` crate, version 0.10.6, which
// is not vendored — restated here from the RFC), the Merkle node hasher, the Fiat-Shamir channel,
// query drawing and proof-of-work. Follows
//   nitroo/crates/stwo/src/core/vcs/blake2_hash.rs:73-118   (hasher wrapper, reduce_to_m31)
//   nitroo/crates/stwo/src/core/vcs/blake2_merkle.rs:18-59  (hash_node, mix_root)
//   nitroo/crates/stwo/src/prover/backend/cpu/blake2s.rs:13-26 (commit_on_layer)
//   nitroo/crates/stwo/src/core/channel/blake2s.rs:20-141   (channel)
//   nitroo/crates/stwo/src/core/queries.rs:11-70            (draw_queries, Queries)
//   nitroo/crates/stwo/src/prover/backend/cpu/grind.rs:6-15 and
//   nitroo/crates/stwo/src/prover/backend/simd/grind.rs:18-25 (smallest nonce wins)
#pragma once
#include "accel.hpp"
#include "fields.hpp"
#include <array>
#include <cstring>
#include <set>
#include <algorithm>

namespace zko {

struct Blake2s {
    uint32_t h[8];
    uint8_t buf[64];
    size_t buflen = 0;
    uint64_t t = 0;
    static constexpr uint32_t IV[8] = {0x6A09E667u, 0xBB67AE85u, 0x3C6EF372u, 0xA54FF53Au,
                                       0x510E527Fu, 0x9B05688Cu, 0x1F83D9ABu, 0x5BE0CD19u};
    static constexpr uint8_t SIGMA[10][16] = {
        {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15},
        {14, 10, 4, 8, 9, 15, 13, 6, 1, 12, 0, 2, 11, 7, 5, 3},
        {11, 8, 12, 0, 5, 2, 15, 13, 10, 14, 3, 6, 7, 1, 9, 4},
        {7, 9, 3, 1, 13, 12, 11, 14, 2, 6, 5, 10, 4, 0, 15, 8},
        {9, 0, 5, 7, 2, 4, 10, 15, 14, 1, 11, 12, 6, 8, 3, 13},
        {2, 12, 6, 10, 0, 11, 8, 3, 4, 13, 7, 5, 15, 14, 1, 9},
        {12, 5, 1, 15, 14, 13, 4, 10, 0, 7, 6, 3, 9, 2, 8, 11},
        {13, 11, 7, 14, 12, 1, 3, 9, 5, 0, 15, 4, 8, 6, 2, 10},
        {6, 15, 14, 9, 11, 3, 0, 8, 12, 2, 13, 7, 1, 4, 10, 5},
        {10, 2, 8, 4, 7, 6, 1, 5, 15, 11, 9, 14, 3, 12, 13, 0}};
    Blake2s() {
        for (int i = 0; i < 8; i++) h[i] = IV[i];
        h[0] ^= 0x01010020u;  // digest length 32, no key, fanout 1, depth 1
    }
    static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
    static void compress(uint32_t h[8], const uint32_t m[16], uint64_t t, bool last) {
        uint32_t v[16];
        for (int i = 0; i < 8; i++) { v[i] = h[i]; v[i + 8] = IV[i]; }
        v[12] ^= (uint32_t)t;
        v[13] ^= (uint32_t)(t >> 32);
        if (last) v[14] = ~v[14];
        auto G = [&](int a, int b, int c, int d, uint32_t x, uint32_t y) {
            v[a] = v[a] + v[b] + x; v[d] = rotr(v[d] ^ v[a], 16);
            v[c] = v[c] + v[d];     v[b] = rotr(v[b] ^ v[c], 12);
            v[a] = v[a] + v[b] + y; v[d] = rotr(v[d] ^ v[a], 8);
            v[c] = v[c] + v[d];     v[b] = rotr(v[b] ^ v[c], 7);
        };
        for (int r = 0; r < 10; r++) {
            const uint8_t* s = SIGMA[r];
            G(0, 4, 8, 12, m[s[0]], m[s[1]]);
            G(1, 5, 9, 13, m[s[2]], m[s[3]]);
            G(2, 6, 10, 14, m[s[4]], m[s[5]]);
            G(3, 7, 11, 15, m[s[6]], m[s[7]]);
            G(0, 5, 10, 15, m[s[8]], m[s[9]]);
            G(1, 6, 11, 12, m[s[10]], m[s[11]]);
            G(2, 7, 8, 13, m[s[12]], m[s[13]]);
            G(3, 4, 9, 14, m[s[14]], m[s[15]]);
        }
        for (int i = 0; i < 8; i++) h[i] ^= v[i] ^ v[i + 8];
    }
    void flush_block(bool last) {
        uint32_t m[16];
        for (int i = 0; i < 16; i++)
            m[i] = (uint32_t)buf[4 * i] | ((uint32_t)buf[4 * i + 1] << 8) | ((uint32_t)buf[4 * i + 2] << 16) |
                   ((uint32_t)buf[4 * i + 3] << 24);
        compress(h, m, t, last);
    }
    void update(const void* data, size_t len) {
        const uint8_t* p = (const uint8_t*)data;
        while (len) {
            if (buflen == 64) {  // only flush a full buffer when more data follows
                t += 64;
                flush_block(false);
                buflen = 0;
            }
            size_t k = std::min(len, 64 - buflen);
            memcpy(buf + buflen, p, k);
            buflen += k; p += k; len -= k;
        }
    }
    void update_u32(uint32_t w) {
        uint8_t b[4] = {(uint8_t)w, (uint8_t)(w >> 8), (uint8_t)(w >> 16), (uint8_t)(w >> 24)};
        update(b, 4);
    }
    std::array<uint8_t, 32> finalize() {
        t += buflen;
        memset(buf + buflen, 0, 64 - buflen);
        flush_block(true);
        std::array<uint8_t, 32> out;
        for (int i = 0; i < 8; i++)
            for (int j = 0; j < 4; j++) out[4 * i + j] = (uint8_t)(h[i] >> (8 * j));
        return out;
    }
};

using Hash = std::array<uint8_t, 32>;

inline uint32_t load_le32(const uint8_t* p) {
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}
inline void store_le32(uint8_t* p, uint32_t w) {
    p[0] = (uint8_t)w; p[1] = (uint8_t)(w >> 8); p[2] = (uint8_t)(w >> 16); p[3] = (uint8_t)(w >> 24);
}

// blake2_hash.rs:111-118
inline Hash reduce_to_m31(const Hash& v) {
    Hash r;
    for (int i = 0; i < 8; i++) store_le32(&r[4 * i], M31::reduce((uint64_t)load_le32(&v[4 * i])).v);
    return r;
}

// blake2_hash.rs:73-108 — `m31` selects Blake2sM31Hasher (every digest word taken mod p).
struct Hasher {
    Blake2s st;
    bool m31;
    explicit Hasher(bool m31_) : m31(m31_) {}
    void update(const void* d, size_t n) { st.update(d, n); }
    Hash finalize() { Hash r = st.finalize(); return m31 ? reduce_to_m31(r) : r; }
    static Hash concat_and_hash(const Hash& a, const Hash& b, bool m31) {
        Hasher h(m31); h.update(a.data(), 32); h.update(b.data(), 32); return h.finalize();
    }
    static Hash hash(const void* d, size_t n, bool m31) { Hasher h(m31); h.update(d, n); return h.finalize(); }
};

// blake2_merkle.rs:18-39
inline Hash hash_node(const Hash* left, const Hash* right, const M31* column_values, size_t n, bool m31) {
    Blake2s st;
    if (left) { st.update(left->data(), 32); st.update(right->data(), 32); }
    for (size_t i = 0; i < n; i++) st.update_u32(column_values[i].v);
    Hash r = st.finalize();
    return m31 ? reduce_to_m31(r) : r;
}

// cpu/blake2s.rs:13-26
inline std::vector<Hash> commit_on_layer(uint32_t log_size, const std::vector<Hash>* prev,
                                         const std::vector<const M31*>& columns, bool m31) {
    size_t n = (size_t)1 << log_size;
    std::vector<Hash> out(n);
    if (accel().leaf_hashes && !prev && !columns.empty() && log_size >= 4) {  // 16 rows per compression (simd.hpp)
        std::vector<const uint32_t*> cp;
        for (auto c : columns) cp.push_back(&c->v);
        accel().leaf_hashes(reinterpret_cast<uint32_t*>(out.data()), cp.data(), cp.size(), n, m31);
        return out;
    }
    if (accel().node_hashes && prev && columns.empty() && log_size >= 4) {
        accel().node_hashes(reinterpret_cast<uint32_t*>(out.data()), reinterpret_cast<const uint32_t*>(prev->data()), n, m31);
        return out;
    }
#pragma omp parallel for schedule(static) if (n >= 1024)
    for (size_t i = 0; i < n; i++) {
        std::vector<M31> row(columns.size());
        for (size_t c = 0; c < columns.size(); c++) row[c] = columns[c][i];
        out[i] = prev ? hash_node(&(*prev)[2 * i], &(*prev)[2 * i + 1], row.data(), row.size(), m31)
                      : hash_node(nullptr, nullptr, row.data(), row.size(), m31);
    }
    return out;
}

// channel/blake2s.rs:20-141
struct Channel {
    Hash digest{};
    uint32_t n_draws = 0;
    bool m31;
    explicit Channel(bool m31_ = true) : m31(m31_) {}
    void update_digest(const Hash& d) { digest = d; n_draws = 0; }
    void mix_root(const Hash& root) { update_digest(Hasher::concat_and_hash(digest, root, m31)); }  // blake2_merkle.rs:53-58
    void mix_u32s(const uint32_t* data, size_t n) {
        Hasher h(m31);
        h.update(digest.data(), 32);
        for (size_t i = 0; i < n; i++) { uint8_t b[4]; store_le32(b, data[i]); h.update(b, 4); }
        update_digest(h.finalize());
    }
    void mix_u64(uint64_t v) { uint32_t d[2] = {(uint32_t)v, (uint32_t)(v >> 32)}; mix_u32s(d, 2); }
    void mix_felts(const QM31* f, size_t n) {
        Hasher h(m31);
        h.update(digest.data(), 32);
        for (size_t i = 0; i < n; i++) {
            uint32_t w[4]; f[i].to_u32(w);
            for (int k = 0; k < 4; k++) { uint8_t b[4]; store_le32(b, w[k]); h.update(b, 4); }
        }
        update_digest(h.finalize());
    }
    void mix_felts(const std::vector<QM31>& f) { mix_felts(f.data(), f.size()); }
    std::array<uint32_t, 8> draw_u32s() {
        uint8_t in[37];
        memcpy(in, digest.data(), 32);
        store_le32(in + 32, n_draws);
        in[36] = 0;
        n_draws++;
        Hash r = Hasher::hash(in, 37, m31);
        std::array<uint32_t, 8> out;
        for (int i = 0; i < 8; i++) out[i] = load_le32(&r[4 * i]);
        return out;
    }
    std::array<M31, 8> draw_base_felts() {
        for (;;) {
            auto u = draw_u32s();
            bool ok = true;
            for (auto x : u) ok = ok && (x < 2 * P);
            if (ok) {
                std::array<M31, 8> r;
                for (int i = 0; i < 8; i++) r[i] = M31::reduce((uint64_t)u[i]);
                return r;
            }
        }
    }
    QM31 draw_secure_felt() {
        auto f = draw_base_felts();
        return QM31::from_m31s(f[0], f[1], f[2], f[3]);
    }
    std::vector<QM31> draw_secure_felts(size_t n) {
        std::vector<QM31> out;
        while (out.size() < n) {
            auto f = draw_base_felts();
            out.push_back(QM31::from_m31s(f[0], f[1], f[2], f[3]));
            if (out.size() < n) out.push_back(QM31::from_m31s(f[4], f[5], f[6], f[7]));
        }
        return out;
    }
    // channel/blake2s.rs:122-140
    Hash pow_prefixed_digest(uint32_t n_bits) const {
        Hasher h(m31);
        uint8_t b[4]; store_le32(b, 0x12345678u);
        h.update(b, 4);
        uint8_t z[12] = {0};
        h.update(z, 12);
        h.update(digest.data(), 32);
        store_le32(b, n_bits);
        h.update(b, 4);
        return h.finalize();
    }
    static bool pow_check(const Hash& prefixed, uint32_t n_bits, uint64_t nonce, bool m31) {
        Hasher h(m31);
        h.update(prefixed.data(), 32);
        uint8_t nb[8];
        for (int i = 0; i < 8; i++) nb[i] = (uint8_t)(nonce >> (8 * i));
        h.update(nb, 8);
        Hash r = h.finalize();
        // trailing zeros of the first 16 bytes read as a little-endian u128
        uint32_t tz = 0;
        for (int i = 0; i < 16; i++) {
            if (r[i] == 0) { tz += 8; continue; }
            uint8_t x = r[i];
            while (!(x & 1)) { tz++; x >>= 1; }
            break;
        }
        return tz >= n_bits;
    }
    bool verify_pow_nonce(uint32_t n_bits, uint64_t nonce) const {
        return pow_check(pow_prefixed_digest(n_bits), n_bits, nonce, m31);
    }
    // The smallest passing nonce of the form (hi << 32) | lo with lo < 2^20, the enumeration of
    // simd/grind.rs:18-25, 62-93 (the parity target). cpu/grind.rs:6-15 counts 0, 1, 2, ... and
    // returns the same nonce whenever one exists below 2^20, which for pow_bits <= 32 fails
    // with probability (1 - 2^-pow_bits)^(2^20).
    uint64_t grind(uint32_t pow_bits) const {
        Hash pre = pow_prefixed_digest(pow_bits);
        for (uint64_t hi = 0;; hi++)
            for (uint64_t lo = 0; lo < (1u << 20); lo++) {
                uint64_t nonce = (hi << 32) | lo;
                if (pow_check(pre, pow_bits, nonce, m31)) return nonce;
            }
    }
};

// queries.rs:11-31
inline std::vector<size_t> draw_queries(Channel& ch, uint32_t log_domain_size, size_t n_queries) {
    std::vector<size_t> raw;
    uint32_t mask = (uint32_t)(((uint64_t)1 << log_domain_size) - 1);
    for (;;) {
        auto words = ch.draw_u32s();
        for (auto w : words) {
            raw.push_back(w & mask);
            if (raw.size() == n_queries) return raw;
        }
    }
}
// queries.rs:43-62
inline std::vector<size_t> sorted_dedup(const std::vector<size_t>& raw) {
    std::set<size_t> s(raw.begin(), raw.end());
    return std::vector<size_t>(s.begin(), s.end());
}
inline std::vector<size_t> fold_queries(const std::vector<size_t>& q, uint32_t n_folds) {
    std::vector<size_t> out;
    for (auto x : q) { size_t y = x >> n_folds; if (out.empty() || out.back() != y) out.push_back(y); }
    return out;
}

}  // namespace zko
