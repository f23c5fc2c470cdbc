// Host-side Fiat-Shamir channel of the prover: Blake2s-256 (RFC 7693) with every digest word
// reduced mod 2^31-1, as the reference's Blake2sM31Channel
// (nitroo/crates/stwo/src/core/channel/blake2s.rs:20-141, core/vcs/blake2_hash.rs:73-118,
// core/vcs/blake2_merkle.rs:53-58). Hashes are held as 8 little-endian words.
#pragma once
#include <array>
#include <cstdint>
#include <cstring>
#include <vector>

#include "../m31.cuh"

namespace b200 {

using HashWords = std::array<uint32_t, 8>;

class Blake2sState {
  public:
    Blake2sState() {
        static const uint32_t iv[8] = {0x6A09E667u, 0xBB67AE85u, 0x3C6EF372u, 0xA54FF53Au, 0x510E527Fu, 0x9B05688Cu, 0x1F83D9ABu, 0x5BE0CD19u};
        for (int i = 0; i < 8; i++) h_[i] = iv[i];
        h_[0] ^= 0x01010020u;
    }
    void update(const uint8_t* p, size_t n) {
        while (n) {
            if (fill_ == 64) { t_ += 64; compress(false); fill_ = 0; }
            size_t k = n < 64 - fill_ ? n : 64 - fill_;
            memcpy(buf_ + fill_, p, k);
            fill_ += k; p += k; n -= k;
        }
    }
    void update_words(const uint32_t* w, size_t n) {
#if defined(__BYTE_ORDER__) && __BYTE_ORDER__ == __ORDER_LITTLE_ENDIAN__
        update(reinterpret_cast<const uint8_t*>(w), 4 * n);  // the words' memory is their little-endian serialisation
#else
        for (size_t i = 0; i < n; i++) {
            uint8_t b[4] = {(uint8_t)w[i], (uint8_t)(w[i] >> 8), (uint8_t)(w[i] >> 16), (uint8_t)(w[i] >> 24)};
            update(b, 4);
        }
#endif
    }
    // Digest with every word taken mod 2^31-1 (the M31 variant of the hasher).
    HashWords finalize_m31() {
        t_ += fill_;
        memset(buf_ + fill_, 0, 64 - fill_);
        compress(true);
        HashWords out;
        for (int i = 0; i < 8; i++) {
            uint32_t w = h_[i], s = (w & zk::P) + (w >> 31);
            out[i] = s >= zk::P ? s - zk::P : s;
        }
        return out;
    }
  private:
    static uint32_t rotr(uint32_t x, int k) { return (x >> k) | (x << (32 - k)); }
    void compress(bool last) {
        static const uint32_t iv[8] = {0x6A09E667u, 0xBB67AE85u, 0x3C6EF372u, 0xA54FF53Au, 0x510E527Fu, 0x9B05688Cu, 0x1F83D9ABu, 0x5BE0CD19u};
        static const uint8_t sigma[10][16] = {
            {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15}, {14, 10, 4, 8, 9, 15, 13, 6, 1, 12, 0, 2, 11, 7, 5, 3},
            {11, 8, 12, 0, 5, 2, 15, 13, 10, 14, 3, 6, 7, 1, 9, 4}, {7, 9, 3, 1, 13, 12, 11, 14, 2, 6, 5, 10, 4, 0, 15, 8},
            {9, 0, 5, 7, 2, 4, 10, 15, 14, 1, 11, 12, 6, 8, 3, 13}, {2, 12, 6, 10, 0, 11, 8, 3, 4, 13, 7, 5, 15, 14, 1, 9},
            {12, 5, 1, 15, 14, 13, 4, 10, 0, 7, 6, 3, 9, 2, 8, 11}, {13, 11, 7, 14, 12, 1, 3, 9, 5, 0, 15, 4, 8, 6, 2, 10},
            {6, 15, 14, 9, 11, 3, 0, 8, 12, 2, 13, 7, 1, 4, 10, 5}, {10, 2, 8, 4, 7, 6, 1, 5, 15, 11, 9, 14, 3, 12, 13, 0}};
        uint32_t m[16], v[16];
#if defined(__BYTE_ORDER__) && __BYTE_ORDER__ == __ORDER_LITTLE_ENDIAN__
        memcpy(m, buf_, 64);
#else
        for (int i = 0; i < 16; i++)
            m[i] = (uint32_t)buf_[4 * i] | ((uint32_t)buf_[4 * i + 1] << 8) | ((uint32_t)buf_[4 * i + 2] << 16) | ((uint32_t)buf_[4 * i + 3] << 24);
#endif
        for (int i = 0; i < 8; i++) { v[i] = h_[i]; v[8 + i] = iv[i]; }
        v[12] ^= (uint32_t)t_;
        v[13] ^= (uint32_t)(t_ >> 32);
        if (last) v[14] = ~v[14];
        auto g = [&](int a, int b, int c, int d, uint32_t x, uint32_t y) {
            v[a] += v[b] + x; v[d] = rotr(v[d] ^ v[a], 16);
            v[c] += v[d];     v[b] = rotr(v[b] ^ v[c], 12);
            v[a] += v[b] + y; v[d] = rotr(v[d] ^ v[a], 8);
            v[c] += v[d];     v[b] = rotr(v[b] ^ v[c], 7);
        };
        for (int r = 0; r < 10; r++) {
            const uint8_t* s = sigma[r];
            g(0, 4, 8, 12, m[s[0]], m[s[1]]);   g(1, 5, 9, 13, m[s[2]], m[s[3]]);
            g(2, 6, 10, 14, m[s[4]], m[s[5]]);  g(3, 7, 11, 15, m[s[6]], m[s[7]]);
            g(0, 5, 10, 15, m[s[8]], m[s[9]]);  g(1, 6, 11, 12, m[s[10]], m[s[11]]);
            g(2, 7, 8, 13, m[s[12]], m[s[13]]); g(3, 4, 9, 14, m[s[14]], m[s[15]]);
        }
        for (int i = 0; i < 8; i++) h_[i] ^= v[i] ^ v[8 + i];
    }
    uint32_t h_[8];
    uint8_t buf_[64];
    size_t fill_ = 0;
    uint64_t t_ = 0;
};

// Blake2sM31Channel.
class Channel {
  public:
    const HashWords& digest() const { return digest_; }
    void mix_root(const HashWords& root) {  // blake2_merkle.rs:53-58
        Blake2sState st;
        st.update_words(digest_.data(), 8);
        st.update_words(root.data(), 8);
        set(st.finalize_m31());
    }
    void mix_u32s(const uint32_t* data, size_t n) {
        Blake2sState st;
        st.update_words(digest_.data(), 8);
        st.update_words(data, n);
        set(st.finalize_m31());
    }
    void mix_u64(uint64_t v) { uint32_t d[2] = {(uint32_t)v, (uint32_t)(v >> 32)}; mix_u32s(d, 2); }
    void mix_felts(const zk::qm31* f, size_t n) { mix_u32s((const uint32_t*)f, 4 * n); }
    void mix_felts(const std::vector<zk::qm31>& f) { mix_felts(f.data(), f.size()); }
    std::array<uint32_t, 8> draw_u32s() {
        uint8_t in[37];
        for (int i = 0; i < 8; i++)
            for (int j = 0; j < 4; j++) in[4 * i + j] = (uint8_t)(digest_[i] >> (8 * j));
        for (int j = 0; j < 4; j++) in[32 + j] = (uint8_t)(n_draws_ >> (8 * j));
        in[36] = 0;
        n_draws_++;
        Blake2sState st;
        st.update(in, 37);
        return st.finalize_m31();
    }
    // channel/blake2s.rs:34-52: retry until all eight words are below 2p.
    std::array<uint32_t, 8> draw_base_felts() {
        for (;;) {
            auto u = draw_u32s();
            bool ok = true;
            for (auto x : u) ok = ok && x < 2 * zk::P;
            if (!ok) continue;
            for (auto& x : u) x = x >= zk::P ? x - zk::P : x;
            return u;
        }
    }
    zk::qm31 draw_secure_felt() {
        auto f = draw_base_felts();
        return {{f[0], f[1], f[2], f[3]}};
    }
    // H(POW_PREFIX, 12 zero bytes, digest, n_bits), channel/blake2s.rs:124-133
    HashWords pow_prefixed_digest(uint32_t n_bits) const {
        Blake2sState st;
        uint32_t head[4] = {0x12345678u, 0, 0, 0};
        st.update_words(head, 4);
        st.update_words(digest_.data(), 8);
        st.update_words(&n_bits, 1);
        return st.finalize_m31();
    }
    // The state as a device-resident copy of the channel holds it (digest, n_draws), and back.
    uint32_t n_draws() const { return n_draws_; }
    void set_state(const HashWords& d, uint32_t n_draws) { digest_ = d; n_draws_ = n_draws; }
  private:
    void set(const HashWords& d) { digest_ = d; n_draws_ = 0; }
    HashWords digest_{};
    uint32_t n_draws_ = 0;
};

// core/queries.rs:11-31
inline std::vector<size_t> draw_queries(Channel& ch, uint32_t log_domain_size, size_t n_queries) {
    std::vector<size_t> raw;
    uint32_t mask = (uint32_t)(((uint64_t)1 << log_domain_size) - 1);
    while (raw.size() < n_queries)
        for (auto w : ch.draw_u32s()) {
            raw.push_back(w & mask);
            if (raw.size() == n_queries) break;
        }
    return raw;
}

}  // namespace b200
