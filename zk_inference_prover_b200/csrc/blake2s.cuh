// Blake2s-256 (RFC 7693) compression for device code: one thread, 16 message words in registers, the ten
// rounds fully unrolled with compile-time message schedules. Shared by the Merkle/grind kernels and by the
// device-resident Fiat-Shamir channel.
#pragma once
#include "common.cuh"

namespace zk {

#define B2S_IV0 0x6A09E667u
#define B2S_IV1 0xBB67AE85u
#define B2S_IV2 0x3C6EF372u
#define B2S_IV3 0xA54FF53Au
#define B2S_IV4 0x510E527Fu
#define B2S_IV5 0x9B05688Cu
#define B2S_IV6 0x1F83D9ABu
#define B2S_IV7 0x5BE0CD19u

__device__ __forceinline__ uint32_t rotr16(uint32_t x) { return __byte_perm(x, 0, 0x1032); }
__device__ __forceinline__ uint32_t rotr8(uint32_t x) { return __byte_perm(x, 0, 0x0321); }
__device__ __forceinline__ uint32_t rotr12(uint32_t x) { return __funnelshift_r(x, x, 12); }
__device__ __forceinline__ uint32_t rotr7(uint32_t x) { return __funnelshift_r(x, x, 7); }

// Where the additions run. Every instruction of a G function (additions, xors, rotations) would go to the integer ALU
// pipe, which issues one warp instruction every two cycles, and the compression is bound by that pipe. A multiply-add
// by one runs on the FMA-heavy pipe instead, in parallel. The compiler moves `c + d` there by itself; forcing
// `(a + x) + b` to add `x` on the ALU and `b` on the FMA pipe as well measured 8% more compressions per second than
// leaving it one three-input ALU addition (all additions on the FMA pipe: 3% fewer). The multiplier is read from
// constant memory so that the compiler can not fold the multiplication away.
static __constant__ uint32_t b2s_one = 1u;
__device__ __forceinline__ uint32_t b2s_fma_add(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b2s_one), "r"(b));
    return r;
}

#define B2S_G(a, b, c, d, x, y)        \
    do {                               \
        a = b2s_fma_add(a + (x), b);   \
        d = rotr16(d ^ a);             \
        c = b2s_fma_add(c, d);         \
        b = rotr12(b ^ c);             \
        a = b2s_fma_add(a + (y), b);   \
        d = rotr8(d ^ a);              \
        c = b2s_fma_add(c, d);         \
        b = rotr7(b ^ c);              \
    } while (0)

#define B2S_ROUND(s0, s1, s2, s3, s4, s5, s6, s7, s8, s9, s10, s11, s12, s13, s14, s15) \
    do {                                                                                 \
        B2S_G(v0, v4, v8, v12, m[s0], m[s1]);                                            \
        B2S_G(v1, v5, v9, v13, m[s2], m[s3]);                                            \
        B2S_G(v2, v6, v10, v14, m[s4], m[s5]);                                           \
        B2S_G(v3, v7, v11, v15, m[s6], m[s7]);                                           \
        B2S_G(v0, v5, v10, v15, m[s8], m[s9]);                                           \
        B2S_G(v1, v6, v11, v12, m[s10], m[s11]);                                         \
        B2S_G(v2, v7, v8, v13, m[s12], m[s13]);                                          \
        B2S_G(v3, v4, v9, v14, m[s14], m[s15]);                                          \
    } while (0)

// One compression (RFC 7693 section 3.2). `t` is the byte count including this block.
__device__ __forceinline__ void blake2s_compress(uint32_t h[8], const uint32_t m[16], uint32_t t, bool last) {
    uint32_t v0 = h[0], v1 = h[1], v2 = h[2], v3 = h[3], v4 = h[4], v5 = h[5], v6 = h[6], v7 = h[7];
    uint32_t v8 = B2S_IV0, v9 = B2S_IV1, v10 = B2S_IV2, v11 = B2S_IV3;
    uint32_t v12 = B2S_IV4 ^ t, v13 = B2S_IV5, v14 = last ? ~B2S_IV6 : B2S_IV6, v15 = B2S_IV7;
    B2S_ROUND(0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15);
    B2S_ROUND(14, 10, 4, 8, 9, 15, 13, 6, 1, 12, 0, 2, 11, 7, 5, 3);
    B2S_ROUND(11, 8, 12, 0, 5, 2, 15, 13, 10, 14, 3, 6, 7, 1, 9, 4);
    B2S_ROUND(7, 9, 3, 1, 13, 12, 11, 14, 2, 6, 5, 10, 4, 0, 15, 8);
    B2S_ROUND(9, 0, 5, 7, 2, 4, 10, 15, 14, 1, 11, 12, 6, 8, 3, 13);
    B2S_ROUND(2, 12, 6, 10, 0, 11, 8, 3, 4, 13, 7, 5, 15, 14, 1, 9);
    B2S_ROUND(12, 5, 1, 15, 14, 13, 4, 10, 0, 7, 6, 3, 9, 2, 8, 11);
    B2S_ROUND(13, 11, 7, 14, 12, 1, 3, 9, 5, 0, 15, 4, 8, 6, 2, 10);
    B2S_ROUND(6, 15, 14, 9, 11, 3, 0, 8, 12, 2, 13, 7, 1, 4, 10, 5);
    B2S_ROUND(10, 2, 8, 4, 7, 6, 1, 5, 15, 11, 9, 14, 3, 12, 13, 0);
    h[0] ^= v0 ^ v8;  h[1] ^= v1 ^ v9;  h[2] ^= v2 ^ v10; h[3] ^= v3 ^ v11;
    h[4] ^= v4 ^ v12; h[5] ^= v5 ^ v13; h[6] ^= v6 ^ v14; h[7] ^= v7 ^ v15;
}

__device__ __forceinline__ void blake2s_init(uint32_t h[8]) {
    h[0] = B2S_IV0 ^ 0x01010020u; h[1] = B2S_IV1; h[2] = B2S_IV2; h[3] = B2S_IV3;
    h[4] = B2S_IV4; h[5] = B2S_IV5; h[6] = B2S_IV6; h[7] = B2S_IV7;
}

// A 32-bit word taken mod 2^31-1 (core/fields/m31.rs:58-60 applied to a u32).
__device__ __forceinline__ uint32_t reduce_word_m31(uint32_t w) {
    uint32_t s = (w & P) + (w >> 31);
    return umin32(s, s - P);
}

}  // namespace zk
