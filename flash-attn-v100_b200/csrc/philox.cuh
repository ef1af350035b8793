// Counter-based dropout stream shared by the forward kernels, the backward
// kernels and the host mask generator.
//
// Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy
// as 1, 2, 3", SC'11) restated from the paper: ten rounds of
//   (c0,c1,c2,c3) <- (hi(M1*c2)^c1^k0, lo(M1*c2), hi(M0*c0)^c3^k1, lo(M0*c0))
// with the key bumped by the Weyl constants between rounds.
//
// One block serves 16 consecutive key positions of one query row:
//   key     = (seed_lo, seed_hi ^ offset_hi)
//   counter = (j / 16, i, b*H + h, offset_lo)
//   byte    = little-endian byte (j % 16) of the four output words
//   keep    = byte >= round(p * 256)
// so the decision is an integer compare and is identical wherever it is
// evaluated, whatever the tile shape of the kernel that asks.
//
// The reference draws tl.rand inside its forward kernel only
// (kernels/forward_kernel.py:198-203) and has no dropout in backward; this
// stream is the new build's own definition.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define FA_HD __host__ __device__ __forceinline__
#else
#define FA_HD inline
#endif

namespace fa {

struct PhiloxKey {
    uint32_t k0, k1;   // key words
    uint32_t c3;       // fourth counter word (offset_lo)
    // the ten round keys (k0 + r W0, k1 + r W1): the same for every block of a call, so they are
    // worked out once on the host and reach the kernels as launch constants
    uint32_t r0[10], r1[10];
};

FA_HD PhiloxKey philox_make_key(uint64_t seed, uint64_t offset) {
    PhiloxKey k;
    k.k0 = (uint32_t)seed;
    k.k1 = (uint32_t)(seed >> 32) ^ (uint32_t)(offset >> 32);
    k.c3 = (uint32_t)offset;
    for (int r = 0; r < 10; ++r) {
        k.r0[r] = k.k0 + (uint32_t)r * 0x9E3779B9u;
        k.r1[r] = k.k1 + (uint32_t)r * 0xBB67AE85u;
    }
    return k;
}

// Which (batch, head) column of the dropout stream a call's local (b, h) is.  A call over a slice of a
// larger problem (a head or batch shard on another GPU, one chunk of a batch) passes the slice's
// origin and the whole problem's head count, and so draws exactly the mask the whole call draws.
struct DropoutOrigin {
    int32_t b0, h0;    // batch and head index of the call's first column in the whole problem
    int32_t heads;     // heads of the whole problem
};

FA_HD uint32_t dropout_column(const DropoutOrigin& o, int b, int h) {
    return (uint32_t)((b + o.b0) * o.heads + h + o.h0);
}

// both halves of the 64-bit product (one wide multiply on the device)
FA_HD void philox_mulhilo(uint32_t a, uint32_t b, uint32_t& hi, uint32_t& lo) {
    uint64_t p = (uint64_t)a * (uint64_t)b;
    lo = (uint32_t)p;
    hi = (uint32_t)(p >> 32);
}

FA_HD void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                         uint32_t k0, uint32_t k1, uint32_t out[4]) {
    const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
    const uint32_t W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        uint32_t hi0, lo0, hi1, lo1;
        philox_mulhilo(M0, c0, hi0, lo0);
        philox_mulhilo(M1, c2, hi1, lo1);
        uint32_t n0 = hi1 ^ c1 ^ k0;
        uint32_t n2 = hi0 ^ c3 ^ k1;
        c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
        k0 += W0; k1 += W1;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// The same ten rounds with the round keys taken from the table in `key`.
FA_HD void philox4x32_10_keyed(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, const PhiloxKey& key, uint32_t out[4]) {
    const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        uint32_t hi0, lo0, hi1, lo1;
        philox_mulhilo(M0, c0, hi0, lo0);
        philox_mulhilo(M1, c2, hi1, lo1);
        uint32_t n0 = hi1 ^ c1 ^ key.r0[r];
        uint32_t n2 = hi0 ^ c3 ^ key.r1[r];
        c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// 16 random bytes for keys [16*jblk, 16*jblk+16) of query row i of head bh.
FA_HD void dropout_block(const PhiloxKey& key, uint32_t bh, uint32_t i, uint32_t jblk,
                         uint32_t out[4]) {
    philox4x32_10_keyed(jblk, i, bh, key.c3, key, out);
}

// Threshold in [0, 256]: a byte is dropped iff byte < threshold.
FA_HD uint32_t dropout_threshold(float p) {
    if (!(p > 0.f)) return 0u;
    float t = p * 256.f + 0.5f;
    uint32_t u = (uint32_t)t;
    return u > 255u ? 255u : u;
}

FA_HD float dropout_effective_p(float p) {
    return (float)dropout_threshold(p) * (1.f / 256.f);
}

// 16-bit keep mask of one block: bit t set iff key 16*jblk + t is kept.
FA_HD uint32_t dropout_keep_bits(const PhiloxKey& key, uint32_t bh, uint32_t i, uint32_t jblk,
                                 uint32_t threshold) {
    uint32_t w[4];
    dropout_block(key, bh, i, jblk, w);
    uint32_t bits = 0;
#if defined(__CUDA_ARCH__)
    // byte >= threshold <=> byte + (256 - threshold) carries out of its eight bits.  The even and the odd
    // bytes of a word go to the two 16-bit lanes of a register each; the add (scaled by 64 or 128, so
    // that the four carries of a word end up at bits 14, 15, 30, 31) cannot cross a lane: (255 + 255) * 128
    // < 2^16.  One high-half multiply per word then moves its four flags to bits 4q .. 4q + 3 (the two
    // partial products that matter land at 32 + 4q and 34 + 4q, the other two below bit 32 and above bit
    // 47).  17 logic operations and 12 multiply-adds for the 16 bytes; 8 % off the kernel that writes a
    // call's bits against four emulated per-byte compares.
    const uint32_t nt = 256u - threshold;                    // threshold is 1 .. 255 here
    const uint32_t k6 = nt * 0x00400040u, k7 = nt * 0x00800080u;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const uint32_t even = w[q] & 0x00FF00FFu;
        const uint32_t odd = __byte_perm(w[q], 0u, 0x4341);  // bytes 1 and 3, each in the low byte of a lane
        const uint32_t se = even * 64u + k6, so = odd * 128u + k7;
        const uint32_t flags = (se & 0x40004000u) | (so & 0x80008000u);
        bits += __umulhi(flags, (1u << (18 + 4 * q)) + (1u << (4 + 4 * q)));
    }
    bits &= 0xFFFFu;
#else
    for (int q = 0; q < 4; ++q) {
        for (int b = 0; b < 4; ++b) {
            uint32_t byte = (w[q] >> (8 * b)) & 0xFFu;
            bits |= (byte >= threshold ? 1u : 0u) << (4 * q + b);
        }
    }
#endif
    return bits;
}

// Single-element form used by code that does not walk a row in key order.
FA_HD bool dropout_keep(const PhiloxKey& key, uint32_t bh, uint32_t i, uint32_t j,
                        uint32_t threshold) {
    uint32_t w[4];
    dropout_block(key, bh, i, j >> 4, w);
    uint32_t t = j & 15u;
    uint32_t byte = (w[t >> 2] >> (8 * (t & 3u))) & 0xFFu;
    return byte >= threshold;
}

}  // namespace fa
