/*
 * philox.h -- Philox4x32-10 keep-mask shared by host and device code.
 *
 * The reference forward kernel takes dropout as a caller-materialised dense
 * float tensor dropout_mask[B*nh, T, T] that it multiplies into exp(s - m)
 * (kernels/attention/fused_attn_forward_kernel_tc_sm89.cu:21-22,321-324); it
 * has no generator.  This header defines the generator the sm_100a kernels
 * evaluate in registers, and the host evaluates to materialise that same dense
 * mask, so the two agree bit for bit (integer arithmetic only).
 *
 * Element (bh, qi, kj) -- qi and kj are GLOBAL sequence positions -- draws from
 *   counter = { kj >> 3, qi, bh, lo32(offset) }
 *   key     = { lo32(seed), hi32(seed) ^ hi32(offset) }
 * and uses 16-bit half number (kj & 7) of the 128 output bits (half h of word
 * (kj & 7) >> 1, low half first), so one Philox call covers eight consecutive
 * keys of a query row.  keep <=> half >= floor(p * 2^16): the drop probability
 * is p rounded down to a multiple of 2^-16.
 */
#ifndef HK_PHILOX_H_
#define HK_PHILOX_H_

#include <stdint.h>

#if defined(__CUDACC__)
#define HK_HD __host__ __device__ __forceinline__
#else
#define HK_HD static inline
#endif

#define HK_PHILOX_M0 0xD2511F53u
#define HK_PHILOX_M1 0xCD9E8D57u
#define HK_PHILOX_W0 0x9E3779B9u
#define HK_PHILOX_W1 0xBB67AE85u

typedef struct { uint32_t v[4]; } hk_philox4_t;

HK_HD void hk_mulhilo32(uint32_t a, uint32_t b, uint32_t* hi, uint32_t* lo) {
#if defined(__CUDA_ARCH__)
    *lo = a * b;
    *hi = __umulhi(a, b);
#else
    uint64_t p = (uint64_t)a * (uint64_t)b;
    *lo = (uint32_t)p;
    *hi = (uint32_t)(p >> 32);
#endif
}

HK_HD hk_philox4_t hk_philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1) {
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
    for (int r = 0; r < 10; ++r) {
        uint32_t hi0, lo0, hi1, lo1;
        hk_mulhilo32(HK_PHILOX_M0, c0, &hi0, &lo0);
        hk_mulhilo32(HK_PHILOX_M1, c2, &hi1, &lo1);
        uint32_t n0 = hi1 ^ c1 ^ k0;
        uint32_t n2 = hi0 ^ c3 ^ k1;
        c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
        k0 += HK_PHILOX_W0;
        k1 += HK_PHILOX_W1;
    }
    hk_philox4_t out;
    out.v[0] = c0; out.v[1] = c1; out.v[2] = c2; out.v[3] = c3;
    return out;
}

/* floor(p * 2^16), in [0, 65535]; p in [0,1). */
HK_HD uint32_t hk_philox_threshold(float p) {
    double t = (double)p * 65536.0;
    if (t <= 0.0) return 0u;
    if (t >= 65535.0) return 65535u;
    return (uint32_t)t;
}

/* The 128 random bits for keys 8*kj8 .. 8*kj8+7 of query row qi. */
HK_HD hk_philox4_t hk_philox_row8(uint64_t seed, uint64_t offset, uint32_t bh, uint32_t qi, uint32_t kj8) {
    return hk_philox4x32_10(kj8, qi, bh, (uint32_t)offset, (uint32_t)seed,
                            (uint32_t)(seed >> 32) ^ (uint32_t)(offset >> 32));
}

/* Keep bits of the eight keys of one Philox call: bit u <=> key 8*kj8+u is kept. */
HK_HD uint32_t hk_philox_keep8(hk_philox4_t r, uint32_t thr) {
    uint32_t m = 0;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
    for (int w = 0; w < 4; ++w) {
        m |= ((r.v[w] & 0xFFFFu) >= thr ? 1u : 0u) << (2 * w);
        m |= ((r.v[w] >> 16) >= thr ? 1u : 0u) << (2 * w + 1);
    }
    return m;
}

HK_HD int hk_philox_keep(uint64_t seed, uint64_t offset, uint32_t bh, uint32_t qi, uint32_t kj, uint32_t thr) {
    hk_philox4_t r = hk_philox_row8(seed, offset, bh, qi, kj >> 3);
    return (int)((hk_philox_keep8(r, thr) >> (kj & 7u)) & 1u);
}

#endif /* HK_PHILOX_H_ */
