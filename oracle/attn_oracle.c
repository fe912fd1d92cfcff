/*
 * attn_oracle.c -- CPU oracle for fused attention forward/backward (fp32 I/O,
 * fp64 dot products).  TEST INFRASTRUCTURE ONLY: this file is the checker the
 * CUDA path is compared against; nothing in the shipped library calls it.
 *
 * It restates, in plain C, the host reference of BlubridgeAI/HyperKernels:
 *   attention forward   kernels/tests/kernels_test.cu:68-98   (attn_ref_forward)
 *   attention backward  kernels/tests/kernels_test.cu:101-139 (attn_ref_backward)
 *   D = rowsum(dO*O)    kernels/tests/kernels_test.cu:465      (precompute_D check)
 *   rand_vec            kernels/tests/kernels_test.cu:48-54    (mt19937_64 uniform)
 * and extends it with the drop-then-renormalise dropout that the reference
 * forward kernel implements but its host reference does not
 * (kernels/attention/fused_attn_forward_kernel_tc_sm89.cu:286-338): the row max
 * runs over all causally-visible scores, e_ij = mask_ij*exp(s_ij-m_i),
 * l_i = sum_j e_ij, O_i = sum_j e_ij v_j / l_i, LSE_i = m_i + log l_i.
 *
 * Parity status: the p=0 paths are pinned bit-for-bit against the reference's
 * own host functions compiled from its sources (see oracle/Makefile, target
 * _ref) and against the committed golden vectors.  The dropout path has no
 * counterpart in the reference's host code or tests.  Its forward is pinned to
 * the reference's GPU forward kernel (recompiled, fed the same dense mask) by
 * tests/test_reference_kernels_gpu.py::test_dropout_forward_pinned_to_the_reference_kernel;
 * its backward has no reference implementation at all ("parity unpinned") and
 * is held by a float64 autograd check and finite differences.
 *
 * Tensors are contiguous [B,H,T,Hd] (LSE, D: [B,H,T]).  Tq query rows attend
 * to Tk key rows; query row i sits at global position q_pos0+i and key row j at
 * k_pos0+j (both 0 for ordinary attention), which is what a sequence-sharded
 * ring step needs.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../hyperkernels_b200/csrc/philox.h"

#define HK_ORACLE_MAX_HD 256

/* mt19937_64 + std::uniform_real_distribution<float>(lo,hi) as libstdc++
 * evaluates it: one 64-bit draw per value, canonical = float(draw) / 2^64,
 * clamped below 1 (kernels_test.cu:48-54). */
typedef struct { uint64_t mt[312]; int idx; } mt64_t;

static void mt64_seed(mt64_t* s, uint64_t seed) {
    s->mt[0] = seed;
    for (int i = 1; i < 312; ++i)
        s->mt[i] = 6364136223846793005ULL * (s->mt[i - 1] ^ (s->mt[i - 1] >> 62)) + (uint64_t)i;
    s->idx = 312;
}

static uint64_t mt64_next(mt64_t* s) {
    if (s->idx >= 312) {
        for (int i = 0; i < 312; ++i) {
            uint64_t x = (s->mt[i] & 0xFFFFFFFF80000000ULL) | (s->mt[(i + 1) % 312] & 0x7FFFFFFFULL);
            uint64_t xa = x >> 1;
            if (x & 1ULL) xa ^= 0xB5026F5AA96619E9ULL;
            s->mt[i] = s->mt[(i + 156) % 312] ^ xa;
        }
        s->idx = 0;
    }
    uint64_t y = s->mt[s->idx++];
    y ^= (y >> 29) & 0x5555555555555555ULL;
    y ^= (y << 17) & 0x71D67FFFEDA60000ULL;
    y ^= (y << 37) & 0xFFF7EEE000000000ULL;
    y ^= (y >> 43);
    return y;
}

void hk_oracle_rand_vec(float* out, size_t n, uint64_t seed, float lo, float hi) {
    mt64_t s;
    mt64_seed(&s, seed);
    for (size_t i = 0; i < n; ++i) {
        float sum = (float)mt64_next(&s);
        float ret = sum / 18446744073709551616.0f;
        if (ret >= 1.0f) ret = nextafterf(1.0f, 0.0f);
        out[i] = ret * (hi - lo) + lo;
    }
}

/* Keep-mask in the reference's dense format: 1.0f keep / 0.0f drop, laid out
 * [BH, Tq, Tk] (fused_attn_forward_kernel_tc_sm89.cu:321-324 indexes it as
 * (bnh*T+qi)*T+kj). */
void hk_oracle_dropout_mask(float* mask, int BH, int Tq, int Tk, float p, uint64_t seed, uint64_t offset,
                            int64_t q_pos0, int64_t k_pos0) {
    const uint32_t thr = hk_philox_threshold(p);
    for (int bh = 0; bh < BH; ++bh)
        for (int i = 0; i < Tq; ++i)
            for (int j = 0; j < Tk; ++j)
                mask[((size_t)bh * Tq + i) * Tk + j] =
                    hk_philox_keep(seed, offset, (uint32_t)bh, (uint32_t)(q_pos0 + i), (uint32_t)(k_pos0 + j), thr) ? 1.0f : 0.0f;
}

/* mask: NULL (no dropout) or dense [B*H, Tq, Tk] floats multiplied into exp(). */
void hk_oracle_attn_forward(const float* Q, const float* K, const float* V, int B, int H, int Tq, int Tk, int Hd,
                            float scale, int causal, int64_t q_pos0, int64_t k_pos0, const float* mask,
                            float* O, float* LSE) {
    for (int b = 0; b < B; ++b)
        for (int h = 0; h < H; ++h) {
            const int64_t bh = (int64_t)b * H + h;
            const int64_t qbase = bh * Tq * Hd, kbase = bh * Tk * Hd, lbase = bh * Tq;
            for (int i = 0; i < Tq; ++i) {
                const float* qi = &Q[qbase + (int64_t)i * Hd];
                int64_t jmax = Tk - 1;
                if (causal) {
                    int64_t lim = q_pos0 + i - k_pos0;
                    if (lim < jmax) jmax = lim;
                }
                float m = -1e30f;
                for (int64_t j = 0; j <= jmax; ++j) {
                    const float* kj = &K[kbase + j * Hd];
                    double d = 0;
                    for (int k = 0; k < Hd; ++k) d += (double)qi[k] * kj[k];
                    float s = (float)(d * scale);
                    if (s > m) m = s;
                }
                double l = 0, oacc[HK_ORACLE_MAX_HD];
                for (int k = 0; k < Hd; ++k) oacc[k] = 0;
                for (int64_t j = 0; j <= jmax; ++j) {
                    const float* kj = &K[kbase + j * Hd];
                    const float* vj = &V[kbase + j * Hd];
                    double d = 0;
                    for (int k = 0; k < Hd; ++k) d += (double)qi[k] * kj[k];
                    float e = expf((float)(d * scale) - m);
                    if (mask) e *= mask[(bh * Tq + i) * (int64_t)Tk + j];
                    l += e;
                    for (int k = 0; k < Hd; ++k) oacc[k] += (double)e * vj[k];
                }
                double inv = (l > 0) ? 1.0 / l : 0.0;
                for (int k = 0; k < Hd; ++k) O[qbase + (int64_t)i * Hd + k] = (float)(oacc[k] * inv);
                LSE[lbase + i] = (l > 0) ? (float)(m + log(l)) : -INFINITY;
            }
        }
}

void hk_oracle_precompute_D(const float* dO, const float* O, int64_t rows, int Hd, float* D) {
    for (int64_t r = 0; r < rows; ++r) {
        double s = 0;
        for (int k = 0; k < Hd; ++k) s += (double)dO[r * Hd + k] * O[r * Hd + k];
        D[r] = (float)s;
    }
}

/* Zero-fills dQ/dK/dV, then accumulates in float like the reference. */
void hk_oracle_attn_backward(const float* Q, const float* K, const float* V, const float* O, const float* dO,
                             const float* LSE, int B, int H, int Tq, int Tk, int Hd, float scale, int causal,
                             int64_t q_pos0, int64_t k_pos0, const float* mask, float* D, float* dQ, float* dK,
                             float* dV) {
    memset(dQ, 0, sizeof(float) * (size_t)B * H * Tq * Hd);
    memset(dK, 0, sizeof(float) * (size_t)B * H * Tk * Hd);
    memset(dV, 0, sizeof(float) * (size_t)B * H * Tk * Hd);
    for (int b = 0; b < B; ++b)
        for (int h = 0; h < H; ++h) {
            const int64_t bh = (int64_t)b * H + h;
            const int64_t qbase = bh * Tq * Hd, kbase = bh * Tk * Hd, lbase = bh * Tq;
            for (int i = 0; i < Tq; ++i) {
                const float* qi = &Q[qbase + (int64_t)i * Hd];
                const float* doi = &dO[qbase + (int64_t)i * Hd];
                const float* oi = &O[qbase + (int64_t)i * Hd];
                double Di = 0;
                for (int k = 0; k < Hd; ++k) Di += (double)doi[k] * oi[k];
                D[lbase + i] = (float)Di;
                const float Li = LSE[lbase + i];
                int64_t jmax = Tk - 1;
                if (causal) {
                    int64_t lim = q_pos0 + i - k_pos0;
                    if (lim < jmax) jmax = lim;
                }
                float* dqi = &dQ[qbase + (int64_t)i * Hd];
                if (Li == -INFINITY) continue; /* fully dropped row: every p_ij is 0 */
                for (int64_t j = 0; j <= jmax; ++j) {
                    const float* kj = &K[kbase + j * Hd];
                    const float* vj = &V[kbase + j * Hd];
                    float* dkj = &dK[kbase + j * Hd];
                    float* dvj = &dV[kbase + j * Hd];
                    double sd = 0, dp = 0;
                    for (int k = 0; k < Hd; ++k) {
                        sd += (double)qi[k] * kj[k];
                        dp += (double)doi[k] * vj[k];
                    }
                    float p = expf((float)(sd * scale) - Li);
                    if (mask) p *= mask[(bh * Tq + i) * (int64_t)Tk + j];
                    float ds = (float)(p * (dp - Di) * scale);
                    for (int k = 0; k < Hd; ++k) {
                        dqi[k] += ds * kj[k];
                        dkj[k] += ds * qi[k];
                        dvj[k] += p * doi[k];
                    }
                }
            }
        }
}

/* ---- inverted ("scaled") dropout -----------------------------------------
 * The usual training-time definition, offered by the library as an option next
 * to the reference's drop-then-renormalise one (the reference has no counterpart):
 *   P = softmax(S) over ALL visible keys,   O_i = sum_j mask_ij * P_ij / (1-p) * v_j,
 *   LSE_i = log sum_j exp(s_ij)   (independent of the mask).
 * Backward: dPd_ij = mask_ij/(1-p) * dO_i.v_j,  D_i = dO_i.O_i,
 *   dS = P * (dPd - D) * scale,  dV_j += mask_ij/(1-p) * P_ij * dO_i.
 * `keep_scale` is 1/(1-p).  Pinned only by the finite-difference test. */
void hk_oracle_attn_forward_scaled_dropout(const float* Q, const float* K, const float* V, int B, int H, int Tq, int Tk,
                                           int Hd, float scale, int causal, int64_t q_pos0, int64_t k_pos0,
                                           const float* mask, float keep_scale, float* O, float* LSE) {
    for (int b = 0; b < B; ++b)
        for (int h = 0; h < H; ++h) {
            const int64_t bh = (int64_t)b * H + h;
            const int64_t qbase = bh * Tq * Hd, kbase = bh * Tk * Hd, lbase = bh * Tq;
            for (int i = 0; i < Tq; ++i) {
                const float* qi = &Q[qbase + (int64_t)i * Hd];
                int64_t jmax = Tk - 1;
                if (causal) {
                    int64_t lim = q_pos0 + i - k_pos0;
                    if (lim < jmax) jmax = lim;
                }
                float m = -1e30f;
                for (int64_t j = 0; j <= jmax; ++j) {
                    const float* kj = &K[kbase + j * Hd];
                    double d = 0;
                    for (int k = 0; k < Hd; ++k) d += (double)qi[k] * kj[k];
                    float s = (float)(d * scale);
                    if (s > m) m = s;
                }
                double l = 0, oacc[HK_ORACLE_MAX_HD];
                for (int k = 0; k < Hd; ++k) oacc[k] = 0;
                for (int64_t j = 0; j <= jmax; ++j) {
                    const float* kj = &K[kbase + j * Hd];
                    const float* vj = &V[kbase + j * Hd];
                    double d = 0;
                    for (int k = 0; k < Hd; ++k) d += (double)qi[k] * kj[k];
                    float e = expf((float)(d * scale) - m);
                    l += e;
                    const double w = (double)e * (mask ? mask[(bh * Tq + i) * (int64_t)Tk + j] * keep_scale : 1.0f);
                    for (int k = 0; k < Hd; ++k) oacc[k] += w * vj[k];
                }
                double inv = (l > 0) ? 1.0 / l : 0.0;
                for (int k = 0; k < Hd; ++k) O[qbase + (int64_t)i * Hd + k] = (float)(oacc[k] * inv);
                LSE[lbase + i] = (l > 0) ? (float)(m + log(l)) : -INFINITY;
            }
        }
}

void hk_oracle_attn_backward_scaled_dropout(const float* Q, const float* K, const float* V, const float* O,
                                            const float* dO, const float* LSE, int B, int H, int Tq, int Tk, int Hd,
                                            float scale, int causal, int64_t q_pos0, int64_t k_pos0, const float* mask,
                                            float keep_scale, float* D, float* dQ, float* dK, float* dV) {
    memset(dQ, 0, sizeof(float) * (size_t)B * H * Tq * Hd);
    memset(dK, 0, sizeof(float) * (size_t)B * H * Tk * Hd);
    memset(dV, 0, sizeof(float) * (size_t)B * H * Tk * Hd);
    for (int b = 0; b < B; ++b)
        for (int h = 0; h < H; ++h) {
            const int64_t bh = (int64_t)b * H + h;
            const int64_t qbase = bh * Tq * Hd, kbase = bh * Tk * Hd, lbase = bh * Tq;
            for (int i = 0; i < Tq; ++i) {
                const float* qi = &Q[qbase + (int64_t)i * Hd];
                const float* doi = &dO[qbase + (int64_t)i * Hd];
                const float* oi = &O[qbase + (int64_t)i * Hd];
                double Di = 0;
                for (int k = 0; k < Hd; ++k) Di += (double)doi[k] * oi[k];
                D[lbase + i] = (float)Di;
                const float Li = LSE[lbase + i];
                int64_t jmax = Tk - 1;
                if (causal) {
                    int64_t lim = q_pos0 + i - k_pos0;
                    if (lim < jmax) jmax = lim;
                }
                float* dqi = &dQ[qbase + (int64_t)i * Hd];
                if (Li == -INFINITY) continue;
                for (int64_t j = 0; j <= jmax; ++j) {
                    const float* kj = &K[kbase + j * Hd];
                    const float* vj = &V[kbase + j * Hd];
                    float* dkj = &dK[kbase + j * Hd];
                    float* dvj = &dV[kbase + j * Hd];
                    double sd = 0, dp = 0;
                    for (int k = 0; k < Hd; ++k) {
                        sd += (double)qi[k] * kj[k];
                        dp += (double)doi[k] * vj[k];
                    }
                    const float w = mask ? mask[(bh * Tq + i) * (int64_t)Tk + j] * keep_scale : 1.0f;
                    float p = expf((float)(sd * scale) - Li);
                    float ds = (float)(p * (dp * w - Di) * scale);
                    float pd = p * w;
                    for (int k = 0; k < Hd; ++k) {
                        dqi[k] += ds * kj[k];
                        dkj[k] += ds * qi[k];
                        dvj[k] += pd * doi[k];
                    }
                }
            }
        }
}
