// attn_fwd_sm100.cu -- fused attention forward for sm_100a.
//
// Computes what fused_attn_forward_kernel_tc_sm89<64,64,64,1> computes
// (kernels/attention/fused_attn_forward_kernel_tc_sm89.cu:72-426 of the
// reference): S = Q K^T on TF32 tensor cores, v = S*scale, causal mask,
// running max m and alpha = exp(m_old - m_new), e = exp(v - m_new), dropout
// mask multiplied into e BEFORE the row sum, l = alpha*l + sum(e),
// O = alpha*O + P V with P rounded to TF32, finally O /= l (0 if l == 0) and
// LSE = m + log l (-inf if l == 0).
//
// Blackwell structure (one CTA = one 128-row query tile, two CTAs per SM):
//   warp 0      TMA producer: Q once, then one K tile and one V tile per step,
//               128-byte-swizzled boxes of 128 rows x 32 floats, mbarrier tx
//               (V with the 32-byte-chunk swizzle an MN-major TF32 operand needs).
//   warp 1      MMA issuer: S = Q K^T as 8 tcgen05.mma (M128 N128 K8, both
//               operands from shared memory), O += P V as 16 tcgen05.mma
//               (M128 N64 K8, A = P read from tensor memory, B = V MN-major
//               from shared memory).  S (128 columns) and O (64 columns) live
//               in tensor memory; P overwrites S in place.
//   warps 2-5   softmax: thread r owns query row r (tensor-memory lane r), so
//               the row max and row sum need no cross-thread reduction.
// While one CTA's softmax warps work, the SM's other CTA keeps the tensor
// pipe busy.
#include "attn_kernels.cuh"
#include "philox.h"

namespace hk {

namespace fwd {

constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 256;
constexpr int COL_S = 0;
constexpr int COL_O = 128;

struct __align__(8) Shared {
    uint64_t q_full, k_full, k_empty, v_full, v_empty, s_full, p_full, o_full;
    uint32_t tmem_base;
    int abort_flag;
};

constexpr int SMEM_TILES = 3 * TILE_BYTES;                      // Q, K, V
constexpr int SMEM_BYTES = SMEM_TILES + sizeof(Shared) + 1024;  // + alignment slack

enum WaitId {
    W_QFULL = 101, W_KFULL, W_KEMPTY, W_VFULL, W_VEMPTY, W_SFULL, W_PFULL, W_OFULL
};

}  // namespace fwd

__global__ void __launch_bounds__(fwd::NUM_THREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                const __grid_constant__ CUtensorMap mapV, const FwdArgs a) {
    using namespace fwd;
    extern __shared__ uint8_t smem_raw[];
    // 128-byte-swizzled tiles need 1024-byte alignment
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sK = smem + TILE_BYTES;
    uint8_t* sV = smem + 2 * TILE_BYTES;
    Shared& sh = *reinterpret_cast<Shared*>(smem + SMEM_TILES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // heavy (late) query tiles first: under the causal mask they have the most key tiles
    const int bh = blockIdx.x % a.BH;
    const int qt = a.n_qtiles - 1 - (int)(blockIdx.x / a.BH);
    const int b = bh / a.H;
    const int h = bh - b * a.H;
    const int q0 = qt * TILE;

    // number of key tiles this query tile attends to
    int kv_end = a.Tk;
    if (a.causal) {
        const int last_row = min(q0 + TILE, a.Tq) - 1;
        const long long lim = (long long)a.q_pos0 + last_row - a.k_pos0 + 1;
        kv_end = (int)max(0ll, min((long long)a.Tk, lim));
    }
    const int n_kv = (kv_end + TILE - 1) / TILE;

    if (threadIdx.x == 0) {
        mbar_init(&sh.q_full, 1);
        mbar_init(&sh.k_full, 1);
        mbar_init(&sh.k_empty, 1);
        mbar_init(&sh.v_full, 1);
        mbar_init(&sh.v_empty, 1);
        mbar_init(&sh.s_full, 1);
        mbar_init(&sh.p_full, 128);
        mbar_init(&sh.o_full, 1);
        sh.abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(&sh.tmem_base, TMEM_COLS);
        tmem_relinquish();
        tc_fence_before_sync();
    }
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sh.tmem_base;
    WaitCtx wc{&sh.abort_flag, a.status};

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0 && n_kv > 0) {
            tma_prefetch_desc(&mapQ);
            tma_prefetch_desc(&mapK);
            tma_prefetch_desc(&mapV);
            mbar_arrive_expect_tx(&sh.q_full, TILE_BYTES);
            tma_load_4d(sQ, &mapQ, &sh.q_full, 0, q0, h, b);
            tma_load_4d(sQ + BOX_BYTES, &mapQ, &sh.q_full, HALF_D, q0, h, b);
            int issued = 0;  // key/value tiles whose loads were issued
            for (int j = 0; j < n_kv; ++j) {
                if (j > 0 && !mbar_wait(wc, &sh.k_empty, (j - 1) & 1, W_KEMPTY, j)) break;
                mbar_arrive_expect_tx(&sh.k_full, TILE_BYTES);
                tma_load_4d(sK, &mapK, &sh.k_full, 0, j * TILE, h, b);
                tma_load_4d(sK + BOX_BYTES, &mapK, &sh.k_full, HALF_D, j * TILE, h, b);
                if (j > 0 && !mbar_wait(wc, &sh.v_empty, (j - 1) & 1, W_VEMPTY, j)) {
                    // K(j) is in flight: let it land before the CTA may exit
                    for (int i = 0; i < 100000 && !mbar_try_wait(&sh.k_full, j & 1); ++i) {}
                    break;
                }
                mbar_arrive_expect_tx(&sh.v_full, TILE_BYTES);
                tma_load_4d(sV, &mapV, &sh.v_full, 0, j * TILE, h, b);
                tma_load_4d(sV + BOX_BYTES, &mapV, &sh.v_full, HALF_D, j * TILE, h, b);
                issued = j + 1;
            }
            // Do not leave the CTA while bulk copies into its shared memory are in flight.
            if (issued > 0) {
                const uint32_t par = (issued - 1) & 1;
                for (int i = 0; i < 100000 && !mbar_try_wait(&sh.q_full, 0); ++i) {}
                for (int i = 0; i < 100000 && !mbar_try_wait(&sh.k_full, par); ++i) {}
                for (int i = 0; i < 100000 && !mbar_try_wait(&sh.v_full, par); ++i) {}
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0 && n_kv > 0) {
            constexpr uint32_t IDESC_S = make_idesc_tf32(TILE, TILE, false, false);
            constexpr uint32_t IDESC_O = make_idesc_tf32(TILE, HEAD_DIM, false, true);
            const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
            bool ok = mbar_wait(wc, &sh.q_full, 0, W_QFULL);
            for (int j = 0; ok && j < n_kv; ++j) {
                const uint32_t par = j & 1;
                if (!(ok = mbar_wait(wc, &sh.k_full, par, W_KFULL, j))) break;
                tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < HEAD_DIM / 8; ++kk) {
                    umma_ss_tf32(tmem + COL_S, kmajor_desc(q_addr, kk, BOX_BYTES), kmajor_desc(k_addr, kk, BOX_BYTES),
                                 IDESC_S, kk > 0);
                }
                umma_commit(&sh.k_empty);
                umma_commit(&sh.s_full);
                if (!(ok = mbar_wait(wc, &sh.v_full, par, W_VFULL, j))) break;
                if (!(ok = mbar_wait(wc, &sh.p_full, par, W_PFULL, j))) break;
                tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < TILE / 8; ++kk) {
                    umma_ts_tf32(tmem + COL_O, tmem + COL_S + kk * 8, mnmajor_desc(v_addr, kk, BOX_BYTES), IDESC_O,
                                 (j > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(&sh.v_empty);
                umma_commit(&sh.o_full);
            }
        }
    } else {
        // ------------------------------ softmax ------------------------------
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;             // row inside the query tile = tensor-memory lane
        const int qrow = q0 + row;                       // row inside this (b,h)
        const bool row_ok = qrow < a.Tq;
        const uint32_t trow = tmem + ((uint32_t)(quarter * 32) << 16);
        // last key index (local to this call's K) this row may see
        long long lim_ll = a.Tk - 1;
        if (a.causal) lim_ll = min(lim_ll, (long long)a.q_pos0 + qrow - a.k_pos0);
        const int kv_lim = row_ok ? (int)max(-1ll, lim_ll) : -1;

        float m = -INFINITY;  // running max, log2 units (score * scale * log2e)
        float l = 0.f;
        bool ok = true;
        uint32_t r[32];

        for (int j = 0; j < n_kv; ++j) {
            // the vote keeps the warp converged for the .sync.aligned tensor-memory accesses below
            ok = __all_sync(0xffffffffu, mbar_wait(wc, &sh.s_full, j & 1, W_SFULL, j));
            if (!ok) break;
            tc_fence_after_sync();
            const int kv0 = j * TILE;
            const bool full = (kv0 + TILE - 1 <= kv_lim);  // no masking needed for this row

            // pass 1: row max of the scaled scores
            float mx = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                tmem_ld32(trow + COL_S + c * 32, r);
                tmem_wait_ld();
                if (full) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]) * a.scale_log2e);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (kv0 + c * 32 + i <= kv_lim) mx = fmaxf(mx, __uint_as_float(r[i]) * a.scale_log2e);
                }
            }
            const float m_new = fmaxf(m, mx);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = (m == -INFINITY) ? 0.f : ex2_approx(m - m_use);

            // rescale the running output (PV of the previous step has completed:
            // s_full of this step was committed after it)
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
                for (int c = 0; c < 2; ++c) {
                    tmem_ld32(trow + COL_O + c * 32, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                    tmem_st32(trow + COL_O + c * 32, r);
                }
            }

            // pass 2: P = exp2(s*scale*log2e - m), masked, dropped, summed, rounded, written over S
            float sum = 0.f;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                tmem_ld32(trow + COL_S + c * 32, r);
                tmem_wait_ld();
                const int kc0 = kv0 + c * 32;
                float e[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float v = ex2_approx(fmaf(__uint_as_float(r[i]), a.scale_log2e, -m_use));
                    if (!full && (kc0 + i > kv_lim)) v = 0.f;
                    e[i] = v;
                }
                if (a.dropout_mode == 2) {
                    if (row_ok) {
#pragma unroll
                        for (int g = 0; g < 8; ++g) {
                            const uint32_t kpos = (uint32_t)(a.k_pos0 + kc0 + g * 4);
                            hk_philox4_t w = hk_philox_row4(a.seed, a.offset, (uint32_t)bh,
                                                            (uint32_t)(a.q_pos0 + qrow), kpos >> 2);
#pragma unroll
                            for (int t = 0; t < 4; ++t)
                                if (w.v[t] < a.drop_thr) e[g * 4 + t] = 0.f;
                        }
                    }
                } else if (a.dropout_mode == 1) {
                    if (row_ok) {
                        const float* mrow = a.mask + ((size_t)bh * a.Tq + qrow) * (size_t)a.Tk;
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (kc0 + i <= kv_lim) e[i] *= __ldg(mrow + kc0 + i);
                    }
                }
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    sum += e[i];
                    r[i] = tf32_round_bits(__float_as_uint(e[i]));
                }
                tmem_st32(trow + COL_S + c * 32, r);
            }
            l = l * alpha + sum;
            m = m_new;
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&sh.p_full);
        }

        // epilogue: O / l and LSE
        if (ok && n_kv > 0) ok = __all_sync(0xffffffffu, mbar_wait(wc, &sh.o_full, (n_kv - 1) & 1, W_OFULL, n_kv));
        tc_fence_after_sync();
        const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
        float* orow = a.O + (int64_t)b * a.o_sB + (int64_t)h * a.o_sH + (int64_t)qrow * a.o_sM;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
            if (ok && n_kv > 0) {
                tmem_ld32(trow + COL_O + c * 32, r);
                tmem_wait_ld();
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) r[i] = 0u;
            }
            if (row_ok) {
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    float4 v;
                    v.x = __uint_as_float(r[i]) * inv_l;
                    v.y = __uint_as_float(r[i + 1]) * inv_l;
                    v.z = __uint_as_float(r[i + 2]) * inv_l;
                    v.w = __uint_as_float(r[i + 3]) * inv_l;
                    *reinterpret_cast<float4*>(orow + c * 32 + i) = v;
                }
            }
        }
        if (row_ok)
            a.LSE[(int64_t)b * a.lse_sB + (int64_t)h * a.lse_sH + qrow] =
                (l > 0.f) ? (m + log2f(l)) * LN2 : -INFINITY;
    }

    // ------------------------------ teardown ------------------------------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

int launch_attn_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const FwdArgs& a,
                    cudaStream_t stream) {
    static bool attr_done[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return HK_ERR_CUDA;
    if (dev < 64 && !attr_done[dev]) {
        if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fwd::SMEM_BYTES) !=
            cudaSuccess)
            return HK_ERR_CUDA;
        attr_done[dev] = true;
    }
    const long long nblocks = (long long)a.n_qtiles * a.BH;
    if (nblocks <= 0 || nblocks > 0x7fffffffLL) return HK_ERR_BAD_SHAPE;
    timing_mark(TIMED_FWD, true, stream);
    attn_fwd_kernel<<<(unsigned)nblocks, fwd::NUM_THREADS, fwd::SMEM_BYTES, stream>>>(mq, mk, mv, a);
    timing_mark(TIMED_FWD, false, stream);
    count_launch();
    return check_launch();
}

}  // namespace hk
