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
// Blackwell structure: one CTA per 256 query rows = two 128-row tiles that take
// turns on the tensor pipe, so that the softmax of one tile runs while the
// MMAs of the other execute.
//   warp 0        TMA producer: both Q tiles once, then K and V tiles through a
//                 two-stage ring (128-byte-swizzled boxes of 128 rows x 32
//                 floats, mbarrier tx; V with the 32-byte-chunk swizzle an
//                 MN-major TF32 operand needs).
//   warp 1        MMA issuer (the whole warp runs the issuing code, one elected lane issues).
//                 S_t = Q_t K^T is 8 tcgen05.mma (M128 N128 K8, operands from
//                 shared memory), O_t += P_t V is 16 (M128 N64 K8, A = P_t read
//                 from tensor memory, B = V MN-major from shared memory).  The
//                 (step, tile) products are numbered in the order (0,0) (0,1) (1,0)
//                 (1,1) ...; product q keeps its S, then its P, in score buffer
//                 q mod 3, and the issue order is S(0) S(1) S(2) | P V(0) S(3) |
//                 P V(1) S(4) | ...: the scores of a tile's NEXT step are computed
//                 while its softmax works on the current one (the tensor pipe
//                 executes in issue order, so S(q+3) cannot overtake the P V(q)
//                 that reads the same buffer).
//   warps 4-7     softmax of tile 0, warps 8-11 softmax of tile 1: thread r owns
//                 query row r (tensor-memory lane r), holds the 128 scores of a
//                 step in registers (one tensor-memory read per score), writes P
//                 back over S.  The running output is rescaled only when the
//                 running maximum grew by more than 2^8 (the final O/l and LSE
//                 use the same maximum, so the result is the same function).
// Tensor memory: three score buffers (128 columns each), O_0, O_1 (64 columns each): 512 of 512 columns.
// Warps 0-3 give most of their registers to the softmax warps (setmaxnreg 56 / 224).
#include <mutex>

#include "attn_kernels.cuh"
#include "philox.h"

namespace hk {

namespace fwd {

constexpr int NUM_THREADS = 384;
constexpr int TMEM_COLS = 512;
constexpr int COL_O0 = 256;  // O_t at COL_O0 + 64 t
// score buffer b of three: columns 0, 128, 384
__device__ __forceinline__ uint32_t score_col(int b) { return b == 2 ? 384u : (uint32_t)b * 128u; }
constexpr int NST = 2;       // K/V ring depth
constexpr float RESCALE_THRESHOLD = 8.f;  // log2 units

struct __align__(8) Shared {
    uint64_t q_full, k_full[NST], k_empty[NST], v_full[NST], v_empty[NST], s_full[3], p_full[3], o_full[3];
    // round_in_smem: warps 2, 3 have rounded the landed tile to TF32; the rounded Q tiles have been read by their store
    uint64_t q_round, k0_round, k_round[NST], v_round[NST], q_stored;
    uint32_t tmem_base;
    int abort_flag;
};

constexpr int OFF_Q = 0;                          // two tiles
constexpr int OFF_K = 2 * TILE_BYTES;             // NST stages
constexpr int OFF_V = OFF_K + NST * TILE_BYTES;   // NST stages
constexpr int OFF_SH = OFF_V + NST * TILE_BYTES;
constexpr int SMEM_BYTES = OFF_SH + sizeof(Shared);
static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KiB a CTA may opt in to");

enum WaitId { W_QFULL = 101, W_KFULL, W_KEMPTY, W_VFULL, W_VEMPTY, W_SFULL, W_PFULL, W_OFULL };

// Timeline slots (SM clock): role 0 = MMA issuer, 1 = softmax thread 0 of tile 0, 2 = of tile 1;
// buffer[1 + (j * 3 + role) * 8 + ph]; buffer[0] = number of KV steps of the recorded CTA.
#ifdef HK_TIMELINE
__device__ __forceinline__ void stamp(const FwdArgs& a, bool on, int j, int role, int ph) {
    if (on && j < 150) a.timeline[1 + (j * 3 + role) * 8 + ph] = clock64();
}
#else
__device__ __forceinline__ void stamp(const FwdArgs&, bool, int, int, int) {}
#endif

// 384 threads x 168 registers at launch = 128 x 56 + 256 x 224 after the hand-over (setmaxnreg.inc can only take what
// the launch-time pool of the CTA holds)
static_assert(128 * 56 + 256 * 224 <= NUM_THREADS * 168, "register hand-over exceeds the CTA's pool");
__device__ __forceinline__ void reg_release() { asm volatile("setmaxnreg.dec.sync.aligned.u32 56;\n"); }
__device__ __forceinline__ void reg_acquire() { asm volatile("setmaxnreg.inc.sync.aligned.u32 224;\n"); }

// number of key tiles the 128-row query tile starting at local row q0 attends to
__device__ __forceinline__ int kv_tiles_for(const FwdArgs& a, int q0) {
    if (q0 >= a.Tq) return 0;
    int kv_end = a.Tk;
    if (a.causal) {
        const int last_row = min(q0 + TILE, a.Tq) - 1;
        const long long lim = (long long)a.q_pos0 + last_row - a.k_pos0 + 1;
        kv_end = (int)max(0ll, min((long long)a.Tk, lim));
    }
    return (kv_end + TILE - 1) / TILE;
}

}  // namespace fwd

__global__ void __launch_bounds__(fwd::NUM_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapO,
                const __grid_constant__ CUtensorMap mapQw, const __grid_constant__ CUtensorMap mapKw,
                const __grid_constant__ CUtensorMap mapVw, const FwdArgs a) {
    using namespace fwd;
    extern __shared__ __align__(1024) uint8_t smem[];
    // schedule trace (timeline_block < 0): {start ns, end ns, SM id, key tiles} of each of the first 1024 CTAs
#ifdef HK_TIMELINE
    const bool trace = a.timeline != nullptr && a.timeline_block < 0 && blockIdx.x < 1024 && threadIdx.x == 0;
#else
    constexpr bool trace = false;
#endif
    if (trace) {
        a.timeline[4 * blockIdx.x] = (long long)globaltimer_ns();
        a.timeline[4 * blockIdx.x + 2] = smid();
    }
    if ((smem_u32(smem) & 1023u) != 0) {  // never expected; refuse to run on a misplaced buffer
        if (threadIdx.x == 0 && atomicCAS(&a.status->code, 0, 199) == 0) a.status->block = blockIdx.x;
        return;
    }
    uint8_t* sQ = smem + OFF_Q;
    uint8_t* sK = smem + OFF_K;
    uint8_t* sV = smem + OFF_V;
    Shared& sh = *reinterpret_cast<Shared*>(smem + OFF_SH);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // heavy (late) query blocks first: under the causal mask they have the most key tiles
    const int bh = blockIdx.x % a.BH;
    const int qb = a.n_qtiles - 1 - (int)(blockIdx.x / a.BH);  // n_qtiles counts 256-row blocks here
    const int b = bh / a.H;
    const int h = bh - b * a.H;
    const int q0 = qb * 2 * TILE;
    const int n0 = kv_tiles_for(a, q0);
    const int n1 = kv_tiles_for(a, q0 + TILE);
    const int n = max(n0, n1);

    // The producer initialises the barriers its copies complete on and issues the first loads at once (Q, and the
    // first NST key/value tiles, which wait for no consumer): the rest of the set-up -- the other barriers, the
    // tensor-memory allocation -- runs under their latency.  The other warps meet these barriers only after the
    // __syncthreads below.
    if (warp == 0 && lane == 0) {
        mbar_init(&sh.q_full, 1);
        for (int s = 0; s < NST; ++s) {
            mbar_init(&sh.k_full[s], 1);
            mbar_init(&sh.v_full[s], 1);
        }
        fence_mbar_init();
        if (n > 0) {
            mbar_arrive_expect_tx(&sh.q_full, 2 * TILE_BYTES);
            for (int t = 0; t < 2; ++t) {
                tma_load_4d(sQ + t * TILE_BYTES, &mapQ, &sh.q_full, 0, q0 + t * TILE, h, b);
                tma_load_4d(sQ + t * TILE_BYTES + BOX_BYTES, &mapQ, &sh.q_full, HALF_D, q0 + t * TILE, h, b);
            }
            for (int j = 0; j < n && j < NST; ++j) {
                mbar_arrive_expect_tx(&sh.k_full[j], TILE_BYTES);
                tma_load_4d(sK + j * TILE_BYTES, &mapK, &sh.k_full[j], 0, j * TILE, h, b);
                tma_load_4d(sK + j * TILE_BYTES + BOX_BYTES, &mapK, &sh.k_full[j], HALF_D, j * TILE, h, b);
                mbar_arrive_expect_tx(&sh.v_full[j], TILE_BYTES);
                tma_load_4d(sV + j * TILE_BYTES, &mapV, &sh.v_full[j], 0, j * TILE, h, b);
                tma_load_4d(sV + j * TILE_BYTES + BOX_BYTES, &mapV, &sh.v_full[j], HALF_D, j * TILE, h, b);
            }
        }
    }
    if (threadIdx.x == 64) {  // an idle warp takes the rest of the barriers
        for (int s = 0; s < NST; ++s) {
            // round_in_smem: a stage is free when the MMAs have read it AND the rounding warps are done with it (they
            // may still have a store of the rounded tile reading it)
            mbar_init(&sh.k_empty[s], a.round_in_smem ? 2 : 1);
            mbar_init(&sh.v_empty[s], a.round_in_smem ? 2 : 1);
        }
        // The score barriers belong to the score BUFFER, not to the tile: the warps of a tile may be a whole step
        // apart (the scores of the next step are there before the slowest warp has finished this one), and a
        // buffer is only refilled after every thread has handed over the P it held.
        for (int bf = 0; bf < 3; ++bf) {
            mbar_init(&sh.s_full[bf], 1);
            mbar_init(&sh.p_full[bf], 128);
            mbar_init(&sh.o_full[bf], 1);
        }
        mbar_init(&sh.q_round, 256);   // Q and the first K tile are rounded by the softmax warps, idle at that point
        mbar_init(&sh.k0_round, 256);
        mbar_init(&sh.q_stored, 1);
        for (int s = 0; s < NST; ++s) {
            mbar_init(&sh.k_round[s], 64);
            mbar_init(&sh.v_round[s], 64);
        }
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
#ifdef HK_TIMELINE
    const bool tl = a.timeline != nullptr && (int)blockIdx.x == a.timeline_block;
#else
    constexpr bool tl = false;
#endif
    if (tl && threadIdx.x == 0) a.timeline[0] = n;

    if (warp < 4) {
        reg_release();
        if (warp == 0) {
            // ------------------------------ TMA producer ------------------------------
            if (lane == 0 && n > 0) {
                // Q and the first NST key/value tiles were issued before the set-up barrier
                int issued = min(n, NST);
                for (int j = NST; j < n; ++j) {
                    const int s = j % NST;
                    const uint32_t par = ((j / NST) - 1) & 1;
                    if (j >= NST && !mbar_wait(wc, &sh.k_empty[s], par, W_KEMPTY, j)) break;
                    mbar_arrive_expect_tx(&sh.k_full[s], TILE_BYTES);
                    tma_load_4d(sK + s * TILE_BYTES, &mapK, &sh.k_full[s], 0, j * TILE, h, b);
                    tma_load_4d(sK + s * TILE_BYTES + BOX_BYTES, &mapK, &sh.k_full[s], HALF_D, j * TILE, h, b);
                    if (j >= NST && !mbar_wait(wc, &sh.v_empty[s], par, W_VEMPTY, j)) {
                        for (int i = 0; i < 100000 && !mbar_try_wait(&sh.k_full[s], (j / NST) & 1); ++i) {}
                        break;
                    }
                    mbar_arrive_expect_tx(&sh.v_full[s], TILE_BYTES);
                    tma_load_4d(sV + s * TILE_BYTES, &mapV, &sh.v_full[s], 0, j * TILE, h, b);
                    tma_load_4d(sV + s * TILE_BYTES + BOX_BYTES, &mapV, &sh.v_full[s], HALF_D, j * TILE, h, b);
                    issued = j + 1;
                }
                // Do not leave the CTA while bulk copies into its shared memory are in flight.
                for (int i = 0; i < 100000 && !mbar_try_wait(&sh.q_full, 0); ++i) {}
                for (int j = max(0, issued - NST); j < issued; ++j) {
                    for (int i = 0; i < 100000 && !mbar_try_wait(&sh.k_full[j % NST], (j / NST) & 1); ++i) {}
                    for (int i = 0; i < 100000 && !mbar_try_wait(&sh.v_full[j % NST], (j / NST) & 1); ++i) {}
                }
            }
        } else if (warp == 1) {
            // ------------------------------ MMA issuer ------------------------------
            // The whole warp runs this code with uniform control flow; only the tcgen05 instructions are predicated
            // on the elected lane (see umma_ss_tf32_lead).
            if (n > 0) {
                const uint32_t leader = elect_one_sync();
                auto wait = [&](uint64_t* bar, uint32_t parity, int id, int aux) -> bool {
                    return __all_sync(0xffffffffu, mbar_wait(wc, bar, parity, id, aux));
                };
                const bool tlm = tl && leader;
                constexpr uint32_t IDESC_S = make_idesc_tf32(TILE, TILE, false, false);
                constexpr uint32_t IDESC_O = make_idesc_tf32(TILE, HEAD_DIM, false, true);
                const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
                auto issue_qk = [&](int t, int s, int buf) {
                    const uint32_t d = tmem + score_col(buf);
#pragma unroll
                    for (int kk = 0; kk < HEAD_DIM / 8; ++kk)
                        umma_ss_tf32_lead(leader, d, kmajor_desc(q_addr + t * TILE_BYTES, kk, BOX_BYTES),
                                     kmajor_desc(k_addr + s * TILE_BYTES, kk, BOX_BYTES), IDESC_S, kk > 0);
                    umma_commit_lead(leader, &sh.s_full[buf]);
                };
                auto issue_pv = [&](int t, int s, int buf, bool first) {  // O_t += P V, P in score buffer buf
                    const uint32_t p = tmem + score_col(buf);
#pragma unroll
                    for (int kk = 0; kk < TILE / 8; ++kk)
                        umma_ts_tf32_lead(leader, tmem + COL_O0 + t * HEAD_DIM, p + kk * 8,
                                     mnmajor_desc(v_addr + s * TILE_BYTES, kk, BOX_BYTES), IDESC_O,
                                     (!first || kk > 0) ? 1u : 0u);
                    umma_commit_lead(leader, &sh.o_full[buf]);
                };
                // products in issue order: step by step, tile 0 before tile 1 (a tile takes part while j < n_t)
                const int total = n0 + n1;
                auto advance = [&](int& j, int& t) {
                    if (t == 0 && j < n1) {
                        t = 1;
                    } else {
                        ++j;
                        t = (j < n0) ? 0 : 1;
                    }
                };
                int jq = 0, tq = (n0 > 0) ? 0 : 1, nq = 0;  // the next S = Q K^T to issue and its number
                auto next_qk = [&]() -> bool {
                    if (nq >= total) return true;
                    const int s = jq % NST;
                    if (tq == 0 || jq >= n0) {  // first product that reads this key tile
                        // round_in_smem: the first key tile has a barrier of its own (other warps round it), so stage 0
                        // of k_round starts counting at key tile NST
                        uint64_t* kbar = !a.round_in_smem ? &sh.k_full[s] : (jq == 0 ? &sh.k0_round : &sh.k_round[s]);
                        const uint32_t kpar = (a.round_in_smem && s == 0 && jq > 0) ? ((jq / NST) - 1) & 1 : (jq / NST) & 1;
                        if (!wait(kbar, kpar, W_KFULL, jq)) return false;
                        tc_fence_after_sync();
                    }
                    issue_qk(tq, s, nq % 3);
                    if (tq == 1 || jq >= n1) umma_commit_lead(leader, &sh.k_empty[s]);  // last one that reads it
                    ++nq;
                    advance(jq, tq);
                    return true;
                };
                bool ok = wait(a.round_in_smem ? &sh.q_round : &sh.q_full, 0, W_QFULL, 0);
                for (int i = 0; ok && i < 3; ++i) ok = next_qk();
                int j = 0, t = (n0 > 0) ? 0 : 1;
                for (int q = 0; ok && q < total; ++q) {
                    const int s = j % NST;
                    stamp(a, tlm, j, 0, 3 * t);
                    if (t == 0 || j >= n0) {
                        if (!(ok = wait(a.round_in_smem ? &sh.v_round[s] : &sh.v_full[s], (j / NST) & 1, W_VFULL, j))) break;
                    }
                    if (!(ok = wait(&sh.p_full[q % 3], (q / 3) & 1, W_PFULL, j))) break;
                    stamp(a, tlm, j, 0, 1 + 3 * t);
                    tc_fence_after_sync();
                    issue_pv(t, s, q % 3, j == 0 && !a.continue_state);
                    if (t == 1 || j >= n1) umma_commit_lead(leader, &sh.v_empty[s]);
                    ok = next_qk();
                    stamp(a, tlm, j, 0, 2 + 3 * t);
                    advance(j, t);
                }
            }
        }
        else if (a.round_in_smem && n > 0) {
            // Warps 2 and 3 round what the TMA has landed to TF32 in place (add 0x1000, clear the low 13 bits: what
            // the HBM pre-pass does, so every result is bit-identical to that path): every K and V tile of the ring
            // but the first K tile, which the softmax warps take together with the two Q tiles while they have
            // nothing else to do.  Short sequences only (the host decides): there the pre-pass costs
            // more than this traffic on the shared-memory port that the S = Q K^T products are bound by.
            const int rt = threadIdx.x - 64;  // 0..63
            auto round_tile = [&](uint8_t* tile, int bytes) {
                uint4* p4 = reinterpret_cast<uint4*>(tile);
#pragma unroll 8
                for (int i = rt; i < bytes / 16; i += 64) {
                    uint4 x = p4[i];
                    x.x = tf32_round_bits(x.x); x.y = tf32_round_bits(x.y);
                    x.z = tf32_round_bits(x.z); x.w = tf32_round_bits(x.w);
                    p4[i] = x;
                }
                fence_proxy_async_smem();
            };
            // Each key/value tile is written out by the first query block that loads it: block qb takes the tiles
            // from where block qb - 1 stops (under the causal mask later blocks see more keys, never fewer).
            int j_store0 = 0;
            if (a.store_q && qb > 0) {
                const int qp = (qb - 1) * 2 * TILE;
                j_store0 = max(kv_tiles_for(a, qp), kv_tiles_for(a, qp + TILE));
            }
            bool rok = true;
            for (int j = 0; rok && j < n; ++j) {
                const int s = j % NST;
                const uint32_t par = (j / NST) & 1;
                const bool store = a.store_q && j >= j_store0;
                if (j > 0) {  // the softmax warps take Q and the first key tile
                    if (!(rok = __all_sync(0xffffffffu, mbar_wait(wc, &sh.k_full[s], par, W_KFULL, 2000 + j)))) break;
                    round_tile(sK + s * TILE_BYTES, TILE_BYTES);
                    mbar_arrive(&sh.k_round[s]);
                }
                if (!(rok = __all_sync(0xffffffffu, mbar_wait(wc, &sh.v_full[s], par, W_VFULL, 2000 + j)))) break;
                round_tile(sV + s * TILE_BYTES, TILE_BYTES);
                mbar_arrive(&sh.v_round[s]);
                if (rt == 0) {
                    // one thread writes the rounded tiles out and hands the stages back.  It has arrived on the
                    // tiles' barriers itself and waits for them: every thread's part is rounded and fenced.
                    bool all_in = true;
                    if (store || (j == 0 && a.store_q)) {
                        if (j == 0 && a.store_q) {
                            all_in = mbar_wait(wc, &sh.q_round, 0, W_QFULL, 2);
                            if (all_in) {
                                for (int t = 0; t < 2; ++t) {
                                    if (q0 + t * TILE < a.Tq) {
                                        tma_store_4d(&mapQw, sQ + t * TILE_BYTES, 0, q0 + t * TILE, h, b);
                                        tma_store_4d(&mapQw, sQ + t * TILE_BYTES + BOX_BYTES, HALF_D, q0 + t * TILE, h, b);
                                    }
                                }
                            }
                        }
                        if (store && all_in)
                            all_in = mbar_wait(wc, j == 0 ? &sh.k0_round : &sh.k_round[s],
                                               (s == 0 && j > 0) ? ((j / NST) - 1) & 1 : par, W_KFULL, 3000 + j) &&
                                     mbar_wait(wc, &sh.v_round[s], par, W_VFULL, 3000 + j);
                        if (store && all_in) {
                            tma_store_4d(&mapKw, sK + s * TILE_BYTES, 0, j * TILE, h, b);
                            tma_store_4d(&mapKw, sK + s * TILE_BYTES + BOX_BYTES, HALF_D, j * TILE, h, b);
                            tma_store_4d(&mapVw, sV + s * TILE_BYTES, 0, j * TILE, h, b);
                            tma_store_4d(&mapVw, sV + s * TILE_BYTES + BOX_BYTES, HALF_D, j * TILE, h, b);
                        }
                        bulk_commit_group();
                        bulk_wait_group_read_all();
                        if (j == 0 && a.store_q) mbar_arrive(&sh.q_stored);  // the epilogue may reuse the Q buffer
                    }
                    mbar_arrive(&sh.k_empty[s]);
                    mbar_arrive(&sh.v_empty[s]);
                }
                __syncwarp();
            }
            if (!rok && a.store_q && rt == 0) mbar_arrive(&sh.q_stored);  // (a second arrival is harmless)
        }
        // teardown of the control warps (kept inside this branch: the two register regimes never
        // share code after the hand-over)
        tc_fence_before_sync();
        __syncthreads();
        if (warp == 1) {
            __syncwarp();
            tc_fence_after_sync();
            tmem_dealloc(tmem, TMEM_COLS);
        }
    } else {
        // ------------------------------ softmax ------------------------------
        reg_acquire();
        const int t = (warp - 4) >> 2;                   // which of the two query tiles
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;             // row inside the query tile = tensor-memory lane
        const int qrow = q0 + t * TILE + row;            // row inside this (b,h)
        const bool row_ok = qrow < a.Tq;
        const int nt = t == 0 ? n0 : n1;
        const uint32_t trow = tmem + ((uint32_t)(quarter * 32) << 16);
        const uint32_t tO = trow + COL_O0 + t * HEAD_DIM;
        const bool tls = tl && row == 0;
        // last key index (local to this call's K) this row may see
        long long lim_ll = a.Tk - 1;
        if (a.causal) lim_ll = min(lim_ll, (long long)a.q_pos0 + qrow - a.k_pos0);
        const int kv_lim = row_ok ? (int)max(-1ll, lim_ll) : -1;
        const float c = a.scale_log2e;
        const float worst = (c >= 0.f) ? -INFINITY : INFINITY;  // raw score that can never win the max

        const bool scaled = a.drop_scaled != 0;
        float m = -INFINITY;  // running max actually used as exponent reference, log2 units
        float l = 0.f;
        bool ok = true;
        uint32_t r[128];
        if (a.continue_state && nt > 0) {
            // The result over the keys seen so far is the starting state: reference LSE, normaliser 1 and the running
            // output O itself (a row that has seen no key starts from nothing).  The output accumulator is written
            // before this thread's first arrival on p_full, which the first P V of the tile waits for.
            const float lse0 = row_ok ? a.LSE[(int64_t)b * a.lse_sB + (int64_t)h * a.lse_sH + qrow] : -INFINITY;
            const bool have = lse0 > -INFINITY;
            m = have ? lse0 * LOG2E : -INFINITY;
            l = have ? 1.f : 0.f;
            const float4* orow = reinterpret_cast<const float4*>(a.O + (int64_t)b * a.o_sB + (int64_t)h * a.o_sH +
                                                                 (int64_t)(row_ok ? qrow : 0) * a.o_sM);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float4 v = have ? orow[i] : make_float4(0.f, 0.f, 0.f, 0.f);
                r[4 * i] = __float_as_uint(v.x); r[4 * i + 1] = __float_as_uint(v.y);
                r[4 * i + 2] = __float_as_uint(v.z); r[4 * i + 3] = __float_as_uint(v.w);
            }
            tmem_st32p(tO, r);
            tmem_st32p(tO + 32, r + 32);
            tmem_wait_st();
        }

        if (a.round_in_smem && n > 0) {
            // Q (both tiles) and the first K tile: rounded by the 256 softmax threads, which wait for the first scores
            // anyway (a tile without keys of its own still takes its share)
            const int st = threadIdx.x - 128;  // 0..255
            auto round_part = [&](uint8_t* buf, int bytes) {
                uint4* p4 = reinterpret_cast<uint4*>(buf);
#pragma unroll 4
                for (int i = st; i < bytes / 16; i += 256) {
                    uint4 x = p4[i];
                    x.x = tf32_round_bits(x.x); x.y = tf32_round_bits(x.y);
                    x.z = tf32_round_bits(x.z); x.w = tf32_round_bits(x.w);
                    p4[i] = x;
                }
                fence_proxy_async_smem();
            };
            if (__all_sync(0xffffffffu, mbar_wait(wc, &sh.q_full, 0, W_QFULL, 4))) {
                round_part(sQ, 2 * TILE_BYTES);
                mbar_arrive(&sh.q_round);
                if (__all_sync(0xffffffffu, mbar_wait(wc, &sh.k_full[0], 0, W_KFULL, 4000))) {
                    round_part(sK, TILE_BYTES);
                    mbar_arrive(&sh.k0_round);
                }
            }
        }
        int q_prev = 0;  // number of this tile's previous product
        for (int j = 0; j < nt; ++j) {
            stamp(a, tls, j, 1 + t, 0);
            // this product's number in the issue order picks its score buffer
            const int q = min(j, n0) + min(j, n1) + ((t == 1 && j < n0) ? 1 : 0);
            const uint32_t tS = trow + score_col(q % 3);
            // the vote keeps the warp converged for the .sync.aligned tensor-memory accesses below
            ok = __all_sync(0xffffffffu, mbar_wait(wc, &sh.s_full[q % 3], (q / 3) & 1, W_SFULL, j));
            if (!ok) break;
            stamp(a, tls, j, 1 + t, 1);
            tc_fence_after_sync();
            tmem_ld32p(tS, r);
            tmem_ld32p(tS + 32, r + 32);
            tmem_ld32p(tS + 64, r + 64);
            tmem_ld32p(tS + 96, r + 96);
            const int kv0 = j * TILE;
            const int lim_local = kv_lim - kv0;  // columns 0..lim_local are visible
            tmem_wait_ld();
            stamp(a, tls, j, 1 + t, 2);
            if (lim_local < TILE - 1) {
#pragma unroll
                for (int i = 0; i < 128; ++i)
                    if (i > lim_local) r[i] = __float_as_uint(worst);
            }
            // row max of the raw scores (min if the scale is negative), four chains
            float mx0 = __uint_as_float(r[0]), mx1 = __uint_as_float(r[1]), mx2 = __uint_as_float(r[2]),
                  mx3 = __uint_as_float(r[3]);
            if (c >= 0.f) {
#pragma unroll
                for (int i = 4; i < 128; i += 4) {
                    mx0 = fmaxf(mx0, __uint_as_float(r[i]));
                    mx1 = fmaxf(mx1, __uint_as_float(r[i + 1]));
                    mx2 = fmaxf(mx2, __uint_as_float(r[i + 2]));
                    mx3 = fmaxf(mx3, __uint_as_float(r[i + 3]));
                }
                mx0 = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
            } else {
#pragma unroll
                for (int i = 4; i < 128; i += 4) {
                    mx0 = fminf(mx0, __uint_as_float(r[i]));
                    mx1 = fminf(mx1, __uint_as_float(r[i + 1]));
                    mx2 = fminf(mx2, __uint_as_float(r[i + 2]));
                    mx3 = fminf(mx3, __uint_as_float(r[i + 3]));
                }
                mx0 = fminf(fminf(mx0, mx1), fminf(mx2, mx3));
            }
            const float m_cand = mx0 * c;  // -inf when nothing is visible
            // raise the reference only when it pays: a stale m makes p at most 2^8 larger, which fp32 absorbs
            const bool raise = (m == -INFINITY) ? (m_cand > -INFINITY) : (m_cand > m + RESCALE_THRESHOLD);
            const float m_new = raise ? m_cand : m;
            const float alpha = raise ? ((m == -INFINITY) ? 0.f : ex2_approx(m - m_cand)) : 1.f;
            if ((j > 0 || a.continue_state) && __any_sync(0xffffffffu, raise)) {
                // rescale the running output, once the P V of the previous step has completed
                if (j > 0) {
                    ok = __all_sync(0xffffffffu, mbar_wait(wc, &sh.o_full[q_prev % 3], (q_prev / 3) & 1, W_OFULL, j));
                    if (!ok) break;
                    tc_fence_after_sync();
                }
#pragma unroll 1
                for (int cc = 0; cc < 2; ++cc) {
                    uint32_t o[32];
                    tmem_ld32(tO + cc * 32, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st32(tO + cc * 32, o);
                }
            }
            const float neg_m = (m_new == -INFINITY) ? 0.f : -m_new;
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
            if (a.dropout_mode == 0) {
                // two scores per FMA and per add (fma.rn.f32x2 / add.rn.f32x2: the same roundings as the scalar forms)
                const float2 c2 = make_float2(c, c), nm2 = make_float2(neg_m, neg_m);
                float2 s01 = make_float2(0.f, 0.f), s23 = make_float2(0.f, 0.f);
#pragma unroll
                for (int i = 0; i < 128; i += 4) {
                    const float2 t01 = __ffma2_rn(make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), c2, nm2);
                    const float2 t23 = __ffma2_rn(make_float2(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])), c2, nm2);
                    const float2 p01 = make_float2(ex2_approx(t01.x), ex2_approx(t01.y));
                    const float2 p23 = make_float2(ex2_approx(t23.x), ex2_approx(t23.y));
                    s01 = __fadd2_rn(s01, p01);
                    s23 = __fadd2_rn(s23, p23);
                    r[i] = tf32_round_bits_mma(__float_as_uint(p01.x));
                    r[i + 1] = tf32_round_bits_mma(__float_as_uint(p01.y));
                    r[i + 2] = tf32_round_bits_mma(__float_as_uint(p23.x));
                    r[i + 3] = tf32_round_bits_mma(__float_as_uint(p23.y));
                }
                s0 = s01.x; s1 = s01.y; s2 = s23.x; s3 = s23.y;
            } else if (a.dropout_mode == 2) {
                // one Philox call per eight keys of this row
#pragma unroll
                for (int g = 0; g < 16; ++g) {
                    const uint32_t kpos = (uint32_t)(a.k_pos0 + kv0 + g * 8);
                    const hk_philox4_t w = hk_philox_row8(a.seed, a.offset, a.bh_pos0 + (uint32_t)bh, (uint32_t)(a.q_pos0 + qrow), kpos >> 3);
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        float p = ex2_approx(fmaf(__uint_as_float(r[g * 8 + u]), c, neg_m));
                        const uint32_t half = (u & 1) ? (w.v[u >> 1] >> 16) : (w.v[u >> 1] & 0xFFFFu);
                        if (scaled) { if (u & 1) s3 += p; else s2 += p; }  // the normaliser ignores the mask
                        if (half < a.drop_thr) p = 0.f;
                        if (u & 1) s1 += p; else s0 += p;
                        r[g * 8 + u] = tf32_round_bits_mma(__float_as_uint(p));
                    }
                }
            } else {
                const float* mrow = a.mask + ((size_t)bh * a.Tq + (row_ok ? qrow : 0)) * (size_t)a.Tk + kv0;
#pragma unroll
                for (int i = 0; i < 128; ++i) {
                    float p = ex2_approx(fmaf(__uint_as_float(r[i]), c, neg_m));
                    if (scaled) s2 += (i <= lim_local) ? p : 0.f;
                    p = (i <= lim_local) ? p * __ldg(mrow + i) : 0.f;
                    s0 += p;
                    r[i] = tf32_round_bits_mma(__float_as_uint(p));
                }
            }
            tmem_st32p(tS, r);
            tmem_st32p(tS + 32, r + 32);
            tmem_st32p(tS + 64, r + 64);
            tmem_st32p(tS + 96, r + 96);
            // inverted dropout: s2, s3 hold the sums over all visible keys, s0, s1 the kept ones
            l = l * alpha + ((scaled && a.dropout_mode != 0) ? (s2 + s3) : ((s0 + s1) + (s2 + s3)));
            m = m_new;
            stamp(a, tls, j, 1 + t, 3);
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&sh.p_full[q % 3]);
            q_prev = q;
            stamp(a, tls, j, 1 + t, 4);
        }

        // epilogue: O / l and LSE
        if (ok && nt > 0) ok = __all_sync(0xffffffffu, mbar_wait(wc, &sh.o_full[q_prev % 3], (q_prev / 3) & 1, W_OFULL, nt));
        tc_fence_after_sync();
        const float inv_l = (l > 0.f) ? a.keep_scale / l : 0.f;
        if (ok && nt > 0) {
            tmem_ld32p(tO, r);
            tmem_ld32p(tO + 32, r + 32);
            tmem_wait_ld();
        } else {
#pragma unroll
            for (int i = 0; i < 64; ++i) r[i] = 0u;
        }
        // O leaves through shared memory and a TMA bulk store (a thread-per-row store would touch 32 lines per
        // instruction).  The tile's own Q buffer is dead -- o_full covered its last S = Q K^T -- and takes the
        // two 32-column boxes of a 128-byte-swizzled TMA tile: 16-byte chunk c of row r at position c ^ (r & 7).
        // Rows past the end of the sequence are clipped by the copy.
        // (a tile that had no key tile to wait for must still let the load of its Q land before reusing the buffer)
        if (nt == 0 && n > 0) __all_sync(0xffffffffu, mbar_wait(wc, &sh.q_full, 0, W_QFULL, 0));
        // ... and the store of the rounded Q tiles must have read it
        if (a.round_in_smem && a.store_q && n > 0) __all_sync(0xffffffffu, mbar_wait(wc, &sh.q_stored, 0, W_QFULL, 3));
        {
            uint8_t* srow = sQ + t * TILE_BYTES + row * 128;
#pragma unroll
            for (int i = 0; i < 64; i += 4) {
                float4 v;
                v.x = __uint_as_float(r[i]) * inv_l;
                v.y = __uint_as_float(r[i + 1]) * inv_l;
                v.z = __uint_as_float(r[i + 2]) * inv_l;
                v.w = __uint_as_float(r[i + 3]) * inv_l;
                const int c = (i >> 2) & 7;
                *reinterpret_cast<float4*>(srow + (i >> 5) * BOX_BYTES + ((c ^ (row & 7)) << 4)) = v;
            }
            fence_proxy_async_smem();
        }
        // a tile that saw no key of this call leaves a continued result untouched
        const bool keep_old = a.continue_state && nt == 0;
        if (row_ok && !keep_old)
            a.LSE[(int64_t)b * a.lse_sB + (int64_t)h * a.lse_sH + qrow] = (l > 0.f) ? (m + log2f(l)) * LN2 : -INFINITY;
        // the 128 threads of this query tile (every one gets here, whatever `ok` is), then one of them stores
        asm volatile("bar.sync %0, 128;" ::"r"(1 + t) : "memory");
        if (row == 0 && q0 + t * TILE < a.Tq && !keep_old) {
            tma_store_4d(&mapO, sQ + t * TILE_BYTES, 0, q0 + t * TILE, h, b);
            tma_store_4d(&mapO, sQ + t * TILE_BYTES + BOX_BYTES, HALF_D, q0 + t * TILE, h, b);
            bulk_commit_group();
            bulk_wait_group_all();
        }
        tc_fence_before_sync();
        __syncthreads();  // pairs with the control warps' barrier before tensor memory is freed
    }
    if (trace) {
        a.timeline[4 * blockIdx.x + 1] = (long long)globaltimer_ns();
        a.timeline[4 * blockIdx.x + 3] = n;
    }
}

int launch_attn_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo,
                    const CUtensorMap& mqw, const CUtensorMap& mkw, const CUtensorMap& mvw, const FwdArgs& a,
                    cudaStream_t stream) {
    // the opt-in to large dynamic shared memory is per device: once per device, safe from any number of host threads
    static std::once_flag attr_once[HK_MAX_DEVICES];
    static cudaError_t attr_rc[HK_MAX_DEVICES];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return HK_ERR_CUDA;
    if (dev < 0 || dev >= HK_MAX_DEVICES) return HK_ERR_UNSUPPORTED;
    std::call_once(attr_once[dev], [dev] {
        attr_rc[dev] = cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fwd::SMEM_BYTES);
    });
    if (attr_rc[dev] != cudaSuccess) return HK_ERR_CUDA;
    const long long nblocks = (long long)a.n_qtiles * a.BH;
    if (nblocks <= 0 || nblocks > 0x7fffffffLL) return HK_ERR_BAD_SHAPE;
    timing_mark(TIMED_FWD, true, stream);
    attn_fwd_kernel<<<(unsigned)nblocks, fwd::NUM_THREADS, fwd::SMEM_BYTES, stream>>>(mq, mk, mv, mo, mqw, mkw, mvw, a);
    timing_mark(TIMED_FWD, false, stream);
    count_launch();
    return check_launch();
}

}  // namespace hk
