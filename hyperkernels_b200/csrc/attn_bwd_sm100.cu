// attn_bwd_sm100.cu -- fused attention backward for sm_100a.
//
// Computes what mem_efficient_bwd_unified_kernel_exp12<64,Causal> computes
// (kernels/attention/mem_efficient_bwd_unified_kernel_exp12.cu:54-329 of the
// reference), one KV tile per CTA, looping over the query tiles that can see it:
//   S = Q K^T, dP = dO V^T                    (:186-212)
//   p = exp2(log2e * (S*scale - LSE)), 0 outside bounds / above the diagonal   (:224-227)
//   dS = p * (dP - D) * scale                 (:228)
//   dQ_i += dS K_j   (accumulated into global memory with atomics, :239-282)
//   dK_j += dS^T Q_i (:261-274)     dV_j += P^T dO_i (:285-299)
// plus the dropout keep-mask (p is multiplied by it), which the reference
// backward lacks but its forward implies.
//
// Blackwell structure (one CTA = one 128-row KV tile, 128-row query tiles):
// the transposed products S^T = K Q^T and dP^T = V dO^T put key rows on the 128
// tensor-memory lanes, so P^T and dS^T -- written back over S^T and dP^T by the
// compute warps -- are directly the tensor-memory A operands of dV += P^T dO and
// dK += dS^T Q.  dS is also staged once through shared memory (MN-major) as the
// A operand of dQ = dS K.  dV, dK (64 columns each) stay in tensor memory for
// the whole CTA; dQ (64 columns) is drained per query tile; V (64 columns) is
// copied into tensor memory once and is the A operand of dP^T, which frees its
// 32 KiB of shared memory for dS.  Everything the kernel writes leaves through
// shared memory and the TMA unit: dQ tiles are added to global memory with bulk
// reductions (per-thread atomics stall the tensor-core instruction issue of the
// same SM), dV and dK are stored with bulk copies at the end (a thread-per-row
// store touches 32 lines per instruction).
//
// Q, dO and K each feed one product that contracts over d (K-major operand,
// 16-byte-chunk swizzle) and one that contracts over the sequence (MN-major
// operand, which for TF32 must use the 32-byte-chunk swizzle; the tensor core
// refuses the 32-byte-chunk swizzle for a K-major operand), so TMA brings each
// of them into shared memory twice, once per swizzle.
//
// Tensor-pipe order per query tile i:
//     dV(i) | S^T(i+1) | dK(i) | dP^T(i+1) | dQ(i)
// dV(i) starts as soon as P^T(i) is in tensor memory, i.e. before the compute
// warps have formed dS(i); dK(i) follows when dS^T(i) is there, dQ(i) when dS(i)
// is staged in shared memory.
// S^T(i+1) only needs the P^T columns back, i.e. dV(i); issuing it before dK(i)
// lets the compute warps start the exponentials of tile i+1 -- the longest
// stretch of scalar work -- while dK(i), dP^T(i+1) and dQ(i) execute.  Two of the
// four 32-column boxes of dS(i) go over the MN-major dO tile as soon as dV(i) has
// consumed it; the other two have a buffer of their own, through which the
// drained dQ(i-1) first leaves by bulk reduction.  No staging touches the K-major
// Q and dO tiles, so their prefetch for tile i+1 starts as soon as S^T(i) and
// dP^T(i) are done.  Measured tensor-pipe time of the 72 instructions of a tile:
// about 3 050 cycles (M128 N128 K8: 74 cycles, M128 N64 K8: 36 from tensor
// memory, 52 from shared memory).
//
//   warps 0-15  compute: four threads per key row (tensor-memory lane), each
//               owning 32 of the 128 query columns, all held in registers so
//               that S^T and dP^T are read from tensor memory exactly once
//   warp 16     TMA loads (K, V once; Q and dO per query tile, each in two layouts)
//   warp 17     MMA issuer (the whole warp runs the issuing code, one elected lane
//               issues)
//   warp 18     TMA reductions of dQ (per query tile) and stores of dK, dV (at the end)
#include <mutex>

#include "attn_kernels.cuh"
#include "philox.h"

namespace hk {

namespace bwd {

constexpr int NUM_COMPUTE = 512;
constexpr int NUM_THREADS = NUM_COMPUTE + 96;  // 16 compute warps, 3 control warps
constexpr int W_LOAD = 16, W_MMA = 17, W_STORE = 18;
constexpr int TMEM_COLS = 512;
constexpr int COL_S = 0;     // S^T, then P^T
constexpr int COL_DP = 128;  // dP^T, then dS^T
constexpr int COL_DV = 256;
constexpr int COL_DK = 320;
constexpr int COL_DQ = 384;
constexpr int COL_V = 448;   // V of this KV tile, A operand of dP^T

struct __align__(16) Shared {
    float lse[2][TILE];   // -LSE * log2e of the query tile (-inf for rows past the end), double-buffered
    float dsum[2][TILE];  // -D * scale of the query tile
    uint64_t k_full, v_full, km_full, q_full, do_full, qm_full, dom_full;  // TMA loads
    uint64_t k_round, km_round;  // round_kv: the compute warps have rounded the K-major / MN-major K tile in place
    uint64_t v_ready;       // V is in tensor memory (and its landing buffer is free)
    uint64_t qk_free, dok_free;  // S^T(i) / dP^T(i) complete: the K-major Q / dO tile may be refilled
    uint64_t s_full, dp_full;
    // per column group (32 query columns = four K = 8 slices of dV and dK): the warps of a group arrive together, the
    // groups one after the other (the schedulers favour the older warps), and each group's slices go as soon as it is in
    uint64_t pt_ready[4];   // P^T of the group is in tensor memory: its slices of dV += P^T dO may go
    uint64_t p_ready[4];    // dS^T of the group is in tensor memory: its slices of dK += dS^T Q may go
    uint64_t dv_done, dk_done;   // dV(i) / dK(i) complete: the MN-major dO / Q tile is free
    uint64_t ds_ready, dq_full, dq_empty, staged;
    uint64_t acc_staged;    // dV, dK of the CTA are staged for the bulk store
    uint64_t dq_staged;     // dQ of a query tile is staged (in the K-major dO tile) for the bulk reduction
    uint64_t dq_out;        // the bulk reduction has read the staged dQ tile: the K-major dO tile may be refilled
    uint32_t tmem_base;
    int abort_flag;
};

constexpr int OFF_KK = 0;                // K, K-major swizzle   (S^T = K Q^T); dK staging at the end
constexpr int OFF_KM = TILE_BYTES;       // K, MN-major swizzle  (dQ = dS K)
constexpr int OFF_QK = 2 * TILE_BYTES;   // Q, K-major           (S^T); staging of the last dQ
constexpr int OFF_DOK = 3 * TILE_BYTES;  // dO, K-major          (dP^T)
constexpr int OFF_QM = 4 * TILE_BYTES;   // Q, MN-major          (dK += dS^T Q); dV staging at the end
constexpr int OFF_DS = 5 * TILE_BYTES;   // dS boxes 0, 1 ([128 kv][32 q] each); first of all the landing buffer of V
constexpr int OFF_DOM = 6 * TILE_BYTES;  // dO, MN-major         (dV += P^T dO); dS boxes 2, 3 once dV is done
static_assert(OFF_DOM == OFF_DS + 2 * BOX_BYTES, "the four dS boxes are one descriptor: equally spaced");
constexpr int OFF_SH = 7 * TILE_BYTES;
// no slack for re-aligning the dynamic shared-memory base: it is declared 1024-byte aligned
// and the kernel checks that it is (the 128-byte swizzles need it)
constexpr int SMEM_BYTES = OFF_SH + sizeof(Shared);
static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KiB a CTA may opt in to");

// Timeline slots (SM clock): role r in {0: MMA issuer, 1: compute thread 0}, iteration it, phase ph:
// buffer[1 + (it * 2 + r) * 8 + ph]; buffer[0] = number of iterations of the recorded CTA.
#ifdef HK_TIMELINE
// fixed-cost stamps of the recorded CTA: buffer[3900 + k]
#define HK_XSTAMP(on, k) do { if (on) a.timeline[3900 + (k)] = clock64(); } while (0)
__device__ __forceinline__ void stamp(const BwdArgs& a, bool on, int it, int role, int ph) {
    if (on && it < 80) a.timeline[1 + (it * 3 + role) * 16 + ph] = clock64();
}
#else
__device__ __forceinline__ void stamp(const BwdArgs&, bool, int, int, int) {}
#define HK_XSTAMP(on, k)
#endif

enum WaitId {
    W_KVFULL = 201, W_QKFULL, W_QKEMPTY, W_QMFULL, W_QMFREE, W_SFULL, W_PREADY, W_BDONE, W_DSREADY, W_DQFULL, W_DQEMPTY,
    W_STAGED, W_DQSTAGED, W_ACCSTAGED, W_VREADY, W_DVDONE, W_DQOUT
};

}  // namespace bwd

__global__ void __launch_bounds__(bwd::NUM_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapdO,
                const __grid_constant__ CUtensorMap mapQm, const __grid_constant__ CUtensorMap mapKm,
                const __grid_constant__ CUtensorMap mapdOm, const __grid_constant__ CUtensorMap mapdQ,
                const __grid_constant__ CUtensorMap mapdK, const __grid_constant__ CUtensorMap mapdV,
                const BwdArgs a) {
    using namespace bwd;
    extern __shared__ __align__(1024) uint8_t smem[];
    // schedule trace (timeline_block < 0): {start ns, end ns, SM id, query tiles} of each of the first 1024 CTAs
#ifdef HK_TIMELINE
    const bool trace = a.timeline != nullptr && a.timeline_block < 0 && blockIdx.x < 1024 && threadIdx.x == 0;
#else
    constexpr bool trace = false;
#endif
    if (trace) {
        a.timeline[4 * blockIdx.x] = (long long)globaltimer_ns();
        a.timeline[4 * blockIdx.x + 2] = clock64();
    }
#ifdef HK_TIMELINE
    const bool tlx = a.timeline != nullptr && (int)blockIdx.x == a.timeline_block && threadIdx.x == 0;
#else
    constexpr bool tlx = false;
#endif
    HK_XSTAMP(tlx, 0);
    if ((smem_u32(smem) & 1023u) != 0) {  // never expected; refuse to run on a misplaced buffer
        if (threadIdx.x == 0 && atomicCAS(&a.status->code, 0, 299) == 0) a.status->block = blockIdx.x;
        return;
    }
    uint8_t* sK = smem + OFF_KK;
    uint8_t* sKm = smem + OFF_KM;
    uint8_t* sV = smem + OFF_DS;  // landing buffer of V, read once into tensor memory
    uint8_t* sQ = smem + OFF_QK;
    uint8_t* sdO = smem + OFF_DOK;
    uint8_t* sQm = smem + OFF_QM;
    uint8_t* sdOm = smem + OFF_DOM;
    uint8_t* sdS = smem + OFF_DS;  // box b at sdS + b * BOX_BYTES
    Shared& sh = *reinterpret_cast<Shared*>(smem + OFF_SH);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // early KV tiles first: under the causal mask they see the most query tiles
    const int bh = blockIdx.x % a.BH;
    const int kt = (int)(blockIdx.x / a.BH);
    const int b = bh / a.H;
    const int h = bh - b * a.H;
    const int kv0 = kt * TILE;
    const int n_qtiles = (a.Tq + TILE - 1) / TILE;

    // first query tile with a row at or below the diagonal of this KV tile
    int it0 = 0;
    if (a.causal) {
        const long long first_q = (long long)kv0 + a.k_pos0 - a.q_pos0;  // smallest local q that sees key kv0
        if (first_q > 0) it0 = (int)min((long long)n_qtiles, first_q / TILE);
    }
    const int n_it = n_qtiles - it0;

    // The load warp initialises the barriers its copies complete on and issues the loads of the first tile at once:
    // the other warps meet those barriers only after the __syncthreads below, and ~1 000 cycles of set-up (the other
    // barriers, the tensor-memory allocation) run under the latency of the first loads instead of before it.
    if (warp == W_LOAD && lane == 0) {
        mbar_init(&sh.k_full, 1);
        mbar_init(&sh.v_full, 1);
        mbar_init(&sh.km_full, 1);
        mbar_init(&sh.q_full, 1);
        mbar_init(&sh.do_full, 1);
        mbar_init(&sh.qm_full, 1);
        mbar_init(&sh.dom_full, 1);
        fence_mbar_init();
        if (n_it > 0) {
            // in the order the first products need them: K, Q (S^T), V, dO (dP^T), MN-major dO (dV), Q (dK), K (dQ)
            const int q0 = it0 * TILE;
            mbar_arrive_expect_tx(&sh.k_full, TILE_BYTES);
            tma_load_4d(sK, &mapK, &sh.k_full, 0, kv0, h, b);
            tma_load_4d(sK + BOX_BYTES, &mapK, &sh.k_full, HALF_D, kv0, h, b);
            mbar_arrive_expect_tx(&sh.q_full, TILE_BYTES);
            tma_load_4d(sQ, &mapQ, &sh.q_full, 0, q0, h, b);
            tma_load_4d(sQ + BOX_BYTES, &mapQ, &sh.q_full, HALF_D, q0, h, b);
            mbar_arrive_expect_tx(&sh.v_full, TILE_BYTES);
            tma_load_4d(sV, &mapV, &sh.v_full, 0, kv0, h, b);
            tma_load_4d(sV + BOX_BYTES, &mapV, &sh.v_full, HALF_D, kv0, h, b);
            mbar_arrive_expect_tx(&sh.do_full, TILE_BYTES);
            tma_load_4d(sdO, &mapdO, &sh.do_full, 0, q0, h, b);
            tma_load_4d(sdO + BOX_BYTES, &mapdO, &sh.do_full, HALF_D, q0, h, b);
            mbar_arrive_expect_tx(&sh.dom_full, TILE_BYTES);
            tma_load_4d(sdOm, &mapdOm, &sh.dom_full, 0, q0, h, b);
            tma_load_4d(sdOm + BOX_BYTES, &mapdOm, &sh.dom_full, HALF_D, q0, h, b);
            mbar_arrive_expect_tx(&sh.qm_full, TILE_BYTES);
            tma_load_4d(sQm, &mapQm, &sh.qm_full, 0, q0, h, b);
            tma_load_4d(sQm + BOX_BYTES, &mapQm, &sh.qm_full, HALF_D, q0, h, b);
            mbar_arrive_expect_tx(&sh.km_full, TILE_BYTES);
            tma_load_4d(sKm, &mapKm, &sh.km_full, 0, kv0, h, b);
            tma_load_4d(sKm + BOX_BYTES, &mapKm, &sh.km_full, HALF_D, kv0, h, b);
        }
    }
    if (threadIdx.x == 0) {
        mbar_init(&sh.v_ready, NUM_COMPUTE);
        mbar_init(&sh.k_round, NUM_COMPUTE);
        mbar_init(&sh.km_round, NUM_COMPUTE);
        mbar_init(&sh.qk_free, 1);
        mbar_init(&sh.dok_free, 1);
        mbar_init(&sh.s_full, 1);
        mbar_init(&sh.dp_full, 1);
        for (int g = 0; g < 4; ++g) {
            mbar_init(&sh.pt_ready[g], TILE);
            mbar_init(&sh.p_ready[g], TILE);
        }
        mbar_init(&sh.dv_done, 1);
        mbar_init(&sh.dk_done, 1);
        mbar_init(&sh.ds_ready, NUM_COMPUTE);
        mbar_init(&sh.dq_full, 1);
        mbar_init(&sh.dq_empty, 256);   // column groups 2, 3 drain dQ
        mbar_init(&sh.dq_staged, 256);
        mbar_init(&sh.dq_out, 1);
        mbar_init(&sh.staged, 256);    // the threads that stage LSE and D
        mbar_init(&sh.acc_staged, NUM_COMPUTE);
        sh.abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == W_MMA) {
        tmem_alloc(&sh.tmem_base, TMEM_COLS);
        tmem_relinquish();
        tc_fence_before_sync();
    }
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sh.tmem_base;
    WaitCtx wc{&sh.abort_flag, a.status};
#ifdef HK_TIMELINE
    const bool tl = a.timeline != nullptr && (int)blockIdx.x == a.timeline_block;  // never in trace mode
#else
    constexpr bool tl = false;
#endif
    if (tl && threadIdx.x == 0) a.timeline[0] = n_it;
    HK_XSTAMP(tlx, 1);

    if (warp == W_LOAD) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0 && n_it > 0) {
            // the loads of the first tile were issued before the set-up barrier
            int issued_q = 1, issued_do = 1, issued_qm = 1, issued_dom = 1;
            auto load_q = [&](int q0) {
                mbar_arrive_expect_tx(&sh.q_full, TILE_BYTES);
                tma_load_4d(sQ, &mapQ, &sh.q_full, 0, q0, h, b);
                tma_load_4d(sQ + BOX_BYTES, &mapQ, &sh.q_full, HALF_D, q0, h, b);
                ++issued_q;
            };
            auto load_do = [&](int q0) {
                mbar_arrive_expect_tx(&sh.do_full, TILE_BYTES);
                tma_load_4d(sdO, &mapdO, &sh.do_full, 0, q0, h, b);
                tma_load_4d(sdO + BOX_BYTES, &mapdO, &sh.do_full, HALF_D, q0, h, b);
                ++issued_do;
            };
            auto load_qm = [&](int q0) {
                mbar_arrive_expect_tx(&sh.qm_full, TILE_BYTES);
                tma_load_4d(sQm, &mapQm, &sh.qm_full, 0, q0, h, b);
                tma_load_4d(sQm + BOX_BYTES, &mapQm, &sh.qm_full, HALF_D, q0, h, b);
                ++issued_qm;
            };
            auto load_dom = [&](int q0) {
                mbar_arrive_expect_tx(&sh.dom_full, TILE_BYTES);
                tma_load_4d(sdOm, &mapdOm, &sh.dom_full, 0, q0, h, b);
                tma_load_4d(sdOm + BOX_BYTES, &mapdOm, &sh.dom_full, HALF_D, q0, h, b);
                ++issued_dom;
            };
            bool tok = true;
            for (int it = 0; it + 1 < n_it; ++it) {
                const int q1 = (it0 + it + 1) * TILE;
                // K-major Q: free as soon as S^T(it) is done
                if (!(tok = mbar_wait(wc, &sh.qk_free, it & 1, W_QKEMPTY, it))) break;
                load_q(q1);
                // K-major dO: dQ(it-1) passes through the tile once dP^T(it) is done; free when the reduction has read it
                if (it == 0) {
                    if (!(tok = mbar_wait(wc, &sh.dok_free, 0, W_QKEMPTY, 1000))) break;
                } else if (!(tok = mbar_wait(wc, &sh.dq_out, (it - 1) & 1, W_DQOUT, it - 1))) break;
                load_do(q1);
                // MN-major Q: free once dK(it) is done
                if (!(tok = mbar_wait(wc, &sh.dk_done, it & 1, W_QMFREE, it))) break;
                load_qm(q1);
                // MN-major dO doubles as staging area of two dS boxes: free once dQ(it) is done
                if (!(tok = mbar_wait(wc, &sh.dq_full, it & 1, W_QMFREE, 1000 + it))) break;
                load_dom(q1);
            }
            // Do not leave the CTA while bulk copies into its shared memory are in flight.
            for (int i = 0; i < 100000 && !mbar_try_wait(&sh.k_full, 0); ++i) {}
            for (int i = 0; i < 100000 && !mbar_try_wait(&sh.v_full, 0); ++i) {}
            for (int i = 0; i < 100000 && !mbar_try_wait(&sh.km_full, 0); ++i) {}
            for (int i = 0; i < 100000 && !mbar_try_wait(&sh.q_full, (issued_q - 1) & 1); ++i) {}
            for (int i = 0; i < 100000 && !mbar_try_wait(&sh.do_full, (issued_do - 1) & 1); ++i) {}
            for (int i = 0; i < 100000 && !mbar_try_wait(&sh.qm_full, (issued_qm - 1) & 1); ++i) {}
            for (int i = 0; i < 100000 && !mbar_try_wait(&sh.dom_full, (issued_dom - 1) & 1); ++i) {}
        }
    } else if (warp == W_MMA) {
        // ------------------------------ MMA issuer ------------------------------
        // The whole warp runs this code with uniform control flow; only the tcgen05 instructions are predicated on
        // the elected lane (see umma_ss_tf32_lead).
        if (n_it > 0) {
            const uint32_t leader = elect_one_sync();
            auto wait = [&](uint64_t* bar, uint32_t parity, int id, int aux) -> bool {
                return __all_sync(0xffffffffu, mbar_wait(wc, bar, parity, id, aux));
            };
            const bool tlm = tl && leader;
            constexpr uint32_t IDESC_ST = make_idesc_tf32(TILE, TILE, false, false);     // K-major x K-major, N = 128
            constexpr uint32_t IDESC_TS = make_idesc_tf32(TILE, HEAD_DIM, false, true);  // tmem A, MN-major B, N = 64
            constexpr uint32_t IDESC_DQ = make_idesc_tf32(TILE, HEAD_DIM, true, true);   // MN-major A and B, N = 64
            const uint32_t k_addr = smem_u32(sK), q_addr = smem_u32(sQ), do_addr = smem_u32(sdO), qm_addr = smem_u32(sQm),
                           dom_addr = smem_u32(sdOm), km_addr = smem_u32(sKm), ds_addr = smem_u32(sdS);
            // S^T of query tile `it` (local index) as soon as K and Q have landed; the exponentials need nothing else
            auto issue_st = [&](int it) -> bool {
                if (it == 0 && !wait(a.round_kv ? &sh.k_round : &sh.k_full, 0, W_KVFULL, 0)) return false;
                if (!wait(&sh.q_full, it & 1, W_QKFULL, it)) return false;
                tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < HEAD_DIM / 8; ++kk)  // S^T = K Q^T
                    umma_ss_tf32_lead(leader, tmem + COL_S, kmajor_desc(k_addr, kk, BOX_BYTES), kmajor_desc(q_addr, kk, BOX_BYTES),
                                 IDESC_ST, kk > 0);
                umma_commit_lead(leader, &sh.s_full);
                umma_commit_lead(leader, &sh.qk_free);
                return true;
            };
            // dP^T = V dO^T, V from tensor memory
            auto issue_dp = [&](int it) -> bool {
                if (it == 0 && !wait(&sh.v_ready, 0, W_VREADY, 0)) return false;
                if (!wait(&sh.do_full, it & 1, W_QKFULL, 1000 + it)) return false;
                tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < HEAD_DIM / 8; ++kk)
                    umma_ts_tf32_lead(leader, tmem + COL_DP, tmem + COL_V + kk * 8, kmajor_desc(do_addr, kk, BOX_BYTES), IDESC_ST, kk > 0);
                umma_commit_lead(leader, &sh.dp_full);
                umma_commit_lead(leader, &sh.dok_free);
                return true;
            };
            bool ok = issue_st(0) && issue_dp(0);
            for (int it = 0; ok && it < n_it; ++it) {
                const uint32_t par = it & 1;
                stamp(a, tlm, it, 0, 0);
                if (!(ok = wait(&sh.dom_full, par, W_QMFULL, it))) break;
                stamp(a, tlm, it, 0, 1);
                for (int g = 0; ok && g < 4; ++g) {  // dV += P^T dO, group by group
                    if (!(ok = wait(&sh.pt_ready[g], par, W_PREADY, 4 * it + g))) break;
                    tc_fence_after_sync();
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4) {
                        const int kk = 4 * g + k4;
                        umma_ts_tf32_lead(leader, tmem + COL_DV, tmem + COL_S + kk * 8, mnmajor_desc(dom_addr, kk, BOX_BYTES),
                                          IDESC_TS, (it > 0 || kk > 0) ? 1u : 0u);
                    }
                }
                if (!ok) break;
                umma_commit_lead(leader, &sh.dv_done);  // MN-major dO consumed: two of the dS boxes may be staged over it
                stamp(a, tlm, it, 0, 2);
                // next tile's S^T: P^T of this tile was consumed by the MMAs just issued
                if (it + 1 < n_it && !(ok = issue_st(it + 1))) break;
                stamp(a, tlm, it, 0, 3);
                if (!(ok = wait(&sh.qm_full, par, W_QMFULL, 1000 + it))) break;
                for (int g = 0; ok && g < 4; ++g) {  // dK += dS^T Q, group by group
                    if (!(ok = wait(&sh.p_ready[g], par, W_PREADY, 1000 + 4 * it + g))) break;
                    tc_fence_after_sync();
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4) {
                        const int kk = 4 * g + k4;
                        umma_ts_tf32_lead(leader, tmem + COL_DK, tmem + COL_DP + kk * 8, mnmajor_desc(qm_addr, kk, BOX_BYTES),
                                          IDESC_TS, (it > 0 || kk > 0) ? 1u : 0u);
                    }
                }
                if (!ok) break;
                umma_commit_lead(leader, &sh.dk_done);  // MN-major Q consumed
                // next tile's dP^T: dS^T of this tile was consumed by the MMAs just issued
                if (it + 1 < n_it && !(ok = issue_dp(it + 1))) break;
                stamp(a, tlm, it, 0, 4);
                // dQ = dS K once dS is staged (shortly after dS^T was stored) and the previous dQ has left tensor memory
                if (!(ok = wait(&sh.ds_ready, par, W_DSREADY, it))) break;
                if (it > 0 && !(ok = wait(&sh.dq_empty, (it - 1) & 1, W_DQEMPTY, it))) break;
                if (it == 0 && !(ok = wait(a.round_kv ? &sh.km_round : &sh.km_full, 0, W_KVFULL, 2))) break;
                stamp(a, tlm, it, 0, 5);
                tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < TILE / 8; ++kk)
                    umma_ss_tf32_lead(leader, tmem + COL_DQ, mnmajor_desc(ds_addr, kk, BOX_BYTES),
                                      mnmajor_desc(km_addr, kk, BOX_BYTES), IDESC_DQ, kk > 0);
                umma_commit_lead(leader, &sh.dq_full);  // also: the dS staging area is free again
                stamp(a, tlm, it, 0, 6);
                stamp(a, tlm, it, 0, 7);
            }
        }
    } else if (warp == W_STORE) {
#ifdef HK_TIMELINE
        // completion monitor (development builds): when each product of a tile is done
        if (lane == 1 && tl) {
            bool mok = true;
            for (int it = 0; mok && it < n_it; ++it) {
                if ((mok = mbar_wait(wc, &sh.dv_done, it & 1, 990, it))) stamp(a, true, it, 2, 0);
                if (mok && it + 1 < n_it && (mok = mbar_wait(wc, &sh.s_full, (it + 1) & 1, 991, it))) stamp(a, true, it, 2, 1);
                if (mok && (mok = mbar_wait(wc, &sh.dk_done, it & 1, 992, it))) stamp(a, true, it, 2, 2);
                if (mok && it + 1 < n_it && (mok = mbar_wait(wc, &sh.dp_full, (it + 1) & 1, 993, it))) stamp(a, true, it, 2, 3);
                if (mok && (mok = mbar_wait(wc, &sh.dq_full, it & 1, 994, it))) stamp(a, true, it, 2, 4);
            }
        }
#endif
        // ------------------------------ store warp ------------------------------
        // Everything that leaves the CTA: the staged dQ tiles (bulk reductions) and, at the end, dV and dK (bulk
        // stores).  A thread of its own, so that a reduction is issued the moment its tile is staged.
        if (lane == 0 && n_it > 0) {
            tma_prefetch_desc(&mapdK);
            tma_prefetch_desc(&mapdV);
            tma_prefetch_desc(&mapdQ);
            // dQ of query tile j, staged in the K-major dO tile: add it to global memory; once the reduction has read
            // the tile, hand it back to the load warp
            auto reduce_dq = [&](int j) -> bool {
                if (!mbar_wait(wc, &sh.dq_staged, j & 1, W_DQSTAGED, j)) return false;
                const int q = (it0 + j) * TILE;
                if (a.det_dq) {  // this KV tile's slab of partial dQ; reduce_dq_slabs adds the slabs in a fixed order
                    tma_store_4d(&mapdQ, sdO, 0, q, h, kt * a.B + b);
                    tma_store_4d(&mapdQ, sdO + BOX_BYTES, HALF_D, q, h, kt * a.B + b);
                } else {
                    tma_reduce_add_4d(&mapdQ, sdO, 0, q, h, b);
                    tma_reduce_add_4d(&mapdQ, sdO + BOX_BYTES, HALF_D, q, h, b);
                }
                bulk_commit_group();
                bulk_wait_group_read_all();
                mbar_arrive(&sh.dq_out);
                return true;
            };
            bool tok = true;
            for (int j = 0; tok && j + 1 < n_it; ++j) tok = reduce_dq(j);  // the last tile's dQ follows dV and dK
            // dV and dK, staged by the compute warps in the MN-major Q tile and the K-major K tile (dead after the last
            // dK and S^T): stored -- added, if the caller accumulates -- with bulk copies; a thread-per-row store would
            // be 32 lines per instruction
            if (tok && (tok = mbar_wait(wc, &sh.acc_staged, 0, W_ACCSTAGED, 0))) {
                if (a.accum_dkdv) {
                    tma_reduce_add_4d(&mapdV, sQm, 0, kv0, h, b);
                    tma_reduce_add_4d(&mapdV, sQm + BOX_BYTES, HALF_D, kv0, h, b);
                    tma_reduce_add_4d(&mapdK, sK, 0, kv0, h, b);
                    tma_reduce_add_4d(&mapdK, sK + BOX_BYTES, HALF_D, kv0, h, b);
                } else {
                    tma_store_4d(&mapdV, sQm, 0, kv0, h, b);
                    tma_store_4d(&mapdV, sQm + BOX_BYTES, HALF_D, kv0, h, b);
                    tma_store_4d(&mapdK, sK, 0, kv0, h, b);
                    tma_store_4d(&mapdK, sK + BOX_BYTES, HALF_D, kv0, h, b);
                }
                bulk_commit_group();
                tok = reduce_dq(n_it - 1);
            }
            // the copies have read their shared-memory sources; they complete on their own
            bulk_wait_group_read_all();
            HK_XSTAMP(tl, 8);
        }
    } else {
        // ------------------------------ compute ------------------------------
        const int quarter = warp & 3;
        const int part = warp >> 2;             // which 32 of the 128 query columns this thread owns
        const int row = quarter * 32 + lane;    // key row inside the tile = tensor-memory lane
        const int tid = threadIdx.x;            // 0..511: the compute warps come first
        const int c0 = part * 32;
        const int kvrow = kv0 + row;
        const bool kv_ok = kvrow < a.Tk;
        const uint32_t trow = tmem + ((uint32_t)(quarter * 32) << 16);
        const float* lse_bh = a.LSE + (int64_t)b * a.lse_sB + (int64_t)h * a.lse_sH;
        const float* d_bh = a.D + (int64_t)b * a.d_sB + (int64_t)h * a.d_sH;
        bool ok = true;
        uint32_t rs[32], rp[32];
#ifndef HK_TL_TID
#define HK_TL_TID 0  // compute thread whose phases a -DHK_TIMELINE build records
#endif
        const bool tlc = tl && tid == HK_TL_TID;
        // -LSE * log2e (threads 0..127; -inf past the end and for a fully dropped row, so that every p is 0) or
        // -D * scale (threads 128..255) of query row q0 + (tid & 127): negated, so that both enter as FMA addends
        auto fetch_lse_or_d = [&](int q0) -> float {
            const int q = q0 + (tid & 127);
            if (tid < TILE) {
                if (q >= a.Tq) return -INFINITY;
                const float l = __ldg(lse_bh + q);
                return (l == -INFINITY) ? -INFINITY : -l * LOG2E;
            }
            return (q < a.Tq) ? -__ldg(d_bh + q) * a.scale : 0.f;
        };
        float staged_val = (tid < 2 * TILE && n_it > 0) ? fetch_lse_or_d(it0 * TILE) : 0.f;

        // dQ of query tile j out of tensor memory into the K-major dO tile (column groups 2 and 3 only: this thread's
        // query row `row`, 32 columns), in the layout of a 128-byte-swizzled TMA box: 16-byte chunk c of row r at
        // position c ^ (r & 7).  Called between the two halves of the NEXT tile's compute, when dP^T of that tile is
        // done: its operand, the K-major dO tile, is then dead until the tile after it is prefetched, long enough for
        // the bulk reduction, which keeps its source for ~1 600 cycles.  Groups 2, 3 run behind groups 0, 1 (the
        // schedulers favour the older warps), late enough for dQ(j) to be complete when they get here.
        auto drain_dq = [&](int j, uint32_t (&v)[32]) -> bool {
            if (!__all_sync(0xffffffffu, mbar_wait(wc, &sh.dq_full, j & 1, W_DQFULL, j))) return false;
            tc_fence_after_sync();
            tmem_ld32(trow + COL_DQ + 32 * (part & 1), v);
            tmem_wait_ld();
            tc_fence_before_sync();
            mbar_arrive(&sh.dq_empty);  // dQ is in registers: the next dQ = dS K may overwrite tensor memory
            uint8_t* srow = sdO + (part & 1) * BOX_BYTES + row * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<uint4*>(srow + ((c ^ (row & 7)) << 4)) =
                    make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
            fence_proxy_async_smem();
            mbar_arrive(&sh.dq_staged);
            return true;
        };

        // V of this KV tile into tensor memory (A operand of dP^T = V dO^T): this thread's key row, 16 of the 64
        // columns, read from the 128-byte-swizzled landing buffer (16-byte chunk c of row r at position c ^ (r & 7))
        // round_kv (short sequences, decided by the host): K and V come straight from the caller's tensors and are
        // rounded to TF32 by the compute warps, once per CTA -- the K-major K tile first (S^T of the first tile waits for
        // it), V on its way into tensor memory, the MN-major K tile inside the first tile (the first dQ needs it).  Same function as the HBM
        // pre-pass, so the results are bit-identical to that path.
        auto round_k_tile = [&](uint8_t* tile) {
            uint4* p4 = reinterpret_cast<uint4*>(tile);
#pragma unroll
            for (int k = 0; k < TILE_BYTES / 16 / NUM_COMPUTE; ++k) {
                uint4 x = p4[tid + k * NUM_COMPUTE];
                x.x = tf32_round_bits(x.x); x.y = tf32_round_bits(x.y);
                x.z = tf32_round_bits(x.z); x.w = tf32_round_bits(x.w);
                p4[tid + k * NUM_COMPUTE] = x;
            }
            fence_proxy_async_smem();
        };
        if (n_it > 0) {
            if (a.round_kv) {
                ok = __all_sync(0xffffffffu, mbar_wait(wc, &sh.k_full, 0, W_KVFULL, 4));
                if (ok) {
                    round_k_tile(sK);
                    mbar_arrive(&sh.k_round);
                }
            }
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(wc, &sh.v_full, 0, W_KVFULL, 3));
            HK_XSTAMP(tlx, 2);
            if (ok) {
                uint32_t rv[16];
                const uint8_t* vrow = sV + (part >> 1) * BOX_BYTES + row * 128;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint4 x = *reinterpret_cast<const uint4*>(vrow + (((4 * (part & 1) + c) ^ (row & 7)) << 4));
                    rv[4 * c] = x.x; rv[4 * c + 1] = x.y; rv[4 * c + 2] = x.z; rv[4 * c + 3] = x.w;
                }
                if (a.round_kv) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) rv[i] = tf32_round_bits(rv[i]);
                }
                tmem_st16(trow + COL_V + 16 * part, rv);
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&sh.v_ready);
            }
            HK_XSTAMP(tlx, 3);
        }

        for (int it = 0; ok && it < n_it; ++it) {
            const int q0 = (it0 + it) * TILE;
            stamp(a, tlc, it, 1, 0);
            // stage LSE (threads 0..127) and D (threads 128..255) of this query tile into buffer it & 1.
            // The buffer was last read two tiles ago; every compute thread passed that tile's ds_ready
            // arrival long before this thread could get here (it has since waited on dq_full or s_full
            // of the previous tile, which follow it).
            // The value was fetched from global memory one tile ahead, so that its latency is not paid here.
            if (tid < 2 * TILE) {
                if (tid < TILE)
                    sh.lse[it & 1][tid] = staged_val;
                else
                    sh.dsum[it & 1][tid - TILE] = staged_val;
                mbar_arrive(&sh.staged);
                if (it + 1 < n_it) staged_val = fetch_lse_or_d(q0 + TILE);
            }
            // an mbarrier rather than bar.sync: its wait is bounded, so a CTA that is
            // winding down after a failed wait cannot strand warps at a barrier
            ok = __all_sync(0xffffffffu, mbar_wait(wc, &sh.staged, it & 1, W_STAGED, it));
            if (!ok) break;
            stamp(a, tlc, it, 1, 1);
            ok = __all_sync(0xffffffffu, mbar_wait(wc, &sh.s_full, it & 1, W_SFULL, it));
            if (!ok) break;
            stamp(a, tlc, it, 1, 2);
            tc_fence_after_sync();

            tmem_ld32(trow + COL_S + c0, rs);
            stamp(a, tlc, it, 1, 8);

            // first query column (local to the tile) this key row is visible to
            int cmin = 0;
            if (a.causal) {
                const long long c = (long long)a.k_pos0 + kvrow - a.q_pos0 - q0;
                cmin = (int)max(0ll, min((long long)TILE, c));
            }
            if (!kv_ok) cmin = TILE;

            // dropout keep bits of this thread's 32 (query, key) pairs
            uint32_t keep = 0xffffffffu;
            if (a.dropout_mode == 2) {
                // One Philox call covers the eight keys kpos & ~7 .. of one query row, i.e. the key rows of eight
                // adjacent lanes (k_pos0 and kv0 are multiples of 8, so row & 7 == lane & 7).  Lane j of such a
                // group evaluates the query columns 8m + j (m = 0..3) and keeps 8 bits per call; the group then
                // swaps them with shuffles, so every lane does 4 calls for its 32 columns instead of 32.
                const int j8 = lane & 7;
                const uint32_t kgrp = (uint32_t)(a.k_pos0 + kvrow) >> 3;
                uint32_t mine = 0u;  // bit 8m + u: query column c0 + 8m + j8, key row (row & ~7) + u
#pragma unroll
                for (int mI = 0; mI < 4; ++mI) {
                    const hk_philox4_t w = hk_philox_row8(a.seed, a.offset, a.bh_pos0 + (uint32_t)bh,
                                                          (uint32_t)(a.q_pos0 + q0 + c0 + 8 * mI + j8), kgrp);
                    mine |= hk_philox_keep8(w, a.drop_thr) << (8 * mI);
                }
                keep = 0u;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t other = __shfl_sync(0xffffffffu, mine, (lane & ~7) | j);  // lane j's columns 8m + j
                    keep |= ((other >> j8) & 0x01010101u) << j;                              // its bit for MY key row
                }
            } else if (a.dropout_mode == 1) {
                keep = 0u;
                if (kv_ok) {
#pragma unroll 4
                    for (int i = 0; i < 32; ++i) {
                        const int q = q0 + c0 + i;
                        if (q < a.Tq && __ldg(a.mask + ((size_t)bh * a.Tq + q) * (size_t)a.Tk + kvrow) != 0.f)
                            keep |= 1u << i;
                    }
                }
            }
            // fold the causal / tail mask into the keep bits: column cc is visible iff cc >= cmin
            uint32_t vis = 0xffffffffu;
            {
                const int lo = cmin - c0;  // first visible local index, may be <= 0 or >= 32
                if (lo > 0) vis = (lo >= 32) ? 0u : (0xffffffffu << lo);
                keep &= vis;
            }
            // pairs whose p is zero: hidden ones, and dropped ones unless the dropout is the inverted kind
            const uint32_t live = a.drop_scaled ? vis : keep;
            tmem_wait_ld();
            stamp(a, tlc, it, 1, 9);

            // p = exp2(s*scale*log2e - LSE*log2e) needs S^T only: dP^T is still being computed.  Two scores per
            // packed FMA (fma.rn.f32x2 gives the same bits as two scalar FMAs).
            {
                const float4* lse4 = reinterpret_cast<const float4*>(sh.lse[it & 1] + c0);
                const float2 c2 = make_float2(a.scale_log2e, a.scale_log2e);
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    const float4 L = lse4[g];
                    const float2 x01 = __ffma2_rn(make_float2(__uint_as_float(rs[4 * g]), __uint_as_float(rs[4 * g + 1])), c2,
                                                  make_float2(L.x, L.y));
                    const float2 x23 = __ffma2_rn(make_float2(__uint_as_float(rs[4 * g + 2]), __uint_as_float(rs[4 * g + 3])), c2,
                                                  make_float2(L.z, L.w));
                    rs[4 * g] = __float_as_uint(ex2_approx(x01.x));
                    rs[4 * g + 1] = __float_as_uint(ex2_approx(x01.y));
                    rs[4 * g + 2] = __float_as_uint(ex2_approx(x23.x));
                    rs[4 * g + 3] = __float_as_uint(ex2_approx(x23.y));
                }
                if (live != 0xffffffffu) {  // tiles on the diagonal, the ragged end, dropout
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (!((live >> i) & 1u)) rs[i] = 0u;
                }
            }
            stamp(a, tlc, it, 1, 10);
            // P^T goes to tensor memory at once (rounded; a pair dropped by inverted dropout counts as zero in dV but
            // keeps its p for dS below): dV += P^T dO and, behind it, the next tile's S^T run while dS is computed,
            // and the store has drained by the time its first reader starts.  rp is free until dP^T is loaded.
            {
                const bool dropped_some = a.drop_scaled && keep != 0xffffffffu;
#pragma unroll
                for (int i = 0; i < 32; ++i) rp[i] = tf32_round_bits_mma(rs[i]);
                if (dropped_some) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (!((keep >> i) & 1u)) rp[i] = 0u;
                }
                tmem_st32(trow + COL_S + c0, rp);
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&sh.pt_ready[part]);
            }
            if (it == 0 && a.round_kv) {
                // the MN-major K tile (last of the first loads, first read by dQ of this tile): rounded here, where
                // the warps would otherwise wait for dP^T
                ok = __all_sync(0xffffffffu, mbar_wait(wc, &sh.km_full, 0, W_KVFULL, 5));
                if (!ok) break;
                round_k_tile(sKm);
                mbar_arrive(&sh.km_round);
            }
            ok = __all_sync(0xffffffffu, mbar_wait(wc, &sh.dp_full, it & 1, W_SFULL, 1000 + it));
            if (!ok) break;
            stamp(a, tlc, it, 1, 11);
            tc_fence_after_sync();
            if (it > 0 && part >= 2 && !(ok = drain_dq(it - 1, rp))) break;  // rp is free until dP^T is loaded
            tmem_ld32(trow + COL_DP + c0, rp);
            tmem_wait_ld();
            stamp(a, tlc, it, 1, 3);

            // dS = p * (dP*scale - D*scale), two elements per packed instruction
            {
                const float4* ds4 = reinterpret_cast<const float4*>(sh.dsum[it & 1] + c0);
                const bool dropped_some = a.drop_scaled && keep != 0xffffffffu;
                if (dropped_some) {
                    // inverted dropout: a dropped pair keeps the -D term of dS but contributes neither dP (zeroed
                    // here) nor to dV (its P^T entry was stored as zero above)
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (!((keep >> i) & 1u)) rp[i] = 0u;
                }
                const float2 dps2 = make_float2(a.dp_scale, a.dp_scale);
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    const float4 Dv = ds4[g];  // -D * scale
#pragma unroll
                    for (int h2 = 0; h2 < 2; ++h2) {
                        const int i = 4 * g + 2 * h2;
                        const float2 nd = h2 ? make_float2(Dv.z, Dv.w) : make_float2(Dv.x, Dv.y);
                        const float2 t = __ffma2_rn(make_float2(__uint_as_float(rp[i]), __uint_as_float(rp[i + 1])), dps2, nd);
                        const float2 ds = __fmul2_rn(make_float2(__uint_as_float(rs[i]), __uint_as_float(rs[i + 1])), t);
                        rp[i] = tf32_round_bits_mma(__float_as_uint(ds.x));
                        rp[i + 1] = tf32_round_bits_mma(__float_as_uint(ds.y));
                    }
                }
            }
            stamp(a, tlc, it, 1, 4);
            tmem_st32(trow + COL_DP + c0, rp);
            stamp(a, tlc, it, 1, 12);
            tmem_wait_st();
            stamp(a, tlc, it, 1, 13);
            tc_fence_before_sync();
            mbar_arrive(&sh.p_ready[part]);  // this group's slices of dK += dS^T Q may go
            stamp(a, tlc, it, 1, 5);

            // dS into shared memory, the MN-major A operand of dQ = dS K: box `part` holds query columns
            // 32*part..32*part+31, one 128-byte row per key row, 32-byte chunks XOR-swizzled with (row & 3).  Boxes 0, 1
            // -- the groups that get here first -- have a buffer of their own, free once dQ of the previous tile is done
            // (before the first tile the buffer held V, which every thread has left once v_ready completes); boxes 2, 3 go over the MN-major dO tile as soon as dV of
            // this tile is done.
            if (part < 2) {
                ok = __all_sync(0xffffffffu, it == 0 ? mbar_wait(wc, &sh.v_ready, 0, W_VREADY, 1)
                                                      : mbar_wait(wc, &sh.dq_full, (it - 1) & 1, W_DQFULL, 1000 + it));
            } else {
                ok = __all_sync(0xffffffffu, mbar_wait(wc, &sh.dv_done, it & 1, W_DVDONE, it));
            }
            if (!ok) break;
            stamp(a, tlc, it, 1, 6);
            {
                // Rows r and r + 4 share a 32-byte chunk position; they store its two halves in opposite order so
                // that the eight lanes of a quarter-warp hit eight different 16-byte bank groups.
                uint8_t* drow = sdS + part * BOX_BYTES + row * 128;
                const bool swap = (row >> 2) & 1;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint4 lo = make_uint4(rp[8 * u], rp[8 * u + 1], rp[8 * u + 2], rp[8 * u + 3]);
                    const uint4 hi = make_uint4(rp[8 * u + 4], rp[8 * u + 5], rp[8 * u + 6], rp[8 * u + 7]);
                    uint8_t* chunk = drow + ((u ^ (row & 3)) << 5);
                    *reinterpret_cast<uint4*>(chunk + (swap ? 16 : 0)) = swap ? hi : lo;
                    *reinterpret_cast<uint4*>(chunk + (swap ? 0 : 16)) = swap ? lo : hi;
                }
            }
            fence_proxy_async_smem();
            mbar_arrive(&sh.ds_ready);
            stamp(a, tlc, it, 1, 7);
        }

        // dV and dK of this KV tile are complete once dK of the last query tile is (dV precedes it on the tensor
        // pipe).  Column groups 0,1 put dV (times 1/(1-p) for inverted dropout) into the MN-major Q tile and groups
        // 2,3 dK into the K-major K tile, both dead by then, as the boxes of a 128-byte-swizzled TMA tile: 16-byte
        // chunk c of row r at position c ^ (r & 7).
        HK_XSTAMP(tlx, 4);
        if (ok && n_it > 0) ok = __all_sync(0xffffffffu, mbar_wait(wc, &sh.dk_done, (n_it - 1) & 1, W_BDONE, n_it));
        HK_XSTAMP(tlx, 5);
        if (ok && n_it > 0) {
            tc_fence_after_sync();
            tmem_ld32(trow + ((part < 2) ? COL_DV + part * 32 : COL_DK + (part - 2) * 32), rs);
            tmem_wait_ld();
            const float f = (part < 2) ? a.dv_scale : 1.f;
            uint8_t* srow = ((part < 2) ? sQm : sK) + (part & 1) * BOX_BYTES + row * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<float4*>(srow + ((c ^ (row & 7)) << 4)) =
                    make_float4(__uint_as_float(rs[4 * c]) * f, __uint_as_float(rs[4 * c + 1]) * f,
                                __uint_as_float(rs[4 * c + 2]) * f, __uint_as_float(rs[4 * c + 3]) * f);
            fence_proxy_async_smem();
            mbar_arrive(&sh.acc_staged);
            HK_XSTAMP(tlx, 6);
        } else if (n_it == 0 && kv_ok && !a.accum_dkdv) {
            // no query sees this KV tile: its dK and dV rows are zero
            float* out_row = (part < 2)
                                 ? a.dV + (int64_t)b * a.dv_sB + (int64_t)h * a.dv_sH + (int64_t)kvrow * a.dv_sM + part * 32
                                 : a.dK + (int64_t)b * a.dk_sB + (int64_t)h * a.dk_sH + (int64_t)kvrow * a.dk_sM + (part - 2) * 32;
#pragma unroll
            for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(out_row + i) = make_float4(0.f, 0.f, 0.f, 0.f);
        }

        // dQ of the last query tile takes the same way out as the others: staged in the K-major dO tile (dead: its
        // last reader was dP^T of this tile) once the reduction of the previous tile has read that buffer, then
        // added to global memory by the store warp.  (From registers with red.global.add it took ~2 500 cycles per
        // CTA and held up the bulk stores of dV and dK behind it.)
        if (ok && n_it > 0 && part >= 2) {
            if (n_it > 1) ok = __all_sync(0xffffffffu, mbar_wait(wc, &sh.dq_out, (n_it - 2) & 1, W_DQOUT, n_it - 2));
            if (ok) ok = drain_dq(n_it - 1, rs);
            HK_XSTAMP(tl && tid == 256, 9);
        }

    }

    // ------------------------------ teardown ------------------------------
    tc_fence_before_sync();
    __syncthreads();
    HK_XSTAMP(tlx, 7);
    if (warp == W_MMA) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem, TMEM_COLS);
    }
    if (trace) {
        a.timeline[4 * blockIdx.x + 1] = (long long)globaltimer_ns();
        a.timeline[4 * blockIdx.x + 2] = smid() | ((clock64() - a.timeline[4 * blockIdx.x + 2]) << 10);  // SM id, SM cycles
        a.timeline[4 * blockIdx.x + 3] = n_it;
    }
}

int launch_attn_bwd(const BwdMaps& m, const BwdArgs& a, cudaStream_t stream) {
    // the opt-in to large dynamic shared memory is per device: once per device, safe from any number of host threads
    static std::once_flag attr_once[HK_MAX_DEVICES];
    static cudaError_t attr_rc[HK_MAX_DEVICES];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return HK_ERR_CUDA;
    if (dev < 0 || dev >= HK_MAX_DEVICES) return HK_ERR_UNSUPPORTED;
    std::call_once(attr_once[dev], [dev] {
        attr_rc[dev] = cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bwd::SMEM_BYTES);
    });
    if (attr_rc[dev] != cudaSuccess) return HK_ERR_CUDA;
    const long long nblocks = (long long)a.n_kvtiles * a.BH;
    if (nblocks <= 0 || nblocks > 0x7fffffffLL) return HK_ERR_BAD_SHAPE;
    timing_mark(TIMED_BWD, true, stream);
    attn_bwd_kernel<<<(unsigned)nblocks, bwd::NUM_THREADS, bwd::SMEM_BYTES, stream>>>(m.q, m.k, m.v, m.dO, m.q_mn, m.k_mn,
                                                                                       m.dO_mn, m.dQ, m.dK, m.dV, a);
    timing_mark(TIMED_BWD, false, stream);
    count_launch();
    return check_launch();
}

}  // namespace hk
