// attn_kernels.cuh -- argument blocks and launchers of the two tensor-core kernels.
#pragma once
#include "attn_common.cuh"

namespace hk {

struct FwdArgs {
    float* O;
    float* LSE;
    const float* mask;  // dense dropout mask [BH, Tq, Tk] or nullptr
    int64_t o_sB, o_sM, o_sH, lse_sB, lse_sH;
    int H, BH;
    int Tq, Tk;
    int n_qtiles;
    int q_pos0, k_pos0;
    float scale_log2e;
    int causal;
    int dropout_mode;  // 0 none, 1 dense mask, 2 Philox
    int drop_scaled;   // 1: inverted dropout (normaliser over all visible keys, kept terms times keep_scale)
    int continue_state;  // 1: O, LSE hold the result over earlier keys and are the starting state
    int round_in_smem;   // 1: Q, K, V arrive unrounded and are rounded to TF32 in shared memory after the TMA landing
    int store_q;         // with round_in_smem: the rounded Q, K and V tiles are also written out (maps mqw, mkw, mvw), where
                         // the HBM pre-pass would have put them, for a backward call that reuses them
    float keep_scale;  // 1/(1-p) when drop_scaled, else 1
    uint32_t drop_thr;
    uint32_t bh_pos0;  // added to the local (batch, head) index in the Philox counter
    uint64_t seed, offset;
    DeviceStatus* status;
    long long* timeline;  // per-phase SM clock stamps of one CTA; only builds with -DHK_TIMELINE read it
    int timeline_block;
};

// mq, mk, mv: TMA maps of the (rounded) operands; mo: map of O, the destination of the kernel's bulk stores.
int launch_attn_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo,
                    const CUtensorMap& mqw, const CUtensorMap& mkw, const CUtensorMap& mvw,
                    const FwdArgs& a, cudaStream_t stream);

struct BwdArgs {
    const float* LSE;
    const float* D;
    float* dQ;
    float* dK;
    float* dV;
    const float* mask;
    int64_t lse_sB, lse_sH, d_sB, d_sH;
    int64_t dq_sB, dq_sM, dq_sH, dk_sB, dk_sM, dk_sH, dv_sB, dv_sM, dv_sH;
    int H, BH;
    int Tq, Tk;
    int n_kvtiles;
    int q_pos0, k_pos0;
    float scale, scale_log2e;
    int causal;
    int accum_dkdv;
    int round_kv;      // 1: K and V arrive unrounded; the compute warps round them to TF32 once they have landed
    int det_dq;        // 1: dQ tiles are stored (map dQ = the slabs [n_kvtiles * B, H, Tq, 64]) instead of added; B below
    int B;
    int dropout_mode;
    int drop_scaled;   // 1: inverted dropout; p below is then the softmax over all visible keys
    float dp_scale;    // factor of dP inside dS: scale, times 1/(1-p) when drop_scaled
    float dv_scale;    // factor of the dV accumulator: 1/(1-p) when drop_scaled, else 1
    uint32_t drop_thr;
    uint32_t bh_pos0;  // added to the local (batch, head) index in the Philox counter
    uint64_t seed, offset;
    DeviceStatus* status;
    long long* timeline;  // per-phase SM clock stamps of one CTA; only builds with -DHK_TIMELINE read it
    int timeline_block;
};

// K-major maps (16-byte-chunk swizzle) of Q, K, V, dO and MN-major maps
// (32-byte-chunk swizzle) of Q, K, dO over the same memory; dQ, dK, dV are
// the destinations of the kernel's bulk reductions and stores (16-byte-chunk
// swizzle).
struct BwdMaps {
    CUtensorMap q, k, v, dO, q_mn, k_mn, dO_mn, dQ, dK, dV;
};

int launch_attn_bwd(const BwdMaps& m, const BwdArgs& a, cudaStream_t stream);

int run_umma_selftest(int which, const float* A, const float* B, float* out, cudaStream_t stream);

}  // namespace hk
