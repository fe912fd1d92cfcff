// attn_prepass.cuh -- launchers of the HBM-bound helper kernels (attn_prepass.cu).
#pragma once
#include "attn_common.cuh"

namespace hk {

struct RoundJob {
    View4 src[4];
    float* dst[4];  // contiguous [BH, T[t], 64]
    int T[4];
    int H, BH;
    int n;
};
int launch_round_tf32(const RoundJob& job, cudaStream_t stream);

struct DJob {
    View4 dO, O;
    float* D;
    int64_t d_sB, d_sH;
    float* dO_rounded;  // contiguous [BH, T, 64] or nullptr
    float* dQ_zero;     // if set: the same rows of dQ are zeroed on the way (dQ is accumulated with atomics)
    int64_t dq_sB, dq_sM, dq_sH;
    int H, BH, T;
};
int launch_precompute_D(const DJob& j, cudaStream_t stream);
// D only, head dimension 16, 32, 48, 64, 80, 96, 128, 160, 192 or 256 (dO_rounded and dQ_zero are ignored)
int launch_precompute_D_hd(const DJob& j, int head_dim, cudaStream_t stream);

int launch_zero_rows(float* ptr, int64_t sB, int64_t sM, int64_t sH, int B, int H, int T, cudaStream_t stream);

// Deterministic dQ: dQ (+)= sum over KV tiles kt, in increasing kt, of slab[kt][b][h][t][:], skipping the (kt, query
// tile) pairs the backward kernel never visits (causal mask: query tiles above the diagonal of the KV tile).
struct DqReduceJob {
    const float* slabs;  // [n_kvtiles][B][H][T][64] contiguous
    float* dQ;
    int64_t dq_sB, dq_sM, dq_sH;
    int B, H, T, n_kvtiles;
    int causal, q_pos0, k_pos0;
    int accumulate;  // 1: add to what dQ holds (HK_FLAG_ACCUM_DQ)
};
int launch_reduce_dq_slabs(const DqReduceJob& j, cudaStream_t stream);

int launch_merge_partial(float* O_acc, float* LSE_acc, const float* O_part, const float* LSE_part, long long rows,
                         cudaStream_t stream);

}  // namespace hk
