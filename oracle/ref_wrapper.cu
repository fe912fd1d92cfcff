// ref_wrapper.cu -- TEST INFRASTRUCTURE ONLY.
//
// Pulls the reference's own test translation unit (kernels/tests/kernels_test.cu)
// into this one with its main() renamed, so that its file-static host functions
// attn_ref_forward / attn_ref_backward / rand_vec (kernels_test.cu:48-54,68-139)
// and its declarations of the three sm_89 attention kernels can be reached
// through a C ABI.  The reference sources are compiled where they lie; nothing
// is copied.  The resulting library is the "reference" CPU baseline and the
// second (GPU) oracle: the unmodified reference kernels recompiled for the
// local architecture.
#include <cstring>

#define main hk_reference_main
#include HK_REF_TEST_CU
#undef main

extern "C" {

void hkref_rand_vec(float* out, size_t n, uint64_t seed, float lo, float hi) {
    std::vector<float> v = rand_vec(n, seed, lo, hi);
    std::memcpy(out, v.data(), n * sizeof(float));
}

void hkref_attn_forward(const float* Q, const float* K, const float* V, int B, int H, int T, int Hd, float scale,
                        int causal, float* O, float* LSE) {
    const size_t n = (size_t)B * H * T * Hd, r = (size_t)B * H * T;
    std::vector<float> q(Q, Q + n), k(K, K + n), v(V, V + n), o(n), lse(r);
    attn_ref_forward(q, k, v, B, H, T, Hd, scale, causal != 0, o, lse);
    std::memcpy(O, o.data(), n * sizeof(float));
    std::memcpy(LSE, lse.data(), r * sizeof(float));
}

void hkref_attn_backward(const float* Q, const float* K, const float* V, const float* O, const float* dO,
                         const float* LSE, int B, int H, int T, int Hd, float scale, int causal, float* D, float* dQ,
                         float* dK, float* dV) {
    const size_t n = (size_t)B * H * T * Hd, r = (size_t)B * H * T;
    std::vector<float> q(Q, Q + n), k(K, K + n), v(V, V + n), o(O, O + n), go(dO, dO + n), lse(LSE, LSE + r);
    std::vector<float> d(r), dq(n), dk(n), dv(n);
    attn_ref_backward(q, k, v, o, go, lse, B, H, T, Hd, scale, causal != 0, d, dq, dk, dv);
    std::memcpy(D, d.data(), r * sizeof(float));
    std::memcpy(dQ, dq.data(), n * sizeof(float));
    std::memcpy(dK, dk.data(), n * sizeof(float));
    std::memcpy(dV, dv.data(), n * sizeof(float));
}

// --- the unmodified reference GPU kernels, launched with the geometry of the
// --- reference test (kernels_test.cu:509-514,529-530,475-477,580-584).
// params192 / params328 point at host copies of the by-value argument blocks.
int hkref_gpu_forward(const void* params192, void* stream) {
    MemEfficientFwdParams fp;
    std::memcpy(&fp, params192, sizeof(fp));
    const int HD_PAD = 64 + 4, BK_STRIDE = 64 + 8;
    size_t smem = sizeof(float) * ((size_t)64 * HD_PAD + 2 * 64 * HD_PAD + 64 * BK_STRIDE + 3 * 64);
    cudaError_t e = cudaFuncSetAttribute(fused_attn_forward_kernel_tc_sm89<64, 64, 64, 1>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grd((unsigned)((fp.T + 63) / 64), (unsigned)(fp.B * fp.nh)), blk(256);
    fused_attn_forward_kernel_tc_sm89<64, 64, 64, 1><<<grd, blk, smem, (cudaStream_t)stream>>>(fp);
    return (int)cudaGetLastError();
}

int hkref_gpu_precompute_D(const void* params328, void* stream) {
    ::MemEfficientBwdParams p;
    std::memcpy(&p, params328, sizeof(p));
    dim3 grd((unsigned)((p.T + 15) / 16), (unsigned)(p.B * p.nh)), blk(256);
    mem_efficient_bwd_precompute_D_sm89<64><<<grd, blk, 0, (cudaStream_t)stream>>>(p);
    return (int)cudaGetLastError();
}

// The caller zeroes dQ first (kernels_test.cu:562); D must already be filled.
int hkref_gpu_backward(const void* params328, void* stream) {
    OwnTensor::MemEfficientBwdParams bp;
    std::memcpy(&bp, params328, sizeof(bp));
    const int HD_PAD = 64 + 4, BKN_PAD = 16 + 4, BM_PAD = 32 + 4;
    size_t smem = sizeof(float) *
                  ((size_t)2 * 32 * HD_PAD + 2 * 16 * HD_PAD + 2 * 32 * BKN_PAD + 2 * 16 * BM_PAD + 32 * HD_PAD + 2 * 32);
    dim3 grd((unsigned)((bp.T + 15) / 16), (unsigned)(bp.B * bp.nh)), blk(256);
    if (bp.is_causal)
        OwnTensor::mem_efficient_bwd_unified_kernel_exp12<64, true><<<grd, blk, smem, (cudaStream_t)stream>>>(bp);
    else
        OwnTensor::mem_efficient_bwd_unified_kernel_exp12<64, false><<<grd, blk, smem, (cudaStream_t)stream>>>(bp);
    return (int)cudaGetLastError();
}

}  // extern "C"
