// umma_rate.cu -- TEST INFRASTRUCTURE: how fast one warp can feed tcgen05.mma.kind::tf32.
//
// The attention kernels rest on two measured facts about the sm_100a tensor pipe, and this probe re-measures them so
// that tests/test_mma_rates_gpu.py can hold them:
//   1. a tcgen05.mma issued from inside a divergent `if (lane == 0)` region costs the issuing thread ~50 cycles, more
//      than an M128 N64 K8 product takes (36): issued by a converged warp with only the instruction predicated on the
//      elected lane, the same products run at the tensor pipe's own rate;
//   2. an MMA shape's cost: M128 N128 ~75 cycles, M128 N64 ~36 (tensor-memory A) / ~52 (both operands in shared
//      memory), M64 shapes at half rate, M128 N256 ~138.
// One CTA per SM; every CTA issues `iters` groups of one shape back to back on operands that are already in place
// (finite garbage: only the rate matters).  Every wait is bounded (sm100_ptx.cuh).
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../hyperkernels_b200/csrc/sm100_ptx.cuh"

using namespace hk;

namespace {

constexpr int BOX = 16384;
constexpr int SMEM = 200 * 1024;

struct __align__(8) PS {
    uint64_t done;
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ uint64_t kdesc(uint32_t base, int kk, uint32_t box) {
    return make_smem_desc(base + (kk >> 2) * box + (kk & 3) * 32, 16, 1024, DESC_SW128);
}
__device__ __forceinline__ uint64_t mdesc(uint32_t base, int kk) {
    return make_smem_desc(base + kk * 1024, BOX, 512, DESC_SW128_32B);
}

// one group of MMAs of shape `MODE`; `lead` != 0 in the issuing lane
template <int MODE>
__device__ __forceinline__ void group(uint32_t lead, uint32_t tmem, uint32_t a, uint32_t b) {
    if constexpr (MODE == 0) {  // 8 x M128 N128 K8, A and B K-major in shared memory (S = Q K^T)
        constexpr uint32_t id = make_idesc_tf32(128, 128, false, false);
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_ss_tf32_lead(lead, tmem, kdesc(a, k, BOX), kdesc(b, k, BOX), id, 1);
    } else if constexpr (MODE == 1) {  // 16 x M128 N64 K8, A in tensor memory, B MN-major (O = P V, dV, dK)
        constexpr uint32_t id = make_idesc_tf32(128, 64, false, true);
#pragma unroll
        for (int k = 0; k < 16; ++k) umma_ts_tf32_lead(lead, tmem, tmem + 256 + k * 8, mdesc(b, k), id, 1);
    } else if constexpr (MODE == 2) {  // 16 x M128 N64 K8, A and B MN-major in shared memory (dQ = dS K)
        constexpr uint32_t id = make_idesc_tf32(128, 64, true, true);
#pragma unroll
        for (int k = 0; k < 16; ++k) umma_ss_tf32_lead(lead, tmem, mdesc(a, k), mdesc(b, k), id, 1);
    } else if constexpr (MODE == 3) {  // 8 x M64 N128 K8
        constexpr uint32_t id = make_idesc_tf32(64, 128, false, false);
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_ss_tf32_lead(lead, tmem, kdesc(a, k, BOX), kdesc(b, k, BOX), id, 1);
    } else if constexpr (MODE == 4) {  // 8 x M64 N256 K8
        constexpr uint32_t id = make_idesc_tf32(64, 256, false, false);
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_ss_tf32_lead(lead, tmem, kdesc(a, k, BOX), kdesc(b, k, 2 * BOX), id, 1);
    } else if constexpr (MODE == 5) {  // 8 x M128 N256 K8
        constexpr uint32_t id = make_idesc_tf32(128, 256, false, false);
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_ss_tf32_lead(lead, tmem, kdesc(a, k, BOX), kdesc(b, k, 2 * BOX), id, 1);
    } else {  // MODE 6: the 72 products of one backward tile in the kernel's order: dV, S^T, dK, dP^T, dQ
        constexpr uint32_t ids = make_idesc_tf32(128, 128, false, false);
        constexpr uint32_t idt = make_idesc_tf32(128, 64, false, true);
        constexpr uint32_t idq = make_idesc_tf32(128, 64, true, true);
#pragma unroll
        for (int k = 0; k < 16; ++k) umma_ts_tf32_lead(lead, tmem + 256, tmem + k * 8, mdesc(b, k), idt, 1);
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_ss_tf32_lead(lead, tmem, kdesc(a, k, BOX), kdesc(b, k, BOX), ids, 1);
#pragma unroll
        for (int k = 0; k < 16; ++k) umma_ts_tf32_lead(lead, tmem + 320, tmem + 128 + k * 8, mdesc(b + 32768, k), idt, 1);
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_ts_tf32_lead(lead, tmem + 128, tmem + 448 + k * 8, kdesc(b + 32768, k, BOX), ids, 1);
#pragma unroll
        for (int k = 0; k < 16; ++k) umma_ss_tf32_lead(lead, tmem + 384, mdesc(a, k), mdesc(b, k), idq, 1);
    }
}

// converged = 1: the whole warp runs the issuing code, the instruction is predicated on the elected lane;
// converged = 0: the issuing code sits inside `if (lane == 0)`, as a first version of the kernels had it
template <int MODE>
__global__ void __launch_bounds__(128, 1) rate_kernel(int iters, int converged, DeviceStatus* status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    PS& sh = *reinterpret_cast<PS*>(smem + SMEM - 64);
    const int warp = threadIdx.x >> 5;
    if ((smem_u32(smem) & 1023u) != 0) return;
    if (threadIdx.x == 0) {
        mbar_init(&sh.done, 1);
        sh.abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(&sh.tmem_base, 512);
        tmem_relinquish();
        tc_fence_before_sync();
    }
    float* s = reinterpret_cast<float*>(smem);
    for (int i = threadIdx.x; i < (SMEM - 1024) / 4; i += blockDim.x) s[i] = 1e-3f * (float)((i * 37) & 63);
    fence_proxy_async_smem();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sh.tmem_base;
    const uint32_t trow = tmem + ((uint32_t)(warp * 32) << 16);
    WaitCtx wc{&sh.abort_flag, status};
    {
        uint32_t r[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(1e-3f * i);
        for (int c = 0; c < 16; ++c) tmem_st32(trow + c * 32, r);
        tmem_wait_st();
        tc_fence_before_sync();
    }
    __syncthreads();
    const uint32_t a = smem_u32(smem), b = smem_u32(smem) + 65536;
    if (warp == 0) {
        if (converged) {
            const uint32_t lead = elect_one_sync();
            tc_fence_after_sync();
#pragma unroll 1
            for (int it = 0; it < iters; ++it) group<MODE>(lead, tmem, a, b);
            umma_commit_lead(lead, &sh.done);
        } else if ((threadIdx.x & 31) == 0) {
            tc_fence_after_sync();
#pragma unroll 1
            for (int it = 0; it < iters; ++it) group<MODE>(1u, tmem, a, b);
            umma_commit_lead(1u, &sh.done);
        }
        __syncwarp();
    }
    mbar_wait(wc, &sh.done, 0, 980);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem, 512);
    }
}

__device__ DeviceStatus g_status;

template <int MODE>
int launch(int iters, int converged, int ctas, cudaStream_t st, DeviceStatus* status) {
    if (cudaFuncSetAttribute(rate_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) return -1;
    rate_kernel<MODE><<<ctas, 128, SMEM, st>>>(iters, converged, status);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace

// mode 0..6 as in group<>; returns 0 or a negative code.  *flops_per_cta_iter receives the FLOP of one group.
extern "C" int umma_rate_run(int mode, int iters, int converged, int ctas, double* flops_per_cta_iter, int* instrs_per_iter,
                             void* stream) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status) != cudaSuccess) return -2;
    if (iters <= 0 || iters > 20000 || ctas <= 0 || ctas > 4096) return -3;
    DeviceStatus* status = static_cast<DeviceStatus*>(p);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    static const double fl[7] = {8 * 2.0 * 128 * 128 * 8, 16 * 2.0 * 128 * 64 * 8, 16 * 2.0 * 128 * 64 * 8, 8 * 2.0 * 64 * 128 * 8,
                                 8 * 2.0 * 64 * 256 * 8,  8 * 2.0 * 128 * 256 * 8, 16 * 2.0 * 128 * 128 * 8 + 48 * 2.0 * 128 * 64 * 8};
    static const int ni[7] = {8, 16, 16, 8, 8, 8, 72};
    if (mode < 0 || mode > 6) return -5;
    if (flops_per_cta_iter) *flops_per_cta_iter = fl[mode];
    if (instrs_per_iter) *instrs_per_iter = ni[mode];
    switch (mode) {
        case 0: return launch<0>(iters, converged, ctas, st, status);
        case 1: return launch<1>(iters, converged, ctas, st, status);
        case 2: return launch<2>(iters, converged, ctas, st, status);
        case 3: return launch<3>(iters, converged, ctas, st, status);
        case 4: return launch<4>(iters, converged, ctas, st, status);
        case 5: return launch<5>(iters, converged, ctas, st, status);
        default: return launch<6>(iters, converged, ctas, st, status);
    }
}

extern "C" int umma_rate_status(void) {
    DeviceStatus h;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&h, g_status, sizeof(h)) != cudaSuccess) return -2;
    return h.code;
}
