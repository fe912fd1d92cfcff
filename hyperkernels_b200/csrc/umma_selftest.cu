// umma_selftest.cu -- one-tile TF32 products through each operand path the
// attention kernels rely on.  A user (or a test) runs these to confirm that
// the shared-memory descriptors, the tensor-memory A operand and the
// accumulator read-out behave on the installed driver/GPU as the attention
// kernels assume; operands are fed WITHOUT rounding so the raw behaviour of
// tcgen05.mma.kind::tf32 on full-mantissa fp32 input is observable.
//
//   case 0  D[128,128] = A[128,64] * B[128,64]^T    A, B K-major in smem (S = Q K^T)
//   case 1  D[128,64]  = A[128,128] * B[128,64]     A in tensor memory, B MN-major (O = P V)
//   case 2  D[128,64]  = A[128,128]^T * B[128,64]   A MN-major in smem, B MN-major (dQ = dS K)
//   case 3  no product: one thread waits on an mbarrier that nothing ever arrives at, to show that
//           a wait that cannot complete ends after HK_WAIT_LIMIT_NS with the device status word
//           set (hk_attn_last_device_status -> HK_ERR_DEVICE_TIMEOUT) and the context still usable
#include "attn_kernels.cuh"

namespace hk {

namespace st {
constexpr int SMEM_BYTES = 4 * BOX_BYTES + TILE_BYTES + 64 + 1024;
struct __align__(8) Shared {
    uint64_t full, done;
    uint32_t tmem_base;
    int abort_flag;
};
}  // namespace st

__global__ void __launch_bounds__(128, 1)
umma_selftest_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, int which,
                     const float* A, float* out, DeviceStatus* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;                  // up to 4 boxes
    uint8_t* sB = smem + 4 * BOX_BYTES;  // 2 boxes
    st::Shared& sh = *reinterpret_cast<st::Shared*>(smem + 4 * BOX_BYTES + TILE_BYTES);
    const int warp = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
        mbar_init(&sh.full, 1);
        mbar_init(&sh.done, 1);
        sh.abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(&sh.tmem_base, 256);
        tmem_relinquish();
        tc_fence_before_sync();
    }
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sh.tmem_base;
    const uint32_t trow = tmem + ((uint32_t)(warp * 32) << 16);
    WaitCtx wc{&sh.abort_flag, status};
    const int N = (which == 0) ? 128 : 64;
    uint32_t r[32];

    if (which == 3) {
        // nothing is in flight: the only thing to wind down after the failed wait is tensor memory
        if (threadIdx.x == 0) mbar_wait(wc, &sh.full, 0, 999);
        tc_fence_before_sync();
        __syncthreads();
        if (warp == 0) {
            __syncwarp();
            tc_fence_after_sync();
            tmem_dealloc(tmem, 256);
        }
        return;
    }

    if (which == 1) {
        // stage A into tensor-memory columns 128..255 (lane = row)
        const float* arow = A + (size_t)threadIdx.x * 128;
        for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(arow[c * 32 + i]);
            tmem_st32(trow + 128 + c * 32, r);
        }
        tmem_wait_st();
        tc_fence_before_sync();
    }
    __syncthreads();

    if (threadIdx.x == 0) {
        const int a_boxes = (which == 0) ? 2 : (which == 2 ? 4 : 0);
        mbar_arrive_expect_tx(&sh.full, (a_boxes + 2) * BOX_BYTES);
        for (int i = 0; i < a_boxes; ++i) tma_load_4d(sA + i * BOX_BYTES, &mapA, &sh.full, i * HALF_D, 0, 0, 0);
        for (int i = 0; i < 2; ++i) tma_load_4d(sB + i * BOX_BYTES, &mapB, &sh.full, i * HALF_D, 0, 0, 0);
        if (mbar_wait(wc, &sh.full, 0, 901)) {
            tc_fence_after_sync();
            const uint32_t a_addr = smem_u32(sA), b_addr = smem_u32(sB);
            if (which == 0) {
                const uint32_t idesc = make_idesc_tf32(128, 128, false, false);
                for (int kk = 0; kk < 8; ++kk) {
                    umma_ss_tf32(tmem, kmajor_desc(a_addr, kk, BOX_BYTES), kmajor_desc(b_addr, kk, BOX_BYTES), idesc, kk > 0);
                }
            } else if (which == 1) {
                const uint32_t idesc = make_idesc_tf32(128, 64, false, true);
                for (int kk = 0; kk < 16; ++kk)
                    umma_ts_tf32(tmem, tmem + 128 + kk * 8, mnmajor_desc(b_addr, kk, BOX_BYTES), idesc, kk > 0);
            } else {
                const uint32_t idesc = make_idesc_tf32(128, 64, true, true);
                for (int kk = 0; kk < 16; ++kk)
                    umma_ss_tf32(tmem, mnmajor_desc(a_addr, kk, BOX_BYTES), mnmajor_desc(b_addr, kk, BOX_BYTES), idesc, kk > 0);
            }
            umma_commit(&sh.done);
        }
    }
    __syncwarp();
    const bool ok = __all_sync(0xffffffffu, mbar_wait(wc, &sh.done, 0, 902));
    tc_fence_after_sync();
    if (ok) {
        for (int c = 0; c < N / 32; ++c) {
            tmem_ld32(trow + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) out[(size_t)threadIdx.x * N + c * 32 + i] = __uint_as_float(r[i]);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem, 256);
    }
}

int run_umma_selftest(int which, const float* A, const float* B, float* out, cudaStream_t stream) {
    if (which < 0 || which > 3) return HK_ERR_UNSUPPORTED;
    if (!A || !B || !out) return HK_ERR_NULL_POINTER;
    CUtensorMap ma, mb;
    int rc;
    // A: case 0 [128 rows][64], case 2 [128 kv][128 q]; case 1 reads A directly
    const int a_inner = (which == 2) ? 128 : 64;
    if ((rc = make_tile_map(&ma, which == 1 ? B : A, a_inner, 1, 1, 128, 128LL * a_inner, a_inner, 128LL * a_inner,
                            TILE, which == 2)) != HK_OK)
        return rc;
    if ((rc = make_tile_map(&mb, B, 64, 1, 1, 128, 128LL * 64, 64, 128LL * 64, TILE, which != 0)) != HK_OK) return rc;
    if (cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, st::SMEM_BYTES) !=
        cudaSuccess)
        return HK_ERR_CUDA;
    DeviceStatus* status = device_status_ptr();
    if (!status) return HK_ERR_CUDA;
    umma_selftest_kernel<<<1, 128, st::SMEM_BYTES, stream>>>(ma, mb, which, A, out, status);
    count_launch();
    return check_launch();
}

}  // namespace hk
