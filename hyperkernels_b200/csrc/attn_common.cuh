// attn_common.cuh -- pieces shared by the attention translation units: tile
// constants, the per-call kernel argument blocks, tensor-map construction and
// the process-wide launch counter / device status word.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hk_attention.h"
#include "sm100_ptx.cuh"

namespace hk {

constexpr int HK_MAX_DEVICES = 64;  // device ordinals the per-device caches cover
constexpr int HEAD_DIM = 64;
constexpr int TILE = 128;                      // query rows and key rows per MMA tile
constexpr int HALF_D = 32;                     // floats per 128-byte swizzle row
constexpr int BOX_BYTES = TILE * HALF_D * 4;   // one TMA box: 128 rows x 32 floats = 16 KiB
constexpr int TILE_BYTES = 2 * BOX_BYTES;      // a 128 x 64 fp32 tile = two boxes = 32 KiB
constexpr float LOG2E = 1.4426950408889634074f;
constexpr float LN2 = 0.6931471805599453094f;

// A [B, H, T, 64] fp32 view with element strides (last-dim stride 1).
struct View4 {
    const float* ptr;
    int64_t sB, sM, sH;
};

// ---- host side -------------------------------------------------------------
// cuTensorMapEncodeTiled fetched through the runtime (no link-time libcuda dependency).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_tiled();

// Tensor map over a [B, H, T, inner] fp32 view (element strides sB, sM, sH; last
// stride 1); box = 32 floats x `box_rows` rows, out-of-range rows read as zero.
// mn_major = false: 128-byte swizzle of 16-byte chunks (K-major MMA operand);
// mn_major = true:  128-byte swizzle of 32-byte chunks (MN-major TF32 operand).
int make_tile_map(CUtensorMap* map, const float* ptr, int inner, int B, int H, int64_t T, int64_t sB, int64_t sM,
                  int64_t sH, int box_rows, bool mn_major = false);

DeviceStatus* device_status_ptr();  // per-device status word (allocated as a __device__ symbol)
void count_launch(int n = 1);

// Optional per-kernel timing (hk_attn_kernel_timing_enable): CUDA events recorded on
// the launching stream around the two tensor-core kernels.
enum TimedKernel { TIMED_FWD = 0, TIMED_BWD = 1, TIMED_KINDS = 2 };
void timing_mark(int kind, bool begin, cudaStream_t stream);
int check_launch();  // cudaGetLastError -> hk_status

}  // namespace hk
