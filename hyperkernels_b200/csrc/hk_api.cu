// hk_api.cu -- the extern "C" boundary declared in include/hk_attention.h:
// argument validation, workspace carving, tensor-map construction and the
// launch sequence of each entry point.  No device memory is allocated here.
#include <atomic>
#include <cmath>
#include <cstddef>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

#include "attn_kernels.cuh"
#include "attn_prepass.cuh"
#include "philox.h"

// The leading bytes of both argument blocks must be the reference's by-value
// structs (fused_attn_forward_kernel_tc_sm89.cu:8-29, 192 bytes;
// mem_efficient_bwd_unified_kernel_exp12.cu:11-38, 328 bytes).
static_assert(offsetof(hk_attn_fwd_params, Q) == 0 && offsetof(hk_attn_fwd_params, LSE) == 32, "fwd head");
static_assert(offsetof(hk_attn_fwd_params, B) == 40 && offsetof(hk_attn_fwd_params, nh) == 44, "fwd head");
static_assert(offsetof(hk_attn_fwd_params, T) == 48 && offsetof(hk_attn_fwd_params, scale) == 56, "fwd head");
static_assert(offsetof(hk_attn_fwd_params, is_causal) == 60 && offsetof(hk_attn_fwd_params, dropout_p) == 64, "fwd head");
static_assert(offsetof(hk_attn_fwd_params, dropout_mask) == 72 && offsetof(hk_attn_fwd_params, q_strideB) == 80, "fwd head");
static_assert(offsetof(hk_attn_fwd_params, lse_strideH) == 184 && offsetof(hk_attn_fwd_params, dropout_seed) == 192, "fwd head");
static_assert(offsetof(hk_attn_bwd_params, D) == 48 && offsetof(hk_attn_bwd_params, dV) == 72, "bwd head");
static_assert(offsetof(hk_attn_bwd_params, B) == 80 && offsetof(hk_attn_bwd_params, T) == 88, "bwd head");
static_assert(offsetof(hk_attn_bwd_params, scale) == 92 && offsetof(hk_attn_bwd_params, is_causal) == 96, "bwd head");
static_assert(offsetof(hk_attn_bwd_params, q_strideB) == 104 && offsetof(hk_attn_bwd_params, d_strideH) == 320, "bwd head");
static_assert(sizeof(hk_attn_fwd_params) == 256 && sizeof(hk_attn_bwd_params) == 408, "block sizes");
static_assert(offsetof(hk_attn_bwd_params, dropout_p) == 328, "bwd tail starts after the 328-byte reference block");

namespace hk {


// ---- process-wide state ------------------------------------------------------
static std::atomic<uint64_t> g_launches{0};
void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

// ---- optional kernel timing -----------------------------------------------------
static std::atomic<int> g_timing_on{0};
static std::mutex g_timing_mu;
struct EventPair { cudaEvent_t a, b; };
static std::vector<EventPair> g_events[TIMED_KINDS];

void timing_mark(int kind, bool begin, cudaStream_t stream) {
    if (!g_timing_on.load(std::memory_order_relaxed)) return;
    std::lock_guard<std::mutex> lock(g_timing_mu);
    if (begin) {
        EventPair e{};
        if (cudaEventCreate(&e.a) != cudaSuccess || cudaEventCreate(&e.b) != cudaSuccess) return;
        cudaEventRecord(e.a, stream);
        g_events[kind].push_back(e);
    } else if (!g_events[kind].empty()) {
        cudaEventRecord(g_events[kind].back().b, stream);
    }
}

int check_launch() {
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return HK_OK;
    fprintf(stderr, "libhk_attention: kernel launch failed: %s\n", cudaGetErrorString(e));
    return HK_ERR_CUDA;
}

__device__ DeviceStatus g_device_status;  // one instance per device that loads the module

DeviceStatus* device_status_ptr() {
    static DeviceStatus* cache[HK_MAX_DEVICES] = {};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= HK_MAX_DEVICES) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!cache[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
        cache[dev] = static_cast<DeviceStatus*>(p);
    }
    return cache[dev];
}

EncodeTiledFn get_encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

int make_tile_map(CUtensorMap* map, const float* ptr, int inner, int B, int H, int64_t T, int64_t sB, int64_t sM,
                  int64_t sH, int box_rows, bool mn_major) {
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) return HK_ERR_CUDA;
    // A size-1 dimension may carry any stride; give it a harmless valid one.
    if (H == 1) sH = sM * T;
    if (B == 1) sB = (sH * H > sM * T) ? sH * H : sM * T;
    cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)T, (cuuint64_t)H, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)sM * 4, (cuuint64_t)sH * 4, (cuuint64_t)sB * 4};
    cuuint32_t box[4] = {(cuuint32_t)HALF_D, (cuuint32_t)box_rows, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE,
                     mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? HK_OK : HK_ERR_CUDA;
}

// ---- optional phase timeline of one CTA (performance debugging) ------------------
static std::atomic<long long*> g_timeline{nullptr};
static std::atomic<int> g_timeline_block{0};

// ---- validation helpers -------------------------------------------------------
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static inline bool stride_ok(int64_t s) { return s >= 0 && (s % 4) == 0; }
// A stride of 0 would broadcast one slice over batches or heads; the TMA tensor maps cannot express that.
static inline bool broadcast_stride(int n, int64_t s) { return n > 1 && s == 0; }
static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace hk

using namespace hk;

extern "C" {

const char* hk_status_string(int s) {
    switch (s) {
        case HK_OK: return "ok";
        case HK_ERR_NULL_POINTER: return "null pointer";
        case HK_ERR_BAD_SHAPE: return "bad shape";
        case HK_ERR_MISALIGNED: return "pointer or stride not 16-byte aligned";
        case HK_ERR_BAD_DROPOUT: return "bad dropout arguments";
        case HK_ERR_WORKSPACE: return "workspace missing or too small";
        case HK_ERR_UNSUPPORTED: return "unsupported combination";
        case HK_ERR_CUDA: return "CUDA error";
        case HK_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel gave up";
        case HK_ERR_STATIC_SCRATCH:
            return "problem needs more scratch than the 24 MiB built into the library; use hk_attn_forward with a workspace";
        default: return "unknown status";
    }
}

void hk_attn_kernel_timing_enable(int on) { g_timing_on.store(on ? 1 : 0); }

int hk_attn_kernel_timing_read(int kind, double* total_ms, int* launches) {
    if (kind < 0 || kind >= TIMED_KINDS || !total_ms || !launches) return HK_ERR_BAD_SHAPE;
    std::lock_guard<std::mutex> lock(g_timing_mu);
    double tot = 0;
    int n = 0;
    for (EventPair& e : g_events[kind]) {
        float ms = 0.f;
        if (cudaEventSynchronize(e.b) == cudaSuccess && cudaEventElapsedTime(&ms, e.a, e.b) == cudaSuccess) {
            tot += ms;
            ++n;
        }
        cudaEventDestroy(e.a);
        cudaEventDestroy(e.b);
    }
    g_events[kind].clear();
    *total_ms = tot;
    *launches = n;
    return HK_OK;
}

uint64_t hk_attn_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int hk_attn_last_device_status(void) {
    DeviceStatus* d = device_status_ptr();
    if (!d) return HK_ERR_CUDA;
    if (cudaDeviceSynchronize() != cudaSuccess) return HK_ERR_CUDA;
    DeviceStatus h;
    if (cudaMemcpy(&h, d, sizeof(h), cudaMemcpyDeviceToHost) != cudaSuccess) return HK_ERR_CUDA;
    if (h.code != 0) {
        DeviceStatus z = {0, 0, 0, 0};
        cudaMemcpy(d, &z, sizeof(z), cudaMemcpyHostToDevice);
        return HK_ERR_DEVICE_TIMEOUT;
    }
    return HK_OK;
}

int hk_attn_dropout_mask(float* mask, int BH, int64_t Tq, int64_t Tk, float p, uint64_t seed, uint64_t offset,
                         int64_t q_pos0, int64_t k_pos0) {
    return hk_attn_dropout_mask_slices(mask, 0u, BH, Tq, Tk, p, seed, offset, q_pos0, k_pos0);
}

int hk_attn_dropout_mask_slices(float* mask, uint32_t bh_pos0, int BH, int64_t Tq, int64_t Tk, float p, uint64_t seed,
                                uint64_t offset, int64_t q_pos0, int64_t k_pos0) {
    if (!mask) return HK_ERR_NULL_POINTER;
    if (!(p >= 0.f && p < 1.f)) return HK_ERR_BAD_DROPOUT;
    if (BH < 0 || Tq < 0 || Tk < 0) return HK_ERR_BAD_SHAPE;
    const uint32_t thr = hk_philox_threshold(p);
    for (int bh = 0; bh < BH; ++bh)
        for (int64_t i = 0; i < Tq; ++i) {
            float* row = mask + ((size_t)bh * Tq + i) * Tk;
            for (int64_t j = 0; j < Tk; ++j)
                row[j] = hk_philox_keep(seed, offset, bh_pos0 + (uint32_t)bh, (uint32_t)(q_pos0 + i), (uint32_t)(k_pos0 + j), thr)
                             ? 1.0f
                             : 0.0f;
        }
    return HK_OK;
}

// Where the operands are rounded to TF32.  For short sequences the kernels do it in shared memory after the TMA has
// landed a tile (forward: Q, K, V; backward: K, V), for long ones an HBM pre-pass writes rounded copies into the
// workspace: the pre-pass costs two passes over every tensor, the in-kernel rounding costs shared-memory bandwidth
// once per tile LOAD, and a K/V tile is loaded once per 256 query rows (and what the pre-pass reads from HBM the
// kernel then reads itself, cold).  Measured on a B200: forward kernel +2.3 us at
// B8 H12 T1024 causal (against 18 us of pre-pass for K and V), +16 % at T16384.  Both give the same bits.
static bool round_in_kernel(uint32_t flags, int64_t Tq, bool causal) {
    if (flags & (HK_FLAG_OPERANDS_PREROUNDED | HK_FLAG_ROUND_IN_HBM)) return false;
    return Tq >= 512 && Tq * (causal ? 1 : 2) <= 2048;  // below 512 rows a CTA has one or two steps and nothing to hide it under
}

size_t hk_attn_fwd_workspace_bytes(const hk_attn_fwd_params* p) {
    if (!p || (p->flags & HK_FLAG_OPERANDS_PREROUNDED)) return 0;
    if (p->B <= 0 || p->nh <= 0 || p->T <= 0) return 0;
    if (round_in_kernel(p->flags, p->T, p->is_causal != 0)) return 0;  // rounded in shared memory: nothing is required
    const int64_t Tk = p->kv_len > 0 ? p->kv_len : p->T;
    const size_t bh = (size_t)p->B * p->nh;
    return align_up(bh * p->T * 256, 256) + 2 * align_up(bh * Tk * 256, 256);
}

// bytes of the rounded operands (Q, dO, K, V) at the head of the backward's workspace
static size_t bwd_rounded_bytes(const hk_attn_bwd_params* p) {
    if (p->flags & HK_FLAG_OPERANDS_PREROUNDED) return 0;
    const int64_t Tk = p->kv_len > 0 ? p->kv_len : p->T;
    const size_t bh = (size_t)p->B * p->nh;
    return 2 * align_up(bh * p->T * 256, 256) + 2 * align_up(bh * Tk * 256, 256);
}

size_t hk_attn_bwd_workspace_bytes(const hk_attn_bwd_params* p) {
    if (!p || p->B <= 0 || p->nh <= 0 || p->T <= 0) return 0;
    size_t n = bwd_rounded_bytes(p);
    if (p->flags & HK_FLAG_DETERMINISTIC_DQ) {  // one slab of partial dQ per KV tile
        const int64_t Tk = p->kv_len > 0 ? p->kv_len : p->T;
        n += (size_t)((Tk + TILE - 1) / TILE) * align_up((size_t)p->B * p->nh * p->T * 256, 256);
    }
    return n;
}

// 1/(1-p) of the inverted-dropout option, with p as the kernels apply it: the Philox mask drops with
// probability floor(p * 65536) / 65536, a caller's dense mask is taken to have been drawn with p itself.
static float keep_scale_of(float p, int mode, uint32_t flags) {
    if (!(flags & HK_FLAG_DROPOUT_SCALED) || mode == 0) return 1.f;
    const double pe = (mode == 2) ? (double)hk_philox_threshold(p) / 65536.0 : (double)p;
    return (float)(1.0 / (1.0 - pe));
}

static int validate_dropout(float p, const float* mask, uint32_t flags, int64_t k_pos0, int* mode) {
    *mode = 0;
    if (!(p >= 0.f && p < 1.f)) return HK_ERR_BAD_DROPOUT;
    const bool philox = (flags & HK_FLAG_PHILOX_DROPOUT) != 0;
    if (philox && mask) return HK_ERR_BAD_DROPOUT;
    if (p > 0.f) {
        if (philox) {
            if (k_pos0 % 8 != 0) return HK_ERR_UNSUPPORTED;  // one Philox call covers keys 8n .. 8n+7
            *mode = 2;
        } else if (mask) {
            *mode = 1;  // reference semantics: active only when p > 0 and mask != nullptr
        }
    }
    return HK_OK;
}

int hk_attn_forward(const hk_attn_fwd_params* p, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!p) return HK_ERR_NULL_POINTER;
    if (!p->Q || !p->K || !p->V || !p->O || !p->LSE) return HK_ERR_NULL_POINTER;
    const int64_t Tq = p->T, Tk = p->kv_len > 0 ? p->kv_len : p->T;
    if (p->B <= 0 || p->nh <= 0 || Tq <= 0 || p->kv_len < 0) return HK_ERR_BAD_SHAPE;
    if (Tq > (1 << 30) || Tk > (1 << 30) || (int64_t)p->B * p->nh > (1 << 24)) return HK_ERR_BAD_SHAPE;
    if (p->q_pos0 < 0 || p->k_pos0 < 0 || p->q_pos0 + Tq > (1LL << 31) - 1 || p->k_pos0 + Tk > (1LL << 31) - 1)
        return HK_ERR_BAD_SHAPE;
    if (!aligned16(p->Q) || !aligned16(p->K) || !aligned16(p->V) || !aligned16(p->O)) return HK_ERR_MISALIGNED;
    const int64_t st[] = {p->q_strideB, p->q_strideM, p->q_strideH, p->k_strideB, p->k_strideM, p->k_strideH,
                          p->v_strideB, p->v_strideM, p->v_strideH, p->o_strideB, p->o_strideM, p->o_strideH};
    for (int64_t s : st)
        if (!stride_ok(s)) return HK_ERR_MISALIGNED;
    if (p->q_strideM < HEAD_DIM || p->k_strideM < HEAD_DIM || p->v_strideM < HEAD_DIM || p->o_strideM < HEAD_DIM)
        return HK_ERR_BAD_SHAPE;
    {
        const int64_t sb[] = {p->q_strideB, p->k_strideB, p->v_strideB, p->o_strideB};
        const int64_t sh[] = {p->q_strideH, p->k_strideH, p->v_strideH, p->o_strideH};
        for (int i = 0; i < 4; ++i)
            if (broadcast_stride(p->B, sb[i]) || broadcast_stride(p->nh, sh[i])) return HK_ERR_UNSUPPORTED;
    }
    if (!std::isfinite(p->scale) || p->scale == 0.f) return HK_ERR_BAD_SHAPE;  // masking multiplies -inf by the scale
    int mode = 0;
    int rc = validate_dropout(p->dropout_p, p->dropout_mask, p->flags, p->k_pos0, &mode);
    if (rc != HK_OK) return rc;

    const int B = p->B, H = p->nh, BH = B * H;
    CUtensorMap mq, mk, mv, mqw, mkw, mvw;
    const bool in_kernel = round_in_kernel(p->flags, Tq, p->is_causal != 0);
    float* q_rounded_out = nullptr;
    if ((p->flags & HK_FLAG_OPERANDS_PREROUNDED) || in_kernel) {
        // the kernel reads the caller's tensors: already rounded, or rounded in shared memory after the TMA landing
        if ((rc = make_tile_map(&mq, p->Q, HEAD_DIM, B, H, Tq, p->q_strideB, p->q_strideM, p->q_strideH, TILE))) return rc;
        if ((rc = make_tile_map(&mk, p->K, HEAD_DIM, B, H, Tk, p->k_strideB, p->k_strideM, p->k_strideH, TILE))) return rc;
        if ((rc = make_tile_map(&mv, p->V, HEAD_DIM, B, H, Tk, p->v_strideB, p->v_strideM, p->v_strideH, TILE, true))) return rc;
        // a workspace, if the caller gave one, receives the rounded Q, K, V where the pre-pass would have put them
        // (HK_FLAG_REUSE_FWD_ROUNDED in the backward)
        const size_t qb = align_up((size_t)BH * Tq * 256, 256), kb = align_up((size_t)BH * Tk * 256, 256);
        if (in_kernel && p->workspace && p->workspace_bytes >= qb + 2 * kb &&
            !(reinterpret_cast<uintptr_t>(p->workspace) & 255u))
            q_rounded_out = static_cast<float*>(p->workspace);
        mqw = mq; mkw = mk; mvw = mv;
        if (q_rounded_out) {
            uint8_t* ws = static_cast<uint8_t*>(p->workspace);
            float* kr = reinterpret_cast<float*>(ws + qb);
            float* vr = reinterpret_cast<float*>(ws + qb + kb);
            if ((rc = make_tile_map(&mqw, q_rounded_out, HEAD_DIM, B, H, Tq, (int64_t)H * Tq * 64, 64, Tq * 64, TILE))) return rc;
            if ((rc = make_tile_map(&mkw, kr, HEAD_DIM, B, H, Tk, (int64_t)H * Tk * 64, 64, Tk * 64, TILE))) return rc;
            if ((rc = make_tile_map(&mvw, vr, HEAD_DIM, B, H, Tk, (int64_t)H * Tk * 64, 64, Tk * 64, TILE, true))) return rc;
        }
    } else {
        const size_t need = hk_attn_fwd_workspace_bytes(p);
        if (!p->workspace || p->workspace_bytes < need || (reinterpret_cast<uintptr_t>(p->workspace) & 255u))
            return HK_ERR_WORKSPACE;
        uint8_t* ws = static_cast<uint8_t*>(p->workspace);
        float* qr = reinterpret_cast<float*>(ws);
        float* kr = reinterpret_cast<float*>(ws + align_up((size_t)BH * Tq * 256, 256));
        float* vr = reinterpret_cast<float*>(ws + align_up((size_t)BH * Tq * 256, 256) + align_up((size_t)BH * Tk * 256, 256));
        RoundJob job{};
        job.src[0] = View4{p->Q, p->q_strideB, p->q_strideM, p->q_strideH};
        job.src[1] = View4{p->K, p->k_strideB, p->k_strideM, p->k_strideH};
        job.src[2] = View4{p->V, p->v_strideB, p->v_strideM, p->v_strideH};
        job.dst[0] = qr; job.dst[1] = kr; job.dst[2] = vr;
        job.T[0] = (int)Tq; job.T[1] = (int)Tk; job.T[2] = (int)Tk;
        job.H = H; job.BH = BH; job.n = 3;
        if ((rc = launch_round_tf32(job, stream))) return rc;
        if ((rc = make_tile_map(&mq, qr, HEAD_DIM, B, H, Tq, (int64_t)H * Tq * 64, 64, Tq * 64, TILE))) return rc;
        if ((rc = make_tile_map(&mk, kr, HEAD_DIM, B, H, Tk, (int64_t)H * Tk * 64, 64, Tk * 64, TILE))) return rc;
        if ((rc = make_tile_map(&mv, vr, HEAD_DIM, B, H, Tk, (int64_t)H * Tk * 64, 64, Tk * 64, TILE, true))) return rc;
        mqw = mq; mkw = mk; mvw = mv;
    }

    FwdArgs a{};
    a.O = p->O; a.LSE = p->LSE;
    a.mask = (mode == 1) ? p->dropout_mask : nullptr;
    a.o_sB = p->o_strideB; a.o_sM = p->o_strideM; a.o_sH = p->o_strideH;
    a.lse_sB = p->lse_strideB; a.lse_sH = p->lse_strideH;
    a.H = H; a.BH = BH; a.Tq = (int)Tq; a.Tk = (int)Tk;
    a.n_qtiles = (int)((Tq + 2 * TILE - 1) / (2 * TILE));  // the forward takes two 128-row tiles per CTA
    a.q_pos0 = (int)p->q_pos0; a.k_pos0 = (int)p->k_pos0;
    a.scale_log2e = p->scale * LOG2E;
    a.causal = p->is_causal ? 1 : 0;
    a.dropout_mode = mode;
    a.keep_scale = keep_scale_of(p->dropout_p, mode, p->flags);
    a.drop_scaled = (mode != 0 && (p->flags & HK_FLAG_DROPOUT_SCALED)) ? 1 : 0;
    a.continue_state = (p->flags & HK_FLAG_CONTINUE_SOFTMAX_STATE) ? 1 : 0;
    a.round_in_smem = in_kernel ? 1 : 0;
    a.store_q = q_rounded_out ? 1 : 0;
    if (a.continue_state && a.drop_scaled) return HK_ERR_UNSUPPORTED;
    a.drop_thr = hk_philox_threshold(p->dropout_p);
    a.seed = p->dropout_seed; a.offset = p->dropout_offset; a.bh_pos0 = p->bh_pos0;
    a.status = device_status_ptr();
    if (!a.status) return HK_ERR_CUDA;
    a.timeline = g_timeline.load();
    a.timeline_block = g_timeline_block.load();
    CUtensorMap mo;
    if ((rc = make_tile_map(&mo, p->O, HEAD_DIM, B, H, Tq, p->o_strideB, p->o_strideM, p->o_strideH, TILE))) return rc;
    return launch_attn_fwd(mq, mk, mv, mo, mqw, mkw, mvw, a, stream);
}

int hk_attn_bwd_precompute_D(const hk_attn_bwd_params* p, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!p) return HK_ERR_NULL_POINTER;
    if (!p->dO || !p->O || !p->D) return HK_ERR_NULL_POINTER;
    if (p->B <= 0 || p->nh <= 0 || p->T <= 0) return HK_ERR_BAD_SHAPE;
    if (!aligned16(p->dO) || !aligned16(p->O)) return HK_ERR_MISALIGNED;
    const int64_t st[] = {p->o_strideB, p->o_strideM, p->o_strideH, p->do_strideB, p->do_strideM, p->do_strideH};
    for (int64_t s : st)
        if (!stride_ok(s)) return HK_ERR_MISALIGNED;
    if (p->o_strideM < HEAD_DIM || p->do_strideM < HEAD_DIM) return HK_ERR_BAD_SHAPE;
    DJob j{};
    j.dO = View4{p->dO, p->do_strideB, p->do_strideM, p->do_strideH};
    j.O = View4{p->O, p->o_strideB, p->o_strideM, p->o_strideH};
    j.D = p->D; j.d_sB = p->d_strideB; j.d_sH = p->d_strideH;
    j.dO_rounded = nullptr;
    j.dQ_zero = nullptr;
    j.H = p->nh; j.BH = p->B * p->nh; j.T = p->T;
    return launch_precompute_D(j, stream);
}

int hk_attn_bwd_precompute_D_hd(const hk_attn_bwd_params* p, int head_dim, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!p) return HK_ERR_NULL_POINTER;
    if (!p->dO || !p->O || !p->D) return HK_ERR_NULL_POINTER;
    if (p->B <= 0 || p->nh <= 0 || p->T <= 0) return HK_ERR_BAD_SHAPE;
    {
        // the ten instantiations of mem_efficient_bwd_precompute_D_sm89.cu:93-102
        static const int dims[] = {16, 32, 48, 64, 80, 96, 128, 160, 192, 256};
        bool known = false;
        for (int d : dims) known = known || d == head_dim;
        if (!known) return HK_ERR_UNSUPPORTED;
    }
    if (!aligned16(p->dO) || !aligned16(p->O)) return HK_ERR_MISALIGNED;
    const int64_t st[] = {p->o_strideB, p->o_strideM, p->o_strideH, p->do_strideB, p->do_strideM, p->do_strideH};
    for (int64_t s : st)
        if (!stride_ok(s)) return HK_ERR_MISALIGNED;
    if (p->o_strideM < head_dim || p->do_strideM < head_dim) return HK_ERR_BAD_SHAPE;
    DJob j{};
    j.dO = View4{p->dO, p->do_strideB, p->do_strideM, p->do_strideH};
    j.O = View4{p->O, p->o_strideB, p->o_strideM, p->o_strideH};
    j.D = p->D; j.d_sB = p->d_strideB; j.d_sH = p->d_strideH;
    j.H = p->nh; j.BH = p->B * p->nh; j.T = p->T;
    return launch_precompute_D_hd(j, head_dim, stream);
}

int hk_attn_backward(const hk_attn_bwd_params* p, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!p) return HK_ERR_NULL_POINTER;
    if (!p->Q || !p->K || !p->V || !p->dO || !p->LSE || !p->D || !p->dQ || !p->dK || !p->dV) return HK_ERR_NULL_POINTER;
    const bool d_given = (p->flags & HK_FLAG_D_PRECOMPUTED) != 0;
    if (!d_given && !p->O) return HK_ERR_NULL_POINTER;
    const int64_t Tq = p->T, Tk = p->kv_len > 0 ? p->kv_len : p->T;
    if (p->B <= 0 || p->nh <= 0 || Tq <= 0 || p->kv_len < 0) return HK_ERR_BAD_SHAPE;
    if (Tk > (1 << 30) || (int64_t)p->B * p->nh > (1 << 24)) return HK_ERR_BAD_SHAPE;
    if (p->q_pos0 < 0 || p->k_pos0 < 0 || p->q_pos0 + Tq > (1LL << 31) - 1 || p->k_pos0 + Tk > (1LL << 31) - 1)
        return HK_ERR_BAD_SHAPE;
    const void* ptrs[] = {p->Q, p->K, p->V, p->dO, p->dQ, p->dK, p->dV};
    for (const void* q : ptrs)
        if (!aligned16(q)) return HK_ERR_MISALIGNED;
    if (!d_given && !aligned16(p->O)) return HK_ERR_MISALIGNED;
    const int64_t st[] = {p->q_strideB,  p->q_strideM,  p->q_strideH,  p->k_strideB,  p->k_strideM,  p->k_strideH,
                          p->v_strideB,  p->v_strideM,  p->v_strideH,  p->o_strideB,  p->o_strideM,  p->o_strideH,
                          p->do_strideB, p->do_strideM, p->do_strideH, p->dq_strideB, p->dq_strideM, p->dq_strideH,
                          p->dk_strideB, p->dk_strideM, p->dk_strideH, p->dv_strideB, p->dv_strideM, p->dv_strideH};
    for (int64_t s : st)
        if (!stride_ok(s)) return HK_ERR_MISALIGNED;
    if (p->q_strideM < HEAD_DIM || p->k_strideM < HEAD_DIM || p->v_strideM < HEAD_DIM || p->do_strideM < HEAD_DIM ||
        p->dq_strideM < HEAD_DIM || p->dk_strideM < HEAD_DIM || p->dv_strideM < HEAD_DIM)
        return HK_ERR_BAD_SHAPE;
    {
        const int64_t sb[] = {p->q_strideB, p->k_strideB, p->v_strideB, p->do_strideB, p->dq_strideB, p->dk_strideB, p->dv_strideB};
        const int64_t sh[] = {p->q_strideH, p->k_strideH, p->v_strideH, p->do_strideH, p->dq_strideH, p->dk_strideH, p->dv_strideH};
        for (int i = 0; i < 7; ++i)
            if (broadcast_stride(p->B, sb[i]) || broadcast_stride(p->nh, sh[i])) return HK_ERR_UNSUPPORTED;
    }
    if (!std::isfinite(p->scale) || p->scale == 0.f) return HK_ERR_BAD_SHAPE;  // as in the forward
    int mode = 0;
    int rc = validate_dropout(p->dropout_p, p->dropout_mask, p->flags, p->k_pos0, &mode);
    if (rc != HK_OK) return rc;

    const int B = p->B, H = p->nh, BH = B * H;
    const View4 vQ{p->Q, p->q_strideB, p->q_strideM, p->q_strideH}, vK{p->K, p->k_strideB, p->k_strideM, p->k_strideH},
        vV{p->V, p->v_strideB, p->v_strideM, p->v_strideH}, vdO{p->dO, p->do_strideB, p->do_strideM, p->do_strideH},
        vO{p->O, p->o_strideB, p->o_strideM, p->o_strideH};
    BwdMaps m;
    float* dO_rounded = nullptr;
    // the tensors the MMAs read: the caller's (pre-rounded) or the rounded copies in the workspace
    View4 tQ = vQ, tK = vK, tV = vV, tdO = vdO;
    bool round_kv = false;
    const bool det_dq = (p->flags & HK_FLAG_DETERMINISTIC_DQ) != 0;
    const int n_kvtiles = (int)((Tk + TILE - 1) / TILE);
    float* dq_slabs = nullptr;
    if (det_dq) {
        if ((int64_t)n_kvtiles * B > (1 << 24)) return HK_ERR_BAD_SHAPE;
        const size_t need = hk_attn_bwd_workspace_bytes(p);
        if (!p->workspace || p->workspace_bytes < need || (reinterpret_cast<uintptr_t>(p->workspace) & 255u))
            return HK_ERR_WORKSPACE;
        dq_slabs = reinterpret_cast<float*>(static_cast<uint8_t*>(p->workspace) + bwd_rounded_bytes(p));
    }
    if (!(p->flags & HK_FLAG_OPERANDS_PREROUNDED)) {
        const size_t need = hk_attn_bwd_workspace_bytes(p);
        if (!p->workspace || p->workspace_bytes < need || (reinterpret_cast<uintptr_t>(p->workspace) & 255u))
            return HK_ERR_WORKSPACE;
        // layout: rounded Q, K, V exactly where hk_attn_forward puts them, then rounded dO
        uint8_t* ws = static_cast<uint8_t*>(p->workspace);
        const size_t qb = align_up((size_t)BH * Tq * 256, 256), kb = align_up((size_t)BH * Tk * 256, 256);
        float* qr = reinterpret_cast<float*>(ws);
        float* kr = reinterpret_cast<float*>(ws + qb);
        float* vr = reinterpret_cast<float*>(ws + qb + kb);
        dO_rounded = reinterpret_cast<float*>(ws + qb + 2 * kb);
        const bool reuse = (p->flags & HK_FLAG_REUSE_FWD_ROUNDED) != 0;
        // a stand-alone backward of a short sequence rounds K and V in shared memory; one that reuses the forward's
        // workspace finds them there (whichever way the forward rounded them)
        round_kv = !reuse && round_in_kernel(p->flags, Tq, p->is_causal != 0);
        RoundJob job{};
        job.H = H; job.BH = BH;
        int n = 0;
        if (!reuse) {
            job.src[n] = vQ; job.dst[n] = qr; job.T[n] = (int)Tq;
            ++n;
            if (!round_kv) {
                job.src[n] = vK; job.dst[n] = kr; job.T[n] = (int)Tk;
                ++n;
                job.src[n] = vV; job.dst[n] = vr; job.T[n] = (int)Tk;
                ++n;
            }
        }
        if (d_given) {  // otherwise the D pre-pass writes the rounded dO while it reads dO
            job.src[n] = vdO; job.dst[n] = dO_rounded; job.T[n] = (int)Tq;
            ++n;
        }
        job.n = n;
        if (n > 0 && (rc = launch_round_tf32(job, stream))) return rc;
        tQ = View4{qr, (int64_t)H * Tq * 64, 64, Tq * 64};
        tdO = View4{dO_rounded, (int64_t)H * Tq * 64, 64, Tq * 64};
        if (!round_kv) {  // otherwise the kernel reads the caller's K and V and rounds them in shared memory
            tK = View4{kr, (int64_t)H * Tk * 64, 64, Tk * 64};
            tV = View4{vr, (int64_t)H * Tk * 64, 64, Tk * 64};
        }
    }
    if ((rc = make_tile_map(&m.q, tQ.ptr, HEAD_DIM, B, H, Tq, tQ.sB, tQ.sM, tQ.sH, TILE, false))) return rc;
    if ((rc = make_tile_map(&m.k, tK.ptr, HEAD_DIM, B, H, Tk, tK.sB, tK.sM, tK.sH, TILE, false))) return rc;
    if ((rc = make_tile_map(&m.v, tV.ptr, HEAD_DIM, B, H, Tk, tV.sB, tV.sM, tV.sH, TILE, false))) return rc;
    if ((rc = make_tile_map(&m.dO, tdO.ptr, HEAD_DIM, B, H, Tq, tdO.sB, tdO.sM, tdO.sH, TILE, false))) return rc;
    if ((rc = make_tile_map(&m.q_mn, tQ.ptr, HEAD_DIM, B, H, Tq, tQ.sB, tQ.sM, tQ.sH, TILE, true))) return rc;
    if ((rc = make_tile_map(&m.k_mn, tK.ptr, HEAD_DIM, B, H, Tk, tK.sB, tK.sM, tK.sH, TILE, true))) return rc;
    if ((rc = make_tile_map(&m.dO_mn, tdO.ptr, HEAD_DIM, B, H, Tq, tdO.sB, tdO.sM, tdO.sH, TILE, true))) return rc;
    if (det_dq) {
        // the slabs as one tensor [n_kvtiles * B, H, Tq, 64]: KV tile kt of batch b is "batch" kt * B + b
        if ((rc = make_tile_map(&m.dQ, dq_slabs, HEAD_DIM, n_kvtiles * B, H, Tq, (int64_t)H * Tq * 64, 64, Tq * 64, TILE, false)))
            return rc;
    } else if ((rc = make_tile_map(&m.dQ, p->dQ, HEAD_DIM, B, H, Tq, p->dq_strideB, p->dq_strideM, p->dq_strideH, TILE, false)))
        return rc;
    if ((rc = make_tile_map(&m.dK, p->dK, HEAD_DIM, B, H, Tk, p->dk_strideB, p->dk_strideM, p->dk_strideH, TILE, false)))
        return rc;
    if ((rc = make_tile_map(&m.dV, p->dV, HEAD_DIM, B, H, Tk, p->dv_strideB, p->dv_strideM, p->dv_strideH, TILE, false)))
        return rc;
    if (!d_given) {
        DJob j{};
        j.dO = vdO; j.O = vO;
        j.D = p->D; j.d_sB = p->d_strideB; j.d_sH = p->d_strideH;
        j.dO_rounded = dO_rounded;
        if (!(p->flags & HK_FLAG_ACCUM_DQ) && !det_dq) {  // the slab reduction overwrites dQ
            j.dQ_zero = p->dQ; j.dq_sB = p->dq_strideB; j.dq_sM = p->dq_strideM; j.dq_sH = p->dq_strideH;
        }
        j.H = H; j.BH = BH; j.T = (int)Tq;
        if ((rc = launch_precompute_D(j, stream))) return rc;
    } else if (!(p->flags & HK_FLAG_ACCUM_DQ) && !det_dq) {
        if ((rc = launch_zero_rows(p->dQ, p->dq_strideB, p->dq_strideM, p->dq_strideH, B, H, (int)Tq, stream))) return rc;
    }

    BwdArgs a{};
    a.LSE = p->LSE; a.D = p->D; a.dQ = p->dQ; a.dK = p->dK; a.dV = p->dV;
    a.mask = (mode == 1) ? p->dropout_mask : nullptr;
    a.lse_sB = p->lse_strideB; a.lse_sH = p->lse_strideH; a.d_sB = p->d_strideB; a.d_sH = p->d_strideH;
    a.dq_sB = p->dq_strideB; a.dq_sM = p->dq_strideM; a.dq_sH = p->dq_strideH;
    a.dk_sB = p->dk_strideB; a.dk_sM = p->dk_strideM; a.dk_sH = p->dk_strideH;
    a.dv_sB = p->dv_strideB; a.dv_sM = p->dv_strideM; a.dv_sH = p->dv_strideH;
    a.H = H; a.BH = BH; a.Tq = (int)Tq; a.Tk = (int)Tk;
    a.n_kvtiles = n_kvtiles;
    a.det_dq = det_dq ? 1 : 0;
    a.B = B;
    a.q_pos0 = (int)p->q_pos0; a.k_pos0 = (int)p->k_pos0;
    a.scale = p->scale; a.scale_log2e = p->scale * LOG2E;
    a.causal = p->is_causal ? 1 : 0;
    a.accum_dkdv = (p->flags & HK_FLAG_ACCUM_DKDV) ? 1 : 0;
    a.round_kv = round_kv ? 1 : 0;
    a.dropout_mode = mode;
    a.drop_scaled = (mode != 0 && (p->flags & HK_FLAG_DROPOUT_SCALED)) ? 1 : 0;
    a.dv_scale = keep_scale_of(p->dropout_p, mode, p->flags);
    a.dp_scale = p->scale * a.dv_scale;
    a.drop_thr = hk_philox_threshold(p->dropout_p);
    a.seed = p->dropout_seed; a.offset = p->dropout_offset; a.bh_pos0 = p->bh_pos0;
    a.status = device_status_ptr();
    if (!a.status) return HK_ERR_CUDA;
    a.timeline = g_timeline.load();
    a.timeline_block = g_timeline_block.load();
    if ((rc = launch_attn_bwd(m, a, stream))) return rc;
    if (det_dq) {
        DqReduceJob r{};
        r.slabs = dq_slabs; r.dQ = p->dQ;
        r.dq_sB = p->dq_strideB; r.dq_sM = p->dq_strideM; r.dq_sH = p->dq_strideH;
        r.B = B; r.H = H; r.T = (int)Tq; r.n_kvtiles = n_kvtiles;
        r.causal = a.causal; r.q_pos0 = a.q_pos0; r.k_pos0 = a.k_pos0;
        r.accumulate = (p->flags & HK_FLAG_ACCUM_DQ) ? 1 : 0;
        return launch_reduce_dq_slabs(r, stream);
    }
    return HK_OK;
}

int hk_attn_merge_partial(float* O_acc, float* LSE_acc, const float* O_part, const float* LSE_part, int64_t rows,
                          void* stream_) {
    if (!O_acc || !LSE_acc || !O_part || !LSE_part) return HK_ERR_NULL_POINTER;
    if (rows < 0) return HK_ERR_BAD_SHAPE;
    if (!aligned16(O_acc) || !aligned16(O_part)) return HK_ERR_MISALIGNED;
    return launch_merge_partial(O_acc, LSE_acc, O_part, LSE_part, rows, static_cast<cudaStream_t>(stream_));
}

int hk_attn_selftest(int which, const float* A, const float* B, float* out, void* stream_) {
    return run_umma_selftest(which, A, B, out, static_cast<cudaStream_t>(stream_));
}

int hk_attn_round_tf32(const float* src, float* dst, int64_t rows, void* stream_) {
    if (!src || !dst) return HK_ERR_NULL_POINTER;
    if (rows < 0 || rows > (1LL << 31) - 1) return HK_ERR_BAD_SHAPE;
    if (!aligned16(src) || !aligned16(dst)) return HK_ERR_MISALIGNED;
    RoundJob job{};
    job.src[0] = View4{src, 0, 64, 0};  // one "head" of `rows` contiguous rows
    job.dst[0] = dst;
    job.T[0] = (int)rows;
    job.H = 1; job.BH = 1; job.n = 1;
    return launch_round_tf32(job, static_cast<cudaStream_t>(stream_));
}

#ifdef HK_TIMELINE
// Development builds only: CTA `block` of every forward/backward launch writes SM-clock stamps of its pipeline
// phases into device_buffer (4096 int64; slot layout in attn_*_sm100.cu); block = -1: every CTA b < 1024 writes
// {start ns, end ns, SM id, tiles} to slots 4b..4b+3.  nullptr turns it off.
void hk_attn_debug_timeline(long long* device_buffer, int block) {
    g_timeline_block.store(block);
    g_timeline.store(device_buffer);
}
#endif

}  // extern "C"
