// attn_fwd_static.cu -- hk_attn_forward_static_scratch: the forward for callers
// that may not allocate device memory.
//
// hk_attn_forward needs scratch (TF32-rounded copies of Q, K and V) and takes it
// from a caller-provided workspace.  Some callers have nowhere to get one: an
// operator plugged into a host framework that owns every byte of device memory
// through its own pool and forbids cudaMalloc from plug-ins, a latency-critical
// serving loop in which cudaMalloc/cudaFree would synchronise the whole device,
// or code that runs where the allocator simply is not reachable.  For them the
// scratch lives in a fixed array inside this library's device image.
//
// Costs and limits, all deliberate:
//   * every GPU that loads the library holds HK_STATIC_SCRATCH_BYTES (24 MiB)
//     until the process exits, used or not;
//   * a call is accepted only if its rounded copies fit: B*nh*(T + 2*kv_len)*256
//     bytes <= 24 MiB, i.e. up to 98 304 rows of 64 floats over Q, K and V
//     together (for example 32 heads x 1024 tokens); larger problems get
//     HK_ERR_STATIC_SCRATCH and must use hk_attn_forward with a workspace;
//   * all calls on a device share the one array.  It keeps whatever the last
//     call left in it; nothing in it needs to start at zero, because each call
//     overwrites exactly the rows it then reads.  Two calls that overlap in time
//     on the same GPU (different streams, or different host threads) race on it
//     and corrupt each other's operands: serialise them.
//   * the first call on each device looks the array's device address up
//     (cudaGetSymbolAddress); make that first call outside any stream capture.
#include <mutex>

#include "attn_common.cuh"

namespace {

constexpr size_t kScratchBytes = HK_STATIC_SCRATCH_BYTES;

// In host code this name is only a handle for the runtime, never a device
// address: it must go through cudaGetSymbolAddress before a kernel can use it.
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

// Device address of g_static_scratch on the current device, resolved once per device.
int static_scratch_ptr(void** out) {
    static void* cache[64] = {};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return HK_ERR_CUDA;
    std::lock_guard<std::mutex> lock(mu);
    if (!cache[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) return HK_ERR_CUDA;
        cache[dev] = p;
    }
    *out = cache[dev];
    return HK_OK;
}

}  // namespace

extern "C" int hk_attn_forward_static_scratch(const hk_attn_fwd_params* p, void* stream) {
    if (!p) return HK_ERR_NULL_POINTER;
    hk_attn_fwd_params q = *p;  // the caller's block is left untouched
    q.workspace = nullptr;
    q.workspace_bytes = 0;
    q.flags |= HK_FLAG_ROUND_IN_HBM;  // this entry point's contract is the pre-pass into the built-in scratch
    const size_t need = hk_attn_fwd_workspace_bytes(&q);
    if (need > kScratchBytes) return HK_ERR_STATIC_SCRATCH;
    if (need > 0) {
        void* scratch = nullptr;
        const int rc = static_scratch_ptr(&scratch);
        if (rc != HK_OK) return rc;
        q.workspace = scratch;
        q.workspace_bytes = kScratchBytes;
    }
    return hk_attn_forward(&q, stream);
}
