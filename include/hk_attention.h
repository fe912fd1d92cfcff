/*
 * hk_attention.h -- C ABI of the sm_100a (B200) fused attention forward/backward.
 *
 * Drop-in boundary for the launch surface of BlubridgeAI/HyperKernels
 * kernels/attention.  The reference exposes no host API: its boundary is
 * "kernel symbol + by-value POD argument block + launch geometry", visible in
 * kernels/tests/kernels_test.cu:509-530 (forward), :475-477 (D pre-pass) and
 * :580-584 (backward).  Each entry point below replaces one of those launches
 * and takes an argument block whose leading bytes are exactly the reference
 * block, followed by an extension tail.  A caller holding a reference block
 * copies it into the head of ours, zeroes the tail, and calls.
 *
 * Conventions
 *   - head_dim is 64, I/O is fp32, MMA operands are TF32 rounded to nearest
 *     exactly as the reference rounds them (bit pattern + 0x1000, low 13 bits
 *     dropped), accumulation is fp32.
 *   - All pointers are device pointers owned by the caller; the library never
 *     allocates device memory.  Scratch comes from `workspace`.
 *   - Strides are in elements; the last-dimension stride is 1.  Every pointer
 *     and every stride*4 must be a multiple of 16 bytes.  A batch or head
 *     stride of 0 (one slice broadcast over several batches or heads, which
 *     the reference's pointer arithmetic allows) is refused with
 *     HK_ERR_UNSUPPORTED when that dimension is larger than 1: the TMA tensor
 *     maps the kernels read through cannot express it.
 *   - Re-entrant: no call keeps state between calls except per-device caches
 *     that are filled once under a lock, so any number of host threads may
 *     drive any number of devices and streams.  Device ordinals 0..63.
 *   - Every function returns HK_OK (0) or a negative hk_status; nothing exits
 *     the process or throws.  Kernel launches are asynchronous on `stream`;
 *     device-side faults surface on the caller's next synchronisation, and the
 *     bounded-wait guard of the kernels is read back with hk_attn_last_device_status.
 *   - No CPU fallback: without a CUDA device every compute call returns
 *     HK_ERR_CUDA.
 */
#ifndef HK_ATTENTION_H_
#define HK_ATTENTION_H_

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum hk_status {
    HK_OK = 0,
    HK_ERR_NULL_POINTER = -1,
    HK_ERR_BAD_SHAPE = -2,     /* B, nh, T <= 0, T too large, kv_len < 0 */
    HK_ERR_MISALIGNED = -3,    /* pointer or stride not 16-byte aligned */
    HK_ERR_BAD_DROPOUT = -4,   /* p outside [0,1), or both mask and Philox requested */
    HK_ERR_WORKSPACE = -5,     /* workspace missing or smaller than hk_attn_*_workspace_bytes */
    HK_ERR_UNSUPPORTED = -6,   /* combination the kernels do not implement */
    HK_ERR_CUDA = -7,          /* CUDA runtime/driver error (no device, launch failure) */
    HK_ERR_DEVICE_TIMEOUT = -8, /* a bounded wait inside a kernel gave up */
    HK_ERR_STATIC_SCRATCH = -9  /* problem too large for the built-in scratch of hk_attn_forward_static_scratch */
} hk_status;

/* Size of the scratch array built into the library for hk_attn_forward_static_scratch. */
#define HK_STATIC_SCRATCH_BYTES ((size_t)24 << 20)

enum {
    /* dropout keep-mask is generated in the kernel from (dropout_seed, dropout_offset)
     * with Philox4x32-10; see hk_attn_dropout_mask for the host twin. */
    HK_FLAG_PHILOX_DROPOUT = 1u << 0,
    /* Q, K, V (and dO) already hold TF32-representable values (low 13 mantissa
     * bits zero): skip the operand rounding and its workspace. */
    HK_FLAG_OPERANDS_PREROUNDED = 1u << 1,
    /* backward: add into dK/dV instead of overwriting them (a K/V block that
     * travels round a sequence-sharded ring carries its gradients with it). */
    HK_FLAG_ACCUM_DKDV = 1u << 2,
    /* backward: do not zero dQ before accumulating into it. */
    HK_FLAG_ACCUM_DQ = 1u << 3,
    /* backward: D is supplied by the caller (reference behaviour of the unified
     * kernel taken alone); otherwise hk_attn_backward computes it from dO and O. */
    HK_FLAG_D_PRECOMPUTED = 1u << 4,
    /* backward: `workspace` is the one hk_attn_forward was given for these same Q, K, V
     * (same shapes, same is_causal, same rounding flags) and still holds what that call left
     * there: do not round again what it holds. */
    HK_FLAG_REUSE_FWD_ROUNDED = 1u << 5,
    /* forward and backward: inverted dropout instead of the reference's drop-then-renormalise
     * (no reference counterpart).  The softmax is normalised over ALL visible keys, the kept
     * probabilities are multiplied by 1/(1-p) and the dropped ones are zero in O; LSE does not
     * depend on the mask.  p is dropout_p for a dense mask and floor(dropout_p * 65536) / 65536
     * for the Philox mask.  Without active dropout the flag changes nothing. */
    HK_FLAG_DROPOUT_SCALED = 1u << 6,
    /* forward: O and LSE already hold the attention result over the keys seen so far (LSE = -inf, any O, for a
     * row that has seen none); the call folds the keys of THIS call in and leaves the combined result in O and
     * LSE -- the previous result acts as one more "key" of weight exp(LSE) and value O.  A caller that shards the
     * key sequence (a KV ring) chains its calls this way instead of merging partial results afterwards.  Not
     * available together with HK_FLAG_DROPOUT_SCALED.  No counterpart in the reference. */
    HK_FLAG_CONTINUE_SOFTMAX_STATE = 1u << 7,
    /* forward and backward: always round the operands with the HBM pre-pass into the workspace.  By default
     * problems of 512 <= T <= 2048 (causal) or <= 1024 (otherwise) are rounded in shared memory after the TMA has
     * landed a tile -- forward: Q, K, V, and no workspace is needed (one that is given and large enough receives
     * the rounded tensors for a backward with HK_FLAG_REUSE_FWD_ROUNDED); stand-alone backward: K and V (Q and dO
     * are still rounded into the workspace) -- because there the pre-pass costs more than the extra
     * shared-memory traffic; both ways give the same bits. */
    HK_FLAG_ROUND_IN_HBM = 1u << 8,
    /* backward: deterministic dQ.  By default the KV-tile CTAs add their dQ tiles into dQ with bulk reductions whose
     * order is not fixed (run-to-run differences of the order of 1e-5); with this flag every CTA stores its tiles
     * into the workspace instead (ceil(kv_len / 128) slabs of B*nh*T*256 bytes behind the rounded operands:
     * hk_attn_bwd_workspace_bytes counts them) and a second kernel adds the slabs in KV-tile order: the same
     * inputs give the same bits on every run.  The slabs are ceil(kv_len / 128) times the size of dQ: meant for
     * the sequence lengths of training batches, not for a 32k-token single sequence.  The reference's own dQ is
     * accumulated with atomicAdd
     * (mem_efficient_bwd_unified_kernel_exp12.cu:239-260) and is not reproducible either. */
    HK_FLAG_DETERMINISTIC_DQ = 1u << 9
};

/* ---- forward ------------------------------------------------------------
 * Head (192 bytes) == MemEfficientFwdParams,
 * kernels/attention/fused_attn_forward_kernel_tc_sm89.cu:8-29. */
typedef struct hk_attn_fwd_params {
    const float* Q;
    const float* K;
    const float* V;
    float* O;
    float* LSE;
    int B;
    int nh;
    int64_t T; /* query rows per (b,h) */
    float scale;
    bool is_causal;
    float dropout_p;
    const float* dropout_mask; /* dense [B*nh, T, kv_len] 1.0/0.0 floats, or NULL */
    int64_t q_strideB, q_strideM, q_strideH;
    int64_t k_strideB, k_strideM, k_strideH;
    int64_t v_strideB, v_strideM, v_strideH;
    int64_t o_strideB, o_strideM, o_strideH;
    int64_t lse_strideB, lse_strideH;
    /* ---- extension tail (all-zero == reference behaviour) ---- */
    uint64_t dropout_seed;
    uint64_t dropout_offset;
    void* workspace;
    size_t workspace_bytes;
    int64_t kv_len; /* key rows per (b,h); 0 means T */
    int64_t q_pos0; /* global position of query row 0 (causal mask, dropout counter) */
    int64_t k_pos0; /* global position of key row 0 */
    uint32_t flags;
    uint32_t bh_pos0; /* global index of (batch 0, head 0) of this call in the Philox counter: a caller that
                       * cuts one problem into several calls over runs of (batch, head) slices passes the
                       * first slice's index, so every cut draws the mask of the single call; 0 otherwise */
} hk_attn_fwd_params;

/* ---- backward -----------------------------------------------------------
 * Head (328 bytes) == MemEfficientBwdParams, declared twice in the reference
 * with one layout: kernels/attention/mem_efficient_bwd_precompute_D_sm89.cu:7-33
 * and OwnTensor:: kernels/attention/mem_efficient_bwd_unified_kernel_exp12.cu:11-38. */
typedef struct hk_attn_bwd_params {
    const float* Q;
    const float* K;
    const float* V;
    const float* O;
    const float* dO;
    const float* LSE;
    float* D;
    float* dQ;
    float* dK;
    float* dV;
    int B;
    int nh;
    int T;
    float scale;
    bool is_causal;
    int64_t q_strideB, q_strideM, q_strideH;
    int64_t k_strideB, k_strideM, k_strideH;
    int64_t v_strideB, v_strideM, v_strideH;
    int64_t o_strideB, o_strideM, o_strideH;
    int64_t do_strideB, do_strideM, do_strideH;
    int64_t dq_strideB, dq_strideM, dq_strideH;
    int64_t dk_strideB, dk_strideM, dk_strideH;
    int64_t dv_strideB, dv_strideM, dv_strideH;
    int64_t lse_strideB, lse_strideH;
    int64_t d_strideB, d_strideH;
    /* ---- extension tail ---- */
    float dropout_p; /* the reference backward has no dropout; 0 reproduces it */
    uint32_t flags;
    const float* dropout_mask; /* dense [B*nh, T, kv_len] or NULL */
    uint64_t dropout_seed;
    uint64_t dropout_offset;
    void* workspace;
    size_t workspace_bytes;
    int64_t kv_len;
    int64_t q_pos0;
    int64_t k_pos0;
    uint32_t bh_pos0; /* as in hk_attn_fwd_params */
    uint32_t reserved;
} hk_attn_bwd_params;

/* Replaces the launch of fused_attn_forward_kernel_tc_sm89<64,64,64,1>
 * (kernels/tests/kernels_test.cu:509-530; kernel at
 * kernels/attention/fused_attn_forward_kernel_tc_sm89.cu:72-426).
 * Writes O and LSE.  `stream` is a cudaStream_t (NULL = default stream). */
int hk_attn_forward(const hk_attn_fwd_params* p, void* stream);

/* hk_attn_forward for callers that cannot allocate device memory (it has no
 * counterpart in the reference, whose kernels need no scratch).  Same arguments
 * and results as hk_attn_forward, but `workspace`/`workspace_bytes` are ignored:
 * the TF32-rounded operand copies go into a 24 MiB array that is part of the
 * library's device image, so the call itself allocates nothing (no cudaMalloc,
 * no cudaFree).  Meant for plug-ins living inside a framework that owns all
 * device memory, and for serving loops where an allocation would stall the GPU.
 * Limits: B*nh*(T + 2*kv_len)*256 bytes must fit in HK_STATIC_SCRATCH_BYTES,
 * otherwise HK_ERR_STATIC_SCRATCH; every GPU that loads the library carries the
 * array until exit; all calls on a GPU share it, so calls that overlap in time
 * on one GPU race (serialise them); the first call on each device resolves the
 * array's address and should be made before any stream capture begins. */
int hk_attn_forward_static_scratch(const hk_attn_fwd_params* p, void* stream);

/* Replaces the launch of mem_efficient_bwd_precompute_D_sm89<64>
 * (kernels/tests/kernels_test.cu:475-477; kernel at
 * kernels/attention/mem_efficient_bwd_precompute_D_sm89.cu:45-91).
 * Reads dO, O and their strides, B, nh, T; writes D. */
int hk_attn_bwd_precompute_D(const hk_attn_bwd_params* p, void* stream);

/* The same pre-pass for the other head dimensions the reference instantiates it for
 * (mem_efficient_bwd_precompute_D_sm89<16|32|48|64|80|96|128|160|192|256>,
 * kernels/attention/mem_efficient_bwd_precompute_D_sm89.cu:93-102): dO and O rows hold
 * `head_dim` floats.  The attention kernels themselves are head_dim 64 only. */
int hk_attn_bwd_precompute_D_hd(const hk_attn_bwd_params* p, int head_dim, void* stream);

/* Replaces the launch of OwnTensor::mem_efficient_bwd_unified_kernel_exp12<64,Causal>
 * (kernels/tests/kernels_test.cu:562-584; kernel at
 * kernels/attention/mem_efficient_bwd_unified_kernel_exp12.cu:54-329) together
 * with the steps its caller performs around it: the D pre-pass (unless
 * HK_FLAG_D_PRECOMPUTED) and the zeroing of dQ (unless HK_FLAG_ACCUM_DQ).
 * Writes dQ, dK, dV (and D). */
int hk_attn_backward(const hk_attn_bwd_params* p, void* stream);

/* Scratch the two calls need for the given block, flags included (0 when none).  Forward: the rounded Q, K, V
 * (3 tensors) when the HBM pre-pass rounds them, nothing when the kernel rounds in shared memory -- though a workspace
 * of hk_attn_bwd_workspace_bytes given to it then receives the rounded tensors for HK_FLAG_REUSE_FWD_ROUNDED.
 * Backward: the rounded Q, K, V, dO (4 tensors, in the forward's order followed by dO), then, with
 * HK_FLAG_DETERMINISTIC_DQ, one slab of partial dQ per 128-key tile. */
size_t hk_attn_fwd_workspace_bytes(const hk_attn_fwd_params* p);
size_t hk_attn_bwd_workspace_bytes(const hk_attn_bwd_params* p);

/* Merges the result of a forward over one more block of keys into a running
 * result: (O_acc, LSE_acc) <- softmax-merge of (O_acc, LSE_acc) and
 * (O_part, LSE_part), rows contiguous [rows, 64] / [rows].  Used by callers that
 * shard the key sequence (ring attention).  No counterpart in the reference,
 * whose forward always sees all keys. */
int hk_attn_merge_partial(float* O_acc, float* LSE_acc, const float* O_part, const float* LSE_part, int64_t rows,
                          void* stream);

/* Rounds `rows` contiguous rows of 64 floats to TF32 (round to nearest, the reference's
 * `+0x1000`, fused_attn_forward_kernel_tc_sm89.cu:197) from src into dst (dst may be src: in place).  A caller
 * that feeds the same tensor to several calls (the ring schedule does) rounds it once and passes
 * HK_FLAG_OPERANDS_PREROUNDED.  No counterpart in the reference, which rounds at every load. */
int hk_attn_round_tf32(const float* src, float* dst, int64_t rows, void* stream);

/* Host twin of the in-kernel Philox keep-mask: fills the dense mask the
 * reference forward consumes (fused_attn_forward_kernel_tc_sm89.cu:321-324),
 * mask[(bh*Tq + i)*Tk + j] = 1.0f keep / 0.0f drop.  `mask` is HOST memory. */
int hk_attn_dropout_mask(float* mask, int BH, int64_t Tq, int64_t Tk, float p, uint64_t seed, uint64_t offset,
                         int64_t q_pos0, int64_t k_pos0);
/* The same for (batch, head) slices bh_pos0 .. bh_pos0 + BH - 1 of a larger problem (the mask a call with that
 * bh_pos0 in its argument block draws). */
int hk_attn_dropout_mask_slices(float* mask, uint32_t bh_pos0, int BH, int64_t Tq, int64_t Tk, float p, uint64_t seed,
                                uint64_t offset, int64_t q_pos0, int64_t k_pos0);

/* Reads (and clears) the status word the kernels of this process wrote on the
 * current device: HK_OK, or HK_ERR_DEVICE_TIMEOUT if a bounded wait gave up.
 * Synchronises the device. */
int hk_attn_last_device_status(void);

/* Number of kernels this library has launched in this process (all devices). */
uint64_t hk_attn_launch_count(void);

/* Per-kernel timing for benchmarks: while enabled, CUDA events are recorded on the
 * launching stream around the forward (kind 0) and backward (kind 1) tensor-core
 * kernels; _read waits for them, returns their summed duration and count since
 * the last read, and releases them.  The reference has no counterpart (its
 * timing lives in its benchmark programs, blas/tests/test_sgemm_addmm_sm89.cu:131-145). */
void hk_attn_kernel_timing_enable(int on);
int hk_attn_kernel_timing_read(int kind, double* total_ms, int* launches);

/* Runs the tensor-core self-test on the current device: small TF32 products
 * through each operand path the attention kernels use (K-major and MN-major
 * shared-memory operands, tensor-memory A operand).  out[0..n) receives the
 * raw results of case `which` (0..2); case 3 computes nothing and makes one
 * bounded wait run out on purpose (about 2 s), after which
 * hk_attn_last_device_status() reports HK_ERR_DEVICE_TIMEOUT once; see
 * hyperkernels_b200/csrc/umma_selftest.cu. */
int hk_attn_selftest(int which, const float* A, const float* B, float* out, void* stream);

const char* hk_status_string(int status);

#ifdef __cplusplus
}
#endif

#endif /* HK_ATTENTION_H_ */
