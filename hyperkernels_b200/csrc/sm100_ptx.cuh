// sm100_ptx.cuh -- thin inline-PTX wrappers for the Blackwell (sm_100a) features
// the attention kernels use: mbarrier, TMA bulk-tensor loads, tensor memory
// (TMEM) allocation / load / store, and tcgen05.mma with TF32 operands.
//
// Every wait is bounded: a spin that does not complete within HK_WAIT_LIMIT_NS
// raises the CTA's abort flag and the global status word and returns false, so
// no kernel built on these helpers can hang a device.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace hk {

// ---------------------------------------------------------------------------
// status word written by kernels when a bounded wait gives up
// ---------------------------------------------------------------------------
struct DeviceStatus {
    int code;        // 0 = ok, otherwise the id of the wait that timed out
    int block;       // blockIdx.x + gridDim.x * blockIdx.y of the first reporter
    int thread;      // threadIdx.x of the first reporter
    int aux;         // loop iteration the wait belonged to
};

constexpr unsigned long long HK_WAIT_LIMIT_NS = 2000000000ull;  // 2 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t elect_one_sync() {
    uint32_t pred = 0;
    asm volatile(
        "{\n"
        ".reg .pred P1;\n"
        "elect.sync _|P1, 0xffffffff;\n"
        "selp.u32 %0, 1, 0, P1;\n"
        "}\n"
        : "=r"(pred));
    return pred;
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_inval(uint64_t* bar) {
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)));
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// makes generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05.mma)
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Per-CTA wait context: `abort` lives in shared memory and is raised by the
// first wait that gives up; every later wait sees it and returns at once.
struct WaitCtx {
    volatile int* abort_flag;  // shared memory
    DeviceStatus* status;      // global memory
};

static __device__ __forceinline__ bool mbar_wait_slow(const WaitCtx& ctx, uint64_t* bar, uint32_t parity, int wait_id, int aux) {
    const unsigned long long t0 = globaltimer_ns();
    while (true) {
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*ctx.abort_flag) return false;
        if (globaltimer_ns() - t0 > HK_WAIT_LIMIT_NS) {
            *ctx.abort_flag = 1;
            if (atomicCAS(&ctx.status->code, 0, wait_id) == 0) {
                ctx.status->block = blockIdx.x + gridDim.x * blockIdx.y;
                ctx.status->thread = threadIdx.x;
                ctx.status->aux = aux;
            }
            __threadfence();
            return false;
        }
    }
}

// Returns false if the wait was abandoned (the CTA must then wind down).
__device__ __forceinline__ bool mbar_wait(const WaitCtx& ctx, uint64_t* bar, uint32_t parity, int wait_id, int aux = 0) {
    for (int i = 0; i < 32; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(ctx, bar, parity, wait_id, aux);
}

__device__ __forceinline__ int smid() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(r));
    return (int)r;
}

// ---------------------------------------------------------------------------
// TMA: tiled bulk-tensor load, global -> shared, completion on an mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// 4-D tile load. Coordinates are element indices, innermost first; c0 must be
// a multiple of 4 floats (16 bytes).
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
        "r"(c3)
        : "memory");
}

// Requests the tile into L2 only (no shared-memory destination, no completion to wait for).
__device__ __forceinline__ void tma_prefetch_l2_4d(const CUtensorMap* map, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}

// 4-D tile reduction, shared -> global: global[tile] += shared tile (fp32 add performed by the
// memory system).  Rows of the box that lie outside the tensor are skipped.  Completion is tracked
// by the issuing thread's bulk async-group.  The shared-memory tile must have been written, and
// fence_proxy_async_smem() executed by its writers, before the issuing thread learnt about it.
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* map, const void* smem_src, int c0, int c1, int c2,
                                                  int c3) {
    asm volatile(
        "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group"
        " [%0, {%2, %3, %4, %5}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
// 4-D tile store, shared -> global; same rules as the reduction above.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* smem_src, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all committed bulk groups of this thread have finished READING shared memory
__device__ __forceinline__ void bulk_wait_group_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// all committed bulk groups of this thread are complete
__device__ __forceinline__ void bulk_wait_group_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---------------------------------------------------------------------------
// tensor memory
// ---------------------------------------------------------------------------
// Executed by ONE full warp. ncols is a power of two in [32, 512]. The base
// address (lane 0, first column) is written to *smem_out.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_out, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_out)),
                 "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tmem_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Each thread of the warp reads 32 consecutive 32-bit columns of its own lane
// (lane = 32*(warp_id%4) + laneid must be encoded in taddr bits [16,32)).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

// 16 consecutive columns of this warp's 32 lanes
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// 16 lanes x 64 consecutive columns in the accumulator-fragment shape (16x256b, eight times): thread t of the warp
// receives, for each group j of eight columns, r[4j], r[4j+1] = lane (t >> 2), columns 8j + 2(t & 3) + {0, 1} and
// r[4j+2], r[4j+3] = lane (t >> 2) + 8, same columns -- four threads hold 32 consecutive bytes of a row, so that
// what they write to global memory falls into whole sectors.  taddr names the first of the 16 lanes.
__device__ __forceinline__ void tmem_ld_16x256b_x8(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

// Pointer flavours for slices of a larger register array (indices must be
// compile-time constants after unrolling so the array stays in registers).
__device__ __forceinline__ void tmem_ld32p(uint32_t taddr, uint32_t* r) {
    tmem_ld32(taddr, *reinterpret_cast<uint32_t(*)[32]>(r));
}
__device__ __forceinline__ void tmem_st32p(uint32_t taddr, const uint32_t* r) {
    tmem_st32(taddr, *reinterpret_cast<const uint32_t(*)[32]>(r));
}

// ---------------------------------------------------------------------------
// tcgen05.mma, kind::tf32, one CTA
// ---------------------------------------------------------------------------
// 32-bit instruction descriptor: fp32 accumulator, TF32 A and B.
//   bits [4,6)  D format (1 = F32)      bits [7,10)  A format (2 = TF32)
//   bits [10,13) B format (2 = TF32)    bit 15 / 16  A / B major (0 = K, 1 = MN)
//   bits [17,23) N >> 3                 bits [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc_tf32(int M, int N, bool a_mn_major, bool b_mn_major) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// 64-bit shared-memory matrix descriptor.
//   bits [0,14)  start address >> 4       bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4  bits [46,48) version (1 on sm_100)
//   bits [61,64) layout: 2 = 128-byte swizzle of 16-byte chunks,
//                        1 = 128-byte swizzle of 32-byte chunks
//
// K-major operand (contraction index contiguous): rows of 32 floats = one
//   128-byte swizzle row, XOR of the 16-byte chunk index with (row & 7); 8-row
//   groups are SBO = 1024 bytes apart, LBO is unused.  TMA writes this layout
//   with CU_TENSOR_MAP_SWIZZLE_128B.
// MN-major operand (M or N index contiguous): for 32-bit operands the tensor
//   core accepts only the 32-byte-chunk flavour: each contraction index is a
//   128-byte row of 32 MN-contiguous floats, XOR of the 32-byte chunk index
//   with (row & 3); 4-row groups are SBO = 512 bytes apart (one K=8 MMA spans
//   two of them), and the next 32 MN elements live LBO bytes further.  TMA
//   writes this layout with CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B.
constexpr uint32_t DESC_SW128 = 2;        // K-major tiles
constexpr uint32_t DESC_SW128_32B = 1;    // MN-major tiles

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t layout) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)layout << 61;
    return d;
}

// K-major 128 x 64 fp32 tile stored as two boxes of [128 rows][32 floats]:
// descriptor of the K = 8 slice number kk (0..7).
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t tile_addr, int kk, uint32_t box_bytes) {
    return make_smem_desc(tile_addr + (kk >> 2) * box_bytes + (kk & 3) * 32, 16, 1024, DESC_SW128);
}

// MN-major tile stored as boxes of [rows = contraction index][32 floats]:
// descriptor of the K = 8 slice number kk (8 rows = 1024 bytes each).
__device__ __forceinline__ uint64_t mnmajor_desc(uint32_t tile_addr, int kk, uint32_t box_bytes) {
    return make_smem_desc(tile_addr + kk * 1024, box_bytes, 512, DESC_SW128_32B);
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts_tf32(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Warp-wide flavours.  A tcgen05.mma is issued by ONE thread, but its 64-bit descriptors and
// addresses are warp-uniform values: when the whole warp runs the issuing code and only the
// instruction itself is predicated on the elected lane (`leader` = elect_one_sync(), nonzero in
// one lane), the compiler keeps that arithmetic on the uniform datapath.  Issued from inside a
// divergent `if (lane == 0)` region instead, every operand is moved lane-wise and one thread
// sustains only one M128 N64 MMA per ~54 cycles (measured) instead of one per ~36.
__device__ __forceinline__ void umma_ss_tf32_lead(uint32_t leader, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                  uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "setp.ne.b32 q, %5, 0;\n"
        "@q tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader)
        : "memory");
}

__device__ __forceinline__ void umma_ts_tf32_lead(uint32_t leader, uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                                  uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "setp.ne.b32 q, %5, 0;\n"
        "@q tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader)
        : "memory");
}

__device__ __forceinline__ void umma_commit_lead(uint32_t leader, uint64_t* bar) {
    asm volatile(
        "{\n"
        ".reg .pred q;\n"
        "setp.ne.b32 q, %1, 0;\n"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
        "}\n"
        ::"r"(smem_u32(bar)), "r"(leader)
        : "memory");
}

// mbarrier arrives once all tcgen05.mma issued so far by this thread have completed
// (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// ---------------------------------------------------------------------------
// misc math
// ---------------------------------------------------------------------------
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Round an fp32 bit pattern to TF32 the way the reference does before every
// MMA (bits + 0x1000; the tensor core then ignores the low 13 bits).
__device__ __forceinline__ uint32_t tf32_round_bits(uint32_t bits) { return (bits + 0x1000u) & 0xFFFFE000u; }
// Same value as seen by the tensor core, which drops the low 13 bits itself:
// for operands written by a kernel straight into tensor or shared memory.
__device__ __forceinline__ uint32_t tf32_round_bits_mma(uint32_t bits) { return bits + 0x1000u; }

__device__ __forceinline__ void red_add_v2(float* gptr, uint32_t a, uint32_t b) {
    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(gptr), "f"(__uint_as_float(a)), "f"(__uint_as_float(b))
                 : "memory");
}

__device__ __forceinline__ void red_add_v4(float* gptr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(gptr), "f"(a), "f"(b), "f"(c), "f"(d)
                 : "memory");
}

}  // namespace hk
