// attn_prepass.cu -- the HBM-bound helper kernels around the two tensor-core
// kernels: TF32 operand rounding, D = rowsum(dO * O), dQ zeroing and the
// softmax merge of two partial forward results.
#include "attn_prepass.cuh"

#include <algorithm>

namespace hk {

// ---------------------------------------------------------------------------
// TF32 operand rounding.  The reference adds 0x1000 to the bit pattern of every
// MMA operand as it loads it from shared memory
// (fused_attn_forward_kernel_tc_sm89.cu:197,209-210,219;
//  mem_efficient_bwd_unified_kernel_exp12.cu:118,127,136), i.e. round to
// nearest, ties away.  tcgen05.mma reads its operands straight from the bytes
// TMA wrote, so the rounding is applied once here, into contiguous
// [BH, T, 64] copies in the caller's workspace.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) round_tf32_kernel(const RoundJob job) {
    const int t = blockIdx.y;
    const int T = job.T[t];
    const int H = job.H;
    const View4 v = job.src[t];
    uint4* dst = reinterpret_cast<uint4*>(job.dst[t]);
    const long long nvec = (long long)job.BH * T * 16;  // 16 float4 per 64-float row
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * blockDim.x) {
        const long long row = i >> 4;
        const int c4 = (int)(i & 15);
        const int bh = (int)(row / T);
        const int r = (int)(row - (long long)bh * T);
        const int b = bh / H, h = bh - b * H;
        // plain load: dst may be src (hk_attn_round_tf32 in place), which rules the read-only path out
        const float4 x =
            *(reinterpret_cast<const float4*>(v.ptr + (int64_t)b * v.sB + (int64_t)h * v.sH + (int64_t)r * v.sM) + c4);
        uint4 y;
        y.x = tf32_round_bits(__float_as_uint(x.x));
        y.y = tf32_round_bits(__float_as_uint(x.y));
        y.z = tf32_round_bits(__float_as_uint(x.z));
        y.w = tf32_round_bits(__float_as_uint(x.w));
        dst[i] = y;
    }
}

int launch_round_tf32(const RoundJob& job, cudaStream_t stream) {
    long long max_vec = 0;
    for (int t = 0; t < job.n; ++t) max_vec = std::max(max_vec, (long long)job.BH * job.T[t] * 16);
    if (max_vec == 0 || job.n == 0) return HK_OK;
    const int blocks = (int)std::min<long long>((max_vec + 255) / 256, 148 * 8);
    round_tf32_kernel<<<dim3(blocks, job.n), 256, 0, stream>>>(job);
    count_launch();
    return check_launch();
}

// ---------------------------------------------------------------------------
// D[b,h,i] = sum_k dO[i,k] * O[i,k]  (mem_efficient_bwd_precompute_D_sm89.cu:45-91),
// 16 lanes per row, one float4 of each operand per lane.  Optionally also
// writes the TF32-rounded copy of dO the backward MMAs consume, so dO is read
// from HBM once, and zeroes the matching rows of dQ (the reference leaves that
// to its caller, kernels_test.cu:562).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) precompute_D_kernel(const DJob j) {
    const long long nrows = (long long)j.BH * j.T;
    const int sub = threadIdx.x & 15;
    for (long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 4; row < ((nrows + 15) & ~15ll);
         row += ((long long)gridDim.x * blockDim.x) >> 4) {
        float s = 0.f;
        if (row < nrows) {
            const int bh = (int)(row / j.T);
            const int r = (int)(row - (long long)bh * j.T);
            const int b = bh / j.H, h = bh - b * j.H;
            const float4 g = __ldg(
                reinterpret_cast<const float4*>(j.dO.ptr + (int64_t)b * j.dO.sB + (int64_t)h * j.dO.sH + (int64_t)r * j.dO.sM) +
                sub);
            const float4 o = __ldg(
                reinterpret_cast<const float4*>(j.O.ptr + (int64_t)b * j.O.sB + (int64_t)h * j.O.sH + (int64_t)r * j.O.sM) + sub);
            s = g.x * o.x + g.y * o.y + g.z * o.z + g.w * o.w;
            if (j.dO_rounded) {
                uint4 y;
                y.x = tf32_round_bits(__float_as_uint(g.x));
                y.y = tf32_round_bits(__float_as_uint(g.y));
                y.z = tf32_round_bits(__float_as_uint(g.z));
                y.w = tf32_round_bits(__float_as_uint(g.w));
                reinterpret_cast<uint4*>(j.dO_rounded)[row * 16 + sub] = y;
            }
            if (j.dQ_zero)
                reinterpret_cast<float4*>(j.dQ_zero + (int64_t)b * j.dq_sB + (int64_t)h * j.dq_sH + (int64_t)r * j.dq_sM)[sub] =
                    make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (row < nrows && sub == 0) {
            const int bh = (int)(row / j.T);
            const int r = (int)(row - (long long)bh * j.T);
            const int b = bh / j.H, h = bh - b * j.H;
            j.D[(int64_t)b * j.d_sB + (int64_t)h * j.d_sH + r] = s;
        }
    }
}

int launch_precompute_D(const DJob& j, cudaStream_t stream) {
    const long long nrows = (long long)j.BH * j.T;
    if (nrows == 0) return HK_OK;
    const int blocks = (int)std::min<long long>((nrows * 16 + 255) / 256, 148 * 8);
    precompute_D_kernel<<<blocks, 256, 0, stream>>>(j);
    count_launch();
    return check_launch();
}

// ---------------------------------------------------------------------------
// The same row sum for the other head dimensions the reference instantiates
// (mem_efficient_bwd_precompute_D_sm89.cu:93-102: 16, 32, 48, 64, 80, 96, 128,
// 160, 192, 256).  A row of HD floats is HD/4 float4; LANES lanes (a power of
// two, at most a warp) share a row and each takes every LANES-th float4, so
// the dimensions that are not powers of two leave some lanes idle in the last
// round; shuffle reduction within the group.
// ---------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(256) precompute_D_hd_kernel(const DJob j) {
    constexpr int NV = HD / 4;                                        // float4 per row
    constexpr int LANES = NV >= 32 ? 32 : NV >= 16 ? 16 : NV >= 8 ? 8 : 4;  // lanes that share a row
    constexpr int ROUNDS = (NV + LANES - 1) / LANES;
    const long long nrows = (long long)j.BH * j.T;
    const int sub = threadIdx.x % LANES;
    const long long stride = ((long long)gridDim.x * blockDim.x) / LANES;
    const long long rows_pad = (nrows + 32 / LANES - 1) / (32 / LANES) * (32 / LANES);  // whole warps iterate together
    for (long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / LANES; row < rows_pad; row += stride) {
        float s = 0.f;
        int b = 0, h = 0, r = 0;
        if (row < nrows) {
            const int bh = (int)(row / j.T);
            r = (int)(row - (long long)bh * j.T);
            b = bh / j.H;
            h = bh - b * j.H;
            const float4* g4 = reinterpret_cast<const float4*>(j.dO.ptr + (int64_t)b * j.dO.sB + (int64_t)h * j.dO.sH +
                                                               (int64_t)r * j.dO.sM);
            const float4* o4 = reinterpret_cast<const float4*>(j.O.ptr + (int64_t)b * j.O.sB + (int64_t)h * j.O.sH +
                                                               (int64_t)r * j.O.sM);
#pragma unroll
            for (int v = 0; v < ROUNDS; ++v) {
                const int c = sub + v * LANES;
                if (NV % LANES == 0 || c < NV) {
                    const float4 g = __ldg(g4 + c), o = __ldg(o4 + c);
                    s += g.x * o.x + g.y * o.y + g.z * o.z + g.w * o.w;
                }
            }
        }
#pragma unroll
        for (int off = LANES / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (row < nrows && sub == 0) j.D[(int64_t)b * j.d_sB + (int64_t)h * j.d_sH + r] = s;
    }
}

template <int HD>
static void launch_D_hd(const DJob& j, cudaStream_t stream) {
    constexpr int NV = HD / 4;
    constexpr int LANES = NV >= 32 ? 32 : NV >= 16 ? 16 : NV >= 8 ? 8 : 4;
    const long long nrows = (long long)j.BH * j.T;
    const int blocks = (int)std::min<long long>((nrows * LANES + 255) / 256, 148 * 8);
    precompute_D_hd_kernel<HD><<<blocks, 256, 0, stream>>>(j);
}

int launch_precompute_D_hd(const DJob& j, int head_dim, cudaStream_t stream) {
    const long long nrows = (long long)j.BH * j.T;
    if (nrows == 0) return HK_OK;
    switch (head_dim) {
        case 16: launch_D_hd<16>(j, stream); break;
        case 32: launch_D_hd<32>(j, stream); break;
        case 48: launch_D_hd<48>(j, stream); break;
        case 64: launch_D_hd<64>(j, stream); break;
        case 80: launch_D_hd<80>(j, stream); break;
        case 96: launch_D_hd<96>(j, stream); break;
        case 128: launch_D_hd<128>(j, stream); break;
        case 160: launch_D_hd<160>(j, stream); break;
        case 192: launch_D_hd<192>(j, stream); break;
        case 256: launch_D_hd<256>(j, stream); break;
        default: return HK_ERR_UNSUPPORTED;
    }
    count_launch();
    return check_launch();
}

// ---------------------------------------------------------------------------
// zero a strided [B, H, T, 64] tensor (dQ is accumulated with atomics; the
// reference leaves this to its caller, kernels_test.cu:562)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) zero_rows_kernel(float* ptr, int64_t sB, int64_t sM, int64_t sH, int H, int T,
                                                        long long nvec) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * blockDim.x) {
        const long long row = i >> 4;
        const int c4 = (int)(i & 15);
        const int bh = (int)(row / T);
        const int r = (int)(row - (long long)bh * T);
        const int b = bh / H, h = bh - b * H;
        reinterpret_cast<float4*>(ptr + (int64_t)b * sB + (int64_t)h * sH + (int64_t)r * sM)[c4] =
            make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

int launch_zero_rows(float* ptr, int64_t sB, int64_t sM, int64_t sH, int B, int H, int T, cudaStream_t stream) {
    const long long nvec = (long long)B * H * T * 16;
    if (nvec == 0) return HK_OK;
    const int blocks = (int)std::min<long long>((nvec + 255) / 256, 148 * 8);
    zero_rows_kernel<<<blocks, 256, 0, stream>>>(ptr, sB, sM, sH, H, T, nvec);
    count_launch();
    return check_launch();
}

// ---------------------------------------------------------------------------
// Deterministic dQ: add the per-KV-tile slabs in KV-tile order.  A query tile is in the slab of KV tile kt only if
// the backward CTA of kt visited it: under the causal mask that is every query tile from
// it0(kt) = clamp((kt*128 + k_pos0 - q_pos0) / 128) on (attn_bwd_sm100.cu computes the same bound).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) reduce_dq_slabs_kernel(DqReduceJob j, long long nvec) {
    const long long slab = (long long)j.B * j.H * j.T * 16;  // float4 per slab
    const int n_qtiles = (j.T + TILE - 1) / TILE;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * blockDim.x) {
        const long long row = i >> 4;
        const int c4 = (int)(i & 15);
        const int bh = (int)(row / j.T);
        const int r = (int)(row - (long long)bh * j.T);
        const int b = bh / j.H, h = bh - b * j.H;
        const int qt = r / TILE;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float4* out = reinterpret_cast<float4*>(j.dQ + (int64_t)b * j.dq_sB + (int64_t)h * j.dq_sH + (int64_t)r * j.dq_sM) + c4;
        if (j.accumulate) acc = *out;
        const float4* src = reinterpret_cast<const float4*>(j.slabs) + i;
        for (int kt = 0; kt < j.n_kvtiles; ++kt) {
            int it0 = 0;
            if (j.causal) {
                const long long first_q = (long long)kt * TILE + j.k_pos0 - j.q_pos0;
                if (first_q > 0) it0 = (int)min((long long)n_qtiles, first_q / TILE);
            }
            if (qt >= it0) {
                const float4 v = __ldg(src + (long long)kt * slab);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
        }
        *out = acc;
    }
}

int launch_reduce_dq_slabs(const DqReduceJob& j, cudaStream_t stream) {
    const long long nvec = (long long)j.B * j.H * j.T * 16;
    if (nvec == 0) return HK_OK;
    const int blocks = (int)std::min<long long>((nvec + 255) / 256, 148 * 8);
    reduce_dq_slabs_kernel<<<blocks, 256, 0, stream>>>(j, nvec);
    count_launch();
    return check_launch();
}

// ---------------------------------------------------------------------------
// (O_acc, LSE_acc) <- merge with (O_part, LSE_part): both are normalised
// softmax outputs over disjoint key sets, so
//   LSE = log(exp(LSE_a) + exp(LSE_p)),  O = O_a * exp(LSE_a - LSE) + O_p * exp(LSE_p - LSE).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) merge_partial_kernel(float* O_acc, float* LSE_acc, const float* O_part,
                                                            const float* LSE_part, long long rows) {
    const int sub = threadIdx.x & 15;
    // both half-warps of a warp run the same number of iterations (bound rounded up to even)
    for (long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 4; row < ((rows + 1) & ~1ll);
         row += ((long long)gridDim.x * blockDim.x) >> 4) {
        const bool valid = row < rows;
        float wa = 0.f, wp = 0.f, lse = -INFINITY;
        if (valid) {
            const float la = LSE_acc[row], lp = LSE_part[row];
            const float mx = fmaxf(la, lp);
            if (mx > -INFINITY) {
                const float ea = expf(la - mx), ep = expf(lp - mx);
                const float inv = 1.f / (ea + ep);
                wa = ea * inv;
                wp = ep * inv;
                lse = mx + logf(ea + ep);
            }
            float4 x = reinterpret_cast<float4*>(O_acc)[row * 16 + sub];
            const float4 y = __ldg(reinterpret_cast<const float4*>(O_part) + row * 16 + sub);
            x.x = x.x * wa + y.x * wp;
            x.y = x.y * wa + y.y * wp;
            x.z = x.z * wa + y.z * wp;
            x.w = x.w * wa + y.w * wp;
            reinterpret_cast<float4*>(O_acc)[row * 16 + sub] = x;
        }
        __syncwarp();  // every lane has read LSE_acc[row] before lane 0 overwrites it
        if (valid && sub == 0) LSE_acc[row] = lse;
    }
}

int launch_merge_partial(float* O_acc, float* LSE_acc, const float* O_part, const float* LSE_part, long long rows,
                         cudaStream_t stream) {
    if (rows == 0) return HK_OK;
    const int blocks = (int)std::min<long long>((rows * 16 + 255) / 256, 148 * 8);
    merge_partial_kernel<<<blocks, 256, 0, stream>>>(O_acc, LSE_acc, O_part, LSE_part, rows);
    count_launch();
    return check_launch();
}

}  // namespace hk
