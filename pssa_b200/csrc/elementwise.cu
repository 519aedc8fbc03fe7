// Token-local stages around the dense products: embedding gather + affine RMSNorm, latent aggregation,
// depth residual, row gather, greedy argmax, fp32 -> bf16 conversion.
#include <cuda_bf16.h>

#include <climits>

#include "context.hpp"
#include "device_math.cuh"
#include "kernels.hpp"

namespace pssa {
namespace {

// One warp per row. src row = embed[ids[row]] (block 0) or feats[row] (deeper blocks).
// src/pssa.rs:1078-1086 / src/gpu_batch.rs:445-472: sum of squares is a sequential scalar f32 sum,
// inv = 1/sqrt(sum/d + 1e-5), x = gamma*(e*inv) + beta.
template <bool EXACT>
__global__ void __launch_bounds__(256) embed_norm_kernel(const float* __restrict__ embed, const uint32_t* __restrict__ ids,
                                                         const float* __restrict__ feats, const float* __restrict__ gamma,
                                                         const float* __restrict__ beta, float* __restrict__ x_norm,
                                                         __nv_bfloat16* __restrict__ x_bf16, size_t rows, int d) {
    extern __shared__ float sm[];  // [8 warps][d]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t row = (size_t)blockIdx.x * 8 + warp;
    if (row >= rows) return;
    const float* src = ids ? embed + (size_t)ids[row] * d : feats + row * d;
    float* buf = sm + (size_t)warp * d;
    float part = 0.0f;
    for (int i = lane; i < d; i += 32) {
        float v = __ldg(src + i);
        buf[i] = v;
        part = fmaf(v, v, part);
    }
    float sum;
    if (EXACT) {
        __syncwarp();
        sum = 0.0f;
        if (lane == 0)
            for (int i = 0; i < d; ++i) sum = __fadd_rn(sum, __fmul_rn(buf[i], buf[i]));
        sum = __shfl_sync(0xffffffffu, sum, 0);
    } else {
        sum = part;
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
    }
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum, (float)d), 1e-5f)));
    for (int i = lane; i < d; i += 32) {
        float v = __fadd_rn(__fmul_rn(__ldg(gamma + i), __fmul_rn(buf[i], inv)), __ldg(beta + i));
        x_norm[row * d + i] = v;
        if (x_bf16) x_bf16[row * d + i] = __float2bfloat16_rn(v);
    }
}

// src/pssa.rs:1179-1196: ad = (U_fast + U_slow) * act (sum over r in order), z = y/sqrt(s) + g*mp + ad.
// One thread per (row, channel); the 16 adapter activations of a row are the same address for a whole warp
// (broadcast), the 16 up-projection weights of a channel are four float4 loads.
__global__ void __launch_bounds__(256) combine_zraw_kernel(const float* __restrict__ y, const float* __restrict__ g,
                                                           size_t ldg, const float* __restrict__ m_proj,
                                                           const float* __restrict__ act, size_t ldact,
                                                           const float* __restrict__ u_eff, float* __restrict__ z_raw,
                                                           __nv_bfloat16* __restrict__ z_bf16, size_t rows, int d, int rank,
                                                           float ssm_scale, int vec) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * (size_t)d) return;
    size_t row = idx / d;
    int i = (int)(idx % d);
    float ad = 0.0f;
    const float* u = u_eff + (size_t)i * rank;
    const float* a = act + row * ldact;
    if (vec) {  // rank % 4 == 0 and 16-byte aligned rows
        for (int r = 0; r < rank; r += 4) {
            float4 uv = __ldg(reinterpret_cast<const float4*>(u + r));
            float4 av = __ldg(reinterpret_cast<const float4*>(a + r));
            ad = __fadd_rn(ad, __fmul_rn(uv.x, av.x));
            ad = __fadd_rn(ad, __fmul_rn(uv.y, av.y));
            ad = __fadd_rn(ad, __fmul_rn(uv.z, av.z));
            ad = __fadd_rn(ad, __fmul_rn(uv.w, av.w));
        }
    } else {
        for (int r = 0; r < rank; ++r) ad = __fadd_rn(ad, __fmul_rn(__ldg(u + r), __ldg(a + r)));
    }
    float z = __fadd_rn(__fadd_rn(__fmul_rn(y[idx], ssm_scale), __fmul_rn(g[row * ldg + i], m_proj[idx])), ad);
    z_raw[idx] = z;
    if (z_bf16) z_bf16[idx] = __float2bfloat16_rn(z);
}

// src/pssa.rs:2332-2337: features += scale * block_out  (prev == nullptr: features = z, block 0)
__global__ void __launch_bounds__(256) residual_kernel(const float* __restrict__ prev, const float* __restrict__ z,
                                                       float* __restrict__ out, size_t n, float scale) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    out[idx] = prev ? __fadd_rn(prev[idx], __fmul_rn(scale, z[idx])) : z[idx];
}

__global__ void __launch_bounds__(256) gather_rows_kernel(const float* __restrict__ src, const uint32_t* __restrict__ rows_idx,
                                                          float* __restrict__ dst, size_t n_rows, int d) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_rows * (size_t)d) return;
    size_t r = idx / d;
    dst[idx] = src[(size_t)rows_idx[r] * d + idx % d];
}

__global__ void __launch_bounds__(256) to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t n) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n) dst[idx] = __float2bfloat16_rn(src[idx]);
}

// src/inference.rs:111-127: argmax over ids 1..V-1 under total_cmp, ties to the lowest id; a non-finite
// logit anywhere in the row is an error (id = UINT32_MAX). One warp per row.
__device__ __forceinline__ int total_order_key(float v) {
    int b = __float_as_int(v);
    return b < 0 ? (b ^ 0x7fffffff) : b;  // monotone signed key of f32::total_cmp
}
__global__ void __launch_bounds__(256) greedy_kernel(const float* __restrict__ logits, uint32_t* __restrict__ out, size_t rows,
                                                     int v) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t row = (size_t)blockIdx.x * 8 + warp;
    if (row >= rows) return;
    const float* lg = logits + row * v;
    long long best = LLONG_MIN;  // (key << 32) | (UINT32_MAX - id): larger is better, lower id wins ties
    bool bad = false;
    for (int i = lane; i < v; i += 32) {
        float x = lg[i];
        if (!isfinite(x)) bad = true;
        if (i >= 1) {
            long long k = ((long long)total_order_key(x) << 32) | (unsigned)(0xffffffffu - (unsigned)i);
            best = k > best ? k : best;
        }
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        long long o = __shfl_xor_sync(0xffffffffu, best, m);
        best = o > best ? o : best;
        bad = bad || __shfl_xor_sync(0xffffffffu, (int)bad, m);
    }
    if (lane == 0) out[row] = (bad || v < 2) ? 0xffffffffu : 0xffffffffu - (unsigned)(best & 0xffffffffll);
}

inline unsigned blocks_for(size_t n, int threads) { return (unsigned)((n + threads - 1) / threads); }

}  // namespace

int32_t launch_embed_norm(pssa_b200_ctx* ctx, const float* embed, const uint32_t* ids, const float* feats, const float* gamma,
                          const float* beta, float* x_norm, void* x_bf16, size_t rows, int d, bool exact) {
    size_t smem = (size_t)8 * d * sizeof(float);
    if (smem > 200 * 1024)
        return fail(ctx, PSSA_B200_ERR_UNSUPPORTED, "B200 norm: latent width %d exceeds one CTA's shared memory; refusing launch", d);
    static bool attr[2] = {false, false};
    if (smem > 48 * 1024 && !attr[exact]) {
        if (exact)
            PSSA_CUDA(ctx, cudaFuncSetAttribute(embed_norm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        else
            PSSA_CUDA(ctx, cudaFuncSetAttribute(embed_norm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr[exact] = true;
    }
    unsigned blocks = blocks_for(rows, 8);
    if (exact)
        embed_norm_kernel<true><<<blocks, 256, smem, ctx->stream>>>(embed, ids, feats, gamma, beta, x_norm, (__nv_bfloat16*)x_bf16, rows, d);
    else
        embed_norm_kernel<false><<<blocks, 256, smem, ctx->stream>>>(embed, ids, feats, gamma, beta, x_norm, (__nv_bfloat16*)x_bf16, rows, d);
    return after_launch(ctx, "embed_norm_kernel");
}

int32_t launch_combine_zraw(pssa_b200_ctx* ctx, const float* y, const float* g, size_t ldg, const float* m_proj, const float* act,
                            size_t ldact, const float* u_eff, float* z_raw, void* z_bf16, size_t rows, int d, int rank,
                            float ssm_scale) {
    int vec = rank % 4 == 0 && ldact % 4 == 0 && ((reinterpret_cast<uintptr_t>(act) | reinterpret_cast<uintptr_t>(u_eff)) & 15) == 0;
    combine_zraw_kernel<<<blocks_for(rows * (size_t)d, 256), 256, 0, ctx->stream>>>(y, g, ldg, m_proj, act, ldact, u_eff, z_raw,
                                                                                 (__nv_bfloat16*)z_bf16, rows, d, rank, ssm_scale, vec);
    return after_launch(ctx, "combine_zraw_kernel");
}

int32_t launch_residual(pssa_b200_ctx* ctx, const float* prev, const float* z, float* out, size_t n, float scale) {
    residual_kernel<<<blocks_for(n, 256), 256, 0, ctx->stream>>>(prev, z, out, n, scale);
    return after_launch(ctx, "residual_kernel");
}

int32_t launch_gather_rows(pssa_b200_ctx* ctx, const float* src, const uint32_t* rows_idx, float* dst, size_t n_rows, int d) {
    gather_rows_kernel<<<blocks_for(n_rows * (size_t)d, 256), 256, 0, ctx->stream>>>(src, rows_idx, dst, n_rows, d);
    return after_launch(ctx, "gather_rows_kernel");
}

int32_t launch_to_bf16(pssa_b200_ctx* ctx, const float* src, void* dst, size_t n) {
    to_bf16_kernel<<<blocks_for(n, 256), 256, 0, ctx->stream>>>(src, (__nv_bfloat16*)dst, n);
    return after_launch(ctx, "to_bf16_kernel");
}

int32_t launch_greedy(pssa_b200_ctx* ctx, const float* logits, uint32_t* out, size_t rows, int v) {
    greedy_kernel<<<blocks_for(rows, 8), 256, 0, ctx->stream>>>(logits, out, rows, v);
    return after_launch(ctx, "greedy_kernel");
}

}  // namespace pssa
