// Token-local stages around the dense products: embedding gather + affine RMSNorm, latent aggregation,
// depth residual, row gather, greedy argmax, fp32 -> bf16 conversion.
#include <cuda_bf16.h>

#include <cfloat>
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
                                                         __nv_bfloat16* __restrict__ x_bf16, size_t rows, int d, uint32_t vocab,
                                                         int* __restrict__ status) {
    pdl_trigger();  // the next kernel in the stream may start its prologue now ...
    pdl_wait();     // ... and this one, if launched as a dependent, waits here for its own predecessor
    extern __shared__ float sm[];  // [8 warps][d]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t row = (size_t)blockIdx.x * 8 + warp;
    if (row >= rows) return;
    uint32_t id = ids ? ids[row] : 0;
    if (id >= vocab) {  // device-resident ids cannot be checked on the host: read row 0 and raise the status word
        if (lane == 0 && status) atomicExch(status, PSSA_B200_ERR_TOKEN);
        id = 0;
    }
    const float* src = ids ? embed + (size_t)id * d : feats + row * d;
    float* buf = sm + (size_t)warp * d;
    float part = 0.0f;
    // 16-byte accesses when every row starts on a 16-byte boundary (the model's widths do)
    const bool vec = (d & 3) == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(x_norm) |
                                       reinterpret_cast<uintptr_t>(gamma) | reinterpret_cast<uintptr_t>(beta)) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(x_bf16) & 7) == 0;
    if (vec) {
#pragma unroll 2
        for (int i = lane * 4; i < d; i += 128) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(src + i));
            *reinterpret_cast<float4*>(buf + i) = v;
            part = fmaf(v.x, v.x, part), part = fmaf(v.y, v.y, part), part = fmaf(v.z, v.z, part), part = fmaf(v.w, v.w, part);
        }
    } else {
        for (int i = lane; i < d; i += 32) {
            float v = __ldg(src + i);
            buf[i] = v;
            part = fmaf(v, v, part);
        }
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
    if (vec) {
        for (int i = lane * 4; i < d; i += 128) {
            const float4 b4 = *reinterpret_cast<const float4*>(buf + i);
            const float4 g4 = __ldg(reinterpret_cast<const float4*>(gamma + i)), t4 = __ldg(reinterpret_cast<const float4*>(beta + i));
            float4 o;
            o.x = __fadd_rn(__fmul_rn(g4.x, __fmul_rn(b4.x, inv)), t4.x), o.y = __fadd_rn(__fmul_rn(g4.y, __fmul_rn(b4.y, inv)), t4.y);
            o.z = __fadd_rn(__fmul_rn(g4.z, __fmul_rn(b4.z, inv)), t4.z), o.w = __fadd_rn(__fmul_rn(g4.w, __fmul_rn(b4.w, inv)), t4.w);
            *reinterpret_cast<float4*>(x_norm + row * d + i) = o;
            if (x_bf16) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(o.x, o.y), hi = __floats2bfloat162_rn(o.z, o.w);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&lo), pk.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(x_bf16 + row * d + i) = pk;
            }
        }
        return;
    }
    for (int i = lane; i < d; i += 32) {
        float v = __fadd_rn(__fmul_rn(__ldg(gamma + i), __fmul_rn(buf[i], inv)), __ldg(beta + i));
        x_norm[row * d + i] = v;
        if (x_bf16) x_bf16[row * d + i] = __float2bfloat16_rn(v);
    }
}

// src/pssa.rs:1179-1196: ad = (U_fast + U_slow) * act (sum over r in order), z = y/sqrt(s) + g*mp + ad.
// One thread owns one channel for ROWS_PER_CTA consecutive rows: its 16 up-projection weights stay in registers,
// the 16 adapter activations of a row are one address for the whole CTA (broadcast), and y / g / m_proj / z are
// read and written as coalesced rows.
constexpr int kCombineRows = 16;
template <int RANK>
__global__ void __launch_bounds__(256) combine_zraw_kernel(const float* __restrict__ y, const float* __restrict__ g,
                                                           size_t ldg, const float* __restrict__ m_proj,
                                                           const float* __restrict__ act, size_t ldact,
                                                           const float* __restrict__ u_eff, float* __restrict__ z_raw,
                                                           __nv_bfloat16* __restrict__ z_bf16, size_t rows, int d, int rank,
                                                           float ssm_scale) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const size_t row0 = (size_t)blockIdx.y * kCombineRows;
    if (i >= d) return;
    float u[RANK > 0 ? RANK : 1];
    if (RANK > 0) {
#pragma unroll
        for (int r = 0; r < RANK; ++r) u[r] = __ldg(u_eff + (size_t)i * RANK + r);
    }
    // rows in groups of four: all global loads of a group are issued before any arithmetic
    for (int r0 = 0; r0 < kCombineRows; r0 += 4) {
        float yv[4], gv[4], mv[4];
        size_t rowv[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            size_t row = row0 + r0 + q;
            rowv[q] = row < rows ? row : rows - 1;  // clamped for the loads; stores are predicated
            yv[q] = y[rowv[q] * d + i];
            gv[q] = g[rowv[q] * ldg + i];
            mv[q] = m_proj[rowv[q] * d + i];
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float* a = act + rowv[q] * ldact;
            float ad = 0.0f;
            if (RANK > 0) {
#pragma unroll
                for (int r = 0; r < RANK; ++r) ad = __fadd_rn(ad, __fmul_rn(u[r], __ldg(a + r)));
            } else {
                for (int r = 0; r < rank; ++r) ad = __fadd_rn(ad, __fmul_rn(__ldg(u_eff + (size_t)i * rank + r), __ldg(a + r)));
            }
            float z = __fadd_rn(__fadd_rn(__fmul_rn(yv[q], ssm_scale), __fmul_rn(gv[q], mv[q])), ad);
            if (row0 + r0 + q < rows) {
                const size_t idx = rowv[q] * d + i;
                z_raw[idx] = z;
                if (z_bf16) z_bf16[idx] = __float2bfloat16_rn(z);
            }
        }
    }
}

// src/pssa.rs:2332-2337: features += scale * block_out  (prev == nullptr: features = z, block 0)
__global__ void __launch_bounds__(256) residual_kernel(const float* __restrict__ prev, const float* __restrict__ z,
                                                       float* __restrict__ out, size_t n, float scale) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    out[idx] = prev ? __fadd_rn(prev[idx], __fmul_rn(scale, z[idx])) : z[idx];
}

// m_inj = g_mem * m_proj (the reference's `sigmoid_mul`, src/cuda/stages.ptx:565-571: a plain product, the gate is
// already a sigmoid)
__global__ void __launch_bounds__(256) multiply_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                                                       size_t n) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n) out[idx] = __fmul_rn(a[idx], b[idx]);
}

// src_rows != 0: indices come from the caller's device memory and are checked here; an index outside the table reads row 0
// and raises PSSA_B200_ERR_TOKEN in the status word (the rule of the embedding kernel)
__global__ void __launch_bounds__(256) gather_rows_kernel(const float* __restrict__ src, const uint32_t* __restrict__ rows_idx,
                                                          float* __restrict__ dst, __nv_bfloat16* __restrict__ dst16, size_t n_rows, int d,
                                                          size_t src_rows, int* status) {
    pdl_trigger();  // the next kernel in the stream may start its prologue now ...
    pdl_wait();     // ... and this one, if launched as a dependent, waits here for its own predecessor
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_rows * (size_t)d) return;
    size_t r = idx / d;
    size_t row = rows_idx[r];
    if (src_rows != 0 && row >= src_rows) {
        if (status && idx % d == 0) atomicExch(status, PSSA_B200_ERR_TOKEN);
        row = 0;
    }
    const float v = src[row * d + idx % d];
    if (dst) dst[idx] = v;
    if (dst16) dst16[idx] = __float2bfloat16_rn(v);  // the tensor-core head reads the gathered rows as bf16 only
}

__global__ void __launch_bounds__(256) to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t n) {
    pdl_trigger();  // the next kernel in the stream may start its prologue now ...
    pdl_wait();     // ... and this one, if launched as a dependent, waits here for its own predecessor
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n) dst[idx] = __float2bfloat16_rn(src[idx]);
}

// src/inference.rs:111-127: argmax over ids 1..V-1 under total_cmp, ties to the lowest id; a non-finite
// logit anywhere in the row is an error (id = UINT32_MAX). One CTA per row.
__device__ __forceinline__ int total_order_key(float v) {
    int b = __float_as_int(v);
    return b < 0 ? (b ^ 0x7fffffff) : b;  // monotone signed key of f32::total_cmp
}
__global__ void __launch_bounds__(256) greedy_kernel(const float* __restrict__ logits, uint32_t* __restrict__ out, size_t rows,
                                                     int v) {
    pdl_trigger();  // the next kernel in the stream may start its prologue now ...
    pdl_wait();     // ... and this one, if launched as a dependent, waits here for its own predecessor
    __shared__ long long s_best[8];
    __shared__ int s_bad[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t row = blockIdx.x;
    const float* lg = logits + row * v;
    long long best = LLONG_MIN;  // (key << 32) | (UINT32_MAX - id): larger is better, lower id wins ties
    bool bad = false;
    auto take = [&](float x, int i) {
        if (!isfinite(x)) bad = true;
        if (i >= 1) {
            long long k = ((long long)total_order_key(x) << 32) | (unsigned)(0xffffffffu - (unsigned)i);
            best = k > best ? k : best;
        }
    };
    if ((v & 3) == 0 && (reinterpret_cast<uintptr_t>(lg) & 15) == 0) {
        for (int i = threadIdx.x * 4; i < v; i += 256 * 4) {
            const float4 x = *reinterpret_cast<const float4*>(lg + i);
            take(x.x, i), take(x.y, i + 1), take(x.z, i + 2), take(x.w, i + 3);
        }
    } else {
        for (int i = threadIdx.x; i < v; i += 256) take(lg[i], i);
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        long long o = __shfl_xor_sync(0xffffffffu, best, m);
        best = o > best ? o : best;
        bad = bad || __shfl_xor_sync(0xffffffffu, (int)bad, m);
    }
    if (lane == 0) s_best[warp] = best, s_bad[warp] = bad;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) {
            best = s_best[w] > best ? s_best[w] : best;
            bad = bad || s_bad[w];
        }
        out[row] = (bad || v < 2) ? 0xffffffffu : 0xffffffffu - (unsigned)(best & 0xffffffffll);
    }
}

// Observer scratch: copy the last row of each lane out of the block's working buffers into
// out[lane] = { weights[cap] | q_pnc[k] | m_val[d] | z_final[d] }. z_final is the block's output before the depth
// residual (src/pssa.rs:1205-1207): z_direct when the caller has it, else (feat_out - feat_in) / scale.
__global__ void __launch_bounds__(256) observe_rows_kernel(const uint32_t* __restrict__ last_rows, const float* __restrict__ weights,
                                                           int cap, const float* __restrict__ q_pnc, int k,
                                                           const float* __restrict__ m_val, const float* __restrict__ z_direct,
                                                           const float* __restrict__ feat_out, const float* __restrict__ feat_in,
                                                           float inv_scale, int d, float* __restrict__ out) {
    const int lane = blockIdx.x;
    const size_t row = last_rows[lane];
    float* o = out + (size_t)lane * (cap + k + 2 * d);
    for (int i = threadIdx.x; i < cap; i += blockDim.x) o[i] = weights[row * cap + i];
    for (int i = threadIdx.x; i < k; i += blockDim.x) o[cap + i] = q_pnc[row * k + i];
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        o[cap + k + i] = m_val[row * d + i];
        float z;
        if (z_direct)
            z = z_direct[row * d + i];
        else if (feat_in)
            z = __fmul_rn(__fsub_rn(feat_out[row * d + i], feat_in[row * d + i]), inv_scale);
        else
            z = feat_out[row * d + i];  // block 0: its output is F0(embed), no residual
        o[cap + k + d + i] = z;
    }
}

// bf16 weight rows with the adapter block appended: dst [n, k + 64] = bf16(src [n, k]) | bf16(tail [n, 16]) | 48 zeros
__global__ void __launch_bounds__(256) pack_weight_cat_kernel(const float* __restrict__ src, const float* __restrict__ tail,
                                                              __nv_bfloat16* __restrict__ dst, size_t n, int k) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int ld = k + 64;
    if (idx >= n * (size_t)ld) return;
    const size_t r = idx / ld;
    const int c = (int)(idx % ld);
    float v = c < k ? src[r * k + c] : (c < k + 16 ? tail[r * 16 + (c - k)] : 0.0f);
    dst[idx] = __float2bfloat16_rn(v);
}

// out [n, 16] = w [n, k] x u [k, 16]  (the adapter's up projection seen through the MLP's first matrix)
__global__ void __launch_bounds__(256) times_adapter_kernel(const float* __restrict__ w, const float* __restrict__ u,
                                                            float* __restrict__ out, size_t n, int k) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n * 16) return;
    const size_t r = idx >> 4;
    const int c = (int)(idx & 15);
    float acc = 0.0f;
    for (int i = 0; i < k; ++i) acc = fmaf(w[r * k + i], u[(size_t)i * 16 + c], acc);
    out[idx] = acc;
}

// Cross entropy of one logits row against its target (src/pssa.rs:2597-2750, the scorer's per-row loss):
// loss = (max - l[target]) + ln(sum exp(l - max)). One CTA per row; a non-finite row or a target outside the
// vocabulary gives NaN, which the host reports.
__global__ void __launch_bounds__(256) cross_entropy_kernel(const float* __restrict__ logits, const uint32_t* __restrict__ targets,
                                                            float* __restrict__ loss, int v) {
    __shared__ float s_red[256];
    const size_t row = blockIdx.x;
    const float* lg = logits + row * (size_t)v;
    float mx = -FLT_MAX;
    for (int i = threadIdx.x; i < v; i += 256) mx = fmaxf(mx, lg[i]);
    s_red[threadIdx.x] = mx;
    __syncthreads();
    for (int w = 128; w > 0; w >>= 1) {
        if (threadIdx.x < w) s_red[threadIdx.x] = fmaxf(s_red[threadIdx.x], s_red[threadIdx.x + w]);
        __syncthreads();
    }
    mx = s_red[0];
    __syncthreads();
    float part = 0.0f;
    for (int i = threadIdx.x; i < v; i += 256) part += expf(__fsub_rn(lg[i], mx));
    s_red[threadIdx.x] = part;
    __syncthreads();
    for (int w = 128; w > 0; w >>= 1) {
        if (threadIdx.x < w) s_red[threadIdx.x] += s_red[threadIdx.x + w];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const uint32_t t = targets[row];
        loss[row] = t < (uint32_t)v ? __fadd_rn(__fsub_rn(mx, lg[t]), logf(s_red[0])) : __int_as_float(0x7fc00000);
    }
}

inline unsigned blocks_for(size_t n, int threads) { return (unsigned)((n + threads - 1) / threads); }

}  // namespace

int32_t launch_embed_norm(pssa_b200_ctx* ctx, const float* embed, const uint32_t* ids, const float* feats, const float* gamma,
                          const float* beta, float* x_norm, void* x_bf16, size_t rows, int d, bool exact, size_t vocab) {
    size_t smem = (size_t)8 * d * sizeof(float);
    if (smem > 200 * 1024)
        return fail(ctx, PSSA_B200_ERR_UNSUPPORTED, "B200 norm: latent width %d exceeds one CTA's shared memory; refusing launch", d);
    static PerDeviceOnce attr[2];
    if (smem > 48 * 1024 && attr[exact].need(ctx->device)) {
        if (exact)
            PSSA_CUDA(ctx, cudaFuncSetAttribute(embed_norm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        else
            PSSA_CUDA(ctx, cudaFuncSetAttribute(embed_norm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr[exact].done(ctx->device);
    }
    unsigned blocks = blocks_for(rows, 8);
    if (exact)
        PSSA_CUDA(ctx, launch_dependent(embed_norm_kernel<true>, dim3(blocks), dim3(256), smem, ctx->stream, embed, ids, feats, gamma, beta,
                                        x_norm, (__nv_bfloat16*)x_bf16, rows, d, (uint32_t)vocab, ctx->status_dev));
    else
        PSSA_CUDA(ctx, launch_dependent(embed_norm_kernel<false>, dim3(blocks), dim3(256), smem, ctx->stream, embed, ids, feats, gamma, beta,
                                        x_norm, (__nv_bfloat16*)x_bf16, rows, d, (uint32_t)vocab, ctx->status_dev));
    return after_launch(ctx, "embed_norm_kernel");
}

int32_t launch_combine_zraw(pssa_b200_ctx* ctx, const float* y, const float* g, size_t ldg, const float* m_proj, const float* act,
                            size_t ldact, const float* u_eff, float* z_raw, void* z_bf16, size_t rows, int d, int rank,
                            float ssm_scale) {
    dim3 grid((unsigned)((d + 255) / 256), (unsigned)((rows + kCombineRows - 1) / kCombineRows));
    if (grid.y > 65535) {
        // very long passes: fall back to several launches of at most 65535 row groups
        size_t step = (size_t)65535 * kCombineRows;
        for (size_t r0 = 0; r0 < rows; r0 += step) {
            size_t n = rows - r0 < step ? rows - r0 : step;
            int32_t rc = launch_combine_zraw(ctx, y + r0 * d, g + r0 * ldg, ldg, m_proj + r0 * d, act + r0 * ldact, ldact, u_eff,
                                             z_raw + r0 * d, z_bf16 ? (char*)z_bf16 + r0 * d * 2 : nullptr, n, d, rank, ssm_scale);
            if (rc) return rc;
        }
        return PSSA_B200_OK;
    }
    if (rank == 16)
        combine_zraw_kernel<16><<<grid, 256, 0, ctx->stream>>>(y, g, ldg, m_proj, act, ldact, u_eff, z_raw, (__nv_bfloat16*)z_bf16,
                                                             rows, d, rank, ssm_scale);
    else
        combine_zraw_kernel<0><<<grid, 256, 0, ctx->stream>>>(y, g, ldg, m_proj, act, ldact, u_eff, z_raw, (__nv_bfloat16*)z_bf16,
                                                            rows, d, rank, ssm_scale);
    return after_launch(ctx, "combine_zraw_kernel");
}

int32_t launch_residual(pssa_b200_ctx* ctx, const float* prev, const float* z, float* out, size_t n, float scale) {
    residual_kernel<<<blocks_for(n, 256), 256, 0, ctx->stream>>>(prev, z, out, n, scale);
    return after_launch(ctx, "residual_kernel");
}

int32_t launch_multiply(pssa_b200_ctx* ctx, const float* a, const float* b, float* out, size_t n) {
    multiply_kernel<<<blocks_for(n, 256), 256, 0, ctx->stream>>>(a, b, out, n);
    return after_launch(ctx, "multiply_kernel");
}

int32_t launch_gather_rows(pssa_b200_ctx* ctx, const float* src, const uint32_t* rows_idx, float* dst, size_t n_rows, int d, size_t src_rows,
                           void* dst_bf16) {
    PSSA_CUDA(ctx, launch_dependent(gather_rows_kernel, dim3(blocks_for(n_rows * (size_t)d, 256)), dim3(256), 0, ctx->stream, src, rows_idx, dst,
                                    (__nv_bfloat16*)dst_bf16, n_rows, d, src_rows, ctx->status_dev));
    return after_launch(ctx, "gather_rows_kernel");
}

int32_t launch_to_bf16(pssa_b200_ctx* ctx, const float* src, void* dst, size_t n) {
    PSSA_CUDA(ctx, launch_dependent(to_bf16_kernel, dim3(blocks_for(n, 256)), dim3(256), 0, ctx->stream, src, (__nv_bfloat16*)dst, n));
    return after_launch(ctx, "to_bf16_kernel");
}

int32_t launch_observe_rows(pssa_b200_ctx* ctx, const uint32_t* last_rows, size_t lanes, const float* weights, int cap, const float* q_pnc,
                            int k, const float* m_val, const float* z_direct, const float* feat_out, const float* feat_in, float scale,
                            int d, float* out) {
    if (lanes == 0) return PSSA_B200_OK;
    observe_rows_kernel<<<(unsigned)lanes, 256, 0, ctx->stream>>>(last_rows, weights, cap, q_pnc, k, m_val, z_direct, feat_out, feat_in,
                                                                 scale != 0.0f ? 1.0f / scale : 0.0f, d, out);
    return after_launch(ctx, "observe_rows_kernel");
}

int32_t launch_pack_weight_cat(pssa_b200_ctx* ctx, const float* src, const float* tail, void* dst, size_t n, int k) {
    pack_weight_cat_kernel<<<blocks_for(n * (size_t)(k + 64), 256), 256, 0, ctx->stream>>>(src, tail, (__nv_bfloat16*)dst, n, k);
    return after_launch(ctx, "pack_weight_cat_kernel");
}

int32_t launch_times_adapter(pssa_b200_ctx* ctx, const float* w, const float* u, float* out, size_t n, int k) {
    times_adapter_kernel<<<blocks_for(n * 16, 256), 256, 0, ctx->stream>>>(w, u, out, n, k);
    return after_launch(ctx, "times_adapter_kernel");
}

int32_t launch_cross_entropy(pssa_b200_ctx* ctx, const float* logits, const uint32_t* targets, float* loss, size_t rows, int v) {
    if (rows == 0) return PSSA_B200_OK;
    if (rows > 0x7fffffffull) return fail(ctx, PSSA_B200_ERR_SHAPE, "cross entropy: %zu rows exceed grid limits; refusing launch", rows);
    cross_entropy_kernel<<<(unsigned)rows, 256, 0, ctx->stream>>>(logits, targets, loss, v);
    return after_launch(ctx, "cross_entropy_kernel");
}

int32_t launch_greedy(pssa_b200_ctx* ctx, const float* logits, uint32_t* out, size_t rows, int v) {
    if (rows > 0x7fffffffull) return fail(ctx, PSSA_B200_ERR_SHAPE, "greedy: %zu rows exceed grid limits; refusing launch", rows);
    PSSA_CUDA(ctx, launch_dependent(greedy_kernel, dim3((unsigned)rows), dim3(256), 0, ctx->stream, logits, out, rows, v));
    return after_launch(ctx, "greedy_kernel");
}

}  // namespace pssa
