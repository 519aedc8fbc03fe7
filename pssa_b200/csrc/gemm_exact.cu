// Y[M,N] = X[M,K] * W[N,K]^T in fp32 with the reference's per-dot reduction order.
//
// Replaces `gemm_cpu_into` / `matvec` (src/backend.rs:832-871, src/pssa.rs:109-116): every output is one
// `dot_slice` (src/linalg.rs:184-298). On an AVX2/FMA host that is 4 accumulators x 8 lanes fed with
// fused multiply-adds over 32-element strides, extra 8-element blocks into accumulator 0, a fixed
// fold ((acc0+acc1)+(acc2+acc3), high half onto low half, two horizontal adds) and a scalar tail; for
// lengths 1..7 and 9..15 it is the portable 4-accumulator loop. A warp reproduces exactly that: lane l
// owns partial sum l of the 32, the fold is the same sequence of additions done with shuffles. This is
// the verification / exact path; the throughput path for the projections is the tensor-core GEMM.
#include "bounds.hpp"
#include "context.hpp"
#include "device_math.cuh"
#include "kernels.hpp"

namespace pssa {
namespace {

constexpr int RT = 4, CT = 4;  // outputs per warp: RT rows x CT columns

__global__ void __launch_bounds__(256) gemm_xwt_exact_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                             float* out, size_t M, int N, int K, size_t ldo, int epi,
                                                             float alpha) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t row0 = ((size_t)blockIdx.x * 4 + (warp >> 1)) * RT;
    const int col0 = (blockIdx.y * 2 + (warp & 1)) * CT;
    if (row0 >= M || col0 >= N) return;
    const float* xr[RT];
    const float* wc[CT];
#pragma unroll
    for (int r = 0; r < RT; ++r) xr[r] = x + (row0 + r < M ? row0 + r : M - 1) * (size_t)K;
#pragma unroll
    for (int c = 0; c < CT; ++c) wc[c] = w + (size_t)(col0 + c < N ? col0 + c : N - 1) * K;
    float acc[RT][CT];
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int c = 0; c < CT; ++c) acc[r][c] = 0.0f;
    int i = 0;
    const unsigned full = 0xffffffffu;
    if (K == 8 || K >= 16) {  // linalg.rs:212-279
        for (; i + 32 <= K; i += 32) {
            float xa[RT], wb[CT];
#pragma unroll
            for (int r = 0; r < RT; ++r) xa[r] = __ldg(xr[r] + i + lane);
#pragma unroll
            for (int c = 0; c < CT; ++c) wb[c] = __ldg(wc[c] + i + lane);
#pragma unroll
            for (int r = 0; r < RT; ++r)
#pragma unroll
                for (int c = 0; c < CT; ++c) acc[r][c] = fmaf(xa[r], wb[c], acc[r][c]);
        }
        for (; i + 8 <= K; i += 8) {  // remaining whole vectors go to accumulator 0 (lanes 0..7)
            if (lane < 8) {
#pragma unroll
                for (int r = 0; r < RT; ++r)
#pragma unroll
                    for (int c = 0; c < CT; ++c) acc[r][c] = fmaf(__ldg(xr[r] + i + lane), __ldg(wc[c] + i + lane), acc[r][c]);
            }
        }
#pragma unroll
        for (int r = 0; r < RT; ++r)
#pragma unroll
            for (int c = 0; c < CT; ++c) {
                float v = acc[r][c];
                v = __fadd_rn(v, __shfl_down_sync(full, v, 8));   // acc0+acc1 (lanes 0-7), acc2+acc3 (lanes 16-23)
                v = __fadd_rn(v, __shfl_down_sync(full, v, 16));  // (acc0+acc1)+(acc2+acc3)
                v = __fadd_rn(v, __shfl_down_sync(full, v, 4));   // low 128 bits + high 128 bits
                v = __fadd_rn(v, __shfl_down_sync(full, v, 1));   // hadd: f0+f1, f2+f3
                v = __fadd_rn(v, __shfl_down_sync(full, v, 2));   // hadd: (f0+f1)+(f2+f3)
                acc[r][c] = v;
            }
    } else {  // linalg.rs:282-298
        for (; i + 4 <= K; i += 4) {
            if (lane < 4) {
#pragma unroll
                for (int r = 0; r < RT; ++r)
#pragma unroll
                    for (int c = 0; c < CT; ++c)
                        acc[r][c] = __fadd_rn(acc[r][c], __fmul_rn(__ldg(xr[r] + i + lane), __ldg(wc[c] + i + lane)));
            }
        }
#pragma unroll
        for (int r = 0; r < RT; ++r)
#pragma unroll
            for (int c = 0; c < CT; ++c) {
                float v = acc[r][c];
                v = __fadd_rn(v, __shfl_down_sync(full, v, 1));  // acc0+acc1, acc2+acc3
                v = __fadd_rn(v, __shfl_down_sync(full, v, 2));  // (acc0+acc1)+(acc2+acc3)
                acc[r][c] = v;
            }
    }
    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < RT; ++r)
#pragma unroll
            for (int c = 0; c < CT; ++c) {
                if (row0 + r >= M || col0 + c >= N) continue;
                float sum = acc[r][c];
                for (int t = i; t < K; ++t) sum = __fadd_rn(sum, __fmul_rn(xr[r][t], wc[c][t]));
                float* o = out + (row0 + r) * ldo + col0 + c;
                *o = apply_epilogue(epi, sum, alpha, epi == EPI_ADD_OUT ? *o : 0.0f);
            }
    }
}

}  // namespace

int32_t launch_gemm_exact(pssa_b200_ctx* ctx, const float* x, const float* w, float* out, size_t M, size_t N, size_t K,
                          size_t ldo, int epi, float alpha) {
    size_t bx = (M + 4 * RT - 1) / (4 * RT), by = (N + 2 * CT - 1) / (2 * CT);
    if (bx > 0x7fffffffull || by > 65535)
        return fail(ctx, PSSA_B200_ERR_SHAPE, "B200 GEMM grid (%zu, %zu) exceeds grid limits; refusing launch", bx, by);
    gemm_xwt_exact_kernel<<<dim3((unsigned)bx, (unsigned)by), 256, 0, ctx->stream>>>(x, w, out, M, (int)N, (int)K, ldo, epi,
                                                                                   alpha);
    return after_launch(ctx, "gemm_xwt_exact_kernel");
}

}  // namespace pssa
