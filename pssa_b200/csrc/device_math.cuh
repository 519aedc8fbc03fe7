// Scalar device functions shared by the kernels: the reference's activation formulas
// (src/linalg.rs:547-555) with every operation separately rounded.
#pragma once
#include <cuda_runtime.h>

namespace pssa {

__device__ __forceinline__ float ref_sigmoid(float x) {  // 1 / (1 + exp(-x))
    return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x)));
}
__device__ __forceinline__ float ref_softplus(float x) {  // x > 20 ? x : ln_1p(exp(x))
    return x > 20.0f ? x : log1pf(expf(x));
}
__device__ __forceinline__ float ref_silu(float h) { return __fmul_rn(h, ref_sigmoid(h)); }

enum Epilogue : int {
    EPI_NONE = 0,
    EPI_SOFTPLUS = 1,
    EPI_SIGMOID = 2,
    EPI_SILU = 3,
    EPI_SCALE = 4,    // out = acc * alpha
    EPI_ADD_OUT = 5,  // out = out + acc   (second half of q = Wqx x + Wqh y; residual adds)
    EPI_RESIDUAL = 6, // tensor-core path only: acc + add_in, then the depth residual (see gemm_tcgen05.cu)
    EPI_GATE = 7,     // tensor-core path only: res_in * acc + alpha * add_in  (gated memory projection + scaled SSM output)
    EPI_POINCARE = 8, // tensor-core path only: acc = p.k; out = Poincare distance from |p|^2 + |k|^2 - 2 acc (see gemm_tcgen05.cu)
};

__device__ __forceinline__ float apply_epilogue(int epi, float acc, float alpha, float prev) {
    switch (epi) {
        case EPI_SOFTPLUS: return ref_softplus(acc);
        case EPI_SIGMOID: return ref_sigmoid(acc);
        case EPI_SILU: return ref_silu(acc);
        case EPI_SCALE: return __fmul_rn(acc, alpha);
        case EPI_ADD_OUT: return __fadd_rn(prev, acc);
        default: return acc;
    }
}

// 2*asinh(sqrt(u)) = log1p(z), z = 2u + 2*sqrt(u*u + u), with the hardware sqrt / log2 / reciprocal approximations:
// log1p(z) = log(w) + (z - (w - 1))/w for w = fl(1 + z). lg2.approx is within 2^-22 absolute near one, 2^-22 relative
// elsewhere, so the distance is good to about 2e-7 absolute near zero and 3e-7 relative beyond.
__device__ __forceinline__ float fast_poincare_distance(float u) {
    float r, lg, rc;
    const float t = fmaf(u, u, u);
    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(t));
    const float z = 2.0f * u + 2.0f * r;
    const float w = 1.0f + z;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(lg) : "f"(w));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rc) : "f"(w));
    return fmaf(lg, 0.69314718055994531f, (z - (w - 1.0f)) * rc);
}

}  // namespace pssa
