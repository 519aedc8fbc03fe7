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

}  // namespace pssa
