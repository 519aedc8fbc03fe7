// Stage-level operators with the reference's `GpuDispatch` argument lists, so that a `GpuDispatch::B200` arm maps one
// method to one call: `memory_forward` (src/backend.rs:1342-1385), and the resident pair `ssm_forward_resident` /
// `memory_forward_after_ssm` (src/backend.rs:1186-1212, 1246-1289). They compose the library's own kernels; the CPU twin
// whose results they reproduce is `stage_memory_impl` (src/gpu_batch.rs:758-929).
#include <cmath>
#include <cstring>
#include <vector>

#include "bounds.hpp"
#include "context.hpp"
#include "kernels.hpp"

using namespace pssa;

namespace {

struct DevBuf {
    void* p = nullptr;
    ~DevBuf() {
        if (p) cudaFree(p);
    }
    cudaError_t alloc(size_t bytes) { return cudaMalloc(&p, bytes ? bytes : 1); }
    float* f() const { return (float*)p; }
};

// src/cuda/stage_bounds.rs:67-152 for the memory stage: every product must fit the u32 element index of the kernels
int32_t memory_stage_shape(pssa_b200_ctx* ctx, size_t seq_len, size_t d_m, size_t d_k, size_t d_val, size_t capacity, size_t count,
                           float tau) {
    if (d_m == 0 || d_m > 0x7fffffff) return fail(ctx, PSSA_B200_ERR_SHAPE, "B200 memory dimensions must be positive and widths fit i32; refusing launch");
    int32_t rc = memory_shape(ctx, seq_len, d_k, d_val, capacity, count, tau);
    if (rc) return rc;
    size_t e;
    return f32_elems(ctx, "memory input", {seq_len, d_m}, &e);
}

}  // namespace

extern "C" {

int32_t pssa_b200_memory_forward_dev(pssa_b200_ctx* ctx, const float* x_norm, const float* y_ssm, const float* w_qx, const float* w_qh,
                                     const float* w_gate, const float* w_proj, const float* keys, const float* norm_sq,
                                     const float* values, size_t seq_len, size_t d_m, size_t d_k, size_t d_val, size_t capacity,
                                     size_t count, float tau, float* q_euc, float* q_pnc, float* q_norm, float* weights, float* m_val,
                                     float* g_mem, float* m_proj, float* m_inj, int32_t precision) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    int32_t rc = memory_stage_shape(ctx, seq_len, d_m, d_k, d_val, capacity, count, tau);
    if (rc) return rc;
    if (!x_norm || !y_ssm || !w_qx || !w_qh || !w_gate || !w_proj || !keys || !norm_sq || !values || !q_euc || !q_pnc || !q_norm ||
        !weights || !m_val || !g_mem || !m_proj || !m_inj)
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 memory forward: null buffer");
    if (precision != PSSA_B200_PRECISION_BF16 && precision != PSSA_B200_PRECISION_FP32_EXACT)
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "unknown precision %d", precision);
    const bool exact = precision == PSSA_B200_PRECISION_FP32_EXACT;
    // q = W_qx x + W_qh y: two products, the second added onto the first (src/gpu_batch.rs:850-880)
    if ((rc = pssa_b200_gemm_xwt_dev(ctx, x_norm, w_qx, seq_len, d_k, d_m, q_euc, d_k, PSSA_B200_EPI_NONE, 1.0f, precision))) return rc;
    if ((rc = pssa_b200_gemm_xwt_dev(ctx, y_ssm, w_qh, seq_len, d_k, d_m, q_euc, d_k, PSSA_B200_EPI_ADD_OUT, 1.0f, precision))) return rc;
    // projection into the ball, distances, softmax over the occupied slots, value read (src/gpu_batch.rs:700-741)
    if ((rc = pssa_b200_memory_read_dev(ctx, q_euc, 1, keys, norm_sq, values, seq_len, d_k, d_val, capacity, count, tau, 0, q_pnc, q_norm,
                                        weights, m_val, nullptr, exact ? PSSA_B200_MEM_EXACT : 0u)))
        return rc;
    // g = sigmoid(W_gate x); m_proj = W_proj m; m_inj = g * m_proj (src/gpu_batch.rs:901-929)
    if ((rc = pssa_b200_gemm_xwt_dev(ctx, x_norm, w_gate, seq_len, d_m, d_m, g_mem, d_m, PSSA_B200_EPI_SIGMOID, 1.0f, precision))) return rc;
    if ((rc = pssa_b200_gemm_xwt_dev(ctx, m_val, w_proj, seq_len, d_m, d_val, m_proj, d_m, PSSA_B200_EPI_NONE, 1.0f, precision))) return rc;
    return launch_multiply(ctx, g_mem, m_proj, m_inj, seq_len * d_m);
}

int32_t pssa_b200_memory_forward(pssa_b200_ctx* ctx, const float* x_norm, const float* y_ssm, const float* w_qx, const float* w_qh,
                                 const float* w_gate, const float* w_proj, const float* keys, const float* norm_sq, const float* values,
                                 size_t seq_len, size_t d_m, size_t d_k, size_t d_val, size_t capacity, size_t count, float tau,
                                 float* q_euc, float* q_pnc, float* q_norm, float* weights, float* m_val, float* g_mem, float* m_proj,
                                 float* m_inj, int32_t precision) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    int32_t rc = memory_stage_shape(ctx, seq_len, d_m, d_k, d_val, capacity, count, tau);
    if (rc) return rc;
    if (!x_norm || !y_ssm || !w_qx || !w_qh || !w_gate || !w_proj || !keys || !norm_sq || !values || !q_euc || !q_pnc || !q_norm ||
        !weights || !m_val || !g_mem || !m_proj || !m_inj)
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 memory forward: null buffer");
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaStream_t st = ctx->stream;
    const size_t T = seq_len, f = sizeof(float);
    struct In { const float* host; size_t n; DevBuf buf; };
    In in[] = {{x_norm, T * d_m, {}}, {y_ssm, T * d_m, {}}, {w_qx, d_k * d_m, {}}, {w_qh, d_k * d_m, {}}, {w_gate, d_m * d_m, {}},
               {w_proj, d_m * d_val, {}}, {keys, capacity * d_k, {}}, {norm_sq, capacity, {}}, {values, capacity * d_val, {}}};
    for (auto& i : in) {
        PSSA_CUDA(ctx, i.buf.alloc(i.n * f));
        PSSA_CUDA(ctx, cudaMemcpyAsync(i.buf.p, i.host, i.n * f, cudaMemcpyHostToDevice, st));
    }
    struct Out { float* host; size_t n; DevBuf buf; };
    Out out[] = {{q_euc, T * d_k, {}}, {q_pnc, T * d_k, {}}, {q_norm, T, {}}, {weights, T * capacity, {}}, {m_val, T * d_val, {}},
                 {g_mem, T * d_m, {}}, {m_proj, T * d_m, {}}, {m_inj, T * d_m, {}}};
    for (auto& o : out) PSSA_CUDA(ctx, o.buf.alloc(o.n * f));
    PSSA_CUDA(ctx, cudaMemsetAsync(out[3].buf.p, 0, out[3].n * f, st));
    rc = pssa_b200_memory_forward_dev(ctx, in[0].buf.f(), in[1].buf.f(), in[2].buf.f(), in[3].buf.f(), in[4].buf.f(), in[5].buf.f(),
                                      in[6].buf.f(), in[7].buf.f(), in[8].buf.f(), seq_len, d_m, d_k, d_val, capacity, count, tau,
                                      out[0].buf.f(), out[1].buf.f(), out[2].buf.f(), out[3].buf.f(), out[4].buf.f(), out[5].buf.f(),
                                      out[6].buf.f(), out[7].buf.f(), precision);
    if (rc == PSSA_B200_OK) rc = pssa_b200_ctx_poll_status(ctx);  // a bounded wait that expired leaves the outputs untouched
    if (rc != PSSA_B200_OK) {
        cudaStreamSynchronize(st);
        return rc;
    }
    for (auto& o : out) PSSA_CUDA(ctx, cudaMemcpyAsync(o.host, o.buf.p, o.n * f, cudaMemcpyDeviceToHost, st));
    PSSA_CUDA(ctx, cudaStreamSynchronize(st));
    return PSSA_B200_OK;
}

int32_t pssa_b200_ssm_forward_resident(pssa_b200_ctx* ctx, const float* delta, const float* delta_raw, const float* b_proj,
                                       const float* x_norm, const float* rates, const float* c_proj, const float* initial,
                                       size_t seq_len, size_t d_m, size_t d_s, uint32_t flags) {
    (void)delta_raw;  // backward-only input of the reference's tape
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    auto& r = ctx->resident;
    r.valid = false;
    if (seq_len == 0 || d_m == 0 || d_s == 0) return fail(ctx, PSSA_B200_ERR_SHAPE, "B200 SSM dimensions must be positive; refusing launch");
    size_t stride, tape, rows_m, rows_s;
    int32_t rc;
    if ((rc = f32_elems(ctx, "SSM stride", {d_m, d_s}, &stride))) return rc;
    if ((rc = f32_elems(ctx, "SSM tape", {seq_len + 1, stride}, &tape))) return rc;
    if ((rc = f32_elems(ctx, "SSM rows", {seq_len, d_m}, &rows_m))) return rc;
    if ((rc = f32_elems(ctx, "SSM state rows", {seq_len, d_s}, &rows_s))) return rc;
    if (!delta || !b_proj || !x_norm || !rates || !c_proj || !initial) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 SSM forward: null buffer");
    if (flags & ~PSSA_B200_SSM_EXACT) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 SSM forward: unknown flags");
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaStream_t st = ctx->stream;
    if (rows_m > r.capacity_rows || tape > r.capacity_stride) {  // capacities in floats: y rows, state tape
        PSSA_CUDA(ctx, cudaStreamSynchronize(st));
        cudaFree(r.y), cudaFree(r.states), cudaFree(r.bar_a), cudaFree(r.bar_b);
        r = pssa_b200_ctx::ResidentSsm{};
        PSSA_CUDA(ctx, cudaMalloc((void**)&r.y, rows_m * 4));
        PSSA_CUDA(ctx, cudaMalloc((void**)&r.states, tape * 4));
        PSSA_CUDA(ctx, cudaMalloc((void**)&r.bar_a, seq_len * stride * 4));
        PSSA_CUDA(ctx, cudaMalloc((void**)&r.bar_b, seq_len * stride * 4));
        r.capacity_rows = rows_m, r.capacity_stride = tape;
    }
    DevBuf dd, db, dc, dx, dr;
    PSSA_CUDA(ctx, dd.alloc(rows_m * 4));
    PSSA_CUDA(ctx, dx.alloc(rows_m * 4));
    PSSA_CUDA(ctx, db.alloc(rows_s * 4));
    PSSA_CUDA(ctx, dc.alloc(rows_s * 4));
    PSSA_CUDA(ctx, dr.alloc(stride * 4));
    PSSA_CUDA(ctx, cudaMemcpyAsync(dd.p, delta, rows_m * 4, cudaMemcpyHostToDevice, st));
    PSSA_CUDA(ctx, cudaMemcpyAsync(dx.p, x_norm, rows_m * 4, cudaMemcpyHostToDevice, st));
    PSSA_CUDA(ctx, cudaMemcpyAsync(db.p, b_proj, rows_s * 4, cudaMemcpyHostToDevice, st));
    PSSA_CUDA(ctx, cudaMemcpyAsync(dc.p, c_proj, rows_s * 4, cudaMemcpyHostToDevice, st));
    PSSA_CUDA(ctx, cudaMemcpyAsync(dr.p, rates, stride * 4, cudaMemcpyHostToDevice, st));
    // states row 0 = the initial carry (src/gpu_batch.rs:392-437); rows 1.. = state after each token
    PSSA_CUDA(ctx, cudaMemcpyAsync(r.states, initial, stride * 4, cudaMemcpyHostToDevice, st));
    DevBuf carry;
    PSSA_CUDA(ctx, carry.alloc(stride * 4));
    PSSA_CUDA(ctx, cudaMemcpyAsync(carry.p, r.states, stride * 4, cudaMemcpyDeviceToDevice, st));
    rc = pssa_b200_ssm_forward_dev(ctx, dd.f(), db.f(), dc.f(), dx.f(), dr.f(), carry.f(), r.y, r.states + stride, r.bar_a, r.bar_b, nullptr,
                                   nullptr, 1, seq_len, d_m, d_s, flags);
    PSSA_CUDA(ctx, cudaStreamSynchronize(st));  // the staged inputs are freed on return
    if (rc != PSSA_B200_OK) return rc;
    r.seq_len = seq_len, r.d_m = d_m, r.d_s = d_s, r.valid = true;
    return PSSA_B200_OK;
}

int32_t pssa_b200_memory_forward_after_ssm(pssa_b200_ctx* ctx, const float* x_norm, const float* w_qx, const float* w_qh, const float* w_gate,
                                           const float* w_proj, const float* keys, const float* norm_sq, const float* values,
                                           size_t seq_len, size_t d_m, size_t d_k, size_t d_val, size_t capacity, size_t count, float tau,
                                           float* bar_a, float* bar_b, float* states, float* y_ssm, float* q_euc, float* q_pnc,
                                           float* q_norm, float* weights, float* m_val, float* g_mem, float* m_proj, float* m_inj,
                                           int32_t precision) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    auto& r = ctx->resident;
    if (!r.valid) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 SSM result is not resident");  // src/cuda/stages.rs:714
    if (r.seq_len != seq_len || r.d_m != d_m) return fail(ctx, PSSA_B200_ERR_SHAPE, "B200 resident SSM shape mismatch");  // src/cuda/stages.rs:733-735
    if (!y_ssm) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 memory forward: null buffer");
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaStream_t st = ctx->stream;
    const size_t stride = r.d_m * r.d_s;
    // publish the resident tape first: it stays recoverable even if the memory stage fails (src/cuda/stages.rs:737-771)
    std::vector<float> y_host(seq_len * d_m);
    PSSA_CUDA(ctx, cudaMemcpyAsync(y_host.data(), r.y, seq_len * d_m * 4, cudaMemcpyDeviceToHost, st));
    if (states) PSSA_CUDA(ctx, cudaMemcpyAsync(states, r.states, (seq_len + 1) * stride * 4, cudaMemcpyDeviceToHost, st));
    if (bar_a) PSSA_CUDA(ctx, cudaMemcpyAsync(bar_a, r.bar_a, seq_len * stride * 4, cudaMemcpyDeviceToHost, st));
    if (bar_b) PSSA_CUDA(ctx, cudaMemcpyAsync(bar_b, r.bar_b, seq_len * stride * 4, cudaMemcpyDeviceToHost, st));
    PSSA_CUDA(ctx, cudaStreamSynchronize(st));
    std::memcpy(y_ssm, y_host.data(), y_host.size() * 4);
    int32_t rc = pssa_b200_memory_forward(ctx, x_norm, y_ssm, w_qx, w_qh, w_gate, w_proj, keys, norm_sq, values, seq_len, d_m, d_k, d_val,
                                          capacity, count, tau, q_euc, q_pnc, q_norm, weights, m_val, g_mem, m_proj, m_inj, precision);
    if (rc == PSSA_B200_OK) r.valid = false;  // consumed
    return rc;
}

}  // extern "C"
