// Launchers implemented in the .cu files; all enqueue on ctx->stream and never synchronise.
#pragma once
#include <cstddef>
#include <cstdint>

#include "context.hpp"

namespace pssa {

// scan_affine.cu
int32_t launch_scan_states(pssa_b200_ctx* ctx, const float* a, const float* b, const float* h0, float* h, float* h_last,
                           size_t lanes, size_t len, size_t stride, int forced_chunks);
int32_t launch_scan_maps(pssa_b200_ctx* ctx, float* scan_a, float* scan_b, size_t lanes, size_t len, size_t stride,
                         int forced_chunks);

// ssm_fused.cu
struct SsmParams {
    const float* delta;    // [rows, d]  softplus already applied
    const float* x_norm;   // [rows, d]
    const float* b_proj;   // [rows, s]
    const float* c_proj;   // [rows, s]
    const float* rates;    // [d, s]     A = -softplus(raw)
    float* carry;          // [lanes, d*s] in/out, may be null (zero carry in, carry out dropped)
    float* y;              // [rows, d]
    float* states;         // optional [rows, d*s]: state after each token
    float* bar_a;          // optional [rows, d*s]
    float* bar_b;          // optional [rows, d*s]
    const uint32_t* offsets;  // per lane first row, null = one lane starting at row 0
    const uint32_t* lengths;  // per lane row count, null = rows
    size_t rows;
    int d, s, lanes;
    int aligned;           // 16-byte vector staging allowed
};
int32_t launch_ssm_fused(pssa_b200_ctx* ctx, const SsmParams& p, bool exact);

// retrieve_poincare.cu
struct RetrieveParams {
    const float* q;        // [rows, dk] Euclidean queries (projected here) or points already in the ball
    int q_is_euclidean;
    float* q_pnc;          // [rows, dk] projected queries, may be null
    float* q_norm;         // [rows] Euclidean norm of q, may be null
    const float* keys;     // [cap, dk]
    const float* norm_sq;  // [cap]
    const float* values;   // [cap, dv]
    float* weights;        // [rows, cap] distances in flight, weights on return
    float* m_val;          // [rows, dv]
    float* min_dist;       // [rows], may be null
    size_t rows;
    int dk, dv, cap, count, top_k;
    float tau;
};
int32_t launch_memory_read(pssa_b200_ctx* ctx, const RetrieveParams& p, bool exact);

}  // namespace pssa
