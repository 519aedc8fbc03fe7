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

}  // namespace pssa
