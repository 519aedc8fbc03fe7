// Driver-free shape validation run before any allocation or launch.
// Same role and wording as the reference's src/cuda/stage_bounds.rs:5-65 ("refusing launch"),
// with this library's limits: element counts are indexed with 64-bit offsets on the device, so the
// only caps are size_t products and a byte size that fits isize.
#pragma once
#include <cstddef>
#include <cstdint>

#include "context.hpp"

namespace pssa {

inline bool checked_mul(size_t a, size_t b, size_t* out) {
    if (a != 0 && b > SIZE_MAX / a) return false;
    *out = a * b;
    return true;
}

// product of dims as an f32 element count whose byte size fits isize (stage_bounds.rs:5-30)
inline int32_t f32_elems(pssa_b200_ctx* ctx, const char* what, std::initializer_list<size_t> dims, size_t* out) {
    size_t n = 1;
    for (size_t d : dims)
        if (!checked_mul(n, d, &n))
            return fail(ctx, PSSA_B200_ERR_SHAPE, "B200 %s: size overflow; refusing launch", what);
    if (n > (size_t)INTPTR_MAX / 4)
        return fail(ctx, PSSA_B200_ERR_SHAPE, "B200 %s: f32 allocation byte size overflow; refusing launch", what);
    *out = n;
    return PSSA_B200_OK;
}

// stage_bounds.rs:45-65
inline int32_t scan_shape(pssa_b200_ctx* ctx, size_t lanes, size_t len, size_t stride, size_t* elems) {
    if (lanes == 0 || len == 0 || stride == 0)
        return fail(ctx, PSSA_B200_ERR_SHAPE, "B200 affine scan dimensions must be positive; refusing launch");
    return f32_elems(ctx, "affine scan elements", {lanes, len, stride}, elems);
}

// stage_bounds.rs:67-105 (SsmShape::new)
struct SsmShape {
    size_t stride, token_m, token_s, token_state;
};
inline int32_t ssm_shape(pssa_b200_ctx* ctx, size_t rows, size_t dm, size_t ds, SsmShape* out) {
    if (rows == 0 || dm == 0 || ds == 0)
        return fail(ctx, PSSA_B200_ERR_SHAPE, "B200 SSM dimensions must be positive; refusing launch");
    if (dm > 0x7fffffff || ds > 0x7fffffff)
        return fail(ctx, PSSA_B200_ERR_SHAPE, "B200 SSM widths must fit i32; refusing launch");
    int32_t rc;
    if ((rc = f32_elems(ctx, "SSM stride", {dm, ds}, &out->stride))) return rc;
    if ((rc = f32_elems(ctx, "SSM latent tape", {rows, dm}, &out->token_m))) return rc;
    if ((rc = f32_elems(ctx, "SSM projection tape", {rows, ds}, &out->token_s))) return rc;
    if ((rc = f32_elems(ctx, "SSM state maps", {rows + 1, out->stride}, &out->token_state))) return rc;
    return PSSA_B200_OK;
}

// stage_bounds.rs:107-152 (MemoryShape::new), for the read alone
inline int32_t memory_shape(pssa_b200_ctx* ctx, size_t rows, size_t dk, size_t dv, size_t cap, size_t count, float tau) {
    if (rows == 0 || cap == 0 || dk == 0 || dv == 0 || dk > 0x7fffffff || dv > 0x7fffffff || cap > 0x7fffffff)
        return fail(ctx, PSSA_B200_ERR_SHAPE, "B200 memory dimensions must be positive and widths fit i32; refusing launch");
    if (count > cap || !(tau > 0.0f) || !(tau <= 3.4028234e38f))
        return fail(ctx, PSSA_B200_ERR_SHAPE,
                    "B200 memory invalid count/capacity (%zu/%zu) or temperature (%g); refusing launch", count, cap, (double)tau);
    size_t n;
    int32_t rc;
    if ((rc = f32_elems(ctx, "memory query", {rows, dk}, &n))) return rc;
    if ((rc = f32_elems(ctx, "memory value", {rows, dv}, &n))) return rc;
    if ((rc = f32_elems(ctx, "memory weights", {rows, cap}, &n))) return rc;
    if ((rc = f32_elems(ctx, "memory keys", {cap, dk}, &n))) return rc;
    if ((rc = f32_elems(ctx, "memory bank values", {cap, dv}, &n))) return rc;
    return PSSA_B200_OK;
}

}  // namespace pssa
