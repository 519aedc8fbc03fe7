// extern "C" entry points: context lifecycle, validation, host staging. Kernels live in the other .cu files.
#include <cstring>

#include "bounds.hpp"
#include "context.hpp"
#include "kernels.hpp"

namespace pssa {
thread_local std::string g_create_error;

int32_t arena_reserve(pssa_b200_ctx* ctx, size_t bytes) {
    if (bytes <= ctx->arena_bytes) return PSSA_B200_OK;
    // growing invalidates earlier carve-outs: callers reserve their total before taking blocks
    if (ctx->arena) {
        PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        PSSA_CUDA(ctx, cudaFree(ctx->arena));
        ctx->arena = nullptr;
        ctx->arena_bytes = 0;
    }
    size_t want = arena_round(bytes);
    cudaError_t e = cudaMalloc((void**)&ctx->arena, want);
    if (e != cudaSuccess) {
        ctx->arena = nullptr;
        return cuda_fail(ctx, e, "scratch arena allocation");
    }
    ctx->arena_bytes = want;
    ctx->arena_used = 0;
    return PSSA_B200_OK;
}

// RAII device buffers for the host-pointer entry points (freed on every exit path)
struct DeviceBuf {
    void* p = nullptr;
    ~DeviceBuf() {
        if (p) cudaFree(p);
    }
    cudaError_t alloc(size_t bytes) { return cudaMalloc(&p, bytes ? bytes : 1); }
    float* f() const { return (float*)p; }
};
}  // namespace pssa

using namespace pssa;

extern "C" {

int32_t pssa_b200_ctx_create(int32_t device, pssa_b200_ctx** out) {
    if (!out) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "pssa_b200_ctx_create: out is null");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return fail(nullptr, PSSA_B200_ERR_CUDA, "no CUDA device available (%s); the B200 path has no CPU fallback",
                    e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0");
    if (device < 0 || device >= count)
        return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "device %d out of range (%d devices)", device, count);
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) return cuda_fail(nullptr, e, "cudaGetDeviceProperties");
    if (prop.major != 10)
        return fail(nullptr, PSSA_B200_ERR_UNSUPPORTED,
                    "device %d (%s) is compute capability %d.%d; this library contains sm_100a code only", device,
                    prop.name, prop.major, prop.minor);
    if ((e = cudaSetDevice(device)) != cudaSuccess) return cuda_fail(nullptr, e, "cudaSetDevice");
    pssa_b200_ctx* ctx = new pssa_b200_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->label = std::string("b200 (") + prop.name + ")";
    if ((e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking)) != cudaSuccess) {
        delete ctx;
        return cuda_fail(nullptr, e, "cudaStreamCreate");
    }
    ctx->owns_stream = true;
    if ((e = cudaMalloc((void**)&ctx->status_dev, sizeof(int))) != cudaSuccess ||
        (e = cudaMemset(ctx->status_dev, 0, sizeof(int))) != cudaSuccess) {
        cudaStreamDestroy(ctx->stream);
        delete ctx;
        return cuda_fail(nullptr, e, "status word allocation");
    }
    *out = ctx;
    return PSSA_B200_OK;
}

void pssa_b200_ctx_destroy(pssa_b200_ctx* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->arena) cudaFree(ctx->arena);
    if (ctx->status_dev) cudaFree(ctx->status_dev);
    if (ctx->owns_stream && ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

const char* pssa_b200_last_error(const pssa_b200_ctx* ctx) { return ctx ? ctx->error.c_str() : g_create_error.c_str(); }

int32_t pssa_b200_ctx_set_stream(pssa_b200_ctx* ctx, void* cuda_stream) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
    ctx->stream = (cudaStream_t)cuda_stream;  // NULL is the legacy default stream
    ctx->owns_stream = false;
    return PSSA_B200_OK;
}

int32_t pssa_b200_ctx_use_own_stream(pssa_b200_ctx* ctx) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->owns_stream) return PSSA_B200_OK;
    PSSA_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
    ctx->owns_stream = true;
    return PSSA_B200_OK;
}

int32_t pssa_b200_ctx_synchronize(pssa_b200_ctx* ctx) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return PSSA_B200_OK;
}

const char* pssa_b200_backend_label(const pssa_b200_ctx* ctx) { return ctx ? ctx->label.c_str() : "b200 (no context)"; }
uint64_t pssa_b200_launch_count(const pssa_b200_ctx* ctx) { return ctx ? ctx->launches : 0; }

int32_t pssa_b200_ctx_reserve(pssa_b200_ctx* ctx, size_t bytes) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    return arena_reserve(ctx, bytes);
}

int32_t pssa_b200_ctx_set_scan_chunks(pssa_b200_ctx* ctx, uint32_t chunks) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    ctx->scan_chunks = (int)chunks;
    return PSSA_B200_OK;
}

// ------------------------------------------------------------------ scan operator

int32_t pssa_b200_affine_scan_dev(pssa_b200_ctx* ctx, float* scan_a, float* scan_b, size_t lanes, size_t len,
                                  size_t stride) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    size_t elems;
    int32_t rc = scan_shape(ctx, lanes, len, stride, &elems);
    if (rc != PSSA_B200_OK) return rc;
    if (!scan_a || !scan_b) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 affine scan: null buffer");
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    return launch_scan_maps(ctx, scan_a, scan_b, lanes, len, stride, ctx->scan_chunks);
}

int32_t pssa_b200_affine_scan(pssa_b200_ctx* ctx, float* scan_a, float* scan_b, size_t lanes, size_t len,
                              size_t stride) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    size_t elems;
    int32_t rc = scan_shape(ctx, lanes, len, stride, &elems);
    if (rc != PSSA_B200_OK) return rc;
    if (!scan_a || !scan_b) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 affine scan: null buffer");
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    DeviceBuf da, db;
    PSSA_CUDA(ctx, da.alloc(elems * 4));
    PSSA_CUDA(ctx, db.alloc(elems * 4));
    PSSA_CUDA(ctx, cudaMemcpyAsync(da.p, scan_a, elems * 4, cudaMemcpyHostToDevice, ctx->stream));
    PSSA_CUDA(ctx, cudaMemcpyAsync(db.p, scan_b, elems * 4, cudaMemcpyHostToDevice, ctx->stream));
    rc = launch_scan_maps(ctx, da.f(), db.f(), lanes, len, stride, ctx->scan_chunks);
    if (rc != PSSA_B200_OK) {
        cudaStreamSynchronize(ctx->stream);
        return rc;
    }
    PSSA_CUDA(ctx, cudaMemcpyAsync(scan_a, da.p, elems * 4, cudaMemcpyDeviceToHost, ctx->stream));
    PSSA_CUDA(ctx, cudaMemcpyAsync(scan_b, db.p, elems * 4, cudaMemcpyDeviceToHost, ctx->stream));
    PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return PSSA_B200_OK;
}

int32_t pssa_b200_scan_states_dev(pssa_b200_ctx* ctx, const float* a, const float* b, const float* h0, float* h,
                                  float* h_last, size_t lanes, size_t len, size_t stride) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    size_t elems;
    int32_t rc = scan_shape(ctx, lanes, len, stride, &elems);
    if (rc != PSSA_B200_OK) return rc;
    if (!a || !b || !h) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 scan states: null buffer");
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    return launch_scan_states(ctx, a, b, h0, h, h_last, lanes, len, stride, ctx->scan_chunks);
}

int32_t pssa_b200_scan_states(pssa_b200_ctx* ctx, const float* a, const float* b, const float* h0, float* h,
                              float* h_last, size_t lanes, size_t len, size_t stride) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    size_t elems;
    int32_t rc = scan_shape(ctx, lanes, len, stride, &elems);
    if (rc != PSSA_B200_OK) return rc;
    if (!a || !b || !h) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 scan states: null buffer");
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    size_t row = lanes * stride * 4;
    DeviceBuf da, db, dh0, dlast;
    PSSA_CUDA(ctx, da.alloc(elems * 4));
    PSSA_CUDA(ctx, db.alloc(elems * 4));
    if (h0) PSSA_CUDA(ctx, dh0.alloc(row));
    if (h_last) PSSA_CUDA(ctx, dlast.alloc(row));
    PSSA_CUDA(ctx, cudaMemcpyAsync(da.p, a, elems * 4, cudaMemcpyHostToDevice, ctx->stream));
    PSSA_CUDA(ctx, cudaMemcpyAsync(db.p, b, elems * 4, cudaMemcpyHostToDevice, ctx->stream));
    if (h0) PSSA_CUDA(ctx, cudaMemcpyAsync(dh0.p, h0, row, cudaMemcpyHostToDevice, ctx->stream));
    // states overwrite the device copy of b: the output needs no third device array
    rc = launch_scan_states(ctx, da.f(), db.f(), h0 ? dh0.f() : nullptr, db.f(), h_last ? dlast.f() : nullptr, lanes,
                            len, stride, ctx->scan_chunks);
    if (rc != PSSA_B200_OK) {
        cudaStreamSynchronize(ctx->stream);
        return rc;
    }
    PSSA_CUDA(ctx, cudaMemcpyAsync(h, db.p, elems * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (h_last) PSSA_CUDA(ctx, cudaMemcpyAsync(h_last, dlast.p, row, cudaMemcpyDeviceToHost, ctx->stream));
    PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return PSSA_B200_OK;
}

}  // extern "C"
