// Per-device context shared by every entry point: stream, scratch arena, error text.
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

#include "../../include/pssa_b200.h"

struct pssa_b200_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    // scratch arena: one growing device allocation, carved per call (no per-call cudaMalloc once warm)
    char* arena = nullptr;
    size_t arena_bytes = 0;
    size_t arena_used = 0;
    // pinned staging for the host-pointer entry points
    std::string error;
    std::string label;
    uint64_t launches = 0;
    int sm_count = 148;
    // device status word for bounded waits (0 = ok)
    int* status_dev = nullptr;
    int scan_chunks = 0;  // 0 = choose automatically; tests force the multi-chunk passes with it
    // lane groups of the model path: up to three side streams beside `stream`, joined by events (model_forward.cu)
    cudaStream_t side[3] = {nullptr, nullptr, nullptr};
    cudaEvent_t fork_ev = nullptr, join_ev[3] = {nullptr, nullptr, nullptr};
    int chain = 0;  // which of those streams `stream` currently is (0 = the caller's); keys the stage profile
    // Resident SSM result (`ssm_forward_resident` -> `memory_forward_after_ssm`, src/backend.rs:1186-1289): the tape of the
    // last resident SSM call stays on the device until the memory stage consumes it.
    struct ResidentSsm {
        float *y = nullptr, *states = nullptr, *bar_a = nullptr, *bar_b = nullptr;  // [T, d], [(T+1), d*s], [T, d*s] x 2
        size_t seq_len = 0, d_m = 0, d_s = 0, capacity_rows = 0, capacity_stride = 0;
        bool valid = false;
    } resident;
    // Stage profile (the role of the reference's StageTrace, src/training_diagnostics.rs:74-125, with device
    // events instead of wall clock): while enabled, an event is recorded after every kernel launch; the time
    // between consecutive events on the (serial) stream is attributed to the kernel launched in between.
    bool profiling = false;
    std::vector<cudaEvent_t> prof_events;      // one per launch, plus one start mark per chain
    std::vector<const char*> prof_names;       // kernel that finished at event i (nullptr: a chain starts here)
    std::vector<int> prof_chain;               // stream (chain) event i was recorded on: times are differences along a chain
    std::vector<cudaEvent_t> prof_pool;        // recycled events
    struct ProfRow {
        std::string name;
        uint64_t launches;
        double ms;
    };
    std::vector<ProfRow> prof_rows;            // result of the last profile_end
};

namespace pssa {

extern thread_local std::string g_create_error;

inline int32_t fail(pssa_b200_ctx* ctx, int32_t code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (ctx)
        ctx->error = buf;
    else
        g_create_error = buf;
    return code;
}

// Fatal classes follow src/cuda.rs:592-602: once seen the context is unusable.
inline bool cuda_error_is_fatal(cudaError_t e) {
    return e == cudaErrorIllegalAddress || e == cudaErrorContextIsDestroyed || e == cudaErrorDevicesUnavailable ||
           e == cudaErrorLaunchTimeout || e == cudaErrorIllegalInstruction || e == cudaErrorMisalignedAddress ||
           e == cudaErrorHardwareStackError || e == cudaErrorLaunchFailure;
}

inline int32_t cuda_fail(pssa_b200_ctx* ctx, cudaError_t e, const char* what) {
    return fail(ctx, cuda_error_is_fatal(e) ? PSSA_B200_ERR_FATAL_CUDA : PSSA_B200_ERR_CUDA, "CUDA %s: %s (%s)", what,
                cudaGetErrorString(e), cudaGetErrorName(e));
}

#define PSSA_CUDA(ctx, call)                                      \
    do {                                                          \
        cudaError_t e__ = (call);                                 \
        if (e__ != cudaSuccess) return pssa::cuda_fail(ctx, e__, #call); \
    } while (0)

// Function attributes such as the opt-in dynamic shared memory size are per DEVICE, while a launcher's static flag is per
// process: a host that opens contexts on several GPUs must set the attribute once on each. One bit per CUDA ordinal.
struct PerDeviceOnce {
    std::atomic<unsigned long long> mask{0};
    bool need(int device) const { return device < 0 || device >= 64 || !(mask.load(std::memory_order_acquire) >> device & 1ull); }
    void done(int device) {
        if (device >= 0 && device < 64) mask.fetch_or(1ull << device, std::memory_order_release);
    }
};

// Arena: reset at the start of an entry point, then bump-allocate 256-byte aligned blocks.
int32_t arena_reserve(pssa_b200_ctx* ctx, size_t bytes);
inline void arena_reset(pssa_b200_ctx* ctx) { ctx->arena_used = 0; }
// Call after the total need is known (arena_reserve) so pointers stay valid.
inline void* arena_take(pssa_b200_ctx* ctx, size_t bytes) {
    size_t off = (ctx->arena_used + 255) & ~size_t(255);
    if (off + bytes > ctx->arena_bytes) return nullptr;
    ctx->arena_used = off + bytes;
    return ctx->arena + off;
}
inline size_t arena_round(size_t bytes) { return (bytes + 255) & ~size_t(255); }

// Launch bookkeeping: every kernel launch of this library goes through here.
// Programmatic dependent launch (stream order preserved, launch latency hidden): a kernel launched with
// `launch_dependent` may start before its predecessor in the stream has finished, and must call pdl_wait() before it
// reads or writes anything the predecessor touches; predecessors call pdl_trigger() early so that the dependent's
// prologue (barrier set-up, TMEM allocation, descriptor fetch) overlaps their own tail. Both calls are no-ops for
// kernels launched the ordinary way.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr, cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#endif
void profile_record(pssa_b200_ctx* ctx, const char* kernel);  // api.cu
inline int32_t after_launch(pssa_b200_ctx* ctx, const char* kernel) {
    ctx->launches += 1;
    if (ctx->profiling) profile_record(ctx, kernel);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(ctx, e, kernel);
    return PSSA_B200_OK;
}

}  // namespace pssa
