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

static cudaEvent_t prof_event(pssa_b200_ctx* ctx) {
    cudaEvent_t e = nullptr;
    if (!ctx->prof_pool.empty()) {
        e = ctx->prof_pool.back();
        ctx->prof_pool.pop_back();
    } else if (cudaEventCreate(&e) != cudaSuccess) {
        e = nullptr;
    }
    return e;
}

void profile_record(pssa_b200_ctx* ctx, const char* kernel) {
    cudaEvent_t e = prof_event(ctx);
    if (!e) return;
    cudaEventRecord(e, ctx->stream);
    ctx->prof_events.push_back(e);
    ctx->prof_names.push_back(kernel);
    ctx->prof_chain.push_back(ctx->chain);
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
    cudaFree(ctx->resident.y), cudaFree(ctx->resident.states), cudaFree(ctx->resident.bar_a), cudaFree(ctx->resident.bar_b);
    for (int i = 0; i < 3; ++i) {
        if (ctx->side[i]) cudaStreamDestroy(ctx->side[i]);
        if (ctx->join_ev[i]) cudaEventDestroy(ctx->join_ev[i]);
    }
    if (ctx->fork_ev) cudaEventDestroy(ctx->fork_ev);
    for (cudaEvent_t e : ctx->prof_events) cudaEventDestroy(e);
    for (cudaEvent_t e : ctx->prof_pool) cudaEventDestroy(e);
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

int32_t pssa_b200_ctx_selftest_wait_expiry(pssa_b200_ctx* ctx, uint32_t polls) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    if (polls == 0 || polls > (1u << 20)) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "selftest: polls must be in 1..2^20");
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    return launch_wait_expiry_selftest(ctx, polls);
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

int32_t pssa_b200_scan_states_noalloc_dev(pssa_b200_ctx* ctx, const float* a, const float* b, const float* h0, float* h,
                                          float* h_last, size_t lanes, size_t len, size_t stride, uint32_t chunks) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    size_t elems;
    int32_t rc = scan_shape(ctx, lanes, len, stride, &elems);
    if (rc != PSSA_B200_OK) return rc;
    if (!a || !b || !h) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 scan states: null buffer");
    if (chunks == 0) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 static scan: chunks must be at least 1");
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    return launch_scan_states_static(ctx, a, b, h0, h, h_last, lanes, len, stride, chunks);
}

// ------------------------------------------------------------------ fused SSM stage


int32_t pssa_b200_ssm_forward_dev(pssa_b200_ctx* ctx, const float* delta, const float* b_proj, const float* c_proj,
                                  const float* x_norm, const float* rates, float* carry, float* y, float* states,
                                  float* bar_a, float* bar_b, const uint32_t* offsets, const uint32_t* lengths,
                                  size_t lanes, size_t rows, size_t d_m, size_t d_s, uint32_t flags) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    SsmShape shape;
    int32_t rc = ssm_shape(ctx, rows, d_m, d_s, &shape);
    if (rc != PSSA_B200_OK) return rc;
    if (lanes == 0 || lanes > 0x7fffffff)
        return fail(ctx, PSSA_B200_ERR_SHAPE, "B200 SSM lane count %zu must be in 1..2^31-1; refusing launch", lanes);
    if (!delta || !b_proj || !c_proj || !x_norm || !rates || !y)
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 SSM forward: null buffer");
    if ((offsets == nullptr) != (lengths == nullptr))
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 SSM forward: offsets and lengths must both be given");
    if (!offsets && lanes != 1)
        return fail(ctx, PSSA_B200_ERR_SHAPE, "B200 SSM forward: %zu lanes need offsets and lengths; refusing launch", lanes);
    if (flags & ~PSSA_B200_SSM_EXACT) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 SSM forward: unknown flags");
    if (offsets) {
        for (size_t l = 0; l < lanes; ++l)
            if ((size_t)offsets[l] + lengths[l] > rows)
                return fail(ctx, PSSA_B200_ERR_SHAPE,
                            "B200 SSM forward: lane %zu covers rows [%u, %u) outside %zu rows; refusing launch", l,
                            offsets[l], offsets[l] + lengths[l], rows);
    }
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    SsmParams p{};
    p.delta = delta, p.x_norm = x_norm, p.b_proj = b_proj, p.c_proj = c_proj, p.rates = rates;
    p.carry = carry, p.y = y, p.states = states, p.bar_a = bar_a, p.bar_b = bar_b;
    p.rows = rows, p.d = (int)d_m, p.s = (int)d_s, p.lanes = (int)lanes;
    p.aligned = ssm_vector_ok(p);
    p.single_token = 1;  // decode-step shape: every lane at most one token
    for (size_t l = 0; l < lanes; ++l) p.single_token = p.single_token && (lengths ? lengths[l] <= 1 : rows <= 1);
    if (offsets) {
        arena_reset(ctx);
        if ((rc = arena_reserve(ctx, arena_round(lanes * 4) * 2)) != PSSA_B200_OK) return rc;
        uint32_t* d_off = (uint32_t*)arena_take(ctx, lanes * 4);
        uint32_t* d_len = (uint32_t*)arena_take(ctx, lanes * 4);
        PSSA_CUDA(ctx, cudaMemcpyAsync(d_off, offsets, lanes * 4, cudaMemcpyHostToDevice, ctx->stream));
        PSSA_CUDA(ctx, cudaMemcpyAsync(d_len, lengths, lanes * 4, cudaMemcpyHostToDevice, ctx->stream));
        p.offsets = d_off, p.lengths = d_len;
    }
    return launch_ssm_fused(ctx, p, (flags & PSSA_B200_SSM_EXACT) != 0);
}

int32_t pssa_b200_ssm_forward(pssa_b200_ctx* ctx, const float* delta, const float* b_proj, const float* x_norm,
                              const float* rates, const float* c_proj, const float* initial, size_t seq_len,
                              size_t d_m, size_t d_s, float* bar_a, float* bar_b, float* states, float* y_ssm,
                              uint32_t flags) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    SsmShape sh;
    int32_t rc = ssm_shape(ctx, seq_len, d_m, d_s, &sh);
    if (rc != PSSA_B200_OK) return rc;
    if (!delta || !b_proj || !c_proj || !x_norm || !rates || !initial || !y_ssm)
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 SSM forward: null buffer");
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    DeviceBuf d_delta, d_b, d_c, d_x, d_rates, d_carry, d_y, d_states, d_ba, d_bb;
    size_t tape = seq_len * sh.stride * 4;
    PSSA_CUDA(ctx, d_delta.alloc(sh.token_m * 4));
    PSSA_CUDA(ctx, d_x.alloc(sh.token_m * 4));
    PSSA_CUDA(ctx, d_y.alloc(sh.token_m * 4));
    PSSA_CUDA(ctx, d_b.alloc(sh.token_s * 4));
    PSSA_CUDA(ctx, d_c.alloc(sh.token_s * 4));
    PSSA_CUDA(ctx, d_rates.alloc(sh.stride * 4));
    PSSA_CUDA(ctx, d_carry.alloc(sh.stride * 4));
    if (states) PSSA_CUDA(ctx, d_states.alloc(tape));
    if (bar_a) PSSA_CUDA(ctx, d_ba.alloc(tape));
    if (bar_b) PSSA_CUDA(ctx, d_bb.alloc(tape));
    cudaStream_t st = ctx->stream;
    PSSA_CUDA(ctx, cudaMemcpyAsync(d_delta.p, delta, sh.token_m * 4, cudaMemcpyHostToDevice, st));
    PSSA_CUDA(ctx, cudaMemcpyAsync(d_x.p, x_norm, sh.token_m * 4, cudaMemcpyHostToDevice, st));
    PSSA_CUDA(ctx, cudaMemcpyAsync(d_b.p, b_proj, sh.token_s * 4, cudaMemcpyHostToDevice, st));
    PSSA_CUDA(ctx, cudaMemcpyAsync(d_c.p, c_proj, sh.token_s * 4, cudaMemcpyHostToDevice, st));
    PSSA_CUDA(ctx, cudaMemcpyAsync(d_rates.p, rates, sh.stride * 4, cudaMemcpyHostToDevice, st));
    PSSA_CUDA(ctx, cudaMemcpyAsync(d_carry.p, initial, sh.stride * 4, cudaMemcpyHostToDevice, st));
    rc = pssa_b200_ssm_forward_dev(ctx, d_delta.f(), d_b.f(), d_c.f(), d_x.f(), d_rates.f(), d_carry.f(), d_y.f(),
                                   states ? d_states.f() : nullptr, bar_a ? d_ba.f() : nullptr,
                                   bar_b ? d_bb.f() : nullptr, nullptr, nullptr, 1, seq_len, d_m, d_s, flags);
    if (rc != PSSA_B200_OK) {
        cudaStreamSynchronize(st);
        return rc;
    }
    PSSA_CUDA(ctx, cudaMemcpyAsync(y_ssm, d_y.p, sh.token_m * 4, cudaMemcpyDeviceToHost, st));
    if (states) {
        memcpy(states, initial, sh.stride * 4);
        PSSA_CUDA(ctx, cudaMemcpyAsync(states + sh.stride, d_states.p, tape, cudaMemcpyDeviceToHost, st));
    }
    if (bar_a) PSSA_CUDA(ctx, cudaMemcpyAsync(bar_a, d_ba.p, tape, cudaMemcpyDeviceToHost, st));
    if (bar_b) PSSA_CUDA(ctx, cudaMemcpyAsync(bar_b, d_bb.p, tape, cudaMemcpyDeviceToHost, st));
    PSSA_CUDA(ctx, cudaStreamSynchronize(st));
    return PSSA_B200_OK;
}

// ------------------------------------------------------------------ episodic memory read

// Shared body of the device-pointer read entry points. `slots_out` / `topk_w_out` [rows, top_k] are the compact results of
// a top-k read (ascending slot order); `handed_over` receives the number of rows the one-kernel read gave to its exact pass.
static int32_t memory_read_impl(pssa_b200_ctx* ctx, const float* q, int32_t q_is_euclidean, const float* keys, const float* norm_sq,
                                const float* values, size_t rows, size_t d_key, size_t d_val, size_t capacity, size_t count, float tau,
                                size_t top_k, float* q_pnc, float* q_norm, float* weights, float* m_val, float* min_dist,
                                uint32_t* slots_out, float* topk_w_out, uint32_t* handed_over, uint32_t flags) {
    int32_t rc = memory_shape(ctx, rows, d_key, d_val, capacity, count, tau);
    if (rc != PSSA_B200_OK) return rc;
    if (!q || !keys || !norm_sq || !values || !m_val)
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 memory read: null buffer");
    const uint32_t known = PSSA_B200_MEM_EXACT | PSSA_B200_MEM_F32_DISTANCE | PSSA_B200_MEM_TC_DISTANCE | PSSA_B200_MEM_NO_FUSED |
                           PSSA_B200_MEM_HANDOVER_SELFTEST | PSSA_B200_MEM_PHASE_CLOCKS;
    if (flags & ~known) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 memory read: unknown flags");
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    // scratch from the arena: the weight rows when the caller does not want them, the bf16 pieces of the weights and of the
    // transposed values for the tensor-core value read (all-slots mode, capacity % 64 == 0), the key pieces of the
    // tensor-core distances / of the one-kernel top-k read with its hand-over list
    const bool exact = (flags & PSSA_B200_MEM_EXACT) != 0;
    const bool topk = top_k != 0 && top_k < count;
    const bool approx = !exact && (flags & (PSSA_B200_MEM_F32_DISTANCE | PSSA_B200_MEM_TC_DISTANCE)) != 0;
    RetrieveParams p{};
    p.q = q, p.q_is_euclidean = q_is_euclidean, p.q_pnc = q_pnc, p.q_norm = q_norm;
    p.keys = keys, p.norm_sq = norm_sq, p.values = values;
    p.m_val = m_val, p.min_dist = min_dist;
    p.rows = rows, p.dk = (int)d_key, p.dv = (int)d_val, p.cap = (int)capacity, p.count = (int)count;
    p.top_k = (int)(top_k > capacity ? capacity : top_k), p.tau = tau;
    p.f32_distance = (flags & (PSSA_B200_MEM_F32_DISTANCE | PSSA_B200_MEM_TC_DISTANCE)) != 0;
    p.no_fused = approx || (flags & PSSA_B200_MEM_NO_FUSED) != 0;
    p.selftest_every = (flags & PSSA_B200_MEM_HANDOVER_SELFTEST) ? 3 : 0;
    // would the one-kernel top-k read take this call? (decided on the shape; its scratch pointers are filled in below)
    RetrieveParams probe = p;
    probe.k_split = probe.k_stat = nullptr;
    unsigned dummy = 0;
    probe.k_split = &dummy, probe.k_stat = reinterpret_cast<const float2*>(&dummy), probe.fixup_count = &dummy;
    const bool fused = topk && !p.no_fused && retrieve_fused_eligible(probe);
    const bool tc_read = !exact && !topk && count > 0 && capacity % 64 == 0;
    const bool tc_dist = !exact && !fused && (flags & PSSA_B200_MEM_TC_DISTANCE) != 0 && d_key % 64 == 0 && count > 0;
    const bool need_dense = !weights && !fused;
    const bool key_pieces = tc_dist || fused;
    size_t need = (need_dense ? arena_round(rows * capacity * 4) : 0) +
                  (tc_read ? arena_round(rows * 3 * capacity * 2) + arena_round(d_val * 3 * capacity * 2) : 0) +
                  (tc_dist ? arena_round(rows * 3 * d_key * 2) + arena_round(rows * 8) : 0) +
                  (key_pieces ? arena_round(capacity * 3 * d_key * 2) + arena_round(capacity * 8) : 0) +
                  (fused ? arena_round((rows + 1) * 4) : 0);
    if (need) {
        arena_reset(ctx);
        if ((rc = arena_reserve(ctx, need)) != PSSA_B200_OK) return rc;
        if (need_dense) weights = (float*)arena_take(ctx, rows * capacity * 4);
        if (tc_read) {
            p.w_split = arena_take(ctx, rows * 3 * capacity * 2);
            void* v_split = arena_take(ctx, d_val * 3 * capacity * 2);
            if ((rc = launch_split_values(ctx, values, v_split, (int)capacity, (int)d_val)) != PSSA_B200_OK) return rc;
            p.v_split = v_split;
        }
        if (key_pieces) {
            void* k_split = arena_take(ctx, capacity * 3 * d_key * 2);
            float2* k_stat = (float2*)arena_take(ctx, capacity * 8);
            if ((rc = launch_split_keys(ctx, keys, norm_sq, k_split, k_stat, (int)capacity, (int)d_key)) != PSSA_B200_OK) return rc;
            p.k_split = k_split, p.k_stat = k_stat;
        }
        if (tc_dist) p.q_split = arena_take(ctx, rows * 3 * d_key * 2), p.q_stat = (float2*)arena_take(ctx, rows * 8);
        if (fused) {
            p.fixup_count = (uint32_t*)arena_take(ctx, 4);
        }
    }
    p.weights = weights;
    if (fused) p.topk_slots = slots_out, p.topk_weights = topk_w_out;
    if (fused && handed_over && (flags & PSSA_B200_MEM_PHASE_CLOCKS)) {
        p.phase_cycles = reinterpret_cast<unsigned long long*>(handed_over + 2);
        PSSA_CUDA(ctx, cudaMemsetAsync(handed_over + 2, 0, kRetrievePhases * sizeof(unsigned long long), ctx->stream));
    }
    if ((rc = launch_memory_read(ctx, p, exact)) != PSSA_B200_OK) return rc;
    if (!fused && topk && (slots_out || topk_w_out) &&
        (rc = launch_compact_topk(ctx, weights, (int)capacity, p.top_k, rows, slots_out, topk_w_out)) != PSSA_B200_OK)
        return rc;
    if (handed_over) {
        if (fused)
            PSSA_CUDA(ctx, cudaMemcpyAsync(handed_over, p.fixup_count, 4, cudaMemcpyDeviceToDevice, ctx->stream));
        else
            PSSA_CUDA(ctx, cudaMemsetAsync(handed_over, 0, 4, ctx->stream));
    }
    return PSSA_B200_OK;
}

int32_t pssa_b200_memory_read_dev(pssa_b200_ctx* ctx, const float* q, int32_t q_is_euclidean, const float* keys,
                                  const float* norm_sq, const float* values, size_t rows, size_t d_key, size_t d_val,
                                  size_t capacity, size_t count, float tau, size_t top_k, float* q_pnc, float* q_norm,
                                  float* weights, float* m_val, float* min_dist, uint32_t flags) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    return memory_read_impl(ctx, q, q_is_euclidean, keys, norm_sq, values, rows, d_key, d_val, capacity, count, tau, top_k, q_pnc, q_norm,
                            weights, m_val, min_dist, nullptr, nullptr, nullptr, flags);
}

int32_t pssa_b200_memory_read_topk_dev(pssa_b200_ctx* ctx, const float* q, int32_t q_is_euclidean, const float* keys,
                                       const float* norm_sq, const float* values, size_t rows, size_t d_key, size_t d_val,
                                       size_t capacity, size_t count, float tau, size_t top_k, float* q_pnc, float* q_norm, float* m_val,
                                       float* min_dist, uint32_t* slots_out, float* weights_out, uint32_t* handed_over, uint32_t flags) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    if (top_k == 0 || top_k >= count)
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 top-k read: top_k must be in 1..count-1 (use the all-slots read otherwise)");
    return memory_read_impl(ctx, q, q_is_euclidean, keys, norm_sq, values, rows, d_key, d_val, capacity, count, tau, top_k, q_pnc, q_norm,
                            nullptr, m_val, min_dist, slots_out, weights_out, handed_over, flags);
}

int32_t pssa_b200_memory_read(pssa_b200_ctx* ctx, const float* q, int32_t q_is_euclidean, const float* keys,
                              const float* norm_sq, const float* values, size_t rows, size_t d_key, size_t d_val,
                              size_t capacity, size_t count, float tau, size_t top_k, float* q_pnc, float* q_norm,
                              float* weights, float* m_val, float* min_dist, uint32_t flags) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    int32_t rc = memory_shape(ctx, rows, d_key, d_val, capacity, count, tau);
    if (rc != PSSA_B200_OK) return rc;
    if (!q || !keys || !norm_sq || !values || !m_val)
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 memory read: null buffer");
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    DeviceBuf dq, dkeys, dns, dvals, dpnc, dqn, dw, dm, dmin;
    cudaStream_t st = ctx->stream;
    PSSA_CUDA(ctx, dq.alloc(rows * d_key * 4));
    PSSA_CUDA(ctx, dkeys.alloc(capacity * d_key * 4));
    PSSA_CUDA(ctx, dns.alloc(capacity * 4));
    PSSA_CUDA(ctx, dvals.alloc(capacity * d_val * 4));
    PSSA_CUDA(ctx, dpnc.alloc(rows * d_key * 4));
    PSSA_CUDA(ctx, dqn.alloc(rows * 4));
    PSSA_CUDA(ctx, dw.alloc(rows * capacity * 4));
    PSSA_CUDA(ctx, dm.alloc(rows * d_val * 4));
    PSSA_CUDA(ctx, dmin.alloc(rows * 4));
    PSSA_CUDA(ctx, cudaMemcpyAsync(dq.p, q, rows * d_key * 4, cudaMemcpyHostToDevice, st));
    PSSA_CUDA(ctx, cudaMemcpyAsync(dkeys.p, keys, capacity * d_key * 4, cudaMemcpyHostToDevice, st));
    PSSA_CUDA(ctx, cudaMemcpyAsync(dns.p, norm_sq, capacity * 4, cudaMemcpyHostToDevice, st));
    PSSA_CUDA(ctx, cudaMemcpyAsync(dvals.p, values, capacity * d_val * 4, cudaMemcpyHostToDevice, st));
    PSSA_CUDA(ctx, cudaMemsetAsync(dw.p, 0, rows * capacity * 4, st));
    rc = pssa_b200_memory_read_dev(ctx, dq.f(), q_is_euclidean, dkeys.f(), dns.f(), dvals.f(), rows, d_key, d_val,
                                   capacity, count, tau, top_k, dpnc.f(), dqn.f(), dw.f(), dm.f(), dmin.f(), flags);
    if (rc != PSSA_B200_OK) {
        cudaStreamSynchronize(st);
        return rc;
    }
    if (q_pnc) PSSA_CUDA(ctx, cudaMemcpyAsync(q_pnc, dpnc.p, rows * d_key * 4, cudaMemcpyDeviceToHost, st));
    if (q_norm) PSSA_CUDA(ctx, cudaMemcpyAsync(q_norm, dqn.p, rows * 4, cudaMemcpyDeviceToHost, st));
    if (weights) PSSA_CUDA(ctx, cudaMemcpyAsync(weights, dw.p, rows * capacity * 4, cudaMemcpyDeviceToHost, st));
    PSSA_CUDA(ctx, cudaMemcpyAsync(m_val, dm.p, rows * d_val * 4, cudaMemcpyDeviceToHost, st));
    if (min_dist) PSSA_CUDA(ctx, cudaMemcpyAsync(min_dist, dmin.p, rows * 4, cudaMemcpyDeviceToHost, st));
    PSSA_CUDA(ctx, cudaStreamSynchronize(st));
    return PSSA_B200_OK;
}

// ------------------------------------------------------------------ bank write and plastic fast weights

int32_t pssa_b200_bank_insert_protected_dev(pssa_b200_ctx* ctx, float* keys, float* norm_sq, float* values, float* confidence,
                                            uint64_t* last_seen_step, uint64_t* meta, size_t capacity, size_t d_key,
                                            size_t d_val, const float* key_pnc, const float* val, const float* surprise,
                                            const uint64_t* step, size_t n, int64_t* slots_out,
                                            const uint32_t* winning_slots, float eta) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    if (capacity == 0 || d_key == 0 || d_val == 0 || capacity > 0x7fffffff || d_key > 0x7fffffff || d_val > 0x7fffffff)
        return fail(ctx, PSSA_B200_ERR_SHAPE, "memory dimensions and capacity must be positive");  // src/memory.rs:36-39
    if (!keys || !norm_sq || !values || !confidence || !last_seen_step || !meta || !key_pnc || !val || !surprise || !step)
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 bank write: null buffer");
    if (winning_slots && !(eta >= 0.0f && eta <= 1.0f))
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 bank write: eta must be in [0, 1]");
    if (n == 0) return PSSA_B200_OK;
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    BankWriteParams p{};
    p.keys = keys, p.norm_sq = norm_sq, p.values = values, p.confidence = confidence;
    p.last_seen = (unsigned long long*)last_seen_step, p.meta = (unsigned long long*)meta;
    p.cap = (int)capacity, p.dk = (int)d_key, p.dv = (int)d_val;
    p.key_pnc = key_pnc, p.val = val, p.surprise = surprise, p.step = (const unsigned long long*)step, p.n = n;
    p.slots_out = (long long*)slots_out, p.winning_slots = winning_slots, p.eta = eta;
    return launch_bank_insert_protected(ctx, p);
}

int32_t pssa_b200_adapter_plastic_update_dev(pssa_b200_ctx* ctx, float* up_fast, const float* value, const float* ad_out,
                                             const float* ad_act, size_t d, size_t rank) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    if (d == 0 || rank == 0 || d > 0x7fffffff / (rank ? rank : 1)) return fail(ctx, PSSA_B200_ERR_SHAPE, "adapter dimensions must be positive and fit i32");
    if (!up_fast || !value || !ad_out || !ad_act) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 plastic update: null buffer");
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    return launch_plastic_update(ctx, up_fast, value, ad_out, ad_act, (int)d, (int)rank);
}

int32_t pssa_b200_adapter_consolidate_dev(pssa_b200_ctx* ctx, float* up_fast, float* up_slow, size_t n, float alpha) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    if (!(alpha >= 0.0f && alpha <= 1.0f)) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "consolidation alpha must be in [0, 1]");
    if (!up_fast || !up_slow) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 consolidate: null buffer");
    if (n == 0) return PSSA_B200_OK;
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    return launch_consolidate(ctx, up_fast, up_slow, n, alpha);
}

// ------------------------------------------------------------------ dense product

// backend.rs:11-38 (checked_gemm_sizes)
static int32_t gemm_sizes(pssa_b200_ctx* ctx, size_t rows, size_t n, size_t k, size_t ldo, int32_t epi, int32_t precision) {
    if (rows == 0 || n == 0 || k == 0) return fail(ctx, PSSA_B200_ERR_SHAPE, "GEMM dimensions must be positive");
    size_t e;
    int32_t rc;
    if ((rc = f32_elems(ctx, "GEMM input", {rows, k}, &e))) return rc;
    if ((rc = f32_elems(ctx, "GEMM weights", {n, k}, &e))) return rc;
    if ((rc = f32_elems(ctx, "GEMM output", {rows, ldo}, &e))) return rc;
    if (ldo < n) return fail(ctx, PSSA_B200_ERR_SHAPE, "GEMM output pitch %zu is smaller than N %zu", ldo, n);
    if (epi < PSSA_B200_EPI_NONE || epi > PSSA_B200_EPI_ADD_OUT) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "unknown GEMM epilogue %d", epi);
    if (precision != PSSA_B200_PRECISION_BF16 && precision != PSSA_B200_PRECISION_FP32_EXACT)
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "unknown GEMM precision %d", precision);
    return PSSA_B200_OK;
}

int32_t pssa_b200_gemm_xwt_dev(pssa_b200_ctx* ctx, const float* x, const float* w, size_t rows, size_t n, size_t k, float* out,
                               size_t ldo, int32_t epilogue, float alpha, int32_t precision) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    int32_t rc = gemm_sizes(ctx, rows, n, k, ldo, epilogue, precision);
    if (rc) return rc;
    if (!x || !w || !out) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "GEMM: null buffer");
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    if (precision == PSSA_B200_PRECISION_FP32_EXACT) return launch_gemm_exact(ctx, x, w, out, rows, n, k, ldo, epilogue, alpha);
    // operands are rounded to bf16 in scratch from the arena
    arena_reset(ctx);
    if ((rc = arena_reserve(ctx, arena_round(rows * k * 2) + arena_round(n * k * 2)))) return rc;
    void* x16 = arena_take(ctx, rows * k * 2);
    void* w16 = arena_take(ctx, n * k * 2);
    if ((rc = launch_to_bf16(ctx, x, x16, rows * k))) return rc;
    if ((rc = launch_to_bf16(ctx, w, w16, n * k))) return rc;
    return launch_gemm_bf16(ctx, x16, w16, out, nullptr, rows, n, k, ldo, epilogue, alpha);
}

int32_t pssa_b200_gemm_xwt(pssa_b200_ctx* ctx, const float* x, const float* w, size_t m, size_t n, size_t k, size_t batch,
                           float* out, int32_t epilogue, float alpha, int32_t precision) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    size_t rows;
    // backend.rs:41-48: the batch shares W and is folded into rows
    if (m == 0 || batch == 0 || !checked_mul(m, batch, &rows)) return fail(ctx, PSSA_B200_ERR_SHAPE, "GEMM row count must be positive and fit usize");
    int32_t rc = gemm_sizes(ctx, rows, n, k, n, epilogue, precision);
    if (rc) return rc;
    if (!x || !w || !out) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "GEMM: null buffer");
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    DeviceBuf dx, dw, dout;
    cudaStream_t st = ctx->stream;
    PSSA_CUDA(ctx, dx.alloc(rows * k * 4));
    PSSA_CUDA(ctx, dw.alloc(n * k * 4));
    PSSA_CUDA(ctx, dout.alloc(rows * n * 4));
    PSSA_CUDA(ctx, cudaMemcpyAsync(dx.p, x, rows * k * 4, cudaMemcpyHostToDevice, st));
    PSSA_CUDA(ctx, cudaMemcpyAsync(dw.p, w, n * k * 4, cudaMemcpyHostToDevice, st));
    if (epilogue == PSSA_B200_EPI_ADD_OUT) PSSA_CUDA(ctx, cudaMemcpyAsync(dout.p, out, rows * n * 4, cudaMemcpyHostToDevice, st));
    rc = pssa_b200_gemm_xwt_dev(ctx, dx.f(), dw.f(), rows, n, k, dout.f(), n, epilogue, alpha, precision);
    if (rc == PSSA_B200_OK) {
        int status = 0;
        PSSA_CUDA(ctx, cudaMemcpyAsync(&status, ctx->status_dev, sizeof(int), cudaMemcpyDeviceToHost, st));
        PSSA_CUDA(ctx, cudaStreamSynchronize(st));
        if (status != 0) {
            cudaMemsetAsync(ctx->status_dev, 0, sizeof(int), st);
            return fail(ctx, status, "B200 GEMM: a bounded device-side wait expired");
        }
        PSSA_CUDA(ctx, cudaMemcpyAsync(out, dout.p, rows * n * 4, cudaMemcpyDeviceToHost, st));
    }
    PSSA_CUDA(ctx, cudaStreamSynchronize(st));
    return rc;
}

int32_t pssa_b200_ctx_profile_begin(pssa_b200_ctx* ctx) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    for (cudaEvent_t e : ctx->prof_events) ctx->prof_pool.push_back(e);
    ctx->prof_events.clear();
    ctx->prof_names.clear();
    ctx->prof_chain.clear();
    cudaEvent_t e = prof_event(ctx);
    if (!e) return fail(ctx, PSSA_B200_ERR_CUDA, "profile: cannot create an event");
    PSSA_CUDA(ctx, cudaEventRecord(e, ctx->stream));
    ctx->prof_events.push_back(e);
    ctx->prof_names.push_back(nullptr);
    ctx->prof_chain.push_back(0);
    ctx->profiling = true;
    return PSSA_B200_OK;
}

int32_t pssa_b200_ctx_profile_end(pssa_b200_ctx* ctx, uint32_t* n_rows) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    ctx->profiling = false;
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    for (int i = 0; i < 3; ++i)
        if (ctx->side[i]) PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->side[i]));
    ctx->prof_rows.clear();
    // time of a kernel = from the previous event on ITS chain (stream) to its own; with several lane groups the chains
    // overlap on the device, so the rows add up to more than the wall time
    cudaEvent_t last[4] = {nullptr, nullptr, nullptr, nullptr};
    for (size_t i = 0; i < ctx->prof_events.size(); ++i) {
        const int chain = ctx->prof_chain[i] & 3;
        cudaEvent_t prev = last[chain];
        last[chain] = ctx->prof_events[i];
        const char* name = ctx->prof_names[i];
        if (!name || !prev) continue;
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, prev, ctx->prof_events[i]) != cudaSuccess) continue;
        bool found = false;
        for (auto& r : ctx->prof_rows)
            if (r.name == name) {
                r.launches += 1, r.ms += ms, found = true;
                break;
            }
        if (!found) ctx->prof_rows.push_back({name, 1, (double)ms});
    }
    for (cudaEvent_t e : ctx->prof_events) ctx->prof_pool.push_back(e);
    ctx->prof_events.clear();
    ctx->prof_names.clear();
    ctx->prof_chain.clear();
    if (n_rows) *n_rows = (uint32_t)ctx->prof_rows.size();
    return PSSA_B200_OK;
}

int32_t pssa_b200_ctx_profile_row(pssa_b200_ctx* ctx, uint32_t index, const char** name, uint64_t* launches, double* ms) {
    if (!ctx || !name || !launches || !ms) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "profile_row: null argument");
    if (index >= ctx->prof_rows.size()) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "profile_row: index %u of %zu", index, ctx->prof_rows.size());
    *name = ctx->prof_rows[index].name.c_str();
    *launches = ctx->prof_rows[index].launches;
    *ms = ctx->prof_rows[index].ms;
    return PSSA_B200_OK;
}

int32_t pssa_b200_sample_dev(pssa_b200_ctx* ctx, float* logits, float* probs, size_t rows, size_t vocab, const pssa_b200_sampling* cfg,
                             const uint32_t* recent_ids, const uint32_t* recent_count, uint64_t* rng_state, uint32_t* ids_out,
                             uint32_t* status_out, float* confidence_out, uint32_t flags) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    if (!logits || !probs || !cfg || !rng_state || !ids_out || !status_out)
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "sampling: null buffer");
    if ((recent_ids == nullptr) != (recent_count == nullptr))
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "sampling: recent ids and their counts must both be given");
    if (flags & ~PSSA_B200_SAMPLE_EXACT) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "sampling: unknown flags");
    // src/inference.rs:87-101
    if (!std::isfinite(cfg->temperature) || cfg->temperature < 0.0f) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "temperature must be finite and >= 0");
    if (!(std::isfinite(cfg->top_p) && cfg->top_p > 0.0f && cfg->top_p <= 1.0f)) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "top-p must be finite in (0, 1]");
    if (cfg->top_k == 0) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "top-k must be positive");
    if (!(std::isfinite(cfg->repetition_penalty) && cfg->repetition_penalty >= 1.0f))
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "repetition penalty must be finite and >= 1");
    if (vocab == 0 || vocab > 0x7fffffff) return fail(ctx, PSSA_B200_ERR_SHAPE, "sampling: vocabulary size %zu outside 1..2^31-1", vocab);
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    SampleParams p{};
    p.logits = logits, p.probs = probs, p.rows = rows, p.vocab = (int)vocab, p.top_k = (int)std::min<uint32_t>(cfg->top_k, 0x7fffffff);
    p.temperature = cfg->temperature, p.top_p = cfg->top_p, p.repetition_penalty = cfg->repetition_penalty;
    p.recent_ids = recent_ids, p.recent_count = recent_count, p.rng_state = (unsigned long long*)rng_state;
    p.ids_out = ids_out, p.status_out = status_out, p.exact = (flags & PSSA_B200_SAMPLE_EXACT) != 0;
    p.confidence_out = confidence_out;
    if ((size_t)p.top_k > vocab) p.top_k = (int)vocab;  // min(candidates, top_k), src/inference.rs:157
    return launch_sample(ctx, p);
}

/* Reads and clears the device status word written by bounded waits (0 = none expired). */
int32_t pssa_b200_ctx_poll_status(pssa_b200_ctx* ctx) {
    if (!ctx) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null context");
    int status = 0;
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    PSSA_CUDA(ctx, cudaMemcpyAsync(&status, ctx->status_dev, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (status != 0) {
        PSSA_CUDA(ctx, cudaMemsetAsync(ctx->status_dev, 0, sizeof(int), ctx->stream));
        if (status == PSSA_B200_ERR_TOKEN)
            return fail(ctx, status, "a device-resident token ID was outside the model vocabulary (row 0 was read in its place)");
        if (status == PSSA_B200_ERR_BANK)
            return fail(ctx, status, "a protected bank write was refused: slot id or bank metadata out of range, or key outside the unit ball");
        return fail(ctx, status, "a bounded device-side wait expired (status %d)", status);
    }
    return PSSA_B200_OK;
}

}  // extern "C"
