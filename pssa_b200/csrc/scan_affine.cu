// Associative scan over diagonal affine maps (a_t, b_t): h_t = a_t * h_{t-1} + b_t.
//
// Replaces the reference's Blelloch tree `affine_scan_in_place` (src/gpu_batch.rs:98-164) and its
// one-thread-per-channel PTX kernel `affine_scan` (src/cuda/stages.ptx:35-53).
//
// Layout in HBM is the reference's: time-major [lanes, len, stride] with the channel fastest, so a
// warp reading one time row of 32 float4 channel groups touches 512 contiguous bytes.
//
// Schedule. The kernel is HBM-bound (12 B per element for states, 16 B for prefix maps), so the job
// is to keep enough loads in flight and to read every input byte once:
//   * one thread owns V channels (float4 when stride % 4 == 0) and walks a time chunk serially,
//     issuing the loads of U rows before the U dependent multiply-adds (U*2 16-byte loads in flight
//     per thread, several hundred KB per SM);
//   * if lanes*stride alone cannot fill the machine, time is split into chunks: pass 1 reduces every
//     chunk to one map (A, B), pass 2 walks the few chunk maps serially to get each chunk's carry-in,
//     pass 3 rescans with that carry. With one chunk only pass 3 runs and inputs are read once.
// There is no inter-CTA waiting anywhere, hence nothing that can spin.
//
// Arithmetic is multiply-then-add with separate roundings (no FMA contraction), which is what the
// reference's scalar recurrence does (src/gpu_batch.rs:564-567); with a single chunk the states are
// therefore bit-identical to the ordered CPU recurrence.
#include "bounds.hpp"
#include "context.hpp"
#include "kernels.hpp"

namespace pssa {
namespace {

template <int V>
struct VecIO;
template <>
struct VecIO<1> {
    static __device__ __forceinline__ void load(const float* p, float (&r)[1]) { r[0] = __ldcs(p); }
    static __device__ __forceinline__ void load_keep(const float* p, float (&r)[1]) { r[0] = __ldg(p); }
    static __device__ __forceinline__ void store(float* p, const float (&r)[1]) { __stcs(p, r[0]); }
    static __device__ __forceinline__ void store_keep(float* p, const float (&r)[1]) { *p = r[0]; }
};
template <>
struct VecIO<4> {
    static __device__ __forceinline__ void load(const float* p, float (&r)[4]) {
        float4 v = __ldcs(reinterpret_cast<const float4*>(p));
        r[0] = v.x, r[1] = v.y, r[2] = v.z, r[3] = v.w;
    }
    static __device__ __forceinline__ void load_keep(const float* p, float (&r)[4]) {
        float4 v = __ldg(reinterpret_cast<const float4*>(p));
        r[0] = v.x, r[1] = v.y, r[2] = v.z, r[3] = v.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&r)[4]) {
        __stcs(reinterpret_cast<float4*>(p), make_float4(r[0], r[1], r[2], r[3]));
    }
    static __device__ __forceinline__ void store_keep(float* p, const float (&r)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(r[0], r[1], r[2], r[3]);
    }
};

struct ScanGeom {
    size_t len, stride;       // time rows, channels per row
    unsigned cvecs;           // stride / V
    unsigned n_chunks;        // time chunks per lane
    unsigned chunk_len;       // rows per chunk (last may be short)
    size_t total;             // lanes * n_chunks * cvecs work items
};

// work item -> (lane, chunk, channel vector); consecutive threads take consecutive channel vectors
struct Item {
    size_t lane;
    unsigned chunk, cv;
};
__device__ __forceinline__ Item decode(const ScanGeom& g, size_t gid) {
    Item it;
    it.cv = (unsigned)(gid % g.cvecs);
    size_t rest = gid / g.cvecs;
    it.chunk = (unsigned)(rest % g.n_chunks);
    it.lane = rest / g.n_chunks;
    return it;
}

// pass 1: each chunk -> one composed map (A, B)
template <int V, int U>
__global__ void __launch_bounds__(128) scan_chunk_reduce(const float* __restrict__ a, const float* __restrict__ b,
                                                         float* __restrict__ agg_a, float* __restrict__ agg_b,
                                                         ScanGeom g) {
    size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= g.total) return;
    Item it = decode(g, gid);
    size_t t0 = (size_t)it.chunk * g.chunk_len;
    size_t t1 = min(g.len, t0 + g.chunk_len);
    size_t base = (it.lane * g.len + t0) * g.stride + (size_t)it.cv * V;
    const float* pa = a + base;
    const float* pb = b + base;
    float A[V], B[V];
#pragma unroll
    for (int v = 0; v < V; ++v) A[v] = 1.0f, B[v] = 0.0f;
    size_t t = t0;
    for (; t + U <= t1; t += U) {
        float av[U][V], bv[U][V];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            VecIO<V>::load_keep(pa + (size_t)u * g.stride, av[u]);
            VecIO<V>::load_keep(pb + (size_t)u * g.stride, bv[u]);
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int v = 0; v < V; ++v) {
                B[v] = __fadd_rn(__fmul_rn(av[u][v], B[v]), bv[u][v]);
                A[v] = __fmul_rn(av[u][v], A[v]);
            }
        pa += (size_t)U * g.stride;
        pb += (size_t)U * g.stride;
    }
    for (; t < t1; ++t) {
        float av[V], bv[V];
        VecIO<V>::load_keep(pa, av);
        VecIO<V>::load_keep(pb, bv);
#pragma unroll
        for (int v = 0; v < V; ++v) {
            B[v] = __fadd_rn(__fmul_rn(av[v], B[v]), bv[v]);
            A[v] = __fmul_rn(av[v], A[v]);
        }
        pa += g.stride;
        pb += g.stride;
    }
    size_t o = (it.lane * g.n_chunks + it.chunk) * g.stride + (size_t)it.cv * V;
    VecIO<V>::store_keep(agg_a + o, A);
    VecIO<V>::store_keep(agg_b + o, B);
}

// pass 2: serial walk over the chunk maps of one (lane, channel vector); writes each chunk's carry-in.
// MAPS = false: carry is a state (carry_b only, seeded from h0). MAPS = true: carry is a map (identity seed).
template <int V, bool MAPS>
__global__ void __launch_bounds__(128) scan_chunk_carry(const float* __restrict__ agg_a, const float* __restrict__ agg_b,
                                                        const float* __restrict__ h0, float* __restrict__ carry_a,
                                                        float* __restrict__ carry_b, ScanGeom g, size_t lanes) {
    size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= lanes * g.cvecs) return;
    unsigned cv = (unsigned)(gid % g.cvecs);
    size_t lane = gid / g.cvecs;
    float pa[V], pb[V];
#pragma unroll
    for (int v = 0; v < V; ++v) pa[v] = 1.0f, pb[v] = 0.0f;
    if (!MAPS && h0 != nullptr) VecIO<V>::load_keep(h0 + lane * g.stride + (size_t)cv * V, pb);
    for (unsigned c = 0; c < g.n_chunks; ++c) {
        size_t o = (lane * g.n_chunks + c) * g.stride + (size_t)cv * V;
        if (MAPS) VecIO<V>::store_keep(carry_a + o, pa);
        VecIO<V>::store_keep(carry_b + o, pb);
        float A[V], B[V];
        VecIO<V>::load_keep(agg_a + o, A);
        VecIO<V>::load_keep(agg_b + o, B);
#pragma unroll
        for (int v = 0; v < V; ++v) {
            pb[v] = __fadd_rn(__fmul_rn(A[v], pb[v]), B[v]);
            if (MAPS) pa[v] = __fmul_rn(A[v], pa[v]);
        }
    }
}

// pass 3 (the only pass when n_chunks == 1): scan a chunk from its carry-in and write the outputs.
// MAPS = false: out_b[t] = h_t (inclusive state).  MAPS = true: (out_a, out_b)[t] = exclusive prefix map.
template <int V, int U, bool MAPS>
__global__ void __launch_bounds__(128, MAPS ? 4 : 7)
    scan_chunk_apply(const float* a, const float* b, const float* __restrict__ carry_a,
                     const float* __restrict__ carry_b, float* out_a, float* out_b, float* __restrict__ last,
                     ScanGeom g) {
    size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= g.total) return;
    Item it = decode(g, gid);
    size_t t0 = (size_t)it.chunk * g.chunk_len;
    size_t t1 = min(g.len, t0 + g.chunk_len);
    size_t base = (it.lane * g.len + t0) * g.stride + (size_t)it.cv * V;
    const float* pa_in = a + base;
    const float* pb_in = b + base;
    float* po_a = MAPS ? out_a + base : nullptr;
    float* po_b = out_b + base;
    float ca[V], cb[V];
#pragma unroll
    for (int v = 0; v < V; ++v) ca[v] = 1.0f, cb[v] = 0.0f;
    size_t co = (it.lane * g.n_chunks + it.chunk) * g.stride + (size_t)it.cv * V;
    if (carry_b != nullptr) VecIO<V>::load_keep(carry_b + co, cb);
    if (MAPS && carry_a != nullptr) VecIO<V>::load_keep(carry_a + co, ca);
    size_t t = t0;
    for (; t + U <= t1; t += U) {
        float av[U][V], bv[U][V];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            VecIO<V>::load(pa_in + (size_t)u * g.stride, av[u]);
            VecIO<V>::load(pb_in + (size_t)u * g.stride, bv[u]);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (MAPS) {
                VecIO<V>::store(po_a + (size_t)u * g.stride, ca);
                VecIO<V>::store(po_b + (size_t)u * g.stride, cb);
            }
#pragma unroll
            for (int v = 0; v < V; ++v) {
                cb[v] = __fadd_rn(__fmul_rn(av[u][v], cb[v]), bv[u][v]);
                if (MAPS) ca[v] = __fmul_rn(av[u][v], ca[v]);
            }
            if (!MAPS) VecIO<V>::store(po_b + (size_t)u * g.stride, cb);
        }
        pa_in += (size_t)U * g.stride;
        pb_in += (size_t)U * g.stride;
        if (MAPS) po_a += (size_t)U * g.stride;
        po_b += (size_t)U * g.stride;
    }
    for (; t < t1; ++t) {
        float av[V], bv[V];
        VecIO<V>::load(pa_in, av);
        VecIO<V>::load(pb_in, bv);
        if (MAPS) {
            VecIO<V>::store(po_a, ca);
            VecIO<V>::store(po_b, cb);
        }
#pragma unroll
        for (int v = 0; v < V; ++v) {
            cb[v] = __fadd_rn(__fmul_rn(av[v], cb[v]), bv[v]);
            if (MAPS) ca[v] = __fmul_rn(av[v], ca[v]);
        }
        if (!MAPS) VecIO<V>::store(po_b, cb);
        pa_in += g.stride;
        pb_in += g.stride;
        if (MAPS) po_a += g.stride;
        po_b += g.stride;
    }
    if (!MAPS && last != nullptr && it.chunk == g.n_chunks - 1)
        VecIO<V>::store_keep(last + it.lane * g.stride + (size_t)it.cv * V, cb);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Split time only when channels alone leave SMs idle. Target: one resident wave of 128-thread CTAs.
unsigned pick_chunks(const pssa_b200_ctx* ctx, size_t lanes, size_t cvecs, size_t len) {
    size_t items = lanes * cvecs;
    size_t capacity = (size_t)ctx->sm_count * 7 * 128;
    if (items * 2 > capacity || len < 128) return 1;
    size_t want = capacity / items;
    size_t max_by_len = len / 64;  // keep chunks long enough that pass 1 + 2 stay cheap
    size_t n = want < max_by_len ? want : max_by_len;
    return (unsigned)(n < 1 ? 1 : n);
}

template <int V, bool MAPS>
int32_t run_scan(pssa_b200_ctx* ctx, const float* a, const float* b, const float* h0, float* out_a, float* out_b,
                 float* last, size_t lanes, size_t len, size_t stride, int forced_chunks) {
    ScanGeom g;
    g.len = len;
    g.stride = stride;
    g.cvecs = (unsigned)(stride / V);
    g.n_chunks = forced_chunks > 0 ? (unsigned)forced_chunks : pick_chunks(ctx, lanes, g.cvecs, len);
    if (g.n_chunks > len) g.n_chunks = (unsigned)len;
    g.chunk_len = (unsigned)((len + g.n_chunks - 1) / g.n_chunks);
    g.n_chunks = (unsigned)((len + g.chunk_len - 1) / g.chunk_len);
    g.total = lanes * g.n_chunks * g.cvecs;
    constexpr int U = MAPS ? 4 : 4;
    const int threads = 128;
    size_t blocks = (g.total + threads - 1) / threads;
    if (blocks > 0x7fffffffull)
        return fail(ctx, PSSA_B200_ERR_SHAPE, "B200 affine scan grid (%zu, 1) exceeds grid limits; refusing launch", blocks);
    const float* carry_a = nullptr;
    const float* carry_b = MAPS ? nullptr : h0;
    if (g.n_chunks > 1) {
        size_t per = lanes * g.n_chunks * stride * sizeof(float);
        arena_reset(ctx);
        int32_t rc = arena_reserve(ctx, arena_round(per) * 4);
        if (rc != PSSA_B200_OK) return rc;
        float* agg_a = (float*)arena_take(ctx, per);
        float* agg_b = (float*)arena_take(ctx, per);
        float* c_a = MAPS ? (float*)arena_take(ctx, per) : nullptr;
        float* c_b = (float*)arena_take(ctx, per);
        scan_chunk_reduce<V, 4><<<(unsigned)blocks, threads, 0, ctx->stream>>>(a, b, agg_a, agg_b, g);
        if ((rc = after_launch(ctx, "scan_chunk_reduce")) != PSSA_B200_OK) return rc;
        size_t cblocks = (lanes * g.cvecs + threads - 1) / threads;
        scan_chunk_carry<V, MAPS><<<(unsigned)cblocks, threads, 0, ctx->stream>>>(agg_a, agg_b, h0, c_a, c_b, g, lanes);
        if ((rc = after_launch(ctx, "scan_chunk_carry")) != PSSA_B200_OK) return rc;
        carry_a = c_a;
        carry_b = c_b;
    }
    scan_chunk_apply<V, U, MAPS><<<(unsigned)blocks, threads, 0, ctx->stream>>>(a, b, carry_a, carry_b, out_a, out_b, last, g);
    return after_launch(ctx, "scan_chunk_apply");
}

}  // namespace

int32_t launch_scan_states(pssa_b200_ctx* ctx, const float* a, const float* b, const float* h0, float* h, float* h_last,
                           size_t lanes, size_t len, size_t stride, int forced_chunks) {
    bool vec = stride % 4 == 0 && aligned16(a) && aligned16(b) && aligned16(h) && (!h0 || aligned16(h0)) &&
               (!h_last || aligned16(h_last));
    if (vec) return run_scan<4, false>(ctx, a, b, h0, nullptr, h, h_last, lanes, len, stride, forced_chunks);
    return run_scan<1, false>(ctx, a, b, h0, nullptr, h, h_last, lanes, len, stride, forced_chunks);
}

// ------------------------------------------------------------------ allocation-free variant
//
// Some hosts cannot let this library allocate device memory while they run: an inference server that
// has handed the whole GPU to its own pool at start-up, or a latency-critical loop in which the
// device-wide synchronisation hidden inside cudaMalloc / cudaFree is not acceptable. For them the
// chunk maps and carries of the multi-chunk scan live in the fixed array below instead of the
// context's growable arena. It is part of the module image, so every GPU that loads this library
// holds these 12 MiB until the process exits.
constexpr size_t kStaticScanFloats = size_t(3) << 20;  // 3 arrays (chunk A, chunk B, carry) x 2^20 floats
static __device__ __align__(256) float g_scan_static_scratch[kStaticScanFloats];

// In host code `g_scan_static_scratch` is only a handle for the runtime, not a device address; the address
// a kernel can use comes from cudaGetSymbolAddress, asked once per device with that device current.
static float* static_scratch_for_current_device(pssa_b200_ctx* ctx, int32_t* rc) {
    constexpr int kMaxDevices = 64;
    static std::atomic<float*> cached[kMaxDevices];  // two host threads may make their first call at once
    *rc = PSSA_B200_OK;
    if (ctx->device < 0 || ctx->device >= kMaxDevices) {
        *rc = fail(ctx, PSSA_B200_ERR_UNSUPPORTED, "static scan scratch: device ordinal %d is outside 0..%d", ctx->device, kMaxDevices - 1);
        return nullptr;
    }
    float* known = cached[ctx->device].load(std::memory_order_acquire);
    if (known == nullptr) {
        float* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_scan_static_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            *rc = cuda_fail(ctx, e, "cudaGetSymbolAddress(g_scan_static_scratch)");
            return nullptr;
        }
        cached[ctx->device].store(ptr, std::memory_order_release);
        known = ptr;
    }
    return known;
}

template <int V>
static int32_t run_scan_states_static(pssa_b200_ctx* ctx, const float* a, const float* b, const float* h0, float* h, float* last,
                                      size_t lanes, size_t len, size_t stride, unsigned chunks) {
    ScanGeom g;
    g.len = len;
    g.stride = stride;
    g.cvecs = (unsigned)(stride / V);
    g.n_chunks = chunks > len ? (unsigned)len : chunks;
    g.chunk_len = (unsigned)((len + g.n_chunks - 1) / g.n_chunks);
    g.n_chunks = (unsigned)((len + g.chunk_len - 1) / g.chunk_len);
    g.total = lanes * g.n_chunks * g.cvecs;
    const int threads = 128;
    size_t blocks = (g.total + threads - 1) / threads;
    if (blocks > 0x7fffffffull)
        return fail(ctx, PSSA_B200_ERR_SHAPE, "B200 affine scan grid (%zu, 1) exceeds grid limits; refusing launch", blocks);
    const float* carry = h0;
    if (g.n_chunks > 1) {
        size_t per = lanes * g.n_chunks * stride;  // floats in each of the three scratch arrays
        if (per > kStaticScanFloats / 3)
            return fail(ctx, PSSA_B200_ERR_SHAPE,
                        "B200 static scan: lanes*chunks*stride = %zu floats exceeds the fixed scratch of %zu floats per array; "
                        "use fewer chunks or the arena-backed entry point; refusing launch",
                        per, kStaticScanFloats / 3);
        int32_t rc;
        float* base = static_scratch_for_current_device(ctx, &rc);
        if (!base) return rc;
        // every element of the three arrays that pass 2 and 3 read is written by pass 1 / 2 of this same call,
        // so nothing left behind by an earlier call is ever observed and no clearing is needed
        float* agg_a = base;
        float* agg_b = base + kStaticScanFloats / 3;
        float* c_b = base + 2 * (kStaticScanFloats / 3);
        scan_chunk_reduce<V, 4><<<(unsigned)blocks, threads, 0, ctx->stream>>>(a, b, agg_a, agg_b, g);
        if ((rc = after_launch(ctx, "scan_chunk_reduce")) != PSSA_B200_OK) return rc;
        size_t cblocks = (lanes * g.cvecs + threads - 1) / threads;
        scan_chunk_carry<V, false><<<(unsigned)cblocks, threads, 0, ctx->stream>>>(agg_a, agg_b, h0, nullptr, c_b, g, lanes);
        if ((rc = after_launch(ctx, "scan_chunk_carry")) != PSSA_B200_OK) return rc;
        carry = c_b;
    }
    scan_chunk_apply<V, 4, false><<<(unsigned)blocks, threads, 0, ctx->stream>>>(a, b, nullptr, carry, nullptr, h, last, g);
    return after_launch(ctx, "scan_chunk_apply");
}

int32_t launch_scan_states_static(pssa_b200_ctx* ctx, const float* a, const float* b, const float* h0, float* h, float* h_last,
                                  size_t lanes, size_t len, size_t stride, unsigned chunks) {
    bool vec = stride % 4 == 0 && aligned16(a) && aligned16(b) && aligned16(h) && (!h0 || aligned16(h0)) &&
               (!h_last || aligned16(h_last));
    if (vec) return run_scan_states_static<4>(ctx, a, b, h0, h, h_last, lanes, len, stride, chunks);
    return run_scan_states_static<1>(ctx, a, b, h0, h, h_last, lanes, len, stride, chunks);
}

int32_t launch_scan_maps(pssa_b200_ctx* ctx, float* scan_a, float* scan_b, size_t lanes, size_t len, size_t stride,
                         int forced_chunks) {
    bool vec = stride % 4 == 0 && aligned16(scan_a) && aligned16(scan_b);
    if (vec) return run_scan<4, true>(ctx, scan_a, scan_b, nullptr, scan_a, scan_b, nullptr, lanes, len, stride, forced_chunks);
    return run_scan<1, true>(ctx, scan_a, scan_b, nullptr, scan_a, scan_b, nullptr, lanes, len, stride, forced_chunks);
}

}  // namespace pssa
