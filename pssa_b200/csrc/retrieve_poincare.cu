// Poincare-ball episodic memory read: project queries into the ball, hyperbolic distance to every
// occupied slot, softmax (all slots or exact top-k) and the weighted value read.
//
// Replaces `retrieve_soft_into` / `diffeomorphic_project` / `poincare_distance`
// (src/memory.rs:198-211, 245-262, 344-426), the per-token loop `retrieve_memory_rows`
// (src/gpu_batch.rs:700-741) and the reference's GPU kernel `memory_forward` (one thread per token,
// src/cuda/stages.ptx:358-446) with its cuBLAS value read (src/cuda/stages.rs:583-614).
//
// Three launches:
//   A  poincare_distance_kernel: 64 queries x 64 slots per CTA pass, 4x4 (query, slot) pairs per
//      thread, squared differences accumulated in f64 exactly like the reference (projection and
//      distance are f64 there, rounded to f32); distances go to the [rows, cap] weights buffer.
//   B  softmax_topk_kernel: one warp per query: min, exp((min-d)/tau), normalise; or exact top-k by
//      (distance bits, slot) with the value read fused (k rows of the bank).
//   C  value_mix_kernel: m = W[rows, count] x V[count, dv] for the all-slots read, fp32, slots
//      accumulated in ascending order like the reference.
// B and C keep the reference's sequential f32 summation order when `exact` is set.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>

#include <algorithm>
#include <cfloat>
#include <math_constants.h>

#include "bounds.hpp"
#include "context.hpp"
#include "device_math.cuh"
#include "kernels.hpp"

namespace pssa {
namespace {

constexpr int QT = 64;   // queries per CTA in kernel A
constexpr int STL = 64;  // slots per pass

// ------------------------------------------------------------------ A: projection + distances
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sa), "l"(gmem));
}

// Shared memory: P as f64 [dimension][query] (a thread's four queries are two 16-byte reads, broadcast over the slot
// threads); key tiles stay fp32, row-major [slot][kpad + 4], in two buffers filled by cp.async one pass ahead and are
// widened to f64 as they are read (exact). A thread owns queries tq*4 + a and slots ts + 16*b.
__global__ void __launch_bounds__(256) poincare_distance_kernel(RetrieveParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int kpad = (p.dk + 3) / 4 * 4;
    const int kpitch = kpad + 4;
    double* Ps = reinterpret_cast<double*>(smem_raw);               // [kpad][QT]
    float* Ks = reinterpret_cast<float*>(Ps + (size_t)kpad * QT);   // [2][STL][kpitch]
    float* qsq = Ks + 2 * (size_t)STL * kpitch;                     // [QT]

    const int tid = threadIdx.x;
    const size_t q0 = (size_t)blockIdx.x * QT;
    const int dk = p.dk, count = p.count;
    const bool vec_in = (dk & 3) == 0 && (reinterpret_cast<uintptr_t>(p.keys) & 15) == 0;

    auto load_keys = [&](int pass, int buf) {
        const int s0 = pass * STL;
        if (s0 < count) {
            float* dst = Ks + (size_t)buf * STL * kpitch;
            if (vec_in) {
                const int c4n = dk >> 2;
                for (int idx = tid; idx < STL * c4n; idx += 256) {
                    const int sl = idx / c4n, c4 = idx % c4n;
                    if (s0 + sl < count)
                        cp_async16(dst + sl * kpitch + c4 * 4, p.keys + (size_t)(s0 + sl) * dk + c4 * 4);
                    else
                        *reinterpret_cast<float4*>(dst + sl * kpitch + c4 * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            } else {
                for (int idx = tid; idx < STL * kpad; idx += 256) {
                    const int sl = idx / kpad, i = idx % kpad;
                    dst[sl * kpitch + i] = (s0 + sl < count && i < dk) ? __ldg(p.keys + (size_t)(s0 + sl) * dk + i) : 0.0f;
                }
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    load_keys(blockIdx.y, 0);

    // zero the padded rows of P
    for (int idx = tid; idx < (kpad - dk) * QT; idx += 256) Ps[(size_t)dk * QT + idx] = 0.0;

    if (tid < QT) {
        const size_t q = q0 + tid;
        const bool publish = blockIdx.y == 0;  // the slot passes of one query tile may be spread over several CTAs
        if (q < p.rows) {
            const float* src = p.q + q * (p.ldq ? p.ldq : (size_t)dk);
            float* dst = (p.q_pnc && publish) ? p.q_pnc + q * dk : nullptr;
            float qs;
            if (p.q_is_euclidean) {
                // memory.rs:198-211: r = sqrt(sum q^2) in f64, sequential; p = q * min(r/(1+r), R)/r
                double r2 = 0.0;
                for (int i = 0; i < dk; ++i) {
                    double v = (double)src[i];
                    r2 = __dadd_rn(r2, __dmul_rn(v, v));
                }
                double r = sqrt(r2);
                const double max_radius = 1.0 - 8.0 * (double)FLT_EPSILON;
                double scale = (r == 0.0) ? 1.0 : fmin(r / (1.0 + r), max_radius) / r;
                double n2 = 0.0;
                for (int i = 0; i < dk; ++i) {
                    float pv = (float)__dmul_rn((double)src[i], scale);
                    if (dst) dst[i] = pv;
                    double pd = (double)pv;
                    Ps[(size_t)i * QT + tid] = pd;
                    n2 = __dadd_rn(n2, __dmul_rn(pd, pd));
                }
                if (p.q_norm && publish) p.q_norm[q] = (float)fmin(r, (double)FLT_MAX);
                qs = (n2 < 1.0 && (float)n2 == 1.0f) ? __uint_as_float(0x3f7fffffu) : (float)n2;  // memory.rs:181-188
            } else {
                double n2 = 0.0;
                for (int i = 0; i < dk; ++i) {
                    float pv = src[i];
                    if (dst) dst[i] = pv;
                    double pd = (double)pv;
                    Ps[(size_t)i * QT + tid] = pd;
                    n2 = __dadd_rn(n2, __dmul_rn(pd, pd));
                }
                qs = (n2 < 1.0 && (float)n2 == 1.0f) ? __uint_as_float(0x3f7fffffu) : (float)n2;
            }
            qsq[tid] = qs;
        } else {
            for (int i = 0; i < dk; ++i) Ps[(size_t)i * QT + tid] = 0.0;
            qsq[tid] = 0.0f;
        }
    }

    const int ts = tid & 15, tq = tid >> 4;  // 16 slot threads x 16 query threads
    const int npass = (count + STL - 1) / STL;
    for (int pass = blockIdx.y, buf = 0; pass < npass; pass += gridDim.y, buf ^= 1) {
        asm volatile("cp.async.wait_group 0;\n" ::);
        __syncthreads();      // this tile (and, first time round, P) visible; everyone is done with the previous tile
        load_keys(pass + gridDim.y, buf ^ 1);  // lands while this tile is consumed
        const float* kt = Ks + (size_t)buf * STL * kpitch;
        double acc[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) acc[a][b] = 0.0;
        for (int i4 = 0; i4 < kpad / 4; ++i4) {
            double kd[4][4];  // [slot b][dimension]
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const float4 k = *reinterpret_cast<const float4*>(kt + (ts + 16 * b) * kpitch + i4 * 4);
                kd[b][0] = (double)k.x, kd[b][1] = (double)k.y, kd[b][2] = (double)k.z, kd[b][3] = (double)k.w;
            }
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                const double2* pp = reinterpret_cast<const double2*>(Ps + (size_t)(i4 * 4 + h) * QT + tq * 4);
                const double2 p01 = pp[0], p23 = pp[1];
                const double pv[4] = {p01.x, p01.y, p23.x, p23.y};
#pragma unroll
                for (int a = 0; a < 4; ++a)
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        const double df = pv[a] - kd[b][h];
                        acc[a][b] = fma(df, df, acc[a][b]);
                    }
            }
        }
        const int s0 = pass * STL;
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const size_t q = q0 + tq * 4 + a;
            if (q >= p.rows) continue;
            const double one_minus_q = 1.0 - (double)qsq[tq * 4 + a];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int slot = s0 + ts + 16 * b;
                if (slot < count) {
                    // memory.rs:245-262: 2*asinh(sqrt(sq/denom)); 2*asinh(z) = log1p(2u + 2*sqrt(u*u + u)), u = z^2
                    double denom = one_minus_q * (1.0 - (double)__ldg(p.norm_sq + slot));
                    double u = acc[a][b] / denom;
                    double dist = log1p(2.0 * u + 2.0 * sqrt(fma(u, u, u)));
                    p.weights[q * p.cap + slot] = (float)dist;
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
}

// ------------------------------------------------------------------ A': fp32 distances (fast mode)
// Same tiling as kernel A with the squared differences accumulated in fp32. Differences are formed first, as in the
// reference, so near-coincident points lose nothing to cancellation: the squared distance carries a relative error of
// about 1e-6 (64 roundings), the distance half of that. The projection is the f64 one (bit-identical q_pnc). Two key
// dimensions travel together as one packed f32x2 register so a (query, slot, dimension pair) costs two instructions.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ float sum2(f32x2 v) {
    float lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
    return lo + hi;
}

// Shared memory: P as [dimension pair][query] float2 (a thread's four queries are one 32-byte read, broadcast over the
// slot threads), key tiles row-major [slot][kpad + 4] in two buffers filled by cp.async one pass ahead. A thread owns
// queries tq*4 + a and slots ts + 16*b: consecutive slot threads sit 68 floats apart, so their 16-byte key reads hit
// disjoint banks and their distance stores are 64-byte runs.
__global__ void __launch_bounds__(256, 3) poincare_distance_f32_kernel(RetrieveParams p) {
    pdl_trigger();  // the next kernel in the stream may start its prologue now ...
    pdl_wait();     // ... and this one, if launched as a dependent, waits here for its own predecessor
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int kpad = (p.dk + 3) / 4 * 4;
    const int kpitch = kpad + 4;
    float2* Pf = reinterpret_cast<float2*>(smem_raw);                 // [kpad/2][QT]
    float* Ks = reinterpret_cast<float*>(Pf + (size_t)(kpad / 2) * QT);  // [2][STL][kpitch]
    float* rq = Ks + 2 * (size_t)STL * kpitch;                        // [QT]     1 / (1 - |p|^2)
    float* rk = rq + QT;                                              // [2][STL] 1 / (1 - |k|^2)

    const int tid = threadIdx.x;
    const size_t q0 = (size_t)blockIdx.x * QT;
    const int dk = p.dk, count = p.count;
    const bool vec_in = (dk & 3) == 0 && (reinterpret_cast<uintptr_t>(p.keys) & 15) == 0;

    // passes over the slots are dealt round-robin to the CTAs of a column (gridDim.y > 1 only when there are too few
    // query tiles to fill the machine: decode steps); `buf` alternates per pass this CTA owns
    auto load_keys = [&](int pass, int buf) {
        const int s0 = pass * STL;
        if (s0 < count) {
            float* dst = Ks + (size_t)buf * STL * kpitch;
            if (vec_in) {
                const int c4n = dk >> 2;
                for (int idx = tid; idx < STL * c4n; idx += 256) {
                    const int sl = idx / c4n, c4 = idx % c4n;
                    if (s0 + sl < count)
                        cp_async16(dst + sl * kpitch + c4 * 4, p.keys + (size_t)(s0 + sl) * dk + c4 * 4);
                    else
                        *reinterpret_cast<float4*>(dst + sl * kpitch + c4 * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            } else {
                for (int idx = tid; idx < STL * kpad; idx += 256) {
                    const int sl = idx / kpad, i = idx % kpad;
                    dst[sl * kpitch + i] = (s0 + sl < count && i < dk) ? __ldg(p.keys + (size_t)(s0 + sl) * dk + i) : 0.0f;
                }
            }
            if (tid < STL)
                rk[buf * STL + tid] = s0 + tid < count ? (float)(1.0 / (1.0 - (double)__ldg(p.norm_sq + s0 + tid))) : 0.0f;
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    load_keys(blockIdx.y, 0);

    float* Pflat = reinterpret_cast<float*>(Pf);
    for (int idx = tid; idx < (kpad - dk) * QT; idx += 256) {  // zero the padded dimensions
        int i = dk + idx / QT, qq = idx % QT;
        Pflat[((size_t)(i >> 1) * QT + qq) * 2 + (i & 1)] = 0.0f;
    }
    if (tid < QT) {
        const size_t q = q0 + tid;
        float qs = 0.0f;
        if (q < p.rows) {
            const float* src = p.q + q * (p.ldq ? p.ldq : (size_t)dk);
            float* dst = (p.q_pnc && blockIdx.y == 0) ? p.q_pnc + q * dk : nullptr;
            double scale = 1.0;
            if (p.q_is_euclidean) {  // memory.rs:198-211
                double r2 = 0.0;
                for (int i = 0; i < dk; ++i) {
                    double v = (double)src[i];
                    r2 = __dadd_rn(r2, __dmul_rn(v, v));
                }
                double r = sqrt(r2);
                const double max_radius = 1.0 - 8.0 * (double)FLT_EPSILON;
                scale = (r == 0.0) ? 1.0 : fmin(r / (1.0 + r), max_radius) / r;
                if (p.q_norm && blockIdx.y == 0) p.q_norm[q] = (float)fmin(r, (double)FLT_MAX);
            }
            double n2 = 0.0;
            for (int i = 0; i < dk; ++i) {
                float pv = p.q_is_euclidean ? (float)__dmul_rn((double)src[i], scale) : src[i];
                if (dst) dst[i] = pv;
                Pflat[((size_t)(i >> 1) * QT + tid) * 2 + (i & 1)] = pv;
                n2 = __dadd_rn(n2, __dmul_rn((double)pv, (double)pv));
            }
            qs = (n2 < 1.0 && (float)n2 == 1.0f) ? __uint_as_float(0x3f7fffffu) : (float)n2;  // memory.rs:181-188
        } else {
            for (int i = 0; i < dk; ++i) Pflat[((size_t)(i >> 1) * QT + tid) * 2 + (i & 1)] = 0.0f;
        }
        rq[tid] = (float)(1.0 / (1.0 - (double)qs));
    }

    const int ts = tid & 15, tq = tid >> 4;
    const int npass = (count + STL - 1) / STL;
    for (int pass = blockIdx.y, buf = 0; pass < npass; pass += gridDim.y, buf ^= 1) {
        asm volatile("cp.async.wait_group 0;\n" ::);
        __syncthreads();      // this tile (and, first time round, P) visible; everyone is done with the previous tile
        load_keys(pass + gridDim.y, buf ^ 1);  // lands while this tile is consumed
        const float* kt = Ks + (size_t)buf * STL * kpitch;
        f32x2 acc[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) acc[a][b] = 0ull;
#pragma unroll 2
        for (int i4 = 0; i4 < kpad / 4; ++i4) {
            f32x2 kv[4][2], pv[4][2];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const ulonglong2 k = *reinterpret_cast<const ulonglong2*>(kt + (ts + 16 * b) * kpitch + i4 * 4);
                kv[b][0] = k.x, kv[b][1] = k.y;
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const ulonglong2* pp = reinterpret_cast<const ulonglong2*>(Pf + (size_t)(i4 * 2 + h) * QT + tq * 4);
                const ulonglong2 p01 = pp[0], p23 = pp[1];
                pv[0][h] = p01.x, pv[1][h] = p01.y, pv[2][h] = p23.x, pv[3][h] = p23.y;
            }
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int a = 0; a < 4; ++a)
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        const f32x2 df = sub2(pv[a][h], kv[b][h]);
                        acc[a][b] = fma2(df, df, acc[a][b]);
                    }
        }
        const int s0 = pass * STL;
        const float* rkt = rk + buf * STL;
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const size_t q = q0 + tq * 4 + a;
            if (q >= p.rows) continue;
            const float rqa = rq[tq * 4 + a];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int slot = s0 + ts + 16 * b;
                // memory.rs:245-262 with u = sq / ((1-|p|^2)(1-|k|^2))
                if (slot < count) p.weights[q * p.cap + slot] = fast_poincare_distance(sum2(acc[a][b]) * (rqa * rkt[ts + 16 * b]));
            }
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
}

// x = x0 + x1 + x2 with bf16 pieces: 24 bits of significand survive, so products of pieces reproduce fp32 products
__device__ __forceinline__ void split3(float x, __nv_bfloat16& a, __nv_bfloat16& b, __nv_bfloat16& c) {
    a = __float2bfloat16_rn(x);
    float r = x - __bfloat162float(a);
    b = __float2bfloat16_rn(r);
    c = __float2bfloat16_rn(r - __bfloat162float(b));
}

__global__ void __launch_bounds__(256) split_values_kernel(const float* __restrict__ values, __nv_bfloat16* __restrict__ out,
                                                           int cap, int dv) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)cap * dv) return;
    int slot = (int)(idx / dv), col = (int)(idx % dv);
    __nv_bfloat16 a, b, c;
    split3(values[idx], a, b, c);
    __nv_bfloat16* row = out + (size_t)col * 3 * cap;
    row[slot] = a, row[cap + slot] = b, row[2 * cap + slot] = c;
}

// keys [cap, dk] fp32 -> k_split [cap, 3*dk] bf16 (three pieces side by side) and k_stat[slot] = (|k|^2, 1/(1-|k|^2))
__global__ void __launch_bounds__(256) split_keys_kernel(const float* __restrict__ keys, const float* __restrict__ norm_sq,
                                                         __nv_bfloat16* __restrict__ out, float2* __restrict__ stat, int cap, int dk) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < (size_t)cap) {
        const float n = __ldg(norm_sq + idx);
        stat[idx] = make_float2(n, (float)(1.0 / (1.0 - (double)n)));
    }
    if (idx >= (size_t)cap * dk) return;
    int slot = (int)(idx / dk), col = (int)(idx % dk);
    __nv_bfloat16 a, b, c;
    split3(keys[idx], a, b, c);
    __nv_bfloat16* row = out + (size_t)slot * 3 * dk;
    row[col] = a, row[dk + col] = b, row[2 * dk + col] = c;
}

// Queries for the tensor-core distance: the reference's projection into the ball (src/memory.rs:198-211, f64, the same
// sequential sums as the distance kernels, so q_pnc has the same bits), then the point as three bf16 pieces
// q_split [rows, 3*dk] and q_stat[row] = (|p|^2, 1/(1-|p|^2)). One CTA = 64 rows: the tile is staged in shared memory
// with coalesced loads, 64 threads walk one row each, all 256 write the pieces.
__global__ void __launch_bounds__(256) project_split_kernel(RetrieveParams p) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float tile[];  // [QT][dk + 1]
    const int dk = p.dk, pitch = dk + 1, tid = threadIdx.x;
    const size_t q0 = (size_t)blockIdx.x * QT;
    const size_t ldq = p.ldq ? p.ldq : (size_t)dk;
    const float* __restrict__ qsrc = p.q;
#pragma unroll 8
    for (int idx = tid; idx < QT * dk; idx += 256) {  // unrolled so that a thread's loads are in flight together
        const int r = idx / dk, c = idx % dk;
        tile[r * pitch + c] = q0 + r < p.rows ? __ldg(qsrc + (q0 + r) * ldq + c) : 0.0f;
    }
    __syncthreads();
    if (tid < QT && q0 + tid < p.rows) {
        float* row = tile + tid * pitch;
        double scale = 1.0;
        if (p.q_is_euclidean) {
            double r2 = 0.0;
            for (int i = 0; i < dk; ++i) {
                double v = (double)row[i];
                r2 = __dadd_rn(r2, __dmul_rn(v, v));
            }
            double r = sqrt(r2);
            const double max_radius = 1.0 - 8.0 * (double)FLT_EPSILON;
            scale = (r == 0.0) ? 1.0 : fmin(r / (1.0 + r), max_radius) / r;
            if (p.q_norm) p.q_norm[q0 + tid] = (float)fmin(r, (double)FLT_MAX);
        }
        double n2 = 0.0;
        for (int i = 0; i < dk; ++i) {
            float pv = p.q_is_euclidean ? (float)__dmul_rn((double)row[i], scale) : row[i];
            row[i] = pv;
            n2 = __dadd_rn(n2, __dmul_rn((double)pv, (double)pv));
        }
        const float qs = (n2 < 1.0 && (float)n2 == 1.0f) ? __uint_as_float(0x3f7fffffu) : (float)n2;  // memory.rs:181-188
        p.q_stat[q0 + tid] = make_float2(qs, (float)(1.0 / (1.0 - (double)qs)));
    }
    __syncthreads();
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.q_split);
    for (int idx = tid; idx < QT * dk / 2; idx += 256) {
        const int r = idx / (dk / 2), c = (idx % (dk / 2)) * 2;
        if (q0 + r >= p.rows) break;
        const float v0 = tile[r * pitch + c], v1 = tile[r * pitch + c + 1];
        if (p.q_pnc) *reinterpret_cast<float2*>(p.q_pnc + (q0 + r) * dk + c) = make_float2(v0, v1);
        __nv_bfloat16 a0, b0, c0, a1, b1, c1;
        split3(v0, a0, b0, c0);
        split3(v1, a1, b1, c1);
        __nv_bfloat16* o = out + (q0 + r) * 3 * dk + c;
        *reinterpret_cast<__nv_bfloat162*>(o) = __halves2bfloat162(a0, a1);
        *reinterpret_cast<__nv_bfloat162*>(o + dk) = __halves2bfloat162(b0, b1);
        *reinterpret_cast<__nv_bfloat162*>(o + 2 * dk) = __halves2bfloat162(c0, c1);
    }
}

// ------------------------------------------------------------------ B: softmax / top-k (+ fused value read)
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, m));
    return v;
}
__device__ __forceinline__ unsigned long long warp_min_u64(unsigned long long v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        unsigned long long o = __shfl_xor_sync(0xffffffffu, v, m);
        v = o < v ? o : v;
    }
    return v;
}

__device__ __forceinline__ float exp2f_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

constexpr int kTopkRegs = 16;  // distances per lane the register path of the top-k selection holds (capacity <= 512)

template <bool EXACT>
__device__ __forceinline__ float weight_of(float min_dist, float d, float tau) {
    // memory.rs:396-398 / 411-414: exp((min - d) / tau), subtraction before division
    float x = __fdiv_rn(__fsub_rn(min_dist, d), tau);
    return expf(x);
}

// All-slots softmax out of registers (non-exact mode, capacity a multiple of 128 and at most 128 * GROUPS, at least one
// stored slot): a lane owns four consecutive slots of every 128 and rows move as 16-byte pieces; a warp walks rows
// q, q + stride, ... with the next row's distances already in flight. Same formulas as the general kernel below (the sum
// is grouped differently). value_terms == 1 or 3: the consumer keeps bf16-grade results (one or two leading pieces of every weight),
// so the weights may use ex2.approx and one reciprocal per row (relative error near 1e-6 instead of 1e-7); a temperature
// too small for a finite reciprocal keeps the division.
template <int GROUPS>
__global__ void __launch_bounds__(256) softmax_all_slots_kernel(RetrieveParams p) {
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cap = p.cap, count = p.count;
    const float tau = p.tau;
    const float inv_tau = 1.0f / tau;
    const bool lite = (p.value_terms == 3 || p.value_terms == 1) && inv_tau < CUDART_INF_F;
    const bool second = p.value_terms != 1;  // the one-term read uses the leading piece only
    const float scale2 = inv_tau * 1.4426950408889634f;
    const size_t stride = (size_t)gridDim.x * 8;
    size_t q = (size_t)blockIdx.x * 8 + warp;
    if (q >= p.rows) return;
    auto load_row = [&](size_t qq, float4* dst) {
        const float* src = p.weights + qq * cap;
#pragma unroll
        for (int g = 0; g < GROUPS; ++g) {
            const int i = g * 128 + lane * 4;
            if (i < count) dst[g] = *reinterpret_cast<const float4*>(src + i);
        }
    };
    float4 nxt[GROUPS];
    load_row(q, nxt);
    for (; q < p.rows; q += stride) {
        float4 dg[GROUPS];
        float mn = FLT_MAX;
#pragma unroll
        for (int g = 0; g < GROUPS; ++g) {
            const int i = g * 128 + lane * 4;
            // slots past `count` hold nothing: an infinite distance gives them weight zero
            float4 d4 = nxt[g];
            d4.x = i + 0 < count ? d4.x : CUDART_INF_F, d4.y = i + 1 < count ? d4.y : CUDART_INF_F;
            d4.z = i + 2 < count ? d4.z : CUDART_INF_F, d4.w = i + 3 < count ? d4.w : CUDART_INF_F;
            dg[g] = d4;
            mn = fminf(fminf(mn, fminf(d4.x, d4.y)), fminf(d4.z, d4.w));
        }
        if (q + stride < p.rows) load_row(q + stride, nxt);
        mn = warp_min(mn);
        if (p.min_dist && lane == 0) p.min_dist[q] = mn;
        auto wt = [&](float d) { return lite ? exp2f_approx((mn - d) * scale2) : weight_of<false>(mn, d, tau); };
        float sum = 0.0f;
#pragma unroll
        for (int g = 0; g < GROUPS; ++g) {
            if (g * 128 < cap) {
                dg[g].x = wt(dg[g].x), dg[g].y = wt(dg[g].y), dg[g].z = wt(dg[g].z), dg[g].w = wt(dg[g].w);
                sum += (dg[g].x + dg[g].y) + (dg[g].z + dg[g].w);
            }
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
        float* row = p.weights + q * cap;
        __nv_bfloat16* ws = p.w_split ? reinterpret_cast<__nv_bfloat16*>(p.w_split) + q * 3 * (size_t)cap : nullptr;
        const float inv_sum = __fdiv_rn(1.0f, sum);
#pragma unroll
        for (int g = 0; g < GROUPS; ++g) {
            const int i = g * 128 + lane * 4;
            if (i < cap) {
                float wn[4] = {dg[g].x, dg[g].y, dg[g].z, dg[g].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) wn[e] = lite ? wn[e] * inv_sum : __fdiv_rn(wn[e], sum);
                if (!p.skip_weights) *reinterpret_cast<float4*>(row + i) = make_float4(wn[0], wn[1], wn[2], wn[3]);
                if (ws && lite) {  // the three-term read never touches the last piece
                    __nv_bfloat16 pa[4], pb[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        pa[e] = __float2bfloat16_rn(wn[e]);
                        pb[e] = __float2bfloat16_rn(wn[e] - __bfloat162float(pa[e]));
                    }
                    *reinterpret_cast<uint2*>(ws + i) = *reinterpret_cast<const uint2*>(pa);
                    if (second) *reinterpret_cast<uint2*>(ws + cap + i) = *reinterpret_cast<const uint2*>(pb);
                } else if (ws) {
                    __nv_bfloat16 pa[4], pb[4], pc[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) split3(wn[e], pa[e], pb[e], pc[e]);
                    *reinterpret_cast<uint2*>(ws + i) = *reinterpret_cast<const uint2*>(pa);
                    *reinterpret_cast<uint2*>(ws + cap + i) = *reinterpret_cast<const uint2*>(pb);
                    *reinterpret_cast<uint2*>(ws + 2 * cap + i) = *reinterpret_cast<const uint2*>(pc);
                }
            }
        }
    }
}

// One token per stream (a decode step): projection, distances, softmax and the weight pieces of the all-slots
// read in ONE launch, one CTA per four queries (a key row is loaded once for the four). With a few hundred rows each of the
// separate kernels is a chain of launch and memory latencies, not work; here the rows never leave the CTA. Same
// formulas as the separate fast-mode kernels: the projection in f64 (lane-partial sums combined in a fixed order
// instead of one sequential sum: the f64 result differs in its last bits, the f32 point almost never), squared
// differences accumulated in fp32 (differences first), the hardware-approximation distance, ex2.approx weights with one
// reciprocal per row, bf16 pieces for the tensor-core value read. Only for the bf16-grade consumers (value_terms 1 or 3).
constexpr int kSmallRows = 4;
__global__ void __launch_bounds__(256) retrieve_small_rows_kernel(RetrieveParams p) {
    pdl_trigger();
    pdl_wait();
    constexpr int R = kSmallRows;
    __shared__ __align__(16) float pt[R][256];  // the queries, then the projected points (dk <= 256)
    __shared__ float red[8][R];
    __shared__ float row_inv[R];                // 1 / (1 - |p|^2)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int dk = p.dk, cap = p.cap, count = p.count;
    const size_t q0 = (size_t)blockIdx.x * R;
    const size_t ldq = p.ldq ? p.ldq : (size_t)dk;
    for (int idx = tid; idx < R * dk; idx += 256) {
        const int r = idx / dk, i = idx - r * dk;
        pt[r][i] = q0 + r < p.rows ? __ldg(p.q + (q0 + r) * ldq + i) : 0.0f;
    }
    __syncthreads();
    if (warp < R) {  // one warp per query: src/memory.rs:198-211, 181-188
        const int r = warp;
        const size_t q = q0 + r;
        double scale = 1.0;
        if (p.q_is_euclidean) {
            double r2 = 0.0;
            for (int i = lane; i < dk; i += 32) r2 += (double)pt[r][i] * (double)pt[r][i];
#pragma unroll
            for (int m = 16; m > 0; m >>= 1) r2 += __shfl_xor_sync(0xffffffffu, r2, m);
            const double rad = sqrt(r2);
            const double max_radius = 1.0 - 8.0 * (double)FLT_EPSILON;
            scale = (rad == 0.0) ? 1.0 : fmin(rad / (1.0 + rad), max_radius) / rad;
            if (p.q_norm && lane == 0 && q < p.rows) p.q_norm[q] = (float)fmin(rad, (double)FLT_MAX);
        }
        double n2 = 0.0;
        for (int i = lane; i < dk; i += 32) {
            const float pv = p.q_is_euclidean ? (float)((double)pt[r][i] * scale) : pt[r][i];
            pt[r][i] = pv;
            if (p.q_pnc && q < p.rows) p.q_pnc[q * dk + i] = pv;
            n2 += (double)pv * (double)pv;
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) n2 += __shfl_xor_sync(0xffffffffu, n2, m);
        if (lane == 0) {
            const float qs = (n2 < 1.0 && (float)n2 == 1.0f) ? __uint_as_float(0x3f7fffffu) : (float)n2;
            row_inv[r] = (float)(1.0 / (1.0 - (double)qs));
        }
    }
    __syncthreads();
    constexpr int PER = 4;  // slots per thread: capacity <= 1024
    float d[R][PER];
    float mn[R];
#pragma unroll
    for (int r = 0; r < R; ++r) mn[r] = FLT_MAX;
    const bool vec = (dk & 3) == 0 && (reinterpret_cast<uintptr_t>(p.keys) & 15) == 0;
#pragma unroll
    for (int u = 0; u < PER; ++u) {
        const int s = tid + u * 256;
#pragma unroll
        for (int r = 0; r < R; ++r) d[r][u] = CUDART_INF_F;  // slots past `count` hold nothing: weight zero
        if (s < count) {
            const float* krow = p.keys + (size_t)s * dk;
            float sq[R];
#pragma unroll
            for (int r = 0; r < R; ++r) sq[r] = 0.0f;
            if (vec && (dk & 31) == 0) {
                // eight 16-byte loads of the key row in flight before they are used: the row comes from L2 and the walk
                // is otherwise one round trip per load
                for (int i0 = 0; i0 < dk; i0 += 32) {
                    float4 kv[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) kv[j] = __ldg(reinterpret_cast<const float4*>(krow + i0) + j);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            const float4 pv = *reinterpret_cast<const float4*>(&pt[r][i0 + 4 * j]);
                            const float a = pv.x - kv[j].x, b = pv.y - kv[j].y, c = pv.z - kv[j].z, e = pv.w - kv[j].w;
                            sq[r] = fmaf(a, a, sq[r]), sq[r] = fmaf(b, b, sq[r]), sq[r] = fmaf(c, c, sq[r]), sq[r] = fmaf(e, e, sq[r]);
                        }
                    }
                }
            } else if (vec) {
                for (int i = 0; i < dk; i += 4) {
                    const float4 kv = __ldg(reinterpret_cast<const float4*>(krow + i));
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const float4 pv = *reinterpret_cast<const float4*>(&pt[r][i]);
                        const float a = pv.x - kv.x, b = pv.y - kv.y, c = pv.z - kv.z, e = pv.w - kv.w;
                        sq[r] = fmaf(a, a, sq[r]), sq[r] = fmaf(b, b, sq[r]), sq[r] = fmaf(c, c, sq[r]), sq[r] = fmaf(e, e, sq[r]);
                    }
                }
            } else {
                for (int i = 0; i < dk; ++i) {
                    const float kv = __ldg(krow + i);
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const float a = pt[r][i] - kv;
                        sq[r] = fmaf(a, a, sq[r]);
                    }
                }
            }
            const float inv_k = __fdividef(1.0f, 1.0f - __ldg(p.norm_sq + s));
#pragma unroll
            for (int r = 0; r < R; ++r) {
                d[r][u] = fast_poincare_distance(sq[r] * (row_inv[r] * inv_k));
                mn[r] = fminf(mn[r], d[r][u]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        mn[r] = warp_min(mn[r]);
        if (lane == 0) red[warp][r] = mn[r];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) {
        float m = red[0][r];
#pragma unroll
        for (int w = 1; w < 8; ++w) m = fminf(m, red[w][r]);
        mn[r] = m;
    }
    __syncthreads();
    if (p.min_dist && tid < R && q0 + tid < p.rows) p.min_dist[q0 + tid] = mn[tid];
    const float inv_tau = 1.0f / p.tau;
    const bool lite = inv_tau < CUDART_INF_F;  // a temperature too small for a finite reciprocal keeps the exact form
    const float scale2 = inv_tau * 1.4426950408889634f;
    float sum[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        sum[r] = 0.0f;
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            d[r][u] = lite ? exp2f_approx((mn[r] - d[r][u]) * scale2) : weight_of<false>(mn[r], d[r][u], p.tau);
            sum[r] += d[r][u];
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], m);
        if (lane == 0) red[warp][r] = sum[r];
    }
    __syncthreads();
    const bool second = p.value_terms != 1;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const size_t q = q0 + r;
        if (q >= p.rows) break;
        const float total = ((red[0][r] + red[1][r]) + (red[2][r] + red[3][r])) + ((red[4][r] + red[5][r]) + (red[6][r] + red[7][r]));
        const float inv_sum = __fdiv_rn(1.0f, total);
        __nv_bfloat16* ws = reinterpret_cast<__nv_bfloat16*>(p.w_split) + q * 3 * (size_t)cap;
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            const int s = tid + u * 256;
            if (s < cap) {
                const float wn = d[r][u] * inv_sum;
                if (!p.skip_weights && p.weights) p.weights[q * cap + s] = wn;
                const __nv_bfloat16 pa = __float2bfloat16_rn(wn);
                ws[s] = pa;
                if (second) ws[cap + s] = __float2bfloat16_rn(wn - __bfloat162float(pa));
            }
        }
    }
}

// One warp per query. Distances are read from `weights` and replaced by the weights.
template <bool EXACT>
__global__ void __launch_bounds__(256) softmax_topk_kernel(RetrieveParams p) {
    pdl_trigger();  // the next kernel in the stream may start its prologue now ...
    pdl_wait();     // ... and this one, if launched as a dependent, waits here for its own predecessor
    extern __shared__ float sm[];  // [8 warps][cap] distances / weights
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t q = (size_t)blockIdx.x * 8 + warp;
    if (q >= p.rows) return;
    const int cap = p.cap, count = p.count, dv = p.dv;
    float* row = p.weights + q * cap;
    float* w = sm + (size_t)warp * cap;
    if (count == 0) {  // memory.rs:363-367
        for (int i = lane; i < cap; i += 32) row[i] = 0.0f;
        for (int j = lane; j < dv; j += 32) {
            if (p.m_val) p.m_val[q * dv + j] = 0.0f;
            if (p.m_bf16) reinterpret_cast<__nv_bfloat16*>(p.m_bf16)[q * dv + j] = __float2bfloat16_rn(0.0f);
        }
        if (p.min_dist) p.min_dist[q] = 0.0f;
        return;
    }
    const float tau = p.tau;
    const int k = p.top_k;
    float mn = FLT_MAX;
    for (int i = lane; i < count; i += 32) {
        float d = row[i];
        w[i] = d;
        mn = fminf(mn, d);
    }
    mn = warp_min(mn);
    if (p.min_dist && lane == 0) p.min_dist[q] = mn;
    __syncwarp();
    if (k != 0 && k < count && k <= 32 && count <= 32 * kTopkRegs && cap >= 64) {
        // Register path of the selection below (same results): each lane keeps its count/32 distances in registers, a
        // round is a local minimum plus one warp-wide minimum of (distance bits, slot); the k winners are then ranked by
        // slot so that the sum, the weights and the value read walk them in ascending slot order (memory.rs:380-408)
        // without touching the other count - k slots.
        unsigned bits[kTopkRegs];
#pragma unroll
        for (int j = 0; j < kTopkRegs; ++j) {
            const int i = lane + 32 * j;
            bits[j] = i < count ? __float_as_uint(w[i]) : 0xffffffffu;  // distances are >= +0: their bits order them
        }
        unsigned my_slot = 0xffffffffu;  // lane r holds the r-th nearest slot
        float my_dist = 0.0f;
        for (int r = 0; r < k; ++r) {
            unsigned best = 0xffffffffu;
            int best_j = 0;
#pragma unroll
            for (int j = 0; j < kTopkRegs; ++j)
                if (bits[j] < best) best = bits[j], best_j = j;  // strict: ties keep the lower slot of this lane
            unsigned long long key = ((unsigned long long)best << 32) | (unsigned)(lane + 32 * best_j);
            key = warp_min_u64(key);
            const unsigned slot = (unsigned)(key & 0xffffffffu);
            if ((int)(slot & 31) == lane) {
#pragma unroll
                for (int j = 0; j < kTopkRegs; ++j)
                    if (j == (int)(slot >> 5)) bits[j] = 0xffffffffu;  // taken
            }
            if (lane == r) my_slot = slot, my_dist = __uint_as_float((unsigned)(key >> 32));
        }
        // rank of this lane's slot among the selected ones = its position in ascending slot order
        int rank = 0;
        for (int j = 0; j < k; ++j) rank += __shfl_sync(0xffffffffu, my_slot, j) < my_slot ? 1 : 0;
        const float my_w = lane < k ? weight_of<EXACT>(mn, my_dist, tau) : 0.0f;
        __syncwarp();  // every lane has read its distances out of w: the row is reused for the compacted list
        unsigned* sel_slot = reinterpret_cast<unsigned*>(w);
        float* sel_w = w + 32;
        if (lane < k) sel_slot[rank] = my_slot, sel_w[rank] = my_w;
        __syncwarp();
        float sum = 0.0f;
        for (int j = 0; j < k; ++j) sum = __fadd_rn(sum, sel_w[j]);  // ascending slot order, like the reference's sum
        for (int i = lane; i < cap; i += 32) row[i] = 0.0f;          // out_weights.fill(0.0)
        __syncwarp();
        if (lane < k) {
            const float wn = __fdiv_rn(my_w, sum);
            row[my_slot] = wn;
            sel_w[rank] = wn;
        }
        __syncwarp();
        for (int j0 = lane; j0 < dv; j0 += 32 * 4) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (int j = 0; j < k; ++j) {
                const float wi = sel_w[j];
                const float* v = p.values + (size_t)sel_slot[j] * dv;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int c = j0 + e * 32;
                    if (c < dv) acc[e] = __fadd_rn(acc[e], __fmul_rn(wi, __ldg(v + c)));
                }
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int c = j0 + e * 32;
                if (c < dv) {
                    if (p.m_val) p.m_val[q * dv + c] = acc[e];
                    if (p.m_bf16) reinterpret_cast<__nv_bfloat16*>(p.m_bf16)[q * dv + c] = __float2bfloat16_rn(acc[e]);
                }
            }
        }
        return;
    }
    if (k != 0 && k < count) {
        // memory.rs:380-408: keep the k smallest (distance bits, slot); weights over those only, slot order
        // selected slots are marked by setting the sign bit of their distance in shared memory
        for (int r = 0; r < k; ++r) {
            unsigned long long local = ~0ull;
            for (int i = lane; i < count; i += 32) {
                unsigned bits = __float_as_uint(w[i]);
                if (bits & 0x80000000u) continue;  // already selected (distances are >= +0)
                unsigned long long key = ((unsigned long long)bits << 32) | (unsigned)i;
                local = key < local ? key : local;
            }
            unsigned long long key = warp_min_u64(local);
            int idx = (int)(key & 0xffffffffu);
            if (lane == 0) w[idx] = __uint_as_float(__float_as_uint(w[idx]) | 0x80000000u);
            __syncwarp();
        }
        // sum in ascending slot order (selected.sort_unstable_by_key(idx); iter().sum()), memory.rs:391-398
        float sum = 0.0f;
        if (lane == 0) {
            for (int i = 0; i < count; ++i) {
                unsigned bits = __float_as_uint(w[i]);
                if (bits & 0x80000000u) sum = __fadd_rn(sum, weight_of<EXACT>(mn, __uint_as_float(bits & 0x7fffffffu), tau));
            }
        }
        sum = __shfl_sync(0xffffffffu, sum, 0);
        // weights: zero everywhere except the selected slots (out_weights.fill(0.0))
        for (int i = lane; i < cap; i += 32) {
            float out = 0.0f;
            if (i < count) {
                unsigned bits = __float_as_uint(w[i]);
                if (bits & 0x80000000u)
                    out = __fdiv_rn(weight_of<EXACT>(mn, __uint_as_float(bits & 0x7fffffffu), tau), sum);
                w[i] = (bits & 0x80000000u) ? out : -1.0f;  // -1 marks "not selected" for the read below
            }
            row[i] = out;
        }
        __syncwarp();
        // fused value read: each lane owns columns j = lane, lane+32, ...; slots in ascending order
        for (int j0 = lane; j0 < dv; j0 += 32 * 4) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (int i = 0; i < count; ++i) {
                float wi = w[i];
                if (wi < 0.0f) continue;
                const float* v = p.values + (size_t)i * dv;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    int j = j0 + e * 32;
                    if (j < dv) acc[e] = __fadd_rn(acc[e], __fmul_rn(wi, __ldg(v + j)));
                }
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int j = j0 + e * 32;
                if (j < dv) {
                    if (p.m_val) p.m_val[q * dv + j] = acc[e];
                    if (p.m_bf16) reinterpret_cast<__nv_bfloat16*>(p.m_bf16)[q * dv + j] = __float2bfloat16_rn(acc[e]);
                }
            }
        }
        return;
    }
    // all-slots read: w = exp((min - d)/tau); sum in slot order; w /= sum   (memory.rs:409-420)
    for (int i = lane; i < count; i += 32) w[i] = weight_of<EXACT>(mn, w[i], tau);
    __syncwarp();
    float sum = 0.0f;
    if (EXACT) {
        if (lane == 0)
            for (int i = 0; i < count; ++i) sum = __fadd_rn(sum, w[i]);
        sum = __shfl_sync(0xffffffffu, sum, 0);
    } else {
        for (int i = lane; i < count; i += 32) sum += w[i];
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
    }
    __nv_bfloat16* ws = p.w_split ? reinterpret_cast<__nv_bfloat16*>(p.w_split) + q * 3 * (size_t)cap : nullptr;
    for (int i = lane; i < cap; i += 32) {
        float wn = i < count ? __fdiv_rn(w[i], sum) : 0.0f;
        row[i] = wn;
        if (ws) {
            __nv_bfloat16 a, b, c;
            split3(wn, a, b, c);
            ws[i] = a, ws[cap + i] = b, ws[2 * cap + i] = c;
        }
    }
}

// ------------------------------------------------------------------ C: dense value read m = W x V
// 64 queries x 64 columns per CTA, 4x4 per thread, slots walked in ascending order.
template <bool EXACT>
__global__ void __launch_bounds__(256) value_mix_kernel(RetrieveParams p) {
    __shared__ __align__(16) float Ws[32][QT + 4];  // [slot][query]
    __shared__ __align__(16) float Vs[32][64 + 4];  // [slot][column]
    const int tid = threadIdx.x;
    const int tc = tid & 15, tq = tid >> 4;
    const size_t q0 = (size_t)blockIdx.x * QT;
    const int c0 = blockIdx.y * 64;
    const int cap = p.cap, count = p.count, dv = p.dv;
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0.0f;
    for (int s0 = 0; s0 < count; s0 += 32) {
        __syncthreads();
        for (int idx = tid; idx < 32 * QT; idx += 256) {
            int qq = idx / 32, sl = idx % 32;  // consecutive threads read consecutive slots of one query row
            size_t q = q0 + qq;
            int slot = s0 + sl;
            Ws[sl][qq] = (q < p.rows && slot < count) ? p.weights[q * cap + slot] : 0.0f;
        }
        for (int idx = tid; idx < 32 * 64; idx += 256) {
            int sl = idx / 64, cc = idx % 64;
            int slot = s0 + sl, col = c0 + cc;
            Vs[sl][cc] = (slot < count && col < dv) ? __ldg(p.values + (size_t)slot * dv + col) : 0.0f;
        }
        __syncthreads();
#pragma unroll 8
        for (int sl = 0; sl < 32; ++sl) {
            float4 wv = *reinterpret_cast<const float4*>(&Ws[sl][tq * 4]);
            float4 vv = *reinterpret_cast<const float4*>(&Vs[sl][tc * 4]);
            float wa[4] = {wv.x, wv.y, wv.z, wv.w};
            float va[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    if (EXACT)
                        acc[a][b] = __fadd_rn(acc[a][b], __fmul_rn(wa[a], va[b]));
                    else
                        acc[a][b] = fmaf(wa[a], va[b], acc[a][b]);
                }
        }
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        size_t q = q0 + tq * 4 + a;
        if (q >= p.rows) continue;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            int col = c0 + tc * 4 + b;
            if (col < dv) {
                if (p.m_val) p.m_val[q * dv + col] = acc[a][b];
                if (p.m_bf16) reinterpret_cast<__nv_bfloat16*>(p.m_bf16)[q * dv + col] = __float2bfloat16_rn(acc[a][b]);
            }
        }
    }
}

}  // namespace

int32_t launch_memory_read(pssa_b200_ctx* ctx, const RetrieveParams& p, bool exact) {
    const int kpad = (p.dk + 3) / 4 * 4;
    size_t smem_a = (size_t)kpad * QT * sizeof(double) + ((size_t)2 * STL * (kpad + 4) + QT) * sizeof(float);
    if (smem_a > 200 * 1024)
        return fail(ctx, PSSA_B200_ERR_UNSUPPORTED, "B200 memory read: key width %d needs %zu bytes of shared memory; refusing launch",
                    p.dk, smem_a);
    size_t smem_b = (size_t)8 * p.cap * sizeof(float);
    if (smem_b > 200 * 1024)
        return fail(ctx, PSSA_B200_ERR_UNSUPPORTED, "B200 memory read: capacity %d exceeds the %d slots one CTA can hold; refusing launch",
                    p.cap, 200 * 1024 / 32);
    size_t qblocks = (p.rows + QT - 1) / QT;
    if (qblocks > 0x7fffffffull) return fail(ctx, PSSA_B200_ERR_SHAPE, "B200 memory read grid exceeds grid limits; refusing launch");
    int32_t rc;
    // top-k reads whose shape fits take the one-kernel path (tensor-core pre-filter, exact f64 decision): same results
    // as the f64 distance kernel below, without the [rows, capacity] matrix in HBM
    if (!p.no_fused && retrieve_fused_eligible(p)) return launch_retrieve_fused(ctx, p);
    // all-slots reads of the bf16-grade consumers whose shape fits: projection, distances, softmax and the bf16 weight rows
    // in one kernel (the caller multiplies the rows by its own operand)
    if (retrieve_all_fused_runs(p, exact)) return launch_retrieve_all_fused(ctx, p);
    if (!p.weights) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 memory read: this shape needs the [rows, capacity] weight rows as scratch");
    // with an empty bank the launch still publishes the projection (gpu_batch.rs:682-698 projects first)
    static PerDeviceOnce attr_a;
    if (smem_a > 48 * 1024 && attr_a.need(ctx->device)) {
        PSSA_CUDA(ctx, cudaFuncSetAttribute(poincare_distance_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_a.done(ctx->device);
    }
    const int kpad4 = (p.dk + 3) / 4 * 4;
    const size_t smem_f = (size_t)(kpad4 / 2) * QT * sizeof(float2) + ((size_t)2 * STL * (kpad4 + 4) + QT + 2 * STL) * sizeof(float);
    const bool tc_dist = !exact && p.q_split && p.k_split && p.q_stat && p.k_stat && p.dk % 64 == 0 && p.dk <= 256 &&
                         (!p.q_pnc || (reinterpret_cast<uintptr_t>(p.q_pnc) & 7) == 0);
    const bool small_rows = !exact && !(p.top_k != 0 && p.top_k < p.count) && p.single_token && p.count > 0 && p.w_split &&
                            (p.value_terms == 1 || p.value_terms == 3) && p.dk <= 256 && p.cap <= 1024 && (p.skip_weights || p.weights) &&
                            (p.f32_distance || tc_dist);
    if (small_rows) {
        // a decode step: projection, distances, softmax and weight pieces in one launch (see the kernel)
        PSSA_CUDA(ctx, launch_dependent(retrieve_small_rows_kernel, dim3((unsigned)((p.rows + kSmallRows - 1) / kSmallRows)), dim3(256), 0, ctx->stream, p));
        if ((rc = after_launch(ctx, "retrieve_small_rows_kernel")) != PSSA_B200_OK) return rc;
    } else if (tc_dist) {
        // distances from the inner product on the tensor cores: projection + three-way split of the queries, then one
        // product against the split keys whose epilogue turns p.k into d(p, k)
        const size_t smem_p = (size_t)QT * (p.dk + 1) * sizeof(float);
        static PerDeviceOnce attr_p;
        if (smem_p > 48 * 1024 && attr_p.need(ctx->device)) {
            PSSA_CUDA(ctx, cudaFuncSetAttribute(project_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            attr_p.done(ctx->device);
        }
        PSSA_CUDA(ctx, launch_dependent(project_split_kernel, dim3((unsigned)qblocks), dim3(256), smem_p, ctx->stream, p));
        if ((rc = after_launch(ctx, "project_split_kernel")) != PSSA_B200_OK) return rc;
        if (p.count > 0 && (rc = launch_gemm_bf16_poincare(ctx, p.q_split, p.k_split, p.q_stat, p.k_stat, p.weights, p.rows,
                                                           (size_t)p.count, (size_t)p.dk, (size_t)p.cap)))
            return rc;
    } else if (p.f32_distance && !exact && smem_f <= 112 * 1024) {  // keys wider than 128 keep the f64 kernel
        static PerDeviceOnce attr_f;
        if (smem_f > 48 * 1024 && attr_f.need(ctx->device)) {
            PSSA_CUDA(ctx, cudaFuncSetAttribute(poincare_distance_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            attr_f.done(ctx->device);
        }
        // few query tiles (decode): spread the slot passes over up to 8 CTAs per tile
        unsigned ysplit = 1;
        const unsigned npass = (unsigned)((p.count + STL - 1) / STL);
        while (qblocks * ysplit < 148 && ysplit < 8 && ysplit * 2 <= (npass ? npass : 1)) ysplit *= 2;
        PSSA_CUDA(ctx, launch_dependent(poincare_distance_f32_kernel, dim3((unsigned)qblocks, ysplit), dim3(256), smem_f, ctx->stream, p));
        if ((rc = after_launch(ctx, "poincare_distance_f32_kernel")) != PSSA_B200_OK) return rc;
    } else {
        unsigned ysplit = 1;  // few query tiles (decode): spread the slot passes over up to 8 CTAs per tile
        const unsigned npass = (unsigned)((p.count + STL - 1) / STL);
        while (qblocks * ysplit < 148 && ysplit < 8 && ysplit * 2 <= (npass ? npass : 1)) ysplit *= 2;
        poincare_distance_kernel<<<dim3((unsigned)qblocks, ysplit), 256, smem_a, ctx->stream>>>(p);
        if ((rc = after_launch(ctx, "poincare_distance_kernel")) != PSSA_B200_OK) return rc;
    }
    size_t wblocks = (p.rows + 7) / 8;
    static PerDeviceOnce attr_b[2];
    if (smem_b > 48 * 1024 && attr_b[exact].need(ctx->device)) {
        if (exact)
            PSSA_CUDA(ctx, cudaFuncSetAttribute(softmax_topk_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        else
            PSSA_CUDA(ctx, cudaFuncSetAttribute(softmax_topk_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_b[exact].done(ctx->device);
    }
    const bool all_regs = !exact && !(p.top_k != 0 && p.top_k < p.count) && p.count > 0 && p.cap % 128 == 0 && p.cap <= 1024 &&
                          (reinterpret_cast<uintptr_t>(p.weights) & 15) == 0;
    if (small_rows) {
        // the weights and their pieces are already formed
    } else if (all_regs) {
        // a few rows per warp, so that a row's loads overlap the arithmetic of the one before
        const size_t want = (p.rows + 31) / 32, full = (size_t)ctx->sm_count * 8;
        const unsigned grid = (unsigned)std::min(wblocks, std::max(want, std::min(wblocks, full)));
        if (p.cap <= 512)
            PSSA_CUDA(ctx, launch_dependent(softmax_all_slots_kernel<4>, dim3(grid), dim3(256), 0, ctx->stream, p));
        else
            PSSA_CUDA(ctx, launch_dependent(softmax_all_slots_kernel<8>, dim3(grid), dim3(256), 0, ctx->stream, p));
        if ((rc = after_launch(ctx, "softmax_all_slots_kernel")) != PSSA_B200_OK) return rc;
    } else {
        if (exact)
            PSSA_CUDA(ctx, launch_dependent(softmax_topk_kernel<true>, dim3((unsigned)wblocks), dim3(256), smem_b, ctx->stream, p));
        else
            PSSA_CUDA(ctx, launch_dependent(softmax_topk_kernel<false>, dim3((unsigned)wblocks), dim3(256), smem_b, ctx->stream, p));
        if ((rc = after_launch(ctx, "softmax_topk_kernel")) != PSSA_B200_OK) return rc;
    }
    bool topk = p.top_k != 0 && p.top_k < p.count;
    if (p.count > 0 && !topk && p.w_split && p.v_split && !exact) {
        // all-slots value read on the tensor cores: m = W x V as six bf16 partial products (fp32-accurate), or the
        // leading three (error near 2^-16 of the row scale) when the caller only keeps a bf16 result
        // (skip_value_read: the caller multiplies the weight pieces by its own operand, e.g. values already carried
        // through the memory projection)
        if (!p.skip_value_read &&
            (rc = launch_gemm_bf16_split3(ctx, p.w_split, p.v_split, p.m_val, p.m_bf16, p.rows, p.dv, p.cap, p.dv,
                                          p.value_terms == 3 ? 3 : p.value_terms == 1 ? 1 : 6)))
            return rc;
    } else if (p.count > 0 && !topk) {
        dim3 grid((unsigned)qblocks, (unsigned)((p.dv + 63) / 64));
        if (exact)
            value_mix_kernel<true><<<grid, 256, 0, ctx->stream>>>(p);
        else
            value_mix_kernel<false><<<grid, 256, 0, ctx->stream>>>(p);
        if ((rc = after_launch(ctx, "value_mix_kernel")) != PSSA_B200_OK) return rc;
    }
    return PSSA_B200_OK;
}

// (PSSA_B200_NO_ALL_SLOTS_FUSED keeps the separate kernels: read at every call, a test compares the two)
bool retrieve_all_fused_runs(const RetrieveParams& p, bool exact) {
    const char* keep_separate = getenv("PSSA_B200_NO_ALL_SLOTS_FUSED");
    return !p.no_fused && !exact && !(keep_separate && *keep_separate && *keep_separate != '0') && retrieve_all_fused_eligible(p);
}

int32_t launch_split_keys(pssa_b200_ctx* ctx, const float* keys, const float* norm_sq, void* k_split, float2* k_stat, int cap, int dk) {
    size_t n = (size_t)cap * dk;
    split_keys_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(keys, norm_sq, (__nv_bfloat16*)k_split, k_stat, cap, dk);
    return after_launch(ctx, "split_keys_kernel");
}

int32_t launch_split_values(pssa_b200_ctx* ctx, const float* values, void* v_split, int cap, int dv) {
    size_t n = (size_t)cap * dv;
    split_values_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(values, (__nv_bfloat16*)v_split, cap, dv);
    return after_launch(ctx, "split_values_kernel");
}

}  // namespace pssa
