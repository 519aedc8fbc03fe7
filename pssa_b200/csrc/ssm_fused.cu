// Fused selective-SSM stage: discretise, scan and read out in one pass, state in registers.
//
//   a = exp(delta_i * A_ij);  b = delta_i * B_j;  h_ij <- a*h_ij + b*x_i;  y_i = sum_j h_ij * C_j
//
// Replaces the reference's three kernels ssm_prepare / affine_scan / ssm_materialize
// (src/cuda/stages.ptx:8-65, launched from src/cuda/stages.rs:260-356), which write three
// [T, d*s] arrays to HBM and read them back twice, and the CPU stage src/gpu_batch.rs:543-680.
// Here the only HBM traffic is the inputs (delta, x, B, C: (2d + 2s) floats per token), y, and the
// carry once per lane; the per-token maps never leave registers. The kernel is therefore bound by
// the exp throughput (d*s per token), not by HBM.
//
// Work split: one CTA = one lane (independent sequence) x CH consecutive channels i; a channel's
// s states are spread over G threads of one warp holding ST states each (G*ST >= s). Inside a warp
// the 32/G threads that own the same state group sit in adjacent lanes, so the B_j / C_j vectors a
// thread needs are one shared-memory address per quarter warp (a broadcast, no bank conflicts; the
// groups are padded apart by 4 floats), and y is completed by a shuffle tree over the G groups.
// Time is walked serially by every thread; token tiles (delta, x, B, C rows) are staged through a
// cp.async ring in shared memory so the global-load latency is hidden behind the previous tile's exps.
//
// Two arithmetic modes:
//   FAST  ex2.approx on delta*(A*log2 e) (the reference's own GPU recipe, stages.ptx:21-22),
//         FMA contraction, y summed per thread then by a shuffle tree over the G threads.
//   EXACT expf, separately rounded multiply/add in the reference's order (src/pssa.rs:1131-1144);
//         with G == 1 the sum over j is the reference's sequential sum.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "bounds.hpp"
#include "context.hpp"
#include "kernels.hpp"

namespace pssa {
namespace {

constexpr int kThreads = 256;  // default CTA size; the 16-state fast configuration also comes with 352 (see launch_ssm_fused)
// tokens per staged tile; the widest state split keeps 8 so its stages stay inside the shared memory of one SM. The
// 64-state configuration (four lanes per channel) takes 32 tokens in two stages: the same shared memory as 16 tokens in
// three, half as many CTA-wide barriers (12.07 against 12.19 ms per step for the twelve launches of the benchmark)
template <int G>
constexpr int kTileTokensFor = G >= 32 ? 8 : (G == 4 ? 32 : 16);
// The 16-state fast configuration is capped at 64 registers so four CTAs (32 warps) share an SM: the kernel is bound by
// dependent-issue latency, not by a pipe, and the extra warps are worth more than the 16 bytes of spill they cost.
constexpr int kMinCtasFast = 4;
constexpr int kStages = 2;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Packed fp32 pairs (one instruction, two IEEE-rounded results): the kernel is bound by instruction issue, and the
// per-state multiply / fma work is half the instruction stream.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

template <int ST, int G, bool EXACT, bool TAPE, int THR = kThreads, int CPT = 1>
__global__ void __launch_bounds__(THR, (ST <= 16 && !TAPE && !EXACT) ? ((THR > 256 || CPT > 1) ? 2 : kMinCtasFast) : 1) ssm_fused_kernel(SsmParams p) {
    // CPT channels per thread (fast mode without tape only): a token's B and C rows are loaded once for both channels and
    // the two recurrences are independent instruction streams, so a warp-token of twice the work takes fewer than twice
    // the instructions.
    static_assert(CPT == 1 || (CPT == 2 && !EXACT && !TAPE), "two channels per thread exist for the fast mode only");
    pdl_trigger();  // the next kernel in the stream may start its prologue now ...
    pdl_wait();     // ... and this one, if launched as a dependent, waits here for its own predecessor
    constexpr int kThreads = THR;     // shadows the default: every stride below follows this instantiation's CTA size
    constexpr int CH = kThreads / G * CPT;  // channels per CTA
    constexpr int kTileTokens = kTileTokensFor<G>;
    constexpr int LPG = 32 / G;       // lanes of a warp that share one state group
    constexpr int SG = ST + 4;        // shared-memory pitch of a state group (bank spreading)
    constexpr int SP = SG * G;        // floats per token row of B / C in shared memory
    extern __shared__ __align__(16) float smem[];
    float* sm_delta = smem;                                   // [kStages][kTileTokens][CH]
    float* sm_x = sm_delta + kStages * kTileTokens * CH;      // [kStages][kTileTokens][CH]
    float* sm_b = sm_x + kStages * kTileTokens * CH;          // [kStages][kTileTokens][SP]
    float* sm_c = sm_b + kStages * kTileTokens * SP;          // [kStages][kTileTokens][SP]

    const int tid = threadIdx.x;
    const int lane_id = tid & 31;
    const int g = lane_id / LPG;
    const int c = (tid >> 5) * LPG + lane_id % LPG;
    const int ncb = (p.d + CH - 1) / CH;
    const int lane = blockIdx.x / ncb;
    const int i0 = (blockIdx.x % ncb) * CH;
    const int i = i0 + CPT * c;  // a two-channel thread owns the adjacent channels CPT * c and CPT * c + 1
    const bool valid = i < p.d;
    const size_t row0 = p.offsets ? p.offsets[lane] : 0;
    const int len = p.lengths ? (int)p.lengths[lane] : (int)p.rows;
    const int d = p.d, s = p.s;
    const size_t ds = (size_t)d * s;
    const int j0 = g * ST;
    const size_t ldd = p.ld_delta ? p.ld_delta : (size_t)d;
    const size_t ldbc = p.ld_bc ? p.ld_bc : (size_t)s;
    float* carry = p.carry ? p.carry + (size_t)(p.lane_slots ? p.lane_slots[lane] : lane) * (p.carry_stride ? p.carry_stride : ds)
                           : nullptr;

    float A[ST], h[ST];
    float A1[CPT > 1 ? ST : 1], h1[CPT > 1 ? ST : 1];  // the second channel of a two-channel thread
    const int i1 = i + 1;
    const bool valid1 = CPT > 1 && i1 < p.d;
    // a thread's states are contiguous in `rates` and in the carry: 16-byte accesses when the layout allows (decode
    // steps are one token long, so this load and the store at the end are most of their traffic)
    const bool vec_state = p.aligned && (s & 3) == 0 && (reinterpret_cast<uintptr_t>(p.rates) & 15) == 0 &&
                           (reinterpret_cast<uintptr_t>(carry) & 15) == 0;
    auto load_state = [&](float* Av, float* hv, int ch, bool ok_ch) {
        if (vec_state) {
#pragma unroll
            for (int q = 0; q < ST / 4; ++q) {
                const bool ok = ok_ch && (j0 + q * 4) < s;
                const float4 r4 = ok ? __ldg(reinterpret_cast<const float4*>(p.rates + (size_t)ch * s + j0) + q) : make_float4(0.f, 0.f, 0.f, 0.f);
                const float4 h4 = (ok && carry) ? *(reinterpret_cast<const float4*>(carry + (size_t)ch * s + j0) + q) : make_float4(0.f, 0.f, 0.f, 0.f);
                Av[q * 4] = r4.x, Av[q * 4 + 1] = r4.y, Av[q * 4 + 2] = r4.z, Av[q * 4 + 3] = r4.w;
                hv[q * 4] = h4.x, hv[q * 4 + 1] = h4.y, hv[q * 4 + 2] = h4.z, hv[q * 4 + 3] = h4.w;
            }
            if (!EXACT) {
#pragma unroll
                for (int jj = 0; jj < ST; ++jj) Av[jj] *= 1.4426950408889634f;
            }
        } else {
#pragma unroll
            for (int jj = 0; jj < ST; ++jj) {
                bool ok = ok_ch && (j0 + jj) < s;
                float rate = ok ? __ldg(p.rates + (size_t)ch * s + j0 + jj) : 0.0f;
                Av[jj] = EXACT ? rate : rate * 1.4426950408889634f;
                hv[jj] = (ok && carry) ? carry[(size_t)ch * s + j0 + jj] : 0.0f;
            }
        }
    };
    load_state(A, h, i, valid);
    if constexpr (CPT > 1) load_state(A1, h1, i1, valid1);

    const int ntiles = (len + kTileTokens - 1) / kTileTokens;

    auto load_tile = [&](int k) {
        if (k < ntiles) {
            const int st = k % kStages;
            const int t0 = k * kTileTokens;
            const int nt = min(kTileTokens, len - t0);
            float* dd = sm_delta + st * kTileTokens * CH;
            float* dx = sm_x + st * kTileTokens * CH;
            float* db = sm_b + st * kTileTokens * SP;
            float* dc = sm_c + st * kTileTokens * SP;
            if (p.aligned) {
                constexpr int CQ = CH / 4 > 0 ? CH / 4 : 1;
                for (int idx = tid; idx < nt * CQ; idx += kThreads) {
                    int tt = idx / CQ, q = idx % CQ;
                    int col = i0 + q * 4;
                    size_t gro = (row0 + t0 + tt) * (size_t)d + col;
                    if (CH >= 4 && col < d) {
                        cp_async16(dd + tt * CH + q * 4, p.delta + (row0 + t0 + tt) * ldd + col);
                        cp_async16(dx + tt * CH + q * 4, p.x_norm + gro);
                    } else if (CH >= 4) {
                        *reinterpret_cast<float4*>(dd + tt * CH + q * 4) = make_float4(0, 0, 0, 0);
                        *reinterpret_cast<float4*>(dx + tt * CH + q * 4) = make_float4(0, 0, 0, 0);
                    }
                }
                constexpr int SQ = ST * G / 4;
                for (int idx = tid; idx < nt * SQ; idx += kThreads) {
                    int tt = idx / SQ, q = idx % SQ;
                    int j = q * 4;
                    int dst = tt * SP + (j / ST) * SG + j % ST;
                    size_t gro = (row0 + t0 + tt) * ldbc + j;
                    if (j < s) {
                        cp_async16(db + dst, p.b_proj + gro);
                        cp_async16(dc + dst, p.c_proj + gro);
                    } else {
                        *reinterpret_cast<float4*>(db + dst) = make_float4(0, 0, 0, 0);
                        *reinterpret_cast<float4*>(dc + dst) = make_float4(0, 0, 0, 0);
                    }
                }
            } else {
                for (int idx = tid; idx < nt * CH; idx += kThreads) {
                    int tt = idx / CH, q = idx % CH;
                    int col = i0 + q;
                    size_t gro = (row0 + t0 + tt) * (size_t)d + col;
                    dd[tt * CH + q] = col < d ? __ldg(p.delta + (row0 + t0 + tt) * ldd + col) : 0.0f;
                    dx[tt * CH + q] = col < d ? __ldg(p.x_norm + gro) : 0.0f;
                }
                for (int idx = tid; idx < nt * ST * G; idx += kThreads) {
                    int tt = idx / (ST * G), j = idx % (ST * G);
                    int dst = tt * SP + (j / ST) * SG + j % ST;
                    size_t gro = (row0 + t0 + tt) * ldbc + j;
                    db[dst] = j < s ? __ldg(p.b_proj + gro) : 0.0f;
                    dc[dst] = j < s ? __ldg(p.c_proj + gro) : 0.0f;
                }
            }
        }
        cp_async_commit();
    };

#pragma unroll
    for (int k = 0; k < kStages - 1; ++k) load_tile(k);

    for (int k = 0; k < ntiles; ++k) {
        // tile k has landed once at most kStages-2 newer groups are in flight; the barrier also means every thread is
        // done with tile k-1 (its stage is the one the prefetch below overwrites)
        cp_async_wait<kStages - 2>();
        __syncthreads();
        load_tile(k + kStages - 1);
        const int st = k % kStages;
        const int t0 = k * kTileTokens;
        const int nt = min(kTileTokens, len - t0);
        float* dd = sm_delta + st * kTileTokens * CH;
        const float* dx = sm_x + st * kTileTokens * CH;
        const float* db = sm_b + st * kTileTokens * SP + g * SG;
        const float* dc = sm_c + st * kTileTokens * SP + g * SG;
        auto token = [&](int tt) {
            float dl, xv, dlb = 0.0f, xvb = 0.0f;
            if constexpr (CPT > 1) {  // both channels' values with one 8-byte load each
                const float2 d2 = *reinterpret_cast<const float2*>(dd + tt * CH + 2 * c);
                const float2 x2 = *reinterpret_cast<const float2*>(dx + tt * CH + 2 * c);
                dl = d2.x, dlb = d2.y, xv = x2.x, xvb = x2.y;
            } else {
                dl = dd[tt * CH + c], xv = dx[tt * CH + c];
            }
            const size_t row = row0 + t0 + tt;
            static_assert(ST % 4 == 0, "states per thread are loaded as float4");
            float bj[ST], cj[ST];
#pragma unroll
            for (int q = 0; q < ST / 4; ++q) {
                float4 vb = *reinterpret_cast<const float4*>(db + tt * SP + q * 4);
                float4 vc = *reinterpret_cast<const float4*>(dc + tt * SP + q * 4);
                bj[q * 4] = vb.x, bj[q * 4 + 1] = vb.y, bj[q * 4 + 2] = vb.z, bj[q * 4 + 3] = vb.w;
                cj[q * 4] = vc.x, cj[q * 4 + 1] = vc.y, cj[q * 4 + 2] = vc.z, cj[q * 4 + 3] = vc.w;
            }
            float yp = 0.0f, ypb = 0.0f;
            float av[TAPE ? ST : 1], bv[TAPE ? ST : 1];
            if (EXACT) {
#pragma unroll
                for (int jj = 0; jj < ST; ++jj) {
                    float a = expf(__fmul_rn(dl, A[jj]));
                    float bb = __fmul_rn(dl, bj[jj]);
                    h[jj] = __fadd_rn(__fmul_rn(a, h[jj]), __fmul_rn(bb, xv));
                    yp = __fadd_rn(yp, __fmul_rn(h[jj], cj[jj]));
                    if (TAPE) av[jj] = a, bv[jj] = bb;
                }
            } else {
                const float w = dl * xv;
                const f32x2 dl2 = pack2(dl, dl), w2 = pack2(w, w);
                f32x2 y2 = pack2(0.0f, 0.0f);
                const float wb = dlb * xvb;
                const f32x2 dlb2 = pack2(dlb, dlb), wb2 = pack2(wb, wb);
                f32x2 yb2 = pack2(0.0f, 0.0f);
#pragma unroll
                for (int jj = 0; jj < ST; jj += 2) {
                    const f32x2 b2 = pack2(bj[jj], bj[jj + 1]), c2 = pack2(cj[jj], cj[jj + 1]);
                    float e0, e1;
                    unpack2(mul2(dl2, pack2(A[jj], A[jj + 1])), e0, e1);
                    const float a0 = ex2_approx(e0), a1 = ex2_approx(e1);
                    f32x2 h2 = fma2(pack2(a0, a1), pack2(h[jj], h[jj + 1]), mul2(w2, b2));
                    unpack2(h2, h[jj], h[jj + 1]);
                    y2 = fma2(h2, c2, y2);
                    if (TAPE) av[jj] = a0, av[jj + 1] = a1, bv[jj] = dl * bj[jj], bv[jj + 1] = dl * bj[jj + 1];
                    if constexpr (CPT > 1) {
                        float f0, f1;
                        unpack2(mul2(dlb2, pack2(A1[jj], A1[jj + 1])), f0, f1);
                        const float g0 = ex2_approx(f0), g1 = ex2_approx(f1);
                        f32x2 hb2 = fma2(pack2(g0, g1), pack2(h1[jj], h1[jj + 1]), mul2(wb2, b2));
                        unpack2(hb2, h1[jj], h1[jj + 1]);
                        yb2 = fma2(hb2, c2, yb2);
                    }
                }
                float y_lo, y_hi;
                unpack2(y2, y_lo, y_hi);
                yp = y_lo + y_hi;
                if constexpr (CPT > 1) {
                    unpack2(yb2, y_lo, y_hi);
                    ypb = y_lo + y_hi;
                }
            }
#pragma unroll
            for (int m = LPG; m < 32; m <<= 1) yp += __shfl_xor_sync(0xffffffffu, yp, m);
            if constexpr (CPT > 1) {
#pragma unroll
                for (int m = LPG; m < 32; m <<= 1) ypb += __shfl_xor_sync(0xffffffffu, ypb, m);
                if (g == 0) *reinterpret_cast<float2*>(dd + tt * CH + 2 * c) = make_float2(yp, ypb);
            } else {
                if (g == 0) dd[tt * CH + c] = yp;  // every reader of this delta slot sits in this warp and has read it
            }
            if (TAPE) {
#pragma unroll
                for (int jj = 0; jj < ST; ++jj) {
                    if (valid && j0 + jj < s) {
                        size_t o = row * ds + (size_t)i * s + j0 + jj;
                        if (p.states) p.states[o] = h[jj];
                        if (p.bar_a) p.bar_a[o] = av[jj];
                        if (p.bar_b) p.bar_b[o] = bv[jj];
                    }
                }
            }
        };
        if (nt == kTileTokens) {
#pragma unroll 4
            for (int tt = 0; tt < kTileTokens; ++tt) token(tt);
        } else {
            for (int tt = 0; tt < nt; ++tt) token(tt);
        }
        __syncthreads();
        // write the tile's y rows out together: 16-byte stores instead of one predicated scalar store per token
        if (p.aligned) {
            constexpr int CQ = CH / 4;
            for (int idx = tid; idx < nt * CQ; idx += kThreads) {
                const int tt = idx / CQ, q = idx % CQ;
                const int col = i0 + q * 4;
                if (col < d) {
                    const float4 v = *reinterpret_cast<const float4*>(dd + tt * CH + q * 4);
                    const size_t o = (row0 + t0 + tt) * (size_t)d + col;
                    *reinterpret_cast<float4*>(p.y + o) = v;
                    if (p.y_bf16) {
                        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
                        uint2 pk;
                        pk.x = *reinterpret_cast<unsigned*>(&lo);
                        pk.y = *reinterpret_cast<unsigned*>(&hi);
                        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.y_bf16) + o) = pk;
                    }
                }
            }
        } else {
            for (int idx = tid; idx < nt * CH; idx += kThreads) {
                const int tt = idx / CH, q = idx % CH;
                if (i0 + q < d) {
                    const size_t o = (row0 + t0 + tt) * (size_t)d + i0 + q;
                    p.y[o] = dd[tt * CH + q];
                    if (p.y_bf16) reinterpret_cast<__nv_bfloat16*>(p.y_bf16)[o] = __float2bfloat16_rn(dd[tt * CH + q]);
                }
            }
        }
    }
    cp_async_wait<0>();
    if (carry && len > 0) {
        auto store_state = [&](const float* hv, int ch, bool ok_ch) {
            if (vec_state) {
#pragma unroll
                for (int q = 0; q < ST / 4; ++q)
                    if (ok_ch && j0 + q * 4 < s)
                        *(reinterpret_cast<float4*>(carry + (size_t)ch * s + j0) + q) = make_float4(hv[q * 4], hv[q * 4 + 1], hv[q * 4 + 2], hv[q * 4 + 3]);
            } else {
#pragma unroll
                for (int jj = 0; jj < ST; ++jj)
                    if (ok_ch && j0 + jj < s) carry[(size_t)ch * s + j0 + jj] = hv[jj];
            }
        };
        store_state(h, i, valid);
        if constexpr (CPT > 1) store_state(h1, i1, valid1);
    }
}

// Decode step: every lane advances by one token, so the launch is one pass over the carries (2 * d * s * 4 bytes per
// lane in and out) and nothing else matters. A thread owns four consecutive states of one channel: rates, carry in and
// carry out are 16-byte accesses that a warp makes over a contiguous 512 bytes; y is finished by a shuffle tree over the
// TPC threads of the channel. Same arithmetic as the fast mode of the tiled kernel (ex2.approx, fused multiply-adds).
template <int TPC>
__global__ void __launch_bounds__(256) ssm_step_kernel(SsmParams p) {
    pdl_trigger();  // the next kernel in the stream may start its prologue now ...
    pdl_wait();     // ... and this one, if launched as a dependent, waits here for its own predecessor
    constexpr int CPB = 256 / TPC;  // channels per CTA
    const int tid = threadIdx.x;
    const int q = tid % TPC, c = tid / TPC;
    const int ncb = (p.d + CPB - 1) / CPB;
    const int lane = blockIdx.x / ncb;
    const int i = (blockIdx.x % ncb) * CPB + c;
    const int len = p.lengths ? (int)p.lengths[lane] : (int)p.rows;
    if (len <= 0) return;  // idle lane: carry and y untouched
    const size_t row = p.offsets ? p.offsets[lane] : 0;
    const int d = p.d, s = p.s;
    const size_t ds = (size_t)d * s;
    const size_t ldd = p.ld_delta ? p.ld_delta : (size_t)d;
    const size_t ldbc = p.ld_bc ? p.ld_bc : (size_t)s;
    float* carry = p.carry ? p.carry + (size_t)(p.lane_slots ? p.lane_slots[lane] : lane) * (p.carry_stride ? p.carry_stride : ds)
                           : nullptr;
    const bool live = i < d && q * 4 < s;
    float yp = 0.0f;
    if (live) {
        const size_t so = (size_t)i * s + q * 4;
        const float4 a4 = __ldg(reinterpret_cast<const float4*>(p.rates + so));
        const float4 h4 = carry ? *reinterpret_cast<const float4*>(carry + so) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 b4 = __ldg(reinterpret_cast<const float4*>(p.b_proj + row * ldbc + q * 4));
        const float4 c4 = __ldg(reinterpret_cast<const float4*>(p.c_proj + row * ldbc + q * 4));
        const float dl = __ldg(p.delta + row * ldd + i);
        const float w = dl * __ldg(p.x_norm + row * d + i);
        const float k = dl * 1.4426950408889634f;
        float4 h;
        h.x = fmaf(ex2_approx(k * a4.x), h4.x, w * b4.x);
        h.y = fmaf(ex2_approx(k * a4.y), h4.y, w * b4.y);
        h.z = fmaf(ex2_approx(k * a4.z), h4.z, w * b4.z);
        h.w = fmaf(ex2_approx(k * a4.w), h4.w, w * b4.w);
        yp = fmaf(h.x, c4.x, fmaf(h.y, c4.y, fmaf(h.z, c4.z, h.w * c4.w)));
        if (carry) *reinterpret_cast<float4*>(carry + so) = h;
    }
#pragma unroll
    for (int m = 1; m < TPC; m <<= 1) yp += __shfl_xor_sync(0xffffffffu, yp, m);
    if (q == 0 && i < d) {
        p.y[row * d + i] = yp;
        if (p.y_bf16) reinterpret_cast<__nv_bfloat16*>(p.y_bf16)[row * d + i] = __float2bfloat16_rn(yp);
    }
}

template <int TPC>
int32_t launch_step(pssa_b200_ctx* ctx, const SsmParams& p) {
    constexpr int CPB = 256 / TPC;
    size_t blocks = (size_t)((p.d + CPB - 1) / CPB) * p.lanes;
    if (blocks > 0x7fffffffull)
        return fail(ctx, PSSA_B200_ERR_SHAPE, "B200 SSM grid (%zu, 1) exceeds grid limits; refusing launch", blocks);
    PSSA_CUDA(ctx, launch_dependent(ssm_step_kernel<TPC>, dim3((unsigned)blocks), dim3(256), 0, ctx->stream, p));
    return after_launch(ctx, "ssm_step_kernel");
}

// Sum of delta over each lane's rows, per channel (the decay half of a time shard's affine map: the product of
// exp(delta_t * A) over the shard is exp(A * sum of delta)). One CTA = one lane x 32 channels; 8 row-strided partial sums
// per channel in f64, combined in a fixed order.
__global__ void __launch_bounds__(256) sum_delta_kernel(const float* __restrict__ delta, size_t ldd, const uint32_t* __restrict__ offsets,
                                                        const uint32_t* __restrict__ lengths, int d, float* __restrict__ out,
                                                        size_t out_stride) {
    __shared__ double part[8][32];
    const int lane = blockIdx.y;
    const int c = threadIdx.x & 31, tq = threadIdx.x >> 5;
    const int i = blockIdx.x * 32 + c;
    const size_t row0 = offsets[lane];
    const int len = (int)lengths[lane];
    double acc = 0.0;
    if (i < d)
        for (int t = tq; t < len; t += 8) acc += (double)__ldg(delta + (row0 + t) * ldd + i);
    part[tq][c] = acc;
    __syncthreads();
    if (tq == 0 && i < d) {
        double sum = 0.0;
#pragma unroll
        for (int k = 0; k < 8; ++k) sum += part[k][c];
        out[(size_t)lane * out_stride + i] = (float)sum;
    }
}

// One thread per (lane, channel, state): walks the shard maps of every rank and time chunk in time order.
__global__ void __launch_bounds__(256) seqpar_fold_kernel(const float* __restrict__ gathered, size_t rec, int world, int rank,
                                                          int chunks, size_t rank_stride, const float* __restrict__ rates,
                                                          float* __restrict__ state, size_t state_stride,
                                                          const uint32_t* __restrict__ lane_slots, float* __restrict__ carry_in,
                                                          int d, int s) {
    const size_t ds = (size_t)d * s;
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int lane = blockIdx.y;
    if (e >= ds) return;
    const int i = (int)(e / s);
    float* st = state + (size_t)(lane_slots ? lane_slots[lane] : lane) * state_stride;
    const float a = rates[e];
    float h = st[e];
    // the records are independent of h: four of them are requested (and their decay factors formed) before the
    // dependent multiply-adds, so the walk is not one memory round trip per record
    const int n = world * chunks;
    for (int j0 = 0; j0 < n; j0 += 4) {
        float pk[4], add[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = j0 + u;
            if (j < n) {
                const int k = j / chunks, c = j - k * chunks;
                const float* r = gathered + (size_t)k * rank_stride + ((size_t)lane * chunks + c) * rec;
                pk[u] = expf(__fmul_rn(a, __ldg(r + i)));
                add[u] = __ldg(r + d + e);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = j0 + u;
            if (j < n) {
                const int k = j / chunks, c = j - k * chunks;
                if (k == rank) carry_in[((size_t)lane * chunks + c) * ds + e] = h;
                h = __fadd_rn(__fmul_rn(pk[u], h), add[u]);
            }
        }
    }
    st[e] = h;
}

template <int ST, int G, bool EXACT, bool TAPE, int THR = kThreads, int CPT = 1>
int32_t launch_cfg(pssa_b200_ctx* ctx, const SsmParams& p) {
    constexpr int kThreads = THR;
    constexpr int CH = kThreads / G * CPT;
    constexpr int SP = (ST + 4) * G;
    constexpr int kTileTokens = kTileTokensFor<G>;
    size_t smem = (size_t)kStages * kTileTokens * (2 * CH + 2 * SP) * sizeof(float);
    auto kern = ssm_fused_kernel<ST, G, EXACT, TAPE, THR, CPT>;
    static PerDeviceOnce attr_set;  // per instantiation and per device
    if (smem > 48 * 1024 && attr_set.need(ctx->device)) {
        PSSA_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set.done(ctx->device);
    }
    int ncb = (p.d + CH - 1) / CH;
    size_t blocks = (size_t)ncb * p.lanes;
    if (blocks > 0x7fffffffull)
        return fail(ctx, PSSA_B200_ERR_SHAPE, "B200 SSM grid (%zu, 1) exceeds grid limits; refusing launch", blocks);
    PSSA_CUDA(ctx, launch_dependent(kern, dim3((unsigned)blocks), dim3(kThreads), smem, ctx->stream, p));
    return after_launch(ctx, "ssm_fused_kernel");
}

// The tape outputs (states, bar_a, bar_b: the reference's training tape) cost d*s floats per token
// each; inference never asks for them, so they live in a separate instantiation.
template <int ST, int G, bool EXACT>
int32_t launch_one(pssa_b200_ctx* ctx, const SsmParams& p) {
    if (p.states || p.bar_a || p.bar_b) return launch_cfg<ST, G, EXACT, true>(ctx, p);
    return launch_cfg<ST, G, EXACT, false>(ctx, p);
}

}  // namespace

int32_t launch_seqpar_fold(pssa_b200_ctx* ctx, const float* gathered, size_t rec, int world, int rank, int chunks, int lanes,
                           size_t rank_stride, const float* rates, float* state, size_t state_stride, const uint32_t* lane_slots,
                           float* carry_in, int d, int s) {
    const size_t ds = (size_t)d * s;
    dim3 grid((unsigned)((ds + 255) / 256), (unsigned)lanes);
    if (lanes < 1 || lanes > 65535) return fail(ctx, PSSA_B200_ERR_SHAPE, "chunk fold: %d lanes outside 1..65535", lanes);
    seqpar_fold_kernel<<<grid, 256, 0, ctx->stream>>>(gathered, rec, world, rank, chunks, rank_stride, rates, state, state_stride,
                                                     lane_slots, carry_in, d, s);
    return after_launch(ctx, "seqpar_fold_kernel");
}

int32_t launch_ssm_fused(pssa_b200_ctx* ctx, const SsmParams& p, bool exact) {
    const int s = p.s;
    if (p.sum_delta) {
        if (!p.offsets || !p.lengths) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "B200 SSM: sum_delta needs lane offsets and lengths");
        if (p.lanes > 65535) return fail(ctx, PSSA_B200_ERR_SHAPE, "B200 SSM: sum_delta supports at most 65535 lanes; refusing launch");
        dim3 grid((unsigned)((p.d + 31) / 32), (unsigned)p.lanes);
        sum_delta_kernel<<<grid, 256, 0, ctx->stream>>>(p.delta, p.ld_delta ? p.ld_delta : (size_t)p.d, p.offsets, p.lengths, p.d,
                                                       p.sum_delta, p.sum_delta_stride);
        int32_t rc = after_launch(ctx, "sum_delta_kernel");
        if (rc != PSSA_B200_OK) return rc;
    }
    const bool tape = p.states || p.bar_a || p.bar_b;
    if (p.single_token && !exact && !tape && p.aligned && s <= 128 && (reinterpret_cast<uintptr_t>(p.rates) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(p.carry) & 15) == 0 && ((p.carry_stride ? p.carry_stride : (size_t)p.d * s) & 3) == 0) {
        if (s <= 16) return launch_step<4>(ctx, p);
        if (s <= 32) return launch_step<8>(ctx, p);
        if (s <= 64) return launch_step<16>(ctx, p);
        return launch_step<32>(ctx, p);
    }
    if (exact) {
        if (s <= 4) return launch_one<4, 1, true>(ctx, p);
        if (s <= 16) return launch_one<16, 1, true>(ctx, p);
        if (s <= 64) return launch_one<64, 1, true>(ctx, p);
        if (s <= 128) return launch_one<16, 8, true>(ctx, p);
        if (s <= 512) return launch_one<16, 32, true>(ctx, p);
    } else {
        if (s <= 4) return launch_one<4, 1, false>(ctx, p);
        if (s <= 8) return launch_one<4, 2, false>(ctx, p);
        if (s <= 16) return launch_one<4, 4, false>(ctx, p);
        if (s <= 32) return launch_one<16, 2, false>(ctx, p);
        if (s <= 64) {
            // CTA shape by wave balance. Every CTA of a launch is resident at once and a warp's time per token is fixed by
            // its exponentials (16 per lane and channel, 8 cycles each on its scheduler's XU pipe), so the launch lasts as
            // long as the busiest scheduler: count, per shape, the channel-warps the fullest SM puts on one scheduler.
            // 256 threads = 64 channels per CTA (4 CTAs per SM), 352 threads = 88 channels (2 per SM), 128 threads with two
            // channels per thread = 64 channels (3 per SM). With d = 768 and 32 lanes: 384 CTAs put 3 x 8 warps on most SMs
            // (6 per scheduler), 288 of 352 threads put 2 x 11 (6 on two schedulers, 5 on the others), 384 two-channel CTAs
            // put 3 x 4 double warps (6). On a tie the two-channel shape wins: a token's B and C rows are loaded once
            // for both channels (11.93 -> 11.67 ms for the 12 launches of the benchmark step).
            if (!tape) {
                auto busiest = [&](int threads, int cpt, int cap) -> long long {
                    const int ch = threads / 4 * cpt;
                    const long long blocks = (long long)((p.d + ch - 1) / ch) * p.lanes;
                    const long long per_sm = (blocks + ctx->sm_count - 1) / ctx->sm_count;
                    if (per_sm > cap) return 1ll << 40;  // more than one wave: not considered
                    return (per_sm * (threads / 32) + 3) / 4 * cpt;
                };
                const long long two = busiest(128, 2, 3), wide = busiest(352, 1, 2), plain = busiest(256, 1, 4);
                if (two <= wide && two <= plain) return launch_cfg<16, 4, false, false, 128, 2>(ctx, p);
                if (wide < plain) return launch_cfg<16, 4, false, false, 352>(ctx, p);
            }
            return launch_one<16, 4, false>(ctx, p);
        }
        if (s <= 128) return launch_one<16, 8, false>(ctx, p);
        if (s <= 256) return launch_one<16, 16, false>(ctx, p);
        if (s <= 512) return launch_one<16, 32, false>(ctx, p);
    }
    return fail(ctx, PSSA_B200_ERR_UNSUPPORTED, "B200 SSM: state width %d exceeds 512; refusing launch", s);
}

}  // namespace pssa
