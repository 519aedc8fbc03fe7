// Exact top-k Poincare memory read in ONE kernel: projection, distances, selection, softmax and value read for a tile
// of 128 queries without the [rows, capacity] distance matrix ever leaving the SM.
//
// Replaces `retrieve_soft_into` with `top_k` set (src/memory.rs:344-408: f64 distances rounded to f32, the k smallest
// `(distance bits, slot)` pairs, weights and value read in ascending slot order) and, like the other read kernels, the
// reference GPU's one-thread-per-token `memory_forward` (src/cuda/stages.ptx:358-446).
//
// The idea: the tensor cores are a PRE-FILTER, the reference's f64 arithmetic decides.
//   1. the CTA's eight warps project the tile's queries into the ball (f64, the reference's sequential sums: same bits) and write
//      the points as three bf16 pieces straight into the 128-byte-swizzled A operand in shared memory;
//   2. one thread issues tcgen05.mma for the three piece products above 2^-16 of p.k against the bank's keys (split the
//      same way once per upload, streamed by TMA through a 3-stage ring by one thread of another warp); the 128 x capacity
//      accumulator fills the SM's TMEM (512 fp32 columns). There are no dedicated producer or issuer warps: nothing else
//      can run while the product is formed (the ring is the other phases' scratch memory), so two of the eight warps take
//      the roles for that phase, and eight warps -- two per scheduler -- may use 255 registers each where ten were held
//      to 168 and spilled in the exact sums (1.22 -> 0.99 ms per 262,144 queries on the same GPU);
//   3. every thread owns one query row (its TMEM lane) and one half of the slots and reads that part of the
//      accumulator twice with tcgen05.ld: a first sweep finds a threshold that at least C = k + 1 slots pass (the C-th
//      smallest of the minima of v = |p-k|^2 / (1-|k|^2) over groups of 32, 16 or 8 slots, both halves merged), a second
//      sweep lists the slots under it (about a dozen of 512); the C smallest of the lists are the row's candidates;
//   4. DK/16 threads per row re-score the candidates as `poincare_distance` does (f64 differences squared and summed, f64
//      log1p form of 2 asinh sqrt, rounded to f32); one thread per row selects k by (bits, slot)
//      and proves the selection: the sweeps
//      also produced v_lb, the smallest (approximate v - its error bound) over every slot that did NOT become a candidate,
//      so the true distance of each of those is at least d(v_lb / (1-|p|^2)); if the k-th selected distance is strictly
//      below that, no other slot can enter or tie. Otherwise (or if the list overflowed) the row is flagged and the CTA
//      recomputes it at the end of the tile with f64 distances to every slot. Rare: a few rows per million.
//   5. softmax over the k selected slots (sum in ascending slot order) and the value read, fused.
// Every mbarrier wait is bounded like the GEMM pipeline's: on expiry the status word gets PSSA_B200_ERR_TIMEOUT and the
// kernel stops issuing work and frees its TMEM.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cfloat>
#include <math_constants.h>

#include "bounds.hpp"
#include "context.hpp"
#include "kernels.hpp"
#include "tcgen05.cuh"

namespace pssa {
namespace {
using namespace tc;

__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// packed fp32 pairs: one instruction, two IEEE-rounded results (the all-slots sweeps are bound by instruction issue next
// to their three hardware approximations per slot)
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
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

constexpr int kListHalf = 32;  // slots one column half of a row can list under its threshold (about 10 expected)
constexpr int kCandMax = 13;   // candidates re-scored per row: top_k + kMargin, at most this many (the kernel is
                               // instantiated for 9 and for 13)
constexpr int kMargin = 1;     // one spare candidate: the proof needs the k-th exact distance strictly under the bound of
                               // everything that is not a candidate, and the (k+1)-th nearest slot is the usual binder
constexpr int kValueBatch = 8;  // value rows a thread has in flight in the value read
constexpr int kWorkWarps = 8;  // every warp works; warps w and w + 4 share the TMEM lanes 32 (w % 4) .. + 31 (one query row per thread)
constexpr int kThreads = 32 * kWorkWarps;  // eight warps, two per scheduler: the whole register file (255 per thread) is usable
constexpr int kStages = 3;
constexpr int kPhases = kRetrievePhases;
constexpr int kRingStage = 256 * BK * 2;  // one key k-block of up to 256 slots: 32 KB
// Error bound of the pre-filter's t = |p - k|^2 = (|p|^2 - p.k) + (|k|^2 - p.k). The tensor cores multiply the three piece
// products above 2^-16 of p.k -- (p0, k0), (p0, k1), (p1, k0) with x = x0 + x1 + x2, |x1| <= 2^-9 |x|, |x2| <= 2^-17 |x| --
// so the dropped products are at most (2^-18 + 2 * 2^-17) sum |p_i k_i| <= 1.9e-5 |p| |k|, and the fp32 accumulation (not
// correctly rounded, about two dozen steps of 2^-23) adds at most 3e-6 |p| |k|: kEpsDot * |p| |k| covers both. The two fp32
// subtractions and the addition are covered by kEpsSum * (|p|^2 + |k|^2). A pre-filter this coarse is enough because its
// only job is to shortlist; the decision is made on exact distances.
constexpr float kEpsDot = 3e-5f;
constexpr float kEpsSum = 8e-7f;

__device__ __forceinline__ void bar_workers() { asm volatile("bar.sync 1, %0;" ::"n"(32 * kWorkWarps) : "memory"); }

__device__ __forceinline__ void split3(float x, __nv_bfloat16& a, __nv_bfloat16& b, __nv_bfloat16& c) {
    a = __float2bfloat16_rn(x);
    float r = x - __bfloat162float(a);
    b = __float2bfloat16_rn(r);
    c = __float2bfloat16_rn(r - __bfloat162float(b));
}

// byte offset of element (row, col) of a [128 rows x 64 bf16] K-major tile with the 128-byte swizzle (what a TMA box load
// with CU_TENSOR_MAP_SWIZZLE_128B produces): 16-byte chunk j of row i sits at chunk j ^ (i % 8)
__device__ __forceinline__ uint32_t sw128_offset(int row, int col) {
    return (uint32_t)(row * 128 + ((((col >> 3) ^ (row & 7)) << 4) | ((col & 7) << 1)));
}

// memory.rs:245-262 given the f64 squared distance: 2 asinh(sqrt(u)) = log1p(2u + 2 sqrt(u^2 + u)), rounded to f32
__device__ __forceinline__ float exact_distance(double sq, double one_minus_q, float key_norm_sq) {
    const double denom = one_minus_q * (1.0 - (double)key_norm_sq);
    const double u = sq / denom;
    return (float)log1p(2.0 * u + 2.0 * sqrt(fma(u, u, u)));
}

__device__ __forceinline__ unsigned long long umin64(unsigned long long a, unsigned long long b) { return a < b ? a : b; }
__device__ __forceinline__ unsigned long long umax64(unsigned long long a, unsigned long long b) { return a < b ? b : a; }

// memory.rs:198-211 + 181-188 for one row, sequential f64 sums: writes the projected point over `row` (dk floats),
// returns |p|^2 as the reference's f32 (nudged below one) and the Euclidean norm
__device__ __forceinline__ float project_row(float* row, int dk, bool euclid, float* q_norm_out) {
    double scale = 1.0;
    if (euclid) {
        double r2 = 0.0;
        for (int i = 0; i < dk; ++i) {
            const double v = (double)row[i];
            r2 = __dadd_rn(r2, __dmul_rn(v, v));
        }
        const double r = sqrt(r2);
        const double max_radius = 1.0 - 8.0 * (double)FLT_EPSILON;
        scale = (r == 0.0) ? 1.0 : fmin(r / (1.0 + r), max_radius) / r;
        if (q_norm_out) *q_norm_out = (float)fmin(r, (double)FLT_MAX);
    }
    double n2 = 0.0;
    for (int i = 0; i < dk; ++i) {
        const float pv = euclid ? (float)__dmul_rn((double)row[i], scale) : row[i];
        row[i] = pv;
        n2 = __dadd_rn(n2, __dmul_rn((double)pv, (double)pv));
    }
    return (n2 < 1.0 && (float)n2 == 1.0f) ? __uint_as_float(0x3f7fffffu) : (float)n2;
}

// Last stage of a row of the exact stage, one warp: the k selected slots arrive in ASCENDING SLOT ORDER (sel_slot / sel_w
// in shared memory, sel_w holding the distances); weights exp((min - d) / tau) summed in that order (memory.rs:391-398),
// normalised, value read in that order with separately rounded multiply and add (memory.rs:399-406).
__device__ __forceinline__ void finish_row(const RetrieveParams& p, size_t q, const unsigned* sel_slot, float* sel_w, int k, float dmin, int lane) {
    const float my_w = lane < k ? expf(__fdiv_rn(__fsub_rn(dmin, sel_w[lane]), p.tau)) : 0.0f;
    __syncwarp();
    if (lane < k) sel_w[lane] = my_w;
    __syncwarp();
    float sum = 0.0f;
    for (int j = 0; j < k; ++j) sum = __fadd_rn(sum, sel_w[j]);
    const float wn = __fdiv_rn(my_w, sum);
    __syncwarp();
    if (lane < k) sel_w[lane] = wn;
    __syncwarp();
    if (p.min_dist && lane == 0) p.min_dist[q] = dmin;
    if (p.topk_slots && lane < k) p.topk_slots[q * k + lane] = sel_slot[lane];
    if (p.topk_weights && lane < k) p.topk_weights[q * k + lane] = wn;
    if (p.weights) {  // the reference's dense row: zero except the selected slots; every address is written once, by the
                      // lane that owns it, so no ordering between a zero and a weight is needed
        float* row = p.weights + q * p.cap;
        for (int i = lane; i < p.cap; i += 32) {
            float w = 0.0f;
            for (int j = 0; j < k; ++j) w = sel_slot[j] == (unsigned)i ? sel_w[j] : w;
            row[i] = w;
        }
    }
    const int dv = p.dv;
    for (int c = lane; c < dv; c += 32) {
        float v[kCandMax - kMargin];  // every selected row's element is requested before the first is used
#pragma unroll
        for (int j = 0; j < kCandMax - kMargin; ++j)
            if (j < k) v[j] = __ldg(p.values + (size_t)sel_slot[j] * dv + c);
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < kCandMax - kMargin; ++j)
            if (j < k) acc = __fadd_rn(acc, __fmul_rn(sel_w[j], v[j]));
        if (p.m_val) p.m_val[q * dv + c] = acc;
        if (p.m_bf16) reinterpret_cast<__nv_bfloat16*>(p.m_bf16)[q * dv + c] = __float2bfloat16_rn(acc);
    }
}

// The exact stage of the one-kernel read, called by all worker threads with the same arguments: for each flagged row of
// the tile, f64 distances to EVERY occupied slot, each the reference's sequential sum (src/memory.rs:245-262), then k
// rounds of a warp-wide minimum over (distance bits, slot) and the row's outputs.
template <int DK>
__device__ __noinline__ void exact_rows(const RetrieveParams& p, size_t q0, const unsigned char* smem_a, const float* stat_qs, const int* flag_rows,
                                        int n_flag, float* fx_p, float* fx_dist, unsigned* fx_slot, float* fx_w, int wtid) {
    constexpr int KB_PIECE = DK / BK;
    constexpr uint32_t A_BLOCK = BM * BK * 2;
    const int lane = wtid & 31, wid = wtid >> 5, count = p.count, k = p.top_k;
    for (int f = 0; f < n_flag; ++f) {
        const int r = flag_rows[f];
        if (wtid < DK) {  // the projected point from its pieces
            const int c = wtid;
            const uint32_t off = sw128_offset(r, c % BK);
            const int kb = c / BK;
            const float x0 = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(smem_a + (0 * KB_PIECE + kb) * A_BLOCK + off));
            const float x1 = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(smem_a + (1 * KB_PIECE + kb) * A_BLOCK + off));
            const float x2 = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(smem_a + (2 * KB_PIECE + kb) * A_BLOCK + off));
            fx_p[c] = x0 + (x1 + x2);
        }
        bar_workers();
        const double one_minus_q = 1.0 - (double)stat_qs[r];
        for (int s = wtid; s < count; s += 2 * 32 * kWorkWarps) {  // two slots per pass: two independent f64 chains
            const int s2 = min(s + 32 * kWorkWarps, count - 1);      // (the last pass may compute a slot twice)
            const float4* ka = reinterpret_cast<const float4*>(p.keys + (size_t)s * DK);
            const float4* kb = reinterpret_cast<const float4*>(p.keys + (size_t)s2 * DK);
            double sa = 0.0, sb = 0.0;
            for (int i = 0; i < DK / 4; ++i) {
                const float4 a = __ldg(ka + i), b = __ldg(kb + i);
                const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const double pe = (double)fx_p[4 * i + e];
                    const double da = pe - (double)av[e], db = pe - (double)bv[e];
                    sa = fma(da, da, sa), sb = fma(db, db, sb);
                }
            }
            const float d_a = exact_distance(sa, one_minus_q, __ldg(p.norm_sq + s));
            const float d_b = exact_distance(sb, one_minus_q, __ldg(p.norm_sq + s2));
            fx_dist[s] = d_a;
            fx_dist[s2] = d_b;
        }
        bar_workers();
        if (wid == 0) {
            unsigned my_slot = 0xffffffffu;
            float my_dist = 0.0f, dmin = 0.0f;
            for (int round = 0; round < k; ++round) {
                unsigned long long local = ~0ull;
                for (int s = lane; s < count; s += 32) {
                    const unsigned bits = __float_as_uint(fx_dist[s]);
                    if (bits & 0x80000000u) continue;  // taken (distances are >= +0)
                    local = umin64(local, ((unsigned long long)bits << 32) | (unsigned)s);
                }
#pragma unroll
                for (int m = 16; m > 0; m >>= 1) local = umin64(local, __shfl_xor_sync(0xffffffffu, local, m));
                const unsigned slot = (unsigned)(local & 0xffffffffu);
                const float d = __uint_as_float((unsigned)(local >> 32));
                if (lane == 0) fx_dist[slot] = __uint_as_float(__float_as_uint(d) | 0x80000000u);
                if (lane == round) my_slot = slot, my_dist = d;
                if (round == 0) dmin = d;
                __syncwarp();
            }
            int srank = 0;
            for (int i = 0; i < k; ++i) srank += __shfl_sync(0xffffffffu, my_slot, i) < my_slot ? 1 : 0;
            if (lane < k) fx_slot[srank] = my_slot, fx_w[srank] = my_dist;
            __syncwarp();
            finish_row(p, q0 + r, fx_slot, fx_w, k, dmin, lane);
            if (lane == 0) atomicAdd(p.fixup_count, 1u);
        }
        bar_workers();
    }
}

// The value read of the proven rows (all worker threads; kept out of line so that the eight rows in flight have registers
// to live in): m = sum over the selected
// slots in ascending slot order of w * v, multiply and add separately rounded (memory.rs:399-406); a thread owns four
// columns of a row and has kValueBatch value rows in flight before the first is used. (Staging the rows in shared memory
// with bulk or 16-byte asynchronous copies measured two to three times slower: the gather is bound by the bytes a thread
// keeps in flight on 512-byte rows of L2.) Then the reference's dense weight row if the caller wants it.
template <int NC>
__device__ __noinline__ void read_selected_values(const float* __restrict__ values, int dv, float* m_val, void* m_bf16, float* weights, int cap, int k,
                                                  size_t q0, const unsigned* sels, const float* selw, const int* row_ok, int wtid) {
    const int dv4 = dv >> 2;
    for (int idx = wtid; idx < BM * dv4; idx += 32 * kWorkWarps) {
        const int r = idx / dv4, c4 = idx - r * dv4;
        if (!row_ok[r]) continue;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j0 = 0; j0 < k; j0 += kValueBatch) {
            float4 vv[kValueBatch];
#pragma unroll
            for (int e = 0; e < kValueBatch; ++e)
                if (j0 + e < k) vv[e] = __ldg(reinterpret_cast<const float4*>(values + (size_t)sels[r * NC + j0 + e] * dv) + c4);
#pragma unroll
            for (int e = 0; e < kValueBatch; ++e) {
                if (j0 + e < k) {
                    const float wi = selw[r * NC + j0 + e];
                    acc.x = __fadd_rn(acc.x, __fmul_rn(wi, vv[e].x)), acc.y = __fadd_rn(acc.y, __fmul_rn(wi, vv[e].y));
                    acc.z = __fadd_rn(acc.z, __fmul_rn(wi, vv[e].z)), acc.w = __fadd_rn(acc.w, __fmul_rn(wi, vv[e].w));
                }
            }
        }
        const size_t o = (q0 + r) * (size_t)dv + (size_t)c4 * 4;
        if (m_val) *reinterpret_cast<float4*>(m_val + o) = acc;
        if (m_bf16) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
            uint2 pk;
            pk.x = *reinterpret_cast<unsigned*>(&lo), pk.y = *reinterpret_cast<unsigned*>(&hi);
            *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(m_bf16) + o) = pk;
        }
    }
    if (weights) {
        for (int idx = wtid; idx < BM * cap; idx += 32 * kWorkWarps) {
            const int r = idx / cap, i = idx % cap;
            if (!row_ok[r]) continue;
            float w = 0.0f;
            for (int j = 0; j < k; ++j) w = sels[r * NC + j] == (unsigned)i ? selw[r * NC + j] : w;
            weights[(q0 + r) * (size_t)cap + i] = w;
        }
    }
}

// ALL: the all-slots read's front end instead of the top-k read. Same projection, split and pre-filter product; then the
// weights of EVERY slot leave as the bf16 operand of the value product, and nothing else: a thread owns one query row
// and one half of the slots, a first sweep over the accumulator finds the row's smallest v (the distance is monotone
// in it), a second one turns every v into exp((d_min - d) / tau) with three hardware approximations per slot
// (sqrt, lg2, ex2: the weight is (1 + z)^(-1/tau) for z = 2u + 2 sqrt(u^2 + u), so the logarithm of the distance
// and the exponential of the weight meet in one multiplication), sums them and parks them as bf16 in the shared memory
// the operands no longer need; a last pass scales the rows by one over their sums and writes them out as whole rows.
// The [rows, capacity] fp32 distance matrix and the projected points never reach HBM.
template <int DK, int NC, bool ALL = false>
__global__ void __launch_bounds__(kThreads, 1) retrieve_topk_fused_kernel(const __grid_constant__ CUtensorMap map_b, RetrieveParams p) {
    constexpr int KB_PIECE = DK / BK;        // k-blocks per bf16 piece
    constexpr int KB_A = 3 * KB_PIECE;       // k-blocks of the A operand (three pieces)
    constexpr uint32_t A_BLOCK = BM * BK * 2;  // 16 KB
    constexpr int PITCH = DK + 1;            // staging pitch in floats (bank spreading for one-thread-per-row walks)
    constexpr int L = DK / 16;               // lanes that share one row's exact sums (four float4 groups each)
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* smem_a = smem;                         // [KB_A][128 x 64 bf16], swizzled
    unsigned char* ring = smem_a + KB_A * A_BLOCK;        // [kStages][<=256 x 64 bf16] while the tensor cores run; otherwise:
    float* staging = reinterpret_cast<float*>(ring);      //   P0-P2: [128][PITCH] raw queries, then the projected points
    float* xbest = reinterpret_cast<float*>(ring);        //   P3: [2][NC][128] each column half's smallest group minima
    uint2* list_e = reinterpret_cast<uint2*>(xbest + 2 * NC * BM);  // P3-P4: [2][kListHalf + 1][128] listed (v bits, slot); the last row
                                                          //   takes the stores of slots that are not listed: no branch in the sweep
    double* sqbuf = reinterpret_cast<double*>(ring);      //   P5: [128][NC] exact squared distances of the candidates (f64)
    float* d32 = reinterpret_cast<float*>(sqbuf + BM * NC);  // P5: [128][NC + 1] exact distances of the candidates
    float* selw = d32 + BM * (NC + 1);                    //   P5: [128][NC] weights of the selected slots, ascending slot order
    unsigned* sels = reinterpret_cast<unsigned*>(selw + BM * NC);  // P5: [128][NC] the selected slots
    float* fx_p = reinterpret_cast<float*>(sels + BM * NC);       //   P5e: [DK] a flagged row's point
    float* fx_dist = fx_p + DK;                                   //   P5e: [512] its distance to every slot
    unsigned* fx_slot = reinterpret_cast<unsigned*>(fx_dist + 512);  // P5e: [32] selected slots, ascending
    float* fx_w = reinterpret_cast<float*>(fx_slot + 32);         //   P5e: [32] their distances, then weights
    int* flag_rows = reinterpret_cast<int*>(fx_w + 32);           //   P5c-P5e: [128] rows of the tile whose selection is not proven
    int* flag_count = flag_rows + BM;                             //   and how many
    unsigned char* tail = ring + kStages * kRingStage;
    float2* kcol_s = reinterpret_cast<float2*>(tail);                      // [cap <= 512] per-slot constants (|k|^2, 1/(1-|k|^2)), see below
    float* kerr_s = reinterpret_cast<float*>(kcol_s + 512);                // [cap <= 512] kEpsDot |k| / (1-|k|^2)
    float* stat_qs = kerr_s + 512;                                         // [128] |p|^2
    float* stat_excl = stat_qs + BM;                                       // [2][128] lower bound of the true v of: the unlisted slots; every non-candidate
    int* stat_cnt = reinterpret_cast<int*>(stat_excl + 2 * BM);            // [2][128] listed slots per column half
    unsigned* stat_dlb = reinterpret_cast<unsigned*>(stat_cnt + 2 * BM);   // [128] bits of the distance no non-candidate can be under
    unsigned* stat_mark = stat_dlb + BM;                                   // [128] 1 = the row's candidates are re-scored; 0 = handed over (or past the end)
    int* row_ok = reinterpret_cast<int*>(stat_mark + BM);                  // [128] 1 = selection proven, results in selw / sels
    unsigned short* cand_slot = reinterpret_cast<unsigned short*>(row_ok + BM);  // [128][kCandMax]
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(cand_slot + BM * kCandMax);
    uint64_t* empty_bar = full_bar + kStages;
    uint64_t* acc_full = empty_bar + kStages;
    long long* phase_clk = reinterpret_cast<long long*>(acc_full + 1);  // [kPhases]
    int* kmax_i = reinterpret_cast<int*>(phase_clk + kPhases);          // [4] maxima over the occupied slots of kcol_s .w, .y, .x (floats >= 0)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(kmax_i + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int dk = DK, cap = p.cap, count = p.count, k = p.top_k;
    const int nh = cap >= 256 ? 256 : cap;   // slots per MMA (N) and per TMA box
    const int halves = cap / nh;
    const int n_cand = min(k + kMargin, NC);
    // columns per group minimum: 32 when that leaves enough fully occupied groups to bound n_cand slots (plus two to
    // keep the bound tight), else 16 or 8; smaller groups give a lower threshold and shorter lists but more insertions
    int group = 32;
    while (group > 8 && count / group < n_cand + 2) group >>= 1;
    const long long n_tiles = (long long)((p.rows + BM - 1) / BM);
    const uint32_t tmem_cols = (uint32_t)cap;  // 128, 256 or 512: a power of two >= 32

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&full_bar[s], 1), mbar_init(&empty_bar[s], 1);
        mbar_init(acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < 4) kmax_i[threadIdx.x] = 0;
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // Per slot, with n = |k|^2 and s = 1 / (1 - n) from the upload: for a row with |p|^2 = q and accumulator a = p.k the
    // pre-filter value is v = (q + n - 2 a) s, computed as fma(-2, a, q + n) * s: nothing is rounded at a size above
    // (q + n) s, which kEpsSum covers; its error bound is (kEpsDot |p| |k| + kEpsSum (q + n)) s. Slots past `count` get
    // n = 3e38, s = 1: v = 3e38, never listed. The maxima of the error-bound terms over the occupied slots give a bound
    // that holds for EVERY slot of a row.
    {
        float m_e = 0.0f, m_s = 0.0f, m_ns = 0.0f;
        for (int i = threadIdx.x; i < cap; i += kThreads) {
            const float2 ks = p.k_stat[i];
            const float kn = sqrtf(ks.x) * 1.0000002f;  // rounded up: it scales an error bound
            const float e = kEpsDot * kn * ks.y * 1.0000002f;
            const float2 kv = i < count ? ks : make_float2(3.0e38f, 1.0f);
            if constexpr (ALL) {  // slot pairs as (n0, n1, s0, s1): one 16-byte load feeds packed arithmetic on two columns
                float* pair = reinterpret_cast<float*>(kcol_s) + 4 * (i >> 1) + (i & 1);
                pair[0] = kv.x, pair[2] = kv.y;
            } else {
                kcol_s[i] = kv;
            }
            kerr_s[i] = i < count ? e : 0.0f;
            if (i < count) m_e = fmaxf(m_e, e), m_s = fmaxf(m_s, ks.y), m_ns = fmaxf(m_ns, ks.x * ks.y * 1.0000002f);
        }
        atomicMax(&kmax_i[0], __float_as_int(m_e));  // non-negative floats order like their bits
        atomicMax(&kmax_i[1], __float_as_int(m_s));
        atomicMax(&kmax_i[2], __float_as_int(m_ns));
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_trigger();
    pdl_wait();

    // Stages per half: every k-block of key piece 0, then of key piece 1. A stage of piece 0 is multiplied with point
    // pieces 0 and 1, a stage of piece 1 with point piece 0: three products from two loads.
    const int n_kb = 2 * KB_PIECE;

    {
        // ---------------- workers
        const int wid = warp;                     // 0..7
        const int wtid = threadIdx.x;             // 0..255
        const int my_row = (warp & 3) * 32 + lane;
        const bool vec_q = (((p.ldq ? p.ldq : (size_t)dk) & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.q) & 15) == 0);
        uint32_t it = 0;
        bool alive = true;
        if (wtid < kPhases) phase_clk[wtid] = 0;  // (ordered before the first lap by the first worker barrier)
        for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
            const size_t q0 = (size_t)tile * BM;
            const size_t ldq = p.ldq ? p.ldq : (size_t)dk;
            long long t_prev = clock64();
            auto lap = [&](int i) {  // one thread's view of the phases; in shared memory to keep registers free
                if (wtid == 0) {
                    const long long now = clock64();
                    phase_clk[i] += now - t_prev, t_prev = now;
                }
            };
            // ---- P0: the tile's raw queries, coalesced, into the staging rows
            if (vec_q) {
                for (int idx = wtid; idx < BM * (DK / 4); idx += 32 * kWorkWarps) {
                    const int r = idx / (DK / 4), c4 = idx % (DK / 4);
                    const float4 v = q0 + r < p.rows ? __ldg(reinterpret_cast<const float4*>(p.q + (q0 + r) * ldq) + c4) : make_float4(0.f, 0.f, 0.f, 0.f);
                    float* dst = staging + r * PITCH + c4 * 4;
                    dst[0] = v.x, dst[1] = v.y, dst[2] = v.z, dst[3] = v.w;
                }
            } else {
                for (int idx = wtid; idx < BM * DK; idx += 32 * kWorkWarps) {
                    const int r = idx / DK, c = idx % DK;
                    staging[r * PITCH + c] = q0 + r < p.rows ? __ldg(p.q + (q0 + r) * ldq + c) : 0.0f;
                }
            }
            bar_workers();
            lap(0);
            // ---- P1: one thread per row projects it (memory.rs:198-211), in place. The all-slots front end, whose consumers
            // keep bf16-grade weights, only forms the row's scale here (two threads per row, fp32 partial sums) and applies
            // it while splitting; |p|^2 follows from the norm and the scale.
            float* row_scale = reinterpret_cast<float*>(stat_dlb);  // [128], all-slots mode only
            if constexpr (ALL) {
                const int r = wtid >> 1, half = wtid & 1;
                const float* row = staging + r * PITCH + half * (DK / 2);
                float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
                for (int i = 0; i < DK / 2; i += 4)
                    s0 = fmaf(row[i], row[i], s0), s1 = fmaf(row[i + 1], row[i + 1], s1), s2 = fmaf(row[i + 2], row[i + 2], s2),
                    s3 = fmaf(row[i + 3], row[i + 3], s3);
                float r2 = (s0 + s1) + (s2 + s3);
                r2 += __shfl_xor_sync(0xffffffffu, r2, 1);
                if (half == 0) {
                    float scale = 1.0f, n2 = r2;
                    if (p.q_is_euclidean) {
                        const double rr = sqrt((double)r2);
                        const double max_radius = 1.0 - 8.0 * (double)FLT_EPSILON;
                        const double sc = (rr == 0.0) ? 1.0 : fmin(rr / (1.0 + rr), max_radius) / rr;
                        scale = (float)sc;
                        n2 = (float)((rr * sc) * (rr * sc));
                        if (p.q_norm && q0 + r < p.rows) p.q_norm[q0 + r] = (float)fmin(rr, (double)FLT_MAX);
                    }
                    row_scale[r] = scale;
                    stat_qs[r] = fminf(n2, __uint_as_float(0x3f7fffffu));
                }
            } else if (wtid < BM) {
                float qn = 0.0f;
                const float qs = project_row(staging + wtid * PITCH, dk, p.q_is_euclidean != 0, &qn);
                stat_qs[wtid] = qs;
                if (p.q_norm && p.q_is_euclidean && q0 + wtid < p.rows) p.q_norm[q0 + wtid] = qn;
            }
            bar_workers();
            lap(1);
            // ---- P2: three bf16 pieces of every coordinate into the swizzled A operand; q_pnc goes out
            for (int idx = wtid; idx < BM * (DK / 2); idx += 32 * kWorkWarps) {
                const int r = idx / (DK / 2), c = (idx % (DK / 2)) * 2;
                float v0 = staging[r * PITCH + c], v1 = staging[r * PITCH + c + 1];
                if constexpr (ALL) v0 *= row_scale[r], v1 *= row_scale[r];
                if (p.q_pnc && q0 + r < p.rows) {
                    p.q_pnc[(q0 + r) * dk + c] = v0;
                    p.q_pnc[(q0 + r) * dk + c + 1] = v1;
                }
                __nv_bfloat16 a0, b0, c0, a1, b1, c1;
                split3(v0, a0, b0, c0);
                split3(v1, a1, b1, c1);
                const int kb = c / BK, cc = c % BK;
                const uint32_t off = sw128_offset(r, cc);
                *reinterpret_cast<__nv_bfloat162*>(smem_a + (0 * KB_PIECE + kb) * A_BLOCK + off) = __halves2bfloat162(a0, a1);
                *reinterpret_cast<__nv_bfloat162*>(smem_a + (1 * KB_PIECE + kb) * A_BLOCK + off) = __halves2bfloat162(b0, b1);
                *reinterpret_cast<__nv_bfloat162*>(smem_a + (2 * KB_PIECE + kb) * A_BLOCK + off) = __halves2bfloat162(c0, c1);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the tensor cores
            tcgen05_fence_before();
            bar_workers();  // the ring is free for key pieces and the operand is complete
            lap(2);
            // ---- the tensor-core phase: while the other warps wait for the accumulator, one thread of warp 0 sends the key
            // pieces through the ring and one thread of warp 1 issues the MMAs (128 x nh x 16 into TMEM columns
            // [h * nh, (h + 1) * nh)). Stages per half: every k-block of key piece 0, then of key piece 1.
            if (wid == 0) {
                if (lane == 0) {
                    uint32_t g = it * (uint32_t)(halves * n_kb);
                    bool ok = true;
                    for (int h = 0; h < halves && ok; ++h)
                        for (int kb = 0; kb < n_kb; ++kb, ++g) {
                            const int s = g % kStages;
                            const uint32_t round = g / kStages;
                            if (round > 0 && !mbar_wait(&empty_bar[s], (round - 1) & 1)) {
                                atomicExch(p.status, PSSA_B200_ERR_TIMEOUT);
                                ok = false;
                                break;
                            }
                            mbar_expect_tx(&full_bar[s], (uint32_t)nh * BK * 2);
                            tma_load_2d(ring + s * kRingStage, &map_b, &full_bar[s], kb * BK, h * nh);  // piece kb / KB_PIECE, block kb % KB_PIECE
                        }
                }
                __syncwarp();
            } else if (wid == 1) {
                if (lane == 0) {
                    const uint32_t idesc = umma_idesc_bf16(BM, nh);
                    uint32_t g = it * (uint32_t)(halves * n_kb);
                    bool ok = true;
                    tcgen05_fence_after();
                    for (int h = 0; h < halves && ok; ++h)
                        for (int kb = 0; kb < n_kb; ++kb, ++g) {
                            const int s = g % kStages;
                            if (!mbar_wait(&full_bar[s], (g / kStages) & 1)) {
                                atomicExch(p.status, PSSA_B200_ERR_TIMEOUT);
                                ok = false;
                                break;
                            }
                            tcgen05_fence_after();
                            const int key_piece = kb / KB_PIECE, within = kb % KB_PIECE;
                            const uint64_t db = umma_desc_sw128(smem_u32(ring + s * kRingStage));
                            for (int a = 0; a < (key_piece == 0 ? 2 : 1); ++a) {
                                const uint64_t da = umma_desc_sw128(smem_u32(smem_a + (a * KB_PIECE + within) * A_BLOCK));
#pragma unroll
                                for (int kk = 0; kk < BK / UMMA_K; ++kk)
                                    tcgen05_mma_bf16(tmem_base + h * nh, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (kb > 0 || a > 0 || kk > 0) ? 1u : 0u);
                            }
                            tcgen05_commit(&empty_bar[s]);
                        }
                    tcgen05_commit(acc_full);  // all products of this tile are in TMEM (or abandoned)
                }
                __syncwarp();
            }
            // ---- P3: two sweeps over the accumulator. All eight warps: a thread owns one query row (its TMEM lane) and one
            // half of the slots (columns): warps 0..3 the lower half, warps 4..7 the upper.
            const int ch = wid >> 2;
            const int c_begin = ch * (cap / 2), c_end = c_begin + cap / 2;
            if (alive) {  // every lane waits (each needs the barrier's acquire); the verdict is made warp-uniform
                const bool ok = mbar_wait(acc_full, it & 1);
                alive = __all_sync(0xffffffffu, ok);
                if (!alive && lane == 0) atomicExch(p.status, PSSA_B200_ERR_TIMEOUT);
            }
            tcgen05_fence_after();
            lap(3);  // waiting for the tensor cores
            if constexpr (ALL) {
                const int ch = wid >> 2;
                const int c_begin = ch * (cap / 2), c_end = c_begin + cap / 2;
                const float qs = stat_qs[my_row];
                const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
                const float inv1mq = __fdividef(1.0f, 1.0f - qs);
                const float inv_tau = __fdividef(1.0f, p.tau);
                constexpr int W_PITCH = 512 + 8;  // bf16 elements per parked row: 16 bytes of padding spread the banks
                __nv_bfloat16* park = reinterpret_cast<__nv_bfloat16*>(smem_a);  // [128][W_PITCH]: over the operand and the ring
                float* row_min = stat_excl;                                     // [2][128] smallest v per column half
                float* row_sum = reinterpret_cast<float*>(stat_cnt);            // [2][128] sum of the weights per column half
                uint32_t buf0[32], buf1[32];
                float vmin = CUDART_INF_F, sum = 0.0f, lg_min_t = 0.0f;
                if (alive) {
                    const f32x2 qs2 = pack2(qs, qs), m2 = pack2(-2.0f, -2.0f);
                    const float4* kpair = reinterpret_cast<const float4*>(kcol_s);
                    auto minimum = [&](const uint32_t (&acc)[32], int c0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            const float4 kc = kpair[(c0 + j) >> 1];
                            float v0, v1;
                            unpack2(mul2(fma2(m2, pack2(__uint_as_float(acc[j]), __uint_as_float(acc[j + 1])), add2(qs2, pack2(kc.x, kc.y))),
                                         pack2(kc.z, kc.w)), v0, v1);
                            vmin = fminf(vmin, fminf(v0, v1));
                        }
                    };
                    tcgen05_ld_32x32_issue(taddr + c_begin, buf0);
                    for (int c0 = c_begin; c0 < c_end; c0 += 64) {
                        tcgen05_wait_ld(buf0);
                        tcgen05_ld_32x32_issue(taddr + c0 + 32, buf1);
                        minimum(buf0, c0);
                        tcgen05_wait_ld(buf1);
                        tcgen05_ld_32x32_issue(taddr + (c0 + 64 < c_end ? c0 + 64 : c_begin), buf0);  // wraps to the second sweep's first columns
                        minimum(buf1, c0 + 32);
                    }
                }
                row_min[ch * BM + my_row] = vmin;
                bar_workers();
                lap(4);
                {
                    // lg2(1 + z) of the row's nearest slot, times 1 / tau: the exponent every weight is measured against
                    const float u = fmaxf(fminf(row_min[my_row], row_min[BM + my_row]), 0.0f) * inv1mq;
                    float r, lg;
                    const float t = fmaf(u, u, u);
                    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(t));
                    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(lg) : "f"(1.0f + fmaf(2.0f, r, 2.0f * u)));
                    lg_min_t = lg * inv_tau;
                }
                lap(5);
                // with row_scale_out the rows leave as they are, straight from this sweep (16 bytes per row and instruction: the
                // stores ride under the sweep's XU work), and the consumer multiplies by 1 / sum; otherwise they are parked
                const bool defer = p.row_scale_out != nullptr;
                if (alive) {
                    __nv_bfloat16* my_park = defer ? reinterpret_cast<__nv_bfloat16*>(p.w_split) + (q0 + my_row) * (size_t)(3 * cap)
                                                   : park + (size_t)my_row * W_PITCH;
                    const f32x2 qs2 = pack2(qs, qs), m2 = pack2(-2.0f, -2.0f), inv1mq2 = pack2(inv1mq, inv1mq), two2 = pack2(2.0f, 2.0f),
                                one2 = pack2(1.0f, 1.0f), ninv_tau2 = pack2(-inv_tau, -inv_tau), lg_min_t2 = pack2(lg_min_t, lg_min_t);
                    const float4* kpair = reinterpret_cast<const float4*>(kcol_s);
                    f32x2 sum2 = pack2(0.0f, 0.0f);
                    const bool row_in = !defer || q0 + my_row < p.rows;
                    auto weights = [&](const uint32_t (&acc)[32], int c0) {
#pragma unroll
                        for (int j0 = 0; j0 < 32; j0 += 16) {
                            float e[16];
#pragma unroll
                            for (int j = 0; j < 16; j += 2) {
                                const float4 kc = kpair[(c0 + j0 + j) >> 1];
                                // slots past the occupied ones carry v = 3e38: every step below keeps the infinity and the weight is 0
                                float u0, u1;
                                unpack2(mul2(mul2(fma2(m2, pack2(__uint_as_float(acc[j0 + j]), __uint_as_float(acc[j0 + j + 1])),
                                                       add2(qs2, pack2(kc.x, kc.y))),
                                                  pack2(kc.z, kc.w)),
                                             inv1mq2),
                                        u0, u1);
                                const f32x2 u2 = pack2(fmaxf(u0, 0.0f), fmaxf(u1, 0.0f));
                                float t0, t1, r0, r1, w0, w1, l0, l1, x0, x1;
                                unpack2(fma2(u2, u2, u2), t0, t1);
                                asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r0) : "f"(t0));
                                asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r1) : "f"(t1));
                                unpack2(fma2(two2, pack2(r0, r1), fma2(two2, u2, one2)), w0, w1);
                                asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(l0) : "f"(w0));
                                asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(l1) : "f"(w1));
                                unpack2(fma2(ninv_tau2, pack2(l0, l1), lg_min_t2), x0, x1);
                                e[j] = ex2_fast(x0), e[j + 1] = ex2_fast(x1);
                                sum2 = add2(sum2, pack2(e[j], e[j + 1]));
                            }
                            uint32_t pk[8];
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                const __nv_bfloat162 hq = __floats2bfloat162_rn(e[2 * q], e[2 * q + 1]);
                                pk[q] = *reinterpret_cast<const uint32_t*>(&hq);
                            }
                            if (defer) {
                                // 32 bytes per thread and instruction: a whole sector of the row at once
                                if (row_in)
                                    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(my_park + c0 + j0), "r"(pk[0]),
                                                 "r"(pk[1]), "r"(pk[2]), "r"(pk[3]), "r"(pk[4]), "r"(pk[5]), "r"(pk[6]), "r"(pk[7])
                                                 : "memory");
                            } else {
                                *reinterpret_cast<uint4*>(my_park + c0 + j0) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                                *reinterpret_cast<uint4*>(my_park + c0 + j0 + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                            }
                        }
                    };
                    for (int c0 = c_begin; c0 < c_end; c0 += 64) {
                        tcgen05_wait_ld(buf0);
                        tcgen05_ld_32x32_issue(taddr + c0 + 32, buf1);
                        weights(buf0, c0);
                        tcgen05_wait_ld(buf1);
                        if (c0 + 64 < c_end) tcgen05_ld_32x32_issue(taddr + c0 + 64, buf0);
                        weights(buf1, c0 + 32);
                    }
                    float s_lo, s_hi;
                    unpack2(sum2, s_lo, s_hi);
                    sum = s_lo + s_hi;
                }
                tcgen05_fence_before();
                row_sum[ch * BM + my_row] = sum;
                bar_workers();
                lap(6);
                if (defer) {
                    if (wtid < BM && q0 + wtid < p.rows) p.row_scale_out[q0 + wtid] = __fdividef(1.0f, row_sum[wtid] + row_sum[BM + wtid]);
                } else {
                    // the rows go out normalised, 16 bytes per thread and consecutive threads along a row: whole 128-byte
                    // lines; four rows per pass, their loads issued before the first is used
                    const int c8n = cap >> 3;                    // 16-byte pieces per row: 16, 32 or 64
                    const int c8 = wtid % c8n, r_first = wtid / c8n, r_step = (32 * kWorkWarps) / c8n;
                    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.w_split);
                    for (int r0 = r_first; r0 < BM; r0 += 4 * r_step) {
                        uint4 pk[4];
                        float inv[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int r = r0 + u * r_step;
                            if (r < BM) {
                                pk[u] = *reinterpret_cast<const uint4*>(park + (size_t)r * W_PITCH + c8 * 8);
                                inv[u] = row_sum[r] + row_sum[BM + r];
                            }
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int r = r0 + u * r_step;
                            if (r < BM && q0 + r < p.rows) {
                                const float sc = __fdividef(1.0f, inv[u]);
                                uint32_t* w4 = reinterpret_cast<uint32_t*>(&pk[u]);
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w4[e]));
                                    const __nv_bfloat162 o = __floats2bfloat162_rn(f.x * sc, f.y * sc);
                                    w4[e] = *reinterpret_cast<const uint32_t*>(&o);
                                }
                                *reinterpret_cast<uint4*>(out + (q0 + r) * (size_t)(3 * cap) + c8 * 8) = pk[u];
                            }
                        }
                    }
                }
                bar_workers();  // the parked rows are consumed: the next tile may overwrite the operand and the ring
                lap(7);
            } else {
                const float qs = stat_qs[my_row];
                const float pn = sqrtf(qs) * 1.0000002f;
                const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
                float best[NC];
    #pragma unroll
                for (int i = 0; i < NC; ++i) best[i] = CUDART_INF_F;
                auto insert_best = [&](float x) {  // keep the NC smallest, sorted; branch-free
    #pragma unroll
                    for (int i = 0; i < NC; ++i) {
                        const float lo = fminf(best[i], x), hi = fmaxf(best[i], x);
                        best[i] = lo, x = hi;
                    }
                };
                // both sweeps read 32 columns per tcgen05.ld into one of two register buffers, the next load in flight while
                // the current buffer is used
                uint32_t buf0[32], buf1[32];
                if (alive) {
                    // sweep 1: group minima
                    auto minima = [&](const uint32_t (&acc)[32], int c0) {
                        float vmin[4] = {CUDART_INF_F, CUDART_INF_F, CUDART_INF_F, CUDART_INF_F};  // minima of the four groups of 8 columns
    #pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float2 kc = kcol_s[c0 + j];
                            vmin[j >> 3] = fminf(vmin[j >> 3], fmaf(-2.0f, __uint_as_float(acc[j]), qs + kc.x) * kc.y);
                        }
                        if (group == 32) {
                            insert_best(fminf(fminf(vmin[0], vmin[1]), fminf(vmin[2], vmin[3])));
                        } else if (group == 16) {
                            insert_best(fminf(vmin[0], vmin[1]));
                            insert_best(fminf(vmin[2], vmin[3]));
                        } else {
    #pragma unroll
                            for (int g = 0; g < 4; ++g) insert_best(vmin[g]);
                        }
                    };
                    tcgen05_ld_32x32_issue(taddr + c_begin, buf0);
                    for (int c0 = c_begin; c0 < c_end; c0 += 64) {
                        tcgen05_wait_ld(buf0);
                        tcgen05_ld_32x32_issue(taddr + c0 + 32, buf1);
                        minima(buf0, c0);
                        tcgen05_wait_ld(buf1);
                        tcgen05_ld_32x32_issue(taddr + (c0 + 64 < c_end ? c0 + 64 : c_begin), buf0);  // wraps to the second sweep's first columns
                        minima(buf1, c0 + 32);
                    }
                }
    #pragma unroll
                for (int i = 0; i < NC; ++i) xbest[(ch * NC + i) * BM + my_row] = best[i];
                bar_workers();
                lap(4);
                // the threshold: the n_cand-th smallest group minimum over BOTH halves (at least n_cand slots lie at or under it)
                {
                    const int other = 1 - ch;
    #pragma unroll
                    for (int i = 0; i < NC; ++i) insert_best(xbest[(other * NC + i) * BM + my_row]);
                }
                float theta = CUDART_INF_F;
    #pragma unroll
                for (int i = 0; i < NC; ++i)
                    if (i == n_cand - 1) theta = best[i];
                // e_cap bounds the pre-filter error of EVERY slot of this row. Slots up to theta + 2.5 e_cap are listed, so an
                // unlisted slot's true v is above theta + 1.5 e_cap; theta + e_cap (rounded) is the bound that goes on.
                const float e_cap = fmaf(pn, __int_as_float(kmax_i[0]), kEpsSum * fmaf(qs, __int_as_float(kmax_i[1]), __int_as_float(kmax_i[2]))) * 1.000001f;
                const float t2 = fmaf(2.5f, e_cap, theta);
                if (ch == 0) stat_excl[my_row] = theta + e_cap;
                lap(5);
                int cnt = 0;
                if (alive) {
                    uint2* const my_list = list_e + (size_t)ch * (kListHalf + 1) * BM + my_row;
                    uint2* const spare = my_list + kListHalf * BM;
                    uint2* wp = my_list;  // the list's end
                    // sweep 2: list the slots at or under the widened threshold: a predicated store at the list's end, which
                    // stops advancing at the spare row (a list that reaches it counts as overflowed)
                    auto listing = [&](const uint32_t (&acc)[32], int c0) {
    #pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float2 kc = kcol_s[c0 + j];
                            const float v = fmaf(-2.0f, __uint_as_float(acc[j]), qs + kc.x) * kc.y;
                            if (v <= t2) {
                                *wp = make_uint2(__float_as_uint(v), (unsigned)(c0 + j));
                                if (wp != spare) wp += BM;
                            }
                        }
                    };
                    for (int c0 = c_begin; c0 < c_end; c0 += 64) {
                        tcgen05_wait_ld(buf0);
                        tcgen05_ld_32x32_issue(taddr + c0 + 32, buf1);
                        listing(buf0, c0);
                        tcgen05_wait_ld(buf1);
                        if (c0 + 64 < c_end) tcgen05_ld_32x32_issue(taddr + c0 + 64, buf0);
                        listing(buf1, c0 + 32);
                    }
                    cnt = (int)((wp - my_list) / BM);
                    if (cnt == kListHalf) cnt = kListHalf + 1;
                }
                tcgen05_fence_before();
                stat_cnt[ch * BM + my_row] = alive ? cnt : kListHalf + 1;
                bar_workers();
                lap(6);
                // ---- P4: one thread per row: the n_cand smallest of the two lists by (v, slot) and the lower bound of the true v
                // of everything else
                if (wtid < BM) {
                    const int r = wtid;
                    const float qs_r = stat_qs[r];
                    const float pn_r = sqrtf(qs_r) * 1.0000002f;
                    float excl_r = stat_excl[r];
                    const int cnt0 = stat_cnt[r], cnt1 = stat_cnt[BM + r];
                    const bool trusted = cnt0 <= kListHalf && cnt1 <= kListHalf;
                    // keys (v bits, slot): v >= -tiny; a value rounded below zero sorts by its magnitude, still among the smallest
                    unsigned long long top[NC];
    #pragma unroll
                    for (int i = 0; i < NC; ++i) top[i] = ~0ull;
                    for (int h = 0; h < 2; ++h) {
                        const int n_list = min(h == 0 ? cnt0 : cnt1, kListHalf);
                        for (int e = 0; e < n_list; ++e) {
                            const uint2 le = list_e[(h * (kListHalf + 1) + e) * BM + r];
                            unsigned long long x = ((unsigned long long)(le.x & 0x7fffffffu) << 32) | le.y;
    #pragma unroll
                            for (int i = 0; i < NC; ++i) {
                                if (i < n_cand) {  // entries past the candidates stay empty: what falls out of the first n_cand is excluded
                                    const unsigned long long lo = umin64(top[i], x), hi = umax64(top[i], x);
                                    top[i] = lo, x = hi;
                                }
                            }
                            if (x != ~0ull) {  // a listed slot that is not (or no longer) a candidate: v minus its own error bound
                                const unsigned slot = (unsigned)(x & 0xffffu);
                                const float2 kc = kcol_s[slot];
                                const float w = (qs_r + kc.x) * kc.y * 1.0000002f;
                                excl_r = fminf(excl_r, fmaf(-pn_r, kerr_s[slot], fmaf(-kEpsSum, w, __uint_as_float((unsigned)(x >> 32)))));
                            }
                        }
                    }
    #pragma unroll
                    for (int i = 0; i < NC; ++i) cand_slot[r * kCandMax + i] = (unsigned short)(top[i] & 0xffffu);
                    stat_excl[BM + r] = excl_r;
                    // untrusted (a list overflowed), nothing to bound with, or past the end: no re-scoring; P5c hands the row over
                    stat_mark[r] = (trusted && excl_r > 0.0f && q0 + r < p.rows) ? 1u : 0u;
                }
                bar_workers();  // the lists are consumed: their memory becomes the exact stage's
                if (wtid == 0) *flag_count = 0;  // (ordered before P5c's increments by the barriers in between)
                lap(7);
                // the next tile's queries towards the L2 while this tile is finished
                {
                    const long long next = tile + gridDim.x;
                    if (next < n_tiles) {
                        constexpr int LPR = DK * 4 / 128;  // 128-byte lines per row
                        for (int idx = wtid; idx < BM * LPR; idx += 32 * kWorkWarps) {
                            const size_t r = (size_t)next * BM + idx / LPR;
                            if (r < p.rows) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.q + r * ldq + (idx % LPR) * 32));
                        }
                    }
                }
                // ---- P5a: exact squared distances, L = DK/16 lanes per row: lane g of a row holds the coordinates 4 (L s + g) .. + 3
                // (s = 0..3) of the projected point as f64 -- the sum of the three bf16 pieces is the fp32 point, exactly -- and walks
                // the row's candidates with the next two candidates' keys in flight: f64 differences to the key, squared and summed in
                // four partial sums that are combined in a fixed order within the lane and then across the L lanes. Like the
                // separate f64 kernel's fused multiply-adds this differs from the reference's one sequential sum only in the last
                // bits of an f64 that is then rounded to f32. Conversions to f64 are the slow instructions here: the point is
                // converted once per row.
                for (int item = wtid; item < BM * L; item += 32 * kWorkWarps) {
                    const int r = item / L, g = item % L;
                    const bool active = stat_mark[r] != 0u;  // uniform over the lanes of a row
                    double pd[4][4];
    #pragma unroll
                    for (int s = 0; s < 4; ++s) {
                        const int c = 4 * (L * s + g);
                        const uint32_t off = sw128_offset(r, c % BK);
                        const int kb = c / BK;
                        const uint2 x0 = *reinterpret_cast<const uint2*>(smem_a + (0 * KB_PIECE + kb) * A_BLOCK + off);
                        const uint2 x1 = *reinterpret_cast<const uint2*>(smem_a + (1 * KB_PIECE + kb) * A_BLOCK + off);
                        const uint2 x2 = *reinterpret_cast<const uint2*>(smem_a + (2 * KB_PIECE + kb) * A_BLOCK + off);
                        // a bf16 is the upper half of its fp32
                        pd[s][0] = (double)(__uint_as_float(x0.x << 16) + (__uint_as_float(x1.x << 16) + __uint_as_float(x2.x << 16)));
                        pd[s][1] = (double)(__uint_as_float(x0.x & 0xffff0000u) + (__uint_as_float(x1.x & 0xffff0000u) + __uint_as_float(x2.x & 0xffff0000u)));
                        pd[s][2] = (double)(__uint_as_float(x0.y << 16) + (__uint_as_float(x1.y << 16) + __uint_as_float(x2.y << 16)));
                        pd[s][3] = (double)(__uint_as_float(x0.y & 0xffff0000u) + (__uint_as_float(x1.y & 0xffff0000u) + __uint_as_float(x2.y & 0xffff0000u)));
                    }
                    const unsigned short* cs = cand_slot + r * kCandMax;
                    float4 kv[3][4];  // a ring of three keys: two in flight ahead of the one in use
                    auto fetch = [&](int j, float4 (&dst)[4]) {
                        const float4* krow = reinterpret_cast<const float4*>(p.keys + (size_t)cs[j] * dk) + g;
    #pragma unroll
                        for (int s = 0; s < 4; ++s) dst[s] = __ldg(krow + L * s);
                    };
                    double tot[NC];
                    if (active) {
                        fetch(0, kv[0]);
                        if (1 < n_cand) fetch(1, kv[1]);
                    }
    #pragma unroll
                    for (int j = 0; j < NC; ++j) {
                        tot[j] = 0.0;
                        if (active && j < n_cand) {
                            if (j + 2 < n_cand) fetch(j + 2, kv[(j + 2) % 3]);
                            double s0 = 0.0, s1 = 0.0, s2 = 0.0, s3 = 0.0;
    #pragma unroll
                            for (int s = 0; s < 4; ++s) {
                                const float4 kk = kv[j % 3][s];
                                const double d0 = pd[s][0] - (double)kk.x, d1 = pd[s][1] - (double)kk.y;
                                const double d2 = pd[s][2] - (double)kk.z, d3 = pd[s][3] - (double)kk.w;
                                s0 = fma(d0, d0, s0), s1 = fma(d1, d1, s1), s2 = fma(d2, d2, s2), s3 = fma(d3, d3, s3);
                            }
                            tot[j] = (s0 + s1) + (s2 + s3);
                        }
                    }
    #pragma unroll
                    for (int j = 0; j < NC; ++j) {
                        if (j < n_cand) {  // uniform over the warp
                            double t = tot[j];
    #pragma unroll
                            for (int m = 1; m < L; m <<= 1) t += __shfl_xor_sync(0xffffffffu, t, m);
                            if (g == 0) sqbuf[r * NC + j] = t;
                        }
                    }
                }
                bar_workers();
                lap(8);
                // ---- P5b: one thread per (row, candidate), three at a time (f64 latency): the distance from the squared distance as
                // `poincare_distance` computes it (f64 log1p form of 2 asinh sqrt, rounded to f32). Item n_cand of a row is the
                // bound: every non-candidate has a true v of at least excl (1 - 4e-7: the f32 rounding of v itself), so its
                // distance is at least d(v_lb / (1 - |p|^2)); the selection is proven when its largest distance is strictly smaller.
                {
                    const int per_row = n_cand + 1, n_items = BM * per_row;
                    auto item_distance = [&](int t) {
                        const int r = t / per_row, j = t - r * per_row;
                        const bool bound = j == n_cand;
                        const double sq = bound ? (double)stat_excl[BM + r] * (1.0 - 4e-7) : sqbuf[r * NC + j];
                        const float ns = bound ? 0.0f : __ldg(p.norm_sq + cand_slot[r * kCandMax + j]);
                        return exact_distance(sq, 1.0 - (double)stat_qs[r], ns);
                    };
                    auto item_store = [&](int t, float d) {
                        const int r = t / per_row, j = t - r * per_row;
                        if (j == n_cand)
                            stat_dlb[r] = __float_as_uint(d);
                        else
                            d32[r * (NC + 1) + j] = d;
                    };
                    for (int t = wtid; t < n_items; t += 3 * 32 * kWorkWarps) {
                        // the last pass may compute an item twice (same value, same address)
                        const int ta = t, tb = min(t + 32 * kWorkWarps, n_items - 1), tc = min(t + 2 * 32 * kWorkWarps, n_items - 1);
                        const float da = item_distance(ta), db = item_distance(tb), dc = item_distance(tc);
                        item_store(ta, da), item_store(tb, db), item_store(tc, dc);
                    }
                }
                bar_workers();
                lap(9);
                // ---- P5c: one thread per row: selection by (distance bits, slot), the proof, softmax over the selected slots
                if (wtid < BM) {
                    const int r = wtid;
                    const size_t q = q0 + r;
                    int ok = 0;
                    if (q < p.rows) {
                        bool decisive = false;
                        if (stat_mark[r] != 0u) {
                            unsigned long long key[NC];
    #pragma unroll
                            for (int j = 0; j < NC; ++j)
                                key[j] = j < n_cand ? (((unsigned long long)__float_as_uint(d32[r * (NC + 1) + j]) << 32) | cand_slot[r * kCandMax + j]) : ~0ull;
                            unsigned kth = 0u, mn = 0xffffffffu;
                            unsigned selected = 0;  // bit j: candidate j is among the k smallest (bits, slot)
    #pragma unroll
                            for (int j = 0; j < NC; ++j) {
                                int rank = 0;
    #pragma unroll
                                for (int i = 0; i < NC; ++i) rank += key[i] < key[j] ? 1 : 0;
                                const unsigned bits = (unsigned)(key[j] >> 32);
                                if (j < n_cand && rank < k) selected |= 1u << j, kth = max(kth, bits);
                                if (j < n_cand) mn = min(mn, bits);
                            }
                            decisive = kth < stat_dlb[r];
                            if (p.selftest_every > 0 && q % (size_t)p.selftest_every == 0) decisive = false;
                            if (decisive) {
                                const float dmin = __uint_as_float(mn);
                                // ascending slot order (memory.rs:389-390), weights exp((min - d) / tau), their sum in that order
    #pragma unroll
                                for (int j = 0; j < NC; ++j) {
                                    if (!(selected >> j & 1u)) continue;
                                    const unsigned slot = (unsigned)key[j] & 0xffffu;
                                    int srank = 0;
    #pragma unroll
                                    for (int i = 0; i < NC; ++i) srank += ((selected >> i & 1u) && ((unsigned)key[i] & 0xffffu) < slot) ? 1 : 0;
                                    sels[r * NC + srank] = slot;
                                    selw[r * NC + srank] = expf(__fdiv_rn(__fsub_rn(dmin, __uint_as_float((unsigned)(key[j] >> 32))), p.tau));
                                }
                                float sum = 0.0f;
                                for (int j = 0; j < k; ++j) sum = __fadd_rn(sum, selw[r * NC + j]);
                                for (int j = 0; j < k; ++j) {
                                    const float wn = __fdiv_rn(selw[r * NC + j], sum);
                                    selw[r * NC + j] = wn;
                                    if (p.topk_slots) p.topk_slots[q * k + j] = sels[r * NC + j];
                                    if (p.topk_weights) p.topk_weights[q * k + j] = wn;
                                }
                                if (p.min_dist) p.min_dist[q] = dmin;
                                ok = 1;
                            }
                        }
                        if (!decisive) flag_rows[atomicAdd(flag_count, 1)] = r;  // the exact stage writes this row
                    }
                    row_ok[r] = ok;
                }
                bar_workers();
                lap(10);
                // ---- P5d: the value read of the proven rows
                read_selected_values<NC>(p.values, p.dv, p.m_val, p.m_bf16, p.weights, cap, k, q0, sels, selw, row_ok, wtid);
                // ---- P5e: the rows whose selection the candidates could not prove (or a list overflowed, or the test hook) are
                // recomputed over every slot. Rare, and uniform over the CTA (the count is shared); kept out of line so that it
                // costs the common path no registers.
                bar_workers();
                if (*flag_count > 0) {
                    const RetrieveParams pc = p;  // a local copy for the out-of-line call: the common path keeps reading the parameter bank
                    exact_rows<DK>(pc, q0, smem_a, stat_qs, flag_rows, *flag_count, fx_p, fx_dist, fx_slot, fx_w, wtid);
                }
                bar_workers();  // the lists and the operand are free for the next tile
                lap(11);
            }
        }
        if (p.phase_cycles && wtid == 0)
            for (int i = 0; i < kPhases; ++i) atomicAdd(p.phase_cycles + i, (unsigned long long)phase_clk[i]);
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

// dense weight rows -> (slots, weights) of the selected slots in ascending slot order; unused entries 0xffffffff / 0
__global__ void __launch_bounds__(256) compact_topk_kernel(const float* __restrict__ weights, int cap, int k, size_t rows,
                                                           unsigned* __restrict__ slots, float* __restrict__ w_out) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t q = (size_t)blockIdx.x * 8 + warp;
    if (q >= rows) return;
    const float* row = weights + q * cap;
    int base = 0;
    for (int s0 = 0; s0 < cap; s0 += 32) {
        const float w = s0 + lane < cap ? row[s0 + lane] : 0.0f;
        const unsigned ballot = __ballot_sync(0xffffffffu, w != 0.0f);
        const int pos = base + __popc(ballot & ((1u << lane) - 1u));
        if (w != 0.0f && pos < k) {
            if (slots) slots[q * k + pos] = (unsigned)(s0 + lane);
            if (w_out) w_out[q * k + pos] = w;
        }
        base += __popc(ballot);
    }
    for (int i = base + lane; i < k; i += 32) {
        if (slots) slots[q * k + i] = 0xffffffffu;
        if (w_out) w_out[q * k + i] = 0.0f;
    }
}

size_t fused_smem(int dk) {
    const size_t a = (size_t)3 * (dk / BK) * BM * BK * 2;
    // tail: per-slot constants, per-row statistics (|p|^2, two bounds, two counts, the proof distance, the flag),
    // candidate slots, barriers
    const size_t tail = 512 * sizeof(float2) + 512 * 4 + (1 + 2 + 2 + 1 + 1 + 1) * BM * 4 + BM * kCandMax * 2 + (2 * kStages + 2 + kPhases) * 8 + 16 + 16;
    return 1024 + a + (size_t)kStages * kRingStage + tail;
}

}  // namespace

bool retrieve_fused_eligible(const RetrieveParams& p) {
    const bool topk = p.top_k != 0 && p.top_k < p.count;
    const int n_cand = p.top_k + kMargin < kCandMax ? p.top_k + kMargin : kCandMax;
    return topk && p.top_k <= kCandMax - kMargin && (p.cap == 128 || p.cap == 256 || p.cap == 512) && (p.dk == 64 || p.dk == 128) &&
           p.count / 8 >= n_cand + 2 && p.k_split && p.k_stat && p.fixup_count && p.rows > 0 &&
           p.rows <= 0xffffffffull && p.dv > 0 && p.dv % 4 == 0 && (reinterpret_cast<uintptr_t>(p.values) & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(p.keys) & 15) == 0 &&
           (!p.m_val || (reinterpret_cast<uintptr_t>(p.m_val) & 15) == 0) && (!p.m_bf16 || (reinterpret_cast<uintptr_t>(p.m_bf16) & 7) == 0);
}

int32_t launch_retrieve_fused(pssa_b200_ctx* ctx, const RetrieveParams& p) {
    if (!retrieve_fused_eligible(p)) return fail(ctx, PSSA_B200_ERR_UNSUPPORTED, "B200 fused top-k read: shape not eligible");
    RetrieveParams q = p;
    q.status = ctx->status_dev;
    CUtensorMap map_b;
    int32_t rc;
    const int nh = p.cap >= 256 ? 256 : p.cap;
    if ((rc = make_map(ctx, &map_b, p.k_split, (size_t)p.cap, (size_t)3 * p.dk, nh))) return rc;
    PSSA_CUDA(ctx, cudaMemsetAsync(p.fixup_count, 0, sizeof(unsigned), ctx->stream));
    const size_t smem = fused_smem(p.dk);
    const long long tiles = (long long)((p.rows + BM - 1) / BM);
    const unsigned grid = (unsigned)(tiles < ctx->sm_count ? tiles : ctx->sm_count);
    static PerDeviceOnce attr[4];
    auto go = [&](auto kernel, int which) -> int32_t {
        if (attr[which].need(ctx->device)) {
            PSSA_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            attr[which].done(ctx->device);
        }
        PSSA_CUDA(ctx, launch_dependent(kernel, dim3(grid), dim3(kThreads), smem, ctx->stream, map_b, q));
        return PSSA_B200_OK;
    };
    const bool few = p.top_k + kMargin <= 9;  // the instantiation with nine candidate registers per thread
    if (p.dk == 64)
        rc = few ? go(retrieve_topk_fused_kernel<64, 9>, 0) : go(retrieve_topk_fused_kernel<64, kCandMax>, 1);
    else
        rc = few ? go(retrieve_topk_fused_kernel<128, 9>, 2) : go(retrieve_topk_fused_kernel<128, kCandMax>, 3);
    if (rc) return rc;
    return after_launch(ctx, "retrieve_topk_fused_kernel");
}

// The all-slots read of the fast modes as one kernel (projection, distances, softmax, bf16 weight rows): for callers
// that keep only the leading bf16 piece of every weight and multiply it themselves (the model's bf16 precision).
bool retrieve_all_fused_eligible(const RetrieveParams& p) {
    const bool topk = p.top_k != 0 && p.top_k < p.count;
    return !topk && !p.single_token && p.count > 0 && p.value_terms == 1 && p.skip_value_read && p.skip_weights && p.w_split && !p.min_dist &&
           (p.cap == 128 || p.cap == 256 || p.cap == 512) && (p.dk == 64 || p.dk == 128) && p.k_split && p.k_stat && p.rows > 0 &&
           p.rows <= 0xffffffffull && p.tau > 0.0f && (reinterpret_cast<uintptr_t>(p.w_split) & 15) == 0;
}

int32_t launch_retrieve_all_fused(pssa_b200_ctx* ctx, const RetrieveParams& p) {
    if (!retrieve_all_fused_eligible(p)) return fail(ctx, PSSA_B200_ERR_UNSUPPORTED, "B200 fused all-slots read: shape not eligible");
    RetrieveParams q = p;
    q.status = ctx->status_dev;
    CUtensorMap map_b;
    int32_t rc;
    const int nh = p.cap >= 256 ? 256 : p.cap;
    if ((rc = make_map(ctx, &map_b, p.k_split, (size_t)p.cap, (size_t)3 * p.dk, nh))) return rc;
    const size_t smem = fused_smem(p.dk);
    const long long tiles = (long long)((p.rows + BM - 1) / BM);
    const unsigned grid = (unsigned)(tiles < ctx->sm_count ? tiles : ctx->sm_count);
    static PerDeviceOnce attr[2];
    auto go = [&](auto kernel, int which) -> int32_t {
        if (attr[which].need(ctx->device)) {
            PSSA_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            attr[which].done(ctx->device);
        }
        PSSA_CUDA(ctx, launch_dependent(kernel, dim3(grid), dim3(kThreads), smem, ctx->stream, map_b, q));
        return PSSA_B200_OK;
    };
    rc = p.dk == 64 ? go(retrieve_topk_fused_kernel<64, 9, true>, 0) : go(retrieve_topk_fused_kernel<128, 9, true>, 1);
    if (rc) return rc;
    return after_launch(ctx, "retrieve_all_fused_kernel");
}

int32_t launch_compact_topk(pssa_b200_ctx* ctx, const float* weights, int cap, int k, size_t rows, unsigned* slots, float* w_out) {
    compact_topk_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, ctx->stream>>>(weights, cap, k, rows, slots, w_out);
    return after_launch(ctx, "compact_topk_kernel");
}

}  // namespace pssa
