// Exact top-k Poincare memory read in ONE kernel: projection, distances, selection, softmax and value read for a tile
// of 128 queries without the [rows, capacity] distance matrix ever leaving the SM.
//
// Replaces `retrieve_soft_into` with `top_k` set (src/memory.rs:344-408: f64 distances rounded to f32, the k smallest
// `(distance bits, slot)` pairs, weights and value read in ascending slot order) and, like the other read kernels, the
// reference GPU's one-thread-per-token `memory_forward` (src/cuda/stages.ptx:358-446).
//
// The idea: the tensor cores are a PRE-FILTER, the reference's f64 arithmetic decides.
//   1. worker warps project the tile's queries into the ball (f64, the reference's sequential sums: same bits) and write
//      the points as three bf16 pieces straight into the 128-byte-swizzled A operand in shared memory;
//   2. one thread issues tcgen05.mma for the six piece products above 2^-24 of p.k against the bank's keys (split the
//      same way once per upload, streamed by TMA through a 3-stage ring); the 128 x capacity accumulator fills the SM's
//      TMEM (512 fp32 columns);
//   3. one thread per query row reads its accumulator row twice with tcgen05.ld: a first sweep finds a threshold that at
//      least C = k + 4 slots pass (the C-th smallest of the minima of v = |p-k|^2 / (1-|k|^2) over groups of 32, 16 or 8
//      slots), a second sweep lists the slots under it (about 20 of 512); the C smallest of the list are the candidates;
//   4. one warp per row re-scores the candidates exactly as `poincare_distance` does (f64 differences and sum, f64
//      log1p form of 2 asinh sqrt, rounded to f32), selects k by (bits, slot) and proves the selection: the sweeps
//      also produced v_lb, the smallest (approximate v - its error bound) over every slot that did NOT become a candidate,
//      so the true distance of each of those is at least d(v_lb / (1-|p|^2)); if the k-th selected distance is strictly
//      below that, no other slot can enter or tie. Otherwise (or if the list overflowed) the row is flagged and a second,
//      tiny kernel recomputes that row with f64 distances to every slot. Rare: a few rows per million.
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

constexpr int kListCap = 48;   // slots a row can list under its threshold (about 20 expected)
constexpr int kCandMax = 16;   // candidates re-scored per row: top_k + kMargin, at most this many
constexpr int kMargin = 4;
constexpr int kWorkWarps = 8;  // warps 2..9; the first four own the 128 TMEM lanes (one query row per thread)
constexpr int kThreads = 64 + 32 * kWorkWarps;
constexpr int kStages = 3;
constexpr int kRingStage = 256 * BK * 2;  // one key k-block of up to 256 slots: 32 KB
// Error bound of the pre-filter's t = |p - k|^2 = (|p|^2 - p.k) + (|k|^2 - p.k): the tensor-core product p.k (six piece
// products, fp32 accumulation that is not correctly rounded) is off by at most kEpsDot * |p| |k| (about fifty accumulation
// steps of 2^-23 relative to sum |p_i k_i| <= |p| |k|; measured below 3.1e-6 |p| |k|, see the tensor-core distance test),
// and the two fp32 subtractions and the addition by kEpsSum * (|p|^2 + |k|^2).
constexpr float kEpsDot = 8e-6f;
constexpr float kEpsSum = 5e-7f;

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

// Last stage of a row, shared by the fused kernel and the exact fix-up: the k selected slots arrive in ASCENDING SLOT ORDER
// (sel_slot / sel_dist in shared memory); weights exp((min - d) / tau) summed in that order (memory.rs:391-398),
// normalised, value read in that order with separately rounded multiply and add (memory.rs:399-406). LANES threads of a
// warp work on one row (32: a warp per row; 16: two rows per warp, `hl` the lane within the half); every lane of the warp
// calls it, `active` says whether its row exists.
template <int LANES>
__device__ __forceinline__ void finish_row(const RetrieveParams& p, size_t q, const unsigned* sel_slot, float* sel_w, int k, float dmin,
                                           int hl, bool active) {
    const float tau = p.tau;
    const float my_w = (active && hl < k) ? expf(__fdiv_rn(__fsub_rn(dmin, sel_w[hl]), tau)) : 0.0f;  // sel_w holds distances on entry
    __syncwarp();
    if (active && hl < k) sel_w[hl] = my_w;
    __syncwarp();
    float sum = 0.0f;
    if (active)
        for (int j = 0; j < k; ++j) sum = __fadd_rn(sum, sel_w[j]);
    const float wn = active ? __fdiv_rn(my_w, sum) : 0.0f;
    __syncwarp();
    if (active && hl < k) sel_w[hl] = wn;
    __syncwarp();
    if (!active) return;  // no warp-wide operation below
    if (p.min_dist && hl == 0) p.min_dist[q] = dmin;
    if (p.topk_slots && hl < k) p.topk_slots[q * k + hl] = sel_slot[hl];
    if (p.topk_weights && hl < k) p.topk_weights[q * k + hl] = wn;
    if (p.weights) {  // the reference's dense row: zero except the selected slots; every address is written once, by the
                      // lane that owns it, so no ordering between a zero and a weight is needed
        float* row = p.weights + q * p.cap;
        for (int i = hl; i < p.cap; i += LANES) {
            float w = 0.0f;
            for (int j = 0; j < k; ++j) w = sel_slot[j] == (unsigned)i ? sel_w[j] : w;
            row[i] = w;
        }
    }
    const int dv = p.dv;
    for (int j0 = hl; j0 < dv; j0 += LANES * 4) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j < k; ++j) {
            const float wi = sel_w[j];
            const float* v = p.values + (size_t)sel_slot[j] * dv;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int c = j0 + e * LANES;
                if (c < dv) acc[e] = __fadd_rn(acc[e], __fmul_rn(wi, __ldg(v + c)));
            }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int c = j0 + e * LANES;
            if (c < dv) {
                if (p.m_val) p.m_val[q * dv + c] = acc[e];
                if (p.m_bf16) reinterpret_cast<__nv_bfloat16*>(p.m_bf16)[q * dv + c] = __float2bfloat16_rn(acc[e]);
            }
        }
    }
}

// lane base + j (j < n) holds (bits, slot): rank of this lane's pair among the n pairs by (bits, slot)
__device__ __forceinline__ int rank_by_key(unsigned long long key, int n, int base) {
    int rank = 0;
    for (int i = 0; i < n; ++i) rank += __shfl_sync(0xffffffffu, key, base + i) < key ? 1 : 0;
    return rank;
}

template <int DK>
__global__ void __launch_bounds__(kThreads, 1) retrieve_topk_fused_kernel(const __grid_constant__ CUtensorMap map_b, RetrieveParams p) {
    constexpr int KB_PIECE = DK / BK;        // k-blocks per bf16 piece
    constexpr int KB_A = 3 * KB_PIECE;       // k-blocks of the A operand (three pieces)
    constexpr uint32_t A_BLOCK = BM * BK * 2;  // 16 KB
    constexpr int PITCH = DK + 1;            // staging pitch in floats (bank spreading for one-thread-per-row walks)
    constexpr int EPL = DK / 16;             // key dimensions per lane in the re-scoring (16 lanes per row)
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* smem_a = smem;                         // [KB_A][128 x 64 bf16], swizzled
    unsigned char* ring = smem_a + KB_A * A_BLOCK;        // [kStages][<=256 x 64 bf16]; between tiles: staging, then the lists
    float* staging = reinterpret_cast<float*>(ring);      // [128][PITCH] raw queries, then the projected points
    float* list_v = reinterpret_cast<float*>(ring);       // [kListCap][128]
    unsigned short* list_s = reinterpret_cast<unsigned short*>(list_v + kListCap * BM);  // [kListCap][128]
    unsigned char* tail = ring + kStages * kRingStage;
    float2* kstat_s = reinterpret_cast<float2*>(tail);                     // [cap <= 512]
    float* stat_qs = reinterpret_cast<float*>(kstat_s + 512);              // [128] |p|^2
    float* stat_vc = stat_qs + BM;                                         // [128] lower bound of the true v of every non-candidate
    int* stat_cnt = reinterpret_cast<int*>(stat_vc + BM);                  // [128] listed slots (> kListCap: overflow)
    float* knorm_s = reinterpret_cast<float*>(stat_cnt + BM);              // [cap <= 512] |k|
    unsigned short* cand_slot = reinterpret_cast<unsigned short*>(knorm_s + 512);  // [128][kCandMax]
    unsigned* sel_slot_s = reinterpret_cast<unsigned*>(cand_slot + BM * kCandMax);  // [kWorkWarps][32]
    float* sel_w_s = reinterpret_cast<float*>(sel_slot_s + kWorkWarps * 32);        // [kWorkWarps][32]
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(sel_w_s + kWorkWarps * 32);
    uint64_t* empty_bar = full_bar + kStages;
    uint64_t* a_ready = empty_bar + kStages;
    uint64_t* acc_full = a_ready + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int dk = DK, cap = p.cap, count = p.count, k = p.top_k;
    const int nh = cap >= 256 ? 256 : cap;   // slots per MMA (N) and per TMA box
    const int halves = cap / nh;
    const int n_cand = min(k + kMargin, kCandMax);
    // columns per group minimum: 32 when that leaves enough fully occupied groups to bound n_cand slots (plus two to
    // keep the bound tight), else 16 or 8; smaller groups give a lower threshold and shorter lists but more insertions
    int group = 32;
    while (group > 8 && count / group < n_cand + 2) group >>= 1;
    const long long n_tiles = (long long)((p.rows + BM - 1) / BM);
    const uint32_t tmem_cols = (uint32_t)cap;  // 128, 256 or 512: a power of two >= 32

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&full_bar[s], 1), mbar_init(&empty_bar[s], 1);
        mbar_init(a_ready, 1);
        mbar_init(acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    for (int i = threadIdx.x; i < cap; i += kThreads) {
        const float2 ks = p.k_stat[i];
        kstat_s[i] = ks;
        knorm_s[i] = sqrtf(ks.x) * 1.0000002f;  // rounded up: it scales an error bound
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_trigger();
    pdl_wait();

    const unsigned char pair_a[6] = {0, 0, 1, 0, 1, 2}, pair_b[6] = {0, 1, 0, 2, 1, 0};
    const int n_kb = 6 * KB_PIECE;  // k-blocks per half

    if (warp == 0) {
        // ---------------- producer: key pieces through the ring, after the workers have released it for this tile
        if (lane == 0) {
            uint32_t g = 0, it = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
                if (!mbar_wait(a_ready, it & 1)) {
                    atomicExch(p.status, PSSA_B200_ERR_TIMEOUT);
                    break;
                }
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
                        const int pair = kb / KB_PIECE, within = kb % KB_PIECE;
                        tma_load_2d(ring + s * kRingStage, &map_b, &full_bar[s], (pair_b[pair] * KB_PIECE + within) * BK, h * nh);
                    }
            }
        }
    } else if (warp == 1) {
        // ---------------- issuer: 128 x nh x 16 MMAs into TMEM columns [h * nh, (h + 1) * nh)
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(BM, nh);
            uint32_t g = 0, it = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
                if (!mbar_wait(a_ready, it & 1)) {
                    atomicExch(p.status, PSSA_B200_ERR_TIMEOUT);
                    break;
                }
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
                        const int pair = kb / KB_PIECE, within = kb % KB_PIECE;
                        const uint64_t da = umma_desc_sw128(smem_u32(smem_a + (pair_a[pair] * KB_PIECE + within) * A_BLOCK));
                        const uint64_t db = umma_desc_sw128(smem_u32(ring + s * kRingStage));
#pragma unroll
                        for (int kk = 0; kk < BK / UMMA_K; ++kk)
                            tcgen05_mma_bf16(tmem_base + h * nh, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                        tcgen05_commit(&empty_bar[s]);
                    }
                tcgen05_commit(acc_full);  // all products of this tile are in TMEM (or abandoned)
            }
        }
    } else {
        // ---------------- workers
        const int wid = warp - 2;                 // 0..7
        const int wtid = threadIdx.x - 64;        // 0..255
        const bool row_warp = wid < 4;            // warps 2..5 own TMEM lane quadrants 2, 3, 0, 1
        const int my_row = (warp & 3) * 32 + lane;
        const bool vec_q = (((p.ldq ? p.ldq : (size_t)dk) & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.q) & 15) == 0);
        uint32_t it = 0;
        bool alive = true;
        long long clk[6] = {0, 0, 0, 0, 0, 0};
        for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
            const size_t q0 = (size_t)tile * BM;
            const size_t ldq = p.ldq ? p.ldq : (size_t)dk;
            long long t_prev = clock64();
            auto lap = [&](int i) {
                const long long now = clock64();
                clk[i] += now - t_prev, t_prev = now;
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
            // ---- P1: one thread per row projects it (memory.rs:198-211), in place
            if (wtid < BM) {
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
                const float v0 = staging[r * PITCH + c], v1 = staging[r * PITCH + c + 1];
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
            bar_workers();
            if (wtid == 0) mbar_arrive(a_ready);  // releases the ring to the producer and the operand to the issuer
            lap(2);
            // ---- P3: two sweeps over the accumulator row (row warps only)
            if (row_warp) {
                if (alive) {  // every lane waits (each needs the barrier's acquire); the verdict is made warp-uniform
                    const bool ok = mbar_wait(acc_full, it & 1);
                    alive = __all_sync(0xffffffffu, ok);
                    if (!alive && lane == 0) atomicExch(p.status, PSSA_B200_ERR_TIMEOUT);
                }
                tcgen05_fence_after();
                lap(3);  // waiting for the tensor cores
                const float qs = stat_qs[my_row];
                const float pn = sqrtf(qs) * 1.0000002f;
                float excl = CUDART_INF_F;  // smallest lower bound of the true v over the slots that do not become candidates
                const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
                float best[kCandMax];
#pragma unroll
                for (int i = 0; i < kCandMax; ++i) best[i] = CUDART_INF_F;
                int cnt = 0;
                float theta = CUDART_INF_F;
                for (int sweep = 0; sweep < 2 && alive; ++sweep) {
                    for (int c0 = 0; c0 < cap; c0 += 32) {
                        float acc[32];
                        tcgen05_ld_32x32(taddr + c0, acc);
                        float gmin = CUDART_INF_F;
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int col = c0 + j;
                            const float2 ks = kstat_s[col];
                            // |p - k|^2 = (|p|^2 - p.k) + (|k|^2 - p.k): nothing rounded at the size of the norms
                            float v = fmaxf(((qs - acc[j]) + (ks.x - acc[j])) * ks.y, 0.0f);
                            v = col < count ? v : CUDART_INF_F;
                            if (sweep == 0) {
                                gmin = fminf(gmin, v);
                                if (((j + 1) & (group - 1)) == 0) {  // end of a group: keep the kCandMax smallest group minima, sorted
                                    float x = gmin;
#pragma unroll
                                    for (int i = 0; i < kCandMax; ++i) {
                                        const float lo = fminf(best[i], x), hi = fmaxf(best[i], x);
                                        best[i] = lo, x = hi;
                                    }
                                    gmin = CUDART_INF_F;
                                }
                            } else if (v <= theta) {
                                if (cnt < kListCap) list_v[cnt * BM + my_row] = v, list_s[cnt * BM + my_row] = (unsigned short)col;
                                ++cnt;
                            } else {
                                // not listed: v minus its own error bound (both scaled by 1/(1-|k|^2))
                                const float err = fmaf(kEpsDot * pn, knorm_s[col], kEpsSum * (qs + ks.x));
                                excl = fminf(excl, fmaf(-err, ks.y, v));
                            }
                        }
                    }
                    if (sweep == 0) {
#pragma unroll
                        for (int i = 0; i < kCandMax; ++i)
                            if (i == n_cand - 1) theta = best[i];  // at least n_cand slots (one per group) lie at or under it
                    }
                }
                tcgen05_fence_before();
                // ---- P4: the n_cand smallest of the list by (v, slot), sorted
                unsigned long long top[kCandMax];
#pragma unroll
                for (int i = 0; i < kCandMax; ++i) top[i] = ~0ull;
                const int n_list = min(cnt, kListCap);
                for (int e = 0; e < n_list; ++e) {
                    unsigned long long x = ((unsigned long long)__float_as_uint(list_v[e * BM + my_row]) << 32) | list_s[e * BM + my_row];
#pragma unroll
                    for (int i = 0; i < kCandMax; ++i) {
                        if (i < n_cand) {  // entries past the candidates stay empty: what falls out of the first n_cand is excluded
                            const unsigned long long lo = umin64(top[i], x), hi = umax64(top[i], x);
                            top[i] = lo, x = hi;
                        }
                    }
                    if (x != ~0ull) {  // a listed slot that is not (or no longer) a candidate
                        const unsigned slot = (unsigned)(x & 0xffffu);
                        const float2 ks = kstat_s[slot];
                        const float err = fmaf(kEpsDot * pn, knorm_s[slot], kEpsSum * (qs + ks.x));
                        excl = fminf(excl, fmaf(-err, ks.y, __uint_as_float((unsigned)(x >> 32))));
                    }
                }
#pragma unroll
                for (int i = 0; i < kCandMax; ++i) cand_slot[my_row * kCandMax + i] = (unsigned short)(top[i] & 0xffffu);
                stat_vc[my_row] = excl;
                stat_cnt[my_row] = alive ? cnt : kListCap + 1;
            }
            bar_workers();
            lap(4);
            // ---- P5: half a warp per row (two rows per warp in flight): exact re-scoring, selection, proof, softmax, value read
            {
                const int half = lane >> 4, hl = lane & 15, base = lane & 16;
                unsigned* sel_slot = sel_slot_s + wid * 32 + half * 16;
                float* sel_w = sel_w_s + wid * 32 + half * 16;
                for (int rb = wid * 2; rb < BM; rb += kWorkWarps * 2) {
                    const int r = rb + half;
                    const size_t q = q0 + r;
                    const bool exists = q < p.rows;
                    // a list overflow (or an abandoned accumulator) leaves no candidates to trust
                    const bool trusted = exists && stat_cnt[r] <= kListCap;
                    // the projected point from its three pieces (their sum is exact); lane hl owns dimensions hl + 16 e
                    float pf[EPL];
#pragma unroll
                    for (int e = 0; e < EPL; ++e) {
                        const int c = hl + 16 * e;
                        const uint32_t off = sw128_offset(r, c % BK);
                        const int kb = c / BK;
                        const float x0 = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(smem_a + (0 * KB_PIECE + kb) * A_BLOCK + off));
                        const float x1 = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(smem_a + (1 * KB_PIECE + kb) * A_BLOCK + off));
                        const float x2 = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(smem_a + (2 * KB_PIECE + kb) * A_BLOCK + off));
                        pf[e] = x0 + (x1 + x2);
                    }
                    double part[kCandMax];
#pragma unroll
                    for (int j = 0; j < kCandMax; ++j) {
                        part[j] = 0.0;
                        if (j < n_cand && trusted) {
                            const float* krow = p.keys + (size_t)cand_slot[r * kCandMax + j] * dk;
#pragma unroll
                            for (int e = 0; e < EPL; ++e) {
                                const double df = (double)pf[e] - (double)__ldg(krow + hl + 16 * e);
                                part[j] = fma(df, df, part[j]);
                            }
                        }
                    }
                    // transpose-reduce over the 16 lanes of the half: after the four steps lane hl holds the full sum of candidate hl
#pragma unroll
                    for (int n = 8, mask = 8; n >= 1; n >>= 1, mask >>= 1) {
                        const bool upper = (lane & mask) != 0;
#pragma unroll
                        for (int i = 0; i < n; ++i) {
                            const double send = upper ? part[i] : part[i + n];
                            const double keep = upper ? part[i + n] : part[i];
                            part[i] = keep + __shfl_xor_sync(0xffffffffu, send, mask);
                        }
                    }
                    const double one_minus_q = 1.0 - (double)stat_qs[r];
                    const bool has = trusted && hl < n_cand;
                    float d_j = CUDART_INF_F;
                    unsigned slot_j = 0xffffu;
                    if (has) {
                        slot_j = cand_slot[r * kCandMax + hl];
                        d_j = exact_distance(part[0], one_minus_q, __ldg(p.norm_sq + slot_j));
                    }
                    const unsigned long long key = has ? (((unsigned long long)__float_as_uint(d_j) << 32) | slot_j) : ~0ull;
                    const int rank = rank_by_key(key, n_cand, base);
                    const bool selected = has && rank < k;
                    // the largest selected distance and the smallest of all, within the half
                    unsigned kth_bits = selected ? __float_as_uint(d_j) : 0u;
                    unsigned min_bits = has ? __float_as_uint(d_j) : 0xffffffffu;
#pragma unroll
                    for (int mk = 8; mk > 0; mk >>= 1) {
                        kth_bits = max(kth_bits, __shfl_xor_sync(0xffffffffu, kth_bits, mk));
                        min_bits = min(min_bits, __shfl_xor_sync(0xffffffffu, min_bits, mk));
                    }
                    // proof that no slot outside the candidate set can enter or tie
                    int decisive = 0;
                    if (hl == 0 && exists) {
                        if (trusted) {
                            // every slot outside the candidate set has a true v of at least this (1 - 4e-7: the f32 rounding of v itself)
                            const double v_lb = (double)stat_vc[r] * (1.0 - 4e-7);
                            if (v_lb > 0.0) {
                                const double u_lb = v_lb / one_minus_q;
                                const float d_lb = (float)log1p(2.0 * u_lb + 2.0 * sqrt(fma(u_lb, u_lb, u_lb)));
                                decisive = kth_bits < __float_as_uint(d_lb);
                            }
                            if (p.selftest_every > 0 && q % (size_t)p.selftest_every == 0) decisive = 0;
                        }
                        if (!decisive) p.fixup_list[atomicAdd(p.fixup_count, 1u)] = (unsigned)q;  // the exact pass writes this row
                    }
                    decisive = __shfl_sync(0xffffffffu, decisive, base);
                    // ascending slot order among the selected
                    int srank = 0;
                    for (int i = 0; i < n_cand; ++i) {
                        const unsigned other_slot = __shfl_sync(0xffffffffu, slot_j, base + i);
                        const bool other_sel = __shfl_sync(0xffffffffu, selected ? 1 : 0, base + i) != 0;
                        srank += (other_sel && other_slot < slot_j) ? 1 : 0;
                    }
                    __syncwarp();
                    if (selected && decisive) sel_slot[srank] = slot_j, sel_w[srank] = d_j;
                    __syncwarp();
                    finish_row<16>(p, q, sel_slot, sel_w, k, __uint_as_float(min_bits), hl, decisive != 0);
                    __syncwarp();
                }
            }
            bar_workers();  // the lists and the operand are free for the next tile
            lap(5);
        }
        if (p.phase_cycles && wtid == 0)
            for (int i = 0; i < 6; ++i) atomicAdd(p.phase_cycles + i, (unsigned long long)clk[i]);
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

// Exact pass for the rows the fused kernel could not prove (or was told to hand over): one warp per flagged row, f64
// distances to every occupied slot, k rounds of a warp-wide minimum over (distance bits, slot).
__global__ void __launch_bounds__(256) retrieve_topk_fixup_kernel(RetrieveParams p) {
    __shared__ float ps[8][256];
    __shared__ float dist[8][512];
    __shared__ unsigned sel_slot_s[8][32];
    __shared__ float sel_w_s[8][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int dk = p.dk, count = p.count, k = p.top_k;
    const size_t ldq = p.ldq ? p.ldq : (size_t)dk;
    const unsigned n_rows = *p.fixup_count;
    for (unsigned item = blockIdx.x * 8 + warp; item < n_rows; item += gridDim.x * 8) {
    const size_t q = p.fixup_list[item];
    __syncwarp();
    for (int i = lane; i < dk; i += 32) ps[warp][i] = p.q[q * ldq + i];
    __syncwarp();
    float qs = 0.0f;
    if (lane == 0) qs = project_row(ps[warp], dk, p.q_is_euclidean != 0, nullptr);
    qs = __shfl_sync(0xffffffffu, qs, 0);
    __syncwarp();
    const double one_minus_q = 1.0 - (double)qs;
    for (int s = lane; s < count; s += 32) {
        const float* krow = p.keys + (size_t)s * dk;
        double sq = 0.0;
        for (int i = 0; i < dk; ++i) {
            const double df = (double)ps[warp][i] - (double)__ldg(krow + i);
            sq = fma(df, df, sq);
        }
        dist[warp][s] = exact_distance(sq, one_minus_q, __ldg(p.norm_sq + s));
    }
    __syncwarp();
    unsigned my_slot = 0xffffffffu;
    float my_dist = 0.0f, dmin = 0.0f;
    for (int r = 0; r < k; ++r) {
        unsigned long long local = ~0ull;
        for (int s = lane; s < count; s += 32) {
            const unsigned bits = __float_as_uint(dist[warp][s]);
            if (bits & 0x80000000u) continue;  // taken (distances are >= +0)
            local = umin64(local, ((unsigned long long)bits << 32) | (unsigned)s);
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) local = umin64(local, __shfl_xor_sync(0xffffffffu, local, m));
        const unsigned slot = (unsigned)(local & 0xffffffffu);
        const float d = __uint_as_float((unsigned)(local >> 32));
        if (lane == 0) dist[warp][slot] = __uint_as_float(__float_as_uint(d) | 0x80000000u);
        if (lane == r) my_slot = slot, my_dist = d;
        if (r == 0) dmin = d;
        __syncwarp();
    }
    int srank = 0;
    for (int i = 0; i < k; ++i) srank += __shfl_sync(0xffffffffu, my_slot, i) < my_slot ? 1 : 0;
    if (lane < k) sel_slot_s[warp][srank] = my_slot, sel_w_s[warp][srank] = my_dist;
    __syncwarp();
    finish_row<32>(p, q, sel_slot_s[warp], sel_w_s[warp], k, dmin, lane, true);
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
    const size_t tail = 512 * sizeof(float2) + 3 * BM * 4 + 512 * 4 + BM * kCandMax * 2 + 2 * kWorkWarps * 32 * 4 + (2 * kStages + 2) * 8 + 16;
    return 1024 + a + (size_t)kStages * kRingStage + tail;
}

}  // namespace

bool retrieve_fused_eligible(const RetrieveParams& p) {
    const bool topk = p.top_k != 0 && p.top_k < p.count;
    const int n_cand = p.top_k + kMargin < kCandMax ? p.top_k + kMargin : kCandMax;
    return topk && p.top_k <= kCandMax - kMargin && (p.cap == 128 || p.cap == 256 || p.cap == 512) && (p.dk == 64 || p.dk == 128) &&
           p.count / 8 >= n_cand + 2 && p.k_split && p.k_stat && p.fixup_list && p.fixup_count && p.rows > 0 &&
           p.rows <= 0xffffffffull && p.dv > 0;
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
    static PerDeviceOnce attr[2];
    if (p.dk == 64) {
        if (attr[0].need(ctx->device)) {
            PSSA_CUDA(ctx, cudaFuncSetAttribute(retrieve_topk_fused_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            attr[0].done(ctx->device);
        }
        PSSA_CUDA(ctx, launch_dependent(retrieve_topk_fused_kernel<64>, dim3(grid), dim3(kThreads), smem, ctx->stream, map_b, q));
    } else {
        if (attr[1].need(ctx->device)) {
            PSSA_CUDA(ctx, cudaFuncSetAttribute(retrieve_topk_fused_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            attr[1].done(ctx->device);
        }
        PSSA_CUDA(ctx, launch_dependent(retrieve_topk_fused_kernel<128>, dim3(grid), dim3(kThreads), smem, ctx->stream, map_b, q));
    }
    if ((rc = after_launch(ctx, "retrieve_topk_fused_kernel"))) return rc;
    // the rows the fused kernel handed over (their count is only known on the device): a fixed small grid walks the list
    retrieve_topk_fixup_kernel<<<(unsigned)ctx->sm_count, 256, 0, ctx->stream>>>(q);
    return after_launch(ctx, "retrieve_topk_fixup_kernel");
}

int32_t launch_compact_topk(pssa_b200_ctx* ctx, const float* weights, int cap, int k, size_t rows, unsigned* slots, float* w_out) {
    compact_topk_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, ctx->stream>>>(weights, cap, k, rows, slots, w_out);
    return after_launch(ctx, "compact_topk_kernel");
}

}  // namespace pssa
