// bf16 tensor-core product for the projections: OUT[M, N] = epilogue(A[M, K] * B[N, K]^T), fp32 accumulate.
//
// Replaces the reference's cuBLAS SGEMM calls for W_delta, W_B, W_C, W_qx, W_qh, W_gate, W_proj, adapter
// down, MLP W1/W2 and the vocabulary head (src/cuda.rs:287-320, src/cuda/stages.rs:183-208) and the
// elementwise kernels that follow them (softplus / sigmoid / sigmoid_mul / add, src/cuda/stages.ptx:541-607),
// which become the epilogue.
//
// Blackwell data path, one persistent CTA per SM walking 128 x BN output tiles (BN = 64, 128 or 256):
//   warp 0   producer: TMA (cp.async.bulk.tensor.2d) loads of 128x64 / BNx64 bf16 boxes, 128-byte swizzle,
//            into a 3- or 4-stage shared-memory ring; completion on per-stage "full" mbarriers.
//   warp 1   issuer: one thread issues tcgen05.mma (cta_group::1, kind::f16, M 128, N BN, K 16) from shared-
//            memory descriptors into one of two TMEM accumulators of BN fp32 columns; tcgen05.commit releases
//            each ring stage ("empty" mbarrier) and finally signals "accumulator full".
//   warps 2-9 epilogue: tcgen05.ld (32 lanes x 32 columns per warp) -> activation -> transpose in shared
//            memory -> whole-line global stores (fp32 and/or bf16); the accumulator is handed back ("accumulator empty") as soon as it is in registers,
//            so the next tile's MMAs overlap this tile's epilogue.
// Both operands are K-major (row-major [rows, K]), so X * W^T needs no transpose anywhere.
// Every mbarrier wait is bounded: on expiry the kernel records PSSA_B200_ERR_TIMEOUT in the context's
// status word, stops issuing work, and still frees its TMEM.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdlib>
#include <cuda_runtime.h>

#include "bounds.hpp"
#include "context.hpp"
#include "device_math.cuh"
#include "kernels.hpp"
#include "tcgen05.cuh"

namespace pssa {
namespace {

using namespace tc;  // BM, BK, UMMA_K, the PTX wrappers and the tensor-map encoder (tcgen05.cuh)
constexpr int EPI_WARPS = 8;  // two warps per TMEM lane quadrant, each draining half of the tile's columns
// Epilogue warps of the 3-stage 128 x 256 products of the block schedule. Sixteen (four per TMEM lane quadrant, 96
// registers per thread) were measured: the products with light epilogues kept their times, the ones that prefetch two
// fp32 inputs spilled and lost 60 %, so the epilogue is not short of warps and eight stay.
constexpr int kWideEpiWarps = EPI_WARPS;
constexpr int STG_PITCH = 32;  // floats per staged row; 16-byte column quads are XOR-swizzled with the row (no padding, so four
                               // 48 KB operand stages fit beside the staging tiles of a 128 x 256 product)

struct GemmEpilogue {
    float* out;            // fp32 [M, ldo] or null
    __nv_bfloat16* out16;  // bf16 [M, ld16] or null
    size_t ldo, ld16;
    int M, N, K;
    int epi;               // Epilogue, or -1 for the column-range table below
    float alpha;
    int c1, c2, c3;        // table: [0,c1) softplus, [c1,c2) none, [c2,c3) sigmoid, [c3,N) silu
    int* status;
    // Split-precision product: A = [A_0 | A_1 | A_2] and B = [B_0 | B_1 | B_2] hold bf16 pieces of fp32 operands
    // (x = x_0 + x_1 + x_2), each piece seg_kb k-blocks wide; the kernel accumulates the listed (A piece, B piece)
    // products into one fp32 accumulator. n_pairs == 0: plain product over K.
    int n_pairs, seg_kb;
    unsigned char pair_a[6], pair_b[6];
    // EPI_RESIDUAL: out = res_in ? res_in + res_scale * (acc + add_in) : acc + add_in   (MLP residual + depth residual)
    const float* add_in;
    const float* res_in;
    size_t ld_add, ld_res;
    float res_scale;
    int add_is_bf16;       // EPI_RESIDUAL: add_in points at bf16 values (row pitch ld_add in elements)
    const float* row_scale;  // EPI_GATE: optional [M] factor on the accumulator's rows (an operand whose rows are not yet
                             // normalised: softmax weights before the division by their sum); null = 1
    // EPI_POINCARE: the accumulator is the inner product p.k of a point in the ball (row) and a bank key (column);
    // row_stat[row] = (|p|^2, 1/(1-|p|^2)), col_stat[col] = (|k|^2, 1/(1-|k|^2)); out = d(p, k)
    const float2* row_stat;
    const float2* col_stat;
    // column-range table only: the last range [c3, N) is also stored as bf16 at column (col - c3) of two side buffers
    // (the adapter activations, which ride as extra K columns of both MLP products); null = not wanted
    __nv_bfloat16* side_a;
    __nv_bfloat16* side_b;
    size_t ld_side_a, ld_side_b;
};

// softplus for the bf16 path (operands already carry 2^-9 relative rounding): x > 20 -> x; x < -4 -> the two-term
// series e^x (1 - e^x / 2) (relative error < e^2x / 3 < 1.2e-4); otherwise log(1 + e^x) with the fast intrinsics
__device__ __forceinline__ float fast_softplus(float x) {
    float ex = __expf(x);
    float mid = __logf(1.0f + ex);
    float low = ex * fmaf(-0.5f, ex, 1.0f);
    return x > 20.0f ? x : (x < -4.0f ? low : mid);
}

__device__ __forceinline__ float fast_epilogue(const GemmEpilogue& e, float acc, int col, float prev) {
    int epi = e.epi;
    if (epi < 0) epi = col < e.c1 ? EPI_SOFTPLUS : col < e.c2 ? EPI_NONE : col < e.c3 ? EPI_SIGMOID : EPI_SILU;
    switch (epi) {
        case EPI_SOFTPLUS: return fast_softplus(acc);
        case EPI_SIGMOID: return 1.0f / (1.0f + __expf(-acc));
        case EPI_SILU: return acc / (1.0f + __expf(-acc));
        case EPI_SCALE: return acc * e.alpha;
        case EPI_ADD_OUT: return prev + acc;
        default: return acc;
    }
}

__device__ __forceinline__ int col_kind(const GemmEpilogue& e, int col) {
    return col < e.c1 ? EPI_SOFTPLUS : col < e.c2 ? EPI_NONE : col < e.c3 ? EPI_SIGMOID : EPI_SILU;
}

// Persistent kernel: CTA c processes tiles c, c + gridDim.x, ... ; tile index -> (m, n) with n fastest, so the
// CTAs running at the same time share A row blocks through L2 and A is read from HBM once. Two TMEM accumulators
// let the epilogue of tile i run while the tensor cores work on tile i + 1.
// MODE fixes the epilogue family at compile time (kRuntimeMode: read it from the launch parameters). The epilogue's
// element loops are unrolled 32 wide, so every family it has to carry costs kilobytes of code in each instantiation and
// the epilogue warps stall on instruction fetch; the products of the model's block schedule get their own instantiations.
constexpr int kRuntimeMode = -100;
// OUTS fixes which outputs exist: 0 = read the pointers at run time, 1 = fp32 only, 2 = bf16 only.
// EW epilogue warps: EW / 4 per TMEM lane quadrant, each draining BN / (EW / 4) of the tile's columns.
// PAIR: the kernel runs as clusters of two CTAs on 256 x BN tiles (cta_group::2): each CTA keeps its own 128 rows of A,
// loads only its half of the B tile (32 KB instead of 48 KB per K block and CTA at BN = 256) and drains its own 128
// accumulator rows; the even CTA issues the MMAs for both and its barriers count both CTAs' operand bytes.
template <int BN, int STAGES, int MODE, int OUTS, int EW, bool PAIR>
__global__ void __launch_bounds__(64 + 32 * EW, 1) gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                            const __grid_constant__ CUtensorMap map_b,
                                                                            GemmEpilogue e) {
    constexpr int B_ROWS = PAIR ? BN / 2 : BN;  // rows of B (output columns) this CTA loads per K block
    constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = B_ROWS * BK * 2;
    constexpr uint32_t TMEM_COLS = 2 * BN;  // 128, 256 or 512: a power of two >= 32
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // 1024-byte alignment is required by the 128-byte swizzle
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* smem_a = smem;
    unsigned char* smem_b = smem + STAGES * A_BYTES;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem_b + STAGES * B_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_full = empty_bar + STAGES;   // [2] accumulator written by the tensor cores
    uint64_t* acc_empty = acc_full + 2;        // [2] accumulator drained by the epilogue warps
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    float* stage = reinterpret_cast<float*>(tmem_slot + 4);  // [EW][32 rows][STG_PITCH]
    float* const out32 = OUTS == 2 ? nullptr : e.out;
    __nv_bfloat16* const out16 = OUTS == 1 ? nullptr : e.out16;
    const bool vec32 = out32 && (e.ldo % 4 == 0) && ((reinterpret_cast<uintptr_t>(out32) & 15) == 0);
    const int epi = MODE == kRuntimeMode ? e.epi : MODE;  // a compile-time constant in the specialised instantiations
    const bool vec_res = (epi == EPI_RESIDUAL || epi == EPI_GATE) && e.ld_add % 4 == 0 && ((reinterpret_cast<uintptr_t>(e.add_in) & (e.add_is_bf16 ? 7 : 15)) == 0) &&
                         (!e.res_in || (e.ld_res % 4 == 0 && ((reinterpret_cast<uintptr_t>(e.res_in) & 15) == 0)));
    const bool vec16 = out16 && (e.ld16 % 4 == 0) && ((reinterpret_cast<uintptr_t>(out16) & 7) == 0);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = e.n_pairs > 0 ? e.n_pairs * e.seg_kb : (e.K + BK - 1) / BK;
    const int n_tiles = (e.N + BN - 1) / BN;
    constexpr int TILE_M = PAIR ? 2 * BM : BM;  // rows of one scheduled tile
    const int m_tiles = (e.M + TILE_M - 1) / TILE_M;
    const long long total_tiles = (long long)n_tiles * m_tiles;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;               // 0: the CTA that issues the MMAs
    const long long first_tile = PAIR ? (blockIdx.x >> 1) : blockIdx.x;  // both CTAs of a pair walk the same tiles
    const long long tile_step = PAIR ? (gridDim.x >> 1) : gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], PAIR ? 2 * EW : EW);  // one arrival per epilogue warp (of both CTAs of a pair)
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // TMEM allocation is a warp-wide operation (for a pair: the same warp of both CTAs, same slot)
        if (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync();  // the peer's barriers are initialised before anything of this CTA can signal them
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // everything above touched only this CTA's shared memory and TMEM; from here on the kernel reads what its
    // predecessor in the stream wrote, so a dependent launch waits for that predecessor here
    pdl_trigger();
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;  // k-block counter across all tiles of this CTA
            bool ok = true;
            const uint32_t leader_full = PAIR ? mapa_shared(smem_u32(full_bar), 0) : 0u;  // the even CTA's full barriers
            for (long long tile = first_tile; tile < total_tiles && ok; tile += tile_step) {
                const int m0 = (int)(tile / n_tiles) * TILE_M + (int)rank * BM, n0 = (int)(tile % n_tiles) * BN + (int)rank * B_ROWS;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t round = it / STAGES;
                    if (round > 0 && !mbar_wait(&empty_bar[s], (round - 1) & 1)) {
                        atomicExch(e.status, PSSA_B200_ERR_TIMEOUT);
                        ok = false;
                        break;
                    }
                    if (!PAIR)
                        mbar_expect_tx(&full_bar[s], A_BYTES + B_BYTES);
                    else if (rank == 0)
                        mbar_expect_tx(&full_bar[s], 2 * (A_BYTES + B_BYTES));  // this CTA's bytes and the peer's
                    int ka = kb, kbb = kb;
                    if (e.n_pairs > 0) {
                        const int pair = kb / e.seg_kb, within = kb % e.seg_kb;
                        ka = e.pair_a[pair] * e.seg_kb + within;
                        kbb = e.pair_b[pair] * e.seg_kb + within;
                    }
                    if (PAIR) {
                        tma_load_2d_pair(smem_a + s * A_BYTES, &map_a, leader_full + s * 8, ka * BK, m0);
                        tma_load_2d_pair(smem_b + s * B_BYTES, &map_b, leader_full + s * 8, kbb * BK, n0);
                    } else {
                        tma_load_2d(smem_a + s * A_BYTES, &map_a, &full_bar[s], ka * BK, m0);
                        tma_load_2d(smem_b + s * B_BYTES, &map_b, &full_bar[s], kbb * BK, n0);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(TILE_M, BN);
            uint32_t it = 0, t = 0;
            bool ok = true;
            for (long long tile = first_tile; tile < total_tiles && ok; tile += tile_step, ++t) {
                const uint32_t buf = t & 1, use = t >> 1;
                if (use > 0 && !mbar_wait(&acc_empty[buf], (use - 1) & 1)) {
                    atomicExch(e.status, PSSA_B200_ERR_TIMEOUT);
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&full_bar[s], (it / STAGES) & 1)) {
                        atomicExch(e.status, PSSA_B200_ERR_TIMEOUT);
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint64_t da = umma_desc_sw128(smem_u32(smem_a + s * A_BYTES));
                    const uint64_t db = umma_desc_sw128(smem_u32(smem_b + s * B_BYTES));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // advance 32 bytes (16 bf16) inside the swizzle atom: +2 in 16-byte units
                        if (PAIR)
                            tcgen05_mma_bf16_pair(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                        else
                            tcgen05_mma_bf16(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    // stage reusable once these MMAs have read it (in both CTAs of a pair)
                    if (PAIR) tcgen05_commit_pair(&empty_bar[s]); else tcgen05_commit(&empty_bar[s]);
                }
                // accumulator complete (or abandoned)
                if (PAIR) tcgen05_commit_pair(&acc_full[buf]); else tcgen05_commit(&acc_full[buf]);
            }
        }
    } else {
        // epilogue warps 2..EW+1: TMEM lane quadrant = warp % 4 (a hardware rule), column part = (warp - 2) / 4
        const int quad = warp & 3;
        const int half = (warp - 2) >> 2;
        constexpr int HALF_COLS = BN / (EW / 4);
        static_assert(EW % 4 == 0 && HALF_COLS % 32 == 0, "every epilogue warp drains whole 32-column chunks");
        float* stg = stage + (warp - 2) * (32 * STG_PITCH);
        const int cq = (lane & 7) * 4;   // column quad this lane stores after the transpose
        const int rsub = lane >> 3;      // row within each group of 4 rows
        uint32_t t = 0;
        const uint32_t leader_acc_empty = PAIR ? mapa_shared(smem_u32(acc_empty), 0) : 0u;
        for (long long tile = first_tile; tile < total_tiles; tile += tile_step, ++t) {
            const int m0 = (int)(tile / n_tiles) * TILE_M + (int)rank * BM, n0 = (int)(tile % n_tiles) * BN + half * HALF_COLS;
            const uint32_t buf = t & 1, use = t >> 1;
            const bool ready = mbar_wait(&acc_full[buf], use & 1);
            if (!ready) {
                if (lane == 0) atomicExch(e.status, PSSA_B200_ERR_TIMEOUT);
                break;
            }
            tcgen05_fence_after();
            const uint32_t taddr = tmem_base + buf * BN + half * HALF_COLS + ((uint32_t)(quad * 32) << 16);
            const int rbase = m0 + quad * 32;
            const bool rows_in = rbase + 32 <= e.M;  // whole 32-row band inside the matrix
            bool released = false;
            // EPI_GATE with row factors: the eight rows a lane stores are the same for every chunk of the tile
            // (kept in registers by the instantiation that carries only this family; the run-time one loads them where used)
            constexpr bool kHoistRowFactors = MODE == EPI_GATE;
            float row_f[kHoistRowFactors ? 8 : 1];
            if constexpr (kHoistRowFactors) {
#pragma unroll
                for (int i = 0; i < 8; ++i) row_f[i] = e.row_scale ? __ldg(e.row_scale + min(rbase + rsub + i * 4, e.M - 1)) : 1.0f;
            }
#pragma unroll 1
            for (int c0 = 0; c0 < HALF_COLS; c0 += 32) {
                const int col0 = n0 + c0;
                // Chunks that lie inside the matrix take the 16-byte path without per-element bounds checks; so does the
                // matrix's last, partial chunk when N is a multiple of 4 (a lane's column quad is then all in or all out)
                const bool interior = rows_in && (col0 + 32 <= e.N || (e.N & 3) == 0);
                const bool lane_in = col0 + (lane & 7) * 4 + 4 <= e.N;
                // EPI_RESIDUAL reads two more fp32 arrays with the output's access pattern: issue those loads first so
                // they are in flight during the TMEM load and the transpose
                float4 pre_add[8], pre_res[8];
                uint2 raw_add[8];
                const bool two_in = epi == EPI_RESIDUAL || epi == EPI_GATE;
                const bool prefetch = two_in && interior && vec_res;
                if (prefetch) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        if (!lane_in) break;
                        const size_t ro = (size_t)(rbase + rsub + i * 4);
                        if (epi == EPI_RESIDUAL && e.add_is_bf16)
                            // kept as raw bits: converting here would wait for the load before the TMEM read is issued
                            raw_add[i] = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(e.add_in) +
                                                                         ro * e.ld_add + col0 + cq);
                        else
                            pre_add[i] = *reinterpret_cast<const float4*>(e.add_in + ro * e.ld_add + col0 + cq);
                        pre_res[i] = e.res_in ? *reinterpret_cast<const float4*>(e.res_in + ro * e.ld_res + col0 + cq)
                                              : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                } else if (epi == EPI_ADD_OUT && interior && out32 && vec32) {
                    // the rows this chunk adds to, requested before the TMEM load instead of one dependent round trip
                    // per row group inside the store loop
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        if (lane_in) pre_add[i] = *reinterpret_cast<const float4*>(out32 + (size_t)(rbase + rsub + i * 4) * e.ldo + col0 + cq);
                }
                float v[32];
                if (col0 < e.N) tcgen05_ld_32x32(taddr + (uint32_t)c0, v);  // warp-uniform
                if (!released && (c0 + 32 >= HALF_COLS || col0 + 32 >= e.N)) {
                    // this warp's last chunk of the accumulator is in registers: hand its share of the buffer back
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (PAIR) mbar_arrive_cluster(leader_acc_empty + buf * 8); else mbar_arrive(&acc_empty[buf]);
                    }
                    released = true;
                }
                if (col0 >= e.N) break;
                // One activation kind per 32-column chunk keeps the element loop free of branches (a per-element
                // switch made the instruction stream jump between kilobytes of unrolled code and stalled on
                // instruction fetch). The column table's boundaries are multiples of 32 for every model shape;
                // a chunk that straddles one is activated element by element after the transpose (kind == -1).
                int kind = epi;
                if (kind < 0) {
                    const int first = col_kind(e, col0), last = col_kind(e, min(col0 + 31, e.N - 1));
                    kind = first == last ? first : -1;
                }
                switch (kind) {
                    case EPI_SOFTPLUS:
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = fast_softplus(v[j]);
                        break;
                    case EPI_SIGMOID:
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __fdividef(1.0f, 1.0f + __expf(-v[j]));
                        break;
                    case EPI_SILU:
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __fdividef(v[j], 1.0f + __expf(-v[j]));
                        break;
                    case EPI_SCALE:
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] *= e.alpha;
                        break;
                    case EPI_POINCARE: {
                        // |p - k|^2 = |p|^2 + |k|^2 - 2 p.k, then u = |p - k|^2 / ((1-|p|^2)(1-|k|^2)) (src/memory.rs:245-262);
                        // this thread's row is one query, the column statistics are warp-wide broadcast loads
                        const float2 rs = __ldg(e.row_stat + min(rbase + lane, e.M - 1));
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float2 cs = __ldg(e.col_stat + min(col0 + j, e.N - 1));
                            // two differences first: both are exact when the points nearly coincide (|p|^2, |k|^2 and p.k
                            // within a factor of two of each other), so no rounding happens at the magnitude of the norms
                            const float sq = fmaxf((rs.x - v[j]) + (cs.x - v[j]), 0.0f);
                            v[j] = fast_poincare_distance(sq * (rs.y * cs.y));
                        }
                        break;
                    }
                    default:
                        break;  // EPI_NONE, EPI_ADD_OUT (added after the transpose)
                }
                // transpose through a warp-private shared-memory tile: global stores become whole 128-byte lines
                // (8 lanes per output row) instead of 32 scattered 16-byte pieces per instruction
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<float4*>(stg + lane * STG_PITCH + (((j >> 2) ^ (lane & 7)) << 2)) =
                        make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                __syncwarp();
                const int gcol = col0 + cq;
                if (interior && kind != -1 && (!out32 || vec32) && (!out16 || vec16) && (!two_in || vec_res)) {
                    float* gp = out32 ? out32 + (size_t)(rbase + rsub) * e.ldo + gcol : nullptr;
                    __nv_bfloat16* bp = out16 ? out16 + (size_t)(rbase + rsub) * e.ld16 + gcol : nullptr;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int sr = i * 4 + rsub;  // staged row; its column quads are swizzled with (row & 7)
                        float4 val = *reinterpret_cast<const float4*>(stg + sr * STG_PITCH + ((((cq >> 2) ^ (sr & 7))) << 2));
                        if (!lane_in) break;
                        {
                            if (epi == EPI_ADD_OUT && gp) {
                                const float4 pv = pre_add[i];
                                val.x += pv.x, val.y += pv.y, val.z += pv.z, val.w += pv.w;
                            } else if (epi == EPI_RESIDUAL) {
                                float4 av = pre_add[i];
                                if (e.add_is_bf16) {
                                    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw_add[i].x));
                                    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw_add[i].y));
                                    av = make_float4(lo.x, lo.y, hi.x, hi.y);
                                }
                                val.x += av.x, val.y += av.y, val.z += av.z, val.w += av.w;
                                if (e.res_in) {
                                    const float4 rv = pre_res[i];
                                    val.x = fmaf(e.res_scale, val.x, rv.x), val.y = fmaf(e.res_scale, val.y, rv.y);
                                    val.z = fmaf(e.res_scale, val.z, rv.z), val.w = fmaf(e.res_scale, val.w, rv.w);
                                }
                            } else if (epi == EPI_GATE) {
                                const float4 av = pre_add[i];
                                float4 gv = pre_res[i];
                                const float rf = kHoistRowFactors ? row_f[kHoistRowFactors ? i : 0]
                                                                  : (e.row_scale ? __ldg(e.row_scale + rbase + rsub + i * 4) : 1.0f);
                                gv.x *= rf, gv.y *= rf, gv.z *= rf, gv.w *= rf;
                                val.x = fmaf(gv.x, val.x, av.x * e.alpha), val.y = fmaf(gv.y, val.y, av.y * e.alpha);
                                val.z = fmaf(gv.z, val.z, av.z * e.alpha), val.w = fmaf(gv.w, val.w, av.w * e.alpha);
                            }
                        }
                        if (gp) *reinterpret_cast<float4*>(gp + (size_t)i * 4 * e.ldo) = val;
                        if (epi < 0 && e.side_a && gcol >= e.c3) {
                            __nv_bfloat162 p0 = __floats2bfloat162_rn(val.x, val.y), p1 = __floats2bfloat162_rn(val.z, val.w);
                            uint2 pk;
                            pk.x = *reinterpret_cast<uint32_t*>(&p0), pk.y = *reinterpret_cast<uint32_t*>(&p1);
                            const size_t srow = (size_t)(rbase + rsub + i * 4);
                            *reinterpret_cast<uint2*>(e.side_a + srow * e.ld_side_a + (gcol - e.c3)) = pk;
                            *reinterpret_cast<uint2*>(e.side_b + srow * e.ld_side_b + (gcol - e.c3)) = pk;
                        }
                        if (bp) {
                            __nv_bfloat162 p0 = __floats2bfloat162_rn(val.x, val.y), p1 = __floats2bfloat162_rn(val.z, val.w);
                            uint2 pk;
                            pk.x = *reinterpret_cast<uint32_t*>(&p0), pk.y = *reinterpret_cast<uint32_t*>(&p1);
                            *reinterpret_cast<uint2*>(bp + (size_t)i * 4 * e.ld16) = pk;
                        }
                    }
                } else {
#pragma unroll 1
                    for (int i = 0; i < 8; ++i) {
                        const int r = i * 4 + rsub;
                        const int grow = rbase + r;
                        if (grow >= e.M || gcol >= e.N) continue;
                        float4 val = *reinterpret_cast<const float4*>(stg + r * STG_PITCH + (((cq >> 2) ^ (r & 7)) << 2));
                        float o[4] = {val.x, val.y, val.z, val.w};
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            if (gcol + q >= e.N) continue;
                            if (kind == -1) o[q] = fast_epilogue(e, o[q], gcol + q, 0.0f);
                            if (epi == EPI_RESIDUAL) {
                                const size_t ai = (size_t)grow * e.ld_add + gcol + q;
                                o[q] += e.add_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(e.add_in)[ai]) : e.add_in[ai];
                                if (e.res_in) o[q] = fmaf(e.res_scale, o[q], e.res_in[(size_t)grow * e.ld_res + gcol + q]);
                            } else if (epi == EPI_GATE) {
                                const float rs = e.row_scale ? e.row_scale[grow] : 1.0f;
                                o[q] = fmaf(e.res_in[(size_t)grow * e.ld_res + gcol + q] * rs, o[q],
                                            e.add_in[(size_t)grow * e.ld_add + gcol + q] * e.alpha);
                            }
                            if (out32) {
                                float* gp = out32 + (size_t)grow * e.ldo + gcol + q;
                                if (epi == EPI_ADD_OUT) o[q] += *gp;
                                *gp = o[q];
                            }
                            if (out16) out16[(size_t)grow * e.ld16 + gcol + q] = __float2bfloat16_rn(o[q]);
                            if (epi < 0 && e.side_a && gcol + q >= e.c3) {
                                e.side_a[(size_t)grow * e.ld_side_a + (gcol + q - e.c3)] = __float2bfloat16_rn(o[q]);
                                e.side_b[(size_t)grow * e.ld_side_b + (gcol + q - e.c3)] = __float2bfloat16_rn(o[q]);
                            }
                        }
                    }
                }
                __syncwarp();
            }
            if (!released) {  // this warp's column half lies entirely outside the matrix
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (PAIR) mbar_arrive_cluster(leader_acc_empty + buf * 8); else mbar_arrive(&acc_empty[buf]);
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync();  // neither CTA leaves (or frees TMEM) while the other may still signal its barriers or read its operands
    if (warp == 1) {
        tcgen05_fence_after();
        if (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---- host side --------------------------------------------------------------------------------
template <int BN, int STAGES, int MODE = kRuntimeMode, int OUTS = 0, int EW = EPI_WARPS, bool PAIR = false>
int32_t launch_tile(pssa_b200_ctx* ctx, const void* a, const void* b, const GemmEpilogue& e) {
    CUtensorMap map_a, map_b;
    int32_t rc;
    constexpr int B_ROWS = PAIR ? BN / 2 : BN;
    if ((rc = make_map(ctx, &map_a, a, e.M, e.K, BM))) return rc;
    if ((rc = make_map(ctx, &map_b, b, e.N, e.K, B_ROWS))) return rc;
    size_t smem = 1024 + (size_t)STAGES * (BM * BK * 2 + B_ROWS * BK * 2) + (2 * STAGES + 4) * 8 + 16 + EW * 32 * STG_PITCH * 4;
    auto kern = gemm_bf16_tcgen05_kernel<BN, STAGES, MODE, OUTS, EW, PAIR>;
    static PerDeviceOnce attr;  // per instantiation and per device
    if (attr.need(ctx->device)) {
        PSSA_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr.done(ctx->device);
    }
    if (PAIR) {
        // one persistent pair per two SMs; both attributes: the cluster of two, and the dependent launch
        const long long tiles = (long long)((e.M + 2 * BM - 1) / (2 * BM)) * ((e.N + BN - 1) / BN);
        const long long pairs = ctx->sm_count / 2;
        const unsigned grid = 2u * (unsigned)(tiles < pairs ? tiles : pairs);
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(grid), cfg.blockDim = dim3(64 + 32 * EW), cfg.dynamicSmemBytes = smem, cfg.stream = ctx->stream;
        cudaLaunchAttribute attrs[2]{};
        attrs[0].id = cudaLaunchAttributeClusterDimension;
        attrs[0].val.clusterDim.x = 2, attrs[0].val.clusterDim.y = 1, attrs[0].val.clusterDim.z = 1;
        attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attrs, cfg.numAttrs = 2;
        PSSA_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, map_a, map_b, e));
    } else {
        long long tiles = (long long)((e.M + BM - 1) / BM) * ((e.N + BN - 1) / BN);
        unsigned grid = (unsigned)(tiles < ctx->sm_count ? tiles : ctx->sm_count);  // one persistent CTA per SM
        PSSA_CUDA(ctx, launch_dependent(kern, dim3(grid), dim3(64 + 32 * EW), smem, ctx->stream, map_a, map_b, e));
    }
    // the profile facility keys on this name: one entry per epilogue family
    const char* name = e.epi == EPI_POINCARE    ? "gemm_bf16_tcgen05_kernel[Poincare distances]"
                       : e.n_pairs > 0          ? "gemm_bf16_tcgen05_kernel[split value read]"
                       : e.epi < 0              ? "gemm_bf16_tcgen05_kernel[x-side concatenated]"
                       : e.epi == EPI_GATE      ? "gemm_bf16_tcgen05_kernel[gated memory projection]"
                       : e.epi == EPI_RESIDUAL  ? "gemm_bf16_tcgen05_kernel[MLP down + residuals]"
                       : e.epi == EPI_SILU      ? "gemm_bf16_tcgen05_kernel[MLP up, SiLU]"
                       : e.epi == EPI_ADD_OUT   ? "gemm_bf16_tcgen05_kernel[accumulate]"
                       : e.epi == EPI_SCALE     ? "gemm_bf16_tcgen05_kernel[scaled]"
                                                : "gemm_bf16_tcgen05_kernel[plain]";
    return after_launch(ctx, name);
}

int32_t check_shape(pssa_b200_ctx* ctx, const void* a, const void* b, size_t M, size_t N, size_t K) {
    if (M == 0 || N == 0 || K == 0) return fail(ctx, PSSA_B200_ERR_SHAPE, "GEMM dimensions must be positive");
    if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff)
        return fail(ctx, PSSA_B200_ERR_SHAPE, "B200 GEMM dimensions must fit i32; refusing launch");
    if (K % 8 != 0 || (reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15))
        return fail(ctx, PSSA_B200_ERR_UNSUPPORTED,
                    "B200 bf16 GEMM needs K %% 8 == 0 and 16-byte aligned operands (TMA row pitch); K = %zu; use the fp32 path", K);
    if ((M + BM - 1) / BM > 0x7fffffff || (N + 63) / 64 > 65535)
        return fail(ctx, PSSA_B200_ERR_SHAPE, "B200 GEMM grid exceeds grid limits; refusing launch");
    return PSSA_B200_OK;
}

int32_t dispatch(pssa_b200_ctx* ctx, const void* a, const void* b, GemmEpilogue& e) {
    e.status = ctx->status_dev;
    // widest tile that still gives every SM work: 256 columns halve the shared-memory operand traffic per flop,
    // narrow outputs (state / key projections) and short batches (decode) use smaller tiles to spread over SMs
    const long long m_tiles = (e.M + BM - 1) / BM;
    const bool only32 = e.out && !e.out16, only16 = !e.out && e.out16;
    // Decode steps (a few hundred rows against a whole weight matrix): 128 x 32 tiles put 48 to 110 CTAs on a product that
    // 128 x 64 tiles covered with 24 to 56, and ten 20 KB stages keep nearly all of a K = 768 product's operands in
    // flight at once. Each CTA is a short chain of latencies (launch, one operand round trip, epilogue), so what counts
    // is how many run side by side and how little code each has to fetch: the step's products get the specialised
    // epilogues here too.
    if (m_tiles <= 2 && e.N >= 256 && e.N <= 4096) {
        if (e.epi == -1 && only32) return launch_tile<32, 10, -1, 1, 4>(ctx, a, b, e);
        if (e.epi == EPI_POINCARE && only32) return launch_tile<32, 10, EPI_POINCARE, 1, 4>(ctx, a, b, e);
        if (e.epi == EPI_GATE && only16) return launch_tile<32, 10, EPI_GATE, 2, 4>(ctx, a, b, e);
        if (e.epi == EPI_SILU && only16) return launch_tile<32, 10, EPI_SILU, 2, 4>(ctx, a, b, e);
        if (e.epi == EPI_RESIDUAL && only32) return launch_tile<32, 10, EPI_RESIDUAL, 1, 4>(ctx, a, b, e);
        return launch_tile<32, 10, kRuntimeMode, 0, 4>(ctx, a, b, e);
    }
    if (e.N <= 64 || m_tiles * ((e.N + 127) / 128) < ctx->sm_count / 2)
        return (e.epi == EPI_ADD_OUT && e.out && !e.out16 && e.n_pairs == 0) ? launch_tile<64, 7, EPI_ADD_OUT, 1>(ctx, a, b, e)
                                                                            : launch_tile<64, 7>(ctx, a, b, e);
    if (e.N <= 128 || m_tiles * ((e.N + 255) / 256) < ctx->sm_count) return launch_tile<128, 5>(ctx, a, b, e);
    // Four 48 KB stages: with three, the issuing thread of the K = 768 products spent 56 % of its cycles waiting for
    // operands (cycle counters around its two waits, 32 x 2048-token lanes) and 40 % with four (its loop 8-14 % shorter);
    // what then limits these products is the epilogue (its warps wait for an accumulator 9 % of the time). The gated
    // split value read and the distance product are bound by their epilogues already (the issuing thread waits for a
    // drained accumulator, not for operands) and measured slower with four stages (1.98 against 1.45 ms per step): three.
    if (e.epi == EPI_POINCARE && only32) return launch_tile<256, 3, EPI_POINCARE, 1, kWideEpiWarps>(ctx, a, b, e);
    if (e.epi == EPI_GATE && e.n_pairs > 0 && only16) return launch_tile<256, 3, EPI_GATE, 2, kWideEpiWarps>(ctx, a, b, e);
    if (e.n_pairs > 0) return (e.epi == EPI_NONE && only16) ? launch_tile<256, 4, EPI_NONE, 2>(ctx, a, b, e) : launch_tile<256, 4>(ctx, a, b, e);
    // Plain products run as CTA pairs (cta_group::2) when there are enough 256-row tiles for every pair of SMs: the
    // operand traffic per SM, the limiter of the 128 x 256 tile's main loop, drops by a third and six 32 KB stages fit:
    // 8192^3 at 1463 TFLOP/s against 1132, 65536 x 1536 x 768 at 1160 against 804. The block schedule's x-side and MLP
    // products were measured as pairs too (same results, parity green) and were not faster (2.27 / 1.72 / 2.05 ms per
    // step against 2.22 / 1.65 / 2.03): their epilogues and output traffic are the limiters, so they stay single CTAs.
    static const bool use_pairs = std::getenv("PSSA_B200_NO_CTA_PAIRS") == nullptr;  // (for comparisons)
    const bool pair_ok = use_pairs && e.n_pairs == 0 && ((e.M + 2 * BM - 1) / (2 * BM)) * ((e.N + 255) / 256) >= ctx->sm_count / 2;
    if (pair_ok && e.epi == EPI_NONE && only32) return launch_tile<256, 6, EPI_NONE, 1, kWideEpiWarps, true>(ctx, a, b, e);
    if (pair_ok && e.epi == EPI_NONE && only16) return launch_tile<256, 6, EPI_NONE, 2, kWideEpiWarps, true>(ctx, a, b, e);
    // the block schedule's products: one epilogue family and one output set per instantiation
    if (e.epi == -1 && only32) return launch_tile<256, 4, -1, 1, kWideEpiWarps>(ctx, a, b, e);
    if (e.epi == EPI_GATE) return only16 ? launch_tile<256, 3, EPI_GATE, 2, kWideEpiWarps>(ctx, a, b, e) : launch_tile<256, 3, EPI_GATE, 0, kWideEpiWarps>(ctx, a, b, e);
    if (e.epi == EPI_RESIDUAL && only32) return launch_tile<256, 4, EPI_RESIDUAL, 1, kWideEpiWarps>(ctx, a, b, e);
    if (e.epi == EPI_SILU && only16) return launch_tile<256, 4, EPI_SILU, 2, kWideEpiWarps>(ctx, a, b, e);
    return launch_tile<256, 3>(ctx, a, b, e);
}

// Self-test of the bounded wait: one warp initialises an mbarrier that nothing ever arrives at (no copy in flight, no
// other CTA) and waits on it with the pipeline's own helper and a caller-chosen poll limit. The wait gives up, the kernel
// records PSSA_B200_ERR_TIMEOUT in the status word exactly as the GEMM pipeline does, and returns normally.
__global__ void __launch_bounds__(32) wait_expiry_selftest_kernel(int* status, unsigned polls) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (!mbar_wait(&bar, 0, polls)) atomicExch(status, PSSA_B200_ERR_TIMEOUT);
    }
}

}  // namespace

int32_t launch_wait_expiry_selftest(pssa_b200_ctx* ctx, unsigned polls) {
    wait_expiry_selftest_kernel<<<1, 32, 0, ctx->stream>>>(ctx->status_dev, polls);
    return after_launch(ctx, "wait_expiry_selftest_kernel");
}

int32_t launch_gemm_bf16(pssa_b200_ctx* ctx, const void* x16, const void* w16, float* out, void* out_bf16, size_t M, size_t N,
                         size_t K, size_t ldo, int epi, float alpha, size_t ld16) {
    int32_t rc = check_shape(ctx, x16, w16, M, N, K);
    if (rc) return rc;
    GemmEpilogue e{};
    e.out = out, e.out16 = (__nv_bfloat16*)out_bf16, e.ldo = ldo, e.ld16 = ld16 ? ld16 : N;
    e.M = (int)M, e.N = (int)N, e.K = (int)K, e.epi = epi, e.alpha = alpha;
    return dispatch(ctx, x16, w16, e);
}

// out = res_in ? res_in + res_scale * (X W^T + add_in) : X W^T + add_in   (all fp32 [M, N] dense)
int32_t launch_gemm_bf16_residual(pssa_b200_ctx* ctx, const void* x16, const void* w16, float* out, const void* add_in,
                                  const float* res_in, float res_scale, size_t M, size_t N, size_t K, size_t ld_add_bf16) {
    int32_t rc = check_shape(ctx, x16, w16, M, N, K);
    if (rc) return rc;
    GemmEpilogue e{};
    e.out = out, e.out16 = nullptr, e.ldo = N, e.ld16 = 0;
    e.M = (int)M, e.N = (int)N, e.K = (int)K, e.epi = EPI_RESIDUAL, e.alpha = 1.0f;
    e.add_in = (const float*)add_in, e.res_in = res_in, e.ld_add = ld_add_bf16 ? ld_add_bf16 : N, e.ld_res = N, e.res_scale = res_scale;
    e.add_is_bf16 = ld_add_bf16 ? 1 : 0;
    return dispatch(ctx, x16, w16, e);
}

// z = gate * (X W^T) + alpha * y: the memory projection with its sigmoid gate and the scaled SSM output folded into the
// epilogue (src/pssa.rs:1189-1192 without the adapter term, which rides in the MLP products as extra K columns).
// gate [M, ld_gate] and y [M, N] fp32; out fp32 [M, N] and out16 bf16 [M, ld16] are both written.
int32_t launch_gemm_bf16_gate(pssa_b200_ctx* ctx, const void* x16, const void* w16, float* out, void* out_bf16, size_t ld16,
                              const float* gate, size_t ld_gate, const float* y, float alpha, size_t M, size_t N, size_t K, bool split_k,
                              const float* row_scale) {
    if (split_k && K % BK != 0) return fail(ctx, PSSA_B200_ERR_UNSUPPORTED, "B200 split GEMM needs K %% 64 == 0; K = %zu", K);
    int32_t rc = check_shape(ctx, x16, w16, M, N, split_k ? 3 * K : K);
    if (rc) return rc;
    GemmEpilogue e{};
    e.out = out, e.out16 = (__nv_bfloat16*)out_bf16, e.ldo = N, e.ld16 = ld16;
    e.M = (int)M, e.N = (int)N, e.K = (int)(split_k ? 3 * K : K), e.epi = EPI_GATE, e.alpha = alpha;
    e.add_in = y, e.res_in = gate, e.ld_add = N, e.ld_res = ld_gate, e.res_scale = 1.0f, e.row_scale = row_scale;
    if (split_k) e.n_pairs = 1, e.seg_kb = (int)(K / BK);  // pair (0, 0): leading piece of each operand
    return dispatch(ctx, x16, w16, e);
}

// fp32-accurate product from three bf16 pieces per operand: a16 [M, 3*K], b16 [N, 3*K], K a multiple of 64.
// The six products whose weight is above 2^-24 are accumulated: (0,0) (0,1) (1,0) (0,2) (1,1) (2,0); `terms` == 3 keeps
// the first three (weight above 2^-16), enough when only the bf16 copy of the result is used.
int32_t launch_gemm_bf16_split3(pssa_b200_ctx* ctx, const void* a16, const void* b16, float* out, void* out_bf16, size_t M,
                                size_t N, size_t K, size_t ldo, int terms) {
    if (K % BK != 0) return fail(ctx, PSSA_B200_ERR_UNSUPPORTED, "B200 split GEMM needs K %% 64 == 0; K = %zu", K);
    int32_t rc = check_shape(ctx, a16, b16, M, N, 3 * K);
    if (rc) return rc;
    GemmEpilogue e{};
    e.out = out, e.out16 = (__nv_bfloat16*)out_bf16, e.ldo = ldo, e.ld16 = N;
    e.M = (int)M, e.N = (int)N, e.K = (int)(3 * K), e.epi = EPI_NONE, e.alpha = 1.0f;
    e.n_pairs = terms == 3 ? 3 : terms == 1 ? 1 : 6, e.seg_kb = (int)(K / BK);
    const unsigned char pa[6] = {0, 0, 1, 0, 1, 2}, pb[6] = {0, 1, 0, 2, 1, 0};
    for (int i = 0; i < 6; ++i) e.pair_a[i] = pa[i], e.pair_b[i] = pb[i];
    return dispatch(ctx, a16, b16, e);
}

// dist[M, ldo] (first N columns) = Poincare distance between M points of the ball and N bank keys, from the inner products
// of their three-piece bf16 splits a16 [M, 3*K], b16 [N, 3*K] (all six partial products: fp32-accurate p.k).
int32_t launch_gemm_bf16_poincare(pssa_b200_ctx* ctx, const void* a16, const void* b16, const float2* row_stat,
                                  const float2* col_stat, float* dist, size_t M, size_t N, size_t K, size_t ldo) {
    if (K % BK != 0) return fail(ctx, PSSA_B200_ERR_UNSUPPORTED, "B200 split GEMM needs K %% 64 == 0; K = %zu", K);
    int32_t rc = check_shape(ctx, a16, b16, M, N, 3 * K);
    if (rc) return rc;
    GemmEpilogue e{};
    e.out = dist, e.out16 = nullptr, e.ldo = ldo, e.ld16 = 0;
    e.M = (int)M, e.N = (int)N, e.K = (int)(3 * K), e.epi = EPI_POINCARE, e.alpha = 1.0f;
    e.n_pairs = 6, e.seg_kb = (int)(K / BK);
    const unsigned char pa[6] = {0, 0, 1, 0, 1, 2}, pb[6] = {0, 1, 0, 2, 1, 0};
    for (int i = 0; i < 6; ++i) e.pair_a[i] = pa[i], e.pair_b[i] = pb[i];
    e.row_stat = row_stat, e.col_stat = col_stat;
    return dispatch(ctx, a16, b16, e);
}

int32_t launch_gemm_bf16_cat(pssa_b200_ctx* ctx, const void* x16, const void* w16, float* out, size_t M, size_t N, size_t K,
                             size_t ldo, int c1, int c2, int c3, void* side_a, size_t ld_side_a, void* side_b, size_t ld_side_b) {
    int32_t rc = check_shape(ctx, x16, w16, M, N, K);
    if (rc) return rc;
    GemmEpilogue e{};
    e.out = out, e.out16 = nullptr, e.ldo = ldo, e.ld16 = 0;
    e.M = (int)M, e.N = (int)N, e.K = (int)K, e.epi = -1, e.alpha = 1.0f, e.c1 = c1, e.c2 = c2, e.c3 = c3;
    if (side_a && side_b) {
        if (c3 % 4 != 0 || ld_side_a % 4 != 0 || ld_side_b % 4 != 0 || (reinterpret_cast<uintptr_t>(side_a) & 7) || (reinterpret_cast<uintptr_t>(side_b) & 7))
            return fail(ctx, PSSA_B200_ERR_UNSUPPORTED, "B200 concatenated GEMM: side buffers need 8-byte aligned rows");
        e.side_a = (__nv_bfloat16*)side_a, e.side_b = (__nv_bfloat16*)side_b, e.ld_side_a = ld_side_a, e.ld_side_b = ld_side_b;
    }
    return dispatch(ctx, x16, w16, e);
}

}  // namespace pssa
