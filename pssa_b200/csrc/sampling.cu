// Device-side token sampling for batched decode: `PSSAInferenceEngine::sample` (src/inference.rs:102-181) for many
// streams at once, so a decode step reads back one id per stream instead of a row of logits.
//
// One CTA per stream, in the reference's order of operations:
//   1. any non-finite logit is an error;
//   2. repetition penalty over the last <= 64 generated ids, applied id by id (an id that repeats in the window is
//      penalised repeatedly, as in the reference's loop);
//   3. temperature 0: argmax over ids 1..V-1 under total order, ties to the lowest id;
//   4. otherwise max over ids 1..V-1, p_i = exp((l_i - max) / T), sum, candidates (p_i / sum), the top_k largest by
//      (probability desc, id asc) selected in order by repeated block-wide maxima, top-p cut on the running sum, mass,
//      one xorshift64* draw (src/linalg.rs:13-26), pick.
// EXACT (flag) keeps the reference's sequential f32 sum over the vocabulary (one thread, V dependent adds); the default
// sums per thread and then over the CTA in a fixed order, which can move the sum by a few ulp.
#include <cuda_runtime.h>

#include <cfloat>

#include "context.hpp"
#include "kernels.hpp"

namespace pssa {
namespace {

constexpr int kSampleThreads = 256;
constexpr int kRecent = 64;

__device__ __forceinline__ int order_key(float v) {  // monotone signed key of f32::total_cmp
    int b = __float_as_int(v);
    return b < 0 ? (b ^ 0x7fffffff) : b;
}

// block-wide maximum of a 64-bit key; every thread gets the result
__device__ __forceinline__ unsigned long long block_max_u64(unsigned long long v, unsigned long long* scratch) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        unsigned long long o = __shfl_xor_sync(0xffffffffu, v, m);
        v = o > v ? o : v;
    }
    __syncthreads();  // scratch may still be read from the previous call
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    unsigned long long r = scratch[0];
#pragma unroll
    for (int w = 1; w < kSampleThreads / 32; ++w) r = scratch[w] > r ? scratch[w] : r;
    return r;
}

__global__ void __launch_bounds__(kSampleThreads) sample_kernel(SampleParams p) {
    extern __shared__ float s_dyn[];  // [top_k] selected probabilities, then [top_k] ids
    __shared__ unsigned long long s_red[kSampleThreads / 32];
    __shared__ float s_part[kSampleThreads];
    __shared__ int s_flag;
    __shared__ unsigned s_pen_id[kRecent];
    __shared__ float s_pen_orig[kRecent];
    __shared__ unsigned s_pen_n;
    __shared__ float s_raw_max, s_raw_sum;
    const int tid = threadIdx.x;
    const size_t row = blockIdx.x;
    const size_t slot = p.slots ? p.slots[row] : row;  // where this row's history and generator live
    const int v = p.vocab;
    float* lg = p.logits + row * (size_t)v;
    float* pr = p.probs + row * (size_t)v;
    float* sel_p = s_dyn;
    unsigned* sel_id = reinterpret_cast<unsigned*>(s_dyn + p.top_k);

    // 1. finite check
    if (tid == 0) s_flag = 0;
    __syncthreads();
    bool bad = false;
    for (int i = tid; i < v; i += kSampleThreads) bad = bad || !isfinite(lg[i]);
    if (bad) s_flag = 1;
    __syncthreads();
    if (s_flag) {
        if (tid == 0) p.ids_out[row] = 0xffffffffu, p.status_out[row] = 1;
        return;
    }
    // raw softmax statistics over ALL ids, before penalty / temperature / exclusion of id 0 (`raw_confidence`,
    // src/inference.rs:526-545); only when the caller wants the selected token's raw probability
    if (p.confidence_out) {
        float mxr = -FLT_MAX;
        for (int i = tid; i < v; i += kSampleThreads) mxr = fmaxf(mxr, lg[i]);
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) mxr = fmaxf(mxr, __shfl_xor_sync(0xffffffffu, mxr, m));
        s_part[tid] = mxr;
        __syncthreads();
        if (tid == 0) {
            for (int t = 0; t < kSampleThreads; t += 32) mxr = fmaxf(mxr, s_part[t]);
            s_raw_max = mxr;
        }
        __syncthreads();
        mxr = s_raw_max;
        float part = 0.0f;
        for (int i = tid; i < v; i += kSampleThreads) part += expf(__fsub_rn(lg[i], mxr));
        s_part[tid] = part;
        __syncthreads();
        if (tid == 0) {
            float sum = 0.0f;
            if (p.exact) {
                for (int i = 0; i < v; ++i) sum = __fadd_rn(sum, expf(__fsub_rn(lg[i], mxr)));  // the reference's order
            } else {
                for (int t = 0; t < kSampleThreads; ++t) sum += s_part[t];
            }
            s_raw_sum = sum;
        }
        __syncthreads();
    }
    if (tid == 0) s_pen_n = 0;
    // 2. repetition penalty, in the order the ids were generated
    if (tid == 0 && p.repetition_penalty > 1.0f && p.recent_ids) {
        const unsigned n = min(p.recent_count[slot], (unsigned)kRecent);
        const unsigned* ids = p.recent_ids + slot * kRecent;
        for (unsigned g = 0; g < n; ++g) {
            const unsigned id = ids[g];
            if (id < (unsigned)v) {
                bool known = false;  // remember the unpenalised value once per id (for the raw confidence)
                for (unsigned q = 0; q < g && !known; ++q) known = ids[q] == id;
                if (!known) s_pen_id[s_pen_n] = id, s_pen_orig[s_pen_n] = lg[id], ++s_pen_n;
                lg[id] = lg[id] > 0.0f ? __fdiv_rn(lg[id], p.repetition_penalty) : __fmul_rn(lg[id], p.repetition_penalty);
            }
        }
    }
    __syncthreads();
    auto publish = [&](unsigned id) {  // thread 0 only: the selected id and, if wanted, its raw softmax probability
        p.ids_out[row] = id, p.status_out[row] = 0;
        if (p.confidence_out) {
            float raw = lg[id];
            for (unsigned q = 0; q < s_pen_n; ++q)
                if (s_pen_id[q] == id) raw = s_pen_orig[q];
            p.confidence_out[row] = __fdiv_rn(expf(__fsub_rn(raw, s_raw_max)), s_raw_sum);
        }
    };
    // 3 / 4a. maximum over ids 1..V-1 as (order key, lowest id wins)
    unsigned long long best = 0;
    for (int i = tid; i < v; i += kSampleThreads)
        if (i >= 1) {
            unsigned long long k = ((unsigned long long)(unsigned)(order_key(lg[i]) ^ 0x80000000) << 32) | (0xffffffffu - (unsigned)i);
            best = k > best ? k : best;
        }
    best = block_max_u64(best, s_red);
    if (v < 2) {
        if (tid == 0) p.ids_out[row] = 0xffffffffu, p.status_out[row] = 3;
        return;
    }
    const unsigned arg_max = 0xffffffffu - (unsigned)(best & 0xffffffffull);
    if (p.temperature == 0.0f) {
        if (tid == 0) publish(arg_max);
        return;
    }
    const float mx = lg[arg_max];
    // 4b. probabilities and their sum
    float part = 0.0f;
    for (int i = tid; i < v; i += kSampleThreads) {
        float e = i >= 1 ? expf(__fdiv_rn(__fsub_rn(lg[i], mx), p.temperature)) : 0.0f;
        pr[i] = e;
        part += e;
    }
    s_part[tid] = part;
    __syncthreads();
    if (tid == 0) {
        float sum = 0.0f;
        if (p.exact) {
            for (int i = 1; i < v; ++i) sum = __fadd_rn(sum, pr[i]);  // the reference's order
        } else {
            for (int t = 0; t < kSampleThreads; ++t) sum += s_part[t];
        }
        s_part[0] = sum;
    }
    __syncthreads();
    const float sum = s_part[0];
    if (!isfinite(sum) || sum <= 0.0f) {
        if (tid == 0) p.ids_out[row] = 0xffffffffu, p.status_out[row] = 2;
        return;
    }
    // candidates carry p_i / sum, and ties of the QUOTIENT go to the lower id (src/inference.rs:150-156)
    for (int i = tid; i < v; i += kSampleThreads)
        if (i >= 1) pr[i] = __fdiv_rn(pr[i], sum);
    // 4c. the top_k candidates by (probability desc, id asc), in order. Probabilities are >= +0, so their bit patterns
    // order them; a taken candidate is marked by setting its sign bit. Each thread caches the best of its own elements
    // and rescans them only after losing that element.
    const int k_want = min(p.top_k, v - 1);
    auto scan_own = [&]() {
        unsigned long long b = 0;
        for (int i = tid; i < v; i += kSampleThreads)
            if (i >= 1) {
                const unsigned bits = __float_as_uint(pr[i]);
                if ((bits & 0x80000000u) || !isfinite(pr[i])) continue;
                unsigned long long k = ((unsigned long long)(bits + 1u) << 32) | (0xffffffffu - (unsigned)i);
                b = k > b ? k : b;
            }
        return b;
    };
    unsigned long long own = scan_own();
    int n_sel = 0;
    for (int r = 0; r < k_want; ++r) {
        const unsigned long long win = block_max_u64(own, s_red);
        if (win == 0) break;  // fewer finite candidates than top_k
        const unsigned id = 0xffffffffu - (unsigned)(win & 0xffffffffull);
        if (own == win) {  // this thread owned the winner
            sel_p[r] = pr[id];
            sel_id[r] = id;
            pr[id] = __uint_as_float(__float_as_uint(pr[id]) | 0x80000000u);
            own = scan_own();
        }
        n_sel = r + 1;
    }
    __syncthreads();
    // 4d. top-p cut, mass, draw, pick (sequential over at most top_k entries)
    if (tid == 0) {
        if (n_sel == 0) {
            p.ids_out[row] = 0xffffffffu, p.status_out[row] = 3;
            return;
        }
        int cutoff = n_sel;
        float cumulative = 0.0f;
        for (int i = 0; i < n_sel; ++i) {
            cumulative = __fadd_rn(cumulative, sel_p[i]);
            if (cumulative >= p.top_p) {
                cutoff = i + 1;
                break;
            }
        }
        const int n = max(cutoff, 1);
        float mass = 0.0f;
        for (int i = 0; i < n; ++i) mass = __fadd_rn(mass, sel_p[i]);
        // src/linalg.rs:13-26
        unsigned long long x = p.rng_state[slot];
        x ^= x >> 12, x ^= x << 25, x ^= x >> 27;
        p.rng_state[slot] = x;
        const unsigned u = (unsigned)((x * 0x2545f4914f6cdd1dull) >> 32);
        const float norm = __fdiv_rn((float)u, 4294967296.0f);  // u32::MAX as f32 rounds to 2^32
        const float draw = __fadd_rn(0.0f, __fmul_rn(norm, __fsub_rn(mass, 0.0f)));
        float running = 0.0f;
        unsigned id = sel_id[n - 1];
        for (int i = 0; i < n; ++i) {
            running = __fadd_rn(running, sel_p[i]);
            if (draw <= running) {
                id = sel_id[i];
                break;
            }
        }
        publish(id);
    }
}

// append each row's new id to its stream's window of the last 64 generated ids (oldest first)
__global__ void push_recent_kernel(const unsigned* __restrict__ ids, const unsigned* __restrict__ slots, unsigned* __restrict__ recent,
                                   unsigned* __restrict__ count, size_t rows) {
    const size_t row = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows || ids[row] == 0xffffffffu) return;
    const size_t slot = slots ? slots[row] : row;
    unsigned* w = recent + slot * kRecent;
    unsigned n = count[slot];
    if (n >= (unsigned)kRecent) {
        for (int i = 1; i < kRecent; ++i) w[i - 1] = w[i];
        n = kRecent - 1;
    }
    w[n] = ids[row];
    count[slot] = n + 1;
}

}  // namespace

int32_t launch_push_recent(pssa_b200_ctx* ctx, const unsigned* ids, const unsigned* slots, unsigned* recent, unsigned* count, size_t rows) {
    push_recent_kernel<<<(unsigned)((rows + 127) / 128), 128, 0, ctx->stream>>>(ids, slots, recent, count, rows);
    return after_launch(ctx, "push_recent_kernel");
}

int32_t launch_sample(pssa_b200_ctx* ctx, const SampleParams& p) {
    if (p.rows == 0 || p.rows > 0x7fffffffull) return fail(ctx, PSSA_B200_ERR_SHAPE, "sampling: row count must be in 1..2^31-1");
    if (p.vocab < 1) return fail(ctx, PSSA_B200_ERR_SHAPE, "sampling: empty vocabulary");
    if (p.top_k < 1 || p.top_k > 4096)
        return fail(ctx, PSSA_B200_ERR_UNSUPPORTED, "sampling: top-k %d outside 1..4096 (the candidates of a stream live in shared memory)", p.top_k);
    sample_kernel<<<(unsigned)p.rows, kSampleThreads, (size_t)p.top_k * 8, ctx->stream>>>(p);
    return after_launch(ctx, "sample_kernel");
}

}  // namespace pssa
