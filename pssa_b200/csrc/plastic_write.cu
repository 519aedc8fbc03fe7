// Write side of the episodic bank and the plastic fast weights.
//
//  * bank_insert_protected_kernel: `insert_protected_with_device` (src/memory.rs:315-342) with the refractory
//    gate `apply_refractory_overwrite` (src/defense.rs:45-67) and the ring insert (src/memory.rs:268-303),
//    for an ORDERED list of writes (the gate is history dependent: src/gpu_batch.rs:742-746). Gate and copy are one
//    kernel; a write costs (k + d + 3) floats of HBM traffic.
//  * the same kernel in "winning slot" mode (the retrieval operator's benchmark configuration, not a reference
//    code path): the gated slot is the caller's nearest slot instead of the ring head and a successful write is the
//    rank-1 update v_slot += eta * (target - v_slot) instead of a full overwrite.
//  * plastic_update_kernel: the Hebbian rank-1 update of the adapter's fast weights `dream_replay_value`
//    (src/pssa.rs:1814-1832) and `consolidate` (src/adapter.rs:65-72).
#include <cuda_runtime.h>

#include <cfloat>

#include "context.hpp"
#include "kernels.hpp"

namespace pssa {
namespace {

// defense.rs:18-22
__device__ __forceinline__ float refractory_gain(unsigned long long delta_tokens, float tau_refractory) {
    float dt = (float)delta_tokens;
    float lin = __fsub_rn(1.0f, expf(__fdiv_rn(-dt, tau_refractory)));
    return fmaxf(__fmul_rn(lin, lin), 0.005f);
}

// One CTA walks the writes in order. meta = {count, write_head}.
// Slot ids and the two meta words live on the device, where the host cannot validate them: a write whose target would
// fall outside the bank (count > cap, head or winning slot >= cap) or whose key is not inside the open unit ball
// (the reference asserts this, src/memory.rs:273-277) is skipped, reported as slot -2 and recorded in the context's
// status word; nothing is read or written out of bounds.
__global__ void __launch_bounds__(256) bank_insert_protected_kernel(BankWriteParams p) {
    __shared__ long long s_slot;   // slot to write, -1 = defended
    __shared__ float s_norm_sq;
    const int tid = threadIdx.x;
    for (size_t w = 0; w < p.n; ++w) {
        const float* key = p.key_pnc + w * p.dk;
        const float* val = p.val + w * p.dv;
        if (tid == 0) {
            unsigned long long count = p.meta[0], head = p.meta[1];
            const unsigned long long step = p.step[w];
            long long slot;
            const unsigned long long target = p.winning_slots ? (unsigned long long)p.winning_slots[w] : head;
            float key_norm_sq = 0.0f;
            bool bad = count > (unsigned long long)p.cap || ((p.winning_slots || count == (unsigned long long)p.cap) && target >= (unsigned long long)p.cap);
            if (!bad && p.winning_slots == nullptr) {
                // memory.rs:181-192: f64 sum of squares, nudged below one
                double n2 = 0.0;
                for (int i = 0; i < p.dk; ++i) {
                    double v = (double)key[i];
                    n2 = __dadd_rn(n2, __dmul_rn(v, v));
                }
                bad = !(n2 < 1.0);  // also catches NaN
                key_norm_sq = (n2 < 1.0 && (float)n2 == 1.0f) ? __uint_as_float(0x3f7fffffu) : (float)n2;
            }
            if (bad) {
                slot = -2;
                if (p.status) atomicExch(p.status, PSSA_B200_ERR_BANK);
            } else if (p.winning_slots == nullptr && count < (unsigned long long)p.cap) {
                slot = (long long)count;  // memory.rs:316-320: append while the bank is not full
                p.meta[0] = count + 1;
                p.confidence[slot] = 1.0f;
                p.last_seen[slot] = step;
            } else {
                const unsigned long long idx = target;
                // defense.rs:45-67
                const unsigned long long seen = p.last_seen[idx];
                const unsigned long long dt = step >= seen ? step - seen : 0;
                const float damage = __fmul_rn(__fmul_rn(0.08f, p.surprise[w]), refractory_gain(dt, 60.0f));
                const float conf = p.confidence[idx];
                if (conf > damage) {
                    p.confidence[idx] = __fsub_rn(conf, damage);
                    p.last_seen[idx] = step;
                    slot = -1;
                } else {
                    p.confidence[idx] = 1.0f;
                    p.last_seen[idx] = step;
                    slot = (long long)idx;
                    if (p.winning_slots == nullptr) p.meta[1] = (head + 1) % (unsigned long long)p.cap;  // memory.rs:279-283
                }
            }
            s_norm_sq = key_norm_sq;
            s_slot = slot;
            if (p.slots_out) p.slots_out[w] = slot;
        }
        __syncthreads();
        const long long slot = s_slot;
        if (slot >= 0) {
            if (p.winning_slots == nullptr) {
                for (int i = tid; i < p.dk; i += blockDim.x) p.keys[slot * p.dk + i] = key[i];
                for (int i = tid; i < p.dv; i += blockDim.x) p.values[slot * p.dv + i] = val[i];
                if (tid == 0) p.norm_sq[slot] = s_norm_sq;
            } else {
                // rank-1 plastic write: pull the winning slot's value towards the target
                for (int i = tid; i < p.dv; i += blockDim.x) {
                    float old = p.values[slot * p.dv + i];
                    p.values[slot * p.dv + i] = __fadd_rn(old, __fmul_rn(p.eta, __fsub_rn(val[i], old)));
                }
            }
        }
        __syncthreads();
    }
}

// src/pssa.rs:1820-1831: rate = 0.02 / (1 + |v|), err_i = clamp(v_i - ad_out_i, -4, 4), U[i, r] += rate*err_i*act_r
__global__ void __launch_bounds__(256) plastic_update_kernel(float* __restrict__ up_fast, const float* __restrict__ value,
                                                             const float* __restrict__ ad_out, const float* __restrict__ ad_act,
                                                             int d, int rank) {
    __shared__ float s_rate;
    if (threadIdx.x == 0) {
        double n2 = 0.0;
        for (int i = 0; i < d; ++i) {
            double v = (double)value[i];
            n2 = __dadd_rn(n2, __dmul_rn(v, v));
        }
        double norm = sqrt(n2);
        s_rate = __fdiv_rn(0.02f, __fadd_rn(1.0f, (float)fmin(norm, (double)FLT_MAX)));
    }
    __syncthreads();
    const float rate = s_rate;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < d * rank; idx += gridDim.x * blockDim.x) {
        int i = idx / rank, r = idx % rank;
        float err = fminf(fmaxf(__fsub_rn(value[i], ad_out[i]), -4.0f), 4.0f);
        up_fast[idx] = __fadd_rn(up_fast[idx], __fmul_rn(__fmul_rn(rate, err), ad_act[r]));
    }
}

// src/adapter.rs:65-72
__global__ void __launch_bounds__(256) consolidate_kernel(float* __restrict__ up_fast, float* __restrict__ up_slow, size_t n,
                                                          float alpha) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    float fast = up_fast[idx];
    up_slow[idx] = __fadd_rn(up_slow[idx], __fmul_rn(alpha, fast));
    up_fast[idx] = __fmul_rn(__fsub_rn(1.0f, alpha), fast);
}

}  // namespace

int32_t launch_bank_insert_protected(pssa_b200_ctx* ctx, const BankWriteParams& p) {
    BankWriteParams q = p;
    q.status = ctx->status_dev;
    bank_insert_protected_kernel<<<1, 256, 0, ctx->stream>>>(q);
    return after_launch(ctx, "bank_insert_protected_kernel");
}

int32_t launch_plastic_update(pssa_b200_ctx* ctx, float* up_fast, const float* value, const float* ad_out, const float* ad_act,
                              int d, int rank) {
    // every block recomputes the (cheap) rate so no second launch is needed
    unsigned blocks = (unsigned)((d * rank + 255) / 256);
    plastic_update_kernel<<<blocks, 256, 0, ctx->stream>>>(up_fast, value, ad_out, ad_act, d, rank);
    return after_launch(ctx, "plastic_update_kernel");
}

int32_t launch_consolidate(pssa_b200_ctx* ctx, float* up_fast, float* up_slow, size_t n, float alpha) {
    consolidate_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(up_fast, up_slow, n, alpha);
    return after_launch(ctx, "consolidate_kernel");
}

}  // namespace pssa
