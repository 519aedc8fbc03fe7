// Model-level entry points: upload, recurrent state, batched prefill and decode.
// The schedule per block is the reference's staged chunk forward (src/gpu_batch.rs:1654-1753):
// embed/norm -> projections -> SSM -> memory -> adapter -> MLP, with the carry in `state`.
#include <cmath>
#include <cstring>

#include "bounds.hpp"
#include "context.hpp"
#include "device_math.cuh"
#include "kernels.hpp"
#include "model.hpp"

using namespace pssa;

namespace {

int32_t mfail(pssa_b200_model* m, int32_t code, const char* msg) { return fail(m ? m->ctx : nullptr, code, "%s", msg); }

size_t tensor_len(const pssa_b200_model* m, int id) {
    size_t d = m->d, s = m->s, k = m->k, r = m->rank;
    switch (id) {
        case T_EMBED: case T_UNEMBED: return m->v * d;
        case T_NORM_GAMMA: case T_NORM_BETA: return d;
        case T_A_MAT: return d * s;
        case T_W_DELTA: case T_W_GATE: case T_W_PROJ: return d * d;
        case T_W_B: case T_W_C: return s * d;
        case T_W_QX: case T_W_QH: return k * d;
        case T_MLP_W1: case T_MLP_W2: return 2 * d * d;
        case T_AD_DOWN: case T_AD_UP: case T_AD_CONS: return r * d;
        case T_BANK_KEYS: return m->cap * k;
        case T_BANK_VALUES: return m->cap * d;
        case T_BANK_NORM_SQ: case T_BANK_CONFIDENCE: return m->cap;
        case T_RESIDUAL_SCALES: return m->depth - 1;
        default: return 0;
    }
}

const int kBlockTensors[] = {T_NORM_GAMMA, T_NORM_BETA, T_A_MAT, T_W_DELTA, T_W_B, T_W_C, T_W_QX, T_W_QH, T_W_GATE,
                             T_W_PROJ, T_MLP_W1, T_MLP_W2, T_AD_DOWN, T_AD_UP, T_AD_CONS, T_BANK_KEYS, T_BANK_VALUES,
                             T_BANK_NORM_SQ};

int32_t dev_alloc(pssa_b200_ctx* ctx, void** p, size_t bytes, bool zero) {
    cudaError_t e = cudaMalloc(p, bytes ? bytes : 4);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "model allocation");
    if (zero) PSSA_CUDA(ctx, cudaMemsetAsync(*p, 0, bytes ? bytes : 4, ctx->stream));
    return PSSA_B200_OK;
}

void free_workspace(Workspace& ws) {
    if (ws.base) cudaFree(ws.base);
    ws = Workspace();
}

}  // namespace

extern "C" {

int32_t pssa_b200_model_create(pssa_b200_ctx* ctx, const pssa_b200_config* cfg, uint32_t max_streams,
                               pssa_b200_model** out) {
    if (!ctx || !cfg || !out) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "pssa_b200_model_create: null argument");
    *out = nullptr;
    // PSSAConfigV2::validate (src/pssa.rs:272-310)
    if (cfg->depth < 1 || cfg->depth > 32) return fail(ctx, PSSA_B200_ERR_SHAPE, "depth must be in 1..=32");
    if (!cfg->d_vocab || !cfg->d_latent || !cfg->d_state || !cfg->d_mem_key || !cfg->mem_capacity)
        return fail(ctx, PSSA_B200_ERR_SHAPE, "all model dimensions, memory capacity, and chunk length must be positive");
    if (!(cfg->tau_mem > 0.0f) || !std::isfinite(cfg->tau_mem))
        return fail(ctx, PSSA_B200_ERR_SHAPE, "lr, eps, and tau_mem must be finite and positive");
    if (max_streams == 0) return fail(ctx, PSSA_B200_ERR_SHAPE, "max_streams must be positive");
    if (cfg->d_state > 512) return fail(ctx, PSSA_B200_ERR_UNSUPPORTED, "B200 SSM: state width exceeds 512; refusing launch");
    if (cfg->d_vocab > 0xfffffffeull || cfg->d_latent > 0x7fffffff || cfg->mem_capacity > 0x7fffffff)
        return fail(ctx, PSSA_B200_ERR_SHAPE, "B200 model dimensions must fit i32; refusing launch");
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    pssa_b200_model* m = new pssa_b200_model();
    m->ctx = ctx;
    m->cfg = *cfg;
    m->d = cfg->d_latent, m->s = cfg->d_state, m->k = cfg->d_mem_key, m->cap = cfg->mem_capacity, m->v = cfg->d_vocab;
    m->depth = cfg->depth;
    m->max_streams = max_streams;
    m->off_delta = 0;
    m->off_b = m->d;
    m->off_c = m->off_b + m->s;
    m->off_q = m->off_c + m->s;
    m->off_gate = m->off_q + m->k;
    m->off_act = m->off_gate + m->d;
    m->ncat = m->off_act + m->rank;
    m->blocks.resize(m->depth);
    m->residual_scales.assign(m->depth - 1, 1.0f / std::sqrt((float)m->depth));  // src/pssa.rs:2059
    m->tensor_set.assign((m->depth + 1) * T_COUNT, false);
    int32_t rc = PSSA_B200_OK;
    auto guard = [&](int32_t r) {
        if (r != PSSA_B200_OK && rc == PSSA_B200_OK) rc = r;
    };
    guard(dev_alloc(ctx, (void**)&m->embed, m->v * m->d * 4, true));
    guard(dev_alloc(ctx, (void**)&m->unembed, m->v * m->d * 4, true));
    guard(dev_alloc(ctx, &m->unembed_bf16, m->v * m->d * 2, true));
    guard(dev_alloc(ctx, (void**)&m->state, (size_t)max_streams * m->depth * m->d * m->s * 4, true));
    for (auto& b : m->blocks) {
        for (int id : kBlockTensors) guard(dev_alloc(ctx, (void**)&b.w[id], tensor_len(m, id) * 4, true));
        guard(dev_alloc(ctx, (void**)&b.rates, m->d * m->s * 4, true));
        guard(dev_alloc(ctx, (void**)&b.u_eff, m->d * m->rank * 4, true));
        guard(dev_alloc(ctx, &b.wcat_bf16, m->ncat * m->d * 2, true));
        guard(dev_alloc(ctx, &b.wqh_bf16, m->k * m->d * 2, true));
        guard(dev_alloc(ctx, &b.wproj_bf16, m->d * m->d * 2, true));
        guard(dev_alloc(ctx, &b.w1cat_bf16, 2 * m->d * (m->d + 64) * 2, true));
        guard(dev_alloc(ctx, &b.w2cat_bf16, m->d * (2 * m->d + 64) * 2, true));
        guard(dev_alloc(ctx, (void**)&b.w1u, 2 * m->d * 16 * 4, true));
        guard(dev_alloc(ctx, &b.vsplit_bf16, m->d * 3 * m->cap * 2, true));
        guard(dev_alloc(ctx, &b.vpsplit_bf16, m->d * 3 * m->cap * 2, true));
        guard(dev_alloc(ctx, (void**)&b.vp, m->cap * m->d * sizeof(float), true));
        guard(dev_alloc(ctx, &b.ksplit_bf16, m->cap * 3 * m->k * 2, true));
        guard(dev_alloc(ctx, (void**)&b.kstat, m->cap * sizeof(float2), true));
        b.host_up.assign(m->d * m->rank, 0.0f);
        b.host_cons.assign(m->d * m->rank, 0.0f);
        b.confidence.assign(m->cap, 1.0f);
        b.last_seen.assign(m->cap, 0);
    }
    if (rc != PSSA_B200_OK) {
        std::string keep = ctx->error;
        pssa_b200_model_destroy(m);
        ctx->error = keep;
        return rc;
    }
    // norm_gamma defaults to one (src/pssa.rs:645)
    std::vector<float> ones(m->d, 1.0f);
    for (auto& b : m->blocks)
        PSSA_CUDA(ctx, cudaMemcpyAsync(b.w[T_NORM_GAMMA], ones.data(), m->d * 4, cudaMemcpyHostToDevice, ctx->stream));
    PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    *out = m;
    return PSSA_B200_OK;
}

void pssa_b200_model_destroy(pssa_b200_model* m) {
    if (!m) return;
    cudaSetDevice(m->ctx->device);
    cudaStreamSynchronize(m->ctx->stream);
    cudaFree(m->embed);
    cudaFree(m->unembed);
    cudaFree(m->unembed_bf16);
    cudaFree(m->state);
    cudaFree(m->obs.q_pnc), cudaFree(m->obs.buf);
    cudaFree(m->score.logits), cudaFree(m->score.targets), cudaFree(m->score.loss);
    cudaFree(m->sampler.recent), cudaFree(m->sampler.count), cudaFree(m->sampler.rng), cudaFree(m->sampler.ids);
    cudaFree(m->sampler.status), cudaFree(m->sampler.head_slot), cudaFree(m->sampler.probs), cudaFree(m->sampler.conf);
    cudaFree(m->chunks.off), cudaFree(m->chunks.len), cudaFree(m->chunks.records), cudaFree(m->chunks.carry_in);
    for (auto& b : m->blocks) {
        for (int id : kBlockTensors) cudaFree(b.w[id]);
        cudaFree(b.rates);
        cudaFree(b.u_eff);
        cudaFree(b.wcat_bf16);
        cudaFree(b.wqh_bf16);
        cudaFree(b.wproj_bf16);
        cudaFree(b.w1cat_bf16);
        cudaFree(b.w2cat_bf16);
        cudaFree(b.w1u);
        cudaFree(b.vsplit_bf16);
        cudaFree(b.vpsplit_bf16);
        cudaFree(b.vp);
        cudaFree(b.ksplit_bf16);
        cudaFree(b.kstat);
    }
    free_workspace(m->ws);
    delete m;
}

int32_t pssa_b200_model_set_tensor(pssa_b200_model* m, int32_t layer, int32_t id, const float* data, size_t len) {
    if (!m || !data) return mfail(m, PSSA_B200_ERR_INVALID_ARGUMENT, "pssa_b200_model_set_tensor: null argument");
    pssa_b200_ctx* ctx = m->ctx;
    bool model_level = id == T_EMBED || id == T_UNEMBED || id == T_RESIDUAL_SCALES;
    bool block_level = id >= T_NORM_GAMMA && id <= T_AD_CONS;
    if (!model_level && !block_level)
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "set_tensor: unknown tensor id %d (banks use set_bank)", id);
    if (block_level && (layer < 0 || (size_t)layer >= m->depth))
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "set_tensor: layer %d outside depth %zu", layer, m->depth);
    size_t want = tensor_len(m, id);
    if (len != want) return fail(ctx, PSSA_B200_ERR_SHAPE, "set_tensor: tensor %d length %zu, expected %zu", id, len, want);
    for (size_t i = 0; i < len; ++i)
        if (!std::isfinite(data[i])) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "set_tensor: non-finite value in tensor %d", id);
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaStream_t st = ctx->stream;
    if (id == T_RESIDUAL_SCALES) {
        m->residual_scales.assign(data, data + len);
        return PSSA_B200_OK;
    }
    if (id == T_EMBED) {
        PSSA_CUDA(ctx, cudaMemcpyAsync(m->embed, data, len * 4, cudaMemcpyHostToDevice, st));
    } else if (id == T_UNEMBED) {
        PSSA_CUDA(ctx, cudaMemcpyAsync(m->unembed, data, len * 4, cudaMemcpyHostToDevice, st));
        m->unembed_dirty = true;
    } else {
        DeviceBlock& b = m->blocks[layer];
        PSSA_CUDA(ctx, cudaMemcpyAsync(b.w[id], data, len * 4, cudaMemcpyHostToDevice, st));
        b.bf16_dirty = true;
        if (id == T_W_PROJ) b.vp_dirty = true;
        if (id == T_A_MAT) {  // refresh_ssm_rates (src/pssa.rs:787-796): A = -softplus(raw), host libm like the reference
            std::vector<float> rates(len);
            for (size_t i = 0; i < len; ++i) rates[i] = -(data[i] > 20.0f ? data[i] : log1pf(expf(data[i])));
            PSSA_CUDA(ctx, cudaMemcpyAsync(b.rates, rates.data(), len * 4, cudaMemcpyHostToDevice, st));
            PSSA_CUDA(ctx, cudaStreamSynchronize(st));
        }
        if (id == T_AD_UP || id == T_AD_CONS) {  // refresh_adapter_up_effective (src/pssa.rs:772-785)
            (id == T_AD_UP ? b.host_up : b.host_cons).assign(data, data + len);
            std::vector<float> eff(len);
            for (size_t i = 0; i < len; ++i) eff[i] = b.host_up[i] + b.host_cons[i];
            PSSA_CUDA(ctx, cudaMemcpyAsync(b.u_eff, eff.data(), len * 4, cudaMemcpyHostToDevice, st));
            PSSA_CUDA(ctx, cudaStreamSynchronize(st));
        }
    }
    PSSA_CUDA(ctx, cudaStreamSynchronize(st));  // `data` may be pageable and reused by the caller
    return PSSA_B200_OK;
}

int32_t pssa_b200_model_get_tensor(pssa_b200_model* m, int32_t layer, int32_t id, float* out, size_t len) {
    if (!m || !out) return mfail(m, PSSA_B200_ERR_INVALID_ARGUMENT, "pssa_b200_model_get_tensor: null argument");
    pssa_b200_ctx* ctx = m->ctx;
    bool model_level = id == T_EMBED || id == T_UNEMBED || id == T_RESIDUAL_SCALES;
    bool block_level = id >= T_NORM_GAMMA && id <= T_AD_CONS;
    if (!model_level && !block_level) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "get_tensor: unknown tensor id %d", id);
    if (block_level && (layer < 0 || (size_t)layer >= m->depth))
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "get_tensor: layer %d outside depth %zu", layer, m->depth);
    size_t want = tensor_len(m, id);
    if (len != want) return fail(ctx, PSSA_B200_ERR_SHAPE, "get_tensor: tensor %d length %zu, expected %zu", id, len, want);
    if (id == T_RESIDUAL_SCALES) {
        for (size_t i = 0; i < len; ++i) out[i] = m->residual_scales[i];
        return PSSA_B200_OK;
    }
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    const float* src = id == T_EMBED ? m->embed : id == T_UNEMBED ? m->unembed : m->blocks[layer].w[id];
    PSSA_CUDA(ctx, cudaMemcpyAsync(out, src, len * 4, cudaMemcpyDeviceToHost, ctx->stream));
    PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return PSSA_B200_OK;
}

int32_t pssa_b200_model_set_bank(pssa_b200_model* m, int32_t layer, const float* keys, const float* norm_sq,
                                 const float* values, uint64_t count, uint64_t write_head, const float* confidence,
                                 const uint64_t* last_seen_step) {
    if (!m || !keys || !norm_sq || !values) return mfail(m, PSSA_B200_ERR_INVALID_ARGUMENT, "pssa_b200_model_set_bank: null argument");
    pssa_b200_ctx* ctx = m->ctx;
    if (layer < 0 || (size_t)layer >= m->depth) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "set_bank: layer %d outside depth %zu", layer, m->depth);
    // src/checkpoint.rs:1060-1066
    if (count > m->cap || write_head >= m->cap || (count < m->cap && write_head != 0))
        return fail(ctx, PSSA_B200_ERR_SHAPE, "memory count/write head invalid");
    for (size_t i = 0; i < count; ++i)  // src/memory.rs:246-250: points must lie inside the open ball
        if (!(norm_sq[i] >= 0.0f && norm_sq[i] < 1.0f))
            return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "Poincare points must be finite and inside the open ball (slot %zu)", i);
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    DeviceBlock& b = m->blocks[layer];
    cudaStream_t st = ctx->stream;
    PSSA_CUDA(ctx, cudaMemcpyAsync(b.w[T_BANK_KEYS], keys, m->cap * m->k * 4, cudaMemcpyHostToDevice, st));
    PSSA_CUDA(ctx, cudaMemcpyAsync(b.w[T_BANK_NORM_SQ], norm_sq, m->cap * 4, cudaMemcpyHostToDevice, st));
    PSSA_CUDA(ctx, cudaMemcpyAsync(b.w[T_BANK_VALUES], values, m->cap * m->d * 4, cudaMemcpyHostToDevice, st));
    b.count = count;
    b.write_head = write_head;
    b.vsplit_dirty = true;
    b.vp_dirty = true;
    b.ksplit_dirty = true;
    if (confidence) b.confidence.assign(confidence, confidence + m->cap);
    if (last_seen_step) b.last_seen.assign(last_seen_step, last_seen_step + m->cap);
    PSSA_CUDA(ctx, cudaStreamSynchronize(st));
    return PSSA_B200_OK;
}

int32_t pssa_b200_model_set_top_k(pssa_b200_model* m, size_t top_k) {
    if (!m) return mfail(m, PSSA_B200_ERR_INVALID_ARGUMENT, "null model");
    m->top_k = top_k;  // 0 = None (full read); the reference rejects Some(0), which has no encoding here
    return PSSA_B200_OK;
}

int32_t pssa_b200_model_set_precision(pssa_b200_model* m, int32_t precision) {
    if (!m) return mfail(m, PSSA_B200_ERR_INVALID_ARGUMENT, "null model");
    if (precision != PSSA_B200_PRECISION_BF16 && precision != PSSA_B200_PRECISION_FP32_EXACT)
        return mfail(m, PSSA_B200_ERR_INVALID_ARGUMENT, "unknown precision");
    m->precision = (uint32_t)precision;
    return PSSA_B200_OK;
}

int32_t pssa_b200_model_set_option(pssa_b200_model* m, int32_t option, int32_t value) {
    if (!m) return mfail(m, PSSA_B200_ERR_INVALID_ARGUMENT, "null model");
    switch (option) {  // messages of src/pssa.rs:2080-2105, 2189-2192, 2232-2243
        case 0:
        case 1:  // enabling is refused on a GPU device; disabling is a no-op (src/pssa.rs:2101-2106)
            if (!value) return PSSA_B200_OK;
            return mfail(m, PSSA_B200_ERR_UNSUPPORTED, "local mixing experiments require CPU single-lane training");
        case 2:
            if (!value) return PSSA_B200_OK;
            return mfail(m, PSSA_B200_ERR_UNSUPPORTED, "hybrid read currently requires the CPU backend");
        case 3: return mfail(m, PSSA_B200_ERR_UNSUPPORTED, "grow memory on the CPU checkpoint before selecting a GPU backend");
        case 4: {  // set_loops (src/pssa.rs:2171-2184): pass 0 keeps its carry, the other passes start from zero
            if (value < 1 || value > 32)
                return mfail(m, PSSA_B200_ERR_INVALID_ARGUMENT, "--loops must be between 1 and 32; use --loops 1 for the original model");
            if ((size_t)value == m->loops) return PSSA_B200_OK;
            pssa_b200_ctx* ctx = m->ctx;
            PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
            PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            const size_t ds = m->d * m->s, nl = (size_t)value, blocks = (size_t)m->max_streams * m->depth;
            float* fresh = nullptr;
            PSSA_CUDA(ctx, cudaMalloc((void**)&fresh, blocks * nl * ds * 4));
            cudaError_t e = cudaMemsetAsync(fresh, 0, blocks * nl * ds * 4, ctx->stream);
            if (e == cudaSuccess)  // [stream][block] rows of `loops` carries: copy the first carry of every row
                e = cudaMemcpy2DAsync(fresh, nl * ds * 4, m->state, m->loops * ds * 4, ds * 4, blocks, cudaMemcpyDeviceToDevice, ctx->stream);
            if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
            if (e != cudaSuccess) {
                cudaFree(fresh);
                return cuda_fail(ctx, e, "resizing the recurrent state for the Ouro passes");
            }
            cudaFree(m->state);
            m->state = fresh;
            m->loops = nl;
            // the extra feature buffer of the passes lives in the activation workspace: rebuild it on the next call
            if (m->ws.base) cudaFree(m->ws.base);
            m->ws = pssa::Workspace();
            m->dev_layout.ws_base = nullptr;
            return PSSA_B200_OK;
        }
        case 5:  // lane groups (not a reference option): 0 = by shape, 1 = one stream, 2..4 = that many groups
            if (value < 0 || value > 4) return mfail(m, PSSA_B200_ERR_INVALID_ARGUMENT, "lane groups must be in 0..4");
            m->lane_groups = (size_t)value;
            return PSSA_B200_OK;
        default: return mfail(m, PSSA_B200_ERR_INVALID_ARGUMENT, "unknown option");
    }
}

int32_t pssa_b200_model_set_max_rows(pssa_b200_model* m, size_t max_rows) {
    if (!m || max_rows == 0) return mfail(m, PSSA_B200_ERR_INVALID_ARGUMENT, "max_rows must be positive");
    m->max_rows = max_rows;
    return PSSA_B200_OK;
}

int32_t pssa_b200_model_reset_state(pssa_b200_model* m, uint32_t stream) {
    if (!m) return mfail(m, PSSA_B200_ERR_INVALID_ARGUMENT, "null model");
    if (stream >= m->max_streams) return fail(m->ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "stream %u outside %u streams", stream, m->max_streams);
    PSSA_CUDA(m->ctx, cudaSetDevice(m->ctx->device));
    size_t n = m->depth * m->loops * m->d * m->s;
    PSSA_CUDA(m->ctx, cudaMemsetAsync(m->state + (size_t)stream * n, 0, n * 4, m->ctx->stream));
    return PSSA_B200_OK;
}

int32_t pssa_b200_model_get_state(pssa_b200_model* m, uint32_t stream, float* out, size_t len) {
    if (!m || !out) return mfail(m, PSSA_B200_ERR_INVALID_ARGUMENT, "null argument");
    size_t n = m->depth * m->loops * m->d * m->s;
    if (stream >= m->max_streams || len != n)
        return fail(m->ctx, PSSA_B200_ERR_SHAPE, "recurrent state: stream %u of %u, length %zu, expected %zu", stream, m->max_streams, len, n);
    PSSA_CUDA(m->ctx, cudaSetDevice(m->ctx->device));
    PSSA_CUDA(m->ctx, cudaMemcpyAsync(out, m->state + (size_t)stream * n, n * 4, cudaMemcpyDeviceToHost, m->ctx->stream));
    PSSA_CUDA(m->ctx, cudaStreamSynchronize(m->ctx->stream));
    return PSSA_B200_OK;
}

int32_t pssa_b200_model_set_state(pssa_b200_model* m, uint32_t stream, const float* data, size_t len) {
    if (!m || !data) return mfail(m, PSSA_B200_ERR_INVALID_ARGUMENT, "null argument");
    size_t n = m->depth * m->loops * m->d * m->s;
    if (stream >= m->max_streams || len != n)
        return fail(m->ctx, PSSA_B200_ERR_SHAPE, "recurrent state: stream %u of %u, length %zu, expected %zu", stream, m->max_streams, len, n);
    PSSA_CUDA(m->ctx, cudaSetDevice(m->ctx->device));
    PSSA_CUDA(m->ctx, cudaMemcpyAsync(m->state + (size_t)stream * n, data, n * 4, cudaMemcpyHostToDevice, m->ctx->stream));
    PSSA_CUDA(m->ctx, cudaStreamSynchronize(m->ctx->stream));
    return PSSA_B200_OK;
}

}  // extern "C"
