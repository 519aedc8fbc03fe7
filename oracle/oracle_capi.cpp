// extern "C" surface of the CPU oracle, bound with ctypes by tests/, the smoke entry and the
// benchmark's CPU-baseline leg. TEST INFRASTRUCTURE ONLY: the shipped library never loads this.
#include <chrono>
#include <cmath>
#include <cstring>
#include <thread>
#include <vector>

#include "pssa_oracle.hpp"

using namespace pssa_oracle;

namespace {
// Tensor numbering shared (by value) with include/pssa_b200.h `pssa_b200_tensor`.
enum TensorId {
    T_EMBED = 0, T_UNEMBED = 1, T_NORM_GAMMA = 2, T_NORM_BETA = 3, T_A_MAT = 4, T_W_DELTA = 5,
    T_W_B = 6, T_W_C = 7, T_W_QX = 8, T_W_QH = 9, T_W_GATE = 10, T_W_PROJ = 11, T_MLP_W1 = 12,
    T_MLP_W2 = 13, T_AD_DOWN = 14, T_AD_UP = 15, T_AD_CONS = 16, T_H_PERSISTENT = 17,
    T_BANK_KEYS = 18, T_BANK_VALUES = 19, T_BANK_NORM_SQ = 20, T_BANK_CONFIDENCE = 21,
    T_RESIDUAL_SCALES = 22,
    // last-token scratch of a block (observer rows, inference.rs:236-313)
    S_X_NORM = 32, S_DELTA = 33, S_B = 34, S_C = 35, S_Y_SSM = 36, S_Q_EUC = 37, S_Q_PNC = 38,
    S_MEM_WEIGHTS = 39, S_M_VAL = 40, S_G_MEM = 41, S_M_PROJ = 42, S_AD_ACT = 43, S_AD_OUT = 44,
    S_Z_RAW = 45, S_MLP_ACT = 46, S_Z_FINAL = 47, S_FEATURES = 48,
};

std::vector<float>* tensor_of(Model* m, int layer, int id) {
    if (id == T_EMBED) return &m->embed;
    if (id == T_UNEMBED) return &m->unembed;
    if (id == T_RESIDUAL_SCALES) return &m->residual_scales;
    if (id == S_FEATURES) return &m->features;
    if (layer < 0 || (size_t)layer >= m->blocks.size()) return nullptr;
    Block& b = m->blocks[layer];
    switch (id) {
        case T_NORM_GAMMA: return &b.norm_gamma;
        case T_NORM_BETA: return &b.norm_beta;
        case T_A_MAT: return &b.a_mat;
        case T_W_DELTA: return &b.w_delta;
        case T_W_B: return &b.w_b;
        case T_W_C: return &b.w_c;
        case T_W_QX: return &b.w_qx;
        case T_W_QH: return &b.w_qh;
        case T_W_GATE: return &b.w_gate;
        case T_W_PROJ: return &b.w_proj;
        case T_MLP_W1: return &b.mlp_w1;
        case T_MLP_W2: return &b.mlp_w2;
        case T_AD_DOWN: return &b.ad_down;
        case T_AD_UP: return &b.ad_up;
        case T_AD_CONS: return &b.ad_cons;
        case T_H_PERSISTENT: return &b.h_persistent;
        case T_BANK_KEYS: return &b.memory.keys;
        case T_BANK_VALUES: return &b.memory.values;
        case T_BANK_NORM_SQ: return &b.memory.norm_sq;
        case T_BANK_CONFIDENCE: return &b.memory.confidence;
        case S_X_NORM: return &b.x_norm;
        case S_DELTA: return &b.delta;
        case S_B: return &b.bp;
        case S_C: return &b.cp;
        case S_Y_SSM: return &b.y_ssm;
        case S_Q_EUC: return &b.q_euc;
        case S_Q_PNC: return &b.q_pnc;
        case S_MEM_WEIGHTS: return &b.mem_weights;
        case S_M_VAL: return &b.m_val;
        case S_G_MEM: return &b.g_mem;
        case S_M_PROJ: return &b.m_proj;
        case S_AD_ACT: return &b.ad_act;
        case S_AD_OUT: return &b.ad_out;
        case S_Z_RAW: return &b.z_raw;
        case S_MLP_ACT: return &b.mlp_act;
        case S_Z_FINAL: return &b.z_final;
        default: return nullptr;
    }
}

template <class F>
void parallel_for(size_t n, int threads, F f) {
    if (threads <= 1 || n <= 1) {
        for (size_t i = 0; i < n; ++i) f(i);
        return;
    }
    size_t nt = std::min<size_t>((size_t)threads, n);
    std::vector<std::thread> pool;
    for (size_t w = 0; w < nt; ++w)
        pool.emplace_back([=] {
            for (size_t i = w; i < n; i += nt) f(i);
        });
    for (auto& t : pool) t.join();
}
}  // namespace

extern "C" {

// dims = depth, d_vocab, d_latent, d_state, d_mem_key, mem_capacity, chunk_len
void* pssa_oracle_model_new(const uint64_t* dims, float tau_mem, uint64_t seed) {
    Config c;
    c.depth = dims[0];
    c.d_vocab = dims[1];
    c.d_latent = dims[2];
    c.d_state = dims[3];
    c.d_mem_key = dims[4];
    c.mem_capacity = dims[5];
    c.chunk_len = dims[6];
    c.tau_mem = tau_mem;
    Model* m = new Model();
    m->init(c, seed);
    return m;
}

void* pssa_oracle_model_load(const uint8_t* bytes, size_t len, char* err, size_t errlen) {
    Model* m = new Model();
    if (!m->load(bytes, len)) {
        if (err && errlen) {
            std::strncpy(err, m->error.c_str(), errlen - 1);
            err[errlen - 1] = 0;
        }
        delete m;
        return nullptr;
    }
    return m;
}

void* pssa_oracle_model_clone(void* h) { return new Model(*(Model*)h); }
void pssa_oracle_model_free(void* h) { delete (Model*)h; }

void pssa_oracle_model_config(void* h, uint64_t* dims, float* tau_mem, uint64_t* step_rng) {
    Model* m = (Model*)h;
    dims[0] = m->cfg.depth;
    dims[1] = m->cfg.d_vocab;
    dims[2] = m->cfg.d_latent;
    dims[3] = m->cfg.d_state;
    dims[4] = m->cfg.d_mem_key;
    dims[5] = m->cfg.mem_capacity;
    dims[6] = m->cfg.chunk_len;
    *tau_mem = m->cfg.tau_mem;
    step_rng[0] = m->step_counter;
    step_rng[1] = m->rng_state;
}

float* pssa_oracle_tensor(void* h, int layer, int id, size_t* len) {
    auto* v = tensor_of((Model*)h, layer, id);
    if (!v) {
        *len = 0;
        return nullptr;
    }
    *len = v->size();
    return v->data();
}

// meta = count, write_head, top_k. set != 0 writes them.
void pssa_oracle_bank_meta(void* h, int layer, uint64_t* meta, int set) {
    Bank& b = ((Model*)h)->blocks[layer].memory;
    if (set) {
        b.count = meta[0];
        b.write_head = meta[1];
        b.top_k = meta[2];
    } else {
        meta[0] = b.count;
        meta[1] = b.write_head;
        meta[2] = b.top_k;
    }
}

uint64_t* pssa_oracle_bank_last_seen(void* h, int layer, size_t* len) {
    Bank& b = ((Model*)h)->blocks[layer].memory;
    *len = b.last_seen_step.size();
    return b.last_seen_step.data();
}

size_t pssa_oracle_bank_insert(void* h, int layer, const float* key, const float* val) {
    return ((Model*)h)->blocks[layer].memory.insert(key, val);
}

long pssa_oracle_bank_insert_protected(void* h, int layer, const float* key, const float* val,
                                       float surprise, uint64_t step) {
    return ((Model*)h)->blocks[layer].memory.insert_protected(key, val, surprise, step);
}

float pssa_oracle_bank_retrieve(void* h, int layer, const float* q_pnc, float tau, float* out_val,
                                float* out_weights, size_t weights_len) {
    return ((Model*)h)->blocks[layer].memory.retrieve_soft_into(q_pnc, tau, out_val, out_weights, weights_len);
}

void pssa_oracle_reset_state(void* h) { ((Model*)h)->reset_recurrent_state(); }
int pssa_oracle_set_loops(void* h, size_t loops) { return ((Model*)h)->set_loops(loops) ? 0 : -1; }
size_t pssa_oracle_state_len(void* h) { return ((Model*)h)->state_len(); }
void pssa_oracle_copy_state_to(void* h, float* out) { ((Model*)h)->copy_state_to(out); }
void pssa_oracle_copy_state_from(void* h, const float* in) { ((Model*)h)->copy_state_from(in); }

int pssa_oracle_forward_inference(void* h, uint64_t id, float* logits) {
    Model* m = (Model*)h;
    if (id >= m->cfg.d_vocab) return -1;
    m->forward_inference((size_t)id, logits);
    return 0;
}

int pssa_oracle_forward_features(void* h, uint64_t id) {
    Model* m = (Model*)h;
    if (id >= m->cfg.d_vocab) return -1;
    m->forward_features((size_t)id);
    return 0;
}

int pssa_oracle_prefill(void* h, const uint64_t* ids, size_t n, float* logits_or_null, size_t* processed) {
    return ((Model*)h)->prefill_inference(ids, n, logits_or_null, processed);
}

float pssa_oracle_chunk_forward(void* h, const uint64_t* ids, const uint64_t* targets, size_t n, float* logits) {
    return ((Model*)h)->chunk_forward(ids, targets, n, logits);
}

// Greedy generation: prefill `n` prompt ids then emit `n_new` tokens (inference.rs:348-418 with
// temperature 0). Returns tokens generated, -1 on error.
long pssa_oracle_generate_greedy(void* h, const uint64_t* ids, size_t n, size_t n_new, uint64_t* out_ids,
                                 float* min_gap) {
    Model* m = (Model*)h;
    std::vector<float> logits(m->cfg.d_vocab);
    if (m->prefill_inference(ids, n, logits.data(), nullptr) != 1) return -1;
    float gap_min = INFINITY;
    for (size_t g = 0; g < n_new; ++g) {
        long tok = greedy_token(logits.data(), m->cfg.d_vocab);
        if (tok < 0) return -1;
        float best = logits[tok], second = -INFINITY;
        for (size_t i = 1; i < m->cfg.d_vocab; ++i)
            if ((long)i != tok && logits[i] > second) second = logits[i];
        gap_min = std::min(gap_min, best - second);
        out_ids[g] = (uint64_t)tok;
        m->forward_inference((size_t)tok, logits.data());
    }
    if (min_gap) *min_gap = gap_min;
    return (long)n_new;
}

// CPU baseline for batched prefill: `n_lanes` independent sequences of `T` tokens (ids [n_lanes, T]) through
// token-serial prefill_inference, lanes spread over `threads` host threads. Every thread works on its own copy of
// the model (the carry is per lane; the weights are duplicated), made before the clock starts. Returns seconds.
double pssa_oracle_prefill_lanes_timed(void* h, const uint64_t* ids, size_t n_lanes, size_t T, int threads, float* last_logits) {
    Model* base = (Model*)h;
    size_t nt = std::max<size_t>(1, std::min<size_t>((size_t)threads, n_lanes));
    std::vector<Model> copies(nt, *base);
    size_t v = base->cfg.d_vocab;
    auto t0 = std::chrono::steady_clock::now();
    std::vector<std::thread> pool;
    for (size_t w = 0; w < nt; ++w)
        pool.emplace_back([&, w] {
            std::vector<float> lg(v);
            for (size_t l = w; l < n_lanes; l += nt) {
                copies[w].reset_recurrent_state();
                copies[w].prefill_inference(ids + l * T, T, lg.data(), nullptr);
                if (last_logits) std::memcpy(last_logits + l * v, lg.data(), v * sizeof(float));
            }
        });
    for (auto& t : pool) t.join();
    return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
}

void pssa_oracle_consolidate(void* h, int layer, float alpha) { ((Model*)h)->blocks[layer].consolidate(alpha); }
void pssa_oracle_dream_replay(void* h, int layer, const float* value) {
    ((Model*)h)->blocks[layer].dream_replay_value(value);
}

// ---- operators -------------------------------------------------------------------------
float pssa_oracle_dot(const float* a, const float* b, size_t len, int kind) {
    if (kind == 1) return dot_slice_avx2_fma(a, b, len);
    if (kind == 2) return dot_slice_portable(a, b, len);
    return dot_slice(a, b, len);
}
float pssa_oracle_softplus(float x) { return softplus(x); }
float pssa_oracle_sigmoid(float x) { return sigmoid(x); }
float pssa_oracle_refractory_gain(uint64_t dt, float tau) { return refractory_gain(dt, tau); }
uint64_t pssa_oracle_fnv1a64(const uint8_t* p, size_t n) { return fnv1a64(p, n); }

void pssa_oracle_rng_fill(uint64_t seed, float low, float high, float* out, size_t n, uint64_t* state_out) {
    SimpleRng rng(seed);
    for (size_t i = 0; i < n; ++i) out[i] = rng.gen_range_f32(low, high);
    if (state_out) *state_out = rng.state;
}

void pssa_oracle_gemm_xwt(const float* x, const float* w, size_t m, size_t n, size_t k, float* out, int threads) {
    parallel_for(m, threads, [=](size_t t) { gemm_xwt(x + t * k, w, 1, n, k, out + t * n); });
}

// in-place exclusive Blelloch scan; arrays hold next_pow2(len) * stride floats
void pssa_oracle_affine_scan(float* a, float* b, size_t len, size_t stride) { affine_scan_in_place(a, b, len, stride); }

// Ordered recurrence h_t = a_t * h_{t-1} + b_t for `lanes` independent [T, stride] problems
// (the scan operator alone; the same mul-then-add as gpu_batch.rs:543-575). h0 may be null (zeros).
void pssa_oracle_scan_states(const float* a, const float* b, const float* h0, float* out, size_t lanes,
                             size_t T, size_t stride, int threads) {
    const size_t block = 256;
    size_t cblocks = (stride + block - 1) / block;
    parallel_for(lanes * cblocks, threads, [=](size_t job) {
        size_t lane = job / cblocks, c0 = (job % cblocks) * block;
        size_t c1 = std::min(stride, c0 + block);
        const float* al = a + lane * T * stride;
        const float* bl = b + lane * T * stride;
        float* ol = out + lane * T * stride;
        float h[256];
        for (size_t c = c0; c < c1; ++c) h[c - c0] = h0 ? h0[lane * stride + c] : 0.0f;
        for (size_t t = 0; t < T; ++t)
            for (size_t c = c0; c < c1; ++c) {
                float v = al[t * stride + c] * h[c - c0] + bl[t * stride + c];
                h[c - c0] = v;
                ol[t * stride + c] = v;
            }
    });
}

// One lane of the SSM stage. states has (len + 1) * d_m * d_s floats, row 0 = carry in.
// mode 0: ordered recurrence (gpu_batch.rs:543-575); mode 1: Blelloch + materialize (622-680).
void pssa_oracle_ssm_forward(const float* delta, const float* b_proj, const float* c_proj, const float* x_norm,
                             const float* rates, float* states, float* y, float* bar_a, float* bar_b, size_t len,
                             size_t d_m, size_t d_s, int mode) {
    if (mode == 1)
        ssm_blelloch(delta, b_proj, c_proj, x_norm, rates, states, y, len, d_m, d_s);
    else
        ssm_sequential(delta, b_proj, c_proj, x_norm, rates, states, y, bar_a, bar_b, len, d_m, d_s);
}

// Lane-batched SSM with only y and the final carry kept (what inference needs). carry [lanes, d*s] in/out.
void pssa_oracle_ssm_lanes(const float* delta, const float* b_proj, const float* c_proj, const float* x_norm,
                           const float* rates, float* carry, float* y, const uint32_t* offsets,
                           const uint32_t* lengths, size_t lanes, size_t d_m, size_t d_s, int threads) {
    parallel_for(lanes, threads, [=](size_t lane) {
        size_t off = offsets[lane], len = lengths[lane], stride = d_m * d_s;
        float* h = carry + lane * stride;
        for (size_t t = 0; t < len; ++t) {
            size_t row = off + t;
            for (size_t i = 0; i < d_m; ++i) {
                float d_i = delta[row * d_m + i], y_i = 0.f;
                for (size_t j = 0; j < d_s; ++j) {
                    size_t idx = i * d_s + j;
                    float a = expf(d_i * rates[idx]);
                    float hv = a * h[idx] + (d_i * b_proj[row * d_s + j]) * x_norm[row * d_m + i];
                    h[idx] = hv;
                    y_i += hv * c_proj[row * d_s + j];
                }
                y[row * d_m + i] = y_i;
            }
        }
    });
}

float pssa_oracle_project(const float* q, float* out, size_t n) { return Bank::diffeomorphic_project(q, out, n); }
float pssa_oracle_squared_norm(const float* p, size_t n) { return Bank::squared_norm(p, n); }
float pssa_oracle_distance(const float* u, float u_sq, const float* v, float v_sq, size_t n) {
    return Bank::poincare_distance(u, u_sq, v, v_sq, n);
}

// Bank read for n queries over a raw bank. q_euc != 0: project first (memory.rs:198-211) and write
// q_pnc_out. weights [n, cap] (rows beyond count left as the reference leaves them: zero-filled here),
// out_val [n, dv], min_dist [n] optional.
void pssa_oracle_memory_read(const float* keys, const float* norm_sq, const float* values, size_t cap,
                             size_t count, size_t dk, size_t dv, size_t top_k, float tau, const float* q,
                             int q_is_euclidean, size_t n, float* q_pnc_out, float* out_val, float* out_weights,
                             float* min_dist, int threads) {
    Bank bank;
    bank.init(cap, dk, dv);
    std::memcpy(bank.keys.data(), keys, cap * dk * 4);
    std::memcpy(bank.values.data(), values, cap * dv * 4);
    std::memcpy(bank.norm_sq.data(), norm_sq, cap * 4);
    bank.count = count;
    bank.top_k = top_k;
    const Bank* bp = &bank;
    parallel_for(n, threads, [=](size_t t) {
        std::vector<float> p(dk);
        if (q_is_euclidean)
            Bank::diffeomorphic_project(q + t * dk, p.data(), dk);
        else
            std::memcpy(p.data(), q + t * dk, dk * 4);
        if (q_pnc_out) std::memcpy(q_pnc_out + t * dk, p.data(), dk * 4);
        std::fill(out_weights + t * cap, out_weights + (t + 1) * cap, 0.f);
        float md = bp->retrieve_soft_into(p.data(), tau, out_val + t * dv, out_weights + t * cap, cap);
        if (min_dist) min_dist[t] = md;
    });
}

// Standalone bank handle for the write-path known-answer tests (memory.rs:268-342).
void* pssa_oracle_bank_new(size_t cap, size_t dk, size_t dv) {
    Bank* b = new Bank();
    b->init(cap, dk, dv);
    return b;
}
void pssa_oracle_bank_free(void* b) { delete (Bank*)b; }
size_t pssa_oracle_rawbank_insert(void* b, const float* key, const float* val) { return ((Bank*)b)->insert(key, val); }
long pssa_oracle_rawbank_insert_protected(void* b, const float* key, const float* val, float surprise, uint64_t step) {
    return ((Bank*)b)->insert_protected(key, val, surprise, step);
}
void pssa_oracle_rawbank_set_top_k(void* b, size_t k) { ((Bank*)b)->top_k = k; }
float pssa_oracle_rawbank_retrieve(void* b, const float* q, float tau, float* out_val, float* out_weights,
                                   size_t weights_len) {
    return ((Bank*)b)->retrieve_soft_into(q, tau, out_val, out_weights, weights_len);
}
// which: 0 keys, 1 values, 2 norm_sq, 3 confidence
float* pssa_oracle_rawbank_array(void* b, int which, size_t* len) {
    Bank* k = (Bank*)b;
    std::vector<float>* v = which == 0 ? &k->keys : which == 1 ? &k->values : which == 2 ? &k->norm_sq : &k->confidence;
    *len = v->size();
    return v->data();
}
void pssa_oracle_rawbank_meta(void* b, uint64_t* meta, uint64_t* last_seen) {
    Bank* k = (Bank*)b;
    meta[0] = k->count;
    meta[1] = k->write_head;
    for (size_t i = 0; i < k->capacity; ++i) last_seen[i] = k->last_seen_step[i];
}
void pssa_oracle_rawbank_set_meta(void* b, uint64_t count, uint64_t head, const float* conf, const uint64_t* last_seen) {
    Bank* k = (Bank*)b;
    k->count = count;
    k->write_head = head;
    for (size_t i = 0; i < k->capacity; ++i) {
        k->confidence[i] = conf[i];
        k->last_seen_step[i] = last_seen[i];
    }
}

// BASELINE config 3's "winning-slot rank-1 write": NOT a reference code path (the reference overwrites the ring
// head, src/memory.rs:315-342). Defined here so the GPU variant has a restatement to be compared with: the gate of
// src/defense.rs:45-67 applied to `slot`; on a successful write values[slot] += eta * (val - values[slot]).
long pssa_oracle_rawbank_plastic_write(void* b, size_t slot, const float* val, float surprise, uint64_t step, float eta) {
    Bank* k = (Bank*)b;
    uint64_t delta_t = step >= k->last_seen_step[slot] ? step - k->last_seen_step[slot] : 0;
    float damage = 0.08f * surprise * refractory_gain(delta_t, 60.0f);
    if (k->confidence[slot] > damage) {
        k->confidence[slot] -= damage;
        k->last_seen_step[slot] = step;
        return -1;
    }
    k->confidence[slot] = 1.0f;
    k->last_seen_step[slot] = step;
    float* v = &k->values[slot * k->dim_val];
    for (size_t i = 0; i < k->dim_val; ++i) v[i] = v[i] + eta * (val[i] - v[i]);
    return (long)slot;
}

long pssa_oracle_greedy(const float* logits, size_t v) { return greedy_token(logits, v); }

// inference.rs:102-181; rng_state is read and written back (one draw when temperature > 0)
long pssa_oracle_sample(uint64_t* rng_state, float temperature, float top_p, size_t top_k, float repetition_penalty,
                        const uint64_t* generated, size_t n_generated, float* logits, size_t v) {
    SimpleRng rng(1);
    rng.state = *rng_state;
    SamplingConfig cfg;
    cfg.temperature = temperature, cfg.top_p = top_p, cfg.top_k = top_k, cfg.repetition_penalty = repetition_penalty;
    long id = sample_token(rng, cfg, generated, n_generated, logits, v);
    *rng_state = rng.state;
    return id;
}

int pssa_oracle_hardware_threads() { return (int)std::thread::hardware_concurrency(); }

}  // extern "C"
