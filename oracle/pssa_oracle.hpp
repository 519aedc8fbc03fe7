// CPU restatement of the PSSA inference forward path (reference crate `pssa` 0.5.0).
//
// TEST INFRASTRUCTURE ONLY. This is the parity oracle and the timed CPU baseline.
// Nothing in the shipped library (pssa_b200/, include/) may include, link or call it;
// only tests/, the smoke entry and the benchmark's CPU-baseline leg use it.
//
// Parity pin: the model restated here reproduces, bit for bit, the reference's own
// golden fixtures (see tests/test_oracle_golden.py): every tensor of
// tests/fixtures/depth_one_main85d9d33_initial.pssa (RNG + init + V7 layout) and words
// [0,22) of tests/fixtures/depth_one_main014f617_avx2_observed.bin (loss + 21 logits of
// the fresh-model chunk forward), plus the bank known-answer tests of
// tests/memory_projection.rs and tests/memory_expansion.rs.
//
// Build: g++ -std=c++17 -O2 -mavx2 -mfma -ffp-contract=off -fno-fast-math
// (the dot product replicates the reference's AVX2/FMA kernel with the same intrinsics;
// everything else must NOT be contracted into FMAs, as rustc does not contract).
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace pssa_oracle {

// src/linalg.rs:1-28
struct SimpleRng {
    uint64_t state;
    explicit SimpleRng(uint64_t seed) : state(seed == 0 ? 0x853c49e6748fea9bULL : seed) {}
    uint32_t next_u32();
    float gen_range_f32(float low, float high);
};

// src/linalg.rs:184-298
float dot_slice(const float* a, const float* b, size_t len);           // runtime rule: AVX2 for len==8 or >=16
float dot_slice_avx2_fma(const float* a, const float* b, size_t len);  // linalg.rs:212-279
float dot_slice_portable(const float* a, const float* b, size_t len);  // linalg.rs:282-298
float sigmoid(float x);   // linalg.rs:547-550
float softplus(float x);  // linalg.rs:552-555

// src/pssa.rs:253-331 (PSSAConfigV2)
struct Config {
    size_t depth = 1, d_vocab = 10000, d_latent = 256, d_state = 16, d_mem_key = 32,
           mem_capacity = 512, chunk_len = 64;
    float lr = 1e-3f, beta1 = 0.9f, beta2 = 0.999f, weight_decay = 0.01f, eps = 1e-8f,
          tau_mem = 0.1f, ema_alpha = 0.01f;
};

// src/memory.rs:4-58 (HyperbolicEpisodicBankV2), persistent fields only
struct Bank {
    size_t capacity = 0, count = 0, dim_key = 0, dim_val = 0, write_head = 0;
    size_t top_k = 0;  // 0 = full soft read (memory.rs:17, None)
    std::vector<float> keys, values, norm_sq, confidence;
    std::vector<uint64_t> last_seen_step;
    void init(size_t cap, size_t dk, size_t dv);
    static float squared_norm(const float* p, size_t n);                       // memory.rs:181-192
    static float diffeomorphic_project(const float* q, float* out, size_t n);  // memory.rs:198-211
    static float poincare_distance(const float* u, float u_sq, const float* v, float v_sq,
                                   size_t n);                                  // memory.rs:245-262
    size_t insert(const float* key, const float* val);                         // memory.rs:268-303
    // returns slot or -1 (memory.rs:315-342, defense.rs:45-67)
    long insert_protected(const float* key, const float* val, float surprise, uint64_t step);
    // memory.rs:344-426; weights has >= count entries (capacity in the model)
    float retrieve_soft_into(const float* q_pnc, float tau, float* out_val, float* out_weights,
                             size_t weights_len) const;
};

// src/defense.rs:18-22
float refractory_gain(uint64_t delta_tokens, float tau_refractory);

// One continuous block: persistent parameters and carry (src/pssa.rs:506-620)
struct Block {
    size_t d = 0, s = 0, k = 0, cap = 0, rank = 16;
    float tau = 0.1f;
    std::vector<float> norm_gamma, norm_beta;
    std::vector<float> a_mat, w_delta, w_b, w_c, w_qx, w_qh, w_gate, w_proj, mlp_w1, mlp_w2;
    std::vector<float> ad_down, ad_up, ad_cons;
    std::vector<float> h_persistent;
    // carries of the Ouro passes 1..loops-1 (pass 0 owns h_persistent): [(loops-1)][d*s], the tail of the reference's
    // tape.h_states (pssa.rs:934-951)
    std::vector<float> loop_carry;
    Bank memory;
    // derived: A = -softplus(raw) (pssa.rs:787-796)
    std::vector<float> rates;
    // last-token scratch (pssa.rs:600-618), published for observers
    std::vector<float> x_norm, delta, bp, cp, y_ssm, q_euc, q_pnc, mem_weights, m_val, g_mem,
        m_proj, ad_act, ad_out, z_raw, mlp_act, mlp_out, z_final;
    void init_shapes(const Config& c);
    void init_random(const Config& c, SimpleRng& rng);  // pssa.rs:630-770
    void refresh_rates();
    // pssa.rs:1072-1209: one token, carry updated in place
    void forward_token(const float* x_features, float* z_out);
    // pssa.rs:1065-1069: one Ouro pass = the same token step on that pass's own carry
    void forward_loop(const float* x_features, float* z_out, size_t loop_index);
    void consolidate(float alpha);                      // adapter.rs:65-72
    void dream_replay_value(const float* target);       // pssa.rs:1814-1832 (uses last ad_act/ad_out)
};

// src/pssa.rs:1931-2075
struct Model {
    Config cfg;
    uint64_t step_counter = 0;
    uint64_t rng_state = 0;
    std::vector<float> embed, unembed;
    std::vector<Block> blocks;
    std::vector<float> residual_scales;
    std::vector<float> features, block_out, continuous_input;
    size_t loops = 1;  // runtime Ouro pass count (pssa.rs:2171-2184); not part of the checkpoint
    std::string error;
    void init(const Config& c, uint64_t seed);                  // pssa.rs:2019-2072
    bool load(const uint8_t* bytes, size_t len);                // checkpoint.rs V7 / V8
    void reset_recurrent_state();                               // pssa.rs:2245-2250
    // pssa.rs:2171-2184 + resize_loop_tape 2147-2167: pass 0 keeps its carry, the other passes start from zero
    bool set_loops(size_t n);
    void forward_features(size_t id);                           // pssa.rs:2312-2377 (single pass and Ouro passes)
    void logits(float* out) const;                              // pssa.rs:2379-2385
    void forward_inference(size_t id, float* logits_out);       // pssa.rs:2387-2391
    // pssa.rs:2399-2442. returns 1 ok, 0 cancelled (never here), -1 error; *processed = tokens advanced
    int prefill_inference(const uint64_t* ids, size_t n, float* logits_or_null, size_t* processed);
    // token-serial training-style forward over one chunk (pssa.rs:2597-2750): fills logits[T*V], returns loss
    float chunk_forward(const uint64_t* ids, const uint64_t* targets, size_t n, float* logits_out);
    size_t state_len() const { return cfg.depth * loops * cfg.d_latent * cfg.d_state; }  // pssa.rs:2255-2261
    void copy_state_to(float* out) const;     // pssa.rs:2263-2286: [block][pass][d*s]
    void copy_state_from(const float* in);    // pssa.rs:2288-2310
};

// src/gpu_batch.rs:84-164
void affine_scan_in_place(float* scan_a, float* scan_b, size_t len, size_t stride);
// src/gpu_batch.rs:392-437
void materialize_ssm_scan(const float* initial, const float* local_a, const float* local_b,
                          const float* x_norm, const float* scan_a, const float* scan_b,
                          const float* c_proj, float* states_out, float* y_out, size_t len,
                          size_t d_m, size_t d_s);
// src/gpu_batch.rs:543-575: ordered recurrence; states has (len+1) rows, row 0 = initial
void ssm_sequential(const float* delta, const float* b_proj, const float* c_proj,
                    const float* x_norm, const float* rates, float* states, float* y, float* bar_a,
                    float* bar_b, size_t len, size_t d_m, size_t d_s);
// src/gpu_batch.rs:622-680: Blelloch form of the same stage
void ssm_blelloch(const float* delta, const float* b_proj, const float* c_proj,
                  const float* x_norm, const float* rates, float* states, float* y, size_t len,
                  size_t d_m, size_t d_s);
// src/backend.rs:832-871 (each output = dot_slice(x_row, w_row))
void gemm_xwt(const float* x, const float* w, size_t m, size_t n, size_t k, float* out);
// inference.rs:123-127: argmax over ids 1..V, ties to the lowest id; -1 on non-finite logits
long greedy_token(const float* logits, size_t v);
// src/inference.rs:102-181 (`sample`): repetition penalty over the last 64 generated ids, temperature softmax over ids
// 1..V-1, candidates sorted by (probability desc, id asc), top-k, top-p, one SimpleRng draw. `logits` is modified by
// the penalty exactly like the reference's slice. Returns the id, or -1 non-finite logits, -2 invalid probability mass,
// -3 no candidates.
struct SamplingConfig {
    float temperature = 0.8f, top_p = 0.95f, repetition_penalty = 1.1f;
    size_t top_k = 40;
};
long sample_token(SimpleRng& rng, const SamplingConfig& cfg, const uint64_t* generated, size_t n_generated, float* logits, size_t v);

uint64_t fnv1a64(const uint8_t* bytes, size_t len);  // checkpoint.rs:89-95

}  // namespace pssa_oracle
