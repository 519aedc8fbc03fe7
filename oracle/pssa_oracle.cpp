// CPU restatement of the PSSA inference forward path. TEST INFRASTRUCTURE ONLY:
// parity oracle + timed CPU baseline; never linked into or called from the shipped library.
// Each function cites the reference file:line it follows. See pssa_oracle.hpp for the pin.
#include "pssa_oracle.hpp"

#include <immintrin.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <queue>
#include <utility>

namespace pssa_oracle {

// ---------------------------------------------------------------- linalg.rs
uint32_t SimpleRng::next_u32() {  // linalg.rs:13-20 (xorshift64*)
    uint64_t x = state;
    x ^= x >> 12;
    x ^= x << 25;
    x ^= x >> 27;
    state = x;
    return (uint32_t)((x * 0x2545f4914f6cdd1dULL) >> 32);
}

float SimpleRng::gen_range_f32(float low, float high) {  // linalg.rs:23-26
    float norm = (float)next_u32() / (float)UINT32_MAX;
    return low + norm * (high - low);
}

float dot_slice_avx2_fma(const float* a, const float* b, size_t len) {  // linalg.rs:212-279
    size_t i = 0;
    __m256 acc0 = _mm256_setzero_ps(), acc1 = _mm256_setzero_ps(), acc2 = _mm256_setzero_ps(),
           acc3 = _mm256_setzero_ps();
    while (i + 32 <= len) {
        acc0 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i), acc0);
        acc1 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i + 8), _mm256_loadu_ps(b + i + 8), acc1);
        acc2 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i + 16), _mm256_loadu_ps(b + i + 16), acc2);
        acc3 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i + 24), _mm256_loadu_ps(b + i + 24), acc3);
        i += 32;
    }
    while (i + 8 <= len) {
        acc0 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i), acc0);
        i += 8;
    }
    __m256 pair01 = _mm256_add_ps(acc0, acc1);
    __m256 pair23 = _mm256_add_ps(acc2, acc3);
    __m256 lanes = _mm256_add_ps(pair01, pair23);
    __m128 folded = _mm_add_ps(_mm256_castps256_ps128(lanes), _mm256_extractf128_ps(lanes, 1));
    __m128 pair = _mm_hadd_ps(folded, folded);
    float sum = _mm_cvtss_f32(_mm_hadd_ps(pair, pair));
    while (i < len) {
        sum += a[i] * b[i];
        i += 1;
    }
    return sum;
}

float dot_slice_portable(const float* a, const float* b, size_t len) {  // linalg.rs:282-298
    size_t i = 0;
    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
    while (i + 4 <= len) {
        acc0 += a[i] * b[i];
        acc1 += a[i + 1] * b[i + 1];
        acc2 += a[i + 2] * b[i + 2];
        acc3 += a[i + 3] * b[i + 3];
        i += 4;
    }
    float sum = (acc0 + acc1) + (acc2 + acc3);
    while (i < len) {
        sum += a[i] * b[i];
        i += 1;
    }
    return sum;
}

float dot_slice(const float* a, const float* b, size_t len) {  // linalg.rs:184-199
    if (len == 8 || len >= 16) return dot_slice_avx2_fma(a, b, len);
    return dot_slice_portable(a, b, len);
}

float sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }            // linalg.rs:547-550
float softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }    // linalg.rs:552-555

static void matvec(const float* w, size_t rows, size_t cols, const float* x, float* out) {
    for (size_t r = 0; r < rows; ++r) out[r] = dot_slice(w + r * cols, x, cols);  // pssa.rs:109-116
}

void gemm_xwt(const float* x, const float* w, size_t m, size_t n, size_t k, float* out) {
    for (size_t t = 0; t < m; ++t)  // backend.rs:832-871: every entry is one dot_slice
        for (size_t j = 0; j < n; ++j) out[t * n + j] = dot_slice(x + t * k, w + j * k, k);
}

// ---------------------------------------------------------------- defense.rs
float refractory_gain(uint64_t delta_tokens, float tau_refractory) {  // defense.rs:18-22
    float dt = (float)delta_tokens;
    float linear = 1.0f - expf(-dt / tau_refractory);
    return std::max(linear * linear, 0.005f);
}

// ---------------------------------------------------------------- memory.rs
void Bank::init(size_t cap, size_t dk, size_t dv) {  // memory.rs:35-58
    capacity = cap;
    count = 0;
    dim_key = dk;
    dim_val = dv;
    write_head = 0;
    top_k = 0;
    keys.assign(cap * dk, 0.f);
    values.assign(cap * dv, 0.f);
    norm_sq.assign(cap, 0.f);
    confidence.assign(cap, 1.f);
    last_seen_step.assign(cap, 0);
}

static double squared_norm_f64(const float* p, size_t n) {  // memory.rs:190-192
    double acc = 0.0;
    for (size_t i = 0; i < n; ++i) acc += (double)p[i] * (double)p[i];
    return acc;
}

float Bank::squared_norm(const float* p, size_t n) {  // memory.rs:181-188
    double norm = squared_norm_f64(p, n);
    if (norm < 1.0 && (float)norm == 1.0f) return std::nextafterf(1.0f, 0.0f);
    return (float)norm;
}

float Bank::diffeomorphic_project(const float* q, float* out, size_t n) {  // memory.rs:198-211
    const double max_radius = 1.0 - 8.0 * (double)std::numeric_limits<float>::epsilon();
    double r = std::sqrt(squared_norm_f64(q, n));
    double scale = (r == 0.0) ? 1.0 : std::min(r / (1.0 + r), max_radius) / r;
    for (size_t i = 0; i < n; ++i) out[i] = (float)((double)q[i] * scale);
    return (float)std::min(r, (double)std::numeric_limits<float>::max());
}

// Rust std f64::asinh: ln_1p(ax + ax / (hypot(1, 1/ax) + 1/ax)) with the sign copied back.
static double rust_asinh(double x) {
    double ax = std::fabs(x);
    double ix = 1.0 / ax;
    return std::copysign(std::log1p(ax + (ax / (std::hypot(1.0, ix) + ix))), x);
}

float Bank::poincare_distance(const float* u, float u_sq, const float* v, float v_sq, size_t n) {
    double sq = 0.0;  // memory.rs:245-262
    for (size_t i = 0; i < n; ++i) {
        double d = (double)u[i] - (double)v[i];
        sq += d * d;
    }
    double denom = (1.0 - (double)u_sq) * (1.0 - (double)v_sq);
    return (float)(2.0 * rust_asinh(std::sqrt(sq / denom)));
}

size_t Bank::insert(const float* key, const float* val) {  // memory.rs:268-303 (no value cap)
    float key_sq = squared_norm(key, dim_key);
    size_t idx;
    if (count < capacity) {
        idx = count++;
    } else {
        idx = write_head;
        write_head = (write_head + 1) % capacity;
    }
    std::memcpy(&keys[idx * dim_key], key, dim_key * sizeof(float));
    norm_sq[idx] = key_sq;
    std::memcpy(&values[idx * dim_val], val, dim_val * sizeof(float));
    confidence[idx] = 1.0f;
    last_seen_step[idx] = 0;
    return idx;
}

long Bank::insert_protected(const float* key, const float* val, float surprise, uint64_t step) {
    if (count < capacity) {  // memory.rs:315-342
        size_t idx = insert(key, val);
        last_seen_step[idx] = step;
        return (long)idx;
    }
    size_t idx = write_head;
    // defense.rs:45-67 apply_refractory_overwrite
    uint64_t delta_t = step >= last_seen_step[idx] ? step - last_seen_step[idx] : 0;
    float damage = 0.08f * surprise * refractory_gain(delta_t, 60.0f);
    if (confidence[idx] > damage) {
        confidence[idx] -= damage;
        last_seen_step[idx] = step;
        return -1;
    }
    confidence[idx] = 1.0f;
    last_seen_step[idx] = step;
    size_t inserted = insert(key, val);
    last_seen_step[inserted] = step;
    return (long)inserted;
}

float Bank::retrieve_soft_into(const float* q_pnc, float tau, float* out_val, float* out_weights,
                               size_t weights_len) const {  // memory.rs:344-426
    float q_sq = squared_norm(q_pnc, dim_key);
    if (count == 0) {
        std::fill(out_val, out_val + dim_val, 0.f);
        std::fill(out_weights, out_weights + weights_len, 0.f);
        return 0.0f;
    }
    float min_dist = std::numeric_limits<float>::max();
    for (size_t idx = 0; idx < count; ++idx) {
        float dist = poincare_distance(q_pnc, q_sq, &keys[idx * dim_key], norm_sq[idx], dim_key);
        min_dist = std::min(min_dist, dist);
        out_weights[idx] = dist;
    }
    if (top_k != 0 && top_k < count) {  // memory.rs:380-408
        // keep the k smallest (distance bits, slot); a max-heap pops the largest pair
        std::priority_queue<std::pair<uint32_t, size_t>> nearest;
        for (size_t idx = 0; idx < count; ++idx) {
            uint32_t bits;
            std::memcpy(&bits, &out_weights[idx], 4);
            nearest.push({bits, idx});
            if (nearest.size() > top_k) nearest.pop();
        }
        std::vector<std::pair<size_t, uint32_t>> selected;
        while (!nearest.empty()) {
            selected.push_back({nearest.top().second, nearest.top().first});
            nearest.pop();
        }
        std::sort(selected.begin(), selected.end());
        std::fill(out_weights, out_weights + weights_len, 0.f);
        float sum = 0.f;
        for (auto& e : selected) {
            float d;
            std::memcpy(&d, &e.second, 4);
            sum += expf((min_dist - d) / tau);
        }
        std::fill(out_val, out_val + dim_val, 0.f);
        for (auto& e : selected) {
            float d;
            std::memcpy(&d, &e.second, 4);
            float weight = expf((min_dist - d) / tau) / sum;
            out_weights[e.first] = weight;
            const float* v = &values[e.first * dim_val];
            for (size_t j = 0; j < dim_val; ++j) out_val[j] += weight * v[j];
        }
        return min_dist;
    }
    float sum = 0.f;
    for (size_t idx = 0; idx < count; ++idx) {
        float w = expf((min_dist - out_weights[idx]) / tau);
        out_weights[idx] = w;
        sum += w;
    }
    std::fill(out_val, out_val + dim_val, 0.f);
    for (size_t idx = 0; idx < count; ++idx) {
        float w = out_weights[idx] / sum;
        out_weights[idx] = w;
        const float* v = &values[idx * dim_val];
        for (size_t j = 0; j < dim_val; ++j) out_val[j] += w * v[j];
    }
    return min_dist;
}

// ---------------------------------------------------------------- pssa.rs: block
static void xavier(std::vector<float>& out, size_t rows, size_t cols, SimpleRng& rng) {
    float limit = std::sqrt(6.0f / (float)(rows + cols));  // pssa.rs:86-101
    out.resize(rows * cols);
    for (auto& x : out) x = rng.gen_range_f32(-limit, limit);
}

void Block::init_shapes(const Config& c) {
    d = c.d_latent;
    s = c.d_state;
    k = c.d_mem_key;
    cap = c.mem_capacity;
    tau = c.tau_mem;
    rank = 16;
    norm_gamma.assign(d, 1.f);
    norm_beta.assign(d, 0.f);
    a_mat.assign(d * s, 0.f);
    w_delta.assign(d * d, 0.f);
    w_b.assign(s * d, 0.f);
    w_c.assign(s * d, 0.f);
    w_qx.assign(k * d, 0.f);
    w_qh.assign(k * d, 0.f);
    w_gate.assign(d * d, 0.f);
    w_proj.assign(d * d, 0.f);
    mlp_w1.assign(2 * d * d, 0.f);
    mlp_w2.assign(d * 2 * d, 0.f);
    ad_down.assign(rank * d, 0.f);
    ad_up.assign(d * rank, 0.f);
    ad_cons.assign(d * rank, 0.f);
    h_persistent.assign(d * s, 0.f);
    memory.init(cap, k, d);
    rates.assign(d * s, 0.f);
    x_norm.assign(d, 0.f);
    delta.assign(d, 0.f);
    bp.assign(s, 0.f);
    cp.assign(s, 0.f);
    y_ssm.assign(d, 0.f);
    q_euc.assign(k, 0.f);
    q_pnc.assign(k, 0.f);
    mem_weights.assign(cap, 0.f);
    m_val.assign(d, 0.f);
    g_mem.assign(d, 0.f);
    m_proj.assign(d, 0.f);
    ad_act.assign(rank, 0.f);
    ad_out.assign(d, 0.f);
    z_raw.assign(d, 0.f);
    mlp_act.assign(2 * d, 0.f);
    mlp_out.assign(d, 0.f);
    z_final.assign(d, 0.f);
}

void Block::init_random(const Config& c, SimpleRng& rng) {  // pssa.rs:630-690
    init_shapes(c);
    float ln_min = logf(1.5f), ln_max = logf(200.0f);
    for (size_t i = 0; i < d; ++i)
        for (size_t j = 0; j < s; ++j) {  // pssa.rs:649-665
            float ratio = s > 1 ? (float)j / (float)(s - 1) : 0.0f;
            float tau_j = expf(ln_min + ratio * (ln_max - ln_min));
            float rate = 1.0f / tau_j;
            a_mat[i * s + j] = logf(expm1f(rate));
        }
    xavier(w_delta, d, d, rng);
    xavier(w_b, s, d, rng);
    xavier(w_c, s, d, rng);
    xavier(w_qx, k, d, rng);
    xavier(w_qh, k, d, rng);
    xavier(w_gate, d, d, rng);
    xavier(w_proj, d, d, rng);
    xavier(ad_down, rank, d, rng);  // adapter.rs:16-24
    xavier(mlp_w1, 2 * d, d, rng);
    // mlp_w2, adapter up/consolidated stay zero (pssa.rs:683, adapter.rs:19-20)
}

void Block::refresh_rates() {  // pssa.rs:787-796
    for (size_t i = 0; i < a_mat.size(); ++i) rates[i] = -softplus(a_mat[i]);
}

void Block::forward_token(const float* e_t, float* z_out) {  // pssa.rs:1072-1209
    refresh_rates();
    float sum_sq = 0.f;
    for (size_t i = 0; i < d; ++i) sum_sq += e_t[i] * e_t[i];
    float inv_rms = 1.0f / std::sqrt(sum_sq / (float)d + 1e-5f);
    for (size_t i = 0; i < d; ++i) x_norm[i] = norm_gamma[i] * (e_t[i] * inv_rms) + norm_beta[i];
    matvec(w_delta.data(), d, d, x_norm.data(), delta.data());
    for (size_t i = 0; i < d; ++i) delta[i] = softplus(delta[i]);
    matvec(w_b.data(), s, d, x_norm.data(), bp.data());
    matvec(w_c.data(), s, d, x_norm.data(), cp.data());
    float ssm_scale = 1.0f / std::sqrt((float)s);
    for (size_t i = 0; i < d; ++i) {  // pssa.rs:1131-1144
        float d_i = delta[i];
        float y_i = 0.f;
        for (size_t j = 0; j < s; ++j) {
            size_t idx = i * s + j;
            float bar_a = expf(d_i * rates[idx]);
            float bar_b = d_i * bp[j];
            float h_val = bar_a * h_persistent[idx] + bar_b * x_norm[i];
            h_persistent[idx] = h_val;
            y_i += h_val * cp[j];
        }
        y_ssm[i] = y_i;
    }
    for (size_t r = 0; r < k; ++r)  // pssa.rs:1147-1152
        q_euc[r] = dot_slice(&w_qx[r * d], x_norm.data(), d) + dot_slice(&w_qh[r * d], y_ssm.data(), d);
    Bank::diffeomorphic_project(q_euc.data(), q_pnc.data(), k);
    memory.retrieve_soft_into(q_pnc.data(), tau, m_val.data(), mem_weights.data(), cap);
    matvec(w_gate.data(), d, d, x_norm.data(), g_mem.data());
    for (size_t i = 0; i < d; ++i) g_mem[i] = sigmoid(g_mem[i]);
    matvec(w_proj.data(), d, d, m_val.data(), m_proj.data());
    matvec(ad_down.data(), rank, d, x_norm.data(), ad_act.data());  // pssa.rs:1179-1186
    for (size_t r = 0; r < rank; ++r) ad_act[r] = ad_act[r] * sigmoid(ad_act[r]);
    for (size_t i = 0; i < d; ++i) {  // adapter.rs:37-48
        float total = 0.f;
        for (size_t r = 0; r < rank; ++r) total += (ad_up[i * rank + r] + ad_cons[i * rank + r]) * ad_act[r];
        ad_out[i] = total;
    }
    for (size_t i = 0; i < d; ++i) z_raw[i] = (y_ssm[i] * ssm_scale) + (g_mem[i] * m_proj[i]) + ad_out[i];
    matvec(mlp_w1.data(), 2 * d, d, z_raw.data(), mlp_act.data());
    for (size_t i = 0; i < 2 * d; ++i) mlp_act[i] = mlp_act[i] * sigmoid(mlp_act[i]);
    matvec(mlp_w2.data(), d, 2 * d, mlp_act.data(), mlp_out.data());
    for (size_t i = 0; i < d; ++i) z_final[i] = z_raw[i] + mlp_out[i];
    std::memcpy(z_out, z_final.data(), d * sizeof(float));
}

void Block::consolidate(float alpha) {  // adapter.rs:65-72
    for (size_t i = 0; i < ad_up.size(); ++i) {
        float fast = ad_up[i];
        ad_cons[i] += alpha * fast;
        ad_up[i] = (1.0f - alpha) * fast;
    }
}

void Block::dream_replay_value(const float* value) {  // pssa.rs:1814-1832
    std::vector<float> out(d);
    forward_token(value, out.data());
    double tn = 0.0;
    for (size_t i = 0; i < d; ++i) tn += (double)value[i] * (double)value[i];
    tn = std::sqrt(tn);
    float rate = 0.02f / (1.0f + (float)std::min(tn, (double)std::numeric_limits<float>::max()));
    for (size_t i = 0; i < d; ++i) {
        float error = std::min(std::max(value[i] - ad_out[i], -4.0f), 4.0f);
        for (size_t r = 0; r < rank; ++r) ad_up[i * rank + r] += rate * error * ad_act[r];
    }
}

// ---------------------------------------------------------------- pssa.rs: model
void Model::init(const Config& c, uint64_t seed) {  // pssa.rs:2019-2072
    cfg = c;
    SimpleRng rng(seed);
    xavier(embed, c.d_vocab, c.d_latent, rng);
    blocks.assign(c.depth, Block());
    blocks[0].init_random(c, rng);
    xavier(unembed, c.d_vocab, c.d_latent, rng);
    for (size_t l = 1; l < c.depth; ++l) blocks[l].init_random(c, rng);
    residual_scales.assign(c.depth - 1, 1.0f / std::sqrt((float)c.depth));
    features.assign(c.d_latent, 0.f);
    block_out.assign(c.d_latent, 0.f);
    rng_state = rng.state;
    step_counter = 0;
}

void Model::reset_recurrent_state() {  // pssa.rs:798-804, 2245-2250
    for (auto& b : blocks) {
        std::fill(b.h_persistent.begin(), b.h_persistent.end(), 0.f);
        std::fill(b.loop_carry.begin(), b.loop_carry.end(), 0.f);
    }
}

bool Model::set_loops(size_t n) {  // pssa.rs:2171-2184
    if (n < 1 || n > 32) {
        error = "--loops must be between 1 and 32; use --loops 1 for the original model";
        return false;
    }
    if (n != loops) {
        loops = n;
        // resize_loop_tape (pssa.rs:2147-2167) builds a fresh tape: the carries of passes >= 1 start from zero
        for (auto& b : blocks) b.loop_carry.assign((n - 1) * b.h_persistent.size(), 0.f);
    }
    return true;
}

void Block::forward_loop(const float* x_features, float* z_out, size_t loop_index) {  // pssa.rs:1065-1069, 940-951
    const size_t hs = h_persistent.size();
    if (loop_index != 0) std::swap_ranges(h_persistent.begin(), h_persistent.end(), loop_carry.begin() + (loop_index - 1) * hs);
    forward_token(x_features, z_out);
    if (loop_index != 0) std::swap_ranges(h_persistent.begin(), h_persistent.end(), loop_carry.begin() + (loop_index - 1) * hs);
}

void Model::copy_state_to(float* out) const {  // pssa.rs:2263-2286
    const size_t hs = cfg.d_latent * cfg.d_state;
    for (size_t l = 0; l < blocks.size(); ++l) {
        float* dst = out + l * loops * hs;
        std::copy(blocks[l].h_persistent.begin(), blocks[l].h_persistent.end(), dst);
        if (loops > 1) std::copy(blocks[l].loop_carry.begin(), blocks[l].loop_carry.end(), dst + hs);
    }
}

void Model::copy_state_from(const float* in) {  // pssa.rs:2288-2310
    const size_t hs = cfg.d_latent * cfg.d_state;
    for (size_t l = 0; l < blocks.size(); ++l) {
        const float* src = in + l * loops * hs;
        std::copy(src, src + hs, blocks[l].h_persistent.begin());
        if (loops > 1) std::copy(src + hs, src + loops * hs, blocks[l].loop_carry.begin());
    }
}

void Model::forward_features(size_t id) {  // pssa.rs:2312-2377
    size_t d = cfg.d_latent;
    if (loops == 1) {
        blocks[0].forward_token(&embed[id * d], features.data());
        for (size_t l = 1; l < blocks.size(); ++l) {
            blocks[l].forward_token(features.data(), block_out.data());
            float scale = residual_scales[l - 1];
            for (size_t i = 0; i < d; ++i) features[i] += scale * block_out[i];
        }
        return;
    }
    // Ouro passes (pssa.rs:2338-2376): the block is applied `loops` times with shared weights and one carry per pass,
    // every pass adding its output / loops to the features it read
    std::copy(&embed[id * d], &embed[id * d] + d, features.begin());
    const float loop_scale = 1.0f / (float)loops;
    for (size_t li = 0; li < loops; ++li) {
        blocks[0].forward_loop(features.data(), block_out.data(), li);
        for (size_t i = 0; i < d; ++i) features[i] += loop_scale * block_out[i];
    }
    continuous_input.resize(d);
    for (size_t l = 1; l < blocks.size(); ++l) {
        const float scale = residual_scales[l - 1];
        std::copy(features.begin(), features.end(), continuous_input.begin());
        for (size_t li = 0; li < loops; ++li) {
            blocks[l].forward_loop(features.data(), block_out.data(), li);
            for (size_t i = 0; i < d; ++i) features[i] += loop_scale * block_out[i];
        }
        for (size_t i = 0; i < d; ++i) features[i] = continuous_input[i] + scale * features[i];
    }
}

void Model::logits(float* out) const {  // pssa.rs:2379-2385
    size_t d = cfg.d_latent;
    matvec(unembed.data(), cfg.d_vocab, d, features.data(), out);
    float scale = 1.0f / std::sqrt((float)d);
    for (size_t i = 0; i < cfg.d_vocab; ++i) out[i] *= scale;
}

void Model::forward_inference(size_t id, float* logits_out) {
    forward_features(id);
    logits(logits_out);
}

int Model::prefill_inference(const uint64_t* ids, size_t n, float* logits_or_null, size_t* processed) {
    // pssa.rs:2399-2442. The 32-token projection tiles keep every dot's reduction order, so the
    // token loop below is bit-identical to the tiled form (inference.rs:1069-1113 asserts that).
    if (processed) *processed = 0;
    if (n == 0) {
        error = "prefill requires at least one token";
        return -1;
    }
    for (size_t i = 0; i < n; ++i) {
        if (ids[i] >= cfg.d_vocab) {
            error = "prompt ID " + std::to_string(ids[i]) + " outside model vocabulary";
            return -1;
        }
        forward_features((size_t)ids[i]);
        if (processed) *processed = i + 1;
    }
    if (logits_or_null) logits(logits_or_null);
    return 1;
}

float Model::chunk_forward(const uint64_t* ids, const uint64_t* targets, size_t n, float* logits_out) {
    // pssa.rs:2597-2750 with loops == 1: token-serial blocks, then head + cross entropy per row.
    size_t d = cfg.d_latent, v = cfg.d_vocab;
    std::vector<float> acts(n * d), next(n * d), z(d);
    if (loops > 1) {
        // Ouro passes: the reference proves its chunk forward equal to token inference (tests/stacked_depth.rs:296-317,
        // src/inference.rs:1069-1113 at loops 3), so the rows are the token-serial features
        for (size_t t = 0; t < n; ++t) {
            forward_features((size_t)ids[t]);
            std::copy(features.begin(), features.end(), &acts[t * d]);
        }
    } else
        for (size_t t = 0; t < n; ++t) blocks[0].forward_token(&embed[ids[t] * d], &acts[t * d]);
    for (size_t l = 1; loops == 1 && l < blocks.size(); ++l) {
        float scale = residual_scales[l - 1];
        for (size_t t = 0; t < n; ++t) {
            blocks[l].forward_token(&acts[t * d], z.data());
            for (size_t i = 0; i < d; ++i) next[t * d + i] = acts[t * d + i] + scale * z[i];
        }
        acts.swap(next);
    }
    float logit_scale = 1.0f / std::sqrt((float)d);
    float total = 0.f;
    for (size_t t = 0; t < n; ++t) {
        float* row = logits_out + t * v;
        matvec(unembed.data(), v, d, &acts[t * d], row);
        for (size_t i = 0; i < v; ++i) row[i] *= logit_scale;
        float max_l = -std::numeric_limits<float>::infinity();
        for (size_t i = 0; i < v; ++i)
            if (row[i] > max_l) max_l = row[i];
        float sum_exp = 0.f;
        for (size_t i = 0; i < v; ++i) sum_exp += expf(row[i] - max_l);
        float loss = (max_l - row[targets[t]]) + logf(sum_exp);
        total += loss;
    }
    return total / (float)n;
}

long greedy_token(const float* logits, size_t v) {  // inference.rs:111-127
    for (size_t i = 0; i < v; ++i)
        if (!std::isfinite(logits[i])) return -1;
    if (v < 2) return -1;
    size_t best = 1;
    for (size_t i = 2; i < v; ++i) {
        // total_cmp: -0.0 orders below +0.0; ties keep the lowest id
        float a = logits[i], b = logits[best];
        bool greater = a > b || (a == b && std::signbit(b) && !std::signbit(a));
        if (greater) best = i;
    }
    return (long)best;
}

// ---------------------------------------------------------------- gpu_batch.rs scan twin
void affine_scan_in_place(float* a, float* b, size_t len, size_t stride) {  // gpu_batch.rs:98-164
    size_t width = 1;
    while (width < len) width <<= 1;
    for (size_t i = len * stride; i < width * stride; ++i) {
        a[i] = 1.0f;
        b[i] = 0.0f;
    }
    for (size_t step = 1; step < width; step *= 2) {  // up-sweep
        size_t chunk = 2 * step * stride;
        for (size_t base = 0; base < width * stride; base += chunk) {
            float* ac = a + base;
            float* bc = b + base;
            size_t left = (step - 1) * stride, right = (2 * step - 1) * stride;
            for (size_t j = 0; j < stride; ++j) {
                // compose_affine(first = left, second = right), gpu_batch.rs:84-86
                float na = ac[right + j] * ac[left + j];
                float nb = ac[right + j] * bc[left + j] + bc[right + j];
                ac[right + j] = na;
                bc[right + j] = nb;
            }
        }
    }
    for (size_t j = 0; j < stride; ++j) {
        a[(width - 1) * stride + j] = 1.0f;
        b[(width - 1) * stride + j] = 0.0f;
    }
    for (size_t step = width / 2; step > 0; step /= 2) {  // down-sweep
        size_t chunk = 2 * step * stride;
        for (size_t base = 0; base < width * stride; base += chunk) {
            float* ac = a + base;
            float* bc = b + base;
            size_t left = (step - 1) * stride, right = (2 * step - 1) * stride;
            for (size_t j = 0; j < stride; ++j) {
                float pa = ac[right + j], pb = bc[right + j];
                float la = ac[left + j], lb = bc[left + j];
                ac[left + j] = pa;
                bc[left + j] = pb;
                // compose_affine(first = parent, second = left)
                ac[right + j] = la * pa;
                bc[right + j] = la * pb + lb;
            }
        }
    }
}

void materialize_ssm_scan(const float* initial, const float* local_a, const float* local_b,
                          const float* x_norm, const float* scan_a, const float* scan_b,
                          const float* c_proj, float* states_out, float* y_out, size_t len,
                          size_t d_m, size_t d_s) {  // gpu_batch.rs:392-437
    size_t stride = d_m * d_s;
    for (size_t t = 0; t < len; ++t) {
        size_t off = t * stride;
        for (size_t i = 0; i < d_m; ++i) {
            float y_i = 0.f;
            for (size_t j = 0; j < d_s; ++j) {
                size_t idx = i * d_s + j;
                float h_before = scan_a[off + idx] * initial[idx] + scan_b[off + idx];
                float h = local_a[off + idx] * h_before + local_b[off + idx] * x_norm[t * d_m + i];
                states_out[off + idx] = h;
                y_i += h * c_proj[t * d_s + j];
            }
            y_out[t * d_m + i] = y_i;
        }
    }
}

void ssm_sequential(const float* delta, const float* b_proj, const float* c_proj,
                    const float* x_norm, const float* rates, float* states, float* y, float* bar_a,
                    float* bar_b, size_t len, size_t d_m, size_t d_s) {  // gpu_batch.rs:543-575
    size_t stride = d_m * d_s;
    for (size_t t = 0; t < len; ++t) {
        const float* hp = states + t * stride;
        float* hn = states + (t + 1) * stride;
        for (size_t i = 0; i < d_m; ++i) {
            float d_i = delta[t * d_m + i];
            float y_i = 0.f;
            for (size_t j = 0; j < d_s; ++j) {
                size_t idx = i * d_s + j;
                float a = expf(d_i * rates[idx]);
                float bb = d_i * b_proj[t * d_s + j];
                if (bar_a) bar_a[t * stride + idx] = a;
                if (bar_b) bar_b[t * stride + idx] = bb;
                float h = a * hp[idx] + bb * x_norm[t * d_m + i];
                hn[idx] = h;
                y_i += h * c_proj[t * d_s + j];
            }
            y[t * d_m + i] = y_i;
        }
    }
}

void ssm_blelloch(const float* delta, const float* b_proj, const float* c_proj,
                  const float* x_norm, const float* rates, float* states, float* y, size_t len,
                  size_t d_m, size_t d_s) {  // gpu_batch.rs:622-680
    size_t stride = d_m * d_s;
    size_t width = 1;
    while (width < len) width <<= 1;
    std::vector<float> bar_a(len * stride), bar_b(len * stride), scan_a(width * stride),
        scan_b(width * stride);
    for (size_t t = 0; t < len; ++t)
        for (size_t i = 0; i < d_m; ++i) {
            float d_i = delta[t * d_m + i];
            for (size_t j = 0; j < d_s; ++j) {
                size_t idx = i * d_s + j;
                float a = expf(d_i * rates[idx]);
                float bb = d_i * b_proj[t * d_s + j];
                bar_a[t * stride + idx] = a;
                bar_b[t * stride + idx] = bb;
                scan_a[t * stride + idx] = a;
                scan_b[t * stride + idx] = bb * x_norm[t * d_m + i];
            }
        }
    affine_scan_in_place(scan_a.data(), scan_b.data(), len, stride);
    materialize_ssm_scan(states, bar_a.data(), bar_b.data(), x_norm, scan_a.data(), scan_b.data(),
                         c_proj, states + stride, y, len, d_m, d_s);
}

long sample_token(SimpleRng& rng, const SamplingConfig& cfg, const uint64_t* generated, size_t n_generated, float* logits,
                  size_t v) {  // inference.rs:102-181
    for (size_t i = 0; i < v; ++i)
        if (!std::isfinite(logits[i])) return -1;
    if (cfg.repetition_penalty > 1.0f) {  // inference.rs:114-122: repeats in the window are penalised repeatedly
        size_t start = n_generated > 64 ? n_generated - 64 : 0;
        for (size_t g = start; g < n_generated; ++g) {
            size_t id = (size_t)generated[g];
            if (logits[id] > 0.0f)
                logits[id] /= cfg.repetition_penalty;
            else
                logits[id] *= cfg.repetition_penalty;
        }
    }
    if (cfg.temperature == 0.0f) return greedy_token(logits, v);
    if (v < 2) return -3;
    float mx = -INFINITY;  // id 0 (<unk>) is not a candidate and must not anchor the softmax (inference.rs:128-136)
    for (size_t i = 1; i < v; ++i) mx = std::max(mx, logits[i]);
    std::vector<float> probs(v, 0.0f);
    float sum = 0.0f;
    for (size_t i = 1; i < v; ++i) {
        probs[i] = expf((logits[i] - mx) / cfg.temperature);  // subtract before dividing (inference.rs:139-143)
        sum += probs[i];
    }
    if (!std::isfinite(sum) || sum <= 0.0f) return -2;
    std::vector<std::pair<size_t, float>> cand;
    cand.reserve(v);
    for (size_t i = 1; i < v; ++i)
        if (std::isfinite(probs[i])) cand.emplace_back(i, probs[i] / sum);
    if (cand.empty()) return -3;
    // probabilities are >= +0, so total_cmp is the ordinary order; ties go to the lower id (inference.rs:156)
    std::sort(cand.begin(), cand.end(), [](const auto& a, const auto& b) { return a.second > b.second || (a.second == b.second && a.first < b.first); });
    size_t k = std::min(cand.size(), cfg.top_k), cutoff = k;
    float cumulative = 0.0f;
    for (size_t i = 0; i < k; ++i) {
        cumulative += cand[i].second;
        if (cumulative >= cfg.top_p) {
            cutoff = i + 1;
            break;
        }
    }
    size_t n = std::max<size_t>(cutoff, 1);
    float mass = 0.0f;
    for (size_t i = 0; i < n; ++i) mass += cand[i].second;
    float draw = rng.gen_range_f32(0.0f, mass);
    float running = 0.0f;
    size_t id = cand[n - 1].first;
    for (size_t i = 0; i < n; ++i) {
        running += cand[i].second;
        if (draw <= running) {
            id = cand[i].first;
            break;
        }
    }
    return (long)id;
}

// ---------------------------------------------------------------- checkpoint.rs reader
uint64_t fnv1a64(const uint8_t* bytes, size_t len) {  // checkpoint.rs:89-95
    uint64_t h = 0xcbf29ce484222325ULL;
    for (size_t i = 0; i < len; ++i) h = (h ^ bytes[i]) * 0x00000100000001b3ULL;
    return h;
}

namespace {
struct Reader {  // checkpoint.rs:520-600
    const uint8_t* p;
    size_t len, off = 0;
    bool ok = true;
    std::string err;
    bool take(size_t n, const char* what) {
        if (!ok) return false;
        if (n > len - off) {
            ok = false;
            err = std::string("truncated while reading ") + what;
            return false;
        }
        return true;
    }
    uint64_t u64(const char* what) {
        if (!take(8, what)) return 0;
        uint64_t v;
        std::memcpy(&v, p + off, 8);
        off += 8;
        return v;
    }
    float f32(const char* what) {
        if (!take(4, what)) return 0;
        float v;
        std::memcpy(&v, p + off, 4);
        off += 4;
        if (!std::isfinite(v)) {
            ok = false;
            err = std::string("non-finite ") + what;
        }
        return v;
    }
    void floats(std::vector<float>& out, const char* what, bool nonneg = false) {
        uint64_t n = u64(what);
        if (!ok) return;
        if (n != out.size()) {
            ok = false;
            err = std::string(what) + " length " + std::to_string(n) + ", expected " + std::to_string(out.size());
            return;
        }
        if (!take(n * 4, what)) return;
        std::memcpy(out.data(), p + off, n * 4);
        off += n * 4;
        for (float x : out)
            if (!std::isfinite(x) || (nonneg && x < 0.f)) {
                ok = false;
                err = std::string("non-finite or negative ") + what;
                return;
            }
    }
    void skip_floats(size_t expect, const char* what) {
        std::vector<float> tmp(expect);
        floats(tmp, what);
    }
    void u64s(std::vector<uint64_t>& out, const char* what) {
        uint64_t n = u64(what);
        if (!ok) return;
        if (n != out.size()) {
            ok = false;
            err = std::string(what) + " length mismatch";
            return;
        }
        if (!take(n * 8, what)) return;
        std::memcpy(out.data(), p + off, n * 8);
        off += n * 8;
    }
    // a parameter is stored as data, grad, m, v (checkpoint.rs:613-657); only data is kept
    void param(std::vector<float>& out, const char* what) {
        floats(out, what);
        skip_floats(out.size(), what);
        skip_floats(out.size(), what);
        skip_floats(out.size(), what);
    }
};

void read_block(Reader& r, Block& b, bool with_embed_slot, std::vector<float>* embed,
                std::vector<float>* unembed) {
    // V7 order (checkpoint.rs:912-956): embed, block matrices, unembed, vectors, carry, bank, adapter.
    // V8 block order (checkpoint.rs:979-1010): the same without the shared endpoints.
    if (with_embed_slot) r.param(*embed, "embed_w");
    r.param(b.a_mat, "a_mat_raw");
    r.param(b.w_delta, "w_delta");
    r.param(b.w_b, "w_b");
    r.param(b.w_c, "w_c");
    r.param(b.w_qx, "w_qx");
    r.param(b.w_qh, "w_qh");
    r.param(b.w_gate, "w_gate");
    r.param(b.w_proj, "w_proj");
    r.param(b.mlp_w1, "mlp_w1");
    r.param(b.mlp_w2, "mlp_w2");
    if (with_embed_slot) r.param(*unembed, "unembed_w");
    r.param(b.norm_gamma, "norm_gamma");
    r.param(b.norm_beta, "norm_beta");
    r.floats(b.h_persistent, "h_persistent");
    b.memory.count = r.u64("memory count");
    b.memory.write_head = r.u64("memory write_head");
    if (r.ok && (b.memory.count > b.memory.capacity || b.memory.write_head >= b.memory.capacity)) {
        r.ok = false;
        r.err = "memory count/write head invalid";
    }
    r.floats(b.memory.keys, "memory keys");
    r.floats(b.memory.values, "memory values");
    r.floats(b.memory.norm_sq, "memory norm_sq", true);
    r.floats(b.memory.confidence, "memory confidence", true);
    r.u64s(b.memory.last_seen_step, "memory last_seen_step");
    r.param(b.ad_down, "adapter.down");
    r.param(b.ad_up, "adapter.up");
    r.floats(b.ad_cons, "adapter.consolidated_up");
}
}  // namespace

bool Model::load(const uint8_t* bytes, size_t len) {  // checkpoint.rs:1-27, 1116-1126, 1344-1411
    error.clear();
    if (len < 22 || std::memcmp(bytes, "PSSA", 4) != 0) {
        error = "not a PSSA container";
        return false;
    }
    uint16_t version;
    uint64_t payload_len, checksum;
    std::memcpy(&version, bytes + 4, 2);
    std::memcpy(&payload_len, bytes + 6, 8);
    std::memcpy(&checksum, bytes + 14, 8);
    if (version != 7 && version != 8 && version != 6) {
        error = "unsupported checkpoint version " + std::to_string(version);
        return false;
    }
    if (payload_len != len - 22) {
        error = "payload length mismatch";
        return false;
    }
    if (fnv1a64(bytes + 22, payload_len) != checksum) {
        error = "checksum mismatch";
        return false;
    }
    Reader r{bytes + 22, (size_t)payload_len, 0, true, {}};
    Config c;
    c.d_vocab = r.u64("d_vocab");
    c.d_latent = r.u64("d_latent");
    c.d_state = r.u64("d_state");
    c.d_mem_key = r.u64("d_mem_key");
    c.mem_capacity = r.u64("mem_capacity");
    c.chunk_len = r.u64("chunk_len");
    c.lr = r.f32("lr");
    c.beta1 = r.f32("beta1");
    c.beta2 = r.f32("beta2");
    c.weight_decay = r.f32("weight_decay");
    c.eps = r.f32("eps");
    c.tau_mem = r.f32("tau_mem");
    c.ema_alpha = r.f32("ema_alpha");
    c.depth = 1;
    if (version == 8) c.depth = r.u64("depth");
    if (!r.ok || c.depth < 1 || c.depth > 32 || c.d_vocab == 0 || c.d_latent == 0 || c.d_state == 0 ||
        c.d_mem_key == 0 || c.mem_capacity == 0 || !(c.tau_mem > 0.f) ||
        c.d_vocab * c.d_latent > (1ull << 31)) {
        error = r.ok ? "invalid configuration" : r.err;
        return false;
    }
    cfg = c;
    residual_scales.assign(c.depth - 1, 0.f);
    if (version == 8) r.floats(residual_scales, "residual scales");
    step_counter = r.u64("step_counter");
    rng_state = r.u64("rng state");
    uint64_t nvocab = r.u64("vocabulary count");
    if (r.ok && nvocab != 0 && nvocab != c.d_vocab) {
        error = "vocabulary count must be zero or d_vocab";
        return false;
    }
    for (uint64_t i = 0; r.ok && i < nvocab; ++i) {
        uint64_t l = r.u64("vocabulary token length");
        if (r.take(l, "vocabulary token")) r.off += l;
    }
    embed.assign(c.d_vocab * c.d_latent, 0.f);
    unembed.assign(c.d_vocab * c.d_latent, 0.f);
    blocks.assign(c.depth, Block());
    for (auto& b : blocks) b.init_shapes(c);
    features.assign(c.d_latent, 0.f);
    block_out.assign(c.d_latent, 0.f);
    if (version == 8) {
        r.param(embed, "embed_w");
        r.param(unembed, "unembed_w");
        for (auto& b : blocks) read_block(r, b, false, nullptr, nullptr);
    } else {
        read_block(r, blocks[0], true, &embed, &unembed);
    }
    std::vector<uint64_t> marks(c.d_vocab);
    r.u64s(marks, "embed_row_marks");
    // tokenizer JSON + optional schedule words (checkpoint.rs:1309-1342) are metadata: skipped
    if (!r.ok) {
        error = r.err;
        return false;
    }
    return true;
}

}  // namespace pssa_oracle
