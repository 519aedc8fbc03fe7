// Random initialisation of a model, as the reference's constructor does it on the host and in its exact draw order, so
// that a model created here from a seed has the tensors of `PSSALayerV2::new(cfg, seed)` bit for bit
// (src/pssa.rs:2019-2072: embedding, block 0, head, then the further blocks; src/pssa.rs:630-690: one block;
// src/linalg.rs:1-28: the xorshift64* generator; src/linalg.rs:338-344: Xavier-uniform fill; src/adapter.rs:16-24).
// Host arithmetic on purpose: the timescale table uses libm's exp / expm1 / ln like the reference's std calls, and the
// draws are one sequential generator. The tensors then go through pssa_b200_model_set_tensor like any upload.
#include <cmath>
#include <cstdint>
#include <vector>

#include "context.hpp"
#include "model.hpp"

namespace pssa {
namespace {

struct SimpleRng {  // src/linalg.rs:1-28
    uint64_t state;
    explicit SimpleRng(uint64_t seed) : state(seed == 0 ? 0x853c49e6748fea9bull : seed) {}
    uint32_t next_u32() {
        uint64_t x = state;
        x ^= x >> 12;
        x ^= x << 25;
        x ^= x >> 27;
        state = x;
        return (uint32_t)((x * 0x2545f4914f6cdd1dull) >> 32);
    }
    float gen_range(float low, float high) {
        const float norm = (float)next_u32() / (float)UINT32_MAX;  // u32 -> f32 rounds to nearest, like `as f32`
        return low + norm * (high - low);
    }
};

int32_t xavier(pssa_b200_model* m, int32_t layer, int32_t id, size_t rows, size_t cols, SimpleRng& rng, std::vector<float>& buf) {
    const float limit = std::sqrt(6.0f / (float)(rows + cols));  // src/linalg.rs:338-344
    buf.resize(rows * cols);
    for (float& v : buf) v = rng.gen_range(-limit, limit);
    return pssa_b200_model_set_tensor(m, layer, id, buf.data(), buf.size());
}

int32_t constant(pssa_b200_model* m, int32_t layer, int32_t id, size_t len, float value, std::vector<float>& buf) {
    buf.assign(len, value);
    return pssa_b200_model_set_tensor(m, layer, id, buf.data(), buf.size());
}

int32_t init_block(pssa_b200_model* m, int32_t layer, SimpleRng& rng, std::vector<float>& buf) {  // src/pssa.rs:630-690
    const size_t d = m->d, s = m->s, k = m->k, rank = m->rank;
    int32_t rc;
    if ((rc = constant(m, layer, T_NORM_GAMMA, d, 1.0f, buf))) return rc;
    if ((rc = constant(m, layer, T_NORM_BETA, d, 0.0f, buf))) return rc;
    // timescales spread geometrically over [1.5, 200] steps; stored raw, the physical rate is -softplus(raw)
    buf.resize(d * s);
    const float ln_min = std::log(1.5f), ln_max = std::log(200.0f);
    for (size_t i = 0; i < d; ++i)
        for (size_t j = 0; j < s; ++j) {
            const float ratio = s > 1 ? (float)j / (float)(s - 1) : 0.0f;
            const float tau = std::exp(ln_min + ratio * (ln_max - ln_min));
            const float rate = 1.0f / tau;
            buf[i * s + j] = std::log(std::expm1(rate));
        }
    if ((rc = pssa_b200_model_set_tensor(m, layer, T_A_MAT, buf.data(), buf.size()))) return rc;
    if ((rc = xavier(m, layer, T_W_DELTA, d, d, rng, buf))) return rc;
    if ((rc = xavier(m, layer, T_W_B, s, d, rng, buf))) return rc;
    if ((rc = xavier(m, layer, T_W_C, s, d, rng, buf))) return rc;
    if ((rc = xavier(m, layer, T_W_QX, k, d, rng, buf))) return rc;
    if ((rc = xavier(m, layer, T_W_QH, k, d, rng, buf))) return rc;
    if ((rc = xavier(m, layer, T_W_GATE, d, d, rng, buf))) return rc;
    if ((rc = xavier(m, layer, T_W_PROJ, d, d, rng, buf))) return rc;
    if ((rc = xavier(m, layer, T_AD_DOWN, rank, d, rng, buf))) return rc;  // src/adapter.rs:16-24: up and consolidated start at zero
    if ((rc = constant(m, layer, T_AD_UP, d * rank, 0.0f, buf))) return rc;
    if ((rc = constant(m, layer, T_AD_CONS, d * rank, 0.0f, buf))) return rc;
    if ((rc = xavier(m, layer, T_MLP_W1, 2 * d, d, rng, buf))) return rc;
    return constant(m, layer, T_MLP_W2, d * 2 * d, 0.0f, buf);  // src/pssa.rs:683
}

}  // namespace
}  // namespace pssa

using namespace pssa;

extern "C" int32_t pssa_b200_model_init_random(pssa_b200_model* m, uint64_t seed, uint64_t* rng_state_out) {
    if (!m) return PSSA_B200_ERR_INVALID_ARGUMENT;
    SimpleRng rng(seed);
    std::vector<float> buf;
    int32_t rc;
    if ((rc = xavier(m, 0, T_EMBED, m->v, m->d, rng, buf))) return rc;
    if ((rc = init_block(m, 0, rng, buf))) return rc;
    if ((rc = xavier(m, 0, T_UNEMBED, m->v, m->d, rng, buf))) return rc;
    for (size_t l = 1; l < m->depth; ++l)
        if ((rc = init_block(m, (int32_t)l, rng, buf))) return rc;
    if (m->depth > 1) {
        buf.assign(m->depth - 1, 1.0f / std::sqrt((float)m->depth));
        if ((rc = pssa_b200_model_set_tensor(m, 0, T_RESIDUAL_SCALES, buf.data(), buf.size()))) return rc;
    }
    if (rng_state_out) *rng_state_out = rng.state;  // the generator the reference keeps for later draws
    return PSSA_B200_OK;
}
