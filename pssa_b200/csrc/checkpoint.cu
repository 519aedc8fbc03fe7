// `.pssa` checkpoint containers (versions 7 and 8, and the single-block version 6 layout they extend) straight into a
// device-resident model: the reference's `load_checkpoint` (src/checkpoint.rs:1344-1411) reduced to what inference needs.
//
// Container (src/checkpoint.rs:1-27): "PSSA", u16 version, u64 payload length, u64 FNV-1a of the payload, payload.
// Payload: configuration words, [v8: depth, residual scales], step counter, RNG state, vocabulary strings, parameters,
// per-block carry / bank / adapter, embedding row marks, tokenizer metadata. A parameter is stored as four equal-length
// f32 arrays (data, grad, Adam m, Adam v; src/checkpoint.rs:613-657); only `data` is uploaded. Everything is validated
// on the host before the first device call, so a rejected file never leaves a half-built model behind.
#include <cmath>
#include <cstring>
#include <string>
#include <vector>

#include "context.hpp"
#include "model.hpp"

namespace pssa {
namespace {

uint64_t fnv1a(const unsigned char* p, size_t n) {  // src/checkpoint.rs:89-95
    uint64_t h = 0xcbf29ce484222325ull;
    for (size_t i = 0; i < n; ++i) h = (h ^ p[i]) * 0x100000001b3ull;
    return h;
}

// Cursor over the payload; the first failure sticks and names the field.
struct Cursor {
    const unsigned char* base;
    size_t len, pos = 0;
    std::string error;

    bool fail_at(const std::string& what) {
        if (error.empty()) error = what;
        return false;
    }
    bool need(size_t n, const char* what) {
        if (!error.empty()) return false;
        if (n > len - pos) return fail_at(std::string("truncated while reading ") + what);
        return true;
    }
    uint64_t word(const char* what) {
        uint64_t v = 0;
        if (need(8, what)) std::memcpy(&v, base + pos, 8), pos += 8;
        return v;
    }
    float scalar(const char* what) {
        float v = 0.0f;
        if (need(4, what)) {
            std::memcpy(&v, base + pos, 4), pos += 4;
            if (!std::isfinite(v)) fail_at(std::string("non-finite ") + what);
        }
        return v;
    }
    // length-prefixed f32 array of exactly `expect` elements
    bool floats(std::vector<float>* out, size_t expect, const char* what, bool non_negative = false) {
        uint64_t n = word(what);
        if (!error.empty()) return false;
        if (n != expect) return fail_at(std::string(what) + " has " + std::to_string(n) + " elements, expected " + std::to_string(expect));
        if (!need(n * 4, what)) return false;
        if (out) {
            out->resize(n);
            std::memcpy(out->data(), base + pos, n * 4);
            for (float x : *out)
                if (!std::isfinite(x) || (non_negative && x < 0.0f)) return fail_at(std::string("non-finite or negative value in ") + what);
        }
        pos += n * 4;
        return true;
    }
    bool words(std::vector<uint64_t>* out, size_t expect, const char* what) {
        uint64_t n = word(what);
        if (!error.empty()) return false;
        if (n != expect) return fail_at(std::string(what) + " has " + std::to_string(n) + " elements, expected " + std::to_string(expect));
        if (!need(n * 8, what)) return false;
        if (out) {
            out->resize(n);
            std::memcpy(out->data(), base + pos, n * 8);
        }
        pos += n * 8;
        return true;
    }
    bool param(std::vector<float>* out, size_t expect, const char* what) {  // data, then grad / m / v skipped
        return floats(out, expect, what) && floats(nullptr, expect, what) && floats(nullptr, expect, what) && floats(nullptr, expect, what);
    }
};

struct HostBlock {
    std::vector<float> t[T_COUNT];
    std::vector<float> carry, keys, values, norm_sq, confidence;
    std::vector<uint64_t> last_seen;
    uint64_t count = 0, write_head = 0;
};

struct Parsed {
    pssa_b200_config cfg{};
    uint32_t version = 0;
    uint64_t step_counter = 0, rng_state = 0;
    std::vector<float> embed, unembed, residual_scales;
    std::vector<HostBlock> blocks;
};

// block record: V7 carries the shared endpoints inside block 0 (src/checkpoint.rs:912-956), V8 does not (979-1010)
bool read_block(Cursor& c, const pssa_b200_config& g, HostBlock& b, std::vector<float>* embed, std::vector<float>* unembed) {
    const size_t d = g.d_latent, s = g.d_state, k = g.d_mem_key, cap = g.mem_capacity, v = g.d_vocab, r = 16;
    if (embed) c.param(embed, v * d, "embed_w");
    c.param(&b.t[T_A_MAT], d * s, "a_mat_raw");
    c.param(&b.t[T_W_DELTA], d * d, "w_delta");
    c.param(&b.t[T_W_B], s * d, "w_b");
    c.param(&b.t[T_W_C], s * d, "w_c");
    c.param(&b.t[T_W_QX], k * d, "w_qx");
    c.param(&b.t[T_W_QH], k * d, "w_qh");
    c.param(&b.t[T_W_GATE], d * d, "w_gate");
    c.param(&b.t[T_W_PROJ], d * d, "w_proj");
    c.param(&b.t[T_MLP_W1], 2 * d * d, "mlp_w1");
    c.param(&b.t[T_MLP_W2], 2 * d * d, "mlp_w2");
    if (unembed) c.param(unembed, v * d, "unembed_w");
    c.param(&b.t[T_NORM_GAMMA], d, "norm_gamma");
    c.param(&b.t[T_NORM_BETA], d, "norm_beta");
    c.floats(&b.carry, d * s, "h_persistent");
    b.count = c.word("memory count");
    b.write_head = c.word("memory write_head");
    if (c.error.empty() && (b.count > cap || b.write_head >= cap)) c.fail_at("memory count / write head outside the bank");
    c.floats(&b.keys, cap * k, "memory keys");
    c.floats(&b.values, cap * d, "memory values");
    c.floats(&b.norm_sq, cap, "memory norm_sq", true);
    c.floats(&b.confidence, cap, "memory confidence", true);
    c.words(&b.last_seen, cap, "memory last_seen_step");
    c.param(&b.t[T_AD_DOWN], r * d, "adapter.down");
    c.param(&b.t[T_AD_UP], d * r, "adapter.up");
    c.floats(&b.t[T_AD_CONS], d * r, "adapter.consolidated_up");
    return c.error.empty();
}

// Host-only: container checks, configuration, and (when `full`) every tensor.
bool parse(const unsigned char* bytes, size_t len, bool full, Parsed& out, std::string& error) {
    if (!bytes || len < 22 || std::memcmp(bytes, "PSSA", 4) != 0) return error = "not a PSSA container", false;
    uint16_t version;
    uint64_t payload_len, checksum;
    std::memcpy(&version, bytes + 4, 2);
    std::memcpy(&payload_len, bytes + 6, 8);
    std::memcpy(&checksum, bytes + 14, 8);
    if (version < 6 || version > 8) return error = "unsupported checkpoint version " + std::to_string(version), false;
    if (payload_len != len - 22) return error = "payload length does not match the file", false;
    if (fnv1a(bytes + 22, payload_len) != checksum) return error = "checksum mismatch", false;
    Cursor c{bytes + 22, (size_t)payload_len};
    pssa_b200_config& g = out.cfg;
    g.d_vocab = c.word("d_vocab"), g.d_latent = c.word("d_latent"), g.d_state = c.word("d_state");
    g.d_mem_key = c.word("d_mem_key"), g.mem_capacity = c.word("mem_capacity");
    c.word("chunk_len");
    for (const char* name : {"lr", "beta1", "beta2", "weight_decay", "eps"}) c.scalar(name);
    g.tau_mem = c.scalar("tau_mem");
    c.scalar("ema_alpha");
    g.depth = version == 8 ? c.word("depth") : 1;
    if (!c.error.empty()) return error = c.error, false;
    if (g.depth < 1 || g.depth > 32 || !g.d_vocab || !g.d_latent || !g.d_state || !g.d_mem_key || !g.mem_capacity || !(g.tau_mem > 0.0f) ||
        g.d_vocab * g.d_latent > (1ull << 31) || g.d_latent * g.d_state > (1ull << 31) || g.mem_capacity * g.d_latent > (1ull << 31))
        return error = "invalid configuration", false;
    out.version = version;
    if (!full) return true;
    if (version == 8) c.floats(&out.residual_scales, g.depth - 1, "residual scales");
    out.step_counter = c.word("step_counter");
    out.rng_state = c.word("rng state");
    const uint64_t n_vocab = c.word("vocabulary count");
    if (c.error.empty() && n_vocab != 0 && n_vocab != g.d_vocab) return error = "vocabulary count must be zero or d_vocab", false;
    for (uint64_t i = 0; c.error.empty() && i < n_vocab; ++i) {
        const uint64_t n = c.word("vocabulary token length");
        if (c.need(n, "vocabulary token")) c.pos += n;
    }
    out.blocks.resize(g.depth);
    if (version == 8) {
        c.param(&out.embed, g.d_vocab * g.d_latent, "embed_w");
        c.param(&out.unembed, g.d_vocab * g.d_latent, "unembed_w");
        for (auto& b : out.blocks)
            if (!read_block(c, g, b, nullptr, nullptr)) break;
    } else {
        read_block(c, g, out.blocks[0], &out.embed, &out.unembed);
    }
    c.words(nullptr, g.d_vocab, "embed_row_marks");
    // tokenizer JSON and schedule words follow (src/checkpoint.rs:1309-1342): metadata, not needed here
    if (!c.error.empty()) return error = c.error, false;
    return true;
}

}  // namespace
}  // namespace pssa

using namespace pssa;

extern "C" {

int32_t pssa_b200_checkpoint_probe(const void* bytes, size_t len, pssa_b200_config* config, uint32_t* version, char* error, size_t error_len) {
    Parsed p;
    std::string err;
    const bool ok = parse((const unsigned char*)bytes, len, false, p, err);
    if (error && error_len) {
        std::strncpy(error, err.c_str(), error_len - 1);
        error[error_len - 1] = 0;
    }
    if (!ok) return PSSA_B200_ERR_INVALID_ARGUMENT;
    if (config) *config = p.cfg;
    if (version) *version = p.version;
    return PSSA_B200_OK;
}

int32_t pssa_b200_model_load_checkpoint(pssa_b200_ctx* ctx, const void* bytes, size_t len, uint32_t max_streams, pssa_b200_model** out) {
    if (!ctx || !out) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "load_checkpoint: null argument");
    *out = nullptr;
    Parsed p;
    std::string err;
    if (!parse((const unsigned char*)bytes, len, true, p, err)) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "invalid checkpoint: %s", err.c_str());
    pssa_b200_model* m = nullptr;
    int32_t rc = pssa_b200_model_create(ctx, &p.cfg, max_streams ? max_streams : 1, &m);
    if (rc != PSSA_B200_OK) return rc;
    auto put = [&](int layer, int id, const std::vector<float>& v) {
        if (rc == PSSA_B200_OK) rc = pssa_b200_model_set_tensor(m, layer, id, v.data(), v.size());
    };
    put(-1, T_EMBED, p.embed);
    put(-1, T_UNEMBED, p.unembed);
    if (p.version == 8 && p.cfg.depth > 1) put(-1, T_RESIDUAL_SCALES, p.residual_scales);
    std::vector<float> carry;
    for (size_t l = 0; l < p.blocks.size() && rc == PSSA_B200_OK; ++l) {
        const HostBlock& b = p.blocks[l];
        for (int id : {T_NORM_GAMMA, T_NORM_BETA, T_A_MAT, T_W_DELTA, T_W_B, T_W_C, T_W_QX, T_W_QH, T_W_GATE, T_W_PROJ, T_MLP_W1, T_MLP_W2,
                       T_AD_DOWN, T_AD_UP, T_AD_CONS})
            put((int)l, id, b.t[id]);
        if (rc == PSSA_B200_OK)
            rc = pssa_b200_model_set_bank(m, (int32_t)l, b.keys.data(), b.norm_sq.data(), b.values.data(), b.count, b.write_head,
                                          b.confidence.data(), b.last_seen.data());
        carry.insert(carry.end(), b.carry.begin(), b.carry.end());
    }
    // the stored carry is stream 0's recurrent state, blocks in order (src/pssa.rs:2255-2310)
    if (rc == PSSA_B200_OK) rc = pssa_b200_model_set_state(m, 0, carry.data(), carry.size());
    if (rc != PSSA_B200_OK) {
        std::string keep = ctx->error;
        pssa_b200_model_destroy(m);
        ctx->error = keep;
        return rc;
    }
    *out = m;
    return PSSA_B200_OK;
}

}  // extern "C"
