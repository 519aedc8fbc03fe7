// Device-resident PSSA model: weights, banks, per-stream recurrent carries and the activation workspace.
// Mirrors the persistent part of `PSSALayerV2` / `PSSAContinuousBlockV2` (src/pssa.rs:506-620, 1931-1966).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "context.hpp"

namespace pssa {

// index = pssa_b200_tensor value (include/pssa_b200.h)
enum TensorId : int {
    T_EMBED = 0, T_UNEMBED = 1, T_NORM_GAMMA = 2, T_NORM_BETA = 3, T_A_MAT = 4, T_W_DELTA = 5, T_W_B = 6, T_W_C = 7,
    T_W_QX = 8, T_W_QH = 9, T_W_GATE = 10, T_W_PROJ = 11, T_MLP_W1 = 12, T_MLP_W2 = 13, T_AD_DOWN = 14, T_AD_UP = 15,
    T_AD_CONS = 16, T_H_PERSISTENT = 17, T_BANK_KEYS = 18, T_BANK_VALUES = 19, T_BANK_NORM_SQ = 20,
    T_BANK_CONFIDENCE = 21, T_RESIDUAL_SCALES = 22, T_COUNT = 23,
};

struct DeviceBlock {
    float* w[T_COUNT] = {};  // fp32 masters (only block-level ids are used)
    float* rates = nullptr;  // A = -softplus(raw)               [d, s]
    float* u_eff = nullptr;  // adapter up: fast + consolidated   [d, rank]
    std::vector<float> host_up, host_cons;
    // bank metadata kept on the host (src/memory.rs:4-33)
    uint64_t count = 0, write_head = 0;
    std::vector<float> confidence;
    std::vector<uint64_t> last_seen;
    // bf16 copies for the tensor-core path
    void* wcat_bf16 = nullptr;  // [ncat, d] rows: W_delta | W_B | W_C | W_qx | W_gate | adapter down
    void* wqh_bf16 = nullptr;
    void* wproj_bf16 = nullptr;
    // MLP matrices with the adapter block appended as 64 extra K columns: [2d, d + 64] = W1 | W1*U | 0 and
    // [d, 2d + 64] = W2 | U | 0 (U = effective adapter up weights); w1u is the fp32 [2d, 16] product W1*U
    void* w1cat_bf16 = nullptr;
    void* w2cat_bf16 = nullptr;
    float* w1u = nullptr;
    void* vsplit_bf16 = nullptr;  // bank values transposed, three bf16 pieces [d, 3*cap] (tensor-core value read)
    void* ksplit_bf16 = nullptr;  // bank keys as three bf16 pieces [cap, 3*k] and (|k|^2, 1/(1-|k|^2)) per slot
    float2* kstat = nullptr;      //   (tensor-core distances); rebuilt together with vsplit_bf16
    // bf16 mode: W_proj (sum_s w_s v_s) = sum_s w_s (W_proj v_s), so the bank's values are carried through the memory
    // projection once per upload: vp = V W_proj^T [cap, d] fp32, vpsplit_bf16 = its transpose as bf16 pieces [d, 3*cap]
    // (the layout of vsplit_bf16; the read uses the leading piece). The all-slots read then yields W_proj m directly.
    float* vp = nullptr;
    void* vpsplit_bf16 = nullptr;
    bool bf16_dirty = true;
    bool vsplit_dirty = true;
    bool vp_dirty = true;
    bool ksplit_dirty = true;
};

struct Workspace {
    size_t rows = 0, lanes = 0;
    uint32_t *ids = nullptr, *lane_off = nullptr, *lane_len = nullptr, *lane_slot = nullptr, *last_rows = nullptr,
             *greedy = nullptr;
    float* feat_c = nullptr;  // Ouro passes only: a block's input features, kept for its depth residual
    float *feat_a = nullptr, *feat_b = nullptr, *x_norm = nullptr, *proj = nullptr, *y = nullptr, *weights = nullptr,
          *m_val = nullptr, *m_proj = nullptr, *z = nullptr, *mlp_act = nullptr, *last_feat = nullptr, *logits = nullptr;
    void *x_bf16 = nullptr, *y_bf16 = nullptr, *m_bf16 = nullptr, *z_bf16 = nullptr, *act_bf16 = nullptr, *w_split = nullptr;
    void* q_split = nullptr;     // projected queries as three bf16 pieces [rows, 3*k] (tensor-core distances)
    float2* q_stat = nullptr;    // [rows] (|p|^2, 1/(1-|p|^2))
    uint32_t* fixup = nullptr;   // [8] rows the fused top-k read recomputed over every slot, per lane group
    // z_bf16 is [rows, d + 64] and act_bf16 [rows, 2d + 64] when the adapter rides in the MLP products (rank 16)
    char* base = nullptr;
    size_t bytes = 0;
};

}  // namespace pssa

struct pssa_b200_model {
    pssa_b200_ctx* ctx = nullptr;
    pssa_b200_config cfg{};
    size_t d = 0, s = 0, k = 0, cap = 0, v = 0, depth = 0, rank = 16;
    size_t ncat = 0;  // d + s + s + k + d + rank
    size_t off_delta = 0, off_b = 0, off_c = 0, off_q = 0, off_gate = 0, off_act = 0;
    uint32_t max_streams = 1;
    uint32_t precision = 0;  // PSSA_B200_PRECISION_*
    size_t top_k = 0;
    size_t loops = 1;  // Ouro passes per block (src/pssa.rs:2171-2184): shared weights, one carry per pass
    size_t lane_groups = 0;  // lane groups on side streams per pass: 0 = choose by shape, 1 = off, 2..4 forced
    size_t max_rows = 65536;
    float* embed = nullptr;
    float* unembed = nullptr;
    void* unembed_bf16 = nullptr;
    bool unembed_dirty = true;
    std::vector<pssa::DeviceBlock> blocks;
    std::vector<float> residual_scales;
    float* state = nullptr;  // [max_streams][depth][loops][d*s]  (src/pssa.rs:2255-2310)
    pssa::Workspace ws;
    // sequence-parallel prefill (world > 1): this process holds time shard `rank` of every lane
    struct SeqPar {
        uint32_t rank = 0, world = 1;
        float* send = nullptr;      // caller-owned device buffer, `capacity` records of (d + d*s) floats
        float* recv = nullptr;      // caller-owned device buffer, world * capacity records
        size_t capacity = 0;        // records (lanes x time chunks) the exchange buffers hold
        pssa_b200_exchange_fn fn = nullptr;
        void* arg = nullptr;
        bool active = false;        // set for the duration of a sharded prefill call only (decode steps stay local)
    } sp;
    // lane description last uploaded by the device-resident entry point (skipped when unchanged: graph capture)
    struct DevLayout {
        const char* ws_base = nullptr;
        std::vector<uint32_t> off, len, slot;
    } dev_layout;
    // scorer buffers: a tile of full-vocabulary logits, targets and per-row losses
    struct Score {
        float* logits = nullptr;   // [tile][vocab]
        uint32_t* targets = nullptr;
        float* loss = nullptr;     // [rows capacity]
        size_t tile = 0, rows = 0;
    } score;
    // observer scratch (src/pssa.rs:609-619: inf_q_pnc, inf_mem_weights, inf_m_val, inf_z_final of the last forward):
    // when enabled, every block publishes those four vectors for the last token of every lane of the last call
    struct Observer {
        bool enabled = false;
        float* q_pnc = nullptr;   // [rows capacity][k]   projected queries of the current block (all rows)
        size_t q_rows = 0;
        float* buf = nullptr;     // [depth][lanes capacity][cap + k + 2d]
        size_t lanes = 0, valid_lanes = 0;
    } obs;
    // per-stream sampler state for device-side sampling (src/inference.rs:37-41: one generator and one list of
    // generated ids per engine); allocated on first use
    struct Sampler {
        unsigned* recent = nullptr;            // [max_streams][64]
        unsigned* count = nullptr;             // [max_streams]
        unsigned long long* rng = nullptr;     // [max_streams]
        unsigned *ids = nullptr, *status = nullptr, *head_slot = nullptr;  // [lanes capacity]
        float* probs = nullptr;                // [lanes capacity][vocab]
        float* conf = nullptr;                 // [lanes capacity]
        size_t lanes = 0;
    } sampler;
    // time chunks ("virtual lanes") of the two-pass SSM: chunk maps, chunk carry-ins and the chunk row ranges
    struct Chunks {
        size_t capacity = 0;        // virtual lanes the buffers hold
        uint32_t *off = nullptr, *len = nullptr;
        std::vector<uint32_t> host_off, host_len;  // what `off` / `len` hold on the device: an unchanged description is not uploaded again
        float* records = nullptr;   // [capacity][d + d*s]  (local mode; the sharded mode uses sp.send)
        float* carry_in = nullptr;  // [capacity][d*s]
    } chunks;
    std::vector<bool> tensor_set;  // [depth * T_COUNT + id] upload bookkeeping
};
