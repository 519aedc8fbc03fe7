// Launchers implemented in the .cu files; all enqueue on ctx->stream and never synchronise.
#pragma once
#include <cstddef>
#include <cstdint>

#include "context.hpp"

namespace pssa {

// scan_affine.cu
int32_t launch_scan_states(pssa_b200_ctx* ctx, const float* a, const float* b, const float* h0, float* h, float* h_last,
                           size_t lanes, size_t len, size_t stride, int forced_chunks);
int32_t launch_scan_maps(pssa_b200_ctx* ctx, float* scan_a, float* scan_b, size_t lanes, size_t len, size_t stride,
                         int forced_chunks);

// allocation-free variant of launch_scan_states: chunk scratch in a fixed __device__ array (scan_affine.cu)
int32_t launch_scan_states_static(pssa_b200_ctx* ctx, const float* a, const float* b, const float* h0, float* h, float* h_last,
                                  size_t lanes, size_t len, size_t stride, unsigned chunks);

// ssm_fused.cu
struct SsmParams {
    const float* delta;    // [rows, d]  softplus already applied
    const float* x_norm;   // [rows, d]
    const float* b_proj;   // [rows, s]
    const float* c_proj;   // [rows, s]
    const float* rates;    // [d, s]     A = -softplus(raw)
    float* carry;          // [lanes, d*s] in/out, may be null (zero carry in, carry out dropped)
    float* y;              // [rows, d]
    void* y_bf16;          // optional bf16 copy of y for the tensor-core query projection
    float* states;         // optional [rows, d*s]: state after each token
    float* bar_a;          // optional [rows, d*s]
    float* bar_b;          // optional [rows, d*s]
    const uint32_t* offsets;  // per lane first row, null = one lane starting at row 0
    const uint32_t* lengths;  // per lane row count, null = rows
    size_t rows;
    int d, s, lanes;
    int aligned;           // 16-byte vector staging allowed
    // row pitches in floats (0 = dense: d for delta, s for b_proj / c_proj)
    size_t ld_delta, ld_bc;
    // carry of lane l lives at carry + slot(l) * carry_stride, slot(l) = lane_slots ? lane_slots[l] : l
    const uint32_t* lane_slots;
    size_t carry_stride;   // 0 = d*s
    int single_token;      // caller's promise that every lane is at most one token long (a decode step)
    // optional (needs offsets / lengths): per lane and channel, the sum of delta over the lane's rows (f64 sum, f32 out) at
    // sum_delta + lane * sum_delta_stride + i. With a zero carry in, (sum_delta, carry out) is the affine map of the
    // lane's time shard: h_out = exp(A * sum_delta) * h_in + carry_out (sequence-parallel prefill).
    float* sum_delta;
    size_t sum_delta_stride;
};
int32_t launch_ssm_fused(pssa_b200_ctx* ctx, const SsmParams& p, bool exact);
// 16-byte staging and stores need 16-byte aligned bases and row pitches / widths that are multiples of 4 floats
inline bool ssm_vector_ok(const SsmParams& p) {
    auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    size_t ldd = p.ld_delta ? p.ld_delta : (size_t)p.d, ldbc = p.ld_bc ? p.ld_bc : (size_t)p.s;
    return p.d % 4 == 0 && p.s % 4 == 0 && ldd % 4 == 0 && ldbc % 4 == 0 && al(p.delta) && al(p.x_norm) && al(p.b_proj) &&
           al(p.c_proj) && al(p.y) && (reinterpret_cast<uintptr_t>(p.y_bf16) & 7) == 0;
}

// Sequence-parallel prefill: fold the gathered per-rank shard maps (records of `rec` floats per lane: d sums of delta,
// then d*s shard states from a zero carry) into this rank's carry-in and into the sequence's final state.
// Each lane's shard is itself `chunks` consecutive time chunks (records ordered [rank][lane][chunk]).
//   h = state(lane); for k in 0..world, c in 0..chunks: { if (k == rank) carry_in(lane, c) = h; h = exp(A * sum_delta) * h + Q };
//   state(lane) = h
// world == 1 is the single-GPU time split of long sequences with few lanes.
int32_t launch_seqpar_fold(pssa_b200_ctx* ctx, const float* gathered, size_t rec, int world, int rank, int chunks, int lanes,
                           size_t rank_stride, const float* rates, float* state, size_t state_stride, const uint32_t* lane_slots,
                           float* carry_in, int d, int s);

// retrieve_poincare.cu
constexpr int kRetrievePhases = 12;  // cycle counters of the one-kernel top-k read (see PSSA_B200_MEM_PHASE_CLOCKS)
struct RetrieveParams {
    const float* q;        // [rows, dk] Euclidean queries (projected here) or points already in the ball
    int q_is_euclidean;
    float* q_pnc;          // [rows, dk] projected queries, may be null
    float* q_norm;         // [rows] Euclidean norm of q, may be null
    const float* keys;     // [cap, dk]
    const float* norm_sq;  // [cap]
    const float* values;   // [cap, dv]
    size_t ldq;            // row pitch of q in floats (0 = dk)
    float* weights;        // [rows, cap] distances in flight, weights on return
    float* m_val;          // [rows, dv]; may be null when m_bf16 is the only result wanted
    void* m_bf16;          // optional bf16 copy of m_val for the tensor-core memory projection
    float* min_dist;       // [rows], may be null
    // tensor-core value read (all-slots mode, non-exact): the softmax kernel also writes each weight row as three
    // bf16 pieces [rows, 3*cap]; v_split is the bank's values transposed and split the same way [dv, 3*cap]
    void* w_split;
    const void* v_split;
    size_t rows;
    int dk, dv, cap, count, top_k;
    float tau;
    int value_terms;       // tensor-core value read: 1 = leading pieces only (a plain bf16 product), 3 = the three leading
                           // partial products (error near 2^-16), else all six (fp32-accurate)
    int f32_distance;      // fast mode: squared differences accumulated in fp32 instead of f64 (ignored when exact)
    int skip_weights;      // all-slots, non-exact, w_split set: do not write the fp32 weight rows back (only the pieces are read)
    float* row_scale_out;  // one-kernel all-slots read only: when set, the weight rows are left as exp((d_min - d) / tau), not
                           // divided by their sum, and 1 / sum goes here ([rows]) for the consumer's epilogue to apply
    int skip_value_read;   // all-slots, non-exact, w_split set: stop after the softmax; the caller multiplies the weight pieces itself
    // tensor-core distances (non-exact, dk % 64 == 0; used when all four are set): q_split [rows, 3*dk] bf16 and
    // q_stat [rows] are scratch written by the projection kernel; k_split [cap, 3*dk] bf16 and k_stat [cap] come from
    // launch_split_keys, once per bank upload
    void* q_split;
    float2* q_stat;
    const void* k_split;
    const float2* k_stat;
    // exact top-k in one kernel (retrieve_fused.cu): compact outputs [rows, top_k] in ascending slot order (either may be
    // null), the counter of rows whose selection the candidates could not prove (recomputed over every slot by the same
    // kernel; one scratch word), and a test hook that treats every n-th row that way regardless (0 = off)
    unsigned* topk_slots;
    float* topk_weights;
    unsigned* fixup_count;
    int selftest_every;
    int no_fused;          // keep the multi-kernel path even where the one-kernel top-k read applies
    int single_token;      // the caller's rows are one token per stream (a decode step): the all-slots read of the fast modes
                           // then takes its one-launch front end, whatever the number of streams -- the choice must not
                           // depend on the row count, or the same stream would see different arithmetic alone and in a batch
    unsigned long long* phase_cycles;  // optional [kRetrievePhases] device counters: clock cycles one worker thread per CTA spent per phase
    int* status;           // context status word (set by the launcher)
};
int32_t launch_memory_read(pssa_b200_ctx* ctx, const RetrieveParams& p, bool exact);
// retrieve_fused.cu: projection, tensor-core pre-filter, exact f64 re-scoring of the candidates, (bits, slot) selection,
// softmax and value read of a top-k read in one kernel; same results as the f64 path of launch_memory_read
bool retrieve_fused_eligible(const RetrieveParams& p);
bool retrieve_all_fused_eligible(const RetrieveParams& p);
// what launch_memory_read decides for this call: true = the one-kernel all-slots read runs (and honours row_scale_out)
bool retrieve_all_fused_runs(const RetrieveParams& p, bool exact);
int32_t launch_retrieve_all_fused(pssa_b200_ctx* ctx, const RetrieveParams& p);
int32_t launch_retrieve_fused(pssa_b200_ctx* ctx, const RetrieveParams& p);
// dense weight rows [rows, cap] -> selected slots and weights [rows, k] in ascending slot order
int32_t launch_compact_topk(pssa_b200_ctx* ctx, const float* weights, int cap, int k, size_t rows, unsigned* slots, float* w_out);
// values [cap, dv] fp32 -> v_split [dv, 3*cap] bf16 (transpose + three-way split); once per bank upload
int32_t launch_split_values(pssa_b200_ctx* ctx, const float* values, void* v_split, int cap, int dv);
// keys [cap, dk] fp32 -> k_split [cap, 3*dk] bf16 pieces and k_stat[slot] = (|k|^2, 1/(1-|k|^2)); once per bank upload
int32_t launch_split_keys(pssa_b200_ctx* ctx, const float* keys, const float* norm_sq, void* k_split, float2* k_stat, int cap, int dk);

// sampling.cu
struct SampleParams {
    float* logits;               // [rows, vocab]; the repetition penalty is applied in place, like the reference
    float* probs;                // [rows, vocab] scratch
    size_t rows;
    int vocab, top_k;
    float temperature, top_p, repetition_penalty;
    const unsigned* recent_ids;  // [rows, 64] last generated ids of each stream in generation order, may be null
    const unsigned* recent_count;  // [rows] how many of them are valid (<= 64)
    unsigned long long* rng_state;  // [rows] xorshift64* state, advanced by one draw when temperature > 0
    unsigned* ids_out;           // [rows] sampled id, UINT32_MAX on error
    unsigned* status_out;        // [rows] 0 ok, 1 non-finite logits, 2 invalid probability mass, 3 no candidates
    int exact;                   // sequential f32 sum over the vocabulary (the reference's order)
    const unsigned* slots;       // optional [rows]: recent_* and rng_state are indexed by slots[row] instead of row
    float* confidence_out;       // optional [rows]: raw softmax probability of the selected id (src/inference.rs:526-545)
};
int32_t launch_sample(pssa_b200_ctx* ctx, const SampleParams& p);
int32_t launch_push_recent(pssa_b200_ctx* ctx, const unsigned* ids, const unsigned* slots, unsigned* recent, unsigned* count, size_t rows);

// plastic_write.cu
struct BankWriteParams {
    float* keys;                 // [cap, dk]
    float* norm_sq;              // [cap]
    float* values;               // [cap, dv]
    float* confidence;           // [cap]
    unsigned long long* last_seen;  // [cap]
    unsigned long long* meta;    // {count, write_head}
    int cap, dk, dv;
    const float* key_pnc;        // [n, dk]
    const float* val;            // [n, dv]
    const float* surprise;       // [n]
    const unsigned long long* step;  // [n]
    size_t n;
    long long* slots_out;        // [n] written slot or -1 (defended); may be null
    const unsigned* winning_slots;  // null = reference behaviour (ring head); else the slot each write targets
    float eta;                   // rank-1 step of the winning-slot mode
    int* status;                 // context status word (set by the launcher): PSSA_B200_ERR_BANK on a refused write
};
int32_t launch_bank_insert_protected(pssa_b200_ctx* ctx, const BankWriteParams& p);
int32_t launch_plastic_update(pssa_b200_ctx* ctx, float* up_fast, const float* value, const float* ad_out, const float* ad_act,
                              int d, int rank);
int32_t launch_consolidate(pssa_b200_ctx* ctx, float* up_fast, float* up_slow, size_t n, float alpha);

// gemm_exact.cu: out[M, ldo] (first N columns) = epilogue(X[M,K] * W[N,K]^T), fp32, dot_slice order
int32_t launch_gemm_exact(pssa_b200_ctx* ctx, const float* x, const float* w, float* out, size_t M, size_t N, size_t K,
                          size_t ldo, int epi, float alpha);

// gemm_tcgen05.cu: one warp waits `polls` polls on an mbarrier nobody arrives at and records the expiry (self-test)
int32_t launch_wait_expiry_selftest(pssa_b200_ctx* ctx, unsigned polls);
// gemm_tcgen05.cu: bf16 operands [rows, K] row-major, fp32 accumulate in TMEM; out fp32 [M, ldo] and/or bf16 [M, N]
int32_t launch_gemm_bf16(pssa_b200_ctx* ctx, const void* x16, const void* w16, float* out, void* out_bf16, size_t M, size_t N,
                         size_t K, size_t ldo, int epi, float alpha, size_t ld16 = 0);  // ld16: row pitch of out_bf16 (0 = N)
// z = gate * (X W^T) + alpha * y, fp32 and bf16 (row pitch ld16) outputs. split_k: both operands are [., 3*K] three-piece
// splits (K % 64 == 0) and only the leading pieces are multiplied.
int32_t launch_gemm_bf16_gate(pssa_b200_ctx* ctx, const void* x16, const void* w16, float* out, void* out_bf16, size_t ld16,
                              const float* gate, size_t ld_gate, const float* y, float alpha, size_t M, size_t N, size_t K,
                              bool split_k = false, const float* row_scale = nullptr);
// MLP output with both residuals fused: out = res_in ? res_in + res_scale*(X W^T + add_in) : X W^T + add_in
// add_in is fp32 [M, N], or bf16 [M, ld_add_bf16] when ld_add_bf16 != 0
int32_t launch_gemm_bf16_residual(pssa_b200_ctx* ctx, const void* x16, const void* w16, float* out, const void* add_in,
                                  const float* res_in, float res_scale, size_t M, size_t N, size_t K, size_t ld_add_bf16 = 0);
// fp32-accurate product of operands pre-split into three bf16 pieces: a16 [M, 3K], b16 [N, 3K] (six partial products)
int32_t launch_gemm_bf16_split3(pssa_b200_ctx* ctx, const void* a16, const void* b16, float* out, void* out_bf16, size_t M,
                                size_t N, size_t K, size_t ldo, int terms = 6);
// Poincare distances of M points of the ball to N bank keys from the inner products of their three-piece splits
// (a16 [M, 3K], b16 [N, 3K]); row_stat / col_stat = (|.|^2, 1/(1-|.|^2)); dist fp32 [M, ldo]
int32_t launch_gemm_bf16_poincare(pssa_b200_ctx* ctx, const void* a16, const void* b16, const float2* row_stat,
                                  const float2* col_stat, float* dist, size_t M, size_t N, size_t K, size_t ldo);
// concatenated x-side projections: columns [0,c1) softplus, [c1,c2) identity, [c2,c3) sigmoid, [c3,N) SiLU
// side_a / side_b (both or neither): the last range is also stored as bf16 at column (col - c3) of two more buffers
int32_t launch_gemm_bf16_cat(pssa_b200_ctx* ctx, const void* x16, const void* w16, float* out, size_t M, size_t N, size_t K,
                             size_t ldo, int c1, int c2, int c3, void* side_a = nullptr, size_t ld_side_a = 0, void* side_b = nullptr,
                             size_t ld_side_b = 0);

// elementwise.cu
int32_t launch_embed_norm(pssa_b200_ctx* ctx, const float* embed, const uint32_t* ids, const float* feats, const float* gamma,
                          const float* beta, float* x_norm, void* x_bf16, size_t rows, int d, bool exact, size_t vocab);
int32_t launch_combine_zraw(pssa_b200_ctx* ctx, const float* y, const float* g, size_t ldg, const float* m_proj, const float* act,
                            size_t ldact, const float* u_eff, float* z_raw, void* z_bf16, size_t rows, int d, int rank,
                            float ssm_scale);
int32_t launch_residual(pssa_b200_ctx* ctx, const float* prev, const float* z, float* out, size_t n, float scale);
int32_t launch_multiply(pssa_b200_ctx* ctx, const float* a, const float* b, float* out, size_t n);
// src_rows != 0: rows_idx is range checked on the device against a table of src_rows rows (row 0 + PSSA_B200_ERR_TOKEN otherwise)
// dst (fp32) and dst_bf16 are both optional
int32_t launch_gather_rows(pssa_b200_ctx* ctx, const float* src, const uint32_t* rows_idx, float* dst, size_t n_rows, int d, size_t src_rows = 0,
                           void* dst_bf16 = nullptr);
int32_t launch_to_bf16(pssa_b200_ctx* ctx, const float* src, void* dst, size_t n);
int32_t launch_observe_rows(pssa_b200_ctx* ctx, const uint32_t* last_rows, size_t lanes, const float* weights, int cap, const float* q_pnc,
                            int k, const float* m_val, const float* z_direct, const float* feat_out, const float* feat_in, float scale,
                            int d, float* out);
// adapter term folded into the MLP products (bf16 mode): see elementwise.cu
int32_t launch_pack_weight_cat(pssa_b200_ctx* ctx, const float* src, const float* tail, void* dst, size_t n, int k);
int32_t launch_times_adapter(pssa_b200_ctx* ctx, const float* w, const float* u, float* out, size_t n, int k);
int32_t launch_cross_entropy(pssa_b200_ctx* ctx, const float* logits, const uint32_t* targets, float* loss, size_t rows, int v);
int32_t launch_greedy(pssa_b200_ctx* ctx, const float* logits, uint32_t* out, size_t rows, int v);

}  // namespace pssa
