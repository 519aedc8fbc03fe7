/*
 * pssa_b200 — C ABI of the B200-native PSSA inference forward path.
 *
 * This is the drop-in boundary: the entry points below are what a `GpuDispatch::B200` /
 * `Device::B200` arm of the reference crate (src/backend.rs:1012-1029) binds over FFI.
 * Plain pointers and sizes only. All matrices are row-major f32 unless stated otherwise.
 *
 * Conventions
 *  - Every function returns a `pssa_b200_status`. On failure the message is available from
 *    `pssa_b200_last_error(ctx)`; caller-owned outputs are left untouched when validation
 *    fails (reference behaviour: src/backend.rs:684-686, tests/backend.rs:66-82).
 *  - Shape validation happens before any allocation or launch and uses the reference's
 *    wording "refusing launch" (src/cuda/stage_bounds.rs:5-65).
 *  - `*_dev` functions take DEVICE pointers, enqueue on the context's stream and return
 *    without synchronising. Functions without the suffix take HOST pointers, stage them
 *    through the context's device arena and return after the result is back on the host,
 *    which is the contract of the reference's `GpuDispatch` methods (src/cuda.rs:517-585).
 *  - There is no CPU fallback anywhere behind this header: without a CUDA device every
 *    compute entry point fails with PSSA_B200_ERR_CUDA.
 *  - A context is single-threaded, like a reference model (`&mut self` on every call).
 */
#ifndef PSSA_B200_H
#define PSSA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum pssa_b200_status {
    PSSA_B200_OK = 0,
    PSSA_B200_ERR_INVALID_ARGUMENT = 1, /* null pointer, bad enum, bad handle */
    PSSA_B200_ERR_SHAPE = 2,            /* dimension / length check failed; nothing launched */
    PSSA_B200_ERR_CUDA = 3,             /* recoverable CUDA error (no device, allocation, ...) */
    PSSA_B200_ERR_FATAL_CUDA = 4,       /* context lost: src/cuda.rs:592-602 classes */
    PSSA_B200_ERR_TIMEOUT = 5,          /* a bounded device-side wait gave up */
    PSSA_B200_ERR_UNSUPPORTED = 6,      /* option the device path refuses (src/pssa.rs:2080-2243) */
    PSSA_B200_ERR_TOKEN = 7,            /* token id outside the vocabulary */
    PSSA_B200_ERR_CANCELLED = 8,        /* the caller's cancellation callback fired */
    PSSA_B200_ERR_BANK = 9              /* device-resident bank metadata / slot id out of range, or a key outside the ball */
} pssa_b200_status;

typedef struct pssa_b200_ctx pssa_b200_ctx;     /* one device, one stream, one scratch arena */
typedef struct pssa_b200_model pssa_b200_model; /* device-resident weights, banks and carries */

/* ------------------------------------------------------------------ context */

/* Replaces `CudaContext::init` (src/cuda.rs:168-196); `device` is a CUDA ordinal. */
int32_t pssa_b200_ctx_create(int32_t device, pssa_b200_ctx** out);
void pssa_b200_ctx_destroy(pssa_b200_ctx* ctx);
/* Message of the last failure on `ctx` (or of the last failed create when ctx is NULL). */
const char* pssa_b200_last_error(const pssa_b200_ctx* ctx);
/* Enqueue on an existing cudaStream_t (e.g. the caller framework's current stream). NULL is the
 * legacy default stream. A fresh context runs on a non-blocking stream of its own. */
int32_t pssa_b200_ctx_set_stream(pssa_b200_ctx* ctx, void* cuda_stream);
/* Go back to a non-blocking stream owned by the context. */
int32_t pssa_b200_ctx_use_own_stream(pssa_b200_ctx* ctx);
int32_t pssa_b200_ctx_synchronize(pssa_b200_ctx* ctx);
/* Replaces `backend_label` (src/backend.rs:1439-1446): "b200 (<device name>)". */
const char* pssa_b200_backend_label(const pssa_b200_ctx* ctx);
/* Number of kernels of this library launched on `ctx` since creation. */
uint64_t pssa_b200_launch_count(const pssa_b200_ctx* ctx);
/* Pre-size the context's scratch arena (bytes) so later calls do not allocate. */
int32_t pssa_b200_ctx_reserve(pssa_b200_ctx* ctx, size_t bytes);

/* Device-side waits (mbarrier phases of the tensor-core pipeline) are bounded; when one expires the kernel
 * records it and returns. This reads and clears that record: PSSA_B200_OK or PSSA_B200_ERR_TIMEOUT. The same word
 * carries PSSA_B200_ERR_TOKEN when a DEVICE-resident token id (which the host cannot check) was outside the vocabulary:
 * the embedding of id 0 was read in its place, so nothing is accessed out of bounds; and PSSA_B200_ERR_BANK when
 * pssa_b200_bank_insert_protected_dev refused a write. */
int32_t pssa_b200_ctx_poll_status(pssa_b200_ctx* ctx);

/* Failure-detection self-test (the role of the reference's host-injected driver failures, tests/backend_cuda.rs:599-649,
 * for the one failure class that lives on the device): enqueues a one-warp kernel that waits at most `polls`
 * (1..2^20) polls on a barrier nothing arrives at, using the tensor-core pipeline's own bounded-wait helper. The wait
 * expires, the kernel records it and returns; pssa_b200_ctx_poll_status then reports PSSA_B200_ERR_TIMEOUT once and
 * the context stays usable. Nothing faults or hangs. */
int32_t pssa_b200_ctx_selftest_wait_expiry(pssa_b200_ctx* ctx, uint32_t polls);

/*
 * Per-kernel device timing, the role of the reference's `StageTrace` spans (src/training_diagnostics.rs:74-125,
 * enabled there by PSSA_CUDA_PROFILE=1) with CUDA events instead of wall clock. Between begin and end an event is
 * recorded after every kernel this library launches on `ctx`; end synchronises and aggregates the time between
 * consecutive events by kernel name. Rows are read back one at a time.
 */
int32_t pssa_b200_ctx_profile_begin(pssa_b200_ctx* ctx);
int32_t pssa_b200_ctx_profile_end(pssa_b200_ctx* ctx, uint32_t* n_rows);
int32_t pssa_b200_ctx_profile_row(pssa_b200_ctx* ctx, uint32_t index, const char** name, uint64_t* launches,
                                  double* ms);

/* Force the number of time chunks of the scan (0 = automatic). A test hook: with more than one
 * chunk the scan runs its reduce / carry / apply passes even on shapes that would not need them. */
int32_t pssa_b200_ctx_set_scan_chunks(pssa_b200_ctx* ctx, uint32_t chunks);

/* ------------------------------------------------------------------ scan operator */

/*
 * In-place EXCLUSIVE prefix of diagonal affine maps over time, `lanes` independent problems.
 * scan_a/scan_b: [lanes, len, stride]; on return row t holds the composition of rows < t
 * (row 0 = identity). Replaces `affine_scan_in_place` (src/gpu_batch.rs:98-164) and the
 * `affine_scan` launch (src/cuda/stages.rs:212-259, shape rule src/cuda/stage_bounds.rs:45-65).
 * No power-of-two padding is needed.
 */
int32_t pssa_b200_affine_scan_dev(pssa_b200_ctx* ctx, float* scan_a, float* scan_b, size_t lanes,
                                  size_t len, size_t stride);
int32_t pssa_b200_affine_scan(pssa_b200_ctx* ctx, float* scan_a, float* scan_b, size_t lanes,
                              size_t len, size_t stride);

/*
 * All prefix states of h_t = a_t * h_{t-1} + b_t (multiply, then add, each rounded: the order
 * of src/gpu_batch.rs:543-575). a, b, h: [lanes, len, stride]; h0 and h_last: [lanes, stride],
 * either may be NULL (zero carry in / carry out not wanted). h may alias b. This is the scan
 * operator "alone": 12 bytes of HBM traffic per element.
 */
int32_t pssa_b200_scan_states_dev(pssa_b200_ctx* ctx, const float* a, const float* b,
                                  const float* h0, float* h, float* h_last, size_t lanes,
                                  size_t len, size_t stride);
int32_t pssa_b200_scan_states(pssa_b200_ctx* ctx, const float* a, const float* b, const float* h0,
                              float* h, float* h_last, size_t lanes, size_t len, size_t stride);

/*
 * Allocation-free form of pssa_b200_scan_states_dev. It has no counterpart in the reference.
 *
 * Who needs it: a host process that must not see this library allocate device memory once it is running --
 * for example a serving process whose own allocator took the whole GPU at start-up, or a loop that cannot
 * afford the device-wide synchronisation that cudaMalloc / cudaFree imply. The scan splits time into `chunks`
 * (>= 1) pieces; the per-chunk maps and carries, which the other entry point keeps in the context's growable
 * arena, live here in a fixed 12 MiB array compiled into the library (held by every GPU that loads the
 * library, until the process exits). Limit: lanes * chunks * stride <= 1,048,576 when chunks > 1; a larger
 * request fails with PSSA_B200_ERR_SHAPE and launches nothing. The call never calls cudaMalloc, cudaFree or
 * any allocating routine; inputs and outputs are the caller's (DEVICE pointers, as for the _dev form).
 *
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress, once per device);
 * make that first call outside any stream capture. All calls on a device share the one array: a call only
 * reads scratch it has itself written, so nothing needs clearing between calls, but two calls whose kernels
 * overlap on the GPU (different streams or contexts of one process) race on it -- serialise them.
 */
int32_t pssa_b200_scan_states_noalloc_dev(pssa_b200_ctx* ctx, const float* a, const float* b, const float* h0,
                                          float* h, float* h_last, size_t lanes, size_t len, size_t stride,
                                          uint32_t chunks);

/* ------------------------------------------------------------------ fused SSM stage */

/* Arithmetic mode of the SSM stage. Default (0): ex2.approx on delta*(A*log2 e) -- the recipe of the
 * reference's own GPU kernel (src/cuda/stages.ptx:21-22) -- with fused multiply-adds. EXACT: expf and
 * separately rounded multiply/add in the order of the CPU reference (src/pssa.rs:1131-1144). */
#define PSSA_B200_SSM_EXACT 1u

/*
 * Discretise + scan + read out for `lanes` independent sequences packed in one row space:
 *   a = exp(delta_i*rates_ij), b = delta_i*B_j, h_ij <- a*h_ij + b*x_i, y_i = sum_j h_ij*C_j.
 * Replaces ssm_prepare + affine_scan + ssm_materialize (src/cuda/stages.rs:260-356), the lane-batched
 * packed_scan / packed_materialize (src/cuda/packed.rs:384-428) and `ssm_forward_resident`
 * (src/backend.rs:1190-1212): the state stays on the device in `carry`.
 * DEVICE pointers: delta, x_norm, y [rows, d_m]; b_proj, c_proj [rows, d_s]; rates [d_m, d_s];
 * carry [lanes, d_m*d_s] read and updated in place (NULL: zero carry in, carry out dropped);
 * optional tape outputs states / bar_a / bar_b [rows, d_m*d_s] (state after each token; NULL = skip).
 * HOST pointers: offsets / lengths [lanes] (u32, first row and row count of each lane; both NULL means
 * one lane covering all rows). Lanes must not overlap and must lie inside [0, rows).
 */
int32_t pssa_b200_ssm_forward_dev(pssa_b200_ctx* ctx, const float* delta, const float* b_proj,
                                  const float* c_proj, const float* x_norm, const float* rates,
                                  float* carry, float* y, float* states, float* bar_a, float* bar_b,
                                  const uint32_t* offsets, const uint32_t* lengths, size_t lanes,
                                  size_t rows, size_t d_m, size_t d_s, uint32_t flags);

/*
 * Host-pointer form with the argument list of `GpuDispatch::ssm_forward` (src/backend.rs:1215-1244)
 * minus the two backward-only inputs (delta_raw, rate_deriv): one lane of seq_len tokens, `initial`
 * [d_m*d_s], states [(seq_len+1)*d_m*d_s] with row 0 = initial, bar_a / bar_b [seq_len*d_m*d_s],
 * y_ssm [seq_len*d_m]. bar_a, bar_b and states may be NULL.
 */
int32_t pssa_b200_ssm_forward(pssa_b200_ctx* ctx, const float* delta, const float* b_proj,
                              const float* x_norm, const float* rates, const float* c_proj,
                              const float* initial, size_t seq_len, size_t d_m, size_t d_s,
                              float* bar_a, float* bar_b, float* states, float* y_ssm, uint32_t flags);

/* ------------------------------------------------------------------ episodic memory read */

/* Keep the reference's sequential f32 summation order for the softmax sum and the value read
 * (src/memory.rs:409-425) instead of tree sums and fused multiply-adds. */
#define PSSA_B200_MEM_EXACT 1u
/* Accumulate the squared differences of the distance in fp32 instead of the reference's f64 (src/memory.rs:245-262).
 * Differences are still formed first, so the distance keeps a relative error near 1e-6; the projection stays f64.
 * About four times faster; what the model's bf16 precision mode uses. Ignored together with PSSA_B200_MEM_EXACT. */
#define PSSA_B200_MEM_F32_DISTANCE 2u
/* Distances from the inner product on the tensor cores: |p - k|^2 = |p|^2 + |k|^2 - 2 p.k with p and k each split into
 * three bf16 pieces and the distance formula in the product's epilogue. The projection stays f64. Absolute error of
 * |p - k|^2 up to about 2e-6 (tensor-core fp32 accumulation is not correctly rounded), so a query that coincides with
 * a key gets a distance of up to 1e-2 instead of 0; meant for queries that already carry bf16 rounding (the model's
 * bf16 precision mode uses it). Needs d_key % 64 == 0, otherwise PSSA_B200_MEM_F32_DISTANCE behaviour applies.
 * Ignored together with PSSA_B200_MEM_EXACT. */
#define PSSA_B200_MEM_TC_DISTANCE 4u
/* Top-k reads whose shape allows it (capacity 128 / 256 / 512, d_key 64 or 128, top_k <= 12, at least 8 * (top_k + 3)
 * occupied slots) run as
 * ONE kernel: tensor-core inner products only pre-filter the slots, the candidates are re-scored with the reference's f64
 * arithmetic and selected by (distance bits, slot), and a row whose selection cannot be proven from the candidates is
 * handed to an exact pass over every slot. Results are those of the default f64 path. This flag keeps the separate
 * distance / selection kernels instead (for comparison). */
#define PSSA_B200_MEM_NO_FUSED 8u
/* Test hook: the one-kernel top-k read hands every third row to its exact pass regardless of the proof. */
#define PSSA_B200_MEM_HANDOVER_SELFTEST 16u
/* Diagnostic of pssa_b200_memory_read_topk_dev: `handed_over` then points at 26 u32 words (8-byte aligned): the count,
 * one pad word, then twelve 64-bit counters of SM clock cycles summed over the CTAs of the one-kernel read: loading the
 * queries, projecting, splitting into bf16 pieces, waiting for the tensor cores, the first sweep (group minima), the
 * threshold, the second sweep (listing), the candidate selection, the exact squared distances, the distances, selection
 * proof + softmax, and the value read. */
#define PSSA_B200_MEM_PHASE_CLOCKS 32u

/*
 * Poincare-ball memory read for `rows` queries against one immutable bank. Replaces
 * `diffeomorphic_project` + `retrieve_soft_into` (src/memory.rs:198-211, 344-426), the row loop
 * `retrieve_memory_rows` (src/gpu_batch.rs:700-741) and the reference GPU's memory_forward kernel +
 * cuBLAS value read (src/cuda/stages.rs:563-614).
 *   q [rows, d_key]: Euclidean queries when q_is_euclidean != 0 (projected with q/(1+|q|), f64), else
 *   points already inside the ball. keys [capacity, d_key], norm_sq [capacity], values [capacity, d_val];
 *   only the first `count` slots are read. score = -distance, weights = softmax(score / tau) over all
 *   occupied slots, or over the exact `top_k` nearest (ties to the lower slot) when 0 < top_k < count.
 * Outputs: q_pnc [rows, d_key] (NULL to skip), q_norm [rows] (NULL to skip), weights [rows, capacity]
 * (zero outside the occupied / selected slots; NULL: scratch from the context arena), m_val [rows, d_val],
 * min_dist [rows] (NULL to skip). count == 0 gives zero weights and values (src/memory.rs:363-367).
 */
int32_t pssa_b200_memory_read_dev(pssa_b200_ctx* ctx, const float* q, int32_t q_is_euclidean,
                                  const float* keys, const float* norm_sq, const float* values,
                                  size_t rows, size_t d_key, size_t d_val, size_t capacity, size_t count,
                                  float tau, size_t top_k, float* q_pnc, float* q_norm, float* weights,
                                  float* m_val, float* min_dist, uint32_t flags);
int32_t pssa_b200_memory_read(pssa_b200_ctx* ctx, const float* q, int32_t q_is_euclidean,
                              const float* keys, const float* norm_sq, const float* values, size_t rows,
                              size_t d_key, size_t d_val, size_t capacity, size_t count, float tau,
                              size_t top_k, float* q_pnc, float* q_norm, float* weights, float* m_val,
                              float* min_dist, uint32_t flags);
/*
 * Top-k read (0 < top_k < count) with COMPACT results instead of the reference's dense weight row (src/memory.rs:380-408
 * zero-fills `out_weights` and sets k entries): slots_out [rows, top_k] (u32) and weights_out [rows, top_k], the selected
 * slots in ascending slot order -- the order the reference sums and mixes them in -- and their normalised weights;
 * either may be NULL. 8 * top_k bytes per query instead of 4 * capacity. handed_over (DEVICE u32, NULL to skip) receives
 * the number of rows the one-kernel read gave to its exact pass. Other arguments as pssa_b200_memory_read_dev. Shapes
 * outside the one-kernel read's range run the separate kernels with scratch weight rows and are compacted afterwards
 * (a selected slot whose weight underflowed to zero is then reported as 0xffffffff).
 */
int32_t pssa_b200_memory_read_topk_dev(pssa_b200_ctx* ctx, const float* q, int32_t q_is_euclidean, const float* keys,
                                       const float* norm_sq, const float* values, size_t rows, size_t d_key, size_t d_val,
                                       size_t capacity, size_t count, float tau, size_t top_k, float* q_pnc, float* q_norm, float* m_val,
                                       float* min_dist, uint32_t* slots_out, float* weights_out, uint32_t* handed_over, uint32_t flags);

/* ------------------------------------------------------------------ memory stage and resident SSM, one call each */

/*
 * `GpuDispatch::memory_forward` (src/backend.rs:1342-1385) with its argument list: the whole memory stage of a block for
 * seq_len token rows, the CPU twin being `stage_memory_impl` (src/gpu_batch.rs:758-929):
 *   q_euc = W_qx x + W_qh y; q_pnc, q_norm = projection into the ball; weights, m_val = all-slots read of the bank;
 *   g_mem = sigmoid(W_gate x); m_proj = W_proj m_val; m_inj = g_mem * m_proj.
 * HOST pointers, row-major fp32: x_norm, y_ssm [seq_len, d_m]; w_qx, w_qh [d_k, d_m]; w_gate [d_m, d_m]; w_proj
 * [d_m, d_val]; keys [capacity, d_k]; norm_sq [capacity]; values [capacity, d_val]. Outputs: q_euc, q_pnc [seq_len, d_k];
 * q_norm [seq_len]; weights [seq_len, capacity]; m_val [seq_len, d_val]; g_mem, m_proj, m_inj [seq_len, d_m]; all left
 * untouched on failure. `precision` (not in the reference's list): PSSA_B200_PRECISION_FP32_EXACT keeps the reference's
 * dot-product and summation orders; PSSA_B200_PRECISION_BF16 runs the four products on the tensor cores (d_m and d_val
 * multiples of 8) with the read's f64 distances unchanged. The _dev form takes DEVICE pointers and only enqueues.
 */
int32_t pssa_b200_memory_forward(pssa_b200_ctx* ctx, const float* x_norm, const float* y_ssm, const float* w_qx, const float* w_qh,
                                 const float* w_gate, const float* w_proj, const float* keys, const float* norm_sq, const float* values,
                                 size_t seq_len, size_t d_m, size_t d_k, size_t d_val, size_t capacity, size_t count, float tau,
                                 float* q_euc, float* q_pnc, float* q_norm, float* weights, float* m_val, float* g_mem, float* m_proj,
                                 float* m_inj, int32_t precision);
int32_t pssa_b200_memory_forward_dev(pssa_b200_ctx* ctx, const float* x_norm, const float* y_ssm, const float* w_qx, const float* w_qh,
                                     const float* w_gate, const float* w_proj, const float* keys, const float* norm_sq,
                                     const float* values, size_t seq_len, size_t d_m, size_t d_k, size_t d_val, size_t capacity,
                                     size_t count, float tau, float* q_euc, float* q_pnc, float* q_norm, float* weights, float* m_val,
                                     float* g_mem, float* m_proj, float* m_inj, int32_t precision);
/*
 * `GpuDispatch::ssm_forward_resident` (src/backend.rs:1186-1212): the SSM stage of one lane whose results (y, every
 * state, the discretised maps) stay on the device, in buffers the context owns, until the memory stage consumes them.
 * HOST pointers as for pssa_b200_ssm_forward; delta_raw is the reference's backward-only input and may be NULL.
 */
int32_t pssa_b200_ssm_forward_resident(pssa_b200_ctx* ctx, const float* delta, const float* delta_raw, const float* b_proj,
                                       const float* x_norm, const float* rates, const float* c_proj, const float* initial,
                                       size_t seq_len, size_t d_m, size_t d_s, uint32_t flags);
/*
 * `GpuDispatch::memory_forward_after_ssm` (src/backend.rs:1246-1289): publishes the resident SSM tape to the host
 * (bar_a, bar_b [seq_len, d_m*d_s], states [(seq_len+1), d_m*d_s] with row 0 the initial carry, y_ssm [seq_len, d_m];
 * the first three may be NULL) and runs pssa_b200_memory_forward on the resident y. Fails with the reference's messages
 * when no SSM result is resident or its shape differs (src/cuda/stages.rs:714, 733-735); the tape is published before
 * the memory stage runs, so it survives a failure of that stage (src/cuda/stages.rs:737-771).
 */
int32_t pssa_b200_memory_forward_after_ssm(pssa_b200_ctx* ctx, const float* x_norm, const float* w_qx, const float* w_qh, const float* w_gate,
                                           const float* w_proj, const float* keys, const float* norm_sq, const float* values,
                                           size_t seq_len, size_t d_m, size_t d_k, size_t d_val, size_t capacity, size_t count, float tau,
                                           float* bar_a, float* bar_b, float* states, float* y_ssm, float* q_euc, float* q_pnc,
                                           float* q_norm, float* weights, float* m_val, float* g_mem, float* m_proj, float* m_inj,
                                           int32_t precision);

/* ------------------------------------------------------------------ bank write and plastic fast weights */

/*
 * `n` ORDERED protected inserts into one bank, gate and copy fused in one kernel. Replaces
 * `insert_protected_with_device` (src/memory.rs:315-342), `apply_refractory_overwrite` (src/defense.rs:45-67) and
 * the ring insert (src/memory.rs:268-303) as called by `insert_training_memory_at` (src/pssa.rs:3705-3737).
 * All DEVICE pointers: keys [cap,d_key], norm_sq [cap], values [cap,d_val], confidence [cap], last_seen_step [cap]
 * (u64), meta = {count, write_head} (u64, updated), key_pnc [n,d_key] (points inside the ball), val [n,d_val],
 * surprise [n], step [n] (u64). slots_out [n] (i64, NULL to skip): the slot written, -1 when the slot defended
 * itself, or -2 when the write was refused: meta and winning_slots live on the device where the host cannot check
 * them, so a count above capacity, a ring head or winning slot >= capacity, or a key that is not inside the open unit
 * ball (the reference asserts it, src/memory.rs:273-277) skips that write, touches nothing out of bounds and raises
 * PSSA_B200_ERR_BANK in the context's status word (pssa_b200_ctx_poll_status). While count < capacity a write appends; afterwards the ring head is gated: gain = max((1-exp(-dt/60))^2,
 * 0.005), damage = 0.08*surprise*gain; confidence > damage keeps the slot (confidence -= damage), otherwise the
 * slot is overwritten, confidence = 1 and the head advances.
 *
 * winning_slots (NULL for the behaviour above) selects the retrieval benchmark's variant, which is NOT a reference
 * code path: write i gates slot winning_slots[i] (the caller's nearest slot) instead of the ring head, and a
 * successful write is the rank-1 update values[slot] += eta * (val - values[slot]); keys are left untouched.
 */
int32_t pssa_b200_bank_insert_protected_dev(pssa_b200_ctx* ctx, float* keys, float* norm_sq, float* values,
                                            float* confidence, uint64_t* last_seen_step, uint64_t* meta,
                                            size_t capacity, size_t d_key, size_t d_val, const float* key_pnc,
                                            const float* val, const float* surprise, const uint64_t* step, size_t n,
                                            int64_t* slots_out, const uint32_t* winning_slots, float eta);
/*
 * Hebbian rank-1 update of the adapter's fast weights, `dream_replay_value` (src/pssa.rs:1814-1832) after the
 * block forward: rate = 0.02/(1+|value|), err = clamp(value - ad_out, -4, 4), up_fast[i,r] += rate*err_i*ad_act[r].
 * DEVICE pointers: up_fast [d, rank], value [d], ad_out [d], ad_act [rank].
 */
int32_t pssa_b200_adapter_plastic_update_dev(pssa_b200_ctx* ctx, float* up_fast, const float* value,
                                             const float* ad_out, const float* ad_act, size_t d, size_t rank);
/* `PlasticAdapterV2::consolidate` (src/adapter.rs:65-72): slow += alpha*fast; fast *= (1-alpha). DEVICE pointers. */
int32_t pssa_b200_adapter_consolidate_dev(pssa_b200_ctx* ctx, float* up_fast, float* up_slow, size_t n, float alpha);

/* ------------------------------------------------------------------ dense product */

/* Epilogue applied to every output of pssa_b200_gemm_xwt (the reference's elementwise kernels
 * softplus_in_place / sigmoid_in_place / add_in_place, src/cuda/stages.ptx:541-607, folded in). */
typedef enum pssa_b200_epilogue {
    PSSA_B200_EPI_NONE = 0,
    PSSA_B200_EPI_SOFTPLUS = 1,
    PSSA_B200_EPI_SIGMOID = 2,
    PSSA_B200_EPI_SILU = 3,
    PSSA_B200_EPI_SCALE = 4,  /* out = acc * alpha */
    PSSA_B200_EPI_ADD_OUT = 5 /* out = out + acc */
} pssa_b200_epilogue;

/* Arithmetic of the dense products and of the whole model path. */
typedef enum pssa_b200_precision {
    PSSA_B200_PRECISION_BF16 = 0, /* bf16 operands on the tensor cores, fp32 accumulate; fp32 scan and retrieval */
    PSSA_B200_PRECISION_FP32_EXACT = 1 /* fp32 everywhere with the CPU reference's reduction order */
} pssa_b200_precision;

/*
 * Y[batch*M, N] = epilogue(X[batch*M, K] * W[N, K]^T): `dispatch_gemm_into` (src/backend.rs:1087-1110,
 * layout contract 41-48: the batch is folded into rows). HOST pointers, fp32. With
 * PSSA_B200_PRECISION_FP32_EXACT every output is the reference's `dot_slice` (src/linalg.rs:184-298) bit for
 * bit; with PSSA_B200_PRECISION_BF16 operands are rounded to bf16 and multiplied on the tensor cores.
 * `out` must hold batch*M*N floats; it is read only by PSSA_B200_EPI_ADD_OUT.
 */
int32_t pssa_b200_gemm_xwt(pssa_b200_ctx* ctx, const float* x, const float* w, size_t m, size_t n, size_t k,
                           size_t batch, float* out, int32_t epilogue, float alpha, int32_t precision);
/* Same on DEVICE pointers; `ldo` is the row pitch of out in floats (>= n). */
int32_t pssa_b200_gemm_xwt_dev(pssa_b200_ctx* ctx, const float* x, const float* w, size_t rows, size_t n, size_t k,
                               float* out, size_t ldo, int32_t epilogue, float alpha, int32_t precision);

/* ------------------------------------------------------------------ model */

/* `PSSAConfigV2` (src/pssa.rs:253-331) reduced to what the forward path reads. */
typedef struct pssa_b200_config {
    uint64_t depth, d_vocab, d_latent, d_state, d_mem_key, mem_capacity;
    float tau_mem;
    uint32_t reserved;
} pssa_b200_config;

/* Parameter / state identifiers for set_tensor and get_tensor (row-major fp32, reference shapes:
 * src/pssa.rs:506-620). EMBED, UNEMBED and RESIDUAL_SCALES are model-level (layer ignored). */
typedef enum pssa_b200_tensor {
    PSSA_B200_T_EMBED = 0,       /* [V, d] */
    PSSA_B200_T_UNEMBED = 1,     /* [V, d] */
    PSSA_B200_T_NORM_GAMMA = 2,  /* [d] */
    PSSA_B200_T_NORM_BETA = 3,   /* [d] */
    PSSA_B200_T_A_MAT = 4,       /* [d, s] raw; A = -softplus(raw) */
    PSSA_B200_T_W_DELTA = 5,     /* [d, d] */
    PSSA_B200_T_W_B = 6,         /* [s, d] */
    PSSA_B200_T_W_C = 7,         /* [s, d] */
    PSSA_B200_T_W_QX = 8,        /* [k, d] */
    PSSA_B200_T_W_QH = 9,        /* [k, d] */
    PSSA_B200_T_W_GATE = 10,     /* [d, d] */
    PSSA_B200_T_W_PROJ = 11,     /* [d, d] */
    PSSA_B200_T_MLP_W1 = 12,     /* [2d, d] */
    PSSA_B200_T_MLP_W2 = 13,     /* [d, 2d] */
    PSSA_B200_T_AD_DOWN = 14,    /* [16, d] */
    PSSA_B200_T_AD_UP = 15,      /* [d, 16] fast */
    PSSA_B200_T_AD_CONS = 16,    /* [d, 16] consolidated */
    PSSA_B200_T_RESIDUAL_SCALES = 22 /* [depth-1] */
} pssa_b200_tensor;

/* Allocates device storage for a model of `cfg` and `max_streams` independent recurrent carries
 * (`PSSALayerV2::new`, src/pssa.rs:2019-2072, without the random init: weights are uploaded, or drawn by
 * pssa_b200_model_init_random below). */
int32_t pssa_b200_model_create(pssa_b200_ctx* ctx, const pssa_b200_config* cfg, uint32_t max_streams,
                               pssa_b200_model** out);
void pssa_b200_model_destroy(pssa_b200_model* model);
/* Upload one parameter (host fp32). Replaces the reference backends' host-pointer-keyed weight cache and
 * its invalidation calls (src/cuda.rs:198-252, src/backend.rs:1113-1133): the caller re-uploads what changed. */
int32_t pssa_b200_model_set_tensor(pssa_b200_model* model, int32_t layer, int32_t tensor, const float* data, size_t len);
/* Read one parameter back (host fp32, `len` must be the tensor's length): what the reference reads straight from its
 * host-resident `ParamMatrix` fields when it saves a checkpoint (src/checkpoint.rs) or inspects a model. */
int32_t pssa_b200_model_get_tensor(pssa_b200_model* model, int32_t layer, int32_t tensor, float* out, size_t len);
/* Random initialisation with the reference's generator and draw order, so that the model holds the tensors of
 * `PSSALayerV2::new(cfg, seed)` bit for bit (src/pssa.rs:2019-2072, 630-690; src/linalg.rs:1-28, 338-344;
 * src/adapter.rs:16-24): embedding, block 0, head, further blocks; norm gain 1, bias 0, MLP down and the adapter's up
 * matrices zero, residual scales 1/sqrt(depth). Banks and carries are left as they are. `rng_state_out` (may be NULL)
 * receives the generator state after the last draw, which the reference keeps in the model for later draws. */
int32_t pssa_b200_model_init_random(pssa_b200_model* model, uint64_t seed, uint64_t* rng_state_out);
/* Upload one block's bank (src/memory.rs:4-33): keys [cap,k], norm_sq [cap], values [cap,d], count,
 * write_head, confidence [cap], last_seen_step [cap]. Checks the invariants of src/checkpoint.rs:1060-1066. */
int32_t pssa_b200_model_set_bank(pssa_b200_model* model, int32_t layer, const float* keys, const float* norm_sq,
                                 const float* values, uint64_t count, uint64_t write_head, const float* confidence,
                                 const uint64_t* last_seen_step);
/* `set_memory_top_k` (src/pssa.rs:2215-2229): 0 restores the all-slots read. The reference refuses this on a
 * GPU device; here it is the one runtime option the device path adds. */
int32_t pssa_b200_model_set_top_k(pssa_b200_model* model, size_t top_k);
int32_t pssa_b200_model_set_precision(pssa_b200_model* model, int32_t precision);
/* Runtime options. 0 local_conv, 1 ssm_skip, 2 hybrid_read, 3 grow_memory: the reference refuses these on any GPU device
 * (src/pssa.rs:2080-2105, 2189-2192, 2232-2243); enabling one returns PSSA_B200_ERR_UNSUPPORTED with the reference's
 * message. 4 = `set_loops` (src/pssa.rs:2171-2184): the runtime number of weight-shared Ouro passes per block, 1..32
 * (src/pssa.rs:2338-2376). Every pass owns a recurrent carry; changing the count keeps pass 0's carries and zeroes the
 * others (`resize_loop_tape`, src/pssa.rs:2147-2167), and the per-stream state becomes [block][pass][d*s].
 * 5 (no counterpart in the reference) = lane groups: a pass over several lanes can be enqueued as up to four groups of
 * consecutive lanes on side streams of the context, joined by events before the call returns (the groups share only
 * read-only weights, so results do not change): 0 = chosen from the shape, 1 = off, 2..4 = that many groups. */
int32_t pssa_b200_model_set_option(pssa_b200_model* model, int32_t option, int32_t value);

/* `reset_recurrent_state` (src/pssa.rs:2245-2250) for one stream. */
int32_t pssa_b200_model_reset_state(pssa_b200_model* model, uint32_t stream);
/* `copy_recurrent_state_to / from` (src/pssa.rs:2263-2310): [block][pass][d*s] fp32, len = depth*loops*d*s. */
int32_t pssa_b200_model_get_state(pssa_b200_model* model, uint32_t stream, float* out, size_t len);
int32_t pssa_b200_model_set_state(pssa_b200_model* model, uint32_t stream, const float* data, size_t len);

/*
 * `prefill_inference` (src/pssa.rs:2399-2442) on one stream: advances the carry over `n` tokens and, when
 * logits is not NULL, writes the last token's logits [V]. Empty input is an error; an id >= V stops after
 * the valid prefix (PSSA_B200_ERR_TOKEN, *processed = prefix length, logits untouched). `cancelled` (may be
 * NULL) is polled before every pass of at most max_rows tokens; a non-zero return stops with
 * PSSA_B200_ERR_CANCELLED, the carry holding the passes already done.
 */
int32_t pssa_b200_model_prefill(pssa_b200_model* model, uint32_t stream, const uint64_t* ids, size_t n, float* logits,
                                size_t* processed, int32_t (*cancelled)(void*), void* cancel_arg);
/*
 * Independent sequences packed in one id array (`SequenceBatch::forward`, src/sequence_batch.rs:233-384, with
 * a per-lane carry): lane l = ids[offsets[l] .. offsets[l]+lengths[l]) continuing stream streams[l]. All lanes
 * are validated before any work. logits (NULL to skip) receives [n_lanes, V]: each lane's last-token logits
 * (rows of zero-length lanes are left untouched). greedy (NULL to skip) receives each lane's greedy next
 * token (src/inference.rs:123-127).
 */
int32_t pssa_b200_model_prefill_batch(pssa_b200_model* model, const uint64_t* ids, const uint32_t* offsets,
                                      const uint32_t* lengths, const uint32_t* streams, size_t n_lanes, float* logits,
                                      uint64_t* greedy);
/*
 * Device-resident form of prefill_batch for callers that already hold token ids on the GPU (and want the logits
 * there): ids_dev [total rows] u32 DEVICE pointer, logits_dev [n_lanes, V] and greedy_dev [n_lanes] u32 DEVICE
 * pointers (either may be NULL); offsets / lengths / streams are HOST arrays as above. Ids are NOT range checked
 * (the caller vouches for ids < V); the whole batch must fit one pass (total rows <= max_rows). Work is only
 * enqueued on the context's stream: nothing is synchronised.
 */
int32_t pssa_b200_model_prefill_batch_dev(pssa_b200_model* model, const uint32_t* ids_dev, const uint32_t* offsets,
                                          const uint32_t* lengths, const uint32_t* streams, size_t n_lanes,
                                          float* logits_dev, uint32_t* greedy_dev);
/* `forward_inference` (src/pssa.rs:2387-2391) for n streams at once: one token each. */
int32_t pssa_b200_model_decode_step(pssa_b200_model* model, const uint32_t* streams, const uint64_t* ids, size_t n,
                                    float* logits, uint64_t* greedy);

/*
 * Token sampling on the device for batched decode: `PSSAInferenceEngine::sample` (src/inference.rs:102-181) for `rows`
 * streams at once. Per stream, in the reference's order: non-finite logits are an error; repetition penalty over the
 * last <= 64 generated ids (an id repeated in the window is penalised repeatedly); temperature 0 is the greedy rule
 * (ids 1..V-1, ties to the lowest id); otherwise softmax((l - max over ids >= 1) / T), candidates sorted by
 * (probability desc, id asc), top-k, top-p on the running sum, one `SimpleRng` draw (src/linalg.rs:13-26), pick.
 * DEVICE pointers: logits [rows, vocab] (modified by the penalty, as the reference modifies its slice), probs
 * [rows, vocab] scratch, recent_ids [rows, 64] + recent_count [rows] (NULL: no history), rng_state [rows] in/out,
 * ids_out [rows] (UINT32_MAX on error), status_out [rows] (0 ok, 1 "model emitted non-finite logits", 2 "invalid
 * sampling probability mass", 3 "no valid generation candidates"). Parameter validation follows
 * `validate` (src/inference.rs:87-101). PSSA_B200_SAMPLE_EXACT keeps the sequential f32 sum over the vocabulary.
 * confidence_out [rows] (NULL to skip): the raw softmax probability of the selected id over ALL ids, before penalty,
 * temperature and filtering (`raw_confidence`, src/inference.rs:526-545; what the scored generation callbacks report).
 */
typedef struct pssa_b200_sampling {
    float temperature;        /* >= 0, finite; 0 = greedy */
    float top_p;              /* (0, 1] */
    uint32_t top_k;           /* 1..4096 */
    float repetition_penalty; /* >= 1, finite */
} pssa_b200_sampling;
#define PSSA_B200_SAMPLE_EXACT 1u
int32_t pssa_b200_sample_dev(pssa_b200_ctx* ctx, float* logits, float* probs, size_t rows, size_t vocab,
                             const pssa_b200_sampling* cfg, const uint32_t* recent_ids, const uint32_t* recent_count,
                             uint64_t* rng_state, uint32_t* ids_out, uint32_t* status_out, float* confidence_out,
                             uint32_t flags);

/*
 * Frozen-model scorer: the forward half of the reference's chunk forward (src/pssa.rs:2597-2750 with one loop), which
 * `pssa score` / `pssa throughput` use on a frozen model (src/evaluation.rs:205-236): logits for EVERY position, then
 * the mean over positions of (max - l[target]) + ln(sum exp(l - max)). The stream's carry advances like a prefill.
 * Full-vocabulary logits are produced a tile of rows at a time and never held for the whole sequence.
 * HOST pointers: ids / targets [n]; mean_loss; token_loss [n] (NULL to skip); logits_out [n, vocab] (NULL to skip).
 */
int32_t pssa_b200_model_score(pssa_b200_model* m, uint32_t stream, const uint64_t* ids, const uint64_t* targets, size_t n,
                              float* mean_loss, float* token_loss, float* logits_out);

/*
 * Observer scratch: the reference keeps, per block, the retrieval state of the last token it processed
 * (`inf_mem_weights`, `inf_q_pnc`, `inf_m_val`, `inf_z_final`, src/pssa.rs:609-619) and hands it to generation
 * observers (src/inference.rs:257-313). With the observer enabled every forward call (prefill, batched prefill, decode
 * step) publishes those four vectors for the LAST token of every lane that has one in the call; `index` counts those
 * lanes in order. Each output may be NULL. HOST pointers: mem_weights [capacity], q_pnc [d_mem_key], m_val and z_final
 * [d_latent]. Costs one small copy kernel per block and the fp32 copy of m in the bf16 mode; off by default.
 */
int32_t pssa_b200_model_set_observer(pssa_b200_model* m, int32_t enabled);
int32_t pssa_b200_model_get_observation(pssa_b200_model* m, uint32_t layer, uint32_t index, float* mem_weights, float* q_pnc,
                                        float* m_val, float* z_final);

/*
 * `insert_training_memory_at` (src/pssa.rs:3705-3737) on the model's device-resident banks: if loss > 3.5, every block
 * gets one protected insert (refractory gate and ring insert of pssa_b200_bank_insert_protected_dev; hybrid read is
 * not supported, so never the gated variant) whose key is `q_poincare` and whose value is `z_final` of the LAST token of
 * observed lane `index` of the previous forward call -- the observer scratch, which must be enabled. `step` is the
 * reference's step counter (the gate's clock). slots_out [depth] (NULL to skip): the slot written, -1 defended, -2
 * refused, -3 nothing attempted (loss <= 3.5). A bank that changed gets its derived copies (key and value pieces, values
 * carried through W_proj) rebuilt before the next forward call. On replicas, apply the same writes in the same order.
 */
int32_t pssa_b200_model_insert_memory(pssa_b200_model* m, uint32_t index, float loss, uint64_t step, int64_t* slots_out);

/*
 * One decode step for `n` streams with the sampling done on the device: forward, vocabulary head, then
 * pssa_b200_sample_dev's kernel on the head's logits, so only `n` ids cross PCIe. Every stream owns a generator
 * (seed 1337 by default, like `PSSAInferenceEngine`, src/inference.rs:70-73) and the window of its last 64 sampled ids
 * that the repetition penalty reads; `sampler_seed` resets both for one stream (seed 0 maps to the reference's
 * non-zero constant, src/linalg.rs:7-11). ids_out [n] and confidence_out [n] (NULL to skip; see pssa_b200_sample_dev)
 * on the HOST.
 */
int32_t pssa_b200_model_sampler_seed(pssa_b200_model* m, uint32_t stream, uint64_t seed);
/* Appends ids to a stream's repetition window without sampling: the reference's penalty reads the last 64 entries of
 * `generated_ids`, which starts as a copy of the PROMPT (src/inference.rs:343-345, 114-121), so a host loop pushes the
 * prompt here before its first sampled step. Ids outside the vocabulary are refused like prompt ids. */
int32_t pssa_b200_model_sampler_push(pssa_b200_model* m, uint32_t stream, const uint64_t* ids, size_t n);
int32_t pssa_b200_model_decode_step_sampled(pssa_b200_model* m, const uint32_t* streams, const uint64_t* ids, size_t n,
                                            const pssa_b200_sampling* cfg, uint32_t flags, uint64_t* ids_out,
                                            float* confidence_out);

/*
 * `.pssa` checkpoint containers, versions 7 and 8 (and the version-6 single-block layout they extend), straight into a
 * device-resident model: the reference's `load_checkpoint` (src/checkpoint.rs:1344-1411; container header 1-27,
 * FNV-1a 89-95, block records 912-1010) reduced to what inference needs. Weights, banks with their metadata, the
 * residual scales and the stored carry (into stream 0) are uploaded; optimizer moments, vocabulary strings and
 * tokenizer metadata are validated for length and skipped. The whole file is checked on the host first (magic,
 * version, payload length, checksum, every array length, finite values), so a rejected file creates nothing.
 * `probe` is the host-only half: it needs no GPU and returns the configuration (error text into `error`).
 */
int32_t pssa_b200_checkpoint_probe(const void* bytes, size_t len, pssa_b200_config* config, uint32_t* version,
                                   char* error, size_t error_len);
int32_t pssa_b200_model_load_checkpoint(pssa_b200_ctx* ctx, const void* bytes, size_t len, uint32_t max_streams,
                                        pssa_b200_model** out);

/*
 * Sequence-parallel prefill: one long sequence (or several) split in TIME over `world` processes, one per GPU, each
 * holding contiguous time shard `rank` of every lane. Not a reference code path; it follows from the reference's scan
 * monoid (`compose_affine`, src/gpu_batch.rs:75-86): per block a rank reduces its shard to one affine map per
 * (channel, state) (the sum of delta and the shard's end state from a zero carry), the maps are all-gathered, every
 * rank folds the lower ranks' maps into its carry-in and runs the fused SSM; everything else in a block is token-local.
 * The library does not link a communication library: the caller supplies the all-gather.
 *   exchange(arg, send, recv, bytes) must, in stream order on the context's stream, place rank k's `bytes` at
 *   recv + k*bytes on every rank (an NCCL all-gather on that stream), and return 0.
 *   send / recv: DEVICE buffers owned by the caller, `capacity` records of (d + d*s) floats and world times that. A
 *   record is one (lane, time chunk): each lane's shard is cut into up to 16 chunks so that a launch fills the GPU
 *   even with few lanes; capacity >= lanes is required, lanes * 16 lets the library choose freely.
 * While enabled (world > 1), pssa_b200_model_prefill_batch_dev treats its lanes as this rank's shards: lane l must be
 * the same sequence on every rank (a rank may hold zero tokens of it), every rank gets the same final recurrent
 * state, and the logits a rank returns are those of ITS last token of each lane (the caller keeps the last
 * non-empty rank's). Every rank must hold at least one token of some lane; the library can only check its own rank, so
 * the caller validates this on all ranks together (from the sequence lengths, which every rank knows) before any rank
 * calls, otherwise the ranks that do hold tokens wait in the exchange for the one that returned an error.
 * world <= 1 or exchange == NULL switches it off.
 */
typedef int32_t (*pssa_b200_exchange_fn)(void* arg, const void* send_dev, void* recv_dev, size_t bytes);
int32_t pssa_b200_model_set_seqpar(pssa_b200_model* m, uint32_t rank, uint32_t world, void* send_dev, void* recv_dev,
                                   size_t capacity, pssa_b200_exchange_fn exchange, void* arg);
/* Upper bound on token rows processed per pass (activation workspace = about 40 KB per row at d 768). */
int32_t pssa_b200_model_set_max_rows(pssa_b200_model* model, size_t max_rows);
/* Allocates now everything a later call of at most `rows` token rows (capped by max_rows per pass) over at most `lanes`
 * lanes would allocate on first use: the activation workspace, the time-chunk buffers and the sampler state. The
 * reference sizes its scratch at construction (`ChunkActivationTape::new`, src/pssa.rs:630-700; packed lanes
 * src/cuda/packed.rs:282-366); here it grows on demand unless reserved, and growth synchronises the stream. */
int32_t pssa_b200_model_reserve(pssa_b200_model* model, size_t rows, size_t lanes);

#ifdef __cplusplus
}
#endif
#endif /* PSSA_B200_H */
