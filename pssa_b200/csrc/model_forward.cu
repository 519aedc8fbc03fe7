// Batched forward over packed lanes: the reference's staged block schedule on device-resident buffers.
#include <algorithm>
#include <cmath>
#include <cstring>

#include "bounds.hpp"
#include "context.hpp"
#include "device_math.cuh"
#include "kernels.hpp"
#include "model.hpp"

using namespace pssa;

namespace {

struct Carver {
    size_t off = 0;
    size_t take(size_t bytes) {
        size_t o = (off + 255) & ~size_t(255);
        off = o + bytes;
        return o;
    }
};

// one allocation carved into the per-row activation buffers; grows when a larger pass is requested
int32_t ensure_workspace(pssa_b200_model* m, size_t rows, size_t lanes) {
    Workspace& ws = m->ws;
    if (ws.base && rows <= ws.rows && lanes <= ws.lanes) return PSSA_B200_OK;
    pssa_b200_ctx* ctx = m->ctx;
    rows = std::max(rows, ws.rows);
    lanes = std::max(lanes, ws.lanes);
    const size_t d = m->d, f = sizeof(float);
    Carver c;
    size_t o_ids = c.take(rows * 4), o_off = c.take(lanes * 4), o_len = c.take(lanes * 4), o_slot = c.take(lanes * 4),
           o_last = c.take(lanes * 4), o_greedy = c.take(lanes * 4);
    size_t o_fc = c.take(m->loops > 1 ? rows * d * f : 0);
    size_t o_fa = c.take(rows * d * f), o_fb = c.take(rows * d * f), o_xn = c.take(rows * d * f),
           o_proj = c.take(rows * m->ncat * f), o_y = c.take(rows * d * f), o_w = c.take(rows * m->cap * f),
           o_mv = c.take(rows * d * f), o_mp = c.take(rows * d * f), o_z = c.take(rows * d * f),
           o_act = c.take(rows * 2 * d * f), o_lf = c.take(lanes * d * f), o_lg = c.take(lanes * m->v * f);
    size_t o_xb = c.take(rows * d * 2), o_yb = c.take(rows * d * 2), o_mb = c.take(rows * d * 2), o_zb = c.take(rows * (d + 64) * 2),
           o_ab = c.take(rows * (2 * d + 64) * 2), o_wsp = c.take(rows * 3 * m->cap * 2), o_qsp = c.take(rows * 3 * m->k * 2),
           o_qst = c.take(rows * sizeof(float2)), o_fix = c.take(8 * 4);  // counters of the one-kernel top-k read, one per lane group
    size_t total = c.take(0);
    PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ws.base) cudaFree(ws.base);
    ws = Workspace();
    cudaError_t e = cudaMalloc((void**)&ws.base, total);
    if (e != cudaSuccess) {
        ws = Workspace();
        return cuda_fail(ctx, e, "activation workspace allocation");
    }
    // the 48 pad columns of the MLP operands' extra K block are never written again and must read as zero
    PSSA_CUDA(ctx, cudaMemsetAsync(ws.base, 0, total, ctx->stream));
    ws.bytes = total, ws.rows = rows, ws.lanes = lanes;
    char* b = ws.base;
    ws.ids = (uint32_t*)(b + o_ids), ws.lane_off = (uint32_t*)(b + o_off), ws.lane_len = (uint32_t*)(b + o_len);
    ws.lane_slot = (uint32_t*)(b + o_slot), ws.last_rows = (uint32_t*)(b + o_last), ws.greedy = (uint32_t*)(b + o_greedy);
    ws.feat_c = m->loops > 1 ? (float*)(b + o_fc) : nullptr;
    ws.feat_a = (float*)(b + o_fa), ws.feat_b = (float*)(b + o_fb), ws.x_norm = (float*)(b + o_xn);
    ws.proj = (float*)(b + o_proj), ws.y = (float*)(b + o_y), ws.weights = (float*)(b + o_w), ws.m_val = (float*)(b + o_mv);
    ws.m_proj = (float*)(b + o_mp), ws.z = (float*)(b + o_z), ws.mlp_act = (float*)(b + o_act);
    ws.last_feat = (float*)(b + o_lf), ws.logits = (float*)(b + o_lg);
    ws.x_bf16 = b + o_xb, ws.y_bf16 = b + o_yb, ws.m_bf16 = b + o_mb, ws.z_bf16 = b + o_zb, ws.act_bf16 = b + o_ab, ws.w_split = b + o_wsp;
    ws.q_split = b + o_qsp, ws.q_stat = (float2*)(b + o_qst), ws.fixup = (uint32_t*)(b + o_fix);
    return PSSA_B200_OK;
}

// buffers of the two-pass (time-chunked) SSM; grow on demand
int32_t ensure_chunks(pssa_b200_model* m, size_t vlanes) {
    auto& c = m->chunks;
    if (vlanes <= c.capacity) return PSSA_B200_OK;
    pssa_b200_ctx* ctx = m->ctx;
    PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    cudaFree(c.off), cudaFree(c.len), cudaFree(c.records), cudaFree(c.carry_in);
    c = pssa_b200_model::Chunks{};
    const size_t ds = m->d * m->s;
    PSSA_CUDA(ctx, cudaMalloc((void**)&c.off, vlanes * 4));
    PSSA_CUDA(ctx, cudaMalloc((void**)&c.len, vlanes * 4));
    PSSA_CUDA(ctx, cudaMalloc((void**)&c.records, vlanes * (m->d + ds) * sizeof(float)));
    PSSA_CUDA(ctx, cudaMalloc((void**)&c.carry_in, vlanes * ds * sizeof(float)));
    c.capacity = vlanes;
    return PSSA_B200_OK;
}

// refresh the bf16 weight copies the tensor-core path reads (concatenated x-side projections)
int32_t refresh_bf16(pssa_b200_model* m) {
    pssa_b200_ctx* ctx = m->ctx;
    const size_t d = m->d;
    int32_t rc;
    for (auto& b : m->blocks) {
        if (!b.bf16_dirty) continue;
        char* cat = (char*)b.wcat_bf16;
        struct Part { int id; size_t row_off, rows; };
        Part parts[] = {{T_W_DELTA, m->off_delta, d}, {T_W_B, m->off_b, m->s},       {T_W_C, m->off_c, m->s},
                        {T_W_QX, m->off_q, m->k},     {T_W_GATE, m->off_gate, d},    {T_AD_DOWN, m->off_act, m->rank}};
        for (auto& p : parts)
            if ((rc = launch_to_bf16(ctx, b.w[p.id], cat + p.row_off * d * 2, p.rows * d))) return rc;
        if ((rc = launch_to_bf16(ctx, b.w[T_W_QH], b.wqh_bf16, m->k * d))) return rc;
        if ((rc = launch_to_bf16(ctx, b.w[T_W_PROJ], b.wproj_bf16, d * d))) return rc;
        // MLP matrices with the adapter block appended (rank 16): W1 | W1*U | 0 and W2 | U | 0
        if ((rc = launch_times_adapter(ctx, b.w[T_MLP_W1], b.u_eff, b.w1u, 2 * d, (int)d))) return rc;
        if ((rc = launch_pack_weight_cat(ctx, b.w[T_MLP_W1], b.w1u, b.w1cat_bf16, 2 * d, (int)d))) return rc;
        if ((rc = launch_pack_weight_cat(ctx, b.w[T_MLP_W2], b.u_eff, b.w2cat_bf16, d, (int)(2 * d)))) return rc;
        b.bf16_dirty = false;
    }
    for (auto& b : m->blocks) {
        if (!b.vsplit_dirty) continue;
        if ((rc = launch_split_values(ctx, b.w[T_BANK_VALUES], b.vsplit_bf16, (int)m->cap, (int)d))) return rc;
        b.vsplit_dirty = false;
    }
    for (auto& b : m->blocks) {
        if (!b.vp_dirty) continue;
        // vp = V W_proj^T in fp32 (every entry one dot product in the reference's order), then transposed bf16 pieces
        if ((rc = launch_gemm_exact(ctx, b.w[T_BANK_VALUES], b.w[T_W_PROJ], b.vp, m->cap, d, d, d, EPI_NONE, 1.0f))) return rc;
        if ((rc = launch_split_values(ctx, b.vp, b.vpsplit_bf16, (int)m->cap, (int)d))) return rc;
        b.vp_dirty = false;
    }
    if (m->unembed_dirty) {
        if ((rc = launch_to_bf16(ctx, m->unembed, m->unembed_bf16, m->v * d))) return rc;
        m->unembed_dirty = false;
    }
    return PSSA_B200_OK;
}

// the bank's keys as bf16 pieces (tensor-core distances of the bf16 mode; the pre-filter of the exact top-k read in both modes)
// side streams and fork / join events of the lane groups, created on first use
int32_t ensure_side_streams(pssa_b200_ctx* ctx, size_t n) {
    for (size_t i = 0; i < n && i < 3; ++i) {
        if (!ctx->side[i]) PSSA_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->side[i], cudaStreamNonBlocking));
        if (!ctx->join_ev[i]) PSSA_CUDA(ctx, cudaEventCreateWithFlags(&ctx->join_ev[i], cudaEventDisableTiming));
    }
    if (!ctx->fork_ev) PSSA_CUDA(ctx, cudaEventCreateWithFlags(&ctx->fork_ev, cudaEventDisableTiming));
    return PSSA_B200_OK;
}

int32_t refresh_key_splits(pssa_b200_model* m) {
    int32_t rc;
    for (auto& b : m->blocks) {
        if (!b.ksplit_dirty) continue;
        if ((rc = launch_split_keys(m->ctx, b.w[T_BANK_KEYS], b.w[T_BANK_NORM_SQ], b.ksplit_bf16, b.kstat, (int)m->cap, (int)m->k))) return rc;
        b.ksplit_dirty = false;
    }
    return PSSA_B200_OK;
}

// out[rows, ldo](first n cols) = epilogue(X * W^T): exact fp32 or bf16 tensor cores
int32_t dense(pssa_b200_model* m, const float* x32, const void* x16, const float* w32, const void* w16, float* out, size_t rows,
              size_t n, size_t k, size_t ldo, int epi, float alpha, void* out_bf16 = nullptr) {
    if (m->precision == PSSA_B200_PRECISION_FP32_EXACT) return launch_gemm_exact(m->ctx, x32, w32, out, rows, n, k, ldo, epi, alpha);
    return launch_gemm_bf16(m->ctx, x16, w16, out, out_bf16, rows, n, k, ldo, epi, alpha);
}

// One pass: `rows` packed token rows of `lanes` lanes already described in the workspace (ids, lane_off, lane_len,
// lane_slot, last_rows). Leaves the final features of every row in ws.feat_a or feat_b (returned).
int32_t forward_rows(pssa_b200_model* m, size_t rows, size_t lanes, const uint32_t* h_off, const uint32_t* h_len, float** feats_out,
                     size_t n_obs = 0) {
    pssa_b200_ctx* ctx = m->ctx;
    Workspace& ws = m->ws;
    const bool exact = m->precision == PSSA_B200_PRECISION_FP32_EXACT;
    const int d = (int)m->d, s = (int)m->s, k = (int)m->k;
    const size_t nc = m->ncat, ds = m->d * m->s;
    const float ssm_scale = 1.0f / std::sqrt((float)s);
    int32_t rc;
    if (!exact && (rc = refresh_bf16(m))) return rc;
    if ((rc = refresh_key_splits(m))) return rc;
    float* feat_in = nullptr;
    float* feat_out = ws.feat_a;
    bool single_token = true;  // a decode step: the SSM stage is then one pass over the carries
    uint32_t max_len = 0;
    for (size_t l = 0; l < lanes; ++l) single_token = single_token && h_len[l] <= 1, max_len = std::max(max_len, h_len[l]);
    // Time chunks. The fused SSM kernel parallelises over lanes x channels only; with few lanes (long sequences) that
    // leaves most SMs idle, so each lane is cut into `n_chunks` consecutive time chunks that run as independent
    // "virtual lanes" in two passes: chunk maps from a zero carry, a fold of the maps in time order, then the real pass
    // with each chunk's carry-in. Every exp is paid twice, so this is only done when the plain launch would occupy at
    // most one CTA per SM -- or in the sequence-parallel mode, where the two passes are paid anyway.
    const size_t ctas = lanes * ((m->d + 63) / 64);
    const size_t slots = (size_t)ctx->sm_count * 4;
    size_t n_chunks = 1;
    if (m->sp.active) {
        // Must be identical on every rank (it sizes the all-gather and the record order the fold walks), so it depends
        // only on quantities every rank shares: the lane count, the model width, the SM count and the exchange capacity --
        // never on this rank's shard lengths, which differ between ranks (a shard may even be a single token).
        n_chunks = std::min<size_t>(16, std::max<size_t>(1, slots / ctas));
        n_chunks = std::min(n_chunks, std::max<size_t>(1, m->sp.capacity / lanes));
    } else if (!single_token && ctas <= (size_t)ctx->sm_count) {
        n_chunks = std::min<size_t>(16, std::max<size_t>(1, slots / ctas));
        n_chunks = std::min(n_chunks, std::max<size_t>(1, max_len / 128));
    }
    const bool two_pass = m->sp.active || n_chunks > 1;
    const size_t vlanes = lanes * n_chunks;
    if (two_pass) {
        if (m->sp.active && vlanes > m->sp.capacity)
            return fail(ctx, PSSA_B200_ERR_SHAPE, "sequence-parallel prefill: %zu lanes exceed the %zu records the exchange buffers hold",
                        lanes, m->sp.capacity);
        if ((rc = ensure_chunks(m, vlanes))) return rc;
        std::vector<uint32_t> v_off(vlanes), v_len(vlanes);
        for (size_t l = 0; l < lanes; ++l)
            for (size_t c = 0; c < n_chunks; ++c) {
                const uint32_t a = (uint32_t)((uint64_t)h_len[l] * c / n_chunks), e = (uint32_t)((uint64_t)h_len[l] * (c + 1) / n_chunks);
                v_off[l * n_chunks + c] = h_off[l] + a, v_len[l * n_chunks + c] = e - a;
            }
        // Uploaded only when the description changed: a repeated call (every step of a benchmark, every pass of a long
        // prompt with equal pass lengths) makes no copy and no synchronisation. The source vectors live in the model;
        // the one wait below is for earlier copies that may still read the vectors about to be replaced.
        if (v_off != m->chunks.host_off || v_len != m->chunks.host_len) {
            PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // earlier copies out of the vectors about to be replaced
            m->chunks.host_off.swap(v_off), m->chunks.host_len.swap(v_len);
            PSSA_CUDA(ctx, cudaMemcpyAsync(m->chunks.off, m->chunks.host_off.data(), vlanes * 4, cudaMemcpyHostToDevice, ctx->stream));
            PSSA_CUDA(ctx, cudaMemcpyAsync(m->chunks.len, m->chunks.host_len.data(), vlanes * 4, cudaMemcpyHostToDevice, ctx->stream));
        }
    }
    const bool observe = m->obs.enabled && n_obs > 0;
    const size_t obs_rec = m->cap + m->k + 2 * m->d;
    if (observe) {
        auto& ob = m->obs;
        if (rows > ob.q_rows) {
            PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            cudaFree(ob.q_pnc), ob.q_pnc = nullptr, ob.q_rows = 0;
            PSSA_CUDA(ctx, cudaMalloc((void**)&ob.q_pnc, rows * m->k * sizeof(float)));
            ob.q_rows = rows;
        }
        if (n_obs > ob.lanes) {
            PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            cudaFree(ob.buf), ob.buf = nullptr, ob.lanes = 0;
            PSSA_CUDA(ctx, cudaMalloc((void**)&ob.buf, m->depth * n_obs * obs_rec * sizeof(float)));
            ob.lanes = n_obs;
        }
        ob.valid_lanes = n_obs;
    }
    // Lane groups. The lanes of a pass can be cut into up to four groups of consecutive lanes, each enqueued on its own
    // stream: the groups share nothing but the read-only weights and banks (every activation buffer is per row, every
    // carry per lane), so the device is free to run one group's tensor-core products beside another group's SSM (the two
    // are bound by different pipes), to fill the tail of one kernel's last wave with the next group's CTAs, and, for a
    // decode step (a chain of small, latency-bound launches), to run the chains side by side. Fork and join are events
    // between the context's stream and the side streams, so a caller capturing the call in a CUDA graph gets the same
    // parallel branches. Off for the two-pass SSM and the observer, whose scratch is not per row.
    size_t n_groups = 1;
    {
        bool contiguous = true;  // groups are row ranges: lane l must start where lane l-1 ends
        size_t expect = 0;
        for (size_t l = 0; l < lanes; ++l) contiguous = contiguous && h_off[l] == expect, expect += h_len[l];
        // Measured at the benchmark's shapes (32 x 2048-token lanes; 256 decode streams) two groups are SLOWER than one
        // stream (24.1 against 23.1 ms per prefill step, 1.70 against 1.37 ms per decode step): every tensor-core CTA
        // takes a whole SM's registers and shared memory, so kernels of different groups queue behind each other instead
        // of sharing SMs, and each is smaller. Kernel variants slim enough for two CTAs per SM (tensor-core CTAs with four
        // epilogue warps and a two-stage ring under 116 KB, SSM CTAs with a two-stage ring) were tried for the grouped case
        // and measured slower still (28.4 ms, 1.77 ms), so they are not kept. The automatic choice is one group; the
        // option stays for other shapes.
        size_t want = m->lane_groups == 0 ? 1 : m->lane_groups;
        if (!two_pass && !observe && contiguous)
            n_groups = std::max<size_t>(1, std::min<size_t>(std::min<size_t>(want, 4), lanes));
    }
    struct Group { size_t r0, nr, l0, nl; };
    Group groups[4];
    {
        size_t lane = 0, row = 0;
        for (size_t g = 0; g < n_groups; ++g) {
            Group& gr = groups[g];
            gr.l0 = lane, gr.r0 = row;
            if (g + 1 == n_groups) {
                lane = lanes, row = rows;
            } else {  // at least one lane, at least one left for every later group, rows as even as whole lanes allow
                const size_t target = rows * (g + 1) / n_groups;
                do row += h_len[lane], ++lane;
                while (lane < lanes - (n_groups - 1 - g) && row + h_len[lane] / 2 <= target);
            }
            gr.nl = lane - gr.l0, gr.nr = row - gr.r0;
        }
    }
    if (n_groups > 1 && (rc = ensure_side_streams(ctx, n_groups - 1))) return rc;
    cudaStream_t const main_stream = ctx->stream;
    // the slice the stages below work on (set per group by the driver loop)
    size_t r0 = 0, nr = rows, l0 = 0, nl = lanes, gi = 0;
    Workspace v = ws;
    auto select = [&](size_t g) {
        const Group& gr = groups[g];
        gi = g, r0 = gr.r0, nr = gr.nr, l0 = gr.l0, nl = gr.nl;
        v = ws;
        const size_t dd = m->d;
        v.ids += r0, v.x_norm += r0 * dd, v.proj += r0 * nc, v.y += r0 * dd, v.weights += r0 * m->cap, v.m_val += r0 * dd, v.m_proj += r0 * dd;
        v.z += r0 * dd, v.mlp_act += r0 * 2 * dd, v.q_stat += r0;
        v.x_bf16 = (char*)ws.x_bf16 + r0 * dd * 2, v.y_bf16 = (char*)ws.y_bf16 + r0 * dd * 2, v.m_bf16 = (char*)ws.m_bf16 + r0 * dd * 2;
        v.z_bf16 = (char*)ws.z_bf16 + r0 * (dd + 64) * 2, v.act_bf16 = (char*)ws.act_bf16 + r0 * (2 * dd + 64) * 2;
        v.w_split = (char*)ws.w_split + r0 * 3 * m->cap * 2, v.q_split = (char*)ws.q_split + r0 * 3 * m->k * 2;
        ctx->stream = g == 0 ? main_stream : ctx->side[g - 1];
        ctx->chain = (int)g;
    };
    auto fork = [&]() -> int32_t {
        if (n_groups <= 1) return PSSA_B200_OK;
        PSSA_CUDA(ctx, cudaEventRecord(ctx->fork_ev, main_stream));
        for (size_t g = 1; g < n_groups; ++g) {
            PSSA_CUDA(ctx, cudaStreamWaitEvent(ctx->side[g - 1], ctx->fork_ev, 0));
            if (ctx->profiling) ctx->stream = ctx->side[g - 1], ctx->chain = (int)g, profile_record(ctx, nullptr);  // a chain starts here
        }
        ctx->stream = main_stream, ctx->chain = 0;
        return PSSA_B200_OK;
    };
    auto join = [&]() -> int32_t {
        ctx->stream = main_stream, ctx->chain = 0;
        for (size_t g = 1; g < n_groups; ++g) {
            PSSA_CUDA(ctx, cudaEventRecord(ctx->join_ev[g - 1], ctx->side[g - 1]));
            PSSA_CUDA(ctx, cudaStreamWaitEvent(main_stream, ctx->join_ev[g - 1], 0));
        }
        return PSSA_B200_OK;
    };
    // One application of block `l` on carry `li` (Ouro pass; 0 for the ordinary model) for the selected group: reads
    // `feat_in` (nullptr: the embedding rows of the ids), writes feat_out = res_in ? res_in + rscale * z : z, z being the
    // block's output. Feature pointers are absolute; the group's row offset is applied here.
    auto run_pass = [&](size_t l, size_t li, const float* feat_in, const float* res_in, float rscale, float* feat_out, bool publish) -> int32_t {
        DeviceBlock& b = m->blocks[l];
        float* const carry_base = m->state + (l * m->loops + li) * ds;
        const size_t carry_stride = m->depth * m->loops * ds;
        if (feat_in) feat_in += r0 * (size_t)d;
        if (res_in) res_in += r0 * (size_t)d;
        feat_out += r0 * (size_t)d;
        // stage 1: gather + RMSNorm (src/gpu_batch.rs:445-472)
        if ((rc = launch_embed_norm(ctx, m->embed, feat_in ? nullptr : v.ids, feat_in, b.w[T_NORM_GAMMA], b.w[T_NORM_BETA],
                                    v.x_norm, exact ? nullptr : v.x_bf16, nr, d, exact, m->v)))
            return rc;
        // stage 2: x-side projections (src/gpu_batch.rs:477-536 plus the query/gate/adapter rows that read x_norm)
        if (exact) {
            struct P { int id; size_t off, n; int epi; };
            P ps[] = {{T_W_DELTA, m->off_delta, m->d, EPI_SOFTPLUS}, {T_W_B, m->off_b, m->s, EPI_NONE},
                      {T_W_C, m->off_c, m->s, EPI_NONE},            {T_W_QX, m->off_q, m->k, EPI_NONE},
                      {T_W_GATE, m->off_gate, m->d, EPI_SIGMOID},   {T_AD_DOWN, m->off_act, m->rank, EPI_SILU}};
            for (auto& p : ps)
                if ((rc = launch_gemm_exact(ctx, v.x_norm, b.w[p.id], v.proj + p.off, nr, p.n, m->d, nc, p.epi, 1.0f))) return rc;
        } else {
            // the adapter activations (last column range) also go, as bf16, into the extra K block of both MLP operands
            if ((rc = launch_gemm_bf16_cat(ctx, v.x_bf16, b.wcat_bf16, v.proj, nr, nc, m->d, nc, (int)m->off_b, (int)m->off_gate,
                                           (int)m->off_act, (char*)v.z_bf16 + m->d * 2, m->d + 64, (char*)v.act_bf16 + 2 * m->d * 2,
                                           2 * m->d + 64)))
                return rc;
        }
        // stage 3: SSM with the lane carries of this block (src/gpu_batch.rs:582-619)
        SsmParams sp{};
        sp.delta = ws.proj + m->off_delta, sp.x_norm = ws.x_norm, sp.b_proj = ws.proj + m->off_b, sp.c_proj = ws.proj + m->off_c;
        sp.rates = b.rates, sp.carry = carry_base, sp.y = ws.y, sp.y_bf16 = exact ? nullptr : ws.y_bf16;
        sp.offsets = ws.lane_off + l0, sp.lengths = ws.lane_len + l0, sp.rows = rows, sp.d = d, sp.s = s, sp.lanes = (int)nl;  // lanes of this group; rows stay absolute
        sp.ld_delta = nc, sp.ld_bc = nc, sp.lane_slots = ws.lane_slot + l0, sp.carry_stride = carry_stride;
        sp.aligned = ssm_vector_ok(sp);
        sp.single_token = single_token;
        if (two_pass) {
            // pass 1: every chunk's affine map (sum of delta, end state from a zero carry), one record per virtual lane
            const size_t rec = (size_t)d + ds;
            float* records = m->sp.active ? m->sp.send : m->chunks.records;
            PSSA_CUDA(ctx, cudaMemsetAsync(records, 0, vlanes * rec * sizeof(float), ctx->stream));
            SsmParams ag = sp;
            ag.offsets = m->chunks.off, ag.lengths = m->chunks.len, ag.lanes = (int)vlanes;
            ag.carry = records + d, ag.carry_stride = rec, ag.lane_slots = nullptr;
            ag.sum_delta = records, ag.sum_delta_stride = rec;
            ag.y_bf16 = nullptr, ag.single_token = 0;  // y of this pass is scratch: the real pass below overwrites it
            if ((rc = launch_ssm_fused(ctx, ag, exact))) return rc;
            const float* gathered = records;
            int world = 1, rank = 0;
            if (m->sp.active) {
                // all-gather of the records over the ranks (the caller's NCCL, in stream order)
                if (m->sp.fn(m->sp.arg, m->sp.send, m->sp.recv, vlanes * rec * sizeof(float)) != 0)
                    return fail(ctx, PSSA_B200_ERR_CUDA, "sequence-parallel prefill: the caller's exchange failed at block %zu", l);
                gathered = m->sp.recv, world = (int)m->sp.world, rank = (int)m->sp.rank;
            }
            // fold in time order: carry-in of each of this rank's chunks, and the lanes' final state
            if ((rc = launch_seqpar_fold(ctx, gathered, rec, world, rank, (int)n_chunks, (int)lanes, vlanes * rec, b.rates,
                                         carry_base, carry_stride, ws.lane_slot, m->chunks.carry_in, d, s)))
                return rc;
            // pass 2: the real one, over the virtual lanes with their carry-ins (carry-outs are scratch)
            sp.offsets = m->chunks.off, sp.lengths = m->chunks.len, sp.lanes = (int)vlanes;
            sp.carry = m->chunks.carry_in, sp.carry_stride = ds, sp.lane_slots = nullptr, sp.single_token = 0;
        }
        if ((rc = launch_ssm_fused(ctx, sp, exact))) return rc;
        // stage 4: query, projection into the ball, bank read, gate (src/gpu_batch.rs:748-929)
        if ((rc = dense(m, v.y, v.y_bf16, b.w[T_W_QH], b.wqh_bf16, v.proj + m->off_q, nr, m->k, m->d, nc, EPI_ADD_OUT, 1.0f))) return rc;
        RetrieveParams rp{};
        const bool obs_now = observe && publish;
        rp.q = v.proj + m->off_q, rp.ldq = nc, rp.q_is_euclidean = 1, rp.q_pnc = obs_now ? m->obs.q_pnc : nullptr, rp.q_norm = nullptr;
        rp.keys = b.w[T_BANK_KEYS], rp.norm_sq = b.w[T_BANK_NORM_SQ], rp.values = b.w[T_BANK_VALUES];
        rp.weights = v.weights, rp.m_val = (exact || obs_now) ? v.m_val : nullptr, rp.m_bf16 = exact ? nullptr : v.m_bf16, rp.min_dist = nullptr;
        // the bf16 mode keeps only the bf16 copy of m (the W_proj operand), so its value read is one plain bf16 product of the
        // leading pieces (the three-term read cost 70 us more per block for a logit error of 9.1e-3 instead of 9.3e-3)
        rp.value_terms = exact ? 6 : 1;
        rp.rows = nr, rp.dk = k, rp.dv = d, rp.cap = (int)m->cap, rp.count = (int)b.count;
        rp.top_k = (int)std::min(m->top_k, m->cap), rp.tau = m->cfg.tau_mem;
        rp.single_token = single_token ? 1 : 0;
        rp.f32_distance = !exact;  // the bf16 mode's queries carry bf16 rounding already; f64 distances buy nothing there
        if (!exact && m->cap % 64 == 0) rp.w_split = v.w_split, rp.v_split = b.vsplit_bf16;
        // only the observer reads the fp32 weight rows after the value read
        rp.skip_weights = rp.w_split && !obs_now && !(rp.top_k != 0 && rp.top_k < rp.count);
        if (k % 64 == 0) rp.k_split = b.ksplit_bf16, rp.k_stat = b.kstat;
        if (!exact && k % 64 == 0) rp.q_split = v.q_split, rp.q_stat = v.q_stat;
        rp.fixup_count = ws.fixup + gi;  // exact top-k in one kernel when the shape allows it
        const bool topk_now = rp.top_k != 0 && rp.top_k < rp.count;
        const bool topk_fused = topk_now && retrieve_fused_eligible(rp);
        if (topk_now && !topk_fused) {
            // A top-k read the one-kernel path cannot take (capacity, key width or fill outside its shapes) keeps the
            // reference's f64 distances in both precisions: a selection made from approximate distances can differ from the
            // reference's where the k-th and (k+1)-th slots are closer than the approximation, and identical slot sets
            // are worth more here than the speed of the fast distances.
            rp.f32_distance = 0, rp.q_split = nullptr, rp.q_stat = nullptr;
        }
        if (!obs_now) rp.weights = topk_fused ? nullptr : v.weights;
        // All-slots read in the bf16 mode: W_proj (sum_s w_s v_s) = sum_s w_s (W_proj v_s). The bank's values were carried
        // through W_proj at upload (vpsplit_bf16), so the product of the weight rows with them IS the memory projection and
        // takes the gate epilogue directly: the value read stops after the softmax (no m, no separate W_proj launch). The
        // observer wants m itself and keeps the two-product schedule.
        const bool proj_in_read = !exact && !(observe && publish) && rp.w_split && !(rp.top_k != 0 && rp.top_k < rp.count) && rp.count > 0;
        rp.skip_value_read = proj_in_read;
        // the one-kernel all-slots read leaves the division by the row sums to the epilogue of the product that follows
        // (its per-row factors borrow the buffer of the separate path's query statistics, which it does not use)
        if (proj_in_read) rp.row_scale_out = reinterpret_cast<float*>(v.q_stat);
        const float* weight_row_scale = (proj_in_read && retrieve_all_fused_runs(rp, exact)) ? rp.row_scale_out : nullptr;
        if ((rc = launch_memory_read(ctx, rp, exact))) return rc;
        // stages 5-6: adapter up + aggregation, then the SiLU MLP with its residual (src/gpu_batch.rs:934-1072)
        if (exact) {
            if ((rc = launch_gemm_exact(ctx, v.m_val, b.w[T_W_PROJ], v.m_proj, nr, m->d, m->d, m->d, EPI_NONE, 1.0f))) return rc;
            if ((rc = launch_combine_zraw(ctx, v.y, v.proj + m->off_gate, nc, v.m_proj, v.proj + m->off_act, nc, b.u_eff, v.z, nullptr,
                                          nr, d, (int)m->rank, ssm_scale)))
                return rc;
            if ((rc = launch_gemm_exact(ctx, v.z, b.w[T_MLP_W1], v.mlp_act, nr, 2 * m->d, m->d, 2 * m->d, EPI_SILU, 1.0f))) return rc;
            // MLP down projection + residual, then depth stacking (src/pssa.rs:2332-2337): block 0 has no outer residual
            if ((rc = launch_gemm_exact(ctx, v.mlp_act, b.w[T_MLP_W2], v.z, nr, m->d, 2 * m->d, m->d, EPI_ADD_OUT, 1.0f))) return rc;
            if ((rc = launch_residual(ctx, res_in, v.z, feat_out, nr * (size_t)d, rscale))) return rc;
        } else {
            // Tensor-core schedule: z = y/sqrt(s) + g*(W_proj m) + U*act never exists as one array. The memory projection's
            // epilogue forms zp = g*acc + y/sqrt(s), kept as bf16 only: it is W1's operand and W2's additive input (an fp32
            // copy for the latter moved 200 MB more per block each way and did not change the logit error); the rank-16 adapter
            // term is one extra K block of both MLP products: W1*(zp + U act) = [W1 | W1 U] [zp; act] and
            // W2*h + U*act = [W2 | U] [h; act]. The combine kernel and the m_proj round trip disappear.
            const size_t ldz = m->d + 64, lda = 2 * m->d + 64;
            if (proj_in_read) {
                if ((rc = launch_gemm_bf16_gate(ctx, v.w_split, b.vpsplit_bf16, nullptr, v.z_bf16, ldz, v.proj + m->off_gate, nc, v.y, ssm_scale,
                                                nr, m->d, m->cap, /*split_k=*/true, weight_row_scale)))
                    return rc;
            } else if ((rc = launch_gemm_bf16_gate(ctx, v.m_bf16, b.wproj_bf16, nullptr, v.z_bf16, ldz, v.proj + m->off_gate, nc, v.y, ssm_scale,
                                                   nr, m->d, m->d)))
                return rc;
            if ((rc = launch_gemm_bf16(ctx, v.z_bf16, b.w1cat_bf16, nullptr, v.act_bf16, nr, 2 * m->d, ldz, 2 * m->d, EPI_SILU, 1.0f, lda)))
                return rc;
            if ((rc = launch_gemm_bf16_residual(ctx, v.act_bf16, b.w2cat_bf16, feat_out, v.z_bf16,
                                                res_in, rscale, nr, m->d, lda, ldz)))
                return rc;
        }
        if (obs_now && (rc = launch_observe_rows(ctx, ws.last_rows, n_obs, v.weights, (int)m->cap, m->obs.q_pnc, k, v.m_val,
                                                 exact ? v.z : nullptr, feat_out, res_in, rscale, d,
                                                 m->obs.buf + l * m->obs.lanes * obs_rec)))
            return rc;
        return PSSA_B200_OK;
    };
    auto other = [&](float* f) { return f == ws.feat_a ? ws.feat_b : ws.feat_a; };
    // every stage is enqueued group by group, so the chains advance together on the host side too
    auto each_group = [&](auto&& fn) -> int32_t {
        int32_t r = PSSA_B200_OK;
        for (size_t g = 0; g < n_groups && r == PSSA_B200_OK; ++g) {
            if (groups[g].nr == 0) continue;  // only empty lanes: nothing to compute, their carries stay as they are
            select(g);
            r = fn();
        }
        ctx->stream = main_stream, ctx->chain = 0;
        return r;
    };
    if ((rc = fork())) return rc;
    if (m->loops == 1) {
        // src/pssa.rs:2327-2337: block 0's output replaces the embedding, every further block adds its scaled output
        for (size_t l = 0; l < m->depth && rc == PSSA_B200_OK; ++l) {
            rc = each_group([&] { return run_pass(l, 0, feat_in, feat_in, l == 0 ? 1.0f : m->residual_scales[l - 1], feat_out, true); });
            feat_in = feat_out;
            feat_out = other(feat_out);
        }
    } else {
        // Ouro passes (src/pssa.rs:2338-2376): features start as the embedding rows; every pass of a block reads the
        // running features and adds its output / loops; a stacked block's passes then fold into the depth residual
        // features = input + scale * features.
        const float loop_scale = 1.0f / (float)m->loops;
        float* feat = ws.feat_a;
        rc = each_group([&] { return launch_gather_rows(ctx, m->embed, v.ids, feat + r0 * (size_t)d, nr, d, m->v); });
        for (size_t l = 0; l < m->depth && rc == PSSA_B200_OK; ++l) {
            if (l > 0)  // keep the block's input
                rc = each_group([&] { return launch_residual(ctx, nullptr, feat + r0 * (size_t)d, ws.feat_c + r0 * (size_t)d, nr * (size_t)d, 1.0f); });
            for (size_t li = 0; li < m->loops && rc == PSSA_B200_OK; ++li) {
                float* next = other(feat);
                rc = each_group([&] { return run_pass(l, li, feat, feat, loop_scale, next, li + 1 == m->loops); });
                feat = next;
            }
            if (l > 0 && rc == PSSA_B200_OK)
                rc = each_group([&] {
                    return launch_residual(ctx, ws.feat_c + r0 * (size_t)d, feat + r0 * (size_t)d, feat + r0 * (size_t)d, nr * (size_t)d,
                                           m->residual_scales[l - 1]);
                });
        }
        feat_in = feat;
    }
    ctx->stream = main_stream, ctx->chain = 0;
    {
        const int32_t jr = join();  // always re-join, even after a failed launch: the side streams must not run past this call
        if (rc == PSSA_B200_OK) rc = jr;
    }
    if (rc) return rc;
    *feats_out = feat_in;
    return PSSA_B200_OK;
}

// head for the last row of every non-empty lane (src/pssa.rs:2379-2385, 2438-2440)
int32_t head_rows(pssa_b200_model* m, const float* feats, size_t n_heads, bool want_greedy) {
    pssa_b200_ctx* ctx = m->ctx;
    Workspace& ws = m->ws;
    int32_t rc;
    const bool exact = m->precision == PSSA_B200_PRECISION_FP32_EXACT;
    // the last rows of the lanes; the tensor-core head takes them as bf16 straight from the gather (in place of the z staging buffer)
    if ((rc = launch_gather_rows(ctx, feats, ws.last_rows, exact ? ws.last_feat : nullptr, n_heads, (int)m->d, 0, exact ? nullptr : ws.z_bf16)))
        return rc;
    const float scale = 1.0f / std::sqrt((float)m->d);
    if (exact) {
        if ((rc = launch_gemm_exact(ctx, ws.last_feat, m->unembed, ws.logits, n_heads, m->v, m->d, m->v, EPI_SCALE, scale))) return rc;
    } else {
        if ((rc = launch_gemm_bf16(ctx, ws.z_bf16, m->unembed_bf16, ws.logits, nullptr, n_heads, m->v, m->d, m->v, EPI_SCALE, scale))) return rc;
    }
    if (want_greedy && (rc = launch_greedy(ctx, ws.logits, ws.greedy, n_heads, (int)m->v))) return rc;
    return PSSA_B200_OK;
}

// Shared driver: lanes described on the host; processes them in passes of at most max_rows rows.
// per-stream sampler state (history window and generator), allocated on first use; generators start from seed 1337 like
// the reference engine's (src/inference.rs:70-73)
int32_t ensure_sampler(pssa_b200_model* m, size_t lanes) {
    pssa_b200_ctx* ctx = m->ctx;
    auto& sm = m->sampler;
    if (!sm.recent) {
        PSSA_CUDA(ctx, cudaMalloc((void**)&sm.recent, (size_t)m->max_streams * 64 * 4));
        PSSA_CUDA(ctx, cudaMalloc((void**)&sm.count, (size_t)m->max_streams * 4));
        PSSA_CUDA(ctx, cudaMalloc((void**)&sm.rng, (size_t)m->max_streams * 8));
        PSSA_CUDA(ctx, cudaMemsetAsync(sm.count, 0, (size_t)m->max_streams * 4, ctx->stream));
        std::vector<unsigned long long> seeds(m->max_streams, 1337ull);
        PSSA_CUDA(ctx, cudaMemcpyAsync(sm.rng, seeds.data(), seeds.size() * 8, cudaMemcpyHostToDevice, ctx->stream));
        PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
    if (lanes > sm.lanes) {
        PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        cudaFree(sm.ids), cudaFree(sm.status), cudaFree(sm.head_slot), cudaFree(sm.probs), cudaFree(sm.conf);
        sm.ids = sm.status = sm.head_slot = nullptr, sm.probs = sm.conf = nullptr, sm.lanes = 0;
        PSSA_CUDA(ctx, cudaMalloc((void**)&sm.ids, lanes * 4));
        PSSA_CUDA(ctx, cudaMalloc((void**)&sm.status, lanes * 4));
        PSSA_CUDA(ctx, cudaMalloc((void**)&sm.head_slot, lanes * 4));
        PSSA_CUDA(ctx, cudaMalloc((void**)&sm.probs, lanes * m->v * sizeof(float)));
        PSSA_CUDA(ctx, cudaMalloc((void**)&sm.conf, lanes * sizeof(float)));
        sm.lanes = lanes;
    }
    return PSSA_B200_OK;
}

int32_t run_lanes(pssa_b200_model* m, const uint64_t* ids, const uint32_t* offsets, const uint32_t* lengths, const uint32_t* streams,
                  size_t n_lanes, float* logits, uint64_t* greedy, int32_t (*cancelled)(void*), void* cancel_arg, size_t* processed,
                  const pssa_b200_sampling* sampling = nullptr, uint32_t sample_flags = 0, float* confidence = nullptr) {
    pssa_b200_ctx* ctx = m->ctx;
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    uint32_t max_len = 0;
    size_t total = 0;
    for (size_t l = 0; l < n_lanes; ++l) {
        max_len = std::max(max_len, lengths[l]);
        total += lengths[l];
    }
    if (processed) *processed = 0;
    if (total == 0) return PSSA_B200_OK;
    // window of tokens per lane per pass
    size_t window = std::max<size_t>(1, m->max_rows / n_lanes);
    if (window > max_len) window = max_len;
    std::vector<uint32_t> h_ids, h_off(n_lanes), h_len(n_lanes), h_slot(n_lanes), h_last;
    int32_t rc;
    for (size_t t0 = 0; t0 < max_len; t0 += window) {
        if (cancelled && cancelled(cancel_arg)) return fail(ctx, PSSA_B200_ERR_CANCELLED, "prefill cancelled after %zu tokens", t0);
        h_ids.clear();
        size_t rows = 0;
        for (size_t l = 0; l < n_lanes; ++l) {
            uint32_t len = lengths[l] > t0 ? (uint32_t)std::min<size_t>(window, lengths[l] - t0) : 0;
            h_off[l] = (uint32_t)rows, h_len[l] = len, h_slot[l] = streams ? streams[l] : (uint32_t)l;
            for (uint32_t t = 0; t < len; ++t) h_ids.push_back((uint32_t)ids[offsets[l] + t0 + t]);
            rows += len;
        }
        const bool final_pass = t0 + window >= max_len;
        // heads: a lane's last token is in this pass iff its length ends inside the window
        h_last.clear();
        std::vector<size_t> head_lane;
        if (logits || greedy || sampling || m->obs.enabled)
            for (size_t l = 0; l < n_lanes; ++l)
                if (lengths[l] > t0 && lengths[l] <= t0 + window) {
                    h_last.push_back(h_off[l] + h_len[l] - 1);
                    head_lane.push_back(l);
                }
        if ((rc = ensure_workspace(m, rows, n_lanes))) return rc;
        Workspace& ws = m->ws;
        cudaStream_t st = ctx->stream;
        m->dev_layout.ws_base = nullptr;  // the cached layout of the device-resident entry no longer holds
        PSSA_CUDA(ctx, cudaMemcpyAsync(ws.ids, h_ids.data(), rows * 4, cudaMemcpyHostToDevice, st));
        PSSA_CUDA(ctx, cudaMemcpyAsync(ws.lane_off, h_off.data(), n_lanes * 4, cudaMemcpyHostToDevice, st));
        PSSA_CUDA(ctx, cudaMemcpyAsync(ws.lane_len, h_len.data(), n_lanes * 4, cudaMemcpyHostToDevice, st));
        PSSA_CUDA(ctx, cudaMemcpyAsync(ws.lane_slot, h_slot.data(), n_lanes * 4, cudaMemcpyHostToDevice, st));
        if (!h_last.empty()) PSSA_CUDA(ctx, cudaMemcpyAsync(ws.last_rows, h_last.data(), h_last.size() * 4, cudaMemcpyHostToDevice, st));
        float* feats = nullptr;
        if ((rc = forward_rows(m, rows, n_lanes, h_off.data(), h_len.data(), &feats, h_last.size()))) return rc;
        if (!h_last.empty() && (logits || greedy || sampling)) {
            if ((rc = head_rows(m, feats, h_last.size(), greedy != nullptr && !sampling))) return rc;
            std::vector<uint32_t> g(h_last.size()), g_status(h_last.size(), 0);
            std::vector<float> g_conf;
            if (sampling) {
                // sample on the device from the logits the head just wrote; only ids come back
                if ((rc = ensure_sampler(m, n_lanes))) return rc;
                std::vector<uint32_t> head_slot(h_last.size());
                for (size_t i = 0; i < head_lane.size(); ++i) head_slot[i] = h_slot[head_lane[i]];
                PSSA_CUDA(ctx, cudaMemcpyAsync(m->sampler.head_slot, head_slot.data(), head_slot.size() * 4, cudaMemcpyHostToDevice, st));
                PSSA_CUDA(ctx, cudaStreamSynchronize(st));  // head_slot is a local vector
                SampleParams sp{};
                sp.logits = ws.logits, sp.probs = m->sampler.probs, sp.rows = h_last.size(), sp.vocab = (int)m->v;
                sp.top_k = (int)std::min<size_t>(sampling->top_k, m->v);
                sp.temperature = sampling->temperature, sp.top_p = sampling->top_p, sp.repetition_penalty = sampling->repetition_penalty;
                sp.recent_ids = m->sampler.recent, sp.recent_count = m->sampler.count, sp.rng_state = m->sampler.rng;
                sp.ids_out = m->sampler.ids, sp.status_out = m->sampler.status, sp.exact = (sample_flags & PSSA_B200_SAMPLE_EXACT) != 0;
                sp.slots = m->sampler.head_slot, sp.confidence_out = confidence ? m->sampler.conf : nullptr;
                if ((rc = launch_sample(ctx, sp))) return rc;
                if ((rc = launch_push_recent(ctx, m->sampler.ids, m->sampler.head_slot, m->sampler.recent, m->sampler.count, h_last.size())))
                    return rc;
                PSSA_CUDA(ctx, cudaMemcpyAsync(g.data(), m->sampler.ids, g.size() * 4, cudaMemcpyDeviceToHost, st));
                PSSA_CUDA(ctx, cudaMemcpyAsync(g_status.data(), m->sampler.status, g.size() * 4, cudaMemcpyDeviceToHost, st));
                if (confidence) {
                    g_conf.resize(g.size());
                    PSSA_CUDA(ctx, cudaMemcpyAsync(g_conf.data(), m->sampler.conf, g.size() * 4, cudaMemcpyDeviceToHost, st));
                }
            } else if (greedy) {
                PSSA_CUDA(ctx, cudaMemcpyAsync(g.data(), ws.greedy, g.size() * 4, cudaMemcpyDeviceToHost, st));
            }
            if (logits) {
                // contiguous runs of lanes are copied in one transfer
                size_t i = 0;
                while (i < head_lane.size()) {
                    size_t j = i;
                    while (j + 1 < head_lane.size() && head_lane[j + 1] == head_lane[j] + 1) ++j;
                    PSSA_CUDA(ctx, cudaMemcpyAsync(logits + head_lane[i] * m->v, ws.logits + i * m->v, (j - i + 1) * m->v * 4,
                                                   cudaMemcpyDeviceToHost, st));
                    i = j + 1;
                }
            }
            PSSA_CUDA(ctx, cudaStreamSynchronize(st));
            if (greedy)
                for (size_t i = 0; i < head_lane.size(); ++i) {
                    if (g[i] == 0xffffffffu) {  // src/inference.rs:111-113, 146-147, 153-154
                        const char* why = g_status[i] == 2 ? "invalid sampling probability mass"
                                          : g_status[i] == 3 ? "no valid generation candidates" : "model emitted non-finite logits";
                        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "%s", why);
                    }
                    greedy[head_lane[i]] = g[i];
                    if (confidence && !g_conf.empty()) confidence[head_lane[i]] = g_conf[i];
                }
        } else if (final_pass || cancelled) {
            PSSA_CUDA(ctx, cudaStreamSynchronize(st));
        }
        if (processed) *processed = std::min<size_t>(max_len, t0 + window);
    }
    PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return PSSA_B200_OK;
}

}  // namespace

extern "C" {

int32_t pssa_b200_model_prefill_batch(pssa_b200_model* m, const uint64_t* ids, const uint32_t* offsets, const uint32_t* lengths,
                                      const uint32_t* streams, size_t n_lanes, float* logits, uint64_t* greedy) {
    if (!m || !ids || !offsets || !lengths) return fail(m ? m->ctx : nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "prefill_batch: null argument");
    pssa_b200_ctx* ctx = m->ctx;
    if (n_lanes == 0 || n_lanes > 0x7fffffff) return fail(ctx, PSSA_B200_ERR_SHAPE, "prefill_batch: lane count must be in 1..2^31-1");
    // validate every lane before any work (src/sequence_batch.rs:250-273)
    std::vector<bool> seen(m->max_streams, false);
    for (size_t l = 0; l < n_lanes; ++l) {
        uint32_t slot = streams ? streams[l] : (uint32_t)l;
        if (slot >= m->max_streams) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "lane %zu uses stream %u outside %u streams", l, slot, m->max_streams);
        if (seen[slot]) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "stream %u appears in more than one lane", slot);
        seen[slot] = true;
        for (uint32_t t = 0; t < lengths[l]; ++t) {
            uint64_t id = ids[(size_t)offsets[l] + t];
            if (id >= m->v) return fail(ctx, PSSA_B200_ERR_TOKEN, "prompt ID %llu outside model vocabulary", (unsigned long long)id);
        }
    }
    return run_lanes(m, ids, offsets, lengths, streams, n_lanes, logits, greedy, nullptr, nullptr, nullptr);
}

int32_t pssa_b200_model_prefill_batch_dev(pssa_b200_model* m, const uint32_t* ids_dev, const uint32_t* offsets, const uint32_t* lengths,
                                          const uint32_t* streams, size_t n_lanes, float* logits_dev, uint32_t* greedy_dev) {
    if (!m || !ids_dev || !offsets || !lengths) return fail(m ? m->ctx : nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "prefill_batch_dev: null argument");
    pssa_b200_ctx* ctx = m->ctx;
    if (n_lanes == 0 || n_lanes > 0x7fffffff) return fail(ctx, PSSA_B200_ERR_SHAPE, "prefill_batch: lane count must be in 1..2^31-1");
    std::vector<bool> seen(m->max_streams, false);
    std::vector<uint32_t> h_off(n_lanes), h_len(n_lanes), h_slot(n_lanes), h_last;
    std::vector<size_t> head_lane;
    size_t rows = 0, span = 0;
    for (size_t l = 0; l < n_lanes; ++l) {
        uint32_t slot = streams ? streams[l] : (uint32_t)l;
        if (slot >= m->max_streams) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "lane %zu uses stream %u outside %u streams", l, slot, m->max_streams);
        if (seen[slot]) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "stream %u appears in more than one lane", slot);
        seen[slot] = true;
        h_off[l] = offsets[l], h_len[l] = lengths[l], h_slot[l] = slot;
        rows += lengths[l];
        span = std::max(span, (size_t)offsets[l] + lengths[l]);
        if (lengths[l] > 0) {
            h_last.push_back(offsets[l] + lengths[l] - 1);
            head_lane.push_back(l);
        }
    }
    // A rank with no token at all cannot take part in the per-block exchange. This check is local: the CALLER must make
    // the same decision on every rank before calling (every rank knows all sequence lengths), or the other ranks would
    // enqueue an all-gather this rank never joins.
    if (rows == 0 && m->sp.world > 1)
        return fail(ctx, PSSA_B200_ERR_SHAPE, "sequence-parallel prefill: rank %u holds no token of any lane", m->sp.rank);
    if (rows == 0) return PSSA_B200_OK;
    if (span > m->max_rows)
        return fail(ctx, PSSA_B200_ERR_SHAPE, "prefill_batch_dev: %zu token rows exceed one pass of %zu rows (set_max_rows)", span, m->max_rows);
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    int32_t rc;
    if ((rc = ensure_workspace(m, span, n_lanes))) return rc;
    Workspace& ws = m->ws;
    cudaStream_t st = ctx->stream;
    PSSA_CUDA(ctx, cudaMemcpyAsync(ws.ids, ids_dev, span * 4, cudaMemcpyDeviceToDevice, st));
    // The lane description is uploaded only when it differs from what the workspace already holds. A repeated call with
    // the same layout (a decode loop) then consists of kernel launches and device-to-device copies only, so the caller can
    // capture it in a CUDA graph on the context's stream.
    auto& lay = m->dev_layout;
    if (lay.ws_base != ws.base || lay.off != h_off || lay.len != h_len || lay.slot != h_slot) {
        PSSA_CUDA(ctx, cudaMemcpyAsync(ws.lane_off, h_off.data(), n_lanes * 4, cudaMemcpyHostToDevice, st));
        PSSA_CUDA(ctx, cudaMemcpyAsync(ws.lane_len, h_len.data(), n_lanes * 4, cudaMemcpyHostToDevice, st));
        PSSA_CUDA(ctx, cudaMemcpyAsync(ws.lane_slot, h_slot.data(), n_lanes * 4, cudaMemcpyHostToDevice, st));
        PSSA_CUDA(ctx, cudaMemcpyAsync(ws.last_rows, h_last.data(), h_last.size() * 4, cudaMemcpyHostToDevice, st));
        lay.ws_base = ws.base, lay.off = h_off, lay.len = h_len, lay.slot = h_slot;
    }
    float* feats = nullptr;
    m->sp.active = m->sp.world > 1;
    rc = forward_rows(m, span, n_lanes, h_off.data(), h_len.data(), &feats, h_last.size());
    m->sp.active = false;
    if (rc) return rc;
    if (logits_dev || greedy_dev) {
        if ((rc = head_rows(m, feats, h_last.size(), greedy_dev != nullptr))) return rc;
        size_t i = 0;
        while (i < head_lane.size()) {  // contiguous runs of non-empty lanes go out in one copy
            size_t j = i;
            while (j + 1 < head_lane.size() && head_lane[j + 1] == head_lane[j] + 1) ++j;
            if (logits_dev)
                PSSA_CUDA(ctx, cudaMemcpyAsync(logits_dev + head_lane[i] * m->v, ws.logits + i * m->v, (j - i + 1) * m->v * 4,
                                               cudaMemcpyDeviceToDevice, st));
            if (greedy_dev)
                PSSA_CUDA(ctx, cudaMemcpyAsync(greedy_dev + head_lane[i], ws.greedy + i, (j - i + 1) * 4, cudaMemcpyDeviceToDevice, st));
            i = j + 1;
        }
    }
    return PSSA_B200_OK;
}

int32_t pssa_b200_model_score(pssa_b200_model* m, uint32_t stream, const uint64_t* ids, const uint64_t* targets, size_t n, float* mean_loss,
                              float* token_loss, float* logits_out) {
    if (!m || !ids || !targets || !mean_loss) return fail(m ? m->ctx : nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "score: null argument");
    pssa_b200_ctx* ctx = m->ctx;
    if (n == 0) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "score requires at least one token");
    if (stream >= m->max_streams) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "stream %u outside %u streams", stream, m->max_streams);
    for (size_t t = 0; t < n; ++t) {
        if (ids[t] >= m->v) return fail(ctx, PSSA_B200_ERR_TOKEN, "token ID %llu outside model vocabulary", (unsigned long long)ids[t]);
        if (targets[t] >= m->v) return fail(ctx, PSSA_B200_ERR_TOKEN, "target ID %llu outside model vocabulary", (unsigned long long)targets[t]);
    }
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t window = std::min(n, m->max_rows);
    // tile of full-vocabulary logits: at most 128 MiB
    const size_t tile = std::max<size_t>(1, std::min(window, ((size_t)128 << 20) / (m->v * sizeof(float))));
    auto& sc = m->score;
    if (tile > sc.tile || window > sc.rows) {
        PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        cudaFree(sc.logits), cudaFree(sc.targets), cudaFree(sc.loss);
        sc = pssa_b200_model::Score{};
        PSSA_CUDA(ctx, cudaMalloc((void**)&sc.logits, tile * m->v * sizeof(float)));
        PSSA_CUDA(ctx, cudaMalloc((void**)&sc.targets, window * 4));
        PSSA_CUDA(ctx, cudaMalloc((void**)&sc.loss, window * 4));
        sc.tile = tile, sc.rows = window;
    }
    const bool exact = m->precision == PSSA_B200_PRECISION_FP32_EXACT;
    const float scale = 1.0f / std::sqrt((float)m->d);
    std::vector<uint32_t> h_ids(window), h_tgt(window);
    std::vector<float> h_loss(window);
    double total = 0.0;
    int32_t rc;
    cudaStream_t st = ctx->stream;
    for (size_t t0 = 0; t0 < n; t0 += window) {
        const size_t rows = std::min(window, n - t0);
        for (size_t t = 0; t < rows; ++t) h_ids[t] = (uint32_t)ids[t0 + t], h_tgt[t] = (uint32_t)targets[t0 + t];
        if ((rc = ensure_workspace(m, rows, 1))) return rc;
        Workspace& ws = m->ws;
        const uint32_t off = 0, len = (uint32_t)rows, slot = stream;
        m->dev_layout.ws_base = nullptr;
        PSSA_CUDA(ctx, cudaMemcpyAsync(ws.ids, h_ids.data(), rows * 4, cudaMemcpyHostToDevice, st));
        PSSA_CUDA(ctx, cudaMemcpyAsync(sc.targets, h_tgt.data(), rows * 4, cudaMemcpyHostToDevice, st));
        PSSA_CUDA(ctx, cudaMemcpyAsync(ws.lane_off, &off, 4, cudaMemcpyHostToDevice, st));
        PSSA_CUDA(ctx, cudaMemcpyAsync(ws.lane_len, &len, 4, cudaMemcpyHostToDevice, st));
        PSSA_CUDA(ctx, cudaMemcpyAsync(ws.lane_slot, &slot, 4, cudaMemcpyHostToDevice, st));
        PSSA_CUDA(ctx, cudaStreamSynchronize(st));  // the three scalars above live on this stack frame
        float* feats = nullptr;
        if ((rc = forward_rows(m, rows, 1, &off, &len, &feats))) return rc;
        for (size_t r0 = 0; r0 < rows; r0 += tile) {
            const size_t nr = std::min(tile, rows - r0);
            if (exact) {
                if ((rc = launch_gemm_exact(ctx, feats + r0 * m->d, m->unembed, sc.logits, nr, m->v, m->d, m->v, EPI_SCALE, scale))) return rc;
            } else {
                if ((rc = launch_to_bf16(ctx, feats + r0 * m->d, ws.z_bf16, nr * m->d))) return rc;
                if ((rc = launch_gemm_bf16(ctx, ws.z_bf16, m->unembed_bf16, sc.logits, nullptr, nr, m->v, m->d, m->v, EPI_SCALE, scale))) return rc;
            }
            if ((rc = launch_cross_entropy(ctx, sc.logits, sc.targets + r0, sc.loss + r0, nr, (int)m->v))) return rc;
            if (logits_out)
                PSSA_CUDA(ctx, cudaMemcpyAsync(logits_out + (t0 + r0) * m->v, sc.logits, nr * m->v * sizeof(float), cudaMemcpyDeviceToHost, st));
        }
        PSSA_CUDA(ctx, cudaMemcpyAsync(h_loss.data(), sc.loss, rows * 4, cudaMemcpyDeviceToHost, st));
        PSSA_CUDA(ctx, cudaStreamSynchronize(st));
        for (size_t t = 0; t < rows; ++t) {
            if (!std::isfinite(h_loss[t])) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "model emitted non-finite logits at token %zu", t0 + t);
            total += (double)h_loss[t];
            if (token_loss) token_loss[t0 + t] = h_loss[t];
        }
    }
    *mean_loss = (float)(total / (double)n);
    return PSSA_B200_OK;
}

int32_t pssa_b200_model_set_observer(pssa_b200_model* m, int32_t enabled) {
    if (!m) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null model");
    m->obs.enabled = enabled != 0;
    if (!m->obs.enabled) m->obs.valid_lanes = 0;
    return PSSA_B200_OK;
}

int32_t pssa_b200_model_get_observation(pssa_b200_model* m, uint32_t layer, uint32_t index, float* mem_weights, float* q_pnc, float* m_val,
                                        float* z_final) {
    if (!m) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null model");
    pssa_b200_ctx* ctx = m->ctx;
    if (!m->obs.enabled || m->obs.valid_lanes == 0)
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "observer scratch is empty: enable the observer and run a forward call first");
    if (layer >= m->depth || index >= m->obs.valid_lanes)
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "observation (block %u, lane %u) outside %zu blocks x %zu lanes", layer, index, m->depth,
                    m->obs.valid_lanes);
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t rec = m->cap + m->k + 2 * m->d;
    const float* src = m->obs.buf + ((size_t)layer * m->obs.lanes + index) * rec;
    cudaStream_t st = ctx->stream;
    if (mem_weights) PSSA_CUDA(ctx, cudaMemcpyAsync(mem_weights, src, m->cap * 4, cudaMemcpyDeviceToHost, st));
    if (q_pnc) PSSA_CUDA(ctx, cudaMemcpyAsync(q_pnc, src + m->cap, m->k * 4, cudaMemcpyDeviceToHost, st));
    if (m_val) PSSA_CUDA(ctx, cudaMemcpyAsync(m_val, src + m->cap + m->k, m->d * 4, cudaMemcpyDeviceToHost, st));
    if (z_final) PSSA_CUDA(ctx, cudaMemcpyAsync(z_final, src + m->cap + m->k + m->d, m->d * 4, cudaMemcpyDeviceToHost, st));
    PSSA_CUDA(ctx, cudaStreamSynchronize(st));
    return PSSA_B200_OK;
}

int32_t pssa_b200_model_insert_memory(pssa_b200_model* m, uint32_t index, float loss, uint64_t step, int64_t* slots_out) {
    if (!m) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null model");
    pssa_b200_ctx* ctx = m->ctx;
    if (slots_out)
        for (size_t l = 0; l < m->depth; ++l) slots_out[l] = -3;  // nothing attempted
    if (!(loss > 3.5f)) return PSSA_B200_OK;  // src/pssa.rs:3706-3708 (also false for NaN)
    if (!m->obs.enabled || m->obs.valid_lanes == 0)
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "insert_memory: enable the observer and run a forward call first (the write takes its key and value from the observer scratch)");
    if (index >= m->obs.valid_lanes)
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "insert_memory: lane %u outside the %zu observed lanes", index, m->obs.valid_lanes);
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t cap = m->cap, rec = m->cap + m->k + 2 * m->d;
    cudaStream_t st = ctx->stream;
    for (size_t l = 0; l < m->depth; ++l) {
        DeviceBlock& b = m->blocks[l];
        if (b.confidence.size() != cap) b.confidence.assign(cap, 0.0f);  // a bank uploaded without metadata: src/memory.rs:44-45
        if (b.last_seen.size() != cap) b.last_seen.assign(cap, 0);
        // the gate's history-dependent words travel to the device for the one write and come back
        arena_reset(ctx);
        int32_t rc_a = arena_reserve(ctx, arena_round(cap * 4) + arena_round(cap * 8) + 4 * 256);
        if (rc_a) return rc_a;
        float* conf = (float*)arena_take(ctx, cap * 4);
        unsigned long long* seen = (unsigned long long*)arena_take(ctx, cap * 8);
        unsigned long long* meta = (unsigned long long*)arena_take(ctx, 16);
        unsigned long long* step_dev = (unsigned long long*)arena_take(ctx, 8);
        float* surprise = (float*)arena_take(ctx, 4);
        long long* slot_dev = (long long*)arena_take(ctx, 8);
        if (!conf || !seen || !meta || !step_dev || !surprise || !slot_dev) return fail(ctx, PSSA_B200_ERR_CUDA, "insert_memory: scratch allocation failed");
        const unsigned long long meta_h[2] = {b.count, b.write_head}, step_h = step;
        PSSA_CUDA(ctx, cudaMemcpyAsync(conf, b.confidence.data(), cap * 4, cudaMemcpyHostToDevice, st));
        PSSA_CUDA(ctx, cudaMemcpyAsync(seen, b.last_seen.data(), cap * 8, cudaMemcpyHostToDevice, st));
        PSSA_CUDA(ctx, cudaMemcpyAsync(meta, meta_h, 16, cudaMemcpyHostToDevice, st));
        PSSA_CUDA(ctx, cudaMemcpyAsync(step_dev, &step_h, 8, cudaMemcpyHostToDevice, st));
        PSSA_CUDA(ctx, cudaMemcpyAsync(surprise, &loss, 4, cudaMemcpyHostToDevice, st));
        const float* obs = m->obs.buf + (l * m->obs.lanes + index) * rec;
        BankWriteParams p{};
        p.keys = b.w[T_BANK_KEYS], p.norm_sq = b.w[T_BANK_NORM_SQ], p.values = b.w[T_BANK_VALUES], p.confidence = conf, p.last_seen = seen, p.meta = meta;
        p.cap = (int)cap, p.dk = (int)m->k, p.dv = (int)m->d;
        p.key_pnc = obs + cap;                    // q_poincare of the lane's last token (src/pssa.rs:3717)
        p.val = obs + cap + m->k + m->d;          // z_final of the same token (src/pssa.rs:3718)
        p.surprise = surprise, p.step = step_dev, p.n = 1, p.slots_out = slot_dev, p.winning_slots = nullptr, p.eta = 0.0f;
        int32_t rc = launch_bank_insert_protected(ctx, p);
        if (rc) return rc;
        unsigned long long meta_back[2];
        long long slot = -1;
        PSSA_CUDA(ctx, cudaMemcpyAsync(b.confidence.data(), conf, cap * 4, cudaMemcpyDeviceToHost, st));
        PSSA_CUDA(ctx, cudaMemcpyAsync(b.last_seen.data(), seen, cap * 8, cudaMemcpyDeviceToHost, st));
        PSSA_CUDA(ctx, cudaMemcpyAsync(meta_back, meta, 16, cudaMemcpyDeviceToHost, st));
        PSSA_CUDA(ctx, cudaMemcpyAsync(&slot, slot_dev, 8, cudaMemcpyDeviceToHost, st));
        PSSA_CUDA(ctx, cudaStreamSynchronize(st));
        b.count = meta_back[0], b.write_head = meta_back[1];
        if (slot >= 0) b.ksplit_dirty = b.vsplit_dirty = b.vp_dirty = true;  // the derived copies of keys and values are stale
        if (slots_out) slots_out[l] = slot;
    }
    return PSSA_B200_OK;
}

int32_t pssa_b200_model_sampler_seed(pssa_b200_model* m, uint32_t stream, uint64_t seed) {
    if (!m) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null model");
    pssa_b200_ctx* ctx = m->ctx;
    if (stream >= m->max_streams) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "stream %u outside %u streams", stream, m->max_streams);
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    int32_t rc = ensure_sampler(m, 1);
    if (rc) return rc;
    const unsigned long long state = seed == 0 ? 0x853c49e6748fea9bull : seed;  // src/linalg.rs:7-11
    const unsigned zero = 0;
    PSSA_CUDA(ctx, cudaMemcpyAsync(m->sampler.rng + stream, &state, 8, cudaMemcpyHostToDevice, ctx->stream));
    PSSA_CUDA(ctx, cudaMemcpyAsync(m->sampler.count + stream, &zero, 4, cudaMemcpyHostToDevice, ctx->stream));
    PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return PSSA_B200_OK;
}

int32_t pssa_b200_model_sampler_push(pssa_b200_model* m, uint32_t stream, const uint64_t* ids, size_t n) {
    if (!m || (!ids && n)) return fail(m ? m->ctx : nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "sampler_push: null argument");
    pssa_b200_ctx* ctx = m->ctx;
    if (stream >= m->max_streams) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "stream %u outside %u streams", stream, m->max_streams);
    for (size_t i = 0; i < n; ++i)
        if (ids[i] >= m->v) return fail(ctx, PSSA_B200_ERR_TOKEN, "prompt ID %llu outside model vocabulary", (unsigned long long)ids[i]);
    if (n == 0) return PSSA_B200_OK;
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    int32_t rc = ensure_sampler(m, 1);
    if (rc) return rc;
    // the window holds the last 64 ids, oldest first (src/inference.rs:114-121 reads `generated_ids[len - 64..]`)
    unsigned count = 0, window[64];
    PSSA_CUDA(ctx, cudaMemcpyAsync(&count, m->sampler.count + stream, 4, cudaMemcpyDeviceToHost, ctx->stream));
    PSSA_CUDA(ctx, cudaMemcpyAsync(window, m->sampler.recent + (size_t)stream * 64, sizeof(window), cudaMemcpyDeviceToHost, ctx->stream));
    PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    std::vector<unsigned> all(window, window + std::min<unsigned>(count, 64u));
    for (size_t i = n > 64 ? n - 64 : 0; i < n; ++i) all.push_back((unsigned)ids[i]);
    const size_t keep = std::min<size_t>(all.size(), 64), from = all.size() - keep;
    for (size_t i = 0; i < keep; ++i) window[i] = all[from + i];
    count = (unsigned)keep;
    PSSA_CUDA(ctx, cudaMemcpyAsync(m->sampler.recent + (size_t)stream * 64, window, keep * 4, cudaMemcpyHostToDevice, ctx->stream));
    PSSA_CUDA(ctx, cudaMemcpyAsync(m->sampler.count + stream, &count, 4, cudaMemcpyHostToDevice, ctx->stream));
    PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return PSSA_B200_OK;
}

int32_t pssa_b200_model_decode_step_sampled(pssa_b200_model* m, const uint32_t* streams, const uint64_t* ids, size_t n,
                                            const pssa_b200_sampling* cfg, uint32_t flags, uint64_t* ids_out, float* confidence_out) {
    if (!m || !ids || !cfg || !ids_out) return fail(m ? m->ctx : nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "decode_step_sampled: null argument");
    pssa_b200_ctx* ctx = m->ctx;
    if (n == 0 || n > 0x7fffffff) return fail(ctx, PSSA_B200_ERR_SHAPE, "decode_step: stream count must be in 1..2^31-1");
    if (flags & ~PSSA_B200_SAMPLE_EXACT) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "sampling: unknown flags");
    // src/inference.rs:87-101
    if (!std::isfinite(cfg->temperature) || cfg->temperature < 0.0f) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "temperature must be finite and >= 0");
    if (!(std::isfinite(cfg->top_p) && cfg->top_p > 0.0f && cfg->top_p <= 1.0f)) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "top-p must be finite in (0, 1]");
    if (cfg->top_k == 0) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "top-k must be positive");
    if (cfg->top_k > 4096 && cfg->top_k < m->v) return fail(ctx, PSSA_B200_ERR_UNSUPPORTED, "sampling: top-k %u outside 1..4096", cfg->top_k);
    if (!(std::isfinite(cfg->repetition_penalty) && cfg->repetition_penalty >= 1.0f))
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "repetition penalty must be finite and >= 1");
    std::vector<bool> seen(m->max_streams, false);
    for (size_t i = 0; i < n; ++i) {
        uint32_t slot = streams ? streams[i] : (uint32_t)i;
        if (slot >= m->max_streams) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "lane %zu uses stream %u outside %u streams", i, slot, m->max_streams);
        if (seen[slot]) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "stream %u appears in more than one lane", slot);
        seen[slot] = true;
        if (ids[i] >= m->v) return fail(ctx, PSSA_B200_ERR_TOKEN, "token ID %llu outside model vocabulary", (unsigned long long)ids[i]);
    }
    std::vector<uint32_t> off(n), len(n, 1);
    for (size_t i = 0; i < n; ++i) off[i] = (uint32_t)i;
    return run_lanes(m, ids, off.data(), len.data(), streams, n, nullptr, ids_out, nullptr, nullptr, nullptr, cfg, flags, confidence_out);
}

int32_t pssa_b200_model_set_seqpar(pssa_b200_model* m, uint32_t rank, uint32_t world, void* send_dev, void* recv_dev, size_t capacity,
                                   pssa_b200_exchange_fn exchange, void* arg) {
    if (!m) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null model");
    pssa_b200_ctx* ctx = m->ctx;
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    PSSA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    m->sp = pssa_b200_model::SeqPar{};
    if (world <= 1 || !exchange) return PSSA_B200_OK;
    if (rank >= world) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "sequence-parallel rank %u outside world of %u", rank, world);
    if (!send_dev || !recv_dev || capacity == 0)
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "sequence-parallel prefill needs exchange buffers and a record capacity");
    if (((uintptr_t)send_dev & 15) || ((uintptr_t)recv_dev & 15))
        return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "sequence-parallel exchange buffers must be 16-byte aligned");
    m->sp.rank = rank, m->sp.world = world, m->sp.send = (float*)send_dev, m->sp.recv = (float*)recv_dev;
    m->sp.capacity = capacity, m->sp.fn = exchange, m->sp.arg = arg;
    return PSSA_B200_OK;
}

int32_t pssa_b200_model_prefill(pssa_b200_model* m, uint32_t stream, const uint64_t* ids, size_t n, float* logits, size_t* processed,
                                int32_t (*cancelled)(void*), void* cancel_arg) {
    if (!m) return fail(nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "null model");
    pssa_b200_ctx* ctx = m->ctx;
    if (processed) *processed = 0;
    if (n == 0 || !ids) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "prefill requires at least one token");  // src/pssa.rs:2405-2407
    if (stream >= m->max_streams) return fail(ctx, PSSA_B200_ERR_INVALID_ARGUMENT, "stream %u outside %u streams", stream, m->max_streams);
    if (n > 0xffffffffull) return fail(ctx, PSSA_B200_ERR_SHAPE, "prefill: %zu tokens exceed the u32 row index", n);
    size_t valid = 0;
    while (valid < n && ids[valid] < m->v) ++valid;
    uint32_t off = 0, len = (uint32_t)valid;
    int32_t rc = PSSA_B200_OK;
    size_t done = 0;
    if (valid > 0) rc = run_lanes(m, ids, &off, &len, &stream, 1, valid == n ? logits : nullptr, nullptr, cancelled, cancel_arg, &done);
    if (processed) *processed = done;
    if (rc != PSSA_B200_OK) return rc;
    if (valid < n)  // the valid prefix has advanced the carry; logits untouched (src/pssa.rs:2414-2416)
        return fail(ctx, PSSA_B200_ERR_TOKEN, "prompt ID %llu outside model vocabulary", (unsigned long long)ids[valid]);
    return PSSA_B200_OK;
}

int32_t pssa_b200_model_decode_step(pssa_b200_model* m, const uint32_t* streams, const uint64_t* ids, size_t n, float* logits,
                                    uint64_t* greedy) {
    if (!m || !ids) return fail(m ? m->ctx : nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "decode_step: null argument");
    if (n == 0 || n > 0x7fffffff) return fail(m->ctx, PSSA_B200_ERR_SHAPE, "decode_step: stream count must be in 1..2^31-1");
    std::vector<uint32_t> off(n), len(n, 1);
    for (size_t i = 0; i < n; ++i) off[i] = (uint32_t)i;
    return pssa_b200_model_prefill_batch(m, ids, off.data(), len.data(), streams, n, logits, greedy);
}

int32_t pssa_b200_model_reserve(pssa_b200_model* m, size_t rows, size_t lanes) {
    if (!m || rows == 0 || lanes == 0) return fail(m ? m->ctx : nullptr, PSSA_B200_ERR_INVALID_ARGUMENT, "reserve: rows and lanes must be positive");
    pssa_b200_ctx* ctx = m->ctx;
    PSSA_CUDA(ctx, cudaSetDevice(ctx->device));
    int32_t rc;
    if ((rc = ensure_workspace(m, std::min(rows, m->max_rows), lanes))) return rc;
    if ((rc = ensure_chunks(m, lanes * 16))) return rc;  // the most time chunks a lane is ever cut into
    return ensure_sampler(m, lanes);
}

}  // extern "C"
