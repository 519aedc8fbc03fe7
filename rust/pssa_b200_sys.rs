//! Raw FFI declarations of `include/pssa_b200.h` for the reference crate: every symbol the C header declares, in the
//! header's order. This file is what `GpuDispatch::B200` / `Device::B200` (see `backend_b200.rs` beside it) binds; link with
//! `cargo:rustc-link-lib=dylib=pssa_b200` from a build script that points at the directory holding `libpssa_b200.so`.
//!
//! Conventions (see the header): every call returns a status (`PSSA_B200_OK` = 0); on failure the text is available from
//! `pssa_b200_last_error`; `*_dev` functions take DEVICE pointers and only enqueue work on the context's stream, the others
//! take host slices and return when the result is back on the host, like the reference's own `GpuDispatch` methods
//! (src/cuda.rs:517-585). There is no CPU fallback behind any of them.
#![allow(non_camel_case_types, clippy::too_many_arguments)]

use std::os::raw::{c_char, c_void};

pub const PSSA_B200_OK: i32 = 0;
pub const PSSA_B200_ERR_INVALID_ARGUMENT: i32 = 1;
pub const PSSA_B200_ERR_SHAPE: i32 = 2;
pub const PSSA_B200_ERR_CUDA: i32 = 3;
pub const PSSA_B200_ERR_FATAL_CUDA: i32 = 4;
pub const PSSA_B200_ERR_TIMEOUT: i32 = 5;
pub const PSSA_B200_ERR_UNSUPPORTED: i32 = 6;
pub const PSSA_B200_ERR_TOKEN: i32 = 7;
pub const PSSA_B200_ERR_CANCELLED: i32 = 8;
pub const PSSA_B200_ERR_BANK: i32 = 9;

pub const PSSA_B200_SSM_EXACT: u32 = 1;
pub const PSSA_B200_MEM_EXACT: u32 = 1;
pub const PSSA_B200_MEM_F32_DISTANCE: u32 = 2;
pub const PSSA_B200_MEM_TC_DISTANCE: u32 = 4;
pub const PSSA_B200_MEM_NO_FUSED: u32 = 8;
pub const PSSA_B200_MEM_HANDOVER_SELFTEST: u32 = 16;
pub const PSSA_B200_MEM_PHASE_CLOCKS: u32 = 32;
pub const PSSA_B200_SAMPLE_EXACT: u32 = 1;

/// `pssa_b200_epilogue`
pub const PSSA_B200_EPI_NONE: i32 = 0;
pub const PSSA_B200_EPI_SOFTPLUS: i32 = 1;
pub const PSSA_B200_EPI_SIGMOID: i32 = 2;
pub const PSSA_B200_EPI_SILU: i32 = 3;
pub const PSSA_B200_EPI_SCALE: i32 = 4;
pub const PSSA_B200_EPI_ADD_OUT: i32 = 5;

/// `pssa_b200_precision`
pub const PSSA_B200_PRECISION_BF16: i32 = 0;
pub const PSSA_B200_PRECISION_FP32_EXACT: i32 = 1;

/// `pssa_b200_tensor`: parameter identifiers of `pssa_b200_model_set_tensor` (reference shapes, src/pssa.rs:506-620)
pub const PSSA_B200_T_EMBED: i32 = 0;
pub const PSSA_B200_T_UNEMBED: i32 = 1;
pub const PSSA_B200_T_NORM_GAMMA: i32 = 2;
pub const PSSA_B200_T_NORM_BETA: i32 = 3;
pub const PSSA_B200_T_A_MAT: i32 = 4;
pub const PSSA_B200_T_W_DELTA: i32 = 5;
pub const PSSA_B200_T_W_B: i32 = 6;
pub const PSSA_B200_T_W_C: i32 = 7;
pub const PSSA_B200_T_W_QX: i32 = 8;
pub const PSSA_B200_T_W_QH: i32 = 9;
pub const PSSA_B200_T_W_GATE: i32 = 10;
pub const PSSA_B200_T_W_PROJ: i32 = 11;
pub const PSSA_B200_T_MLP_W1: i32 = 12;
pub const PSSA_B200_T_MLP_W2: i32 = 13;
pub const PSSA_B200_T_AD_DOWN: i32 = 14;
pub const PSSA_B200_T_AD_UP: i32 = 15;
pub const PSSA_B200_T_AD_CONS: i32 = 16;
pub const PSSA_B200_T_RESIDUAL_SCALES: i32 = 22;

/// Opaque: one device, one stream, one scratch arena.
#[repr(C)]
pub struct pssa_b200_ctx {
    _private: [u8; 0],
}
/// Opaque: device-resident weights, banks and recurrent carries.
#[repr(C)]
pub struct pssa_b200_model {
    _private: [u8; 0],
}

/// `PSSAConfigV2` (src/pssa.rs:253-331) reduced to what the forward path reads.
#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct pssa_b200_config {
    pub depth: u64,
    pub d_vocab: u64,
    pub d_latent: u64,
    pub d_state: u64,
    pub d_mem_key: u64,
    pub mem_capacity: u64,
    pub tau_mem: f32,
    pub reserved: u32,
}

/// Sampling parameters of `PSSAInferenceEngine::sample` (src/inference.rs:87-181).
#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct pssa_b200_sampling {
    pub temperature: f32,
    pub top_p: f32,
    pub top_k: u32,
    pub repetition_penalty: f32,
}

/// All-gather supplied by the caller for sequence-parallel prefill: place rank k's `bytes` at `recv + k * bytes` on every
/// rank, in stream order on the context's stream; return 0.
pub type pssa_b200_exchange_fn =
    Option<unsafe extern "C" fn(arg: *mut c_void, send_dev: *const c_void, recv_dev: *mut c_void, bytes: usize) -> i32>;

#[link(name = "pssa_b200")]
extern "C" {
    pub fn pssa_b200_ctx_create(device: i32, out: *mut *mut pssa_b200_ctx) -> i32;
    pub fn pssa_b200_ctx_destroy(ctx: *mut pssa_b200_ctx);
    pub fn pssa_b200_last_error(ctx: *const pssa_b200_ctx) -> *const c_char;
    pub fn pssa_b200_ctx_set_stream(ctx: *mut pssa_b200_ctx, cuda_stream: *mut c_void) -> i32;
    pub fn pssa_b200_ctx_use_own_stream(ctx: *mut pssa_b200_ctx) -> i32;
    pub fn pssa_b200_ctx_synchronize(ctx: *mut pssa_b200_ctx) -> i32;
    pub fn pssa_b200_backend_label(ctx: *const pssa_b200_ctx) -> *const c_char;
    pub fn pssa_b200_launch_count(ctx: *const pssa_b200_ctx) -> u64;
    pub fn pssa_b200_ctx_reserve(ctx: *mut pssa_b200_ctx, bytes: usize) -> i32;
    pub fn pssa_b200_ctx_poll_status(ctx: *mut pssa_b200_ctx) -> i32;
    pub fn pssa_b200_ctx_selftest_wait_expiry(ctx: *mut pssa_b200_ctx, polls: u32) -> i32;
    pub fn pssa_b200_ctx_profile_begin(ctx: *mut pssa_b200_ctx) -> i32;
    pub fn pssa_b200_ctx_profile_end(ctx: *mut pssa_b200_ctx, n_rows: *mut u32) -> i32;
    pub fn pssa_b200_ctx_profile_row(
        ctx: *mut pssa_b200_ctx,
        index: u32,
        name: *const *const c_char,
        launches: *mut u64,
        ms: *mut f64,
    ) -> i32;
    pub fn pssa_b200_ctx_set_scan_chunks(ctx: *mut pssa_b200_ctx, chunks: u32) -> i32;
    pub fn pssa_b200_affine_scan_dev(
        ctx: *mut pssa_b200_ctx,
        scan_a: *mut f32,
        scan_b: *mut f32,
        lanes: usize,
        len: usize,
        stride: usize,
    ) -> i32;
    pub fn pssa_b200_affine_scan(
        ctx: *mut pssa_b200_ctx,
        scan_a: *mut f32,
        scan_b: *mut f32,
        lanes: usize,
        len: usize,
        stride: usize,
    ) -> i32;
    pub fn pssa_b200_scan_states_dev(
        ctx: *mut pssa_b200_ctx,
        a: *const f32,
        b: *const f32,
        h0: *const f32,
        h: *mut f32,
        h_last: *mut f32,
        lanes: usize,
        len: usize,
        stride: usize,
    ) -> i32;
    pub fn pssa_b200_scan_states(
        ctx: *mut pssa_b200_ctx,
        a: *const f32,
        b: *const f32,
        h0: *const f32,
        h: *mut f32,
        h_last: *mut f32,
        lanes: usize,
        len: usize,
        stride: usize,
    ) -> i32;
    pub fn pssa_b200_scan_states_noalloc_dev(
        ctx: *mut pssa_b200_ctx,
        a: *const f32,
        b: *const f32,
        h0: *const f32,
        h: *mut f32,
        h_last: *mut f32,
        lanes: usize,
        len: usize,
        stride: usize,
        chunks: u32,
    ) -> i32;
    pub fn pssa_b200_ssm_forward_dev(
        ctx: *mut pssa_b200_ctx,
        delta: *const f32,
        b_proj: *const f32,
        c_proj: *const f32,
        x_norm: *const f32,
        rates: *const f32,
        carry: *mut f32,
        y: *mut f32,
        states: *mut f32,
        bar_a: *mut f32,
        bar_b: *mut f32,
        offsets: *const u32,
        lengths: *const u32,
        lanes: usize,
        rows: usize,
        d_m: usize,
        d_s: usize,
        flags: u32,
    ) -> i32;
    pub fn pssa_b200_ssm_forward(
        ctx: *mut pssa_b200_ctx,
        delta: *const f32,
        b_proj: *const f32,
        x_norm: *const f32,
        rates: *const f32,
        c_proj: *const f32,
        initial: *const f32,
        seq_len: usize,
        d_m: usize,
        d_s: usize,
        bar_a: *mut f32,
        bar_b: *mut f32,
        states: *mut f32,
        y_ssm: *mut f32,
        flags: u32,
    ) -> i32;
    pub fn pssa_b200_memory_read_dev(
        ctx: *mut pssa_b200_ctx,
        q: *const f32,
        q_is_euclidean: i32,
        keys: *const f32,
        norm_sq: *const f32,
        values: *const f32,
        rows: usize,
        d_key: usize,
        d_val: usize,
        capacity: usize,
        count: usize,
        tau: f32,
        top_k: usize,
        q_pnc: *mut f32,
        q_norm: *mut f32,
        weights: *mut f32,
        m_val: *mut f32,
        min_dist: *mut f32,
        flags: u32,
    ) -> i32;
    pub fn pssa_b200_memory_read(
        ctx: *mut pssa_b200_ctx,
        q: *const f32,
        q_is_euclidean: i32,
        keys: *const f32,
        norm_sq: *const f32,
        values: *const f32,
        rows: usize,
        d_key: usize,
        d_val: usize,
        capacity: usize,
        count: usize,
        tau: f32,
        top_k: usize,
        q_pnc: *mut f32,
        q_norm: *mut f32,
        weights: *mut f32,
        m_val: *mut f32,
        min_dist: *mut f32,
        flags: u32,
    ) -> i32;
    pub fn pssa_b200_memory_read_topk_dev(
        ctx: *mut pssa_b200_ctx,
        q: *const f32,
        q_is_euclidean: i32,
        keys: *const f32,
        norm_sq: *const f32,
        values: *const f32,
        rows: usize,
        d_key: usize,
        d_val: usize,
        capacity: usize,
        count: usize,
        tau: f32,
        top_k: usize,
        q_pnc: *mut f32,
        q_norm: *mut f32,
        m_val: *mut f32,
        min_dist: *mut f32,
        slots_out: *mut u32,
        weights_out: *mut f32,
        handed_over: *mut u32,
        flags: u32,
    ) -> i32;
    pub fn pssa_b200_memory_forward(
        ctx: *mut pssa_b200_ctx,
        x_norm: *const f32,
        y_ssm: *const f32,
        w_qx: *const f32,
        w_qh: *const f32,
        w_gate: *const f32,
        w_proj: *const f32,
        keys: *const f32,
        norm_sq: *const f32,
        values: *const f32,
        seq_len: usize,
        d_m: usize,
        d_k: usize,
        d_val: usize,
        capacity: usize,
        count: usize,
        tau: f32,
        q_euc: *mut f32,
        q_pnc: *mut f32,
        q_norm: *mut f32,
        weights: *mut f32,
        m_val: *mut f32,
        g_mem: *mut f32,
        m_proj: *mut f32,
        m_inj: *mut f32,
        precision: i32,
    ) -> i32;
    pub fn pssa_b200_memory_forward_dev(
        ctx: *mut pssa_b200_ctx,
        x_norm: *const f32,
        y_ssm: *const f32,
        w_qx: *const f32,
        w_qh: *const f32,
        w_gate: *const f32,
        w_proj: *const f32,
        keys: *const f32,
        norm_sq: *const f32,
        values: *const f32,
        seq_len: usize,
        d_m: usize,
        d_k: usize,
        d_val: usize,
        capacity: usize,
        count: usize,
        tau: f32,
        q_euc: *mut f32,
        q_pnc: *mut f32,
        q_norm: *mut f32,
        weights: *mut f32,
        m_val: *mut f32,
        g_mem: *mut f32,
        m_proj: *mut f32,
        m_inj: *mut f32,
        precision: i32,
    ) -> i32;
    pub fn pssa_b200_ssm_forward_resident(
        ctx: *mut pssa_b200_ctx,
        delta: *const f32,
        delta_raw: *const f32,
        b_proj: *const f32,
        x_norm: *const f32,
        rates: *const f32,
        c_proj: *const f32,
        initial: *const f32,
        seq_len: usize,
        d_m: usize,
        d_s: usize,
        flags: u32,
    ) -> i32;
    pub fn pssa_b200_memory_forward_after_ssm(
        ctx: *mut pssa_b200_ctx,
        x_norm: *const f32,
        w_qx: *const f32,
        w_qh: *const f32,
        w_gate: *const f32,
        w_proj: *const f32,
        keys: *const f32,
        norm_sq: *const f32,
        values: *const f32,
        seq_len: usize,
        d_m: usize,
        d_k: usize,
        d_val: usize,
        capacity: usize,
        count: usize,
        tau: f32,
        bar_a: *mut f32,
        bar_b: *mut f32,
        states: *mut f32,
        y_ssm: *mut f32,
        q_euc: *mut f32,
        q_pnc: *mut f32,
        q_norm: *mut f32,
        weights: *mut f32,
        m_val: *mut f32,
        g_mem: *mut f32,
        m_proj: *mut f32,
        m_inj: *mut f32,
        precision: i32,
    ) -> i32;
    pub fn pssa_b200_bank_insert_protected_dev(
        ctx: *mut pssa_b200_ctx,
        keys: *mut f32,
        norm_sq: *mut f32,
        values: *mut f32,
        confidence: *mut f32,
        last_seen_step: *mut u64,
        meta: *mut u64,
        capacity: usize,
        d_key: usize,
        d_val: usize,
        key_pnc: *const f32,
        val: *const f32,
        surprise: *const f32,
        step: *const u64,
        n: usize,
        slots_out: *mut i64,
        winning_slots: *const u32,
        eta: f32,
    ) -> i32;
    pub fn pssa_b200_adapter_plastic_update_dev(
        ctx: *mut pssa_b200_ctx,
        up_fast: *mut f32,
        value: *const f32,
        ad_out: *const f32,
        ad_act: *const f32,
        d: usize,
        rank: usize,
    ) -> i32;
    pub fn pssa_b200_adapter_consolidate_dev(
        ctx: *mut pssa_b200_ctx,
        up_fast: *mut f32,
        up_slow: *mut f32,
        n: usize,
        alpha: f32,
    ) -> i32;
    pub fn pssa_b200_gemm_xwt(
        ctx: *mut pssa_b200_ctx,
        x: *const f32,
        w: *const f32,
        m: usize,
        n: usize,
        k: usize,
        batch: usize,
        out: *mut f32,
        epilogue: i32,
        alpha: f32,
        precision: i32,
    ) -> i32;
    pub fn pssa_b200_gemm_xwt_dev(
        ctx: *mut pssa_b200_ctx,
        x: *const f32,
        w: *const f32,
        rows: usize,
        n: usize,
        k: usize,
        out: *mut f32,
        ldo: usize,
        epilogue: i32,
        alpha: f32,
        precision: i32,
    ) -> i32;
    pub fn pssa_b200_model_create(
        ctx: *mut pssa_b200_ctx,
        cfg: *const pssa_b200_config,
        max_streams: u32,
        out: *mut *mut pssa_b200_model,
    ) -> i32;
    pub fn pssa_b200_model_destroy(model: *mut pssa_b200_model);
    pub fn pssa_b200_model_set_tensor(
        model: *mut pssa_b200_model,
        layer: i32,
        tensor: i32,
        data: *const f32,
        len: usize,
    ) -> i32;
    pub fn pssa_b200_model_insert_memory(model: *mut pssa_b200_model, index: u32, loss: f32, step: u64, slots_out: *mut i64) -> i32;
    pub fn pssa_b200_model_sampler_push(model: *mut pssa_b200_model, stream: u32, ids: *const u64, n: usize) -> i32;
    pub fn pssa_b200_model_reserve(model: *mut pssa_b200_model, rows: usize, lanes: usize) -> i32;
    pub fn pssa_b200_model_get_tensor(
        model: *mut pssa_b200_model,
        layer: i32,
        tensor: i32,
        out: *mut f32,
        len: usize,
    ) -> i32;
    pub fn pssa_b200_model_init_random(
        model: *mut pssa_b200_model,
        seed: u64,
        rng_state_out: *mut u64,
    ) -> i32;
    pub fn pssa_b200_model_set_bank(
        model: *mut pssa_b200_model,
        layer: i32,
        keys: *const f32,
        norm_sq: *const f32,
        values: *const f32,
        count: u64,
        write_head: u64,
        confidence: *const f32,
        last_seen_step: *const u64,
    ) -> i32;
    pub fn pssa_b200_model_set_top_k(model: *mut pssa_b200_model, top_k: usize) -> i32;
    pub fn pssa_b200_model_set_precision(model: *mut pssa_b200_model, precision: i32) -> i32;
    pub fn pssa_b200_model_set_option(model: *mut pssa_b200_model, option: i32, value: i32) -> i32;
    pub fn pssa_b200_model_reset_state(model: *mut pssa_b200_model, stream: u32) -> i32;
    pub fn pssa_b200_model_get_state(model: *mut pssa_b200_model, stream: u32, out: *mut f32, len: usize) -> i32;
    pub fn pssa_b200_model_set_state(model: *mut pssa_b200_model, stream: u32, data: *const f32, len: usize) -> i32;
    pub fn pssa_b200_model_prefill(
        model: *mut pssa_b200_model,
        stream: u32,
        ids: *const u64,
        n: usize,
        logits: *mut f32,
        processed: *mut usize,
        cancelled: Option<unsafe extern "C" fn(*mut c_void) -> i32>,
        cancel_arg: *mut c_void,
    ) -> i32;
    pub fn pssa_b200_model_prefill_batch(
        model: *mut pssa_b200_model,
        ids: *const u64,
        offsets: *const u32,
        lengths: *const u32,
        streams: *const u32,
        n_lanes: usize,
        logits: *mut f32,
        greedy: *mut u64,
    ) -> i32;
    pub fn pssa_b200_model_prefill_batch_dev(
        model: *mut pssa_b200_model,
        ids_dev: *const u32,
        offsets: *const u32,
        lengths: *const u32,
        streams: *const u32,
        n_lanes: usize,
        logits_dev: *mut f32,
        greedy_dev: *mut u32,
    ) -> i32;
    pub fn pssa_b200_model_decode_step(
        model: *mut pssa_b200_model,
        streams: *const u32,
        ids: *const u64,
        n: usize,
        logits: *mut f32,
        greedy: *mut u64,
    ) -> i32;
    pub fn pssa_b200_sample_dev(
        ctx: *mut pssa_b200_ctx,
        logits: *mut f32,
        probs: *mut f32,
        rows: usize,
        vocab: usize,
        cfg: *const pssa_b200_sampling,
        recent_ids: *const u32,
        recent_count: *const u32,
        rng_state: *mut u64,
        ids_out: *mut u32,
        status_out: *mut u32,
        confidence_out: *mut f32,
        flags: u32,
    ) -> i32;
    pub fn pssa_b200_model_score(
        m: *mut pssa_b200_model,
        stream: u32,
        ids: *const u64,
        targets: *const u64,
        n: usize,
        mean_loss: *mut f32,
        token_loss: *mut f32,
        logits_out: *mut f32,
    ) -> i32;
    pub fn pssa_b200_model_set_observer(m: *mut pssa_b200_model, enabled: i32) -> i32;
    pub fn pssa_b200_model_get_observation(
        m: *mut pssa_b200_model,
        layer: u32,
        index: u32,
        mem_weights: *mut f32,
        q_pnc: *mut f32,
        m_val: *mut f32,
        z_final: *mut f32,
    ) -> i32;
    pub fn pssa_b200_model_sampler_seed(m: *mut pssa_b200_model, stream: u32, seed: u64) -> i32;
    pub fn pssa_b200_model_decode_step_sampled(
        m: *mut pssa_b200_model,
        streams: *const u32,
        ids: *const u64,
        n: usize,
        cfg: *const pssa_b200_sampling,
        flags: u32,
        ids_out: *mut u64,
        confidence_out: *mut f32,
    ) -> i32;
    pub fn pssa_b200_checkpoint_probe(
        bytes: *const c_void,
        len: usize,
        config: *mut pssa_b200_config,
        version: *mut u32,
        error: *mut c_char,
        error_len: usize,
    ) -> i32;
    pub fn pssa_b200_model_load_checkpoint(
        ctx: *mut pssa_b200_ctx,
        bytes: *const c_void,
        len: usize,
        max_streams: u32,
        out: *mut *mut pssa_b200_model,
    ) -> i32;
    pub fn pssa_b200_model_set_seqpar(
        m: *mut pssa_b200_model,
        rank: u32,
        world: u32,
        send_dev: *mut c_void,
        recv_dev: *mut c_void,
        capacity: usize,
        exchange: pssa_b200_exchange_fn,
        arg: *mut c_void,
    ) -> i32;
    pub fn pssa_b200_model_set_max_rows(model: *mut pssa_b200_model, max_rows: usize) -> i32;
}
