//! `B200Context`: what a `GpuDispatch::B200(B200Context)` / `Device::B200(B200Context)` arm of the reference crate
//! (src/backend.rs:1012-1029) holds and delegates to, method for method, for the inference forward path. Source only:
//! the build image has no Rust toolchain, so this file is checked against the C header by the tests of the Python
//! binding (same symbols, same argument order), not compiled there.
//!
//! How it plugs in (additions to src/backend.rs, behind a cargo feature `b200`):
//!
//! ```ignore
//! pub enum Device { Cpu, Gpu(WgpuContext), #[cfg(feature = "cuda")] Cuda(CudaContext),
//!                   #[cfg(feature = "b200")] B200(crate::backend_b200::B200Context) }
//! pub enum GpuDispatch { Wgpu(WgpuContext), #[cfg(feature = "cuda")] Cuda(CudaContext),
//!                        #[cfg(feature = "b200")] B200(crate::backend_b200::B200Context) }
//! // every `match self { .. }` of `impl GpuDispatch` gains `Self::B200(ctx) => ctx.<same method>(<same arguments>)`;
//! // `Device::gpu()` gains `Device::B200(ctx) => Some(GpuDispatch::B200(ctx.clone()))`;
//! // `Device::try_gpu()` tries `B200Context::init(0)` first.
//! ```
//!
//! Differences from the CUDA arm, all deliberate: there is NO CPU fallback (`dispatch_gemm_into` returns the error
//! instead of calling `gemm_cpu_into`); weights are not cached by host pointer at this level (the model-level API,
//! `B200Model` below, keeps weights, banks and carries resident and is what inference should use); the backward
//! methods of `GpuDispatch` are not provided (training is outside this path) and return `Err`.
use std::ffi::CStr;
use std::os::raw::c_void;
use std::ptr;
use std::sync::{Arc, Mutex};

use crate::pssa_b200_sys as sys;

/// Owns one `pssa_b200_ctx`. `Clone` shares it; calls serialise on the mutex, like `CudaContext` (src/cuda.rs:155-166).
#[derive(Clone)]
pub struct B200Context {
    inner: Arc<Mutex<CtxHandle>>,
    label: String,
}

struct CtxHandle(*mut sys::pssa_b200_ctx);
// The library's context is single-threaded; the mutex above provides that.
unsafe impl Send for CtxHandle {}

impl Drop for CtxHandle {
    fn drop(&mut self) {
        unsafe { sys::pssa_b200_ctx_destroy(self.0) }
    }
}

fn last_error(ctx: *const sys::pssa_b200_ctx) -> String {
    unsafe {
        let p = sys::pssa_b200_last_error(ctx);
        if p.is_null() { "unknown B200 error".into() } else { CStr::from_ptr(p).to_string_lossy().into_owned() }
    }
}

/// Fatal classes follow src/cuda.rs:592-602: once seen the context is unusable and the caller should stop.
pub fn panic_if_fatal_b200_error(status: i32, message: &str) {
    if status == sys::PSSA_B200_ERR_FATAL_CUDA {
        panic!("fatal B200 error: {message}");
    }
}

impl B200Context {
    /// Replaces `CudaContext::init` (src/cuda.rs:168-196).
    pub fn init(device: i32) -> Result<Self, String> {
        let mut raw = ptr::null_mut();
        let rc = unsafe { sys::pssa_b200_ctx_create(device, &mut raw) };
        if rc != sys::PSSA_B200_OK {
            return Err(last_error(ptr::null()));
        }
        let label = unsafe { CStr::from_ptr(sys::pssa_b200_backend_label(raw)).to_string_lossy().into_owned() };
        Ok(Self { inner: Arc::new(Mutex::new(CtxHandle(raw))), label })
    }

    fn with<R>(&self, f: impl FnOnce(*mut sys::pssa_b200_ctx) -> i32, ok: R) -> Result<R, String> {
        let guard = self.inner.lock().map_err(|_| "B200 context poisoned".to_string())?;
        let rc = f(guard.0);
        if rc == sys::PSSA_B200_OK {
            Ok(ok)
        } else {
            let message = last_error(guard.0);
            panic_if_fatal_b200_error(rc, &message);
            Err(message)
        }
    }

    /// `backend_label` (src/backend.rs:1439-1446): "b200 (<device name>)".
    pub fn backend_label(&self) -> String {
        self.label.clone()
    }

    /// `try_dispatch_gemm_into` (src/backend.rs:1051-1083): Y[batch,M,N] = X[batch,M,K] * W[N,K]^T, fp32 with the
    /// reference's `dot_slice` reduction order (bit-equal to `gemm_cpu_into`). Output untouched on a shape error.
    pub fn try_dispatch_gemm_into(&self, x: &[f32], w: &[f32], m: usize, n: usize, k: usize, batch: usize, out: &mut [f32]) -> Result<(), String> {
        let (_, _, expected) = crate::backend::checked_gemm_sizes(m, n, k, batch, x.len(), w.len())?;
        if out.len() != expected {
            return Err("GEMM output length mismatch".into());
        }
        self.with(
            |c| unsafe {
                sys::pssa_b200_gemm_xwt(c, x.as_ptr(), w.as_ptr(), m, n, k, batch, out.as_mut_ptr(), sys::PSSA_B200_EPI_NONE, 1.0, sys::PSSA_B200_PRECISION_FP32_EXACT)
            },
            (),
        )
    }

    /// `dispatch_gemm_into` (src/backend.rs:1087-1110) WITHOUT the CPU fallback: a device failure is returned.
    pub fn dispatch_gemm_into(&self, x: &[f32], w: &[f32], m: usize, n: usize, k: usize, batch: usize, out: &mut [f32]) -> Result<(), String> {
        self.try_dispatch_gemm_into(x, w, m, n, k, batch, out)
    }

    pub fn try_dispatch_gemm(&self, x: &[f32], w: &[f32], m: usize, n: usize, k: usize, batch: usize) -> Result<Vec<f32>, String> {
        let (_, _, expected) = crate::backend::checked_gemm_sizes(m, n, k, batch, x.len(), w.len())?;
        let mut out = vec![0.0f32; expected];
        self.try_dispatch_gemm_into(x, w, m, n, k, batch, &mut out)?;
        Ok(out)
    }

    pub fn dispatch_gemm(&self, x: &[f32], w: &[f32], m: usize, n: usize, k: usize, batch: usize) -> Vec<f32> {
        self.try_dispatch_gemm(x, w, m, n, k, batch).unwrap_or_else(|e| panic!("B200 GEMM failed (no CPU fallback on this path): {e}"))
    }

    /// `softplus_in_place` (src/backend.rs:1419-1425). The device path applies softplus as the epilogue of the projection
    /// that produces the values; a bare elementwise call gains nothing from a round trip, so it runs the reference's
    /// scalar formula on the host, as the reference's own CUDA arm does for short vectors.
    pub fn softplus_in_place(&self, values: &mut [f32]) -> Result<(), String> {
        for v in values {
            *v = crate::linalg::softplus(*v);
        }
        Ok(())
    }

    /// `invalidate_weights` / `invalidate_weights_only` (src/backend.rs:1113-1133): nothing is cached by host pointer at
    /// this level; `B200Model::set_tensor` re-uploads what changed.
    pub fn invalidate_weights(&self) {}
    pub fn invalidate_weights_only(&self, _keys: &[(usize, usize)]) {}

    /// `accelerates_backward` (src/backend.rs:1431-1437): training is outside this path.
    pub fn accelerates_backward(&self) -> bool {
        false
    }

    /// `ssm_forward` (src/backend.rs:1215-1244); delta_raw and rate_deriv are backward-only inputs and are not read.
    #[allow(clippy::too_many_arguments)]
    pub fn ssm_forward(&self, delta: &[f32], _delta_raw: &[f32], b_proj: &[f32], x_norm: &[f32], rates: &[f32], _rate_deriv: &[f32], c_proj: &[f32],
                       initial: &[f32], seq_len: usize, d_m: usize, d_s: usize, bar_a: &mut [f32], bar_b: &mut [f32], states: &mut [f32],
                       y_ssm: &mut [f32]) -> Result<(), String> {
        let stride = d_m.checked_mul(d_s).ok_or("SSM stride overflow")?;
        if delta.len() != seq_len * d_m || x_norm.len() != seq_len * d_m || y_ssm.len() != seq_len * d_m || b_proj.len() != seq_len * d_s
            || c_proj.len() != seq_len * d_s || rates.len() != stride || initial.len() != stride || bar_a.len() != seq_len * stride
            || bar_b.len() != seq_len * stride || states.len() != (seq_len + 1) * stride {
            return Err("B200 SSM forward buffer lengths do not match the shape; refusing launch".into());
        }
        self.with(
            |c| unsafe {
                sys::pssa_b200_ssm_forward(c, delta.as_ptr(), b_proj.as_ptr(), x_norm.as_ptr(), rates.as_ptr(), c_proj.as_ptr(), initial.as_ptr(), seq_len, d_m,
                                           d_s, bar_a.as_mut_ptr(), bar_b.as_mut_ptr(), states.as_mut_ptr(), y_ssm.as_mut_ptr(), sys::PSSA_B200_SSM_EXACT)
            },
            (),
        )
    }

    /// `ssm_forward_resident` (src/backend.rs:1186-1212): the tape stays on the device for `memory_forward_after_ssm`.
    #[allow(clippy::too_many_arguments)]
    pub fn ssm_forward_resident(&self, delta: &[f32], delta_raw: &[f32], b_proj: &[f32], x_norm: &[f32], rates: &[f32], c_proj: &[f32], initial: &[f32],
                                seq_len: usize, d_m: usize, d_s: usize) -> Result<(), String> {
        let stride = d_m.checked_mul(d_s).ok_or("SSM stride overflow")?;
        if delta.len() != seq_len * d_m || x_norm.len() != seq_len * d_m || b_proj.len() != seq_len * d_s || c_proj.len() != seq_len * d_s
            || rates.len() != stride || initial.len() != stride {
            return Err("B200 SSM forward buffer lengths do not match the shape; refusing launch".into());
        }
        self.with(
            |c| unsafe {
                sys::pssa_b200_ssm_forward_resident(c, delta.as_ptr(), delta_raw.as_ptr(), b_proj.as_ptr(), x_norm.as_ptr(), rates.as_ptr(), c_proj.as_ptr(),
                                                    initial.as_ptr(), seq_len, d_m, d_s, sys::PSSA_B200_SSM_EXACT)
            },
            (),
        )
    }

    /// `memory_forward` (src/backend.rs:1342-1385), same 24 arguments.
    #[allow(clippy::too_many_arguments)]
    pub fn memory_forward(&self, x_norm: &[f32], y_ssm: &[f32], w_qx: &[f32], w_qh: &[f32], w_gate: &[f32], w_proj: &[f32], keys: &[f32], norm_sq: &[f32],
                          values: &[f32], seq_len: usize, d_m: usize, d_k: usize, d_val: usize, capacity: usize, count: usize, tau: f32, q_euc: &mut [f32],
                          q_pnc: &mut [f32], q_norm: &mut [f32], weights: &mut [f32], m_val: &mut [f32], g_mem: &mut [f32], m_proj: &mut [f32],
                          m_inj: &mut [f32]) -> Result<(), String> {
        memory_lengths(x_norm, Some(y_ssm), w_qx, w_qh, w_gate, w_proj, keys, norm_sq, values, seq_len, d_m, d_k, d_val, capacity, q_euc, q_pnc, q_norm,
                       weights, m_val, g_mem, m_proj, m_inj)?;
        self.with(
            |c| unsafe {
                sys::pssa_b200_memory_forward(c, x_norm.as_ptr(), y_ssm.as_ptr(), w_qx.as_ptr(), w_qh.as_ptr(), w_gate.as_ptr(), w_proj.as_ptr(), keys.as_ptr(),
                                              norm_sq.as_ptr(), values.as_ptr(), seq_len, d_m, d_k, d_val, capacity, count, tau, q_euc.as_mut_ptr(),
                                              q_pnc.as_mut_ptr(), q_norm.as_mut_ptr(), weights.as_mut_ptr(), m_val.as_mut_ptr(), g_mem.as_mut_ptr(),
                                              m_proj.as_mut_ptr(), m_inj.as_mut_ptr(), sys::PSSA_B200_PRECISION_FP32_EXACT)
            },
            (),
        )
    }

    /// `memory_forward_after_ssm` (src/backend.rs:1246-1289), same 27 arguments.
    #[allow(clippy::too_many_arguments)]
    pub fn memory_forward_after_ssm(&self, x_norm: &[f32], w_qx: &[f32], w_qh: &[f32], w_gate: &[f32], w_proj: &[f32], keys: &[f32], norm_sq: &[f32],
                                    values: &[f32], seq_len: usize, d_m: usize, d_k: usize, d_val: usize, capacity: usize, count: usize, tau: f32,
                                    bar_a: &mut [f32], bar_b: &mut [f32], states: &mut [f32], y_ssm: &mut [f32], q_euc: &mut [f32], q_pnc: &mut [f32],
                                    q_norm: &mut [f32], weights: &mut [f32], m_val: &mut [f32], g_mem: &mut [f32], m_proj: &mut [f32], m_inj: &mut [f32])
                                    -> Result<(), String> {
        memory_lengths(x_norm, None, w_qx, w_qh, w_gate, w_proj, keys, norm_sq, values, seq_len, d_m, d_k, d_val, capacity, q_euc, q_pnc, q_norm, weights,
                       m_val, g_mem, m_proj, m_inj)?;
        if y_ssm.len() != seq_len * d_m {
            return Err("B200 memory forward buffer lengths do not match the shape; refusing launch".into());
        }
        self.with(
            |c| unsafe {
                sys::pssa_b200_memory_forward_after_ssm(c, x_norm.as_ptr(), w_qx.as_ptr(), w_qh.as_ptr(), w_gate.as_ptr(), w_proj.as_ptr(), keys.as_ptr(),
                                                        norm_sq.as_ptr(), values.as_ptr(), seq_len, d_m, d_k, d_val, capacity, count, tau, bar_a.as_mut_ptr(),
                                                        bar_b.as_mut_ptr(), states.as_mut_ptr(), y_ssm.as_mut_ptr(), q_euc.as_mut_ptr(), q_pnc.as_mut_ptr(),
                                                        q_norm.as_mut_ptr(), weights.as_mut_ptr(), m_val.as_mut_ptr(), g_mem.as_mut_ptr(), m_proj.as_mut_ptr(),
                                                        m_inj.as_mut_ptr(), sys::PSSA_B200_PRECISION_FP32_EXACT)
            },
            (),
        )
    }

    /// The backward half of `GpuDispatch` (src/backend.rs:1136-1185, 1291-1417) is training and not on this path.
    pub fn backward_unsupported<T>(&self) -> Result<T, String> {
        Err("the B200 path implements the inference forward path only".into())
    }

    /// Model-level entry: device-resident weights, banks and carries (`PSSALayerV2` inference API, src/pssa.rs:2245-2442).
    pub fn create_model(&self, cfg: &sys::pssa_b200_config, max_streams: u32) -> Result<B200Model, String> {
        let guard = self.inner.lock().map_err(|_| "B200 context poisoned".to_string())?;
        let mut raw = ptr::null_mut();
        let rc = unsafe { sys::pssa_b200_model_create(guard.0, cfg, max_streams, &mut raw) };
        if rc != sys::PSSA_B200_OK {
            return Err(last_error(guard.0));
        }
        Ok(B200Model { ctx: self.clone(), raw, vocab: cfg.d_vocab as usize, carry_len: (cfg.depth * cfg.d_latent * cfg.d_state) as usize, loops: 1 })
    }
}

#[allow(clippy::too_many_arguments)]
fn memory_lengths(x_norm: &[f32], y_ssm: Option<&[f32]>, w_qx: &[f32], w_qh: &[f32], w_gate: &[f32], w_proj: &[f32], keys: &[f32], norm_sq: &[f32],
                  values: &[f32], seq_len: usize, d_m: usize, d_k: usize, d_val: usize, capacity: usize, q_euc: &[f32], q_pnc: &[f32], q_norm: &[f32],
                  weights: &[f32], m_val: &[f32], g_mem: &[f32], m_proj: &[f32], m_inj: &[f32]) -> Result<(), String> {
    let ok = x_norm.len() == seq_len * d_m && y_ssm.map_or(true, |y| y.len() == seq_len * d_m) && w_qx.len() == d_k * d_m && w_qh.len() == d_k * d_m
        && w_gate.len() == d_m * d_m && w_proj.len() == d_m * d_val && keys.len() == capacity * d_k && norm_sq.len() == capacity
        && values.len() == capacity * d_val && q_euc.len() == seq_len * d_k && q_pnc.len() == seq_len * d_k && q_norm.len() == seq_len
        && weights.len() == seq_len * capacity && m_val.len() == seq_len * d_val && g_mem.len() == seq_len * d_m && m_proj.len() == seq_len * d_m
        && m_inj.len() == seq_len * d_m;
    if ok { Ok(()) } else { Err("B200 memory forward buffer lengths do not match the shape; refusing launch".into()) }
}

/// A device-resident model: what `PSSALayerV2` keeps in `self.device` terms when the device is `Device::B200`.
pub struct B200Model {
    ctx: B200Context,
    raw: *mut sys::pssa_b200_model,
    vocab: usize,
    carry_len: usize,  // depth * d_latent * d_state: the carries of one pass
    loops: usize,
}

impl Drop for B200Model {
    fn drop(&mut self) {
        let _guard = self.ctx.inner.lock();
        unsafe { sys::pssa_b200_model_destroy(self.raw) }
    }
}

impl B200Model {
    fn call(&self, f: impl FnOnce(*mut sys::pssa_b200_model) -> i32) -> Result<(), String> {
        let guard = self.ctx.inner.lock().map_err(|_| "B200 context poisoned".to_string())?;
        let rc = f(self.raw);
        if rc == sys::PSSA_B200_OK {
            Ok(())
        } else {
            let message = last_error(guard.0);
            panic_if_fatal_b200_error(rc, &message);
            Err(message)
        }
    }

    /// Upload one parameter (`ParamMatrix::data`), replacing the reference backends' weight caches.
    pub fn set_tensor(&self, layer: i32, tensor: i32, data: &[f32]) -> Result<(), String> {
        self.call(|m| unsafe { sys::pssa_b200_model_set_tensor(m, layer, tensor, data.as_ptr(), data.len()) })
    }

    /// `insert_training_memory_at` on the device-resident banks; returns the per-block slots.
    pub fn insert_memory(&self, index: u32, loss: f32, step: u64, slots_out: &mut [i64]) -> Result<(), String> {
        self.call(|m| unsafe { sys::pssa_b200_model_insert_memory(m, index, loss, step, slots_out.as_mut_ptr()) })
    }

    /// Appends the prompt to a stream's repetition window (`generated_ids` starts as a copy of the prompt).
    pub fn sampler_push(&self, stream: u32, ids: &[u64]) -> Result<(), String> {
        self.call(|m| unsafe { sys::pssa_b200_model_sampler_push(m, stream, ids.as_ptr(), ids.len()) })
    }

    /// Reads a parameter back into a host slice (what checkpoint saving reads from `ParamMatrix` fields).
    pub fn get_tensor(&self, layer: i32, tensor: i32, out: &mut [f32]) -> Result<(), String> {
        self.call(|m| unsafe { sys::pssa_b200_model_get_tensor(m, layer, tensor, out.as_mut_ptr(), out.len()) })
    }

    /// `PSSALayerV2::new(cfg, seed)`'s random init on the device model; returns the generator state to keep.
    pub fn init_random(&self, seed: u64) -> Result<u64, String> {
        let mut state = 0u64;
        self.call(|m| unsafe { sys::pssa_b200_model_init_random(m, seed, &mut state) })?;
        Ok(state)
    }

    /// Upload one block's `HyperbolicEpisodicBankV2` (src/memory.rs:4-33).
    #[allow(clippy::too_many_arguments)]
    pub fn set_bank(&self, layer: i32, keys: &[f32], norm_sq: &[f32], values: &[f32], count: usize, write_head: usize, confidence: &[f32],
                    last_seen_step: &[u64]) -> Result<(), String> {
        self.call(|m| unsafe {
            sys::pssa_b200_model_set_bank(m, layer, keys.as_ptr(), norm_sq.as_ptr(), values.as_ptr(), count as u64, write_head as u64, confidence.as_ptr(),
                                          last_seen_step.as_ptr())
        })
    }

    /// `set_loops` (src/pssa.rs:2171-2184).
    pub fn set_loops(&mut self, loops: usize) -> Result<(), String> {
        if !(1..=32).contains(&loops) {
            return Err("--loops must be between 1 and 32; use --loops 1 for the original model".into());
        }
        self.call(|m| unsafe { sys::pssa_b200_model_set_option(m, 4, loops as i32) })?;
        self.loops = loops;
        Ok(())
    }

    /// `set_memory_top_k` (src/pssa.rs:2215-2229); the one runtime option the device path adds.
    pub fn set_memory_top_k(&self, top_k: Option<usize>) -> Result<(), String> {
        if top_k == Some(0) {
            return Err("memory top-k must be positive".into());
        }
        self.call(|m| unsafe { sys::pssa_b200_model_set_top_k(m, top_k.unwrap_or(0)) })
    }

    /// `reset_recurrent_state` (src/pssa.rs:2245-2250) for stream 0.
    pub fn reset_recurrent_state(&self) -> Result<(), String> {
        self.call(|m| unsafe { sys::pssa_b200_model_reset_state(m, 0) })
    }

    /// `copy_recurrent_state_to / from` (src/pssa.rs:2263-2310): `[block][pass][d*s]`.
    pub fn copy_recurrent_state_to(&self, out: &mut [f32]) -> Result<(), String> {
        self.call(|m| unsafe { sys::pssa_b200_model_get_state(m, 0, out.as_mut_ptr(), out.len()) })
    }
    pub fn copy_recurrent_state_from(&self, state: &[f32]) -> Result<(), String> {
        self.call(|m| unsafe { sys::pssa_b200_model_set_state(m, 0, state.as_ptr(), state.len()) })
    }

    /// `forward_inference` (src/pssa.rs:2387-2391). Panics on a bad id or length like the reference (src/pssa.rs:2317, 2388).
    pub fn forward_inference(&self, x_id: usize, logits_out: &mut [f32]) {
        assert_eq!(logits_out.len(), self.vocab);
        assert!(x_id < self.vocab, "token ID must be in vocabulary");
        let id = x_id as u64;
        self.call(|m| unsafe { sys::pssa_b200_model_decode_step(m, ptr::null(), &id, 1, logits_out.as_mut_ptr(), ptr::null_mut()) })
            .unwrap_or_else(|e| panic!("B200 forward_inference failed: {e}"));
    }

    /// `prefill_inference` (src/pssa.rs:2399-2442): `Ok(false)` on cancellation, `Err` for an empty prompt or an id outside
    /// the vocabulary (after the valid prefix has advanced the carry); logits untouched in both cases.
    pub fn prefill_inference<C: Fn() -> bool>(&self, token_ids: &[usize], logits_out: Option<&mut [f32]>, cancelled: C) -> Result<bool, String> {
        unsafe extern "C" fn trampoline<C: Fn() -> bool>(arg: *mut c_void) -> i32 {
            let f = &*(arg as *const C);
            if f() { 1 } else { 0 }
        }
        let ids: Vec<u64> = token_ids.iter().map(|&t| t as u64).collect();
        let logits_ptr = logits_out.map_or(ptr::null_mut(), |l| {
            assert_eq!(l.len(), self.vocab);
            l.as_mut_ptr()
        });
        let mut processed = 0usize;
        let guard = self.ctx.inner.lock().map_err(|_| "B200 context poisoned".to_string())?;
        let rc = unsafe {
            sys::pssa_b200_model_prefill(self.raw, 0, ids.as_ptr(), ids.len(), logits_ptr, &mut processed, Some(trampoline::<C>),
                                         &cancelled as *const C as *mut c_void)
        };
        match rc {
            sys::PSSA_B200_OK => Ok(true),
            sys::PSSA_B200_ERR_CANCELLED => Ok(false),
            _ => {
                let message = last_error(guard.0);
                panic_if_fatal_b200_error(rc, &message);
                Err(message)
            }
        }
    }

    /// Independent sequences as lanes (`SequenceBatch::forward`, src/sequence_batch.rs:233-384): last-token logits per lane.
    pub fn prefill_batch(&self, ids: &[u64], offsets: &[u32], lengths: &[u32], logits: &mut [f32]) -> Result<(), String> {
        assert_eq!(logits.len(), lengths.len() * self.vocab);
        self.call(|m| unsafe {
            sys::pssa_b200_model_prefill_batch(m, ids.as_ptr(), offsets.as_ptr(), lengths.as_ptr(), ptr::null(), lengths.len(), logits.as_mut_ptr(),
                                               ptr::null_mut())
        })
    }

    /// `recurrent_state_len` (src/pssa.rs:2255-2261) without the local-conv histories the device path refuses.
    pub fn recurrent_state_len(&self) -> usize {
        self.carry_len * self.loops
    }
}
