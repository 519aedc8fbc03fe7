"""Host-side mirror of the reference's device seam (`Device` / `GpuDispatch`, src/backend.rs:1012-1482).

Method names, argument meaning and error behaviour follow the reference; every method is a thin call
into the C ABI. numpy arrays are host buffers (the reference's `&[f32]` slices); the `*_dev` methods
take device pointers (ints) or objects with `.data_ptr()` (torch tensors) and only enqueue work.
"""
import ctypes as C
import weakref

import numpy as np

from . import _native as N


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, int):
        return C.c_void_p(x)
    if isinstance(x, np.ndarray):
        return C.c_void_p(x.ctypes.data)
    if hasattr(x, "data_ptr"):
        return C.c_void_p(x.data_ptr())
    raise TypeError(f"cannot take a pointer of {type(x)}")


def _host(a, name, shape=None):
    if not isinstance(a, np.ndarray) or a.dtype != np.float32 or not a.flags["C_CONTIGUOUS"]:
        raise TypeError(f"{name} must be a C-contiguous float32 numpy array")
    if shape is not None and tuple(a.shape) != tuple(shape):
        raise ValueError(f"{name} has shape {a.shape}, expected {shape}")
    return a


class B200Dispatch:
    """One context on one B200 (`GpuDispatch::B200`)."""

    def __init__(self, device: int = 0, stream=None):
        self._lib = N.lib()
        h = C.c_void_p()
        rc = self._lib.pssa_b200_ctx_create(device, C.byref(h))
        if rc != N.OK:
            raise N.B200Error(rc, self._lib.pssa_b200_last_error(None).decode())
        self._h = h
        self.device = device
        if stream is not None:
            self.set_stream(stream)

    def _adopt(self, child):
        """Objects that hold a pointer to this context (models) are closed before the context is."""
        if not hasattr(self, "_children"):
            self._children = weakref.WeakSet()
        self._children.add(child)

    def close(self):
        for child in list(getattr(self, "_children", ())):
            child.close()
        if getattr(self, "_h", None):
            self._lib.pssa_b200_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc != N.OK:
            raise N.B200Error(rc, self._lib.pssa_b200_last_error(self._h).decode())

    # ---- context
    def set_stream(self, stream):
        """`stream`: a cudaStream_t as int (0 = legacy default stream), a torch.cuda.Stream, or None to
        return to the context's own non-blocking stream."""
        if stream is None:
            self._check(self._lib.pssa_b200_ctx_use_own_stream(self._h))
            return
        raw = getattr(stream, "cuda_stream", stream)
        self._check(self._lib.pssa_b200_ctx_set_stream(self._h, C.c_void_p(raw)))

    def synchronize(self):
        self._check(self._lib.pssa_b200_ctx_synchronize(self._h))

    def backend_label(self) -> str:  # src/backend.rs:1439-1446
        return self._lib.pssa_b200_backend_label(self._h).decode()

    def launch_count(self) -> int:
        return int(self._lib.pssa_b200_launch_count(self._h))

    def reserve(self, nbytes: int):
        self._check(self._lib.pssa_b200_ctx_reserve(self._h, nbytes))

    def set_scan_chunks(self, chunks: int):
        self._check(self._lib.pssa_b200_ctx_set_scan_chunks(self._h, chunks))

    # ---- scan operator
    def affine_scan_in_place(self, scan_a: np.ndarray, scan_b: np.ndarray, length: int, stride: int, lanes: int = 1):
        """Exclusive prefix of affine maps, in place (src/gpu_batch.rs:98-164). Host arrays."""
        _host(scan_a, "scan_a")
        _host(scan_b, "scan_b")
        if scan_a.size != lanes * length * stride or scan_b.size != lanes * length * stride:
            raise N.B200Error(N.ERR_SHAPE, "B200 affine scan: buffers must hold lanes*len*stride elements; refusing launch")
        self._check(self._lib.pssa_b200_affine_scan(self._h, _ptr(scan_a), _ptr(scan_b), lanes, length, stride))

    def affine_scan_dev(self, scan_a, scan_b, lanes: int, length: int, stride: int):
        self._check(self._lib.pssa_b200_affine_scan_dev(self._h, _ptr(scan_a), _ptr(scan_b), lanes, length, stride))

    def scan_states(self, a: np.ndarray, b: np.ndarray, h0=None, want_last=False):
        """All states of h_t = a_t*h_{t-1} + b_t for host arrays [lanes, len, stride]."""
        _host(a, "a")
        _host(b, "b", a.shape)
        lanes, length, stride = a.shape
        if h0 is not None:
            _host(h0, "h0", (lanes, stride))
        h = np.empty_like(a)
        last = np.empty((lanes, stride), np.float32) if want_last else None
        self._check(self._lib.pssa_b200_scan_states(self._h, _ptr(a), _ptr(b), _ptr(h0), _ptr(h), _ptr(last), lanes,
                                                    length, stride))
        return (h, last) if want_last else h

    def scan_states_dev(self, a, b, h0, h, h_last, lanes: int, length: int, stride: int):
        self._check(self._lib.pssa_b200_scan_states_dev(self._h, _ptr(a), _ptr(b), _ptr(h0), _ptr(h), _ptr(h_last),
                                                        lanes, length, stride))


    def scan_states_noalloc_dev(self, a, b, h0, h, h_last, lanes: int, length: int, stride: int, chunks: int):
        """Same result as `scan_states_dev` without any device allocation: for hosts that own all GPU memory
        themselves or cannot tolerate the synchronisation of cudaMalloc. Scratch is a fixed array inside the
        library (lanes*chunks*stride <= 2**20 when chunks > 1); concurrent calls on one GPU must be serialised."""
        self._check(self._lib.pssa_b200_scan_states_noalloc_dev(self._h, _ptr(a), _ptr(b), _ptr(h0), _ptr(h), _ptr(h_last),
                                                                lanes, length, stride, chunks))

    # ---- fused SSM stage
    def ssm_forward(self, delta, b_proj, x_norm, rates, c_proj, initial, seq_len, d_m, d_s, bar_a=None, bar_b=None,
                    states=None, y_ssm=None, exact=False):
        """`GpuDispatch::ssm_forward` (src/backend.rs:1215-1244) on host arrays; outputs are written in place.
        Lengths are checked like the reference's "CUDA SSM forward shape mismatch" (src/cuda/stages.rs:281-290)."""
        stride = d_m * d_s
        want = [("delta", delta, seq_len * d_m), ("b_proj", b_proj, seq_len * d_s), ("x_norm", x_norm, seq_len * d_m),
                ("rates", rates, stride), ("c_proj", c_proj, seq_len * d_s), ("initial", initial, stride),
                ("y_ssm", y_ssm, seq_len * d_m)]
        for name, arr, n in want:
            _host(arr, name)
            if arr.size != n:
                raise N.B200Error(N.ERR_SHAPE, f"B200 SSM forward shape mismatch: {name} has {arr.size} elements, "
                                               f"expected {n}; refusing launch")
        for name, arr, n in (("bar_a", bar_a, seq_len * stride), ("bar_b", bar_b, seq_len * stride),
                             ("states", states, (seq_len + 1) * stride)):
            if arr is not None and (_host(arr, name).size != n):
                raise N.B200Error(N.ERR_SHAPE, f"B200 SSM forward shape mismatch: {name}; refusing launch")
        self._check(self._lib.pssa_b200_ssm_forward(self._h, _ptr(delta), _ptr(b_proj), _ptr(x_norm), _ptr(rates),
                                                    _ptr(c_proj), _ptr(initial), seq_len, d_m, d_s, _ptr(bar_a),
                                                    _ptr(bar_b), _ptr(states), _ptr(y_ssm), N.SSM_EXACT if exact else 0))

    def ssm_forward_dev(self, delta, b_proj, c_proj, x_norm, rates, carry, y, offsets, lengths, rows, d_m, d_s,
                        states=None, bar_a=None, bar_b=None, exact=False):
        """Lane-batched, device-resident form: `offsets` / `lengths` are host uint32 arrays (or None for one lane)."""
        lanes = 1
        if offsets is not None:
            offsets = np.ascontiguousarray(offsets, np.uint32)
            lengths = np.ascontiguousarray(lengths, np.uint32)
            lanes = len(offsets)
        self._check(self._lib.pssa_b200_ssm_forward_dev(
            self._h, _ptr(delta), _ptr(b_proj), _ptr(c_proj), _ptr(x_norm), _ptr(rates), _ptr(carry), _ptr(y),
            _ptr(states), _ptr(bar_a), _ptr(bar_b), _ptr(offsets), _ptr(lengths), lanes, rows, d_m, d_s,
            N.SSM_EXACT if exact else 0))


    # ---- episodic memory read
    @staticmethod
    def _mem_flags(exact, f32_distance, tc_distance=False, no_fused=False, handover_selftest=False, phase_clocks=False):
        return ((N.MEM_EXACT if exact else 0) | (N.MEM_F32_DISTANCE if f32_distance else 0) |
                (N.MEM_TC_DISTANCE if tc_distance else 0) | (N.MEM_NO_FUSED if no_fused else 0) |
                (N.MEM_HANDOVER_SELFTEST if handover_selftest else 0) | (N.MEM_PHASE_CLOCKS if phase_clocks else 0))

    def memory_read_topk_dev(self, q, keys, norm_sq, values, rows, dk, dv, cap, count, tau, top_k, m_val, slots_out=None,
                             weights_out=None, q_pnc=None, q_norm=None, min_dist=None, handed_over=None, q_is_euclidean=True,
                             exact=False, no_fused=False, handover_selftest=False, phase_clocks=False):
        """Top-k read with compact results (device buffers): see pssa_b200_memory_read_topk_dev in include/pssa_b200.h."""
        self._check(self._lib.pssa_b200_memory_read_topk_dev(
            self._h, _ptr(q), 1 if q_is_euclidean else 0, _ptr(keys), _ptr(norm_sq), _ptr(values), rows, dk, dv, cap, count, tau,
            top_k, _ptr(q_pnc), _ptr(q_norm), _ptr(m_val), _ptr(min_dist), _ptr(slots_out), _ptr(weights_out), _ptr(handed_over),
            self._mem_flags(exact, False, False, no_fused, handover_selftest, phase_clocks)))

    def memory_read(self, q, keys, norm_sq, values, count, tau, top_k=0, q_is_euclidean=True, exact=False,
                    f32_distance=False, tc_distance=False, no_fused=False, handover_selftest=False):
        """Bank read on host arrays: returns (q_pnc, q_norm, weights, m_val, min_dist). Mirrors
        `retrieve_memory_rows` (src/gpu_batch.rs:700-741): project, distances, softmax / top-k, value read."""
        _host(q, "q")
        _host(keys, "keys")
        _host(values, "values")
        _host(norm_sq, "norm_sq")
        rows, dk = q.shape
        cap, dk2 = keys.shape
        dv = values.shape[1]
        if dk2 != dk or values.shape[0] != cap or norm_sq.size != cap:
            raise N.B200Error(N.ERR_SHAPE, "B200 memory read shape mismatch; refusing launch")
        q_pnc = np.empty((rows, dk), np.float32)
        q_norm = np.empty(rows, np.float32)
        weights = np.empty((rows, cap), np.float32)
        m_val = np.empty((rows, dv), np.float32)
        md = np.empty(rows, np.float32)
        self._check(self._lib.pssa_b200_memory_read(
            self._h, _ptr(q), 1 if q_is_euclidean else 0, _ptr(keys), _ptr(norm_sq), _ptr(values), rows, dk, dv, cap,
            count, tau, top_k or 0, _ptr(q_pnc), _ptr(q_norm), _ptr(weights), _ptr(m_val), _ptr(md),
            self._mem_flags(exact, f32_distance, tc_distance, no_fused, handover_selftest)))
        return q_pnc, q_norm, weights, m_val, md

    def memory_read_dev(self, q, keys, norm_sq, values, rows, dk, dv, cap, count, tau, m_val, top_k=0, q_pnc=None,
                        q_norm=None, weights=None, min_dist=None, q_is_euclidean=True, exact=False, f32_distance=False,
                        tc_distance=False, no_fused=False):
        self._check(self._lib.pssa_b200_memory_read_dev(
            self._h, _ptr(q), 1 if q_is_euclidean else 0, _ptr(keys), _ptr(norm_sq), _ptr(values), rows, dk, dv, cap,
            count, tau, top_k or 0, _ptr(q_pnc), _ptr(q_norm), _ptr(weights), _ptr(m_val), _ptr(min_dist),
            self._mem_flags(exact, f32_distance, tc_distance, no_fused)))


    # ---- stage-level operators with the reference's argument lists (src/backend.rs:1186-1289, 1342-1385)
    def _memory_outputs(self, seq_len, d_m, d_k, d_val, capacity):
        z = lambda *shape: np.zeros(shape, np.float32)  # noqa: E731
        return dict(q_euc=z(seq_len, d_k), q_pnc=z(seq_len, d_k), q_norm=z(seq_len), weights=z(seq_len, capacity),
                    m_val=z(seq_len, d_val), g_mem=z(seq_len, d_m), m_proj=z(seq_len, d_m), m_inj=z(seq_len, d_m))

    def memory_forward(self, x_norm, y_ssm, w_qx, w_qh, w_gate, w_proj, keys, norm_sq, values, seq_len, d_m, d_k, d_val,
                       capacity, count, tau, precision=N.PRECISION_FP32_EXACT, out=None):
        """`GpuDispatch::memory_forward` (src/backend.rs:1342-1385) on host arrays; returns the eight outputs as a dict
        (or fills `out`, a dict of preallocated arrays, which stays untouched on failure)."""
        ins = [x_norm, y_ssm, w_qx, w_qh, w_gate, w_proj, keys, norm_sq, values]
        for name, arr in zip(("x_norm", "y_ssm", "w_qx", "w_qh", "w_gate", "w_proj", "keys", "norm_sq", "values"), ins):
            _host(arr, name)
        o = out or self._memory_outputs(seq_len, d_m, d_k, d_val, capacity)
        self._check(self._lib.pssa_b200_memory_forward(
            self._h, *[_ptr(a) for a in ins], seq_len, d_m, d_k, d_val, capacity, count, tau,
            *[_ptr(o[k]) for k in ("q_euc", "q_pnc", "q_norm", "weights", "m_val", "g_mem", "m_proj", "m_inj")], precision))
        return o

    def ssm_forward_resident(self, delta, b_proj, x_norm, rates, c_proj, initial, seq_len, d_m, d_s, delta_raw=None, exact=False):
        """`GpuDispatch::ssm_forward_resident` (src/backend.rs:1186-1212): results stay on the device."""
        self._check(self._lib.pssa_b200_ssm_forward_resident(
            self._h, _ptr(delta), _ptr(delta_raw), _ptr(b_proj), _ptr(x_norm), _ptr(rates), _ptr(c_proj), _ptr(initial), seq_len,
            d_m, d_s, N.SSM_EXACT if exact else 0))

    def memory_forward_after_ssm(self, x_norm, w_qx, w_qh, w_gate, w_proj, keys, norm_sq, values, seq_len, d_m, d_s, d_k, d_val,
                                 capacity, count, tau, precision=N.PRECISION_FP32_EXACT):
        """`GpuDispatch::memory_forward_after_ssm` (src/backend.rs:1246-1289): publishes the resident SSM tape and runs the
        memory stage on it; returns (tape dict, memory outputs dict)."""
        ins = [x_norm, w_qx, w_qh, w_gate, w_proj, keys, norm_sq, values]
        stride = d_m * d_s
        tape = dict(bar_a=np.zeros((seq_len, stride), np.float32), bar_b=np.zeros((seq_len, stride), np.float32),
                    states=np.zeros((seq_len + 1, stride), np.float32), y_ssm=np.zeros((seq_len, d_m), np.float32))
        o = self._memory_outputs(seq_len, d_m, d_k, d_val, capacity)
        self._check(self._lib.pssa_b200_memory_forward_after_ssm(
            self._h, *[_ptr(a) for a in ins], seq_len, d_m, d_k, d_val, capacity, count, tau,
            *[_ptr(tape[k]) for k in ("bar_a", "bar_b", "states", "y_ssm")],
            *[_ptr(o[k]) for k in ("q_euc", "q_pnc", "q_norm", "weights", "m_val", "g_mem", "m_proj", "m_inj")], precision))
        return tape, o

    # ---- device-side sampling (src/inference.rs:102-181)
    def sample_dev(self, logits, probs, rows, vocab, rng_state, ids_out, status_out, temperature=0.70, top_p=0.85, top_k=24,
                   repetition_penalty=1.25, recent_ids=None, recent_count=None, exact=False, confidence_out=None):
        """One sampled id per stream; all buffers are device buffers (torch tensors or raw pointers)."""
        cfg = N.Sampling(temperature, top_p, top_k, repetition_penalty)
        self._check(self._lib.pssa_b200_sample_dev(self._h, _ptr(logits), _ptr(probs), rows, vocab, C.byref(cfg), _ptr(recent_ids),
                                                   _ptr(recent_count), _ptr(rng_state), _ptr(ids_out), _ptr(status_out),
                                                   _ptr(confidence_out),
                                                   N.SAMPLE_EXACT if exact else 0))

    # ---- bank write / plastic fast weights (device pointers)
    def bank_insert_protected_dev(self, keys, norm_sq, values, confidence, last_seen_step, meta, capacity, d_key, d_val,
                                  key_pnc, val, surprise, step, n, slots_out=None, winning_slots=None, eta=0.0):
        """Ordered protected inserts (`insert_protected`, src/memory.rs:305-342); see include/pssa_b200.h."""
        self._check(self._lib.pssa_b200_bank_insert_protected_dev(
            self._h, _ptr(keys), _ptr(norm_sq), _ptr(values), _ptr(confidence), _ptr(last_seen_step), _ptr(meta), capacity,
            d_key, d_val, _ptr(key_pnc), _ptr(val), _ptr(surprise), _ptr(step), n, _ptr(slots_out), _ptr(winning_slots), eta))

    def adapter_plastic_update_dev(self, up_fast, value, ad_out, ad_act, d, rank):
        self._check(self._lib.pssa_b200_adapter_plastic_update_dev(self._h, _ptr(up_fast), _ptr(value), _ptr(ad_out),
                                                                   _ptr(ad_act), d, rank))

    def adapter_consolidate_dev(self, up_fast, up_slow, n, alpha):
        self._check(self._lib.pssa_b200_adapter_consolidate_dev(self._h, _ptr(up_fast), _ptr(up_slow), n, alpha))

    # ---- dense product
    def dispatch_gemm_into(self, x, w, m, n, k, batch, out, epilogue=N.EPI_NONE, alpha=1.0, precision=N.PRECISION_FP32_EXACT):
        """`GpuDispatch::dispatch_gemm_into` (src/backend.rs:1087-1110): Y[batch,M,N] = X[batch,M,K] * W[N,K]^T on host
        arrays. Lengths are validated before anything runs and `out` is left untouched on failure
        (src/backend.rs:11-38, tests/backend.rs:66-82)."""
        if 0 in (m, n, k, batch):
            raise N.B200Error(N.ERR_SHAPE, "GEMM dimensions must be positive")
        for name, arr in (("x", x), ("w", w), ("out", out)):
            _host(arr, name)
        if x.size != batch * m * k or w.size != n * k:
            raise N.B200Error(N.ERR_SHAPE, f"GEMM operand lengths must be {batch * m * k} and {n * k}, got {x.size} and {w.size}")
        if out.size != batch * m * n:
            raise N.B200Error(N.ERR_SHAPE, "GEMM output length mismatch")
        self._check(self._lib.pssa_b200_gemm_xwt(self._h, _ptr(x), _ptr(w), m, n, k, batch, _ptr(out), epilogue, alpha,
                                                 precision))

    def dispatch_gemm(self, x, w, m, n, k, batch, **kw):  # src/backend.rs:1031-1046
        out = np.empty(batch * m * n, np.float32)
        self.dispatch_gemm_into(x, w, m, n, k, batch, out, **kw)
        return out

    def gemm_xwt_dev(self, x, w, rows, n, k, out, ldo=None, epilogue=N.EPI_NONE, alpha=1.0, precision=N.PRECISION_BF16):
        self._check(self._lib.pssa_b200_gemm_xwt_dev(self._h, _ptr(x), _ptr(w), rows, n, k, _ptr(out), ldo or n, epilogue,
                                                     alpha, precision))

    def profile_begin(self):
        """Start per-kernel device timing (the reference's StageTrace spans, src/training_diagnostics.rs:74-125)."""
        self._check(self._lib.pssa_b200_ctx_profile_begin(self._h))

    def profile_end(self):
        """Stop timing; returns {kernel name: (launches, total ms)}."""
        n = C.c_uint32()
        self._check(self._lib.pssa_b200_ctx_profile_end(self._h, C.byref(n)))
        rows = {}
        for i in range(n.value):
            name, launches, ms = C.c_char_p(), C.c_uint64(), C.c_double()
            self._check(self._lib.pssa_b200_ctx_profile_row(self._h, i, C.byref(name), C.byref(launches), C.byref(ms)))
            rows[name.value.decode()] = (int(launches.value), float(ms.value))
        return rows

    def poll_status(self):
        self._check(self._lib.pssa_b200_ctx_poll_status(self._h))

    def selftest_wait_expiry(self, polls=4096):
        """Enqueue the bounded-wait self-test: a wait that nothing satisfies runs out after `polls` polls and is
        recorded; the next poll_status() raises with status ERR_TIMEOUT, and the context stays usable."""
        self._check(self._lib.pssa_b200_ctx_selftest_wait_expiry(self._h, polls))


class Device:
    """`Device` of src/backend.rs:1012-1018 reduced to the arm this package adds."""

    def __init__(self, dispatch: B200Dispatch):
        self._dispatch = dispatch

    @classmethod
    def try_gpu(cls, device: int = 0) -> "Device":  # src/backend.rs:1467-1481
        return cls(B200Dispatch(device))

    def is_gpu(self) -> bool:
        return True

    def gpu(self) -> B200Dispatch:
        return self._dispatch
