"""ctypes binding of the CPU oracle (oracle/_build/libpssa_oracle.so).

TEST INFRASTRUCTURE ONLY. Imported by tests/, by the smoke entry and by the benchmark's
CPU-baseline leg as the checker / the timed CPU reference. The shipped package never imports it.
"""
import ctypes as C
import pathlib
import subprocess

import numpy as np

_DIR = pathlib.Path(__file__).resolve().parent
_LIB_PATH = _DIR / "_build" / "libpssa_oracle.so"
_lib = None

# tensor ids: same values as `pssa_b200_tensor` in include/pssa_b200.h
EMBED, UNEMBED, NORM_GAMMA, NORM_BETA, A_MAT, W_DELTA, W_B, W_C, W_QX, W_QH, W_GATE, W_PROJ, \
    MLP_W1, MLP_W2, AD_DOWN, AD_UP, AD_CONS, H_PERSISTENT, BANK_KEYS, BANK_VALUES, BANK_NORM_SQ, \
    BANK_CONFIDENCE, RESIDUAL_SCALES = range(23)
S_X_NORM, S_DELTA, S_B, S_C, S_Y_SSM, S_Q_EUC, S_Q_PNC, S_MEM_WEIGHTS, S_M_VAL, S_G_MEM, S_M_PROJ, \
    S_AD_ACT, S_AD_OUT, S_Z_RAW, S_MLP_ACT, S_Z_FINAL, S_FEATURES = range(32, 49)

BLOCK_TENSORS = [NORM_GAMMA, NORM_BETA, A_MAT, W_DELTA, W_B, W_C, W_QX, W_QH, W_GATE, W_PROJ,
                 MLP_W1, MLP_W2, AD_DOWN, AD_UP, AD_CONS]

_fp = C.POINTER(C.c_float)
_u64p = C.POINTER(C.c_uint64)
_u32p = C.POINTER(C.c_uint32)


def build(force: bool = False) -> pathlib.Path:
    """Compile the oracle with the flags its header states."""
    srcs = [_DIR / "pssa_oracle.cpp", _DIR / "oracle_capi.cpp", _DIR / "pssa_oracle.hpp"]
    if force or not _LIB_PATH.exists() or any(s.stat().st_mtime > _LIB_PATH.stat().st_mtime for s in srcs):
        subprocess.run(["make", "-C", str(_DIR), "-B" if force else "-s"], check=True)
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        try:
            build()
        except Exception:
            if not _LIB_PATH.exists():
                raise
        L = C.CDLL(str(_LIB_PATH))
        L.pssa_oracle_model_new.restype = C.c_void_p
        L.pssa_oracle_model_new.argtypes = [_u64p, C.c_float, C.c_uint64]
        L.pssa_oracle_model_load.restype = C.c_void_p
        L.pssa_oracle_model_load.argtypes = [C.c_char_p, C.c_size_t, C.c_char_p, C.c_size_t]
        L.pssa_oracle_model_clone.restype = C.c_void_p
        L.pssa_oracle_model_clone.argtypes = [C.c_void_p]
        L.pssa_oracle_model_free.argtypes = [C.c_void_p]
        L.pssa_oracle_set_loops.argtypes = [C.c_void_p, C.c_size_t]
        L.pssa_oracle_state_len.restype = C.c_size_t
        L.pssa_oracle_state_len.argtypes = [C.c_void_p]
        L.pssa_oracle_copy_state_to.argtypes = [C.c_void_p, _fp]
        L.pssa_oracle_copy_state_from.argtypes = [C.c_void_p, _fp]
        L.pssa_oracle_model_config.argtypes = [C.c_void_p, _u64p, _fp, _u64p]
        L.pssa_oracle_tensor.restype = _fp
        L.pssa_oracle_tensor.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_size_t)]
        L.pssa_oracle_bank_meta.argtypes = [C.c_void_p, C.c_int, _u64p, C.c_int]
        L.pssa_oracle_bank_last_seen.restype = _u64p
        L.pssa_oracle_bank_last_seen.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_size_t)]
        L.pssa_oracle_bank_insert.restype = C.c_size_t
        L.pssa_oracle_bank_insert.argtypes = [C.c_void_p, C.c_int, _fp, _fp]
        L.pssa_oracle_bank_insert_protected.restype = C.c_long
        L.pssa_oracle_bank_insert_protected.argtypes = [C.c_void_p, C.c_int, _fp, _fp, C.c_float, C.c_uint64]
        L.pssa_oracle_reset_state.argtypes = [C.c_void_p]
        L.pssa_oracle_forward_inference.argtypes = [C.c_void_p, C.c_uint64, _fp]
        L.pssa_oracle_forward_features.argtypes = [C.c_void_p, C.c_uint64]
        L.pssa_oracle_prefill.argtypes = [C.c_void_p, _u64p, C.c_size_t, _fp, C.POINTER(C.c_size_t)]
        L.pssa_oracle_chunk_forward.restype = C.c_float
        L.pssa_oracle_chunk_forward.argtypes = [C.c_void_p, _u64p, _u64p, C.c_size_t, _fp]
        L.pssa_oracle_generate_greedy.restype = C.c_long
        L.pssa_oracle_generate_greedy.argtypes = [C.c_void_p, _u64p, C.c_size_t, C.c_size_t, _u64p, _fp]
        L.pssa_oracle_prefill_lanes_timed.restype = C.c_double
        L.pssa_oracle_prefill_lanes_timed.argtypes = [C.c_void_p, _u64p, C.c_size_t, C.c_size_t, C.c_int, _fp]
        L.pssa_oracle_consolidate.argtypes = [C.c_void_p, C.c_int, C.c_float]
        L.pssa_oracle_dream_replay.argtypes = [C.c_void_p, C.c_int, _fp]
        L.pssa_oracle_dot.restype = C.c_float
        L.pssa_oracle_dot.argtypes = [_fp, _fp, C.c_size_t, C.c_int]
        L.pssa_oracle_softplus.restype = C.c_float
        L.pssa_oracle_softplus.argtypes = [C.c_float]
        L.pssa_oracle_sigmoid.restype = C.c_float
        L.pssa_oracle_sigmoid.argtypes = [C.c_float]
        L.pssa_oracle_refractory_gain.restype = C.c_float
        L.pssa_oracle_refractory_gain.argtypes = [C.c_uint64, C.c_float]
        L.pssa_oracle_fnv1a64.restype = C.c_uint64
        L.pssa_oracle_fnv1a64.argtypes = [C.c_char_p, C.c_size_t]
        L.pssa_oracle_rng_fill.argtypes = [C.c_uint64, C.c_float, C.c_float, _fp, C.c_size_t, _u64p]
        L.pssa_oracle_gemm_xwt.argtypes = [_fp, _fp, C.c_size_t, C.c_size_t, C.c_size_t, _fp, C.c_int]
        L.pssa_oracle_affine_scan.argtypes = [_fp, _fp, C.c_size_t, C.c_size_t]
        L.pssa_oracle_scan_states.argtypes = [_fp, _fp, _fp, _fp, C.c_size_t, C.c_size_t, C.c_size_t, C.c_int]
        L.pssa_oracle_ssm_forward.argtypes = [_fp] * 9 + [C.c_size_t] * 3 + [C.c_int]
        L.pssa_oracle_ssm_lanes.argtypes = [_fp] * 7 + [_u32p, _u32p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_int]
        L.pssa_oracle_project.restype = C.c_float
        L.pssa_oracle_project.argtypes = [_fp, _fp, C.c_size_t]
        L.pssa_oracle_squared_norm.restype = C.c_float
        L.pssa_oracle_squared_norm.argtypes = [_fp, C.c_size_t]
        L.pssa_oracle_distance.restype = C.c_float
        L.pssa_oracle_distance.argtypes = [_fp, C.c_float, _fp, C.c_float, C.c_size_t]
        L.pssa_oracle_memory_read.argtypes = [_fp, _fp, _fp, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t,
                                              C.c_size_t, C.c_float, _fp, C.c_int, C.c_size_t, _fp, _fp, _fp,
                                              _fp, C.c_int]
        L.pssa_oracle_bank_new.restype = C.c_void_p
        L.pssa_oracle_bank_new.argtypes = [C.c_size_t] * 3
        L.pssa_oracle_bank_free.argtypes = [C.c_void_p]
        L.pssa_oracle_rawbank_insert.restype = C.c_size_t
        L.pssa_oracle_rawbank_insert.argtypes = [C.c_void_p, _fp, _fp]
        L.pssa_oracle_rawbank_insert_protected.restype = C.c_long
        L.pssa_oracle_rawbank_insert_protected.argtypes = [C.c_void_p, _fp, _fp, C.c_float, C.c_uint64]
        L.pssa_oracle_rawbank_set_top_k.argtypes = [C.c_void_p, C.c_size_t]
        L.pssa_oracle_rawbank_retrieve.restype = C.c_float
        L.pssa_oracle_rawbank_retrieve.argtypes = [C.c_void_p, _fp, C.c_float, _fp, _fp, C.c_size_t]
        L.pssa_oracle_rawbank_array.restype = _fp
        L.pssa_oracle_rawbank_array.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_size_t)]
        L.pssa_oracle_rawbank_meta.argtypes = [C.c_void_p, _u64p, _u64p]
        L.pssa_oracle_rawbank_set_meta.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, _fp, _u64p]
        L.pssa_oracle_rawbank_plastic_write.restype = C.c_long
        L.pssa_oracle_rawbank_plastic_write.argtypes = [C.c_void_p, C.c_size_t, _fp, C.c_float, C.c_uint64, C.c_float]
        L.pssa_oracle_greedy.restype = C.c_long
        L.pssa_oracle_greedy.argtypes = [_fp, C.c_size_t]
        L.pssa_oracle_sample.restype = C.c_long
        L.pssa_oracle_sample.argtypes = [C.POINTER(C.c_uint64), C.c_float, C.c_float, C.c_size_t, C.c_float,
                                         C.POINTER(C.c_uint64), C.c_size_t, _fp, C.c_size_t]
        L.pssa_oracle_hardware_threads.restype = C.c_int
        _lib = L
    return _lib


def fptr(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_fp)


def u64ptr(a: np.ndarray):
    assert a.dtype == np.uint64 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_u64p)


def u32ptr(a: np.ndarray):
    assert a.dtype == np.uint32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_u32p)


class Model:
    """Reference-shaped model (`PSSALayerV2`, src/pssa.rs:1931-2075) evaluated by the oracle."""

    def __init__(self, handle):
        if not handle:
            raise RuntimeError("oracle model handle is null")
        self.h = C.c_void_p(handle)
        dims = (C.c_uint64 * 7)()
        tau = C.c_float()
        sr = (C.c_uint64 * 2)()
        lib().pssa_oracle_model_config(self.h, dims, C.byref(tau), sr)
        (self.depth, self.d_vocab, self.d_latent, self.d_state, self.d_mem_key, self.mem_capacity,
         self.chunk_len) = [int(x) for x in dims]
        self.tau_mem = float(tau.value)
        self.step_counter, self.rng_state = int(sr[0]), int(sr[1])

    @classmethod
    def new(cls, depth, d_vocab, d_latent, d_state, d_mem_key, mem_capacity, chunk_len=64, tau_mem=0.1, seed=1):
        dims = (C.c_uint64 * 7)(depth, d_vocab, d_latent, d_state, d_mem_key, mem_capacity, chunk_len)
        return cls(lib().pssa_oracle_model_new(dims, tau_mem, seed))

    @classmethod
    def load(cls, data: bytes):
        err = C.create_string_buffer(256)
        h = lib().pssa_oracle_model_load(data, len(data), err, 256)
        if not h:
            raise ValueError("invalid checkpoint: " + err.value.decode())
        return cls(h)

    def clone(self):
        return Model(lib().pssa_oracle_model_clone(self.h))

    def __del__(self):
        try:
            lib().pssa_oracle_model_free(self.h)
        except Exception:
            pass

    def tensor(self, layer: int, tid: int) -> np.ndarray:
        """Writable numpy view of a parameter / carry / scratch vector owned by the oracle."""
        n = C.c_size_t()
        p = lib().pssa_oracle_tensor(self.h, layer, tid, C.byref(n))
        if not p and n.value == 0:
            if tid == RESIDUAL_SCALES:
                return np.zeros(0, np.float32)
            raise KeyError((layer, tid))
        return np.ctypeslib.as_array(p, shape=(n.value,))

    def bank_meta(self, layer: int):
        meta = (C.c_uint64 * 3)()
        lib().pssa_oracle_bank_meta(self.h, layer, meta, 0)
        return int(meta[0]), int(meta[1]), int(meta[2])

    def set_bank_meta(self, layer: int, count: int, write_head: int, top_k: int = 0):
        meta = (C.c_uint64 * 3)(count, write_head, top_k)
        lib().pssa_oracle_bank_meta(self.h, layer, meta, 1)

    def bank_last_seen(self, layer: int) -> np.ndarray:
        n = C.c_size_t()
        p = lib().pssa_oracle_bank_last_seen(self.h, layer, C.byref(n))
        return np.ctypeslib.as_array(p, shape=(n.value,))

    def bank_insert(self, layer, key, val) -> int:
        key = np.ascontiguousarray(key, np.float32)
        val = np.ascontiguousarray(val, np.float32)
        return int(lib().pssa_oracle_bank_insert(self.h, layer, fptr(key), fptr(val)))

    def bank_insert_protected(self, layer, key, val, surprise, step) -> int:
        """`insert_protected_with_device` (src/memory.rs:315-342): the slot written, or -1 when the slot defended itself."""
        key = np.ascontiguousarray(key, np.float32)
        val = np.ascontiguousarray(val, np.float32)
        return int(lib().pssa_oracle_bank_insert_protected(self.h, layer, fptr(key), fptr(val), surprise, step))

    def reset_recurrent_state(self):
        lib().pssa_oracle_reset_state(self.h)

    def forward_inference(self, token: int) -> np.ndarray:
        out = np.empty(self.d_vocab, np.float32)
        if lib().pssa_oracle_forward_inference(self.h, token, fptr(out)) != 0:
            raise ValueError("token ID must be in vocabulary")
        return out

    def forward_features(self, token: int) -> np.ndarray:
        if lib().pssa_oracle_forward_features(self.h, token) != 0:
            raise ValueError("token ID must be in vocabulary")
        return self.tensor(-1, S_FEATURES).copy()

    def prefill_inference(self, ids, want_logits=True):
        ids = np.ascontiguousarray(ids, np.uint64)
        out = np.empty(self.d_vocab, np.float32) if want_logits else None
        done = C.c_size_t()
        rc = lib().pssa_oracle_prefill(self.h, u64ptr(ids), len(ids), fptr(out) if want_logits else None,
                                       C.byref(done))
        return rc, int(done.value), out

    def chunk_forward(self, ids, targets):
        ids = np.ascontiguousarray(ids, np.uint64)
        targets = np.ascontiguousarray(targets, np.uint64)
        logits = np.empty((len(ids), self.d_vocab), np.float32)
        loss = lib().pssa_oracle_chunk_forward(self.h, u64ptr(ids), u64ptr(targets), len(ids), fptr(logits))
        return float(np.float32(loss)), logits

    def generate_greedy(self, ids, n_new):
        ids = np.ascontiguousarray(ids, np.uint64)
        out = np.empty(n_new, np.uint64)
        gap = C.c_float()
        rc = lib().pssa_oracle_generate_greedy(self.h, u64ptr(ids), len(ids), n_new, u64ptr(out), C.byref(gap))
        if rc < 0:
            raise RuntimeError("oracle generation failed")
        return out, float(gap.value)

    def prefill_lanes_timed(self, ids, threads):
        """Token-serial prefill of independent lanes ids [n, T] on `threads` host threads; returns (seconds, logits)."""
        ids = np.ascontiguousarray(ids, np.uint64)
        n, T = ids.shape
        logits = np.empty((n, self.d_vocab), np.float32)
        sec = lib().pssa_oracle_prefill_lanes_timed(self.h, u64ptr(ids), n, T, threads, fptr(logits))
        return float(sec), logits

    def set_loops(self, loops: int):
        """Runtime Ouro pass count (pssa.rs:2171-2184); passes >= 1 start from zero carries."""
        if lib().pssa_oracle_set_loops(self.h, loops) != 0:
            raise ValueError("--loops must be between 1 and 32; use --loops 1 for the original model")

    def state(self) -> np.ndarray:
        """Recurrent carry in the reference's `[block][pass][d*s]` order (pssa.rs:2263-2310)."""
        out = np.empty(lib().pssa_oracle_state_len(self.h), np.float32)
        lib().pssa_oracle_copy_state_to(self.h, fptr(out))
        return out

    def set_state(self, flat: np.ndarray):
        flat = np.ascontiguousarray(flat, np.float32)
        assert flat.size == lib().pssa_oracle_state_len(self.h)
        lib().pssa_oracle_copy_state_from(self.h, fptr(flat))


def rng_fill(seed: int, low: float, high: float, n: int) -> np.ndarray:
    """`SimpleRng::gen_range_f32` stream (src/linalg.rs:1-28)."""
    out = np.empty(n, np.float32)
    lib().pssa_oracle_rng_fill(seed, low, high, fptr(out), n, None)
    return out


def scan_states(a, b, h0=None, threads=1):
    """h_t = a_t*h_{t-1} + b_t, ordered (mul then add), for [lanes, T, stride] inputs."""
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    lanes, T, stride = a.shape
    out = np.empty_like(a)
    h0p = fptr(np.ascontiguousarray(h0, np.float32)) if h0 is not None else None
    lib().pssa_oracle_scan_states(fptr(a), fptr(b), h0p, fptr(out), lanes, T, stride, threads)
    return out


def affine_scan_exclusive(a, b):
    """Blelloch exclusive prefix of affine maps (src/gpu_batch.rs:98-164) for [T, stride] arrays."""
    T, stride = a.shape
    width = 1 << max(0, (T - 1).bit_length())
    pa = np.zeros((width, stride), np.float32)
    pb = np.zeros((width, stride), np.float32)
    pa[:T] = a
    pb[:T] = b
    lib().pssa_oracle_affine_scan(fptr(pa), fptr(pb), T, stride)
    return pa[:T].copy(), pb[:T].copy()


def ssm_forward(delta, b_proj, c_proj, x_norm, rates, h0, mode=0):
    """One lane of the SSM stage; returns (states[(T+1), d*s], y[T, d], bar_a, bar_b)."""
    T, d = delta.shape
    s = b_proj.shape[1]
    states = np.zeros((T + 1, d * s), np.float32)
    states[0] = h0
    y = np.empty((T, d), np.float32)
    bar_a = np.empty((T, d * s), np.float32)
    bar_b = np.empty((T, d * s), np.float32)
    args = [np.ascontiguousarray(x, np.float32) for x in (delta, b_proj, c_proj, x_norm, rates)]
    lib().pssa_oracle_ssm_forward(*[fptr(x) for x in args], fptr(states), fptr(y), fptr(bar_a), fptr(bar_b),
                                  T, d, s, mode)
    return states, y, bar_a, bar_b


def ssm_lanes(delta, b_proj, c_proj, x_norm, rates, carry, offsets, lengths, threads=1):
    """Packed lanes: rows [sum(len), d]; carry [lanes, d*s] updated in place; returns y."""
    n, d = delta.shape
    s = b_proj.shape[1]
    y = np.zeros((n, d), np.float32)
    args = [np.ascontiguousarray(x, np.float32) for x in (delta, b_proj, c_proj, x_norm, rates)]
    offsets = np.ascontiguousarray(offsets, np.uint32)
    lengths = np.ascontiguousarray(lengths, np.uint32)
    assert carry.dtype == np.float32 and carry.flags["C_CONTIGUOUS"]
    lib().pssa_oracle_ssm_lanes(*[fptr(x) for x in args], fptr(carry), fptr(y), u32ptr(offsets), u32ptr(lengths),
                                len(lengths), d, s, threads)
    return y


def memory_read(keys, norm_sq, values, count, q, tau, top_k=0, q_is_euclidean=False, threads=1):
    """Bank read for n queries (src/memory.rs:344-426). Returns (q_pnc, m_val, weights, min_dist)."""
    keys = np.ascontiguousarray(keys, np.float32)
    values = np.ascontiguousarray(values, np.float32)
    norm_sq = np.ascontiguousarray(norm_sq, np.float32)
    q = np.ascontiguousarray(q, np.float32)
    cap, dk = keys.shape
    dv = values.shape[1]
    n = q.shape[0]
    q_pnc = np.empty((n, dk), np.float32)
    m_val = np.empty((n, dv), np.float32)
    weights = np.empty((n, cap), np.float32)
    md = np.empty(n, np.float32)
    lib().pssa_oracle_memory_read(fptr(keys), fptr(norm_sq), fptr(values), cap, count, dk, dv, top_k, tau,
                                  fptr(q), 1 if q_is_euclidean else 0, n, fptr(q_pnc), fptr(m_val),
                                  fptr(weights), fptr(md), threads)
    return q_pnc, m_val, weights, md


def gemm_xwt(x, w, threads=1):
    """Y = X * W^T with every entry one `dot_slice` (src/backend.rs:832-871)."""
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    m, k = x.shape
    n = w.shape[0]
    out = np.empty((m, n), np.float32)
    lib().pssa_oracle_gemm_xwt(fptr(x), fptr(w), m, n, k, fptr(out), threads)
    return out


class RawBank:
    """Standalone `HyperbolicEpisodicBankV2` (src/memory.rs) for the write/read known-answer tests."""

    def __init__(self, cap, dk, dv):
        self.cap, self.dk, self.dv = cap, dk, dv
        self.h = C.c_void_p(lib().pssa_oracle_bank_new(cap, dk, dv))

    def __del__(self):
        try:
            lib().pssa_oracle_bank_free(self.h)
        except Exception:
            pass

    def insert(self, key, val):
        return int(lib().pssa_oracle_rawbank_insert(self.h, fptr(np.asarray(key, np.float32)),
                                                    fptr(np.asarray(val, np.float32))))

    def insert_protected(self, key, val, surprise, step):
        r = lib().pssa_oracle_rawbank_insert_protected(self.h, fptr(np.asarray(key, np.float32)),
                                                       fptr(np.asarray(val, np.float32)), surprise, step)
        return None if r < 0 else int(r)

    def plastic_write(self, slot, val, surprise, step, eta):
        """Winning-slot rank-1 write of the retrieval benchmark configuration (restatement only, not in the reference)."""
        r = lib().pssa_oracle_rawbank_plastic_write(self.h, slot, fptr(np.asarray(val, np.float32)), surprise, step, eta)
        return None if r < 0 else int(r)

    def set_top_k(self, k):
        lib().pssa_oracle_rawbank_set_top_k(self.h, k or 0)

    def retrieve(self, q, tau):
        out = np.full(self.dv, 9.0, np.float32)
        w = np.full(self.cap, 9.0, np.float32)
        md = lib().pssa_oracle_rawbank_retrieve(self.h, fptr(np.asarray(q, np.float32)), tau, fptr(out), fptr(w),
                                                self.cap)
        return out, w, float(md)

    def array(self, which):
        n = C.c_size_t()
        p = lib().pssa_oracle_rawbank_array(self.h, which, C.byref(n))
        return np.ctypeslib.as_array(p, shape=(n.value,))

    def meta(self):
        meta = (C.c_uint64 * 2)()
        ls = np.zeros(self.cap, np.uint64)
        lib().pssa_oracle_rawbank_meta(self.h, meta, u64ptr(ls))
        return int(meta[0]), int(meta[1]), ls

    def set_meta(self, count, head, conf, last_seen):
        lib().pssa_oracle_rawbank_set_meta(self.h, count, head, fptr(np.asarray(conf, np.float32)),
                                           u64ptr(np.asarray(last_seen, np.uint64)))


def sample(rng_state: int, logits, generated, temperature=0.8, top_p=0.95, top_k=40, repetition_penalty=1.1):
    """`sample` (src/inference.rs:102-181). Returns (id or negative error, new rng state, logits after the penalty)."""
    lg = np.ascontiguousarray(logits, np.float32).copy()
    gen = np.ascontiguousarray(generated, np.uint64)
    st = C.c_uint64(rng_state)
    tok = lib().pssa_oracle_sample(C.byref(st), temperature, top_p, top_k, repetition_penalty, u64ptr(gen), len(gen), fptr(lg),
                                   lg.size)
    return int(tok), int(st.value), lg
