"""Host-side mirror of the reference's model-level inference API (`PSSALayerV2`, src/pssa.rs:2245-2442) on top of
the C ABI's device-resident model. Weights, banks and carries live on the GPU; token ids go in, logits come out."""
import ctypes as C

import numpy as np

from . import _native as N
from .dispatch import B200Dispatch, _ptr

# tensor ids of include/pssa_b200.h
EMBED, UNEMBED, NORM_GAMMA, NORM_BETA, A_MAT, W_DELTA, W_B, W_C, W_QX, W_QH, W_GATE, W_PROJ, MLP_W1, MLP_W2, AD_DOWN, \
    AD_UP, AD_CONS = range(17)
RESIDUAL_SCALES = 22
BLOCK_TENSORS = (NORM_GAMMA, NORM_BETA, A_MAT, W_DELTA, W_B, W_C, W_QX, W_QH, W_GATE, W_PROJ, MLP_W1, MLP_W2, AD_DOWN,
                 AD_UP, AD_CONS)


class PSSAModel:
    """One model on one B200. `streams` independent recurrent carries (lanes) share the weights and banks."""

    def __init__(self, gpu: B200Dispatch, depth, d_vocab, d_latent, d_state, d_mem_key, mem_capacity, tau_mem=0.1,
                 streams=1, precision=N.PRECISION_BF16):
        self.gpu = gpu
        self._lib = gpu._lib
        self.depth, self.d_vocab, self.d_latent, self.d_state = depth, d_vocab, d_latent, d_state
        self.d_mem_key, self.mem_capacity, self.tau_mem, self.streams = d_mem_key, mem_capacity, tau_mem, streams
        cfg = N.Config(depth, d_vocab, d_latent, d_state, d_mem_key, mem_capacity, tau_mem, 0)
        h = C.c_void_p()
        gpu._check(self._lib.pssa_b200_model_create(gpu._h, C.byref(cfg), streams, C.byref(h)))
        self._h = h
        gpu._adopt(self)
        self.set_precision(precision)

    @staticmethod
    def probe_checkpoint(data: bytes):
        """Host-only validation of a `.pssa` container: returns (config dict, version); raises ValueError otherwise."""
        cfg, ver, err = N.Config(), C.c_uint32(), C.create_string_buffer(256)
        if N.lib().pssa_b200_checkpoint_probe(data, len(data), C.byref(cfg), C.byref(ver), err, 256) != N.OK:
            raise ValueError("invalid checkpoint: " + err.value.decode())
        return ({f: getattr(cfg, f) for f, _ in cfg._fields_ if f != "reserved"}, int(ver.value))

    @classmethod
    def from_checkpoint(cls, gpu: B200Dispatch, data: bytes, streams=1, precision=N.PRECISION_BF16):
        """`load_checkpoint` (src/checkpoint.rs:1344-1411) into a device-resident model; stream 0 gets the stored carry."""
        cfg, _ = cls.probe_checkpoint(data)
        self = cls.__new__(cls)
        self.gpu, self._lib = gpu, gpu._lib
        self.depth, self.d_vocab, self.d_latent, self.d_state = cfg["depth"], cfg["d_vocab"], cfg["d_latent"], cfg["d_state"]
        self.d_mem_key, self.mem_capacity, self.tau_mem, self.streams = cfg["d_mem_key"], cfg["mem_capacity"], cfg["tau_mem"], streams
        h = C.c_void_p()
        gpu._check(self._lib.pssa_b200_model_load_checkpoint(gpu._h, data, len(data), streams, C.byref(h)))
        self._h = h
        gpu._adopt(self)
        self.set_precision(precision)
        return self

    def close(self):
        if getattr(self, "_h", None):
            if getattr(self.gpu, "_h", None):  # a model never outlives its context
                self._lib.pssa_b200_model_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- upload
    def set_tensor(self, layer: int, tensor: int, data):
        a = np.ascontiguousarray(data, np.float32).ravel()
        self.gpu._check(self._lib.pssa_b200_model_set_tensor(self._h, layer, tensor, _ptr(a), a.size))

    def reserve(self, rows: int, lanes: int):
        """Allocate now what calls of at most `rows` rows over `lanes` lanes would allocate on first use."""
        self.gpu._check(self._lib.pssa_b200_model_reserve(self._h, rows, lanes))

    def get_tensor(self, layer: int, tensor: int, length: int):
        out = np.empty(length, np.float32)
        self.gpu._check(self._lib.pssa_b200_model_get_tensor(self._h, layer, tensor, _ptr(out), out.size))
        return out

    def init_random(self, seed: int) -> int:
        """`PSSALayerV2::new(cfg, seed)`'s tensors (src/pssa.rs:2019-2072); returns the generator state after the last draw."""
        state = C.c_uint64()
        self.gpu._check(self._lib.pssa_b200_model_init_random(self._h, seed, C.byref(state)))
        return int(state.value)

    def set_bank(self, layer, keys, norm_sq, values, count, write_head=0, confidence=None, last_seen_step=None):
        keys = np.ascontiguousarray(keys, np.float32)
        norm_sq = np.ascontiguousarray(norm_sq, np.float32)
        values = np.ascontiguousarray(values, np.float32)
        if keys.size != self.mem_capacity * self.d_mem_key or values.size != self.mem_capacity * self.d_latent or \
                norm_sq.size != self.mem_capacity:
            raise N.B200Error(N.ERR_SHAPE, "memory bank arrays do not match the configured capacity and widths")
        conf = None if confidence is None else np.ascontiguousarray(confidence, np.float32)
        seen = None if last_seen_step is None else np.ascontiguousarray(last_seen_step, np.uint64)
        self.gpu._check(self._lib.pssa_b200_model_set_bank(self._h, layer, _ptr(keys), _ptr(norm_sq), _ptr(values), count,
                                                           write_head, _ptr(conf), _ptr(seen)))

    # ---- runtime options (src/pssa.rs:2080-2243)
    def set_memory_top_k(self, top_k):
        if top_k == 0:
            raise N.B200Error(N.ERR_INVALID_ARGUMENT, "memory top-k must be positive")
        self.gpu._check(self._lib.pssa_b200_model_set_top_k(self._h, top_k or 0))

    def set_precision(self, precision):
        self.gpu._check(self._lib.pssa_b200_model_set_precision(self._h, precision))

    def set_local_conv(self, enabled):
        self.gpu._check(self._lib.pssa_b200_model_set_option(self._h, 0, int(enabled)))

    def set_ssm_skip(self, enabled):
        self.gpu._check(self._lib.pssa_b200_model_set_option(self._h, 1, int(enabled)))

    def set_hybrid_read(self, enabled, lam=1.0):
        if not (np.isfinite(lam) and 0.0 < lam <= 1.0):
            raise N.B200Error(N.ERR_INVALID_ARGUMENT, "hybrid decay lam must be in (0.0, 1.0]")
        self.gpu._check(self._lib.pssa_b200_model_set_option(self._h, 2, int(enabled)))

    def grow_memory(self, capacity):
        self.gpu._check(self._lib.pssa_b200_model_set_option(self._h, 3, int(capacity)))

    def set_loops(self, loops):
        if not 1 <= loops <= 32:
            raise N.B200Error(N.ERR_INVALID_ARGUMENT, "--loops must be between 1 and 32; use --loops 1 for the original model")
        self.gpu._check(self._lib.pssa_b200_model_set_option(self._h, 4, int(loops)))
        self.loops = int(loops)

    def set_lane_groups(self, groups):
        """Lane groups on side streams per pass: 0 = chosen from the shape, 1 = off, 2..4 = that many groups."""
        self.gpu._check(self._lib.pssa_b200_model_set_option(self._h, 5, int(groups)))

    def set_max_rows(self, rows):
        self.gpu._check(self._lib.pssa_b200_model_set_max_rows(self._h, rows))

    # ---- recurrent state (src/pssa.rs:2245-2310)
    def recurrent_state_len(self):
        return self.depth * getattr(self, "loops", 1) * self.d_latent * self.d_state

    def reset_recurrent_state(self, stream=None):
        for s in (range(self.streams) if stream is None else [stream]):
            self.gpu._check(self._lib.pssa_b200_model_reset_state(self._h, s))

    def copy_recurrent_state_to(self, stream=0):
        out = np.empty(self.recurrent_state_len(), np.float32)
        self.gpu._check(self._lib.pssa_b200_model_get_state(self._h, stream, _ptr(out), out.size))
        return out

    def copy_recurrent_state_from(self, state, stream=0):
        a = np.ascontiguousarray(state, np.float32)
        self.gpu._check(self._lib.pssa_b200_model_set_state(self._h, stream, _ptr(a), a.size))

    # ---- forward
    def forward_inference(self, x_id: int, stream=0):
        """`forward_inference` (src/pssa.rs:2387-2391): one token, returns logits [V]. A bad id raises, as the
        reference panics (src/pssa.rs:2317)."""
        return self.decode_step([x_id], [stream])[0]

    def prefill_inference(self, token_ids, want_logits=True, cancelled=None, stream=0):
        """`prefill_inference` (src/pssa.rs:2399-2442). Returns (completed, logits or None). Raises B200Error for an
        empty prompt or an id outside the vocabulary (after the valid prefix has advanced the carry)."""
        ids = np.ascontiguousarray(token_ids, np.uint64)
        logits = np.empty(self.d_vocab, np.float32) if want_logits else None
        done = C.c_size_t()
        cb = N.CANCEL_FN(lambda _arg: 1 if cancelled() else 0) if cancelled else None
        rc = self._lib.pssa_b200_model_prefill(self._h, stream, _ptr(ids) if ids.size else None, ids.size, _ptr(logits),
                                               C.byref(done), cb, None)
        self.processed = int(done.value)
        if rc == N.ERR_CANCELLED:
            return False, None
        self.gpu._check(rc)
        return True, logits

    def prefill_batch(self, lanes, streams=None, want_logits=True, want_greedy=False):
        """Independent sequences (`SequenceBatch::forward`, src/sequence_batch.rs:233-384): `lanes` is a list of id
        sequences; lane l continues stream streams[l] (default l). Returns (logits [n, V] or None, greedy ids or None)."""
        lengths = np.array([len(x) for x in lanes], np.uint32)
        offsets = np.concatenate([[0], np.cumsum(lengths)[:-1]]).astype(np.uint32)
        ids = np.ascontiguousarray(np.concatenate([np.asarray(x, np.uint64) for x in lanes]) if lengths.sum() else
                                   np.zeros(1, np.uint64), np.uint64)
        st = None if streams is None else np.ascontiguousarray(streams, np.uint32)
        logits = np.zeros((len(lanes), self.d_vocab), np.float32) if want_logits else None
        greedy = np.zeros(len(lanes), np.uint64) if want_greedy else None
        self.gpu._check(self._lib.pssa_b200_model_prefill_batch(self._h, _ptr(ids), _ptr(offsets), _ptr(lengths), _ptr(st),
                                                                len(lanes), _ptr(logits), _ptr(greedy)))
        return logits, greedy

    def prefill_batch_dev(self, ids_dev, offsets, lengths, streams=None, logits_dev=None, greedy_dev=None):
        """Device-resident form: `ids_dev` (uint32), `logits_dev` [n, V] fp32 and `greedy_dev` [n] uint32 are device
        buffers (torch tensors or raw pointers); offsets / lengths / streams are host arrays. Only enqueues work."""
        offsets = np.ascontiguousarray(offsets, np.uint32)
        lengths = np.ascontiguousarray(lengths, np.uint32)
        st = None if streams is None else np.ascontiguousarray(streams, np.uint32)
        self.gpu._check(self._lib.pssa_b200_model_prefill_batch_dev(self._h, _ptr(ids_dev), _ptr(offsets), _ptr(lengths),
                                                                    _ptr(st), len(lengths), _ptr(logits_dev), _ptr(greedy_dev)))

    def capture_greedy_decode_graph(self, ids_dev, streams=None):
        """One greedy decode step for len(ids_dev) streams as a CUDA graph (torch.cuda.CUDAGraph).

        `ids_dev` (int32 device tensor, one token per stream) is both the step's input and its output: every replay
        feeds the ids of the previous one, so a generation loop is `graph.replay()` per token with no host round trip.
        Works because the device-resident entry point only launches kernels and device-to-device copies once the lane
        layout is on the device. The capture takes ONE real step first (it uploads the layout and sizes every buffer),
        so on return ids and states have advanced by one token; the context's stream is switched to a capture stream for
        the duration of the call.
        """
        import torch
        n = int(ids_dev.numel())
        offsets = np.arange(n, dtype=np.uint32)
        lengths = np.ones(n, dtype=np.uint32)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        self.gpu.set_stream(side)
        try:
            with torch.cuda.stream(side):
                self.prefill_batch_dev(ids_dev, offsets, lengths, streams, None, ids_dev)
                side.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side, capture_error_mode="relaxed"):
                    self.prefill_batch_dev(ids_dev, offsets, lengths, streams, None, ids_dev)
        finally:
            side.synchronize()
            self.gpu.set_stream(torch.cuda.current_stream())
        return graph

    def decode_step(self, ids, streams=None, want_logits=True, want_greedy=False):
        ids = np.ascontiguousarray(ids, np.uint64)
        st = None if streams is None else np.ascontiguousarray(streams, np.uint32)
        logits = np.empty((ids.size, self.d_vocab), np.float32) if want_logits else None
        greedy = np.empty(ids.size, np.uint64) if want_greedy else None
        self.gpu._check(self._lib.pssa_b200_model_decode_step(self._h, _ptr(st), _ptr(ids), ids.size, _ptr(logits),
                                                              _ptr(greedy)))
        if want_logits and want_greedy:
            return logits, greedy
        return logits if want_logits else greedy

    def score(self, ids, targets, stream=0, want_logits=False):
        """Mean next-token cross entropy of a frozen model over `ids` (the forward half of the chunk forward,
        src/pssa.rs:2597-2750). Returns (mean loss, per-token losses[, logits [n, vocab]])."""
        ids = np.ascontiguousarray(ids, np.uint64)
        targets = np.ascontiguousarray(targets, np.uint64)
        mean = C.c_float()
        per = np.empty(ids.size, np.float32)
        logits = np.empty((ids.size, self.d_vocab), np.float32) if want_logits else None
        self.gpu._check(self._lib.pssa_b200_model_score(self._h, stream, _ptr(ids), _ptr(targets), ids.size, C.byref(mean), _ptr(per),
                                                        _ptr(logits)))
        return (float(mean.value), per, logits) if want_logits else (float(mean.value), per)

    def set_observer(self, enabled=True):
        """Publish each block's retrieval scratch of the last token of every lane (src/pssa.rs:609-619)."""
        self.gpu._check(self._lib.pssa_b200_model_set_observer(self._h, 1 if enabled else 0))

    def observation(self, layer, index=0):
        """(mem_weights [cap], q_pnc [k], m_val [d], z_final [d]) of block `layer` for emitting lane `index`."""
        w = np.empty(self.mem_capacity, np.float32)
        q = np.empty(self.d_mem_key, np.float32)
        mv = np.empty(self.d_latent, np.float32)
        z = np.empty(self.d_latent, np.float32)
        self.gpu._check(self._lib.pssa_b200_model_get_observation(self._h, layer, index, _ptr(w), _ptr(q), _ptr(mv), _ptr(z)))
        return w, q, mv, z

    def sampler_seed(self, stream=0, seed=1337):
        """Reset a stream's generator and its window of generated ids (`SimpleRng::new(seed)`, src/linalg.rs:7-11)."""
        self.gpu._check(self._lib.pssa_b200_model_sampler_seed(self._h, stream, seed))

    def decode_step_sampled(self, ids, streams=None, temperature=0.70, top_p=0.85, top_k=24, repetition_penalty=1.25, exact=False,
                            want_confidence=False):
        """Decode step with `sample` (src/inference.rs:102-181) on the device; returns the sampled ids (and, if asked,
        the raw softmax probability of each: `raw_confidence`, src/inference.rs:526-545)."""
        ids = np.ascontiguousarray(ids, np.uint64)
        st = None if streams is None else np.ascontiguousarray(streams, np.uint32)
        out = np.empty(ids.size, np.uint64)
        cfg = N.Sampling(temperature, top_p, top_k, repetition_penalty)
        conf = np.empty(ids.size, np.float32) if want_confidence else None
        self.gpu._check(self._lib.pssa_b200_model_decode_step_sampled(self._h, _ptr(st), _ptr(ids), ids.size, C.byref(cfg),
                                                                      N.SAMPLE_EXACT if exact else 0, _ptr(out), _ptr(conf)))
        return (out, conf) if want_confidence else out

    def insert_memory(self, loss: float, step: int, index=0):
        """`insert_training_memory_at` (src/pssa.rs:3705-3737) with the last observed token of lane `index`; returns the
        per-block slots (written slot, -1 defended, -2 refused, -3 loss not above 3.5)."""
        slots = np.empty(self.depth, np.int64)
        self.gpu._check(self._lib.pssa_b200_model_insert_memory(self._h, index, loss, step, _ptr(slots)))
        return slots

    def sampler_push(self, ids, stream=0):
        """Append ids (the prompt) to a stream's repetition window (`generated_ids` starts as the prompt, src/inference.rs:343-345)."""
        ids = np.ascontiguousarray(ids, np.uint64)
        self.gpu._check(self._lib.pssa_b200_model_sampler_push(self._h, stream, _ptr(ids), ids.size))

    def generate(self, prompt_ids, max_new_tokens=50, temperature=0.70, top_p=0.85, top_k=24, repetition_penalty=1.25, seed=1337,
                 stream=0, cancelled=None, on_token=None, scored=False, exact=False):
        """The id-level loop of `PSSAInferenceEngine::try_generate_chat_turn_impl` (src/inference.rs:317-418; tokenizer and
        text assembly stay with the caller): reset the carry, seed the generator, the prompt becomes the head of the
        repetition window, prefill, then `max_new_tokens` steps of forward + `sample` on the device. The first sampled
        token comes from the logits of the last prompt token, which is run as the first sampled step (prefill == token
        loop, src/inference.rs:1069-1113). `cancelled()` is polled before the prompt and before every step and returns
        what was generated so far; `on_token(count, previous_id, selected_id, probability)` follows the reference's
        callback / observer order. Returns (ids, raw probabilities or None)."""
        prompt = np.ascontiguousarray(prompt_ids, np.uint64)
        if prompt.size == 0:
            raise ValueError("prompt is empty after tokenization")  # src/inference.rs:333-335
        if cancelled is not None and cancelled():
            return np.zeros(0, np.uint64), (np.zeros(0, np.float32) if scored else None)
        self.reset_recurrent_state(stream)
        self.sampler_seed(stream, seed)
        self.sampler_push(prompt, stream)
        if prompt.size > 1:
            ok, _ = self.prefill_inference(prompt[:-1], want_logits=False, cancelled=cancelled, stream=stream)
            if not ok:
                return np.zeros(0, np.uint64), (np.zeros(0, np.float32) if scored else None)
        out, probs, tok = [], [], int(prompt[-1])
        for step in range(max_new_tokens):
            if cancelled is not None and cancelled():
                break
            got = self.decode_step_sampled([tok], [stream], temperature, top_p, top_k, repetition_penalty, exact=exact,
                                           want_confidence=scored)
            nxt, p = (int(got[0][0]), float(got[1][0])) if scored else (int(got[0]), 0.0)
            if on_token is not None:
                on_token(step + 1, tok, nxt, p)
            out.append(nxt), probs.append(p)
            tok = nxt
        return np.array(out, np.uint64), (np.array(probs, np.float32) if scored else None)

    def generate_greedy(self, prompt_ids, n_new, stream=0):
        """Prefill + greedy decode (src/inference.rs:348-418 at temperature 0): returns the generated ids."""
        _, g = self.prefill_batch([prompt_ids], [stream], want_logits=False, want_greedy=True)
        out = [int(g[0])]
        for _ in range(n_new - 1):
            g = self.decode_step([out[-1]], [stream], want_logits=False, want_greedy=True)
            out.append(int(g[0]))
        return np.array(out, np.uint64)
