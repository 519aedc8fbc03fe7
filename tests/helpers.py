"""Test helpers: copy an oracle model onto the GPU model, synthetic model fills."""
import numpy as np

import oracle as O


def fill_synthetic(m: "O.Model", seed: int, bank_fill: float = 1.0, std: float = 0.02):
    """Give every matrix (including the zero-initialised MLP W2 and adapter up weights) seeded values, decays
    exp(A) ~ U(0.9, 0.999), and fill the bank with keys inside the ball (radius < 0.9) and N(0,1) values."""
    rng = np.random.default_rng(seed)
    d, s, k, cap = m.d_latent, m.d_state, m.d_mem_key, m.mem_capacity
    for tid in (O.EMBED, O.UNEMBED):
        t = m.tensor(-1, tid)
        t[:] = rng.normal(0, std, t.size).astype(np.float32)
    for l in range(m.depth):
        for tid in (O.W_DELTA, O.W_B, O.W_C, O.W_QX, O.W_QH, O.W_GATE, O.W_PROJ, O.MLP_W1, O.MLP_W2, O.AD_DOWN, O.AD_UP,
                    O.AD_CONS):
            t = m.tensor(l, tid)
            t[:] = rng.normal(0, std, t.size).astype(np.float32)
        u = rng.uniform(0.9, 0.999, d * s)
        m.tensor(l, O.A_MAT)[:] = np.log(np.expm1(-np.log(u))).astype(np.float32)
        count = int(round(cap * bank_fill))
        dirs = rng.standard_normal((cap, k))
        dirs /= np.linalg.norm(dirs, axis=1, keepdims=True)
        keys = (dirs * rng.uniform(0, 0.9, (cap, 1))).astype(np.float32)
        vals = rng.standard_normal((cap, d)).astype(np.float32)
        for i in range(count):
            m.bank_insert(l, keys[i], vals[i])
    return m


def upload(oracle_model: "O.Model", gpu_model):
    """Copy every parameter, bank and carry of an oracle model into a pssa_b200.PSSAModel."""
    from pssa_b200 import model as M
    gpu_model.set_tensor(-1, M.EMBED, oracle_model.tensor(-1, O.EMBED))
    gpu_model.set_tensor(-1, M.UNEMBED, oracle_model.tensor(-1, O.UNEMBED))
    if oracle_model.depth > 1:
        gpu_model.set_tensor(-1, M.RESIDUAL_SCALES, oracle_model.tensor(-1, O.RESIDUAL_SCALES))
    for l in range(oracle_model.depth):
        for tid in M.BLOCK_TENSORS:
            gpu_model.set_tensor(l, tid, oracle_model.tensor(l, tid))
        count, head, _ = oracle_model.bank_meta(l)
        gpu_model.set_bank(l, oracle_model.tensor(l, O.BANK_KEYS), oracle_model.tensor(l, O.BANK_NORM_SQ),
                           oracle_model.tensor(l, O.BANK_VALUES), count, head, oracle_model.tensor(l, O.BANK_CONFIDENCE),
                           oracle_model.bank_last_seen(l))
    gpu_model.copy_recurrent_state_from(oracle_model.state(), 0)


def write_pssa_v8(m: "O.Model", step_counter: int = 0, rng_state: int = 1) -> bytes:
    """Serialise an oracle model as a version-8 `.pssa` container (src/checkpoint.rs:979-1087 layout): config words,
    depth, residual scales, counters, empty vocabulary, shared endpoints, one record per block, row marks. Optimizer
    moments are written as zeros. Written independently of both readers under test."""
    import struct
    out = bytearray()

    def u64(v):
        out.extend(struct.pack("<Q", int(v)))

    def f32(v):
        out.extend(struct.pack("<f", float(v)))

    def floats(a):
        a = np.ascontiguousarray(a, np.float32).ravel()
        u64(a.size)
        out.extend(a.tobytes())

    def param(a):
        floats(a)
        for _ in range(3):
            floats(np.zeros(np.asarray(a).size, np.float32))

    for v in (m.d_vocab, m.d_latent, m.d_state, m.d_mem_key, m.mem_capacity, m.chunk_len):
        u64(v)
    for v in (1e-3, 0.9, 0.999, 0.01, 1e-8, m.tau_mem, 0.99):
        f32(v)
    u64(m.depth)
    floats(m.tensor(-1, O.RESIDUAL_SCALES) if m.depth > 1 else np.zeros(0, np.float32))
    u64(step_counter)
    u64(rng_state)
    u64(0)  # vocabulary strings: none
    param(m.tensor(-1, O.EMBED))
    param(m.tensor(-1, O.UNEMBED))
    state = m.state().reshape(m.depth, -1)
    for l in range(m.depth):
        for tid in (O.A_MAT, O.W_DELTA, O.W_B, O.W_C, O.W_QX, O.W_QH, O.W_GATE, O.W_PROJ, O.MLP_W1, O.MLP_W2, O.NORM_GAMMA,
                    O.NORM_BETA):
            param(m.tensor(l, tid))
        floats(state[l])
        count, head, _ = m.bank_meta(l)
        u64(count)
        u64(head)
        for tid in (O.BANK_KEYS, O.BANK_VALUES, O.BANK_NORM_SQ, O.BANK_CONFIDENCE):
            floats(m.tensor(l, tid))
        seen = np.ascontiguousarray(m.bank_last_seen(l), np.uint64)
        u64(seen.size)
        out.extend(seen.tobytes())
        param(m.tensor(l, O.AD_DOWN))
        param(m.tensor(l, O.AD_UP))
        floats(m.tensor(l, O.AD_CONS))
    marks = np.zeros(m.d_vocab, np.uint64)
    u64(marks.size)
    out.extend(marks.tobytes())
    payload = bytes(out)
    h = 0xcbf29ce484222325
    for byte in payload:
        h = ((h ^ byte) * 0x100000001b3) & 0xFFFFFFFFFFFFFFFF
    return b"PSSA" + struct.pack("<HQQ", 8, len(payload), h) + payload
