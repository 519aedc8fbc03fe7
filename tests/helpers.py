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
