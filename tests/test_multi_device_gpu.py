"""One host process, contexts on two GPUs: what a Rust `Device::B200` per GPU would do. Kernel attributes such as the
opt-in dynamic shared-memory size are per device, so every launcher must set them on each device it meets, not once per
process. Runs a tensor-core product, the fused SSM and a memory read (all of which need more than 48 KB of shared memory
per CTA) on devices 0 and 1 in turn. Skipped below two GPUs."""
import numpy as np
import pytest

import oracle as O
from parity import chan_err

pytestmark = pytest.mark.gpu


def test_contexts_on_two_devices_in_one_process_both_launch_large_shared_memory_kernels():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import pssa_b200
    from pssa_b200 import _native as N
    rng = np.random.default_rng(4)
    x = rng.standard_normal((300, 256)).astype(np.float32)
    w = rng.standard_normal((384, 256)).astype(np.float32)
    want = x @ w.T
    T, d, s = 64, 192, 64
    delta = np.log1p(np.exp(rng.normal(-2.0, 1.0, (T, d)))).astype(np.float32)
    bp, cp = rng.normal(0, 1, (T, s)).astype(np.float32), rng.normal(0, 1, (T, s)).astype(np.float32)
    xs = rng.normal(0, 1, (T, d)).astype(np.float32)
    rates = -np.exp(rng.uniform(np.log(0.005), np.log(0.7), d * s)).astype(np.float32)
    h0 = rng.normal(0, 1, d * s).astype(np.float32)
    _, ref_y, _, _ = O.ssm_forward(delta, bp, cp, xs, rates, h0, mode=0)
    cap, dk, dv = 512, 64, 96
    dirs = rng.standard_normal((cap, dk))
    keys = (dirs / np.linalg.norm(dirs, axis=1, keepdims=True) * rng.uniform(0, 0.9, (cap, 1))).astype(np.float32)
    norm_sq = (keys.astype(np.float64) ** 2).sum(1).astype(np.float32)
    vals = rng.standard_normal((cap, dv)).astype(np.float32)
    q = rng.standard_normal((70, dk)).astype(np.float32)
    _, ref_m, ref_w, _ = O.memory_read(keys, norm_sq, vals, cap, q, 0.1, top_k=8, q_is_euclidean=True)
    gpus = [pssa_b200.B200Dispatch(i) for i in (0, 1)]
    try:
        for rounds in range(2):  # the second round finds every attribute already set on both devices
            for g in gpus:
                out = np.zeros_like(want)
                g.dispatch_gemm_into(x, w, 300, 384, 256, 1, out, precision=N.PRECISION_BF16)
                assert float(np.max(np.abs(out - want))) <= 0.02 * float(np.abs(want).max())
                y = np.empty((T, d), np.float32)
                g.ssm_forward(delta, bp, xs, rates, cp, h0, T, d, s, None, None, None, y)
                assert chan_err(y, ref_y, 0) <= 1e-5
                res = g.memory_read(q, keys, norm_sq, vals, cap, 0.1, top_k=8, q_is_euclidean=True)
                got_w, got_m = res[2], res[3]
                assert np.array_equal(got_w != 0, ref_w != 0)
                assert float(np.max(np.abs(got_m - ref_m))) <= 1e-5 * float(np.abs(ref_m).max())
                g.poll_status()
    finally:
        for g in gpus:
            g.close()
