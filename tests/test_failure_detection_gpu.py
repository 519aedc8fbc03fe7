"""Failure detection on the device without a fault: a bounded wait that nothing satisfies expires, the kernel records
PSSA_B200_ERR_TIMEOUT and returns, the host reads the record, and the context keeps working. The waiting kernel uses
the tensor-core pipeline's own wait helper with a poll limit of a few thousand; nothing traps, faults or spins without
bound. Host-side failure injection (bad shapes, bad handles, no device) is in test_abi.py and the operator tests."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_an_expired_device_side_wait_is_reported_once_and_the_context_survives():
    import torch

    import pssa_b200
    from pssa_b200 import _native as N
    gpu = pssa_b200.B200Dispatch(0)
    try:
        gpu.poll_status()  # clean to begin with
        gpu.selftest_wait_expiry(4096)
        with pytest.raises(pssa_b200.B200Error) as e:
            gpu.poll_status()
        assert e.value.status == N.ERR_TIMEOUT and "bounded device-side wait expired" in str(e.value)
        gpu.poll_status()  # reading the record cleared it
        # the next calls on the same context work: a tensor-core product (the pipeline whose waits are bounded) and a scan
        rng = np.random.default_rng(0)
        x = rng.standard_normal((200, 128)).astype(np.float32)
        w = rng.standard_normal((96, 128)).astype(np.float32)
        out = np.zeros((200, 96), np.float32)
        gpu.dispatch_gemm_into(x, w, 200, 96, 128, 1, out, precision=N.PRECISION_BF16)
        want = x @ w.T
        assert float(np.max(np.abs(out - want))) <= 0.02 * float(np.abs(want).max())
        a = rng.uniform(0.9, 0.999, (1, 50, 8)).astype(np.float32)
        b = rng.standard_normal((1, 50, 8)).astype(np.float32)
        h = gpu.scan_states(a, b, None)
        assert np.isfinite(h).all()
        gpu.poll_status()
        # argument validation of the self-test itself
        for polls in (0, (1 << 20) + 1):
            with pytest.raises(pssa_b200.B200Error):
                gpu.selftest_wait_expiry(polls)
        # a GEMM whose host entry point sees the record reports it too (and clears it)
        gpu.selftest_wait_expiry(64)
        with pytest.raises(pssa_b200.B200Error) as e:
            gpu.dispatch_gemm_into(x, w, 200, 96, 128, 1, out, precision=N.PRECISION_BF16)
        assert e.value.status == N.ERR_TIMEOUT
        gpu.poll_status()
    finally:
        gpu.close()
    torch.cuda.synchronize()
