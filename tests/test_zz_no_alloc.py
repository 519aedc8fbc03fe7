"""The allocation-free scan entry point against the arena-backed one (collected last on purpose: if it fails,
a run that stops at the first failure has already run every other test).

Callers it serves: processes that may not allocate device memory after start-up (their own pool owns the GPU)
or that cannot accept the implicit device synchronisation of cudaMalloc / cudaFree in a latency-critical loop.
"""
import numpy as np
import pytest

import oracle as O

pytestmark = pytest.mark.gpu


def test_noalloc_scan_matches_the_arena_backed_scan_on_two_calls_in_a_row():
    import torch

    import pssa_b200
    gpu = pssa_b200.B200Dispatch(0)
    gpu.set_stream(torch.cuda.current_stream())
    try:
        lanes, T, stride, chunks = 2, 1024, 256, 8
        g = torch.Generator(device="cuda").manual_seed(17)
        for call in range(2):  # second call reuses the fixed scratch with different data and a different chunking
            a = torch.empty(lanes, T, stride, device="cuda").uniform_(0.9, 0.999, generator=g)
            b = torch.randn(lanes, T, stride, device="cuda", generator=g)
            h0 = torch.randn(lanes, stride, device="cuda", generator=g)
            want, want_last = torch.empty_like(a), torch.empty_like(h0)
            got, got_last = torch.full_like(a, float("nan")), torch.full_like(h0, float("nan"))
            gpu.set_scan_chunks(chunks)
            gpu.scan_states_dev(a, b, h0, want, want_last, lanes, T, stride)
            gpu.set_scan_chunks(0)
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
            gpu.scan_states_noalloc_dev(a, b, h0, got, got_last, lanes, T, stride, chunks)
            torch.cuda.synchronize()
            # the property the entry point exists for: the device's free memory does not move across the call (the
            # first call only looks up the address of the array that was loaded with the library)
            assert torch.cuda.mem_get_info()[0] == free_before, f"call {call}: device memory in use changed"
            # against the CPU oracle's ordered recurrence, not only against the library's other entry point
            ref = O.scan_states(a.cpu().numpy(), b.cpu().numpy(), h0.cpu().numpy())
            ref_scale = np.maximum(1e-6, np.abs(ref).max(axis=1, keepdims=True))
            assert float(np.max(np.abs(got.cpu().numpy() - ref) / ref_scale)) <= 1e-5
            assert float(np.max(np.abs(got_last.cpu().numpy() - ref[:, -1]) / ref_scale[:, 0])) <= 1e-5
            # same kernels, same chunking: the tolerance of the chunked-scan tests (1e-5 of the channel's scale)
            scale = want.abs().amax(dim=1, keepdim=True).clamp_min(1e-6)
            assert float(((got - want).abs() / scale).max()) <= 1e-5
            assert float(((got_last - want_last).abs() / scale[:, 0]).max()) <= 1e-5
            chunks = 3
        # one chunk needs no scratch at all
        gpu.scan_states_noalloc_dev(a, b, h0, got, None, lanes, T, stride, 1)
        gpu.set_scan_chunks(1)
        gpu.scan_states_dev(a, b, h0, want, None, lanes, T, stride)
        gpu.set_scan_chunks(0)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        # beyond the fixed maximum: a clear error, nothing launched
        with pytest.raises(pssa_b200.B200Error) as e:
            gpu.scan_states_noalloc_dev(a, b, h0, got, None, 64, 4096, 8192, 4)
        assert e.value.status == 2 and "exceeds the fixed scratch" in str(e.value)
    finally:
        gpu.set_stream(None)
        gpu.close()
