"""Parity of the CUDA scan operator with the CPU oracle, through the C ABI (needs a B200)."""
import numpy as np
import pytest

import oracle as O

pytestmark = pytest.mark.gpu

from parity import REL_TOL, chan_err, rel_err, rel_p99  # fp32 scan within 1e-5 relative


@pytest.fixture(scope="module")
def gpu():
    import pssa_b200
    d = pssa_b200.B200Dispatch(0)
    yield d
    d.close()


def make(lanes, T, stride, seed):
    rng = np.random.default_rng(seed)
    a = rng.uniform(0.9, 0.999, (lanes, T, stride)).astype(np.float32)
    b = rng.standard_normal((lanes, T, stride), dtype=np.float32)
    h0 = rng.standard_normal((lanes, stride), dtype=np.float32)
    return a, b, h0


@pytest.mark.parametrize("T", [1, 2, 3, 31, 32, 33, 255, 256, 257, 1000])
@pytest.mark.parametrize("stride", [1, 3, 8, 36, 100])
def test_states_single_chunk_is_bit_identical_to_the_ordered_recurrence(gpu, T, stride):
    a, b, h0 = make(2, T, stride, T * 131 + stride)
    gpu.set_scan_chunks(1)
    h, last = gpu.scan_states(a, b, h0, want_last=True)
    ref = O.scan_states(a, b, h0)
    assert np.array_equal(h.view(np.uint32), ref.view(np.uint32))
    assert np.array_equal(last.view(np.uint32), ref[:, -1].view(np.uint32))


@pytest.mark.parametrize("chunks", [2, 3, 7, 64])
@pytest.mark.parametrize("T,stride", [(2, 4), (33, 5), (257, 12), (1024, 64), (4096, 8)])
def test_states_chunked_passes_match_within_tolerance(gpu, chunks, T, stride):
    a, b, h0 = make(3, T, stride, chunks * 7 + T)
    gpu.set_scan_chunks(chunks)
    h, last = gpu.scan_states(a, b, h0, want_last=True)
    gpu.set_scan_chunks(0)
    ref = O.scan_states(a, b, h0)
    # chunk boundaries reassociate the recurrence: per-channel-scale bound (tests/parity.py)
    assert chan_err(h, ref, 1) <= REL_TOL
    assert h.size < 100_000 or rel_p99(h, ref) <= REL_TOL
    scale = np.maximum(1e-6, np.abs(ref).max(axis=1))
    assert float(np.max(np.abs(last - ref[:, -1]) / scale)) <= REL_TOL


def test_states_without_carry_in_start_from_zero(gpu):
    a, b, _ = make(1, 300, 16, 5)
    gpu.set_scan_chunks(1)
    got = gpu.scan_states(a, b)
    gpu.set_scan_chunks(0)
    assert np.array_equal(got, O.scan_states(a, b))


@pytest.mark.parametrize("chunks", [0, 1, 4])
@pytest.mark.parametrize("T,stride", [(1, 1), (3, 2), (7, 3), (33, 4), (129, 8), (1024, 20)])
def test_exclusive_map_scan_matches_the_blelloch_oracle(gpu, chunks, T, stride):
    # contract of src/gpu_batch.rs:3808-3835 with the tolerances of tests/associative_scan.rs:10
    a, b, _ = make(1, T, stride, T + stride)
    pa, pb = a[0].copy(), b[0].copy()
    gpu.set_scan_chunks(chunks)
    gpu.affine_scan_in_place(pa, pb, T, stride)
    gpu.set_scan_chunks(0)
    ra, rb = O.affine_scan_exclusive(a[0], b[0])
    assert np.all(pa[0] == 1.0) and np.all(pb[0] == 0.0)
    assert rel_err(pa, ra) <= REL_TOL
    assert np.max(np.abs(pb - rb)) <= 2e-5 * max(1.0, float(np.max(np.abs(rb))))


def test_device_pointer_entry_with_automatic_chunking(gpu):
    import torch
    lanes, T, stride = 2, 2048, 256  # few channels: the automatic policy splits time
    a, b, h0 = make(lanes, T, stride, 99)
    ta, tb, th0 = (torch.from_numpy(x).cuda() for x in (a, b, h0))
    th = torch.empty_like(ta)
    tlast = torch.empty_like(th0)
    gpu.set_stream(torch.cuda.current_stream())
    gpu.scan_states_dev(ta, tb, th0, th, tlast, lanes, T, stride)
    torch.cuda.synchronize()
    ref = O.scan_states(a, b, h0)
    assert chan_err(th.cpu().numpy(), ref, 1) <= REL_TOL and rel_p99(th.cpu().numpy(), ref) <= REL_TOL
    scale = np.maximum(1e-6, np.abs(ref).max(axis=1))
    assert float(np.max(np.abs(tlast.cpu().numpy() - ref[:, -1]) / scale)) <= REL_TOL
    # in place over b
    gpu.scan_states_dev(ta, tb, th0, tb, None, lanes, T, stride)
    torch.cuda.synchronize()
    assert torch.equal(tb, th)
    gpu.set_stream(None)


def test_full_size_property_linearity_and_last_row(gpu):
    """At a size the oracle cannot finish quickly: the scan is linear in b, and constant maps have a
    closed form (h_T = a^T h0 + b (1 - a^T) / (1 - a))."""
    import torch
    lanes, T, stride = 8, 4096, 8192
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.empty(lanes, T, stride, device="cuda").uniform_(0.9, 0.999, generator=g)
    b1 = torch.randn(lanes, T, stride, device="cuda", generator=g)
    b2 = torch.randn(lanes, T, stride, device="cuda", generator=g)
    h1, h2, h12 = torch.empty_like(a), torch.empty_like(a), torch.empty_like(a)
    gpu.set_stream(torch.cuda.current_stream())
    gpu.scan_states_dev(a, b1, None, h1, None, lanes, T, stride)
    gpu.scan_states_dev(a, b2, None, h2, None, lanes, T, stride)
    gpu.scan_states_dev(a, b1 + b2, None, h12, None, lanes, T, stride)
    torch.cuda.synchronize()
    scale = float(h12.abs().max())
    assert float((h1 + h2 - h12).abs().max()) <= 2e-5 * scale
    a.fill_(0.5)
    b1.fill_(1.0)
    gpu.scan_states_dev(a, b1, None, h1, None, lanes, T, stride)
    torch.cuda.synchronize()
    gpu.set_stream(None)
    assert float((h1[:, -1] - 2.0).abs().max()) <= 1e-6 and float((h1[:, 0] - 1.0).abs().max()) == 0.0


def test_shape_errors_leave_outputs_untouched(gpu):
    import pssa_b200
    a = np.ones((1, 4, 4), np.float32)
    with pytest.raises(pssa_b200.B200Error) as e:
        gpu._check(gpu._lib.pssa_b200_scan_states(gpu._h, a.ctypes.data, a.ctypes.data, None, a.ctypes.data, None, 0, 4, 4))
    assert e.value.status == 2 and "refusing launch" in str(e.value)
    assert np.all(a == 1.0)
    with pytest.raises(pssa_b200.B200Error) as e:
        gpu._check(gpu._lib.pssa_b200_scan_states(gpu._h, a.ctypes.data, a.ctypes.data, None, a.ctypes.data, None,
                                                  1 << 40, 1 << 40, 1 << 40))
    assert e.value.status == 2 and "overflow" in str(e.value)
