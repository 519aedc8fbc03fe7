"""Parity of the Poincare memory read (project, distance, softmax / exact top-k, value read) with the CPU
oracle, through the C ABI."""
import numpy as np
import pytest

import oracle as O
from parity import REL_TOL, rel_err

pytestmark = pytest.mark.gpu

TINY = float(np.frombuffer(np.uint32(1).tobytes(), np.float32)[0])


@pytest.fixture(scope="module")
def gpu():
    import pssa_b200
    d = pssa_b200.B200Dispatch(0)
    yield d
    d.close()


def make_bank(cap, dk, dv, seed, max_radius=0.9):
    """Keys: direction N(0,I)/|.| times radius U(0, max_radius); norm_sq by the reference's rule."""
    rng = np.random.default_rng(seed)
    dirs = rng.standard_normal((cap, dk))
    dirs /= np.linalg.norm(dirs, axis=1, keepdims=True)
    keys = (dirs * rng.uniform(0, max_radius, (cap, 1))).astype(np.float32)
    norm_sq = np.array([O.lib().pssa_oracle_squared_norm(O.fptr(k), dk) for k in keys], np.float32)
    values = rng.standard_normal((cap, dv)).astype(np.float32)
    return keys, norm_sq, values


def check(gpu, q, keys, norm_sq, values, count, tau, top_k, euclid, exact):
    ref_p, ref_m, ref_w, ref_md = O.memory_read(keys, norm_sq, values, count, q, tau, top_k, euclid)
    q_pnc, q_norm, w, m, md = gpu.memory_read(q, keys, norm_sq, values, count, tau, top_k, euclid, exact)
    assert np.array_equal(q_pnc.view(np.uint32), ref_p.view(np.uint32)), "projection differs"
    if count == 0:
        assert not w.any() and not m.any()
        return
    # distances are f64 rounded to f32 on both sides
    assert np.array_equal(md.view(np.uint32), ref_md.view(np.uint32)) or rel_err(md, ref_md) <= 1.2e-7
    assert np.array_equal(w != 0, ref_w != 0), "selected slot sets differ"
    assert np.max(np.abs(w - ref_w)) <= (2e-7 if exact else 1e-6)  # weights are in [0, 1]
    scale = np.maximum(1e-6, np.abs(values[:max(count, 1)]).max())
    assert np.max(np.abs(m - ref_m)) / scale <= (2e-6 if exact else REL_TOL)


@pytest.mark.parametrize("rows,dk,dv,cap,count", [(1, 1, 1, 1, 1), (3, 2, 4, 3, 2), (65, 16, 64, 32, 32),
                                                  (130, 33, 70, 100, 77), (64, 64, 192, 512, 512),
                                                  (17, 128, 128, 512, 300)])
def test_fp32_distance_mode_stays_within_its_stated_error(gpu, rows, dk, dv, cap, count):
    """Fast mode (fp32 accumulation of the squared differences): the projection is still bit-exact, distances are
    within 2e-6 relative, so weights exp(-d/tau) move by at most d*2e-6/tau of themselves."""
    keys, norm_sq, values = make_bank(cap, dk, dv, rows + dk + cap)
    rng = np.random.default_rng(rows * 7)
    q = (rng.standard_normal((rows, dk)) * rng.uniform(0.05, 3.0, (rows, 1))).astype(np.float32)
    q[0] = keys[0] / (1.0 - np.linalg.norm(keys[0]))  # projects back onto slot 0 up to rounding: distance near zero
    tau = 0.1
    ref_p, ref_m, ref_w, ref_md = O.memory_read(keys, norm_sq, values, count, q, tau, 0, True)
    q_pnc, _, w, m, md = gpu.memory_read(q, keys, norm_sq, values, count, tau, 0, True, False, f32_distance=True)
    assert np.array_equal(q_pnc.view(np.uint32), ref_p.view(np.uint32))
    assert np.max(np.abs(md - ref_md)) <= 2e-6 * np.maximum(1.0, np.abs(ref_md).max()) + 1e-5
    assert np.max(np.abs(w - ref_w)) <= 2e-4
    scale = np.maximum(1e-6, np.abs(values[:count]).max())
    assert np.max(np.abs(m - ref_m)) / scale <= 4e-4
    assert abs(float(w[0].sum()) - 1.0) <= 1e-5


@pytest.mark.parametrize("top_k", [0, 8])
@pytest.mark.parametrize("rows,dk,dv,cap,count", [(1, 64, 64, 64, 1), (65, 64, 64, 32, 32), (300, 64, 192, 512, 512),
                                                  (130, 64, 70, 100, 77), (17, 128, 128, 512, 300), (64, 33, 16, 64, 64)])
def test_tensor_core_distance_mode_stays_within_its_stated_error(gpu, rows, dk, dv, cap, count, top_k):
    """Distances from |p|^2 + |k|^2 - 2 p.k with the inner product on the tensor cores (three bf16 pieces per operand):
    the projection is still bit-exact; |p - k|^2 carries an absolute error below 2.5e-6 (the tensor cores' fp32 accumulation is not correctly rounded), so u = |p - k|^2 / ((1-|p|^2)(1-|k|^2))
    is off by at most 2.5e-6 / ((1-|p|^2)(1-|k|^2)) and the distance by that over sqrt(u^2 + u), or by 2*sqrt of it near zero.
    A key width that is not a multiple of 64 (last case) falls back to the fp32 difference kernel."""
    keys, norm_sq, values = make_bank(cap, dk, dv, rows + dk + cap)
    rng = np.random.default_rng(rows * 11 + top_k)
    q = (rng.standard_normal((rows, dk)) * rng.uniform(0.02, 0.5, (rows, 1))).astype(np.float32)
    q[0] = keys[0] / (1.0 - np.linalg.norm(keys[0]))  # projects back onto slot 0 up to rounding: distance near zero
    tau = 0.1
    ref_p, ref_m, ref_w, ref_md = O.memory_read(keys, norm_sq, values, count, q, tau, top_k, True)
    q_pnc, _, w, m, md = gpu.memory_read(q, keys, norm_sq, values, count, tau, top_k, True, False, tc_distance=True)
    assert np.array_equal(q_pnc.view(np.uint32), ref_p.view(np.uint32))
    pn = (ref_p.astype(np.float64) ** 2).sum(1)
    conf = 1.0 / ((1.0 - pn) * (1.0 - float(norm_sq[:count].max())))
    du = 2.5e-6 * conf
    # d(u) = log1p(2u + 2 sqrt(u^2 + u)) is concave with d(0) = 0: |d(u + du) - d(u)| <= d(du)
    bound = np.log1p(2 * du + 2 * np.sqrt(du * du + du)) + 1e-5
    assert np.all(np.abs(md - ref_md) <= bound), (np.abs(md - ref_md).max(), bound.max())
    assert bound.max() <= 2.5e-2
    # weights exp(-d / tau) / sum: a distance error e moves a weight by at most about e / tau of itself (twice with the sum)
    if top_k == 0:
        assert np.all(np.abs(w - ref_w).max(1) <= 2.5 * bound / tau + 1e-6)
        scale = np.maximum(1e-6, np.abs(values[:count]).max())
        assert np.all(np.abs(m - ref_m).max(1) / scale <= 2.5 * bound / tau + 1e-5)
    else:
        same = (w != 0) == (ref_w != 0)
        assert same.all(1).mean() >= 0.97  # near-ties at the k-th place may swap
    assert abs(float(w[0].sum()) - 1.0) <= 1e-5


@pytest.mark.parametrize("exact", [False, True])
@pytest.mark.parametrize("top_k", [0, 1, 2, 8])
@pytest.mark.parametrize("rows,dk,dv,cap,count", [(1, 1, 1, 1, 1), (3, 2, 4, 3, 2), (65, 16, 64, 32, 32),
                                                  (130, 33, 70, 100, 77), (64, 64, 192, 512, 512),
                                                  (17, 128, 128, 512, 300)])
def test_read_matches_oracle(gpu, rows, dk, dv, cap, count, top_k, exact):
    keys, norm_sq, values = make_bank(cap, dk, dv, rows + dk + cap)
    rng = np.random.default_rng(rows * 7 + top_k)
    q = (rng.standard_normal((rows, dk)) * rng.uniform(0.05, 3.0, (rows, 1))).astype(np.float32)
    check(gpu, q, keys, norm_sq, values, count, 0.1, top_k, True, exact)


def test_queries_already_in_the_ball_and_other_temperatures(gpu):
    keys, norm_sq, values = make_bank(64, 8, 16, 3)
    q, _, _ = make_bank(40, 8, 16, 4)
    for tau in (0.8, 0.1, 1e-3, TINY):
        for top_k in (0, 3):
            check(gpu, q, keys, norm_sq, values, 64, tau, top_k, False, True)


def test_empty_bank_gives_zeros_but_publishes_the_projection(gpu):
    keys, norm_sq, values = make_bank(8, 4, 4, 1)
    q = np.random.default_rng(0).standard_normal((5, 4)).astype(np.float32)
    check(gpu, q, keys, norm_sq, values, 0, 0.1, 0, True, False)
    check(gpu, q, keys, norm_sq, values, 0, 0.1, 2, True, True)


def test_reference_known_answers(gpu):
    # tests/memory_projection.rs:37-53: subnormal temperature, two tied nearest slots
    keys = np.array([[0.5], [-0.5], [0.75]], np.float32)
    norm_sq = (keys[:, 0] ** 2).astype(np.float32)
    values = np.array([[1.0, 2.0], [3.0, -2.0], [100.0, 100.0]], np.float32)
    q = np.zeros((1, 1), np.float32)
    for exact in (False, True):
        _, _, w, m, _ = gpu.memory_read(q, keys, norm_sq, values, 3, TINY, 0, False, exact)
        assert w.tolist() == [[0.5, 0.5, 0.0]] and m.tolist() == [[2.0, 0.0]]
    # tests/memory_expansion.rs:79-92: top-1 with a tie keeps the lowest slot
    keys = np.array([[0.2], [-0.2], [0.0], [0.0]], np.float32)
    norm_sq = (keys[:, 0] ** 2).astype(np.float32)
    values = np.array([[1.0], [2.0], [0.0], [0.0]], np.float32)
    _, _, w, m, _ = gpu.memory_read(q, keys, norm_sq, values, 2, TINY, 1, False, True)
    assert w.tolist() == [[1.0, 0.0, 0.0, 0.0]] and m.tolist() == [[1.0]]
    # tests/memory_expansion.rs:52-77: top-k >= count is the full read
    keys = np.array([[0.0], [0.1], [0.6], [0.0], [0.0]], np.float32)
    norm_sq = (keys[:, 0].astype(np.float64) ** 2).astype(np.float32)
    values = np.array([[2.0], [4.0], [100.0], [0.0], [0.0]], np.float32)
    full = gpu.memory_read(q, keys, norm_sq, values, 3, 1.0, 0, False, True)
    for k in (3, 9):
        got = gpu.memory_read(q, keys, norm_sq, values, 3, 1.0, k, False, True)
        assert np.array_equal(got[2], full[2]) and np.array_equal(got[3], full[3])
    _, _, w, m, _ = gpu.memory_read(q, keys, norm_sq, values, 3, 1.0, 1, False, True)
    assert m.tolist() == [[2.0]] and w.tolist() == [[1.0, 0.0, 0.0, 0.0, 0.0]]


def test_extreme_queries_stay_in_the_ball(gpu):
    # tests/memory_projection.rs:3-35
    fmax = np.finfo(np.float32).max
    for vec in ([0.0], [16_777_216.0], [-fmax], [fmax, -fmax, fmax], [TINY, -TINY]):
        q = np.array([vec], np.float32)
        ref_p, _, _, _ = O.memory_read(np.zeros((1, len(vec)), np.float32), np.zeros(1, np.float32),
                                       np.zeros((1, 1), np.float32), 1, q, 0.1, 0, True)
        got = gpu.memory_read(q, np.zeros((1, len(vec)), np.float32), np.zeros(1, np.float32),
                              np.zeros((1, 1), np.float32), 1, 0.1, 0, True, True)
        assert np.array_equal(got[0].view(np.uint32), ref_p.view(np.uint32))
        assert np.isfinite(got[1]).all() and float((got[0].astype(np.float64) ** 2).sum()) < 1.0


def test_operator_shape_top8_device_resident(gpu):
    """The retrieval operator's own shape (512 slots, key/value dim 128, tau 0.1, top-8) on device buffers:
    a sample of rows against the oracle plus whole-batch properties (weights sum to one, at most 8 nonzero)."""
    import torch
    rows, dk, dv, cap = 64 * 1024, 128, 128, 512
    keys, norm_sq, values = make_bank(cap, dk, dv, 11)
    qk, _, _ = make_bank(4096, dk, dv, 12)
    q = np.tile(qk, (rows // 4096, 1))
    tq, tk, tn, tv = (torch.from_numpy(x).cuda() for x in (q, keys, norm_sq, values))
    w = torch.zeros(rows, cap, device="cuda")
    m = torch.zeros(rows, dv, device="cuda")
    gpu.set_stream(torch.cuda.current_stream())
    for top_k in (8, 0):
        gpu.memory_read_dev(tq, tk, tn, tv, rows, dk, dv, cap, cap, 0.1, m, top_k=top_k, weights=w,
                            q_is_euclidean=False)
        torch.cuda.synchronize()
        sums = w.sum(dim=1)
        assert float((sums - 1.0).abs().max()) <= 1e-5
        if top_k:
            assert int((w != 0).sum(dim=1).max()) <= top_k
        sample = slice(4000, 4256)
        _, ref_m, ref_w, _ = O.memory_read(keys, norm_sq, values, cap, q[sample], 0.1, top_k, False)
        assert np.array_equal(w[sample].cpu().numpy() != 0, ref_w != 0)
        assert np.max(np.abs(w[sample].cpu().numpy() - ref_w)) <= 1e-6
        assert np.max(np.abs(m[sample].cpu().numpy() - ref_m)) <= REL_TOL * np.abs(values).max()
    gpu.set_stream(None)


def test_shape_errors(gpu):
    import pssa_b200
    keys, norm_sq, values = make_bank(8, 4, 4, 1)
    q = np.zeros((2, 4), np.float32)
    with pytest.raises(pssa_b200.B200Error) as e:
        gpu.memory_read(q, keys, norm_sq, values, 9, 0.1)
    assert e.value.status == 2 and "invalid count/capacity (9/8)" in str(e.value)
    with pytest.raises(pssa_b200.B200Error) as e:
        gpu.memory_read(q, keys, norm_sq, values, 8, 0.0)
    assert "temperature" in str(e.value)
