"""Parity of the fused SSM stage (discretise + scan + read out) with the CPU oracle, through the C ABI."""
import numpy as np
import pytest

import oracle as O
from parity import REL_TOL, chan_err, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    import pssa_b200
    d = pssa_b200.B200Dispatch(0)
    yield d
    d.close()


def inputs(T, d, s, seed):
    rng = np.random.default_rng(seed)
    delta = np.log1p(np.exp(rng.normal(-2.0, 1.0, (T, d)))).astype(np.float32)  # softplus of a projection
    bp = rng.normal(0, 1, (T, s)).astype(np.float32)
    cp = rng.normal(0, 1, (T, s)).astype(np.float32)
    x = rng.normal(0, 1, (T, d)).astype(np.float32)
    # decay exp(delta*A) mostly in (0.9, 0.999) like the model's log-spaced rates (src/pssa.rs:649-665)
    rates = -np.exp(rng.uniform(np.log(0.005), np.log(0.7), d * s)).astype(np.float32)
    h0 = rng.normal(0, 1, d * s).astype(np.float32)
    return delta, bp, cp, x, rates, h0


SHAPES = [(1, 4, 2), (2, 7, 3), (3, 16, 16), (31, 12, 4), (32, 64, 64), (33, 20, 8), (257, 32, 64), (130, 9, 5),
          (64, 8, 128), (40, 192, 64)]


@pytest.mark.parametrize("exact", [False, True])
@pytest.mark.parametrize("T,d,s", SHAPES)
def test_single_lane_matches_ordered_recurrence(gpu, T, d, s, exact):
    delta, bp, cp, x, rates, h0 = inputs(T, d, s, T * 1000 + d * 10 + s)
    ref_states, ref_y, ref_a, ref_b = O.ssm_forward(delta, bp, cp, x, rates, h0, mode=0)
    y = np.empty((T, d), np.float32)
    states = np.empty((T + 1, d * s), np.float32)
    bar_a = np.empty((T, d * s), np.float32)
    bar_b = np.empty((T, d * s), np.float32)
    gpu.ssm_forward(delta, bp, x, rates, cp, h0, T, d, s, bar_a, bar_b, states, y, exact=exact)
    assert np.array_equal(states[0], h0)
    assert np.array_equal(bar_b.view(np.uint32), ref_b.view(np.uint32))  # one rounded product in both modes
    assert rel_err(bar_a, ref_a) <= (2e-7 if exact else 6e-7)
    tol = 5e-6 if exact else REL_TOL  # CUDA expf (<= 2 ulp) vs glibc expf, both within their documented error
    assert chan_err(states, ref_states, 0) <= tol
    assert chan_err(y, ref_y, 0) <= tol
    # without the tape outputs (the inference form) y is the same
    y2 = np.empty_like(y)
    gpu.ssm_forward(delta, bp, x, rates, cp, h0, T, d, s, None, None, None, y2, exact=exact)
    assert np.array_equal(y2, y)


def test_packed_ragged_lanes_with_an_idle_lane(gpu):
    # lanes as in src/sequence_batch.rs:233-384: packed rows, per-lane carry; an omitted lane keeps its carry
    import torch
    d, s = 48, 16
    lengths = np.array([5, 0, 33, 1, 70], np.uint32)
    offsets = np.concatenate([[0], np.cumsum(lengths)[:-1]]).astype(np.uint32)
    rows = int(lengths.sum())
    delta, bp, cp, x, rates, _ = inputs(rows, d, s, 77)
    carry = np.random.default_rng(1).normal(size=(len(lengths), d * s)).astype(np.float32)
    ref_carry = carry.copy()
    ref_y = O.ssm_lanes(delta, bp, cp, x, rates, ref_carry, offsets, lengths)
    t = {k: torch.from_numpy(v).cuda() for k, v in dict(delta=delta, bp=bp, cp=cp, x=x, rates=rates, carry=carry).items()}
    y = torch.zeros(rows, d, device="cuda")
    gpu.set_stream(torch.cuda.current_stream())
    for exact in (False, True):
        c = t["carry"].clone()
        gpu.ssm_forward_dev(t["delta"], t["bp"], t["cp"], t["x"], t["rates"], c, y, offsets, lengths, rows, d, s,
                            exact=exact)
        torch.cuda.synchronize()
        got_c = c.cpu().numpy()
        assert np.array_equal(got_c[1], carry[1])  # idle lane untouched
        assert chan_err(y.cpu().numpy(), ref_y, 0) <= REL_TOL
        scale = np.maximum(1e-6, np.abs(ref_carry).max())
        assert float(np.max(np.abs(got_c - ref_carry))) / scale <= REL_TOL
    gpu.set_stream(None)


def test_decode_step_shape_one_token_per_lane_with_an_idle_lane(gpu):
    """Every lane one token long (the decode step, which has its own kernel in the fast mode): y and the carries
    match the oracle, the idle lane keeps its carry, and a second step continues from the first."""
    import torch
    for d, s in ((48, 16), (768, 64), (20, 8), (32, 128)):
        lengths = np.array([1, 1, 0, 1, 1, 1], np.uint32)
        offsets = np.concatenate([[0], np.cumsum(lengths)[:-1]]).astype(np.uint32)
        rows = int(lengths.sum())
        carry = np.random.default_rng(d).normal(size=(len(lengths), d * s)).astype(np.float32)
        ref_carry = carry.copy()
        c = torch.from_numpy(carry).cuda()
        gpu.set_stream(torch.cuda.current_stream())
        for step in range(2):
            delta, bp, cp, x, rates, _ = inputs(rows, d, s, 100 + step)
            ref_y = O.ssm_lanes(delta, bp, cp, x, rates, ref_carry, offsets, lengths)
            t = {k: torch.from_numpy(v).cuda() for k, v in dict(delta=delta, bp=bp, cp=cp, x=x, rates=rates).items()}
            y = torch.zeros(rows, d, device="cuda")
            gpu.ssm_forward_dev(t["delta"], t["bp"], t["cp"], t["x"], t["rates"], c, y, offsets, lengths, rows, d, s)
            torch.cuda.synchronize()
            got_c = c.cpu().numpy()
            assert np.array_equal(got_c[2], carry[2])  # idle lane untouched
            assert chan_err(y.cpu().numpy(), ref_y, 0) <= REL_TOL
            scale = np.maximum(1e-6, np.abs(ref_carry).max())
            assert float(np.max(np.abs(got_c - ref_carry))) / scale <= REL_TOL
        gpu.set_stream(None)


def test_continuation_equals_one_pass_bitwise_at_model_size(gpu):
    """Size-independent property at the stacked model's shape (d 768, state 64): running a sequence in two
    calls with the carry handed over gives bit-identical y and carry to one call (src/pssa.rs:1245-1247)."""
    import torch
    lanes, T, d, s = 4, 512, 768, 64
    g = torch.Generator(device="cuda").manual_seed(5)
    delta = torch.nn.functional.softplus(torch.randn(lanes * T, d, device="cuda", generator=g) - 2.0)
    x = torch.randn(lanes * T, d, device="cuda", generator=g)
    bp = torch.randn(lanes * T, s, device="cuda", generator=g)
    cp = torch.randn(lanes * T, s, device="cuda", generator=g)
    rates = -torch.exp(torch.empty(d, s, device="cuda").uniform_(-5.0, -0.4, generator=g))
    off = (np.arange(lanes) * T).astype(np.uint32)
    full = np.full(lanes, T, np.uint32)
    half = np.full(lanes, T // 2, np.uint32)
    gpu.set_stream(torch.cuda.current_stream())
    c1 = torch.zeros(lanes, d * s, device="cuda")
    y1 = torch.zeros(lanes * T, d, device="cuda")
    gpu.ssm_forward_dev(delta, bp, cp, x, rates, c1, y1, off, full, lanes * T, d, s)
    c2 = torch.zeros(lanes, d * s, device="cuda")
    y2 = torch.zeros(lanes * T, d, device="cuda")
    gpu.ssm_forward_dev(delta, bp, cp, x, rates, c2, y2, off, half, lanes * T, d, s)
    gpu.ssm_forward_dev(delta, bp, cp, x, rates, c2, y2, off + T // 2, half, lanes * T, d, s)
    torch.cuda.synchronize()
    gpu.set_stream(None)
    assert torch.equal(y1, y2) and torch.equal(c1, c2)
    assert bool(torch.isfinite(y1).all())


def test_shape_and_lane_errors(gpu):
    import pssa_b200
    delta, bp, cp, x, rates, h0 = inputs(4, 8, 4, 0)
    y = np.full((4, 8), 7.0, np.float32)
    with pytest.raises(pssa_b200.B200Error) as e:
        gpu.ssm_forward(delta[:3], bp, x, rates, cp, h0, 4, 8, 4, y_ssm=y)
    assert e.value.status == 2 and "shape mismatch" in str(e.value) and np.all(y == 7.0)
    with pytest.raises(pssa_b200.B200Error) as e:
        gpu.ssm_forward(delta[:0], bp[:0], x[:0], rates, cp[:0], h0, 0, 8, 4, y_ssm=y[:0])
    assert "must be positive" in str(e.value)
    import torch
    z = torch.zeros(4, 8, device="cuda")
    with pytest.raises(pssa_b200.B200Error) as e:
        gpu.ssm_forward_dev(z, z, z, z, z, None, z, np.array([0, 3], np.uint32), np.array([3, 2], np.uint32), 4, 8, 4)
    assert e.value.status == 2 and "outside 4 rows" in str(e.value)
