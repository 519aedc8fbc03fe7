"""The stage-level operators that carry the reference's `GpuDispatch` argument lists -- `memory_forward`
(src/backend.rs:1342-1385) and the resident pair `ssm_forward_resident` / `memory_forward_after_ssm`
(src/backend.rs:1186-1289) -- against the CPU oracle's stage arithmetic (`stage_memory_impl`, src/gpu_batch.rs:758-929)."""
import numpy as np
import pytest

import oracle as O
from parity import chan_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    import pssa_b200
    d = pssa_b200.B200Dispatch(0)
    yield d
    d.close()


def _case(T, d_m, d_k, d_val, cap, count, seed):
    rng = np.random.default_rng(seed)
    f = lambda *s: rng.normal(0, 1, s).astype(np.float32)  # noqa: E731
    x, y = f(T, d_m), f(T, d_m)
    w_qx, w_qh = f(d_k, d_m) * 0.2, f(d_k, d_m) * 0.2
    w_gate, w_proj = f(d_m, d_m) * 0.2, f(d_m, d_val) * 0.2
    dirs = rng.standard_normal((cap, d_k))
    keys = (dirs / np.linalg.norm(dirs, axis=1, keepdims=True) * rng.uniform(0, 0.9, (cap, 1))).astype(np.float32)
    keys[count:] = 0
    norm_sq = (keys.astype(np.float64) ** 2).sum(1).astype(np.float32)
    values = f(cap, d_val)
    return x, y, w_qx, w_qh, w_gate, w_proj, keys, norm_sq, values


def _oracle_memory_stage(x, y, w_qx, w_qh, w_gate, w_proj, keys, norm_sq, values, count, tau):
    """src/gpu_batch.rs:850-929 from the oracle's operators: every product entry is one `dot_slice`."""
    q_euc = O.gemm_xwt(x, w_qx) + O.gemm_xwt(y, w_qh)  # f32 add of the two dots (src/gpu_batch.rs:874-876)
    q_pnc, m_val, weights, _ = O.memory_read(keys, norm_sq, values, count, q_euc, tau, q_is_euclidean=True)
    q_norm = np.sqrt((q_euc.astype(np.float64) ** 2).sum(1)).astype(np.float32)
    sig = np.vectorize(lambda v: O.lib().pssa_oracle_sigmoid(float(v)), otypes=[np.float32])
    g = sig(O.gemm_xwt(x, w_gate))
    m_proj = O.gemm_xwt(m_val, w_proj)
    return dict(q_euc=q_euc, q_pnc=q_pnc, q_norm=q_norm, weights=weights, m_val=m_val, g_mem=g, m_proj=m_proj, m_inj=g * m_proj)


@pytest.mark.parametrize("T,d_m,d_k,d_val,cap,count", [(37, 40, 12, 40, 20, 13), (5, 16, 8, 24, 8, 8), (130, 64, 64, 64, 128, 128), (3, 24, 4, 8, 4, 0)])
def test_memory_forward_matches_the_stage_arithmetic_of_the_reference(gpu, T, d_m, d_k, d_val, cap, count):
    case = _case(T, d_m, d_k, d_val, cap, count, seed=T + d_m)
    ref = _oracle_memory_stage(*case, count, 0.1)
    got = gpu.memory_forward(*case, T, d_m, d_k, d_val, cap, count, 0.1)
    # the products keep the reference's dot-product order: bit-equal
    for name in ("q_euc", "m_proj") if count else ("q_euc",):
        if name == "q_euc":
            assert np.array_equal(got[name].view(np.uint32), ref[name].view(np.uint32)), name
    for name, want in ref.items():
        scale = max(1e-6, float(np.abs(want).max()))
        assert float(np.max(np.abs(got[name] - want))) / scale <= 1e-5, name
    if count == 0:  # src/memory.rs:363-367
        assert not got["weights"].any() and not got["m_val"].any() and not got["m_inj"].any()


def test_memory_forward_on_the_tensor_cores(gpu):
    from pssa_b200 import _native as N
    T, d_m, d_k, d_val, cap, count = 200, 64, 16, 64, 64, 64
    case = _case(T, d_m, d_k, d_val, cap, count, seed=9)
    ref = _oracle_memory_stage(*case, count, 0.5)
    got = gpu.memory_forward(*case, T, d_m, d_k, d_val, cap, count, 0.5, precision=N.PRECISION_BF16)
    for name, want in ref.items():
        scale = max(1e-6, float(np.abs(want).max()))
        assert float(np.max(np.abs(got[name] - want))) / scale <= (6e-2 if name in ("weights", "m_val", "m_proj", "m_inj") else 2e-2), name


def test_bad_shapes_leave_the_outputs_untouched(gpu):
    import pssa_b200
    T, d_m, d_k, d_val, cap, count = 4, 8, 4, 8, 4, 4
    case = _case(T, d_m, d_k, d_val, cap, count, seed=1)
    out = gpu._memory_outputs(T, d_m, d_k, d_val, cap)
    for v in out.values():
        v[...] = 7.0
    with pytest.raises(pssa_b200.B200Error, match="refusing launch"):
        gpu.memory_forward(*case, T, d_m, d_k, d_val, cap, cap + 1, 0.1, out=out)
    with pytest.raises(pssa_b200.B200Error, match="refusing launch"):
        gpu.memory_forward(*case, T, d_m, d_k, d_val, cap, count, 0.0, out=out)
    assert all((v == 7.0).all() for v in out.values())


def test_resident_ssm_then_memory_stage(gpu):
    import pssa_b200
    T, d_m, d_s, d_k, cap = 33, 24, 8, 8, 16
    rng = np.random.default_rng(3)
    delta = np.log1p(np.exp(rng.normal(-2.0, 1.0, (T, d_m)))).astype(np.float32)
    bp, cp = rng.normal(0, 1, (T, d_s)).astype(np.float32), rng.normal(0, 1, (T, d_s)).astype(np.float32)
    _, _, w_qx, w_qh, w_gate, w_proj, keys, norm_sq, values = _case(T, d_m, d_k, d_m, cap, cap, seed=4)
    x = rng.normal(0, 1, (T, d_m)).astype(np.float32)
    rates = -np.exp(rng.uniform(np.log(0.005), np.log(0.7), d_m * d_s)).astype(np.float32)
    h0 = rng.normal(0, 1, d_m * d_s).astype(np.float32)
    mem_args = (x, w_qx, w_qh, w_gate, w_proj, keys, norm_sq, values)
    # nothing resident yet: the reference's message (src/cuda/stages.rs:714)
    with pytest.raises(pssa_b200.B200Error, match="SSM result is not resident"):
        gpu.memory_forward_after_ssm(*mem_args, T, d_m, d_s, d_k, d_m, cap, cap, 0.1)
    gpu.ssm_forward_resident(delta, bp, x, rates, cp, h0, T, d_m, d_s, exact=True)
    with pytest.raises(pssa_b200.B200Error, match="resident SSM shape mismatch"):  # src/cuda/stages.rs:733-735
        gpu.memory_forward_after_ssm(x[:-1], *mem_args[1:], T - 1, d_m, d_s, d_k, d_m, cap, cap, 0.1)
    tape, got = gpu.memory_forward_after_ssm(*mem_args, T, d_m, d_s, d_k, d_m, cap, cap, 0.1)
    ref_states, ref_y, ref_a, ref_b = O.ssm_forward(delta, bp, cp, x, rates, h0, mode=0)
    assert np.array_equal(tape["states"][0], h0)
    assert chan_err(tape["states"], ref_states, 0) <= 5e-6 and chan_err(tape["y_ssm"], ref_y, 0) <= 5e-6
    assert np.array_equal(tape["bar_b"].view(np.uint32), ref_b.view(np.uint32))
    assert float(np.max(np.abs(tape["bar_a"] - ref_a) / np.maximum(1e-6, np.abs(ref_a)))) <= 2e-7
    want = gpu.memory_forward(x, tape["y_ssm"], *mem_args[1:], T, d_m, d_k, d_m, cap, cap, 0.1)
    for name in want:
        assert np.array_equal(got[name], want[name]), name
    ref = _oracle_memory_stage(x, ref_y, w_qx, w_qh, w_gate, w_proj, keys, norm_sq, values, cap, 0.1)
    for name, w in ref.items():
        assert float(np.max(np.abs(got[name] - w))) / max(1e-6, float(np.abs(w).max())) <= 2e-5, name
    # consumed: a second call finds nothing resident
    with pytest.raises(pssa_b200.B200Error, match="SSM result is not resident"):
        gpu.memory_forward_after_ssm(*mem_args, T, d_m, d_s, d_k, d_m, cap, cap, 0.1)
