"""Parity of the dense products through the C ABI: the exact fp32 kernel against the reference's dot_slice bit
for bit, the bf16 tensor-core kernel against an fp32 product of the bf16-rounded operands."""
import numpy as np
import pytest

import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    import pssa_b200
    d = pssa_b200.B200Dispatch(0)
    yield d
    d.close()


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


@pytest.mark.parametrize("k", [1, 3, 4, 7, 8, 9, 15, 16, 17, 31, 32, 33, 40, 63, 64, 71, 100, 192, 257, 768])
def test_exact_gemm_is_dot_slice_bit_for_bit(gpu, k):
    # tests/backend.rs:84-100 (blocked GEMM == dot_slice bitwise) for every tail length of src/linalg.rs:184-298
    rng = np.random.default_rng(k)
    m, n = 9, 11
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = rng.standard_normal((n, k)).astype(np.float32)
    got = gpu.dispatch_gemm(x, w, m, n, k, 1).reshape(m, n)
    assert np.array_equal(bits(got), bits(O.gemm_xwt(x, w)))


def test_batch_folds_into_rows_and_bad_lengths_leave_output_untouched(gpu):
    # tests/backend.rs:9-82
    import pssa_b200
    rng = np.random.default_rng(0)
    b, m, n, k = 3, 5, 6, 24
    x = rng.standard_normal((b, m, k)).astype(np.float32)
    w = rng.standard_normal((n, k)).astype(np.float32)
    got = gpu.dispatch_gemm(x, w, m, n, k, b).reshape(b * m, n)
    assert np.array_equal(bits(got), bits(O.gemm_xwt(x.reshape(b * m, k), w)))
    out = np.full(b * m * n, 5.0, np.float32)
    for bad in (lambda: gpu.dispatch_gemm_into(x.ravel()[:-1].copy(), w, m, n, k, b, out),
                lambda: gpu.dispatch_gemm_into(x, w, m, n, k, b, out[:-1].copy()),
                lambda: gpu.dispatch_gemm_into(x, w, 0, n, k, b, out)):
        with pytest.raises(pssa_b200.B200Error):
            bad()
    assert np.all(out == 5.0)


def test_exact_epilogues_follow_the_reference_formulas(gpu):
    from pssa_b200 import _native as N
    rng = np.random.default_rng(1)
    m, n, k = 7, 33, 48
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = rng.standard_normal((n, k)).astype(np.float32)
    acc = O.gemm_xwt(x, w)
    sp = np.vectorize(O.lib().pssa_oracle_softplus)(acc).astype(np.float32)
    sg = np.vectorize(O.lib().pssa_oracle_sigmoid)(acc).astype(np.float32)
    got = gpu.dispatch_gemm(x, w, m, n, k, 1, epilogue=N.EPI_SOFTPLUS).reshape(m, n)
    assert np.max(np.abs(got - sp) / np.maximum(1e-6, np.abs(sp))) <= 3e-7
    got = gpu.dispatch_gemm(x, w, m, n, k, 1, epilogue=N.EPI_SIGMOID).reshape(m, n)
    assert np.max(np.abs(got - sg)) <= 2e-7
    got = gpu.dispatch_gemm(x, w, m, n, k, 1, epilogue=N.EPI_SCALE, alpha=0.25).reshape(m, n)
    assert np.array_equal(bits(got), bits(acc * np.float32(0.25)))
    prev = rng.standard_normal((m, n)).astype(np.float32)
    out = prev.copy().ravel()
    gpu.dispatch_gemm_into(x, w, m, n, k, 1, out, epilogue=N.EPI_ADD_OUT)
    assert np.array_equal(bits(out.reshape(m, n)), bits(prev + acc))


def bf16_round(a):
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7fff + ((u >> 16) & 1)) & 0xffff0000
    return u.astype(np.uint32).view(np.float32)


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (128, 64, 128), (1, 16, 8), (130, 200, 72), (257, 1744, 768), (300, 64, 768),
                                   (512, 768, 1536), (5, 4096, 192)])
def test_bf16_tensor_core_gemm(gpu, m, n, k):
    from pssa_b200 import _native as N
    rng = np.random.default_rng(m + n + k)
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    ref = bf16_round(x).astype(np.float64) @ bf16_round(w).astype(np.float64).T
    got = gpu.dispatch_gemm(x, w, m, n, k, 1, precision=N.PRECISION_BF16).reshape(m, n)
    gpu.poll_status()
    scale = np.abs(ref).max()
    assert np.max(np.abs(got - ref)) <= 2e-5 * scale + 1e-6  # fp32 accumulation of exact bf16 products
    # against the unrounded fp32 product the error is the bf16 operand rounding
    full = x.astype(np.float64) @ w.astype(np.float64).T
    assert np.max(np.abs(got - full)) <= 2e-2 * max(1.0, np.abs(full).max())


def test_bf16_gemm_epilogues_and_k_alignment(gpu):
    import pssa_b200
    from pssa_b200 import _native as N
    rng = np.random.default_rng(4)
    m, n, k = 200, 96, 64
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.2).astype(np.float32)
    acc = bf16_round(x).astype(np.float64) @ bf16_round(w).astype(np.float64).T
    got = gpu.dispatch_gemm(x, w, m, n, k, 1, precision=N.PRECISION_BF16, epilogue=N.EPI_SILU).reshape(m, n)
    assert np.max(np.abs(got - acc / (1 + np.exp(-acc)))) <= 1e-4
    got = gpu.dispatch_gemm(x, w, m, n, k, 1, precision=N.PRECISION_BF16, epilogue=N.EPI_SOFTPLUS).reshape(m, n)
    assert np.max(np.abs(got - np.log1p(np.exp(acc)))) <= 1e-4
    with pytest.raises(pssa_b200.B200Error) as e:
        gpu.dispatch_gemm(x[:, :60].copy(), w[:, :60].copy(), m, n, 60, 1, precision=N.PRECISION_BF16)
    assert e.value.status == 6 and "K % 8" in str(e.value)


@pytest.mark.parametrize("m,n,k", [(4096, 2304, 512), (3900, 2000, 264), (5000, 4104, 128)])
def test_bf16_gemm_as_cta_pairs(gpu, m, n, k):
    """Plain products with enough 256-row tiles for every pair of SMs run as clusters of two CTAs (cta_group::2: the
    even CTA issues the MMAs over both CTAs' operand halves). Full and ragged shapes (rows and columns that are not
    multiples of the 256 x 256 tile, an odd number of 128-row blocks, K that is not a multiple of the 64-wide K block)
    against an f64 product of the bf16-rounded operands; the profile shows which kernel ran."""
    from pssa_b200 import _native as N
    rng = np.random.default_rng(m + n + k)
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    ref = bf16_round(x).astype(np.float64) @ bf16_round(w).astype(np.float64).T
    got = gpu.dispatch_gemm(x, w, m, n, k, 1, precision=N.PRECISION_BF16).reshape(m, n)
    gpu.poll_status()
    scale = np.abs(ref).max()
    assert np.max(np.abs(got - ref)) <= 2e-5 * scale + 1e-6
