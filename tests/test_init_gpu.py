"""Random initialisation inside the library (`pssa_b200_model_init_random`): the tensors of `PSSALayerV2::new(cfg, seed)`
bit for bit. Pinned to the reference's own vector: its initial V7 fixture (seed 192) read by the library's checkpoint
reader must hold exactly the tensors the library draws itself; stacked depth (the head is drawn before the further
blocks, src/pssa.rs:2019-2072) is checked against the oracle, which reproduces the same fixture."""
import pathlib

import numpy as np
import pytest

import oracle as O

pytestmark = pytest.mark.gpu

GOLDEN = pathlib.Path(__file__).parent / "golden"
BLOCK_TENSORS = ("NORM_GAMMA", "NORM_BETA", "A_MAT", "W_DELTA", "W_B", "W_C", "W_QX", "W_QH", "W_GATE", "W_PROJ", "MLP_W1", "MLP_W2",
                 "AD_DOWN", "AD_UP", "AD_CONS")


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


@pytest.fixture(scope="module")
def gpu():
    import pssa_b200
    d = pssa_b200.B200Dispatch(0)
    yield d
    d.close()


def _lengths(cfg):
    d, s, k, v = cfg["d_latent"], cfg["d_state"], cfg["d_mem_key"], cfg["d_vocab"]
    return dict(EMBED=v * d, UNEMBED=v * d, NORM_GAMMA=d, NORM_BETA=d, A_MAT=d * s, W_DELTA=d * d, W_B=s * d, W_C=s * d, W_QX=k * d,
                W_QH=k * d, W_GATE=d * d, W_PROJ=d * d, MLP_W1=2 * d * d, MLP_W2=2 * d * d, AD_DOWN=16 * d, AD_UP=16 * d, AD_CONS=16 * d)


def test_init_equals_the_reference_initial_checkpoint(gpu):
    import pssa_b200
    from pssa_b200 import _native as N
    from pssa_b200 import model as M
    data = (GOLDEN / "depth_one_main85d9d33_initial.pssa").read_bytes()
    ref = pssa_b200.PSSAModel.from_checkpoint(gpu, data, precision=N.PRECISION_FP32_EXACT)
    cfg, _ = pssa_b200.PSSAModel.probe_checkpoint(data)
    own = pssa_b200.PSSAModel(gpu, cfg["depth"], cfg["d_vocab"], cfg["d_latent"], cfg["d_state"], cfg["d_mem_key"], cfg["mem_capacity"],
                              tau_mem=cfg["tau_mem"], streams=1, precision=N.PRECISION_FP32_EXACT)
    own.init_random(192)  # the fixture's seed (tests/depth_one_reference.rs)
    lens = _lengths(cfg)
    # every randomly initialised tensor of the fixture (its recipe, tests/depth_one_reference.rs, afterwards fills the
    # MLP's second matrix and the adapter's up matrices with a fixed pattern: those are not part of the init)
    drawn = [n for n in BLOCK_TENSORS if n not in ("MLP_W2", "AD_UP", "AD_CONS")]
    for name in ["EMBED", "UNEMBED"] + drawn:
        tid = getattr(M, name)
        assert np.array_equal(bits(own.get_tensor(0, tid, lens[name])), bits(ref.get_tensor(0, tid, lens[name]))), name
    own.close()
    ref.close()


@pytest.mark.parametrize("seed", [192, 0, 7])
def test_stacked_init_draw_order_and_generator_state(gpu, seed):
    import pssa_b200
    from pssa_b200 import _native as N
    from pssa_b200 import model as M
    cfg = dict(depth=3, d_vocab=37, d_latent=24, d_state=8, d_mem_key=8, mem_capacity=16)
    om = O.Model.new(cfg["depth"], cfg["d_vocab"], cfg["d_latent"], cfg["d_state"], cfg["d_mem_key"], cfg["mem_capacity"], tau_mem=0.1,
                     seed=seed)
    gm = pssa_b200.PSSAModel(gpu, tau_mem=0.1, streams=1, precision=N.PRECISION_FP32_EXACT, **cfg)
    state = gm.init_random(seed)
    assert state == om.rng_state
    lens = _lengths(cfg)
    for name in ("EMBED", "UNEMBED"):
        assert np.array_equal(bits(gm.get_tensor(0, getattr(M, name), lens[name])), bits(om.tensor(-1, getattr(O, name)))), name
    for layer in range(cfg["depth"]):
        for name in BLOCK_TENSORS:
            got = gm.get_tensor(layer, getattr(M, name), lens[name])
            assert np.array_equal(bits(got), bits(om.tensor(layer, getattr(O, name)))), (layer, name)
    scales = gm.get_tensor(0, M.RESIDUAL_SCALES, cfg["depth"] - 1)
    assert np.array_equal(bits(scales), bits(np.full(cfg["depth"] - 1, np.float32(1.0) / np.sqrt(np.float32(cfg["depth"])), np.float32)))
    # a freshly initialised model runs: first-token logits equal the oracle's in the exact mode
    ok, logits = gm.prefill_inference([3, 5, 2])
    rc, done, ref_logits = om.prefill_inference([3, 5, 2])
    assert ok and rc == 1 and np.max(np.abs(logits - ref_logits)) <= 1e-5 * max(1.0, float(np.abs(ref_logits).max()))
    gm.close()
