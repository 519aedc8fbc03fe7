"""Runtime Ouro passes (`set_loops`, src/pssa.rs:2171-2184, 2338-2376) on the GPU path against the CPU oracle: prefill,
token steps, carries in [block][pass][d*s] order, the reference's "first pass keeps the single-pass math" property
(tests/loops.rs:42-62) and the frozen-model scorer."""
import numpy as np
import pytest

import oracle as O
from helpers import fill_synthetic, upload
from parity import scale_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    import pssa_b200
    d = pssa_b200.B200Dispatch(0)
    yield d
    d.close()


def pair(gpu, depth, v, d, s, k, cap, seed, loops, precision=1, streams=1):
    import pssa_b200
    om = O.Model.new(depth, v, d, s, k, cap, tau_mem=0.1, seed=seed)
    fill_synthetic(om, seed)
    gm = pssa_b200.PSSAModel(gpu, depth, v, d, s, k, cap, tau_mem=0.1, streams=streams, precision=precision)
    upload(om, gm)
    om.set_loops(loops)
    gm.set_loops(loops)
    return om, gm


@pytest.mark.parametrize("depth,loops,v,d,s,k,cap,n", [(1, 2, 50, 16, 4, 4, 8, 9), (2, 3, 97, 32, 16, 8, 16, 40), (3, 2, 64, 40, 8, 12, 10, 33),
                                                       (1, 3, 300, 192, 64, 64, 64, 70)])
def test_fp32_prefill_token_steps_and_carries_match_the_oracle(gpu, depth, loops, v, d, s, k, cap, n):
    om, gm = pair(gpu, depth, v, d, s, k, cap, seed=depth * 10 + loops, loops=loops)
    assert gm.recurrent_state_len() == depth * loops * d * s
    ids = (np.arange(n) * 7 + 3) % v
    ok, logits = gm.prefill_inference(ids)
    _, _, ref = om.prefill_inference(ids)
    assert ok and scale_err(logits, ref) <= 1e-5
    st, ref_st = gm.copy_recurrent_state_to(), om.state()
    assert st.shape == ref_st.shape
    assert np.max(np.abs(st - ref_st)) <= 1e-5 * max(1.0, np.abs(ref_st).max())
    tok = int(np.argmax(ref[1:]) + 1)
    for _ in range(5):
        lg, gr = gm.decode_step([tok], [0], want_greedy=True)
        ref = om.forward_inference(tok)
        assert scale_err(lg[0], ref) <= 1e-5
        nxt = int(O.lib().pssa_oracle_greedy(O.fptr(ref), v))
        assert int(gr[0]) == nxt
        tok = nxt
    gm.close()


def test_first_pass_keeps_the_single_pass_math_and_set_loops_keeps_pass_zero(gpu):
    om1, gm1 = pair(gpu, 1, 61, 32, 8, 8, 12, seed=5, loops=1)
    om2, gm2 = pair(gpu, 1, 61, 32, 8, 8, 12, seed=5, loops=2)
    ids = (np.arange(50) * 3 + 2) % 61
    gm1.prefill_inference(ids)
    gm2.prefill_inference(ids)
    hs = 32 * 8
    s1, s2 = gm1.copy_recurrent_state_to(), gm2.copy_recurrent_state_to()
    assert np.array_equal(s2[:hs].view(np.uint32), s1.view(np.uint32))  # tests/loops.rs:42-62
    assert np.any(s2[hs:] != 0)
    gm2.set_loops(3)  # src/pssa.rs:2147-2167: a fresh tape, pass 0's carry survives
    s3 = gm2.copy_recurrent_state_to()
    assert s3.size == 3 * hs and np.array_equal(s3[:hs], s2[:hs]) and not s3[hs:].any()
    import pssa_b200
    with pytest.raises(pssa_b200.B200Error, match="--loops must be between 1 and 32"):
        gm2.set_loops(0)
    gm1.close()
    gm2.close()


def test_bf16_mode_lanes_and_scorer_with_passes(gpu):
    om, gm = pair(gpu, 2, 512, 192, 64, 64, 64, seed=21, loops=2, precision=0, streams=3)
    rng = np.random.default_rng(1)
    prompts = [rng.integers(1, 512, n) for n in (70, 9, 33)]
    logits, _ = gm.prefill_batch([list(p) for p in prompts])
    for j, p in enumerate(prompts):
        ref_m = om.clone()
        ref_m.reset_recurrent_state()
        _, _, ref = ref_m.prefill_inference(p)
        assert float(np.max(np.abs(logits[j] - ref))) <= 2e-2, j
    # scorer in the fp32 mode: every position's logits and the mean loss
    om2, gm2 = pair(gpu, 2, 97, 32, 16, 8, 16, seed=23, loops=3)
    ids = (np.arange(120) * 7 + 1) % 97
    targets = (ids * 3 + 5) % 97
    ref_loss, ref_logits = om2.chunk_forward(ids, targets)
    gm2.set_max_rows(50)  # three passes over the rows
    loss, per, got = gm2.score(ids, targets, want_logits=True)
    assert abs(loss - ref_loss) <= 1e-5 * abs(ref_loss) and scale_err(got, ref_logits) <= 1e-5
    assert np.max(np.abs(gm2.copy_recurrent_state_to(0) - om2.state())) <= 1e-5 * max(1.0, np.abs(om2.state()).max())
    gm.close()
    gm2.close()


def test_observer_publishes_the_last_pass(gpu):
    om, gm = pair(gpu, 2, 80, 48, 16, 16, 20, seed=17, loops=2)
    gm.set_observer(True)
    ids = (np.arange(23) * 7 + 2) % 80
    gm.prefill_inference(ids)
    om.prefill_inference(ids)
    for l in range(2):
        w, q, mv, z = gm.observation(l, 0)
        ref = [om.tensor(l, t).copy() for t in (O.S_MEM_WEIGHTS, O.S_Q_PNC, O.S_M_VAL, O.S_Z_FINAL)]
        for got, want, name in zip((w, q, mv, z), ref, ("weights", "q_pnc", "m_val", "z_final")):
            assert np.max(np.abs(got - want)) / max(1e-6, float(np.abs(want).max())) <= 1e-5, (l, name)
    gm.close()
