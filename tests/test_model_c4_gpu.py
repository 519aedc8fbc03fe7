"""Parity of the GPU path with the CPU oracle on the configuration the benchmark times: the stacked 12-block model
(d 768, state 64, key 64, 512 full slots, vocabulary 16384) over 2048-token sequences, in both precisions, with the
all-slots read and with memory top-8; plus one long recurrence (8192 tokens through 2 blocks at d 768) that takes the
time-chunked SSM path. The reference proves prefill == token loop up to 1024 tokens (src/inference.rs:1069-1113) and
token inference == chunk forward for stacked depth (tests/stacked_depth.rs:296-317); the oracle here is the
token-serial restatement, one host thread per lane (about a minute on the GPU box's host cores).
"""
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import pytest

import oracle as O
from parity import scale_err

pytestmark = pytest.mark.gpu

T = 2048
LANES = 4          # all-slots lanes
TOPK_LANES = 2     # lanes re-run with memory top-8
LONG_T = 8192


def _greedy(row):
    return int(O.lib().pssa_oracle_greedy(O.fptr(np.ascontiguousarray(row, np.float32)), row.size))


def _gap(row):
    order = np.sort(row[1:])
    return float(order[-1] - order[-2])


@pytest.fixture(scope="module")
def c4():
    """The benchmark's model (same generator and seed as bench.py) and the oracle's results for every case."""
    import bench
    tensors, banks = bench.synth_weights(1234)
    om = bench.oracle_model(tensors, banks)
    ids = np.random.default_rng(100).integers(1, bench.CFG["d_vocab"], (bench.LANES, T)).astype(np.uint64)[:LANES]
    long_ids = np.random.default_rng(101).integers(1, bench.CFG["d_vocab"], LONG_T).astype(np.uint64)
    # the 2-block model of the long recurrence: blocks 0 and 1 of the same weights
    cfg2 = dict(bench.CFG, depth=2)
    om2 = O.Model.new(2, cfg2["d_vocab"], cfg2["d_latent"], cfg2["d_state"], cfg2["d_mem_key"], cfg2["mem_capacity"], tau_mem=0.1, seed=1)
    for (layer, tid), arr in tensors.items():
        if layer < 2:
            om2.tensor(layer, tid)[:] = arr.ravel()
    for l in range(2):
        keys, norm_sq, values = banks[l]
        om2.tensor(l, O.BANK_KEYS)[:] = keys.ravel()
        om2.tensor(l, O.BANK_NORM_SQ)[:] = norm_sq
        om2.tensor(l, O.BANK_VALUES)[:] = values.ravel()
        om2.set_bank_meta(l, cfg2["mem_capacity"], 0)

    def run(model, seq, top_k):
        m = model.clone()
        if top_k:
            for l in range(m.depth):
                c, h, _ = m.bank_meta(l)
                m.set_bank_meta(l, c, h, top_k)
        m.reset_recurrent_state()
        rc, done, logits = m.prefill_inference(seq)
        assert rc == 1 and done == len(seq)
        scratch = [(m.tensor(l, O.S_MEM_WEIGHTS).copy(), m.tensor(l, O.S_Q_PNC).copy()) for l in range(m.depth)]
        return logits, m.state().copy(), scratch

    jobs = [(om, ids[l], 0) for l in range(LANES)] + [(om, ids[l], 8) for l in range(TOPK_LANES)] + [(om2, long_ids, 0)]
    with ThreadPoolExecutor(len(jobs)) as pool:  # the oracle's C entry points run without the interpreter lock
        res = list(pool.map(lambda j: run(*j), jobs))
    return dict(bench=bench, tensors=tensors, banks=banks, ids=ids, long_ids=long_ids, full=res[:LANES],
                top8=res[LANES:LANES + TOPK_LANES], long=res[-1])


@pytest.fixture(scope="module")
def gpu():
    import pssa_b200
    d = pssa_b200.B200Dispatch(0)
    yield d
    d.close()


def _gpu_model(gpu, c4, precision, depth=12, streams=LANES):
    import pssa_b200
    cfg = dict(c4["bench"].CFG, depth=depth)
    gm = pssa_b200.PSSAModel(gpu, tau_mem=0.1, streams=streams, precision=precision, **cfg)
    for (layer, tid), arr in c4["tensors"].items():
        if layer < depth:
            gm.set_tensor(layer, tid, arr)
    for l in range(depth):  # residual scales keep the default 1/sqrt(depth) on both sides (src/pssa.rs:2059)
        keys, norm_sq, values = c4["banks"][l]
        gm.set_bank(l, keys, norm_sq, values, cfg["mem_capacity"])
    return gm


def _check_fp32(logits, states, want, tol=1e-5):
    for l, (ref_logits, ref_state, _) in enumerate(want):
        assert scale_err(logits[l], ref_logits) <= tol, f"lane {l}: last-token logits after {T} tokens"
        s_scale = max(1.0, float(np.abs(ref_state).max()))
        assert float(np.max(np.abs(states[l] - ref_state))) / s_scale <= tol, f"lane {l}: final recurrent state"
        assert int(np.argmax(logits[l][1:]) + 1) == _greedy(ref_logits) or _gap(ref_logits) <= 2 * tol * float(np.abs(ref_logits).max())


def _distances_f64(p, keys):
    """Poincare distances of one projected query to every key in f64 (src/memory.rs:245-262), for measuring near-ties."""
    p, keys = p.astype(np.float64), keys.astype(np.float64)
    u = ((p - keys) ** 2).sum(1) / ((1.0 - (p ** 2).sum()) * (1.0 - (keys ** 2).sum(1)))
    return 2.0 * np.arcsinh(np.sqrt(u))


def _check_bf16(logits, want, record):
    errs, gaps = [], []
    for l, (ref_logits, _, _) in enumerate(want):
        err = float(np.max(np.abs(logits[l] - ref_logits)))
        gap = _gap(ref_logits)
        errs.append(err), gaps.append(gap)
        assert err <= 2e-2, f"lane {l}: max |logit difference| {err} after {T} tokens through 12 blocks"
        if gap > 2 * err:
            assert int(np.argmax(logits[l][1:]) + 1) == _greedy(ref_logits), f"lane {l}: greedy token (gap {gap}, error {err})"
    record(max_abs_logit_err=max(errs), min_top2_gap=min(gaps), logit_scale=float(max(np.abs(w[0]).max() for w in want)))


def test_fp32_mode_at_the_benchmark_configuration(gpu, c4):
    gm = _gpu_model(gpu, c4, precision=1)
    logits, _ = gm.prefill_batch([list(x) for x in c4["ids"]])
    _check_fp32(logits, [gm.copy_recurrent_state_to(l) for l in range(LANES)], c4["full"])
    gm.close()


def test_bf16_mode_at_the_benchmark_configuration(gpu, c4, record_property):
    gm = _gpu_model(gpu, c4, precision=0)
    logits, _ = gm.prefill_batch([list(x) for x in c4["ids"]])
    _check_bf16(logits, c4["full"], lambda **kw: [record_property(k, v) for k, v in kw.items()])
    # the recurrent state itself is fp32 arithmetic on bf16-projected inputs: same order of error as the logits
    for l, (_, ref_state, _) in enumerate(c4["full"]):
        s_scale = max(1.0, float(np.abs(ref_state).max()))
        assert float(np.max(np.abs(gm.copy_recurrent_state_to(l) - ref_state))) / s_scale <= 5e-2
    gm.close()


@pytest.mark.parametrize("precision", [1, 0])
def test_memory_top_8_on_the_model_path(gpu, c4, precision, record_property):
    """Top-8 read inside the 12-block model (the reference refuses this option on a GPU device, src/pssa.rs:2215-2218;
    only bank-level known answers exist there): logits and state against the oracle with top_k = 8, and the slots the
    last token of each lane selected in every block.

    Selection is a discontinuous function of the query: the fp32 mode's queries agree with the CPU's to about 1e-6, and
    over 2 x 2048 x 12 selections among 512 slots a few land where the 8th and 9th nearest slots are closer than that,
    so the two sides legitimately keep different slots there and the difference (two nearly equal weights on different
    values) travels on through the recurrent state. Given IDENTICAL queries the selection is identical (the operator
    tests in test_memory_gpu.py assert set equality). Here the fp32 bar is therefore 1e-3 of scale instead of 1e-5, and
    a last-token slot set may differ from the oracle's only where the oracle's own 8th/9th distances are a near-tie."""
    gm = _gpu_model(gpu, c4, precision=precision, streams=TOPK_LANES)
    gm.set_memory_top_k(8)
    gm.set_observer(True)
    logits, _ = gm.prefill_batch([list(x) for x in c4["ids"][:TOPK_LANES]])
    if precision == 1:
        _check_fp32(logits, [gm.copy_recurrent_state_to(l) for l in range(TOPK_LANES)], c4["top8"], tol=1e-3)
        record_property("fp32_top8_logit_scale_err", max(scale_err(logits[l], c4["top8"][l][0]) for l in range(TOPK_LANES)))
    else:
        _check_bf16(logits, c4["top8"], lambda **kw: [record_property(k, v) for k, v in kw.items()])
    same = total = 0
    for lane, (_, _, scratch) in enumerate(c4["top8"]):
        for l in range(12):
            w, q, _, _ = gm.observation(l, lane)
            ref_w, ref_q = scratch[l]
            assert np.count_nonzero(w) == 8 and np.count_nonzero(ref_w) == 8
            total += 1
            equal = np.array_equal(w != 0, ref_w != 0)
            same += int(equal)
            if precision == 1:
                # earlier flips have moved the state a little, so the last token's queries agree to 1e-3, not 1e-6
                dq = float(np.max(np.abs(q - ref_q)))
                assert dq <= 1e-3
                if not equal:  # only a near-tie at the selection boundary (on the scale of the query difference) may flip
                    dist = np.sort(_distances_f64(ref_q, c4["banks"][l][0]))
                    assert (dist[8] - dist[7]) <= 50 * dq, (lane, l, dq, dist[6:10])
    record_property("blocks_with_the_oracle_slot_set", f"{same}/{total}")
    if precision == 1:
        assert same >= total - 2
    gm.close()


@pytest.mark.parametrize("precision", [1, 0])
def test_long_recurrence_through_the_time_chunked_path(gpu, c4, precision):
    """One lane of 8192 tokens, 2 blocks at d 768: 12 CTAs cannot fill the GPU, so the SSM runs as time chunks (chunk
    maps, fold, second pass). Decays reach 0.999, so the state carries about a thousand steps of history."""
    gm = _gpu_model(gpu, c4, precision=precision, depth=2, streams=1)
    gpu.profile_begin()
    ok, logits = gm.prefill_inference(c4["long_ids"])
    rows = gpu.profile_end()
    assert ok and "seqpar_fold_kernel" in rows
    ref_logits, ref_state, _ = c4["long"]
    state = gm.copy_recurrent_state_to(0)
    s_scale = max(1.0, float(np.abs(ref_state).max()))
    if precision == 1:
        assert scale_err(logits, ref_logits) <= 1e-5
        assert float(np.max(np.abs(state - ref_state))) / s_scale <= 1e-5
    else:
        assert float(np.max(np.abs(logits - ref_logits))) <= 2e-2
        assert float(np.max(np.abs(state - ref_state))) / s_scale <= 5e-2
    gm.close()
