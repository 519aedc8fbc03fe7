"""Device-side sampling against the CPU restatement of the reference's `sample` (src/inference.rs:102-181)."""
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


def run(gpu, logits, recent, states, exact=True, **cfg):
    import torch
    rows, v = logits.shape
    lg = torch.from_numpy(logits.copy()).cuda()
    probs = torch.zeros(rows, v, device="cuda")
    rid = np.zeros((rows, 64), np.uint32)
    rcount = np.zeros(rows, np.uint32)
    for r, ids in enumerate(recent):
        ids = list(ids)[-64:]
        rid[r, :len(ids)] = ids
        rcount[r] = len(ids)
    st = torch.from_numpy(np.asarray(states, np.uint64).view(np.int64).copy()).cuda()
    out = torch.zeros(rows, dtype=torch.int32, device="cuda")
    status = torch.zeros(rows, dtype=torch.int32, device="cuda")
    conf = torch.zeros(rows, device="cuda")
    gpu.set_stream(torch.cuda.current_stream())
    gpu.sample_dev(lg, probs, rows, v, st, out, status, recent_ids=torch.from_numpy(rid.view(np.int32)).cuda(),
                   recent_count=torch.from_numpy(rcount.view(np.int32)).cuda(), exact=exact, confidence_out=conf, **cfg)
    torch.cuda.synchronize()
    gpu.set_stream(None)
    run.confidence = conf.cpu().numpy()
    return (out.cpu().numpy().view(np.uint32), status.cpu().numpy(), st.cpu().numpy().view(np.uint64), lg.cpu().numpy())


CONFIGS = [dict(temperature=0.70, top_p=0.85, top_k=24, repetition_penalty=1.25),   # the reference's defaults
           dict(temperature=0.0, top_p=1.0, top_k=1, repetition_penalty=1.0),       # greedy
           dict(temperature=1.3, top_p=1.0, top_k=4096, repetition_penalty=1.0),    # wide open
           dict(temperature=0.05, top_p=0.5, top_k=3, repetition_penalty=2.0),
           dict(temperature=1e-6, top_p=0.9, top_k=10, repetition_penalty=1.1)]


@pytest.mark.parametrize("cfg", CONFIGS)
@pytest.mark.parametrize("v", [2, 50, 1000, 16384])
def test_sampled_ids_rng_state_and_penalised_logits_match_the_restatement(gpu, cfg, v):
    rng = np.random.default_rng(v)
    rows = 24
    logits = (rng.standard_normal((rows, v)) * rng.uniform(0.1, 6.0, (rows, 1))).astype(np.float32)
    logits[3, : min(v, 9)] = 1.5  # exact ties
    logits[4] = 0.0               # all equal: id 1 in the greedy rule
    recent = [rng.integers(0, v, rng.integers(0, 90)).tolist() for _ in range(rows)]
    recent[5] = [min(7, v - 1)] * 80  # one id repeated through the whole window
    states = rng.integers(1, 2**63, rows, dtype=np.uint64)
    ids, status, new_states, lg_after = run(gpu, logits, recent, states, **cfg)
    # raw confidence: softmax of the UNpenalised logits over all ids, at the selected id (src/inference.rs:526-545)
    raw = np.exp(logits - logits.max(1, keepdims=True)).astype(np.float32)
    raw /= np.cumsum(raw, axis=1, dtype=np.float32)[:, -1:]  # the reference sums in id order
    assert np.max(np.abs(run.confidence - raw[np.arange(rows), ids.astype(np.int64)])) <= 1e-6
    mismatches = 0
    for r in range(rows):
        ref_id, ref_state, ref_lg = O.sample(int(states[r]), logits[r], recent[r], **cfg)
        assert status[r] == 0 and ref_id >= 0
        assert np.array_equal(lg_after[r].view(np.uint32), ref_lg.view(np.uint32)), "penalty differs"
        assert int(new_states[r]) == ref_state, "rng stream differs"
        if int(ids[r]) != ref_id:
            mismatches += 1
    # CUDA expf and glibc expf may differ in the last bit of a probability; a draw that lands within that of a boundary
    # can then fall on the neighbouring candidate. With 24 streams that should be rare.
    assert mismatches <= 1, mismatches


def test_errors_and_validation(gpu):
    import pssa_b200
    v = 64
    logits = np.zeros((3, v), np.float32)
    logits[1, 5] = np.inf
    logits[2, 0] = np.nan  # id 0 is not a candidate, but a non-finite logit anywhere is an error
    ids, status, _, _ = run(gpu, logits, [[], [], []], [1, 2, 3], temperature=0.7, top_p=0.9, top_k=5, repetition_penalty=1.0)
    assert ids[0] == 1 or 1 <= ids[0] < v
    assert status.tolist() == [0, 1, 1] and ids[1] == 0xFFFFFFFF and ids[2] == 0xFFFFFFFF
    for bad, msg in ((dict(temperature=-1.0), "temperature must be finite"), (dict(top_p=0.0), "top-p must be finite in"),
                     (dict(top_k=0), "top-k must be positive"), (dict(repetition_penalty=0.5), "repetition penalty must be finite")):
        cfg = dict(temperature=0.7, top_p=0.9, top_k=5, repetition_penalty=1.0)
        cfg.update(bad)
        with pytest.raises(pssa_b200.B200Error, match=msg):
            run(gpu, logits[:1], [[]], [1], **cfg)


def test_fast_sum_mode_keeps_the_distribution(gpu):
    """Without the sequential sum the chosen ids may differ only where the draw sits on a boundary."""
    rng = np.random.default_rng(1)
    rows, v = 64, 16384
    logits = (rng.standard_normal((rows, v)) * 3).astype(np.float32)
    states = rng.integers(1, 2**63, rows, dtype=np.uint64)
    cfg = dict(temperature=0.8, top_p=0.95, top_k=40, repetition_penalty=1.0)
    a = run(gpu, logits, [[]] * rows, states, exact=True, **cfg)
    b = run(gpu, logits, [[]] * rows, states, exact=False, **cfg)
    assert np.array_equal(a[2], b[2]) and int(np.sum(a[0] != b[0])) <= 1


def test_model_level_sampled_decode_follows_the_restatement(gpu):
    """Forward + head + sampling on the device, ids only back to the host: two streams with their own generators and
    repetition windows follow the CPU model sampled by the restatement with the same seeds."""
    import pssa_b200
    from helpers import fill_synthetic, upload
    v = 300
    om = O.Model.new(2, v, 48, 16, 16, 20, tau_mem=0.1, seed=8)
    fill_synthetic(om, 8, std=0.3)  # wide logits so the distribution is far from uniform
    gm = pssa_b200.PSSAModel(gpu, 2, v, 48, 16, 16, 20, tau_mem=0.1, streams=2, precision=1)
    upload(om, gm)
    cfg = dict(temperature=0.9, top_p=0.9, top_k=12, repetition_penalty=1.3)
    oms = [om.clone(), om.clone()]
    seeds = [1337, 99]
    gm.sampler_seed(0, seeds[0])
    gm.sampler_seed(1, seeds[1])
    prompts = [np.array([5, 9, 2, 77]), np.array([11, 3])]
    gm.prefill_batch([list(p) for p in prompts], want_logits=False)
    states = list(seeds)
    history = [[], []]
    for s_, p_ in enumerate(prompts):  # the CPU replicas consume the same prompts
        oms[s_].reset_recurrent_state()
        oms[s_].prefill_inference(p_)
    # both sides then decode from the same fixed tokens
    toks = [7, 8]
    mismatches = 0
    for step in range(24):
        got, conf = gm.decode_step_sampled(toks, [0, 1], exact=True, want_confidence=True, **cfg)
        nxt = []
        for s in range(2):
            lg = oms[s].forward_inference(toks[s])
            raw = np.exp(lg - lg.max())
            # logits of magnitude ~100 here: the 1e-5 relative agreement of the logits becomes ~1e-4 on a probability
            assert abs(float(conf[s]) - float(raw[int(got[s])] / raw.sum())) <= 2e-4
            ref_id, states[s], _ = O.sample(states[s], lg, history[s], **cfg)
            if int(got[s]) != ref_id:
                mismatches += 1
            history[s].append(int(got[s]))  # follow the device's choice so the two sides stay on one sequence
            nxt.append(int(got[s]))
        toks = nxt
    assert mismatches <= 1, mismatches
    assert len(set(history[0])) > 3  # it really samples
    # an id repeated in the window is what the penalty sees: windows are per stream
    with pytest.raises(pssa_b200.B200Error, match="top-p must be finite"):
        gm.decode_step_sampled(toks, [0, 1], top_p=1.5)
    gm.close()


def test_generate_loop_follows_the_engine_order_with_the_prompt_in_the_repetition_window(gpu):
    """`PSSAModel.generate`: reset, seed, the PROMPT heads the repetition window (`generated_ids` starts as a copy of it,
    src/inference.rs:343-345), prefill, then forward + sample per step. The CPU side replays the engine's loop with the
    restatement of `sample` on the oracle's logits, following the device's choice after each step so that a draw landing
    within an ulp of a candidate boundary cannot fork the two sequences."""
    import pssa_b200
    from helpers import fill_synthetic, upload
    v = 200
    om = O.Model.new(2, v, 48, 16, 16, 20, tau_mem=0.1, seed=5)
    fill_synthetic(om, 5, std=0.3)
    gm = pssa_b200.PSSAModel(gpu, 2, v, 48, 16, 16, 20, tau_mem=0.1, streams=1, precision=1)
    upload(om, gm)
    cfg = dict(temperature=0.9, top_p=0.9, top_k=12, repetition_penalty=1.4)
    prompt = [5, 9, 2, 77, 9, 9, 31]
    ref = om.clone()
    ref.reset_recurrent_state()
    _, _, logits = ref.prefill_inference(prompt)
    state = {"rng": 4242, "logits": logits, "history": list(prompt), "mismatch": 0, "calls": 0, "prob_err": 0.0}

    def on_token(count, previous, selected, probability):
        state["calls"] += 1
        assert count == state["calls"] and previous == state["history"][-1]
        lg = state["logits"].copy()
        raw = np.exp(lg - lg.max())
        state["prob_err"] = max(state["prob_err"], abs(probability - float(raw[selected] / raw.sum())))
        ref_id, state["rng"], _ = O.sample(state["rng"], lg, state["history"], **cfg)
        state["mismatch"] += int(ref_id != selected)
        state["history"].append(int(selected))
        state["logits"] = ref.forward_inference(int(selected))

    ids, probs = gm.generate(prompt, max_new_tokens=24, seed=4242, on_token=on_token, scored=True, exact=True, **cfg)
    assert len(ids) == 24 and state["calls"] == 24 and state["mismatch"] <= 1 and state["prob_err"] <= 2e-4
    assert list(ids) == state["history"][len(prompt):] and probs.shape == (24,)
    # the prompt really is in the window: without it the penalised logits of the first step, and so the ids, differ
    gm.reset_recurrent_state(0)
    gm.sampler_seed(0, 4242)
    gm.prefill_inference(prompt[:-1], want_logits=False)
    first_without = int(gm.decode_step_sampled([prompt[-1]], [0], exact=True, **dict(cfg, temperature=0.0))[0])
    gm.reset_recurrent_state(0)
    gm.sampler_seed(0, 4242)
    gm.sampler_push(prompt, 0)
    gm.prefill_inference(prompt[:-1], want_logits=False)
    first_with = int(gm.decode_step_sampled([prompt[-1]], [0], exact=True, **dict(cfg, temperature=0.0))[0])
    lg = logits.copy()
    greedy_plain = int(np.argmax(lg[1:]) + 1)
    pen = lg.copy()
    for t in prompt[-64:]:
        pen[t] = pen[t] / cfg["repetition_penalty"] if pen[t] > 0 else pen[t] * cfg["repetition_penalty"]
    assert first_without == greedy_plain and first_with == int(np.argmax(pen[1:]) + 1)
    # cancellation before the first step returns nothing; ids outside the vocabulary are refused when pushed
    ids, _ = gm.generate(prompt, max_new_tokens=5, cancelled=lambda: True)
    assert len(ids) == 0
    with pytest.raises(pssa_b200.B200Error, match="outside model vocabulary"):
        gm.sampler_push([v + 3], 0)
    gm.close()
