"""End-to-end parity of prefill and decode with the CPU oracle, through the C ABI's device-resident model."""
import numpy as np
import pytest

import oracle as O
from helpers import fill_synthetic, upload
from parity import rel_err, scale_err

pytestmark = pytest.mark.gpu

N_ERR_TOKEN = 7  # PSSA_B200_ERR_TOKEN


@pytest.fixture(scope="module")
def gpu():
    import pssa_b200
    d = pssa_b200.B200Dispatch(0)
    yield d
    d.close()


def make_pair(gpu, depth, v, d, s, k, cap, seed, streams=1, bank_fill=1.0, precision=1, tau=0.1):
    import pssa_b200
    om = O.Model.new(depth, v, d, s, k, cap, tau_mem=tau, seed=seed)
    fill_synthetic(om, seed, bank_fill)
    gm = pssa_b200.PSSAModel(gpu, depth, v, d, s, k, cap, tau_mem=tau, streams=streams, precision=precision)
    upload(om, gm)
    return om, gm


def test_golden_fixture_logits_through_the_gpu_model(gpu, golden_dir):
    """The reference's own golden rows (tests/depth_one_parity.rs, AVX2 set words [1,22)) on the GPU path in fp32."""
    import pssa_b200
    om = O.Model.load((golden_dir / "depth_one_main85d9d33_initial.pssa").read_bytes())
    obs = np.frombuffer((golden_dir / "depth_one_main014f617_avx2_observed.bin").read_bytes(), np.uint32)[1:22]
    want = obs.view(np.float32).reshape(3, 7)
    gm = pssa_b200.PSSAModel(gpu, 1, 7, 4, 2, 2, 3, tau_mem=om.tau_mem, precision=1)
    upload(om, gm)
    rows = [gm.forward_inference(t) for t in (1, 2, 1)]
    assert scale_err(np.stack(rows), want) <= 1e-5 and rel_err(np.stack(rows), want) <= 1e-4


@pytest.mark.parametrize("depth,v,d,s,k,cap,n", [(1, 50, 16, 4, 4, 8, 5), (2, 97, 32, 16, 8, 16, 40), (1, 300, 192, 64, 64, 64, 70),
                                                 (3, 64, 40, 8, 12, 10, 33), (4, 128, 64, 64, 32, 32, 17)])
def test_fp32_prefill_and_token_loop_match_the_oracle(gpu, depth, v, d, s, k, cap, n):
    om, gm = make_pair(gpu, depth, v, d, s, k, cap, seed=depth * 100 + d)
    ids = (np.arange(n) * 7 + 3) % v
    ok, logits = gm.prefill_inference(ids)
    rc, done, ref = om.prefill_inference(ids)
    assert ok and rc == 1 and gm.processed == n
    assert scale_err(logits, ref) <= 1e-5, "last-token logits"
    st = gm.copy_recurrent_state_to()
    assert np.max(np.abs(st - om.state())) <= 1e-5 * max(1.0, np.abs(om.state()).max())
    # decode continues from the prefilled carry; greedy tokens agree
    tok = int(np.argmax(ref[1:]) + 1)
    for _ in range(6):
        lg, gr = gm.decode_step([tok], [0], want_greedy=True)
        ref = om.forward_inference(tok)
        assert scale_err(lg[0], ref) <= 1e-5
        nxt = int(O.lib().pssa_oracle_greedy(O.fptr(ref), v))
        assert int(gr[0]) == nxt
        tok = nxt


def test_prefill_equals_token_loop_on_the_gpu(gpu):
    # src/inference.rs:1069-1113: prefill == decode loop, with a non-reset carry
    om, gm = make_pair(gpu, 2, 61, 32, 8, 8, 12, seed=9, streams=2)
    ids = (np.arange(67) * 5 + 1) % 61
    gm.copy_recurrent_state_from(om.state(), 1)
    _, a = gm.prefill_inference(ids, stream=0)
    for t in ids:
        b = gm.forward_inference(int(t), stream=1)
    assert scale_err(a, b) <= 1e-6
    assert np.max(np.abs(gm.copy_recurrent_state_to(0) - gm.copy_recurrent_state_to(1))) <= 1e-6


def test_independent_lanes_ragged_with_partial_bank_and_top_k(gpu):
    om, gm = make_pair(gpu, 2, 80, 48, 16, 16, 20, seed=4, streams=4, bank_fill=0.6)
    lanes = [list((np.arange(n) * 3 + j) % 80) for j, n in enumerate([9, 0, 31, 1])]
    for top_k in (None, 3):
        if top_k:
            gm.set_memory_top_k(top_k)
            for l in range(2):
                c, h, _ = om.bank_meta(l)
                om.set_bank_meta(l, c, h, top_k)
        gm.reset_recurrent_state()
        logits, greedy = gm.prefill_batch(lanes, want_greedy=True)
        for j, lane in enumerate(lanes):
            if not lane:
                assert not logits[j].any()
                continue
            ref_m = om.clone()
            ref_m.reset_recurrent_state()
            _, _, ref = ref_m.prefill_inference(lane)
            assert scale_err(logits[j], ref) <= 1e-5, (top_k, j)
            assert int(greedy[j]) == int(O.lib().pssa_oracle_greedy(O.fptr(ref), 80))
            assert np.max(np.abs(gm.copy_recurrent_state_to(j) - ref_m.state())) <= 1e-5


def test_passes_split_long_prompts_without_changing_results(gpu):
    om, gm = make_pair(gpu, 2, 40, 24, 8, 8, 8, seed=2, streams=2)
    ids = (np.arange(100) * 11) % 40
    _, a = gm.prefill_inference(ids, stream=0)
    gm.set_max_rows(16)
    _, b = gm.prefill_inference(ids, stream=1)
    gm.set_max_rows(65536)
    assert np.array_equal(a, b)
    assert np.array_equal(gm.copy_recurrent_state_to(0), gm.copy_recurrent_state_to(1))


def test_error_semantics_follow_the_reference(gpu):
    import pssa_b200
    om, gm = make_pair(gpu, 1, 30, 16, 4, 4, 4, seed=3)
    with pytest.raises(pssa_b200.B200Error, match="at least one token"):  # src/pssa.rs:2405-2407
        gm.prefill_inference([])
    before = gm.copy_recurrent_state_to()
    with pytest.raises(pssa_b200.B200Error, match="prompt ID 99 outside model vocabulary") as e:
        gm.prefill_inference([3, 4, 99, 5])
    assert e.value.status == 7 and gm.processed == 2
    ref = om.clone()
    ref.prefill_inference([3, 4], want_logits=False)
    assert np.max(np.abs(gm.copy_recurrent_state_to() - ref.state())) <= 1e-6 and not np.array_equal(before, ref.state())
    calls = []
    gm.set_max_rows(4)
    done, lg = gm.prefill_inference(np.arange(12) % 30, cancelled=lambda: len(calls) >= 2 or calls.append(1))
    gm.set_max_rows(65536)
    assert done is False and lg is None and gm.processed == 8  # two passes of 4 ran before the third poll cancelled
    for fn, msg in ((lambda: gm.set_local_conv(True), "local mixing experiments require CPU"),
                    (lambda: gm.set_hybrid_read(True, 0.5), "hybrid read currently requires the CPU backend"),
                    (lambda: gm.grow_memory(64), "grow memory on the CPU checkpoint"),
                    (lambda: gm.set_memory_top_k(0), "memory top-k must be positive")):
        with pytest.raises(pssa_b200.B200Error, match=msg):
            fn()
    with pytest.raises(pssa_b200.B200Error, match="outside model vocabulary"):
        gm.forward_inference(30)


def test_bf16_path_logits_within_tolerance_and_greedy_tokens(gpu):
    """bf16 projections, fp32 scan and retrieval: logits within 2e-2 max-abs of the fp32 CPU reference; greedy
    tokens identical wherever the reference's top-1/top-2 gap exceeds twice the observed error."""
    om, gm = make_pair(gpu, 2, 512, 192, 64, 64, 64, seed=21, precision=0)
    ids = (np.arange(96) * 37 + 5) % 512
    ok, logits = gm.prefill_inference(ids)
    _, _, ref = om.prefill_inference(ids)
    err = float(np.max(np.abs(logits - ref)))
    assert err <= 2e-2, err
    tok = int(O.lib().pssa_oracle_greedy(O.fptr(ref), 512))
    agree = total = 0
    for _ in range(24):
        lg, gr = gm.decode_step([tok], [0], want_greedy=True)
        ref = om.forward_inference(tok)
        e = float(np.max(np.abs(lg[0] - ref)))
        assert e <= 2e-2
        order = np.sort(ref[1:])
        nxt = int(O.lib().pssa_oracle_greedy(O.fptr(ref), 512))
        if order[-1] - order[-2] > 2 * e:
            total += 1
            agree += int(gr[0]) == nxt
        tok = nxt
    assert agree == total


def test_a_stream_decodes_the_same_alone_and_inside_a_large_batch(gpu):
    """Kernel choices (tile shapes, the one-launch front end of a decode step's read) follow the shape of the step,
    never the number of rows in it in a way that changes arithmetic: the first 8 of 96 streams, run as a batch of 8
    on a second model with the same weights, give bit-identical logits after the 16-token prompts (1536 rows against
    128) and after every one of 12 greedy steps (96 rows against 8)."""
    import pssa_b200
    om, big = make_pair(gpu, 2, 512, 192, 64, 64, 64, seed=33, streams=96, precision=0)
    small = pssa_b200.PSSAModel(gpu, 2, 512, 192, 64, 64, 64, tau_mem=0.1, streams=8, precision=0)
    upload(om, small)
    rng = np.random.default_rng(3)
    prompts = [rng.integers(1, 512, 16) for _ in range(96)]
    lb, gb = big.prefill_batch(prompts, want_greedy=True)
    ls, gs = small.prefill_batch(prompts[:8], want_greedy=True)
    assert np.array_equal(lb[:8], ls) and np.array_equal(gb[:8], gs)
    for _ in range(12):
        lb, gb = big.decode_step(gb, want_greedy=True)
        ls, gs = small.decode_step(gs, want_greedy=True)
        assert np.array_equal(lb[:8], ls) and np.array_equal(gb[:8], gs)
    big.close(), small.close()


def test_closing_the_context_first_closes_its_models():
    """A model holds a pointer into its context; closing the context must retire the model rather than
    leave it to free device memory through a dead context later."""
    import pssa_b200
    g = pssa_b200.B200Dispatch(0)
    m = pssa_b200.PSSAModel(g, 1, 32, 16, 4, 4, 8)
    g.close()
    assert m._h is None
    m.close()  # idempotent
    del m


def test_sharded_prefill_single_rank_matches_the_oracle(gpu):
    """The lane-sharding front end on one rank (no process group): one logits row per prompt, empty prompts zero."""
    from pssa_b200 import lanes as L
    om, gm = make_pair(gpu, 2, 61, 24, 4, 8, 16, seed=5, streams=8)
    rng = np.random.default_rng(3)
    prompts = [rng.integers(1, 61, n) for n in (9, 0, 4, 17, 1, 6, 6)]
    gm.reset_recurrent_state()
    got = L.sharded_prefill(gm, prompts, 1, 0)
    assert got.shape == (7, 61) and not got[1].any()
    for j, p in enumerate(prompts):
        if len(p):
            ref_m = om.clone()
            ref_m.reset_recurrent_state()
            _, _, ref = ref_m.prefill_inference(p)
            assert scale_err(got[j], ref) <= 1e-5, j


def test_device_resident_prefill_equals_the_host_entry_and_profile_rows_add_up(gpu):
    """`prefill_batch_dev` (ids and logits stay in HBM, work only enqueued) returns the host entry's bits, and the
    per-kernel profile counts every launch the context counted."""
    import torch
    om, gm = make_pair(gpu, 2, 80, 48, 16, 16, 20, seed=9, streams=3, precision=0)
    lanes = [list((np.arange(n) * 5 + j) % 79 + 1) for j, n in enumerate([33, 7, 64])]
    gm.reset_recurrent_state()
    host_logits, host_greedy = gm.prefill_batch(lanes, want_greedy=True)
    gm.reset_recurrent_state()
    lengths = np.array([len(x) for x in lanes], np.uint32)
    offsets = np.concatenate([[0], np.cumsum(lengths)[:-1]]).astype(np.uint32)
    ids_dev = torch.tensor(np.concatenate(lanes).astype(np.int32), device="cuda", dtype=torch.int32)
    logits_dev = torch.zeros(3, 80, device="cuda")
    greedy_dev = torch.zeros(3, device="cuda", dtype=torch.int32)
    gpu.set_stream(torch.cuda.current_stream())
    n0 = gpu.launch_count()
    gpu.profile_begin()
    gm.prefill_batch_dev(ids_dev, offsets, lengths, None, logits_dev, greedy_dev)
    torch.cuda.synchronize()
    rows = gpu.profile_end()
    launched = gpu.launch_count() - n0
    gpu.set_stream(None)
    assert np.array_equal(logits_dev.cpu().numpy().view(np.uint32), host_logits.view(np.uint32))
    assert np.array_equal(greedy_dev.cpu().numpy().astype(np.uint64), host_greedy)
    assert launched > 0 and sum(n for n, _ in rows.values()) == launched
    assert all(ms >= 0 for _, ms in rows.values()) and any("ssm_fused" in k for k in rows)


def test_long_single_sequence_uses_time_chunks_and_matches_the_oracle(gpu):
    """One lane of 700 tokens cannot fill the GPU by channels alone: the library cuts it into time chunks (chunk maps,
    fold, second pass). Logits and the final state still match the token-serial oracle in the fp32 mode."""
    om, gm = make_pair(gpu, 2, 61, 32, 8, 8, 12, seed=13, streams=1)
    ids = (np.arange(700) * 7 + 3) % 61
    gpu.profile_begin()
    _, logits = gm.prefill_inference(ids)
    rows = gpu.profile_end()
    assert "seqpar_fold_kernel" in rows and rows["seqpar_fold_kernel"][0] == 2  # once per block
    _, _, ref = om.prefill_inference(ids)
    assert scale_err(logits, ref) <= 1e-5
    ref_state = om.state()
    assert np.max(np.abs(gm.copy_recurrent_state_to(0) - ref_state)) <= 1e-5 * max(1.0, np.abs(ref_state).max())
    # continuing token by token from the chunked prefill equals continuing on the CPU
    a = gm.forward_inference(5)
    b = om.forward_inference(5)
    assert scale_err(a, b) <= 1e-5


def test_reference_cpu_case_prefill_512_then_200_greedy_tokens(gpu):
    """The reference's own CPU-runnable configuration: one block, vocabulary 8192, d 192, state 64, 512 slots (key
    dim 64), ids uniform in [1, 8192); prefill 512 tokens, then 200 greedy tokens. The fp32 mode emits the oracle's
    token sequence; the bf16 mode agrees wherever the oracle's top-1/top-2 gap exceeds the bf16 error bound."""
    v, n_prompt, n_new = 8192, 512, 200
    ids = np.random.default_rng(0).integers(1, v, n_prompt)
    om, gm = make_pair(gpu, 1, v, 192, 64, 64, 512, seed=41)
    ref_tokens, min_gap = om.clone().generate_greedy(ids, n_new)
    got = gm.generate_greedy(ids, n_new)
    assert np.array_equal(got, ref_tokens), f"first difference at {int(np.argmax(got != ref_tokens))}, min gap {min_gap}"
    om2, gm16 = make_pair(gpu, 1, v, 192, 64, 64, 512, seed=41, precision=0)
    got16 = gm16.generate_greedy(ids, n_new)
    # walk the oracle along ITS sequence and compare only while the bf16 path has followed it
    om2.reset_recurrent_state()
    _, _, ref = om2.prefill_inference(ids)
    followed = 0
    for t in range(n_new):
        order = np.sort(ref[1:])
        gap = order[-1] - order[-2]
        if int(got16[t]) != int(ref_tokens[t]):
            assert gap <= 4e-2, f"bf16 path left the reference sequence at step {t} with a gap of {gap}"
            break
        followed += 1
        ref = om2.forward_inference(int(ref_tokens[t]))
    assert followed >= 1


@pytest.mark.parametrize("top_k", [0, 3])
def test_observer_scratch_matches_the_reference_buffers(gpu, top_k):
    """`inf_mem_weights / inf_q_pnc / inf_m_val / inf_z_final` of every block for the last token processed
    (src/pssa.rs:609-619), after a prefill and after decode steps, in both precision modes."""
    for precision, tol in ((1, 1e-5), (0, 3e-2)):
        om, gm = make_pair(gpu, 3, 80, 48, 16, 16, 20, seed=17, streams=2, bank_fill=0.8, precision=precision)
        if top_k:
            gm.set_memory_top_k(top_k)
            for l in range(3):
                c, h, _ = om.bank_meta(l)
                om.set_bank_meta(l, c, h, top_k)
        gm.set_observer(True)
        ids = (np.arange(23) * 7 + 2) % 80

        def check(where):
            for l in range(3):
                w, q, mv, z = gm.observation(l, 0)
                ref = [om.tensor(l, t).copy() for t in (O.S_MEM_WEIGHTS, O.S_Q_PNC, O.S_M_VAL, O.S_Z_FINAL)]
                for got, want, name in zip((w, q, mv, z), ref, ("weights", "q_pnc", "m_val", "z_final")):
                    scale = max(1e-6, float(np.abs(want).max()))
                    assert np.max(np.abs(got - want)) / scale <= tol, (where, l, name, precision)
                if precision == 1 and top_k:
                    assert np.array_equal(w != 0, ref[0] != 0)  # the same slots selected

        gm.prefill_inference(ids)
        om.prefill_inference(ids)
        check("prefill")
        for tok in (5, 9):
            gm.forward_inference(tok)
            om.forward_inference(tok)
            check("decode")
        gm.set_observer(False)
        with pytest.raises(Exception, match="observer scratch is empty"):
            gm.observation(0, 0)
        gm.close()


def test_scorer_reproduces_the_reference_golden_loss_and_logits(gpu, golden_dir):
    """The frozen-model scorer (all-position logits + cross entropy) against the reference's own vector: word 0 of the
    golden file is the chunk-forward loss of the fresh depth-one model on ids [1, 2, 1] / targets [2, 1, 3], words
    [1, 22) its logits (tests/depth_one_parity.rs)."""
    import pssa_b200
    data = (golden_dir / "depth_one_main85d9d33_initial.pssa").read_bytes()
    obs = np.frombuffer((golden_dir / "depth_one_main014f617_avx2_observed.bin").read_bytes(), np.uint32)
    want_loss = float(obs[:1].view(np.float32)[0])
    want_logits = obs[1:22].view(np.float32).reshape(3, 7)
    gm = pssa_b200.PSSAModel.from_checkpoint(gpu, data, precision=1)
    loss, per, logits = gm.score([1, 2, 1], [2, 1, 3], want_logits=True)
    assert abs(loss - want_loss) <= 1e-5 * abs(want_loss)
    assert scale_err(logits, want_logits) <= 1e-5
    assert abs(float(per.mean()) - loss) <= 1e-6
    gm.close()


def test_scorer_matches_the_oracle_over_passes_and_tiles(gpu):
    om, gm = make_pair(gpu, 2, 97, 32, 16, 8, 16, seed=23)
    ids = (np.arange(300) * 7 + 1) % 97
    targets = (ids * 3 + 5) % 97
    ref_loss, ref_logits = om.chunk_forward(ids, targets)
    gm.set_max_rows(128)  # three passes
    loss, per, logits = gm.score(ids, targets, want_logits=True)
    assert abs(loss - ref_loss) <= 1e-5 * abs(ref_loss)
    assert scale_err(logits, ref_logits) <= 1e-5
    assert np.max(np.abs(gm.copy_recurrent_state_to(0) - om.state())) <= 1e-5 * max(1.0, np.abs(om.state()).max())
    import pssa_b200
    with pytest.raises(pssa_b200.B200Error, match="target ID 97 outside"):
        gm.score([1, 2], [3, 97])
    gm.close()


def test_greedy_decode_step_as_a_cuda_graph_equals_the_eager_steps(gpu):
    """The device-resident entry is capturable once its lane layout is on the device: replays of the captured step
    (ids fed back on the device) produce the tokens of eager decode steps."""
    import torch
    gpu.set_stream(torch.cuda.current_stream())
    om, gm = make_pair(gpu, 2, 97, 32, 16, 8, 16, seed=31, streams=3, precision=0)
    _, gm2 = make_pair(gpu, 2, 97, 32, 16, 8, 16, seed=31, streams=3, precision=0)
    prompts = [[5, 9, 2], [11, 3], [7]]
    _, g0 = gm.prefill_batch(prompts, want_logits=False, want_greedy=True)
    _, g0b = gm2.prefill_batch(prompts, want_logits=False, want_greedy=True)
    assert np.array_equal(g0, g0b)
    # eager reference: 6 steps
    eager = [g0b]
    for _ in range(6):
        eager.append(gm2.decode_step(eager[-1], want_logits=False, want_greedy=True))
    ids_dev = torch.tensor(g0.astype(np.int32), device="cuda", dtype=torch.int32)
    graph = gm.capture_greedy_decode_graph(ids_dev)          # takes one real step
    torch.cuda.synchronize()
    assert np.array_equal(ids_dev.cpu().numpy().astype(np.uint64), eager[1])
    for step in range(2, 7):
        graph.replay()
        torch.cuda.synchronize()
        assert np.array_equal(ids_dev.cpu().numpy().astype(np.uint64), eager[step]), step
    gpu.poll_status()
    gpu.set_stream(None)
    gm.close()
    gm2.close()


def test_device_resident_ids_outside_the_vocabulary_raise_the_status_word(gpu):
    import pssa_b200
    import torch
    gpu.set_stream(torch.cuda.current_stream())
    _, gm = make_pair(gpu, 1, 50, 16, 4, 4, 8, seed=3, precision=1)
    ids_dev = torch.tensor([3, 50, 4], device="cuda", dtype=torch.int32)
    logits = torch.zeros(1, 50, device="cuda")
    gm.prefill_batch_dev(ids_dev, np.array([0], np.uint32), np.array([3], np.uint32), None, logits, None)
    torch.cuda.synchronize()
    with pytest.raises(pssa_b200.B200Error) as e:
        gpu.poll_status()
    assert e.value.status == N_ERR_TOKEN
    gpu.poll_status()  # cleared
    gpu.set_stream(None)
    gm.close()


@pytest.mark.parametrize("precision", [1, 0])
def test_lane_groups_on_side_streams_do_not_change_results(gpu, precision):
    """A pass over several lanes may be enqueued as up to four groups of consecutive lanes on side streams (the groups
    share only read-only weights). Logits, greedy tokens and carries must be bit-identical to the single-stream schedule,
    for ragged prefill (including an empty lane), for decode steps, with top-k reads, and under the stage profile."""
    om, gm = make_pair(gpu, 2, 300, 192, 64, 64, 512, seed=77, streams=7, precision=precision)
    rng = np.random.default_rng(8)
    lanes = [list(rng.integers(1, 300, n)) for n in (40, 3, 0, 65, 17, 1, 30)]
    results = []
    for groups, top_k in ((1, None), (2, None), (4, None), (3, None), (1, 8), (4, 8)):
        if top_k:
            gm.set_memory_top_k(top_k)
        gm.set_lane_groups(groups)
        gm.reset_recurrent_state()
        if groups == 4:
            gpu.profile_begin()
        logits, greedy = gm.prefill_batch(lanes, want_greedy=True)
        ids = np.where(np.array([len(x) for x in lanes]) > 0, greedy, 1)
        for _ in range(3):
            step_logits, ids = gm.decode_step(ids, want_logits=True, want_greedy=True)
        if groups == 4:
            rows = gpu.profile_end()
            assert any("ssm" in k for k in rows)
        states = np.stack([gm.copy_recurrent_state_to(s) for s in range(7)])
        results.append((top_k, logits, greedy, step_logits, ids, states))
    for top_k in (None, 8):
        same = [r for r in results if r[0] == top_k]
        for other in same[1:]:
            for a, b in zip(same[0][1:], other[1:]):
                assert np.array_equal(a.view(np.uint32) if a.dtype == np.float32 else a, b.view(np.uint32) if b.dtype == np.float32 else b)
    gm.set_lane_groups(0)
    gpu.poll_status()
    gm.close()


def test_decode_graph_with_lane_groups_replays_the_eager_tokens(gpu):
    """Fork and join of the lane groups are events between streams, so the captured step keeps its parallel branches."""
    import torch
    gpu.set_stream(torch.cuda.current_stream())
    _, gm = make_pair(gpu, 2, 97, 32, 16, 8, 16, seed=31, streams=6, precision=0)
    _, gm2 = make_pair(gpu, 2, 97, 32, 16, 8, 16, seed=31, streams=6, precision=0)
    gm.set_lane_groups(3)
    gm2.set_lane_groups(1)
    prompts = [[5, 9, 2], [11, 3], [7], [8, 8], [1, 2, 3, 4], [9]]
    _, g0 = gm.prefill_batch(prompts, want_logits=False, want_greedy=True)
    _, g0b = gm2.prefill_batch(prompts, want_logits=False, want_greedy=True)
    assert np.array_equal(g0, g0b)
    eager = [g0b]
    for _ in range(5):
        eager.append(gm2.decode_step(eager[-1], want_logits=False, want_greedy=True))
    ids_dev = torch.tensor(g0.astype(np.int32), device="cuda", dtype=torch.int32)
    graph = gm.capture_greedy_decode_graph(ids_dev)
    torch.cuda.synchronize()
    assert np.array_equal(ids_dev.cpu().numpy().astype(np.uint64), eager[1])
    for step in range(2, 6):
        graph.replay()
        torch.cuda.synchronize()
        assert np.array_equal(ids_dev.cpu().numpy().astype(np.uint64), eager[step]), step
    gpu.poll_status()
    gpu.set_stream(None)
    gm.close()
    gm2.close()


def test_reserved_model_allocates_nothing_during_calls(gpu):
    """`pssa_b200_model_reserve`: after it, prefill (plain and time-chunked) and decode calls within the reserved size
    leave the device's free memory unchanged (growth of the workspace, the chunk buffers and the sampler state is what
    would otherwise allocate, and synchronise, in the middle of a call)."""
    import torch
    import pssa_b200
    cfg = dict(depth=2, d_vocab=101, d_latent=64, d_state=16, d_mem_key=16, mem_capacity=64)
    om = O.Model.new(cfg["depth"], cfg["d_vocab"], cfg["d_latent"], cfg["d_state"], cfg["d_mem_key"], cfg["mem_capacity"], tau_mem=0.1, seed=2)
    fill_synthetic(om, 2)
    gm = pssa_b200.PSSAModel(gpu, tau_mem=0.1, streams=4, precision=1, **cfg)
    upload(om, gm)
    gm.reserve(4 * 700, 4)
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    rng = np.random.default_rng(3)
    gm.prefill_batch([rng.integers(1, cfg["d_vocab"], n) for n in (700, 50, 1, 333)])
    gm.prefill_inference(rng.integers(1, cfg["d_vocab"], 700))  # one long lane: the time-chunked path
    gm.decode_step([1, 2, 3, 4], want_logits=True, want_greedy=True)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0
    gm.close()


@pytest.mark.parametrize("k,cap,tau", [(64, 256, 0.1), (128, 128, 0.13), (128, 512, 0.1), (64, 512, 0.25)])
def test_one_kernel_all_slots_read_agrees_with_the_separate_kernels(gpu, monkeypatch, k, cap, tau):
    """The bf16 mode's all-slots read runs projection, distances, softmax and the bf16 weight rows as one kernel when
    the shape allows it (three bf16 piece products instead of six, hardware sqrt / lg2 / ex2, weights rounded to bf16
    before and after normalisation). Against the separate kernels (same weights, same prompts): logits within 2e-3
    max-abs of each other, and both within the bf16 mode's 2e-2 of the fp32 CPU reference; a partly filled bank gives
    its empty slots weight zero in both."""
    import pssa_b200
    om = O.Model.new(2, 512, 192, 64, k, cap, tau_mem=tau, seed=17)
    fill_synthetic(om, 17, 0.6)
    rng = np.random.default_rng(5)
    prompts = [rng.integers(1, 512, n) for n in (300, 257, 128, 40)]
    ref = np.stack([om_prefill(om, ids) for ids in prompts])
    out = []
    for keep in ("1", "0"):
        monkeypatch.setenv("PSSA_B200_NO_ALL_SLOTS_FUSED", keep)
        gm = pssa_b200.PSSAModel(gpu, 2, 512, 192, 64, k, cap, tau_mem=tau, streams=4, precision=0)
        upload(om, gm)
        logits, _ = gm.prefill_batch(prompts, want_greedy=True)
        out.append(logits.copy())
        gm.close()
    assert float(np.max(np.abs(out[0] - out[1]))) <= 2e-3
    assert float(np.max(np.abs(out[0] - ref))) <= 2e-2 and float(np.max(np.abs(out[1] - ref))) <= 2e-2


def om_prefill(om, ids):
    om.reset_recurrent_state()
    _, _, logits = om.prefill_inference(ids)
    return np.array(logits, copy=True)
