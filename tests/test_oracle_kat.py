"""Known-answer tests the reference holds for the bank, the scan and the numeric tails, run on the oracle
(no GPU). Each test names the reference test it restates."""
import numpy as np
import pytest

import oracle as O

F32_MAX = np.finfo(np.float32).max
TINY = np.frombuffer(np.uint32(1).tobytes(), np.float32)[0]  # f32::from_bits(1)


def project(q):
    q = np.asarray(q, np.float32)
    out = np.empty_like(q)
    norm = O.lib().pssa_oracle_project(O.fptr(q), O.fptr(out), len(q))
    return out, float(norm)


def sqnorm(p):
    p = np.ascontiguousarray(p, np.float32)
    return float(O.lib().pssa_oracle_squared_norm(O.fptr(p), len(p)))


def test_extreme_queries_project_strictly_inside_the_ball():
    # tests/memory_projection.rs:3-35
    for q in ([0.0], [16_777_216.0], [-F32_MAX], [F32_MAX, -F32_MAX, F32_MAX], [F32_MAX] * 4096, [TINY, -TINY]):
        p, norm = project(q)
        assert np.isfinite(norm) and np.all(np.isfinite(p))
        assert sqnorm(p) < 1.0
        if any(abs(x) > 1.0 for x in q):
            assert sqnorm(p) > 0.99
        bank = O.RawBank(1, len(q), 2)
        bank.insert(p, [2.0, -3.0])
        out, w, _ = bank.retrieve(p, float(TINY))
        assert out.tolist() == [2.0, -3.0] and w.tolist() == [1.0]


def test_tiny_temperature_keeps_nearest_entries_and_ties_finite():
    # tests/memory_projection.rs:37-53
    bank = O.RawBank(3, 1, 2)
    bank.insert([0.5], [1.0, 2.0])
    for tau in (np.float32(1e-40), TINY):
        out, w, _ = bank.retrieve([0.0], float(tau))
        assert out.tolist() == [1.0, 2.0] and w[0] == 1.0
    bank.insert([-0.5], [3.0, -2.0])
    bank.insert([0.75], [100.0, 100.0])
    out, w, _ = bank.retrieve([0.0], float(TINY))
    assert w.tolist() == [0.5, 0.5, 0.0]
    assert out.tolist() == [2.0, 0.0]


def test_nearest_read_masks_other_slots_and_full_k_is_exact():
    # tests/memory_expansion.rs:52-77
    bank = O.RawBank(5, 1, 1)
    for key, value in ((0.0, 2.0), (0.1, 4.0), (0.6, 100.0)):
        bank.insert([key], [value])
    full_out, full_w, _ = bank.retrieve([0.0], 1.0)
    full_w[3:] = 0.0  # rows beyond count are not written by the full read (memory.rs:409-425)
    for k in (3, 9):
        bank.set_top_k(k)
        out, w, _ = bank.retrieve([0.0], 1.0)
        w[3:] = 0.0
        assert np.array_equal(out, full_out) and np.array_equal(w, full_w)
    bank.set_top_k(1)
    out, w, _ = bank.retrieve([0.0], 1.0)
    assert out.tolist() == [2.0] and w.tolist() == [1.0, 0.0, 0.0, 0.0, 0.0]
    bank.set_top_k(2)
    out, w, _ = bank.retrieve([0.0], 1.0)
    assert 2.0 < out[0] < 4.0 and abs(float(w.sum()) - 1.0) < 1e-6 and w[2] == 0.0


def test_nearest_ties_tiny_temperature_and_empty_are_stable():
    # tests/memory_expansion.rs:79-92
    b = O.RawBank(4, 1, 1)
    b.set_top_k(1)
    out, w, _ = b.retrieve([0.0], float(TINY))
    assert out.tolist() == [0.0] and w.tolist() == [0.0] * 4
    b.insert([0.2], [1.0])
    b.insert([-0.2], [2.0])
    out, w, _ = b.retrieve([0.0], float(TINY))
    assert out.tolist() == [1.0] and w.tolist() == [1.0, 0.0, 0.0, 0.0]


def test_protected_write_defends_then_overwrites_with_exact_metadata():
    # src/memory.rs:715-735 (value cap off) + src/defense.rs:45-67
    bank = O.RawBank(1, 1, 2)
    assert bank.insert_protected([0.1], [3.0, 4.0], 0.0, 1) == 0
    before = (bank.array(0).copy(), bank.array(1).copy(), bank.array(2).copy())
    assert bank.insert_protected([0.2], [30.0, 40.0], 0.0, 2) is None
    assert np.array_equal(bank.array(0), before[0]) and np.array_equal(bank.array(1), before[1])
    assert np.array_equal(bank.array(2), before[2])
    assert bank.insert_protected([0.2], [-30.0, 40.0], 1e6, 1000) == 0
    assert bank.array(0).tolist() == [np.float32(0.2)]
    assert bank.array(1).tolist() == [-30.0, 40.0]
    assert bank.array(2)[0] == np.float32(sqnorm([0.2]))
    assert bank.array(3).tolist() == [1.0]
    count, head, last_seen = bank.meta()
    assert (count, head, last_seen.tolist()) == (1, 0, [1000])


def test_refractory_gain_floor_and_saturation():
    # src/defense.rs:18-22
    g = O.lib().pssa_oracle_refractory_gain
    assert g(0, 60.0) == np.float32(0.005)
    assert abs(g(10_000, 60.0) - 1.0) < 1e-6
    expect = (1.0 - np.exp(np.float32(-30.0 / 60.0), dtype=np.float32)) ** 2
    assert abs(g(30, 60.0) - expect) < 1e-7


def test_ring_overwrite_order_matches_growth_test_prefix():
    # tests/memory_expansion.rs:12-20 (insert order / write head only; growth itself is out of scope)
    bank = O.RawBank(3, 1, 1)
    for i in range(5):
        bank.insert([i / 10.0], [float(i)])
    assert bank.array(1).tolist() == [3.0, 4.0, 2.0]
    assert bank.meta()[:2] == (3, 2)


@pytest.mark.parametrize("length,stride", [(1, 1), (3, 2), (7, 3), (33, 4)])
def test_affine_scan_exclusive_prefix_contract(length, stride):
    # src/gpu_batch.rs:3808-3835
    t = np.arange(length, dtype=np.float32)[:, None]
    c = np.arange(stride, dtype=np.float32)[None, :]
    a = (0.8 + 0.01 * (t + c)).astype(np.float32)
    b = (-0.2 + 0.03 * (2 * t + c)).astype(np.float32)
    pa, pb = O.affine_scan_exclusive(a, b)
    ra = np.ones(stride, np.float32)
    rb = np.zeros(stride, np.float32)
    for i in range(length):
        assert np.all(np.abs(pa[i] - ra) < 2e-6) and np.all(np.abs(pb[i] - rb) < 1e-4)
        rb = a[i] * rb + b[i]
        ra = ra * a[i]


@pytest.mark.parametrize("T", [1, 2, 3, 31, 32, 33, 129, 300])
def test_blelloch_stage_matches_ordered_recurrence(T):
    # tests/associative_scan.rs:186-233 (FORWARD_TOL = 2e-5, :10)
    rng = np.random.default_rng(T)
    d, s = 7, 3
    delta = rng.uniform(0.01, 0.5, (T, d)).astype(np.float32)
    bp = rng.normal(size=(T, s)).astype(np.float32)
    cp = rng.normal(size=(T, s)).astype(np.float32)
    x = rng.normal(size=(T, d)).astype(np.float32)
    rates = -rng.uniform(0.01, 1.0, d * s).astype(np.float32)
    h0 = rng.normal(size=d * s).astype(np.float32)
    st0, y0, _, _ = O.ssm_forward(delta, bp, cp, x, rates, h0, mode=0)
    st1, y1, _, _ = O.ssm_forward(delta, bp, cp, x, rates, h0, mode=1)
    assert np.max(np.abs(st0 - st1)) < 2e-5 and np.max(np.abs(y0 - y1)) < 2e-5


def test_softplus_tails_and_decay_closed_forms():
    # tests/numeric_recurrence.rs:47-137 (forward halves)
    for raw in (-17.0, -20.0):
        got = float(O.lib().pssa_oracle_softplus(raw))
        expect = np.log1p(np.exp(raw))
        assert got > 0.0 and abs(got / expect - 1.0) < 2.0e-7
    assert O.lib().pssa_oracle_softplus(25.0) == 25.0
    m = O.Model.new(depth=1, d_vocab=2, d_latent=1, d_state=1, d_mem_key=1, mem_capacity=1, chunk_len=2, seed=19)
    m.tensor(0, O.NORM_GAMMA)[:] = 0.0
    m.tensor(0, O.NORM_BETA)[:] = 1.0
    m.tensor(0, O.W_B)[:] = 0.0
    m.tensor(0, O.W_C)[:] = 1.0
    m.tensor(0, O.W_QX)[:] = 0.0
    m.tensor(0, O.W_QH)[:] = 0.0
    m.tensor(-1, O.UNEMBED)[:] = [0.0, 1.0]
    for raw_rate in (-17.0, -20.0):
        m.tensor(0, O.A_MAT)[:] = raw_rate
        m.tensor(0, O.W_DELTA)[:] = 1.0e7
        m.tensor(0, O.H_PERSISTENT)[:] = 1.0
        m.forward_inference(0)
        m.forward_inference(0)
        rate = np.log1p(np.exp(raw_rate))
        decay = np.exp(-1.0e7 * rate)
        assert abs(float(m.tensor(0, O.H_PERSISTENT)[0]) - decay ** 2) < 2.0e-7


def test_greedy_excludes_id_zero_and_breaks_ties_low():
    # src/inference.rs:111-127, test at :569-571
    g = lambda v: O.lib().pssa_oracle_greedy(O.fptr(np.asarray(v, np.float32)), len(v))
    assert g([100.0, 0.5, 0.5, 0.25]) == 1
    assert g([9.0, -1.0, 3.0, 3.0]) == 2
    assert g([0.0, np.nan, 1.0]) == -1
    assert g([0.0, -0.0, 0.0]) == 2  # total_cmp orders -0.0 below +0.0


def test_prefill_error_semantics():
    # src/pssa.rs:2405-2417, tests at src/inference.rs:1115-1160
    m = O.Model.new(depth=2, d_vocab=11, d_latent=8, d_state=4, d_mem_key=4, mem_capacity=4, seed=5)
    rc, done, _ = m.prefill_inference(np.zeros(0, np.uint64))
    assert rc == -1 and done == 0
    ref = m.clone()
    ref.prefill_inference([3, 4], want_logits=False)
    rc, done, _ = m.prefill_inference([3, 4, 99, 5])
    assert rc == -1 and done == 2
    assert np.array_equal(m.state(), ref.state())  # valid prefix advanced, nothing after it


def test_stacked_prefill_equals_token_loop_bitwise():
    # src/inference.rs:1069-1113 (depth 2, non-reset carries, lengths around the 32-token tile)
    for n in (1, 31, 32, 33, 67):
        m = O.Model.new(depth=2, d_vocab=23, d_latent=16, d_state=4, d_mem_key=4, mem_capacity=6, seed=11)
        for l in range(2):
            m.tensor(l, O.MLP_W2)[:] = O.rng_fill(100 + l, -0.1, 0.1, 16 * 32)
            m.tensor(l, O.AD_UP)[:] = O.rng_fill(200 + l, -0.1, 0.1, 16 * 16)
            for j in range(4):
                key, _ = project(O.rng_fill(300 + 10 * l + j, -1, 1, 4))
                m.bank_insert(l, key, O.rng_fill(400 + 10 * l + j, -1, 1, 16))
        ids = (np.arange(n) * 7 + 3) % 23
        b = m.clone()
        rc, done, last = m.prefill_inference(ids)
        for t in ids:
            row = b.forward_inference(int(t))
        assert rc == 1 and done == n
        assert np.array_equal(last.view(np.uint32), row.view(np.uint32))
        assert np.array_equal(m.state().view(np.uint32), b.state().view(np.uint32))


def test_reference_cpu_scans_differ_elementwise_at_cancellations():
    """The reference's two CPU forms of the SSM stage (ordered and Blelloch) agree to its own absolute
    2e-5 (tests/associative_scan.rs:10) but not to 1e-5 elementwise-relative: states that are
    near-cancellations of O(1) terms carry an absolute roundoff of ~1e-7. This is why reassociated
    GPU paths are held to a per-channel-scale bound (tests/parity.py)."""
    from parity import chan_err, rel_err
    rng = np.random.default_rng(7)
    T, d, s = 1024, 8, 4
    delta = rng.uniform(0.001, 0.1, (T, d)).astype(np.float32)
    bp = rng.normal(size=(T, s)).astype(np.float32)
    cp = rng.normal(size=(T, s)).astype(np.float32)
    x = rng.normal(size=(T, d)).astype(np.float32)
    rates = -rng.uniform(0.01, 1.0, d * s).astype(np.float32)
    st0, y0, _, _ = O.ssm_forward(delta, bp, cp, x, rates, np.zeros(d * s, np.float32), mode=0)
    st1, y1, _, _ = O.ssm_forward(delta, bp, cp, x, rates, np.zeros(d * s, np.float32), mode=1)
    assert np.max(np.abs(st0 - st1)) < 2e-5
    assert rel_err(st0[1:], st1[1:]) > 1e-5
    assert chan_err(st1[1:], st0[1:], 0) < 1e-5


def test_ouro_passes_first_pass_keeps_the_single_pass_math_and_prefill_equals_the_token_loop():
    """Runtime Ouro passes (src/pssa.rs:2338-2376). Reference-held properties: the first shared pass preserves the
    single-pass math (tests/loops.rs:42-62: pass 0 of a loops-2 model reproduces the loops-1 states bit for bit, because it
    reads the same embedding rows on its own carry), prefill == token loop bitwise at loops 3 with non-reset carries
    (src/inference.rs:1069-1113), and set_loops keeps pass 0's carry while the new passes start from zero."""
    from helpers import fill_synthetic
    ids = (np.arange(40) * 5 + 1) % 31
    one = O.Model.new(1, 31, 8, 4, 4, 6, seed=0xfeed)
    fill_synthetic(one, 2)
    two = one.clone()
    two.set_loops(2)
    assert two.state().size == 2 * one.state().size
    for t in ids:
        one.forward_inference(int(t))
        two.forward_inference(int(t))
    hs = one.state().size
    assert np.array_equal(two.state()[:hs].view(np.uint32), one.state().view(np.uint32))
    assert np.any(two.state()[hs:] != 0)
    # prefill == token loop at loops 3, depth 2, carries not reset in between
    a = O.Model.new(2, 31, 8, 4, 4, 6, seed=11)
    fill_synthetic(a, 3)
    a.set_loops(3)
    b = a.clone()
    a.prefill_inference(ids[:7])
    for t in ids[:7]:
        b.forward_inference(int(t))
    _, _, la = a.prefill_inference(ids[7:])
    for t in ids[7:]:
        lb = b.forward_inference(int(t))
    assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
    assert np.array_equal(a.state().view(np.uint32), b.state().view(np.uint32))
    assert a.state().size == 2 * 3 * 8 * 4
    # the state round-trips in [block][pass][d*s] order, and changing the count keeps pass 0 only
    st = a.state()
    c = a.clone()
    c.set_state(st[::-1].copy())
    assert np.array_equal(c.state(), st[::-1])
    c.set_state(st)
    c.set_loops(2)
    got = c.state().reshape(2, 2, 32)
    assert np.array_equal(got[:, 0], st.reshape(2, 3, 32)[:, 0]) and not got[:, 1].any()
    with pytest.raises(ValueError, match="--loops must be between 1 and 32"):
        c.set_loops(33)
