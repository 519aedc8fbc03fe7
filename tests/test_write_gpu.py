"""Parity of the bank write (refractory gate + ring insert) and of the plastic fast-weight update with the CPU
oracle, through the C ABI."""
import numpy as np
import pytest

import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    import torch

    import pssa_b200
    d = pssa_b200.B200Dispatch(0)
    d.set_stream(torch.cuda.current_stream())
    yield d
    d.set_stream(None)
    d.close()


class DeviceBank:
    def __init__(self, cap, dk, dv):
        import torch
        self.cap, self.dk, self.dv = cap, dk, dv
        self.keys = torch.zeros(cap, dk, device="cuda")
        self.norm_sq = torch.zeros(cap, device="cuda")
        self.values = torch.zeros(cap, dv, device="cuda")
        self.conf = torch.ones(cap, device="cuda")
        self.seen = torch.zeros(cap, dtype=torch.int64, device="cuda")
        self.meta = torch.zeros(2, dtype=torch.int64, device="cuda")

    def write(self, gpu, keys, vals, surprise, steps, winning=None, eta=0.0):
        import torch
        n = len(steps)
        tk = torch.tensor(np.asarray(keys, np.float32).reshape(n, self.dk), device="cuda")
        tv = torch.tensor(np.asarray(vals, np.float32).reshape(n, self.dv), device="cuda")
        ts = torch.tensor(np.asarray(surprise, np.float32), device="cuda")
        tt = torch.tensor(np.asarray(steps, np.int64), device="cuda")
        out = torch.full((n,), -7, dtype=torch.int64, device="cuda")
        tw = None if winning is None else torch.tensor(np.asarray(winning, np.int32), device="cuda")
        gpu.bank_insert_protected_dev(self.keys, self.norm_sq, self.values, self.conf, self.seen, self.meta, self.cap,
                                      self.dk, self.dv, tk, tv, ts, tt, n, out, tw, eta)
        torch.cuda.synchronize()
        return out.cpu().numpy()


def assert_same(bank: DeviceBank, ref: "O.RawBank", conf_tol=0.0):
    count, head, seen = ref.meta()
    assert bank.meta.cpu().tolist() == [count, head]
    assert np.array_equal(bank.keys.cpu().numpy().ravel().view(np.uint32), ref.array(0).view(np.uint32))
    assert np.array_equal(bank.values.cpu().numpy().ravel().view(np.uint32), ref.array(1).view(np.uint32))
    assert np.array_equal(bank.norm_sq.cpu().numpy().view(np.uint32), ref.array(2).view(np.uint32))
    assert np.max(np.abs(bank.conf.cpu().numpy() - ref.array(3))) <= conf_tol
    assert bank.seen.cpu().numpy().astype(np.uint64).tolist() == seen.tolist()


def test_reference_known_answer_defend_then_overwrite(gpu):
    # src/memory.rs:715-735 without the value cap
    bank, ref = DeviceBank(1, 1, 2), O.RawBank(1, 1, 2)
    seq = [([0.1], [3.0, 4.0], 0.0, 1), ([0.2], [30.0, 40.0], 0.0, 2), ([0.2], [-30.0, 40.0], 1e6, 1000)]
    want = [ref.insert_protected(k, v, s, t) for k, v, s, t in seq]
    got = bank.write(gpu, [k for k, *_ in seq], [v for _, v, *_ in seq], [s for *_, s, _ in seq], [t for *_, t in seq])
    assert want == [0, None, 0] and got.tolist() == [0, -1, 0]
    assert_same(bank, ref)
    assert bank.conf.cpu().tolist() == [1.0] and bank.seen.cpu().tolist() == [1000]


def test_ordered_writes_fill_then_gate_the_ring_head(gpu):
    rng = np.random.default_rng(0)
    cap, dk, dv, n = 5, 8, 12, 40
    bank, ref = DeviceBank(cap, dk, dv), O.RawBank(cap, dk, dv)
    dirs = rng.standard_normal((n, dk))
    keys = (dirs / np.linalg.norm(dirs, axis=1, keepdims=True) * rng.uniform(0, 0.95, (n, 1))).astype(np.float32)
    vals = rng.standard_normal((n, dv)).astype(np.float32)
    surprise = rng.uniform(3.5, 40.0, n).astype(np.float32)
    steps = np.cumsum(rng.integers(1, 90, n)).astype(np.int64)
    want = [ref.insert_protected(keys[i], vals[i], float(surprise[i]), int(steps[i])) for i in range(n)]
    got = bank.write(gpu, keys, vals, surprise, steps)  # one launch, ordered
    assert got.tolist() == [-1 if w is None else w for w in want]
    assert any(w is None for w in want) and sum(w is not None for w in want) > cap  # both gate outcomes occurred
    assert_same(bank, ref, conf_tol=3e-7)  # the gate's expf is the only inexact operation
    # split into two launches: same state (the carry is the bank itself)
    bank2 = DeviceBank(cap, dk, dv)
    bank2.write(gpu, keys[:17], vals[:17], surprise[:17], steps[:17])
    bank2.write(gpu, keys[17:], vals[17:], surprise[17:], steps[17:])
    assert np.array_equal(bank2.values.cpu().numpy(), bank.values.cpu().numpy())
    assert np.array_equal(bank2.conf.cpu().numpy(), bank.conf.cpu().numpy())


def test_winning_slot_rank_one_write_matches_the_restatement(gpu):
    """The retrieval benchmark's write variant (nearest slot, rank-1 value update): not a reference code path, so
    parity is against the oracle's explicit restatement only."""
    rng = np.random.default_rng(3)
    cap, dk, dv, n = 16, 4, 6, 30
    bank, ref = DeviceBank(cap, dk, dv), O.RawBank(cap, dk, dv)
    init_k = (rng.uniform(-0.4, 0.4, (cap, dk))).astype(np.float32)
    init_v = rng.standard_normal((cap, dv)).astype(np.float32)
    for i in range(cap):
        ref.insert(init_k[i], init_v[i])
    bank.write(gpu, init_k, init_v, np.zeros(cap, np.float32), np.zeros(cap, np.int64))
    slots = rng.integers(0, cap, n)
    vals = rng.standard_normal((n, dv)).astype(np.float32)
    surprise = rng.uniform(0.0, 60.0, n).astype(np.float32)
    steps = np.cumsum(rng.integers(1, 50, n)).astype(np.int64)
    want = [ref.plastic_write(int(slots[i]), vals[i], float(surprise[i]), int(steps[i]), 0.25) for i in range(n)]
    got = bank.write(gpu, np.zeros((n, dk), np.float32), vals, surprise, steps, winning=slots, eta=0.25)
    assert got.tolist() == [-1 if w is None else w for w in want]
    assert np.max(np.abs(bank.values.cpu().numpy().ravel() - ref.array(1))) <= 1e-6
    assert np.max(np.abs(bank.conf.cpu().numpy() - ref.array(3))) <= 3e-7
    assert np.array_equal(bank.keys.cpu().numpy().ravel(), ref.array(0))  # keys untouched in this mode


def test_plastic_update_and_consolidation_match_the_oracle(gpu):
    # src/pssa.rs:1814-1832 and src/adapter.rs:65-72
    import torch
    m = O.Model.new(1, 20, 16, 4, 4, 4, seed=5)
    m.tensor(0, O.AD_UP)[:] = O.rng_fill(1, -0.1, 0.1, 16 * 16)
    m.tensor(0, O.AD_CONS)[:] = O.rng_fill(2, -0.1, 0.1, 16 * 16)
    value = O.rng_fill(3, -6.0, 6.0, 16)  # large enough that the +-4 clamp engages
    before = m.tensor(0, O.AD_UP).copy()
    O.lib().pssa_oracle_dream_replay(m.h, 0, O.fptr(value))
    act, out = m.tensor(0, O.S_AD_ACT).copy(), m.tensor(0, O.S_AD_OUT).copy()
    up = torch.tensor(before, device="cuda")
    gpu.adapter_plastic_update_dev(up, torch.tensor(value, device="cuda"), torch.tensor(out, device="cuda"),
                                   torch.tensor(act, device="cuda"), 16, 16)
    torch.cuda.synchronize()
    assert np.array_equal(up.cpu().numpy().view(np.uint32), m.tensor(0, O.AD_UP).view(np.uint32))
    slow = torch.tensor(m.tensor(0, O.AD_CONS).copy(), device="cuda")
    O.lib().pssa_oracle_consolidate(m.h, 0, 0.01)
    gpu.adapter_consolidate_dev(up, slow, 256, 0.01)
    torch.cuda.synchronize()
    assert np.array_equal(up.cpu().numpy().view(np.uint32), m.tensor(0, O.AD_UP).view(np.uint32))
    assert np.array_equal(slow.cpu().numpy().view(np.uint32), m.tensor(0, O.AD_CONS).view(np.uint32))


def test_write_argument_errors(gpu):
    import pssa_b200
    bank = DeviceBank(2, 2, 2)
    with pytest.raises(pssa_b200.B200Error, match="eta must be in"):
        bank.write(gpu, [[0.0, 0.0]], [[0.0, 0.0]], [0.0], [1], winning=[0], eta=2.0)
    with pytest.raises(pssa_b200.B200Error, match="must be positive"):
        gpu.bank_insert_protected_dev(bank.keys, bank.norm_sq, bank.values, bank.conf, bank.seen, bank.meta, 0, 2, 2,
                                      bank.keys, bank.values, bank.conf, bank.seen, 1)


def test_out_of_range_device_metadata_is_refused_without_touching_memory(gpu):
    """Slot ids and {count, write_head} live on the device, where the host cannot check them. A winning slot or ring
    head >= capacity, a count above capacity, or a key outside the open unit ball (src/memory.rs:273-277 asserts it)
    must skip that write, report slot -2, raise PSSA_B200_ERR_BANK in the status word and leave the bank alone."""
    import torch

    import pssa_b200
    cap, dk, dv = 4, 3, 5
    rng = np.random.default_rng(2)
    bank = DeviceBank(cap, dk, dv)
    keys = rng.uniform(-0.3, 0.3, (cap, dk)).astype(np.float32)
    vals = rng.standard_normal((cap, dv)).astype(np.float32)
    assert bank.write(gpu, keys, vals, np.ones(cap), np.arange(cap)).tolist() == [0, 1, 2, 3]
    gpu.poll_status()
    snap = [t.clone() for t in (bank.keys, bank.values, bank.norm_sq, bank.conf, bank.seen, bank.meta)]

    def unchanged():
        return all(torch.equal(a, b) for a, b in zip(snap, (bank.keys, bank.values, bank.norm_sq, bank.conf, bank.seen, bank.meta)))

    def refused():
        with pytest.raises(pssa_b200.B200Error) as e:
            gpu.poll_status()
        assert e.value.status == 9
        gpu.poll_status()  # cleared

    # winning slot outside the bank
    assert bank.write(gpu, keys[:1], vals[:1], [1.0], [9], winning=[cap + 3], eta=0.5).tolist() == [-2]
    refused()
    assert unchanged()
    # key on / outside the unit sphere
    assert bank.write(gpu, [[1.0, 0.0, 0.0]], vals[:1], [50.0], [10]).tolist() == [-2]
    refused()
    assert bank.write(gpu, [[np.nan, 0.0, 0.0]], vals[:1], [50.0], [10]).tolist() == [-2]
    refused()
    assert unchanged()
    # corrupted metadata: ring head beyond the bank, then a count beyond capacity
    bank.meta.copy_(torch.tensor([cap, cap + 1], dtype=torch.int64))
    assert bank.write(gpu, keys[:1], vals[:1], [50.0], [11]).tolist() == [-2]
    refused()
    bank.meta.copy_(torch.tensor([cap + 2, 0], dtype=torch.int64))
    assert bank.write(gpu, keys[:1], vals[:1], [50.0], [12]).tolist() == [-2]
    refused()
    bank.meta.copy_(snap[5])
    assert unchanged()
    # a good write still works afterwards
    assert bank.write(gpu, keys[:1] * 0.5, vals[:1], [50.0], [1000]).tolist() == [0]
    gpu.poll_status()


def test_model_level_memory_insert_follows_insert_training_memory_at(gpu):
    """`pssa_b200_model_insert_memory`: if loss > 3.5 every block's bank gets a protected insert of (q_poincare, z_final)
    of the lane's last token (src/pssa.rs:3705-3737). A small bank fills up and then the refractory gate decides, so the
    sequence of slots (including defended writes) must equal the oracle's, and so must the logits of forward calls
    made after the writes (they read the rewritten banks)."""
    import pssa_b200
    from helpers import fill_synthetic, upload
    cfg = dict(depth=2, d_vocab=61, d_latent=32, d_state=8, d_mem_key=16, mem_capacity=6)
    om = O.Model.new(cfg["depth"], cfg["d_vocab"], cfg["d_latent"], cfg["d_state"], cfg["d_mem_key"], cfg["mem_capacity"], tau_mem=0.1, seed=4)
    fill_synthetic(om, 4, bank_fill=0.5)
    gm = pssa_b200.PSSAModel(gpu, tau_mem=0.1, streams=1, precision=1, **cfg)
    upload(om, gm)
    gm.set_observer(True)
    rng = np.random.default_rng(9)
    # below the threshold nothing is attempted (and no observation is needed for that verdict)
    assert list(gm.insert_memory(3.5, 10)) == [-3, -3]
    step = 0
    for round_ in range(14):
        tok = int(rng.integers(1, cfg["d_vocab"]))
        ok, logits = gm.prefill_inference([tok])
        ref_logits = om.forward_inference(tok)
        assert ok and np.max(np.abs(logits - ref_logits)) <= 1e-5 * max(1.0, float(np.abs(ref_logits).max())), round_
        loss = float(rng.uniform(3.0, 9.0))
        step += int(rng.integers(1, 90))  # some writes come soon after the last one (small refractory gain), some late
        got = gm.insert_memory(loss, step)
        for l in range(cfg["depth"]):
            if loss > 3.5:
                want = om.bank_insert_protected(l, om.tensor(l, O.S_Q_PNC), om.tensor(l, O.S_Z_FINAL), loss, step)
                assert int(got[l]) == want, (round_, l, got, want)
            else:
                assert int(got[l]) == -3
    # without the observer the entry point refuses (its key and value live in the observer scratch)
    gm.set_observer(False)
    with pytest.raises(pssa_b200.B200Error, match="observer"):
        gm.insert_memory(5.0, step + 1)
    gm.close()
