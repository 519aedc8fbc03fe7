"""Sequence-parallel prefill, host side: time sharding, owner selection, and the exchange-and-fold algorithm the
library runs per block, restated with numpy on two gloo ranks and checked against the oracle's single-pass SSM."""
import os
import socket

import numpy as np
import pytest

import oracle as O
from parity import REL_TOL, chan_err
from pssa_b200 import seqpar as SP


def test_time_shards_are_contiguous_balanced_and_cover_the_sequence():
    for world in (1, 2, 3, 8):
        for n in (0, 1, 7, 8, 9, 65536, 65537):
            sh = SP.time_shards(n, world)
            assert len(sh) == world and sh[0][0] == 0 and sh[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(sh, sh[1:]))
            sizes = [b - a for a, b in sh]
            assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
            owner = SP.last_token_owner(n, world)
            assert owner == (-1 if n == 0 else max(r for r, z in enumerate(sizes) if z))
    with pytest.raises(ValueError):
        SP.time_shards(4, 0)


def test_pack_shard_and_owner_selection():
    prompts = [np.arange(10, 21), np.arange(3), np.zeros(0, np.int64), np.arange(100, 105)]
    seen = [[] for _ in prompts]
    for rank in range(3):
        ids, off, ln = SP.pack_shard(prompts, 3, rank)
        assert ids.dtype == np.uint32 and len(ids) == int(ln.sum())
        for lane in range(len(prompts)):
            seen[lane] += ids[off[lane]:off[lane] + ln[lane]].tolist()
    assert all(s == list(p) for s, p in zip(seen, prompts))
    rows = np.arange(3 * 4 * 2, dtype=np.float32).reshape(3, 4, 2)
    got = SP.select_owner_rows(rows, [11, 3, 0, 5], 3)
    assert np.array_equal(got[0], rows[2, 0]) and np.array_equal(got[1], rows[2, 1])
    assert not got[2].any() and np.array_equal(got[3], rows[2, 3])
    assert np.array_equal(SP.select_owner_rows(rows, [2, 1, 0, 3], 3)[1], rows[0, 1])


T, D, S = 90, 12, 8


def _inputs():
    rng = np.random.default_rng(11)
    delta = np.log1p(np.exp(rng.normal(-2.0, 1.0, (T, D)))).astype(np.float32)
    bp = rng.normal(0, 1, (T, S)).astype(np.float32)
    cp = rng.normal(0, 1, (T, S)).astype(np.float32)
    x = rng.normal(0, 1, (T, D)).astype(np.float32)
    rates = -np.exp(rng.uniform(np.log(0.005), np.log(0.7), D * S)).astype(np.float32)
    h0 = rng.normal(0, 1, D * S).astype(np.float32)
    return delta, bp, cp, x, rates, h0


def _one_lane(delta, bp, cp, x, rates, carry):
    c = carry.reshape(1, -1).copy()
    n = len(delta)
    y = O.ssm_lanes(delta, bp, cp, x, rates, c, np.zeros(1, np.uint32), np.array([n], np.uint32)) if n else np.zeros((0, D), np.float32)
    return y, c[0]


def _rank_main(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        delta, bp, cp, x, rates, h0 = _inputs()
        a, b = SP.time_shards(T, world)[rank]
        sl = slice(a, b)
        # 1. the shard's affine map from a zero carry: (sum of delta per channel, end state)
        _, q_state = _one_lane(delta[sl], bp[sl], cp[sl], x[sl], rates, np.zeros(D * S, np.float32))
        rec = np.concatenate([delta[sl].astype(np.float64).sum(0).astype(np.float32), q_state])
        # 2. all-gather of the records
        got = [torch.empty(len(rec)) for _ in range(world)]
        dist.all_gather(got, torch.from_numpy(rec))
        # 3. fold in time order: carry-in of this rank, and the final state
        h = h0.copy()
        for k in range(world):
            if k == rank:
                carry_in = h.copy()
            r = got[k].numpy()
            pk = np.exp((rates * np.repeat(r[:D], S)).astype(np.float32)).astype(np.float32)
            h = (pk * h).astype(np.float32) + r[D:]
        # 4. the real pass
        y, _ = _one_lane(delta[sl], bp[sl], cp[sl], x[sl], rates, carry_in)
        q.put((rank, y, h))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_ranks_exchange_and_fold_reproduce_the_single_pass():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = {}
    for _ in procs:
        rank, y, h = q.get(timeout=120)
        res[rank] = (y, h)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    delta, bp, cp, x, rates, h0 = _inputs()
    ref_y, ref_h = _one_lane(delta, bp, cp, x, rates, h0)
    y = np.concatenate([res[0][0], res[1][0]])
    assert chan_err(y, ref_y, 0) <= REL_TOL
    scale = np.abs(ref_h).max()
    for r in (0, 1):  # both ranks end with the same, correct, final state
        assert np.max(np.abs(res[r][1] - ref_h)) / scale <= REL_TOL
    assert np.array_equal(res[0][1], res[1][1])


def test_the_empty_shard_verdict_is_the_same_on_every_rank():
    """A prompt shorter than the world leaves the last ranks without tokens. The check runs on the global lengths, so
    every rank raises (or none does) before any of them enqueues the per-block all-gather."""
    for lengths, world, ok in (([3], 4, False), ([3, 0, 2], 4, False), ([4], 4, True), ([1, 9], 4, True), ([5, 7], 2, True),
                               ([0, 0], 2, False), ([2, 3], 2, True), ([1], 1, True)):
        verdicts = []
        for rank in range(world):  # what each rank would conclude: the function does not look at the rank at all
            try:
                SP.check_every_rank_has_tokens(lengths, world)
                verdicts.append(True)
            except ValueError:
                verdicts.append(False)
        assert verdicts == [ok] * world, (lengths, world)
        # and it agrees with what the ranks' packed shards actually hold
        holds = [int(SP.pack_shard([np.zeros(n, np.int64) for n in lengths], world, r)[2].sum()) > 0 for r in range(world)]
        assert all(holds) == ok


def test_shard_lengths_between_world_and_twice_world_differ_by_rank():
    """With world <= len < 2*world some ranks hold two tokens and some one: anything a rank derives for the exchange
    (record counts, chunking) must therefore not depend on its own shard length."""
    world = 4
    sizes = [[b - a for a, b in SP.time_shards(n, world)] for n in (4, 5, 7)]
    assert sizes == [[1, 1, 1, 1], [2, 1, 1, 1], [2, 2, 2, 1]]
