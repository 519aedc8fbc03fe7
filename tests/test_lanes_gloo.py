"""Host logic of the multi-rank path: lanes are partitioned over ranks with no data-path collective, and the
per-lane results gathered over `torch.distributed`. Runs as two gloo ranks on CPU; the CPU oracle stands in for
each rank's model replica (the GPU model has the same `prefill_batch` contract)."""
import os
import socket

import numpy as np
import pytest

import oracle as O
from helpers import fill_synthetic
from pssa_b200 import lanes as L

CFG = dict(depth=2, d_vocab=61, d_latent=24, d_state=4, d_mem_key=8, mem_capacity=16)


def test_partition_covers_every_lane_once_and_balances_tokens():
    rng = np.random.default_rng(0)
    for world in (1, 2, 3, 8):
        for n in (0, 1, 5, 37):
            lengths = rng.integers(0, 200, n)
            parts = L.partition_lanes(lengths, world)
            assert len(parts) == world
            allidx = np.concatenate(parts) if n else np.zeros(0, np.int64)
            assert sorted(allidx.tolist()) == list(range(n))
            assert all(np.all(np.diff(p) > 0) for p in parts if len(p) > 1)
            loads = [int(lengths[p].sum()) for p in parts]
            if n:
                assert max(loads) - min(loads) <= int(lengths.max())  # the LPT bound
    with pytest.raises(ValueError):
        L.partition_lanes([1, 2], 0)
    with pytest.raises(ValueError):
        L.partition_lanes([1, -2], 2)


def test_equal_lanes_split_evenly_and_deterministically():
    parts = L.partition_lanes([2048] * 64, 8)
    assert all(len(p) == 8 for p in parts)
    again = L.partition_lanes([2048] * 64, 8)
    assert all(np.array_equal(a, b) for a, b in zip(parts, again))


def test_shard_packing_matches_the_batched_entry_point_layout():
    prompts = [np.arange(1, 6), np.zeros(0, np.int64), np.arange(7, 10), np.arange(20, 31)]
    seen = []
    for rank in range(2):
        sh = L.shard_prompts(prompts, 2, rank)
        assert sh.ids.dtype == np.uint64 and sh.offsets.dtype == np.uint32 and sh.lengths.dtype == np.uint32
        for j, lane in enumerate(sh.lane_ids):
            o, n = int(sh.offsets[j]), int(sh.lengths[j])
            assert np.array_equal(sh.ids[o:o + n], np.asarray(prompts[lane], np.uint64))
        assert len(sh.ids) == int(sh.lengths.sum())
        seen += sh.lane_ids.tolist()
    assert sorted(seen) == [0, 1, 2, 3]
    with pytest.raises(ValueError):
        L.shard_prompts(prompts, 2, 2)


class OracleReplica:
    """One rank's model replica on the CPU: token-serial prefill of each owned lane from a zero state."""

    def __init__(self):
        self.d_vocab = CFG["d_vocab"]
        self.model = O.Model.new(CFG["depth"], CFG["d_vocab"], CFG["d_latent"], CFG["d_state"], CFG["d_mem_key"],
                                 CFG["mem_capacity"])
        fill_synthetic(self.model, 5)

    def prefill_batch(self, lanes):
        out = np.zeros((len(lanes), self.d_vocab), np.float32)
        for j, ids in enumerate(lanes):
            if len(ids):
                self.model.reset_recurrent_state()
                rc, done, logits = self.model.prefill_inference(np.asarray(ids, np.uint64))
                assert rc == 1 and done == len(ids)  # 1 = completed
                out[j] = logits
        return out, None


def _prompts():
    rng = np.random.default_rng(3)
    return [rng.integers(1, CFG["d_vocab"], n) for n in (9, 0, 4, 17, 1, 6, 6)]


def _rank_main(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        got = L.sharded_prefill(OracleReplica(), _prompts(), world, rank)
        q.put((rank, got))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_single_process_result():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    single = L.sharded_prefill(OracleReplica(), _prompts(), 1, 0)  # no process group: reorder only
    assert np.array_equal(results[0], results[1])
    assert np.array_equal(results[0].view(np.uint32), single.view(np.uint32))
    assert np.all(single[1] == 0) and np.any(single[0] != 0)
