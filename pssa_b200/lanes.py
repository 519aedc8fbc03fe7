"""Sharding independent sequences (lanes) over ranks, one process per GPU.

The reference batches independent sequences as lanes of one packed row matrix (`SequenceBatch`,
src/sequence_batch.rs:233-384): every lane has its own recurrent state and nothing flows between lanes. That
independence is what makes the path data parallel: each rank prefills its own lanes against a replicated copy of
the weights and banks, and no collective runs on the data path. The only exchange is the optional gather of the
per-lane results (last-token logits or greedy tokens) back to every rank, which is host logic and works over any
`torch.distributed` backend (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


def partition_lanes(lengths, world: int):
    """Deterministic balanced assignment of lanes to ranks.

    Longest-processing-time-first on token counts: lanes are taken longest first (ties by index) and each goes to
    the rank with the fewest tokens so far (ties by rank). Returns a list of `world` sorted index arrays that
    together cover every lane exactly once; empty lanes are assigned too so results keep one row per lane.
    """
    if world < 1:
        raise ValueError(f"world size {world} must be positive")
    lengths = np.asarray(lengths, dtype=np.int64)
    if lengths.ndim != 1:
        raise ValueError("lane lengths must be one-dimensional")
    if np.any(lengths < 0):
        raise ValueError("lane lengths must be non-negative")
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    load = [0] * world
    count = [0] * world
    owned = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda q: (load[q], count[q], q))
        owned[r].append(i)
        load[r] += int(lengths[i])
        count[r] += 1
    return [np.array(sorted(o), dtype=np.int64) for o in owned]


@dataclass
class LaneShard:
    """The lanes one rank owns, packed the way the batched entry points take them."""
    lane_ids: np.ndarray   # global lane indices, ascending
    ids: np.ndarray        # packed token ids of the owned lanes (uint64)
    offsets: np.ndarray    # first packed row of each owned lane (uint32)
    lengths: np.ndarray    # tokens per owned lane (uint32)


def shard_prompts(prompts, world: int, rank: int) -> LaneShard:
    """Pack the prompts (a list of 1-D integer arrays) this rank owns."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    lengths = np.array([len(p) for p in prompts], dtype=np.int64)
    mine = partition_lanes(lengths, world)[rank]
    own_len = lengths[mine].astype(np.uint32)
    offsets = np.zeros(len(mine), dtype=np.uint32)
    if len(mine) > 1:
        offsets[1:] = np.cumsum(own_len[:-1], dtype=np.uint64).astype(np.uint32)
    if len(mine) and int(own_len.sum()) > 0:
        ids = np.concatenate([np.asarray(prompts[i], dtype=np.uint64) for i in mine])
    else:
        ids = np.zeros(0, dtype=np.uint64)
    return LaneShard(mine, ids, offsets, own_len)


def gather_lane_rows(local_rows, lane_ids, n_lanes: int, group=None):
    """All ranks receive the [n_lanes, width] matrix assembled from every rank's per-lane rows.

    `local_rows` is this rank's [len(lane_ids), width] float32 result (last-token logits, say). Ranks may own
    different numbers of lanes, so rows travel padded to the largest shard together with their lane indices.
    Without an initialised process group (one process) the rows are only reordered.
    """
    import torch
    import torch.distributed as dist

    local_rows = np.ascontiguousarray(local_rows, dtype=np.float32)
    lane_ids = np.asarray(lane_ids, dtype=np.int64)
    if local_rows.ndim != 2 or local_rows.shape[0] != len(lane_ids):
        raise ValueError(f"expected one row per owned lane: rows {local_rows.shape}, lanes {len(lane_ids)}")
    width = local_rows.shape[1]
    out = np.zeros((n_lanes, width), dtype=np.float32)
    if not (dist.is_available() and dist.is_initialized()):
        out[lane_ids] = local_rows
        return out
    world = dist.get_world_size(group)
    device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else torch.device("cpu")
    n_max = torch.tensor([len(lane_ids)], dtype=torch.int64, device=device)
    dist.all_reduce(n_max, op=dist.ReduceOp.MAX, group=group)
    n_max = int(n_max.item())
    pad_ids = torch.full((n_max,), -1, dtype=torch.int64, device=device)
    pad_rows = torch.zeros((n_max, width), dtype=torch.float32, device=device)
    if len(lane_ids):
        pad_ids[: len(lane_ids)] = torch.from_numpy(lane_ids).to(device)
        pad_rows[: len(lane_ids)] = torch.from_numpy(local_rows).to(device)
    all_ids = [torch.empty_like(pad_ids) for _ in range(world)]
    all_rows = [torch.empty_like(pad_rows) for _ in range(world)]
    dist.all_gather(all_ids, pad_ids, group=group)
    dist.all_gather(all_rows, pad_rows, group=group)
    seen = np.zeros(n_lanes, dtype=bool)
    for ids_t, rows_t in zip(all_ids, all_rows):
        ids_np = ids_t.cpu().numpy()
        keep = ids_np >= 0
        if np.any(seen[ids_np[keep]]):
            raise RuntimeError("a lane was reported by two ranks: the partition is not the same on every rank")
        seen[ids_np[keep]] = True
        out[ids_np[keep]] = rows_t.cpu().numpy()[keep]
    if not seen.all():
        raise RuntimeError(f"{int((~seen).sum())} lanes were reported by no rank")
    return out


def sharded_prefill(model, prompts, world: int, rank: int, group=None):
    """Prefill `prompts` across `world` ranks and return the [n_lanes, vocab] last-token logits on every rank.

    `model` is this rank's replica: anything whose `prefill_batch(list_of_id_sequences)` returns
    `(logits [n, vocab], greedy)` with one row per sequence, like `PSSAModel.prefill_batch`. Owned lane l runs on the
    replica's stream l. Lanes with no tokens return a zero row, as the batched entry point leaves them.
    """
    shard = shard_prompts(prompts, world, rank)
    if len(shard.lane_ids):
        logits, _ = model.prefill_batch([prompts[i] for i in shard.lane_ids])
        rows = np.asarray(logits, dtype=np.float32)
    else:
        rows = np.zeros((0, model.d_vocab), dtype=np.float32)
    return gather_lane_rows(rows, shard.lane_ids, len(prompts), group)
