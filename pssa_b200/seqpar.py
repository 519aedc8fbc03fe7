"""Sequence-parallel prefill: long sequences split in time over the ranks, one process per GPU.

Every rank holds a contiguous time shard of every sequence. Per block the library reduces a shard to one affine map
per (channel, state) (`compose_affine`, src/gpu_batch.rs:75-86: the sum of delta and the shard's end state from a zero
carry), asks this module for an all-gather of those maps (NCCL through `torch.distributed`, on the stream the library
runs on), folds the lower ranks' maps into its carry-in and runs the fused SSM; the rest of a block is token-local.
After the call every rank holds the same final recurrent state, so batched decode can continue on any of them.

The host logic here is the time sharding, the exchange callback, and picking each sequence's logits from the rank that
owns its last token.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _native as N


def time_shards(length: int, world: int):
    """Balanced contiguous split of `length` tokens over `world` ranks: [(start, stop)] per rank, earlier ranks take the
    remainder, so the first `length % world` shards are one token longer and empty shards only appear at the end."""
    if world < 1:
        raise ValueError(f"world size {world} must be positive")
    if length < 0:
        raise ValueError("sequence length must be non-negative")
    base, rem = divmod(int(length), world)
    out, start = [], 0
    for r in range(world):
        n = base + (1 if r < rem else 0)
        out.append((start, start + n))
        start += n
    return out


def last_token_owner(length: int, world: int) -> int:
    """Rank whose shard holds the last token (-1 for an empty sequence)."""
    owner = -1
    for r, (a, b) in enumerate(time_shards(length, world)):
        if b > a:
            owner = r
    return owner


def check_every_rank_has_tokens(lengths, world: int):
    """Raise unless every rank's packed shard holds at least one token. Decided from the global sequence lengths, which
    every rank holds identically, so that all ranks raise together and none is left waiting in the per-block all-gather
    for a peer that returned early."""
    for rank in range(world):
        if not any(time_shards(int(n), world)[rank][1] > time_shards(int(n), world)[rank][0] for n in lengths):
            raise ValueError(f"every rank needs at least one token: rank {rank} of {world} would hold none "
                             f"(longest sequence has {max([int(n) for n in lengths], default=0)} tokens)")


def pack_shard(prompts, world: int, rank: int):
    """This rank's shards of all prompts in the batched entry point's packed layout: (ids uint32, offsets, lengths)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    parts, lengths = [], []
    for p in prompts:
        a, b = time_shards(len(p), world)[rank]
        parts.append(np.asarray(p[a:b], dtype=np.uint32))
        lengths.append(b - a)
    lengths = np.asarray(lengths, dtype=np.uint32)
    offsets = np.zeros(len(prompts), dtype=np.uint32)
    if len(prompts) > 1:
        offsets[1:] = np.cumsum(lengths[:-1], dtype=np.uint64).astype(np.uint32)
    ids = np.concatenate(parts) if parts and int(lengths.sum()) else np.zeros(0, np.uint32)
    return ids, offsets, lengths


def select_owner_rows(per_rank_rows, lengths, world: int):
    """per_rank_rows [world, lanes, width]: keep, for every lane, the row of the rank that owns its last token
    (zeros for an empty sequence)."""
    per_rank_rows = np.asarray(per_rank_rows)
    out = np.zeros(per_rank_rows.shape[1:], dtype=per_rank_rows.dtype)
    for lane, n in enumerate(lengths):
        owner = last_token_owner(int(n), world)
        if owner >= 0:
            out[lane] = per_rank_rows[owner, lane]
    return out


class SequenceParallelPrefill:
    """Binds a `PSSAModel` replica to a process group for time-sharded prefill.

    Needs an initialised NCCL process group, the model's context on the calling thread's current torch stream
    (`gpu.set_stream(torch.cuda.current_stream())`), and the same weights, banks and recurrent state on every rank.
    """

    def __init__(self, model, group=None, max_lanes: int = 8):
        import torch
        import torch.distributed as dist

        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("sequence-parallel prefill needs an initialised torch.distributed process group")
        self.model, self.group = model, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.max_lanes = max_lanes
        rec = model.d_latent + model.d_latent * model.d_state
        capacity = max_lanes * 16  # records: the library cuts each lane's shard into up to 16 time chunks
        dev = torch.device("cuda", torch.cuda.current_device())
        self._send = torch.zeros(capacity * rec, dtype=torch.float32, device=dev)
        self._recv = torch.zeros(self.world * capacity * rec, dtype=torch.float32, device=dev)
        self._error = None

        def exchange(_arg, _send, _recv, nbytes):
            # the library has just written `nbytes` of self._send on the current stream; NCCL runs on that stream too
            try:
                n = nbytes // 4
                dist.all_gather_into_tensor(self._recv[: self.world * n], self._send[:n], group=self.group)
                return 0
            except Exception as exc:  # surfaces as an error status of the prefill call
                self._error = exc
                return 1

        self._callback = N.EXCHANGE_FN(exchange)  # keep alive as long as the library may call it
        model.gpu._check(model._lib.pssa_b200_model_set_seqpar(
            model._h, self.rank, self.world, C.c_void_p(self._send.data_ptr()), C.c_void_p(self._recv.data_ptr()),
            capacity, self._callback, None))

    def close(self):
        if self.model is not None and getattr(self.model, "_h", None):
            self.model._lib.pssa_b200_model_set_seqpar(self.model._h, 0, 1, None, None, 0, N.EXCHANGE_FN(0), None)
        self.model = None

    def prefill(self, prompts):
        """Prefill `prompts` (full sequences, identical on every rank; lane l uses stream l). Returns the
        [lanes, vocab] last-token logits on every rank."""
        import torch
        import torch.distributed as dist

        if len(prompts) > self.max_lanes:
            raise ValueError(f"{len(prompts)} sequences exceed the {self.max_lanes} lanes the exchange buffers hold")
        lengths = [len(p) for p in prompts]
        check_every_rank_has_tokens(lengths, self.world)  # the same verdict on every rank, before any device work
        ids, offsets, shard_len = pack_shard(prompts, self.world, self.rank)
        dev = self._send.device
        ids_dev = torch.from_numpy(ids.astype(np.int64)).to(torch.int32).to(dev)
        logits = torch.zeros(len(prompts), self.model.d_vocab, dtype=torch.float32, device=dev)
        try:
            self.model.prefill_batch_dev(ids_dev, offsets, shard_len, None, logits, None)
        except N.B200Error:
            if self._error is not None:
                raise self._error
            raise
        gathered = torch.empty(self.world, *logits.shape, dtype=torch.float32, device=dev)
        dist.all_gather_into_tensor(gathered, logits, group=self.group)
        return select_owner_rows(gathered.cpu().numpy(), lengths, self.world)
