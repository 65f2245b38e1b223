"""Host-side sharding of independent sequences over ranks (one process per GPU).

Sequences never interact, so the token path has no collective: each rank owns a
contiguous block of global sequence ids, derives that block's prompts and sampler
draws from per-sequence seeds (so a sequence is identical whichever GPU it lands
on), and the finished ids are collected once at the end.
"""
from __future__ import annotations

import numpy as np


def shard_range(n_total: int, world: int, rank: int):
    """Contiguous block of global sequence ids owned by `rank` (sizes differ by at most one)."""
    base, extra = divmod(n_total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def seq_prompt(seed: int, global_seq: int, vocab: int, n: int):
    return np.random.default_rng([seed, global_seq]).integers(0, vocab, n).astype(np.int32)


def seq_draws(seed: int, global_seq: int, n: int):
    return np.random.default_rng([seed + 1, global_seq]).random(n, dtype=np.float32)


def pad_ids(seqs, width: int, fill: int = -1):
    out = np.full((len(seqs), width), fill, np.int32)
    for i, s in enumerate(seqs):
        out[i, :len(s)] = s
    return out


def gather_ids(local_table, world: int, device=None):
    """All ranks' id tables stacked in rank order: one all_gather (NCCL on GPU tensors, gloo on CPU).
    Ranks must hold equally many rows; returns a numpy array [world * rows, width]."""
    import torch
    import torch.distributed as dist

    if world == 1:
        return np.ascontiguousarray(local_table)  # nothing to exchange
    t = torch.from_numpy(np.ascontiguousarray(local_table))
    if device is not None:
        t = t.to(device)
    parts = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(parts, t)
    return torch.cat(parts).cpu().numpy()


def max_over_ranks(values, world: int, device=None):
    """Element-wise maximum of a small list of floats over all ranks (timings)."""
    import torch
    import torch.distributed as dist

    t = torch.tensor(list(values), dtype=torch.float64, device=device if device is not None else "cpu")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.cpu()]
