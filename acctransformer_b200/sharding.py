"""Sharding of (batch, head) units over the GPUs of one box.

Every (batch, head) slice of q, k, v, dropout mask, alibi, O, L, dQ, dK, dV is independent (the
reference encodes exactly this in its shard strategy: tensors mapped on [dp, mp, 1, 1], the mask on
dp only -- train/acctransformer/flash_attention/nn/layer/flash_attention.py:146-177), so a rank
takes a contiguous run of units and no data crosses between ranks.  The only communication is the
reduction of the timing (max over ranks), which works on any torch.distributed backend.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def unit_slice(total_units, rank, world):
    """Contiguous [start, stop) of the flattened (batch*head) units owned by ``rank``; the first
    ``total_units % world`` ranks get one extra unit."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(total_units, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_bnsd(t, rank, world):
    """View of units [start, stop) of a [B, N, S, D] tensor as [1, units, S, D] (no copy when contiguous)."""
    B, N = t.shape[0], t.shape[1]
    start, stop = unit_slice(B * N, rank, world)
    return t.reshape(1, B * N, *t.shape[2:])[:, start:stop]


def max_over_ranks(value, device="cpu"):
    """Max of a python float over all ranks (identity when torch.distributed is not initialised)."""
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
