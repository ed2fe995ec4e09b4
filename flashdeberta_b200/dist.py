"""Sequence sharding for multi-GPU inference: one process per GPU, no per-layer collective.

Every sequence's encoder forward is independent of every other one, so a batch is split across ranks by whole
sequences, balanced by token count; each rank runs the unmodified single-GPU path on its shard and the results are
brought together once at the end.  (The reference has no multi-device code at all.)
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def partition_by_tokens(lengths: Sequence[int], world_size: int, quadratic_weight: float = 0.0) -> List[List[int]]:
    """Split sequence indices into `world_size` bins with near-equal cost, longest first (LPT).

    cost(len) = len + quadratic_weight * len^2.  With the default weight 0 this is the balanced-token-count contract;
    a positive weight also balances the attention term.  Deterministic: ties go to the lower sequence index and the
    lower rank.  Returns, per rank, the indices it owns in increasing order.
    """
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    cost = [float(n) + quadratic_weight * float(n) * float(n) for n in lengths]
    order = sorted(range(len(lengths)), key=lambda i: (-cost[i], i))
    load = [0.0] * world_size
    bins: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda r: (load[r], r))
        bins[r].append(i)
        load[r] += cost[i]
    return [sorted(b) for b in bins]


def shard_batch(input_ids: torch.Tensor, attention_mask: torch.Tensor, rank: int, world_size: int,
                quadratic_weight: float = 0.0) -> Tuple[torch.Tensor, torch.Tensor, List[int]]:
    """This rank's rows of a right-padded (B, L) batch, cut to the longest sequence it owns."""
    lengths = attention_mask.sum(-1).tolist()
    mine = partition_by_tokens([int(x) for x in lengths], world_size, quadratic_weight)[rank]
    if not mine:
        return input_ids[:0], attention_mask[:0], mine
    idx = torch.tensor(mine, dtype=torch.long, device=input_ids.device)
    Lr = max(int(lengths[i]) for i in mine)
    return input_ids[idx, :Lr], attention_mask[idx, :Lr], mine


def gather_sequences(local: torch.Tensor, owned: Sequence[int], batch: int, seqlen: int,
                     group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """The single collective of a sharded forward: every rank contributes its (b_r, L_r, hid) result and receives the
    full (batch, seqlen, hid) tensor in the original sequence order (zeros where nothing was computed).

    Shards differ in size, so they are padded to the largest and exchanged with one all_gather; the index lists travel
    with all_gather_object.  Works on NCCL (GPU tensors) and gloo (CPU tensors)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        out = local.new_zeros(batch, seqlen, local.shape[-1])
        if len(owned):
            out[torch.tensor(list(owned), device=local.device), : local.shape[1]] = local
        return out
    world = dist.get_world_size(group)
    meta: List = [None] * world
    dist.all_gather_object(meta, (list(owned), tuple(local.shape)), group=group)
    hid = local.shape[-1]
    max_b = max(m[1][0] for m in meta)
    max_l = max(m[1][1] for m in meta)
    padded = local.new_zeros(max_b, max_l, hid)
    padded[: local.shape[0], : local.shape[1]] = local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded.contiguous(), group=group)
    out = local.new_zeros(batch, seqlen, hid)
    for (idx, shape), part in zip(meta, parts):
        if idx:
            out[torch.tensor(idx, device=local.device), : shape[1]] = part[: shape[0], : shape[1]]
    return out


@torch.no_grad()
def sharded_forward(model, input_ids: torch.Tensor, attention_mask: torch.Tensor, *, gather: bool = True,
                    quadratic_weight: float = 0.0, group: Optional[dist.ProcessGroup] = None):
    """Run `model` (replicated on every rank) on this rank's share of the batch.  Returns the gathered
    last_hidden_state (B, L, hid) when `gather` is set, else (local_hidden, owned_indices)."""
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    ids, mask, owned = shard_batch(input_ids, attention_mask, rank, world, quadratic_weight)
    if len(owned):
        hidden = model(input_ids=ids, attention_mask=mask).last_hidden_state
    else:
        hid = model.config.hidden_size
        hidden = torch.zeros(0, 1, hid, device=input_ids.device, dtype=next(model.parameters()).dtype)
    if not gather:
        return hidden, owned
    return gather_sequences(hidden, owned, input_ids.shape[0], input_ids.shape[1], group)
