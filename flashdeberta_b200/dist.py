"""Sequence sharding for multi-GPU inference: one process per GPU, no per-layer collective.

Every sequence's encoder forward is independent of every other one, so a batch is split across ranks by whole
sequences, balanced by token count (or by a cost that also counts the attention's quadratic term); each rank runs the
unmodified single-GPU path on its shard of packed tokens and the results are brought together once at the end, as packed
rows: one ``all_gather`` of (T_r, hidden) shards padded to the largest T_r (the shards are balanced, so the padding is a
few rows), then one row gather back into the original sequence order.  (The reference has no multi-device code at all.)

Nothing but the result rows crosses ranks: the partition is a deterministic function of the sequence lengths, which every
rank has, so each rank works out everybody's share by itself.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

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


def quadratic_weight_from_times(step_ms: float, attn_ms: float, lengths: Sequence[int], head_dim: int = 64,
                                att_span: int = 256) -> float:
    """The weight of len^2 against len in a sequence's cost, from one measured step over `lengths`: the part of the
    attention time that belongs to Q.K^T and P.V (4 l^2 D of the attention's 4 l^2 D + 4 l 2S D FLOPs) grows with l^2,
    everything else (the rest of the attention, the linear layers) with l."""
    s1 = float(sum(lengths))
    s2 = float(sum(n * n for n in lengths))
    if s1 <= 0 or s2 <= 0 or step_ms <= 0:
        return 0.0
    f_quad = 4.0 * s2 * head_dim
    f_pos = 4.0 * s1 * 2 * att_span * head_dim
    t_quad = attn_ms * f_quad / (f_quad + f_pos)
    t_lin = max(step_ms - t_quad, 1e-9)
    return (t_quad / s2) / (t_lin / s1)


class ShardPlan:
    """Who owns what, for one list of sequence lengths and one world size: per rank the sequences it owns, its packed
    ``cu_seqlens``, and the row permutation that puts the gathered shards back into the original packed order."""

    def __init__(self, lengths: Sequence[int], world_size: int, quadratic_weight: float = 0.0):
        self.lengths = [int(n) for n in lengths]
        self.world = int(world_size)
        self.bins = partition_by_tokens(self.lengths, self.world, quadratic_weight)
        self.tokens = [sum(self.lengths[i] for i in b) for b in self.bins]
        self.max_tokens = max(self.tokens) if self.tokens else 0
        self.total = sum(self.lengths)
        self._perm: Dict[str, torch.Tensor] = {}

    def cu_seqlens(self, rank: int) -> List[int]:
        cu = [0]
        for i in self.bins[rank]:
            cu.append(cu[-1] + self.lengths[i])
        return cu

    def max_seqlen(self, rank: int) -> int:
        return max((self.lengths[i] for i in self.bins[rank]), default=0)

    def local_rows(self, rank: int) -> torch.Tensor:
        """Rows of the original packed batch (all sequences back to back) that `rank` owns, in its own packed order."""
        start = [0]
        for n in self.lengths:
            start.append(start[-1] + n)
        pieces = [torch.arange(start[i], start[i + 1]) for i in self.bins[rank]]
        return torch.cat(pieces) if pieces else torch.zeros(0, dtype=torch.long)

    def gather_permutation(self, device) -> torch.Tensor:
        """perm[t] = row of the (world * max_tokens) gathered buffer that holds row t of the original packed batch."""
        key = str(device)
        if key not in self._perm:
            perm = torch.empty(self.total, dtype=torch.long)
            for r in range(self.world):
                rows = self.local_rows(r)
                perm[rows] = r * self.max_tokens + torch.arange(rows.numel())
            self._perm[key] = perm.to(device)
        return self._perm[key]


def gather_packed(local: torch.Tensor, plan: ShardPlan, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """The single collective of a sharded forward.  `local`: this rank's (T_r, hidden) result rows in its own packed order.
    Returns the (T, hidden) rows of the whole batch in the original packed order, on every rank."""
    world = plan.world
    if world == 1 or not dist.is_initialized():
        return local  # one rank owns every sequence, in the original order
    hid = local.shape[-1]
    buf = local.new_empty(world, plan.max_tokens, hid)
    mine = buf[dist.get_rank(group)]
    mine[: local.shape[0]].copy_(local)
    if local.shape[0] < plan.max_tokens:
        mine[local.shape[0]:].zero_()
    dist.all_gather(list(buf.unbind(0)), mine, group=group)
    return buf.view(world * plan.max_tokens, hid).index_select(0, plan.gather_permutation(local.device))


@torch.no_grad()
def sharded_forward_packed(model, packed_ids: torch.Tensor, plan: ShardPlan, *, gather: bool = True,
                           group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Run `model` (replicated on every rank) on this rank's share of a packed batch.  `packed_ids`: (T_r,) token ids
    of the sequences this rank owns, back to back in the order of ``plan.bins[rank]`` (take ``ids[plan.local_rows(rank)]``
    of the whole batch).  Returns the gathered (T, hidden) last hidden state in the original packed order, or this rank's
    own (T_r, hidden) rows when `gather` is off."""
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    cu = torch.tensor(plan.cu_seqlens(rank), dtype=torch.int32, device=packed_ids.device)
    if packed_ids.numel():
        hidden = model(input_ids=packed_ids.view(1, -1), cu_seqlens=cu, max_seqlen=plan.max_seqlen(rank)).last_hidden_state[0]
    else:
        hidden = torch.zeros(0, model.config.hidden_size, device=packed_ids.device, dtype=next(model.parameters()).dtype)
    return gather_packed(hidden, plan, group) if gather else hidden


# ---------------------------------------------------------------------------------------------------------------------
# padded batches: the same exchange behind a (B, L) interface
# ---------------------------------------------------------------------------------------------------------------------
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


def gather_sequences(local: torch.Tensor, lengths: Sequence[int], seqlen: int, rank: int, world_size: int,
                     quadratic_weight: float = 0.0, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Padded form of the final exchange: `local` is this rank's (b_r, L_r, hidden) result for the sequences
    ``partition_by_tokens(lengths, world_size)[rank]`` (right-padded); returns (batch, seqlen, hidden) in the original
    order with zeros in the padding.  Only the valid rows travel: the shard is packed, exchanged by ``gather_packed`` and
    unpacked once."""
    plan = ShardPlan(lengths, world_size, quadratic_weight)
    owned = plan.bins[rank]
    hid = local.shape[-1]
    rows = [local[b, : plan.lengths[i]] for b, i in enumerate(owned)]
    packed = torch.cat(rows) if rows else local.new_zeros(0, hid)
    full = gather_packed(packed, plan, group)  # (T, hid), original packed order
    out = local.new_zeros(len(plan.lengths) * seqlen, hid)
    dest = torch.cat([torch.arange(n) + b * seqlen for b, n in enumerate(plan.lengths)]) if plan.total else torch.zeros(0, dtype=torch.long)
    out.index_copy_(0, dest.to(local.device), full)
    return out.view(len(plan.lengths), seqlen, hid)


@torch.no_grad()
def sharded_forward(model, input_ids: torch.Tensor, attention_mask: torch.Tensor, *, gather: bool = True,
                    quadratic_weight: float = 0.0, group: Optional[dist.ProcessGroup] = None):
    """Run `model` (replicated on every rank) on this rank's share of a right-padded batch.  Returns the gathered
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
    lengths = [int(x) for x in attention_mask.sum(-1).tolist()]
    return gather_sequences(hidden, lengths, input_ids.shape[1], rank, world, quadratic_weight, group)
