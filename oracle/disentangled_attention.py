"""CPU oracle for DeBERTa-v2/v3 disentangled self-attention (forward only).

TEST INFRASTRUCTURE ONLY.  This file is a plain fp32 restatement of the eager
algorithm the reference falls back to (HuggingFace ``transformers``
``models/deberta_v2/modeling_deberta_v2.py``, version 5.5.0, which the
reference wires in at ``src/flashdeberta/model.py:11,254-257``).  Nothing in the
shipped package imports it; it is used by the tests, by the smoke check and by
the CPU-baseline leg of the benchmark as the checker.

Pinning: ``tests/golden/make_golden.py`` imports the real HuggingFace module in
a container that has it and stores its inputs and outputs as fixtures; the
CPU-only tests compare every function below against those fixtures.

Layout conventions used throughout:
  q, k, v       (rows, H, D) float32, ``rows`` = all tokens of all sequences
  pos_key/query (H, 2*span, D) float32 (already projected, per head)
  seq_start/len per-sequence first row and number of valid rows
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import numpy as np
import torch


# --------------------------------------------------------------------------- #
# integer path: log-bucket relative index
# --------------------------------------------------------------------------- #
def log_bucket_position(rel: np.ndarray, bucket_size: int, max_position: int) -> np.ndarray:
    """Signed bucket of a relative distance ``rel = q_pos - k_pos``.

    Follows ``make_log_bucket_position`` (modeling_deberta_v2.py:56-69): the
    identity for ``|rel| <= bucket_size//2``; beyond that
    ``sign * (ceil(log(|rel|/mid) / log((max_position-1)/mid) * (mid-1)) + mid)``
    evaluated in float32, exactly as torch does for an int64 input.
    """
    rel = np.asarray(rel, dtype=np.int64)
    mid = bucket_size // 2
    sign = np.sign(rel)
    inside = (rel < mid) & (rel > -mid)
    abs_pos = np.where(inside, mid - 1, np.abs(rel))
    # int64 / int -> float32 (torch default dtype), log in float32
    ratio = (abs_pos.astype(np.float32) / np.float32(mid)).astype(np.float32)
    denom = np.log(np.float32((max_position - 1) / mid)).astype(np.float32)
    with np.errstate(divide="ignore"):
        log_pos = np.ceil((np.log(ratio).astype(np.float32) / denom).astype(np.float32)
                          * np.float32(mid - 1)).astype(np.float32) + np.float32(mid)
    bucket = np.where(abs_pos <= mid, rel.astype(np.float32), log_pos * sign.astype(np.float32))
    return bucket.astype(np.int64)


def att_span(position_buckets: int, max_relative_positions: int) -> int:
    """Half the number of rows of the relative-embedding table
    (modeling_deberta_v2.py:168-174, ``pos_ebd_size``)."""
    return position_buckets if position_buckets > 0 else max_relative_positions


def relative_index(rel: np.ndarray, position_buckets: int, max_relative_positions: int) -> np.ndarray:
    """Row of the position tables addressed by distance ``rel``.

    ``clamp(bucket(rel) + span, 0, 2*span-1)`` — modeling_deberta_v2.py:96-98
    (bucketing only when both sizes are positive), :318 (c2p) and :336 (p2c; the
    bucket function is odd, so the p2c index of (q, k) equals the c2p index).
    """
    rel = np.asarray(rel, dtype=np.int64)
    span = att_span(position_buckets, max_relative_positions)
    if position_buckets > 0 and max_relative_positions > 0:
        b = log_bucket_position(rel, position_buckets, max_relative_positions)
    else:
        b = rel
    return np.clip(b + span, 0, 2 * span - 1).astype(np.int64)


# --------------------------------------------------------------------------- #
# floating-point path
# --------------------------------------------------------------------------- #
def sm_scale_for(head_dim: int, c2p: bool, p2c: bool) -> float:
    """1/sqrt(D * (1 + [c2p] + [p2c])) — modeling_deberta_v2.py:237-243."""
    return 1.0 / math.sqrt(head_dim * (1 + int(c2p) + int(p2c)))


@torch.no_grad()
def attention_core(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    pos_key: Optional[torch.Tensor],
    pos_query: Optional[torch.Tensor],
    seq_start: Sequence[int],
    seq_len: Sequence[int],
    sm_scale: float,
    position_buckets: int,
    max_relative_positions: int,
    row_block: int = 512,
    return_lse: bool = False,
):
    """softmax((QK^T + c2p + p2c) * sm_scale) V per sequence, fp32, blockwise.

    Restates modeling_deberta_v2.py:243-264 (scores, softmax, PV) and :313-343
    (the two gathered bias terms) without ever holding more than
    ``row_block x len`` scores.  Rows outside every sequence are left zero.
    Returns ``out`` (rows, H, D) and optionally the natural-log LSE (rows, H).
    """
    q = q.float(); k = k.float(); v = v.float()
    rows, H, D = q.shape
    out = torch.zeros(rows, H, D, dtype=torch.float32)
    lse = torch.zeros(rows, H, dtype=torch.float32)
    span = att_span(position_buckets, max_relative_positions)
    if pos_key is not None:
        pos_key = pos_key.float()[:, : 2 * span]
    if pos_query is not None:
        pos_query = pos_query.float()[:, : 2 * span]
    for s0, ln in zip(seq_start, seq_len):
        s0 = int(s0); ln = int(ln)
        if ln <= 0:
            continue
        ks = k[s0:s0 + ln].permute(1, 0, 2)  # (H, ln, D)
        vs = v[s0:s0 + ln].permute(1, 0, 2)
        p2c_all = None
        if pos_query is not None:
            p2c_all = torch.bmm(ks, pos_query.transpose(1, 2))  # (H, ln, 2span) rows = key
        kpos = np.arange(ln, dtype=np.int64)
        for m0 in range(0, ln, row_block):
            m1 = min(ln, m0 + row_block)
            qs = q[s0 + m0:s0 + m1].permute(1, 0, 2)  # (H, mb, D)
            scores = torch.bmm(qs, ks.transpose(1, 2))  # (H, mb, ln)
            if pos_key is not None or pos_query is not None:
                rel = np.arange(m0, m1, dtype=np.int64)[:, None] - kpos[None, :]
                idx = torch.from_numpy(relative_index(rel, position_buckets, max_relative_positions))
                idx_h = idx.unsqueeze(0).expand(H, -1, -1)
                if pos_key is not None:
                    c2p = torch.bmm(qs, pos_key.transpose(1, 2))  # (H, mb, 2span)
                    scores = scores + torch.gather(c2p, 2, idx_h)
                if pos_query is not None:
                    # p2c[m, n] = (K[n] . pos_query[idx(m - n)])
                    scores = scores + torch.gather(p2c_all, 2, idx_h.transpose(1, 2)).transpose(1, 2)
            scores = scores * sm_scale
            mx = scores.max(dim=-1, keepdim=True).values
            p = torch.exp(scores - mx)
            l = p.sum(dim=-1, keepdim=True)
            o = torch.bmm(p / l, vs)  # (H, mb, D)
            out[s0 + m0:s0 + m1] = o.permute(1, 0, 2)
            lse[s0 + m0:s0 + m1] = (mx + torch.log(l)).squeeze(-1).permute(1, 0)
    if return_lse:
        return out, lse
    return out


@torch.no_grad()
def project_positions(rel_embeddings: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                      num_heads: int) -> torch.Tensor:
    """Per-head projection of the relative-embedding table: (2span, hid) -> (H, 2span, D).
    modeling_deberta_v2.py:295-311."""
    y = torch.nn.functional.linear(rel_embeddings.float(), weight.float(), None if bias is None else bias.float())
    return y.view(y.shape[0], num_heads, -1).permute(1, 0, 2).contiguous()


@torch.no_grad()
def module_forward(
    hidden_states: torch.Tensor,
    seq_len: Sequence[int],
    rel_embeddings: Optional[torch.Tensor],
    state: dict,
    num_heads: int,
    position_buckets: int,
    max_relative_positions: int,
    pos_att_type: Sequence[str],
    share_att_key: bool,
    relative_attention: bool = True,
    query_states: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Whole attention sub-layer (modeling_deberta_v2.py:191-274) on a right-padded
    (B, L, hid) batch; ``state`` holds the module's parameters by their HuggingFace names
    (query_proj.weight, ..., pos_key_proj.weight, ...).  Padded rows come back zero."""
    B, L, hid = hidden_states.shape
    lin = torch.nn.functional.linear
    hs = hidden_states.float()
    qs = hs if query_states is None else query_states.float()
    g = lambda n: state[n].float() if n in state and state[n] is not None else None
    q = lin(qs, g("query_proj.weight"), g("query_proj.bias")).view(B * L, num_heads, -1)
    k = lin(hs, g("key_proj.weight"), g("key_proj.bias")).view(B * L, num_heads, -1)
    v = lin(hs, g("value_proj.weight"), g("value_proj.bias")).view(B * L, num_heads, -1)
    D = q.shape[-1]
    c2p = relative_attention and "c2p" in pos_att_type
    p2c = relative_attention and "p2c" in pos_att_type
    pos_key = pos_query = None
    if relative_attention:
        span = att_span(position_buckets, max_relative_positions)
        rel = rel_embeddings[: 2 * span]
        if share_att_key:
            if c2p:
                pos_key = project_positions(rel, g("key_proj.weight"), g("key_proj.bias"), num_heads)
            if p2c:
                pos_query = project_positions(rel, g("query_proj.weight"), g("query_proj.bias"), num_heads)
        else:
            if c2p:
                pos_key = project_positions(rel, g("pos_key_proj.weight"), g("pos_key_proj.bias"), num_heads)
            if p2c:
                pos_query = project_positions(rel, g("pos_query_proj.weight"), g("pos_query_proj.bias"), num_heads)
    out = attention_core(
        q, k, v, pos_key, pos_query,
        [b * L for b in range(B)], list(seq_len),
        sm_scale_for(D, c2p, p2c), position_buckets, max_relative_positions,
    )
    return out.view(B, L, num_heads * D)


# --------------------------------------------------------------------------- #
# FP8 (e4m3) expectation model: same math on operands rounded through e4m3
# --------------------------------------------------------------------------- #
def fake_quant_e4m3(x: torch.Tensor, dims: Sequence[int]):
    """Round ``x`` through float8-e4m3 with one scale per slab reduced over ``dims``
    (scale = amax/448).  Returns (dequantised x, scale).  Used to tell quantisation
    noise from kernel bugs; there is no FP8 code in the reference to follow."""
    amax = x.abs().amax(dim=tuple(dims), keepdim=True).clamp_min(1e-12)
    scale = amax / 448.0
    xq = (x / scale).to(torch.float8_e4m3fn).to(torch.float32)
    return xq * scale, scale
