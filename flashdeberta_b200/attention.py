"""Disentangled self-attention module with the fused sm_100a core.

Same constructor, parameter names and ``forward`` signature as the reference's ``FlashDisentangledSelfAttention``
(src/flashdeberta/model.py:97-252), which itself subclasses transformers' ``DisentangledSelfAttention``
(models/deberta_v2/modeling_deberta_v2.py:137-184 for the parameters), so checkpoints and call sites carry over.
What differs inside:

* no ``q @ pos_key^T`` / ``k @ pos_query^T`` bias tensors (model.py:189-192, :210-214): the kernel takes the projected
  position tables and contracts them per tile;
* no pack / unpack per layer (model.py:216-231, :249): padded batches are handled in place from per-sequence lengths;
* the mask may arrive as (B, L), as the (B, 1, L, L) tensor transformers' encoder builds, or as a (B,) int tensor of
  lengths (what this package's encoder passes); right padding is assumed, as in the reference's varlen path.
"""
from __future__ import annotations

import math
import warnings
from typing import Optional

import torch
from transformers.models.deberta_v2.modeling_deberta_v2 import DisentangledSelfAttention

from . import _lib, ops

_warned_general = False


class PackedSequences:
    """What travels through the layers in place of the attention mask when the encoder runs on packed tokens: the
    batch is one (1, T, hidden) row of all valid tokens, sequence b owning rows cu_seqlens[b] .. cu_seqlens[b+1]
    (same role as the (cu_seqlens, max_seqlen) pair of src/flashdeberta/model.py:233-234, made once per model forward
    instead of once per layer)."""

    def __init__(self, cu_seqlens: torch.Tensor, max_seqlen: int, indices: torch.Tensor, batch: int, seqlen: int):
        self.cu_seqlens, self.max_seqlen, self.indices = cu_seqlens, int(max_seqlen), indices
        self.batch, self.seqlen = int(batch), int(seqlen)

    @classmethod
    def from_mask(cls, mask2d: torch.Tensor, device=None) -> Optional["PackedSequences"]:
        """None when the batch has no padding.  One host read (total tokens and longest sequence) per model forward; the
        reference does one per sequence per layer (src/flashdeberta/ops/flash_attention_varlen.py:71-83) plus one per
        layer (padding.py:82).  With a mask on the host the read waits for nothing; ``device`` is then where the index
        tensors go."""
        m = mask2d != 0
        lens = m.sum(dim=-1, dtype=torch.int32)
        if lens.numel() == 0:
            return None
        total, max_len = torch.stack([lens.sum(), lens.max()]).tolist()
        if total == mask2d.numel():
            return None
        cu = torch.zeros(lens.numel() + 1, dtype=torch.int32, device=mask2d.device)
        cu[1:] = torch.cumsum(lens, 0)
        indices = torch.nonzero(m.flatten(), as_tuple=False).flatten()
        if device is not None and cu.device != torch.device(device):
            cu, indices = cu.to(device, non_blocking=True), indices.to(device, non_blocking=True)
        return cls(cu, max_len, indices, mask2d.shape[0], mask2d.shape[1])

    def pack(self, x: torch.Tensor) -> torch.Tensor:
        """(B, L, ...) -> (1, T, ...)"""
        return x.reshape(self.batch * self.seqlen, *x.shape[2:]).index_select(0, self.indices).unsqueeze(0)

    def unpack(self, x: torch.Tensor) -> torch.Tensor:
        """(1, T, ...) -> (B, L, ...) with zeros in the padding (src/flashdeberta/padding.py:30-44)."""
        out = x.new_zeros(self.batch * self.seqlen, *x.shape[2:])
        out.index_copy_(0, self.indices, x[0])
        return out.view(self.batch, self.seqlen, *x.shape[2:])


def lengths_from_mask(attention_mask: Optional[torch.Tensor], check: bool = True) -> Optional[torch.Tensor]:
    """Per-sequence valid lengths (int32, on the mask's device) from any of the mask forms the module is handed.
    Returns None for "everything valid".  No host synchronisation.

    The dense kernel path addresses a sequence by its length alone, so the valid tokens must be a prefix of each row
    (right padding).  The reference un-pads through the mask's indices and takes any layout
    (src/flashdeberta/padding.py:113-166); here other layouts go through ``PackedSequences`` (what the encoder does for any
    padded batch), and a mask that is not a prefix is refused: a ValueError for a mask on the host, the FDB_DEV_BAD_MASK bit
    of the device status word (raised by ``ops.check_status``) for a mask on the device."""
    if attention_mask is None:
        return None
    m = attention_mask
    if m.dim() == 1:  # already lengths
        return m.to(torch.int32)
    if m.dim() == 4:  # (B, 1, L, L), entry (i, j) = valid_i * valid_j: the diagonal says which tokens are valid
        m = torch.diagonal(m[:, 0], dim1=-2, dim2=-1)
    elif m.dim() == 3:  # (B, L, L)
        m = torch.diagonal(m, dim1=-2, dim2=-1)
    elif m.dim() != 2:
        raise ValueError(f"attention_mask with {attention_mask.dim()} dims is not supported")
    valid = m != 0
    lens = valid.sum(dim=-1, dtype=torch.int32)
    if check and not torch.compiler.is_compiling():
        prefix = torch.arange(m.shape[-1], device=m.device)[None, :] < lens[:, None]
        bad = (valid != prefix).any()
        if m.device.type == "cpu":
            if bool(bad):
                raise ValueError("attention_mask is not right-padded: the valid tokens of every row must come first "
                                 "(pack the batch, e.g. through FlashDebertaV2Model, to use other layouts)")
        else:
            ops.flag_status(m.device, bad, _lib.FDB_DEV_BAD_MASK)
    return lens


class FlashDisentangledSelfAttention(DisentangledSelfAttention):
    """Drop-in for src/flashdeberta/model.py:97 of the reference."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._pos_cache = None
        self._prepared = ops.PreparedWorkspace()  # this module's workspace: gathered tables and tile order are kept
        config = args[0] if args else kwargs.get("config")
        # FP8-e4m3 attention (per-head amax scales); a new switch, the reference has no FP8 path
        self.attn_fp8 = bool(getattr(config, "attn_fp8", False))

    # -- position tables ------------------------------------------------------------------------------------------------
    def _heads_first(self, x: torch.Tensor) -> torch.Tensor:
        # (rows, H*D) -> (H, rows, D)
        return x.view(x.shape[0], self.num_attention_heads, -1).permute(1, 0, 2).contiguous()

    def _position_tables(self, rel_embeddings: torch.Tensor, dtype: torch.dtype):
        """pos_key_layer / pos_query_layer of model.py:159-177, head-major (H, 2*span, D).  They do not depend on the
        input, so in eval mode they are kept until a parameter or the embedding table changes."""
        c2p = "c2p" in self.pos_att_type
        p2c = "p2c" in self.pos_att_type
        if self.share_att_key:
            wk, wq = self.key_proj, self.query_proj
        else:
            wk, wq = getattr(self, "pos_key_proj", None), getattr(self, "pos_query_proj", None)
        key = None
        if not self.training and not torch.is_grad_enabled() and not torch.compiler.is_compiling():
            # the table is kept alive below, so its identity stays its own
            key = (id(rel_embeddings), ops.tensor_stamp(rel_embeddings, held=True), rel_embeddings.device, dtype,
                   tuple(ops.tensor_stamp(p, held=True) for m in (wk, wq) if m is not None for p in m.parameters()))
            if self._pos_cache is not None and self._pos_cache[0] == key:
                return self._pos_cache[1], self._pos_cache[2]
        span2 = 2 * self.pos_ebd_size
        rel = self.pos_dropout(rel_embeddings)[:span2]
        pos_key = self._heads_first(wk(rel)).to(dtype) if c2p else None
        pos_query = self._heads_first(wq(rel)).to(dtype) if p2c else None
        if key is not None:
            self._pos_cache = (key, pos_key, pos_query, rel_embeddings)  # keep the table alive so id() stays unique
        return pos_key, pos_query

    def _forward_general(self, q, k, v, pos_key, pos_query, attention_mask, sm_scale, buckets, max_rel, in_dtype):
        """Head sizes other than 64 (up to 128; the reference's test has one such shape, tests/attention.py:87-89, no
        DeBERTa checkpoint has): the library's general kernel, fp32 arithmetic on CUDA cores.  Correct and slow (it is the
        kernel the fused one is validated with); forward only."""
        B, L, H, D = q.shape
        if D > 128:
            raise ValueError(f"head size {D} is not supported (64 on the fused kernel, up to 128 on the general one)")
        if ops.wants_grad(q, k, v, pos_key, pos_query) or self.attn_fp8:
            raise RuntimeError("training and e4m3 attention need a head size of 64")
        global _warned_general
        if not _warned_general:
            warnings.warn(f"flashdeberta_b200: head size {D} runs on the general CUDA-core kernel, far below the speed of the "
                          "fused kernel (head size 64)")
            _warned_general = True
        if isinstance(attention_mask, PackedSequences):
            pk = attention_mask
            out = ops.disentangled_attention_check(q.view(L, H, D), k.view(L, H, D), v.view(L, H, D), pos_key, pos_query,
                                                   cu_seqlens=pk.cu_seqlens, max_seqlen=pk.max_seqlen, sm_scale=sm_scale,
                                                   position_buckets=buckets, max_relative_positions=max_rel)
        else:
            out = ops.disentangled_attention_check(q, k, v, pos_key, pos_query, seq_lens=lengths_from_mask(attention_mask),
                                                   max_seqlen=L, sm_scale=sm_scale, position_buckets=buckets,
                                                   max_relative_positions=max_rel)
        out = out.reshape(B, L, H * D)
        return (out if out.dtype == in_dtype else out.to(in_dtype), None)

    # -- forward -------------------------------------------------------------------------------------------------------------
    def forward(self, hidden_states, attention_mask, output_attentions=False, query_states=None, relative_pos=None,
                rel_embeddings=None):
        """Returns ``(context (B, L, hidden), None)`` like model.py:252.  ``relative_pos`` is ignored, as in the
        reference (model.py:105): positions are always 0..len-1 inside each sequence.  Padded rows come back zero."""
        if output_attentions:
            raise ValueError("the fused attention never materialises attention probabilities; "
                             "use the eager implementation for output_attentions=True")
        if query_states is None:
            query_states = hidden_states
        B, L, _ = hidden_states.shape
        H, D = self.num_attention_heads, self.attention_head_size
        in_dtype = hidden_states.dtype

        q = self.query_proj(query_states).view(B, L, H, D)
        k = self.key_proj(hidden_states).view(B, L, H, D)
        v = self.value_proj(hidden_states).view(B, L, H, D)

        scale_factor = 1 + int("c2p" in self.pos_att_type) + int("p2c" in self.pos_att_type)
        sm_scale = 1.0 / math.sqrt(D * scale_factor)

        pos_key = pos_query = None
        buckets, max_rel = -1, -1
        if self.relative_attention and scale_factor > 1:
            if rel_embeddings is None:
                raise ValueError("rel_embeddings is required when relative_attention is on")
            # the general kernel (head sizes other than 64) also computes in fp32 from fp32 inputs: no rounding at all
            table_dtype = torch.float32 if (D != 64 and in_dtype == torch.float32) else torch.bfloat16
            pos_key, pos_query = self._position_tables(rel_embeddings, table_dtype)
            buckets, max_rel = self.position_buckets, self.max_relative_positions

        if D != 64:
            if in_dtype not in (torch.float32, torch.bfloat16):
                q, k, v = q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)
            return self._forward_general(q, k, v, pos_key, pos_query, attention_mask, sm_scale, buckets, max_rel, in_dtype)
        if in_dtype != torch.bfloat16:
            q, k, v = q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)
        if isinstance(attention_mask, PackedSequences):
            # packed tokens: hidden_states is (1, T, hidden); every sequence is addressed through cu_seqlens
            pk = attention_mask
            kw = dict(cu_seqlens=pk.cu_seqlens, max_seqlen=pk.max_seqlen, sm_scale=sm_scale, position_buckets=buckets,
                      max_relative_positions=max_rel)
            if self.attn_fp8:
                out = ops.disentangled_attention_fp8(q.view(L, H, D), k.view(L, H, D), v.view(L, H, D), pos_key, pos_query, **kw)
            elif ops.wants_grad(q, k, v, pos_key, pos_query):  # training: the op with a backward
                out = ops.attn_fwd_train_op(q.view(L, H, D), k.view(L, H, D), v.view(L, H, D), pos_key, pos_query,
                                            pk.cu_seqlens, None, pk.max_seqlen, sm_scale, buckets, max_rel)[0]
            else:
                out = ops.disentangled_attention(q.view(L, H, D), k.view(L, H, D), v.view(L, H, D), pos_key, pos_query,
                                                 prepared=self._prepared, **kw)
            out = out.view(B, L, H * D)
            return (out if in_dtype == torch.bfloat16 else out.to(in_dtype), None)
        seq_lens = lengths_from_mask(attention_mask)
        if self.attn_fp8:
            out = ops.disentangled_attention_fp8(q, k, v, pos_key, pos_query, seq_lens=seq_lens, max_seqlen=L,
                                                 sm_scale=sm_scale, position_buckets=buckets,
                                                 max_relative_positions=max_rel)
        elif ops.wants_grad(q, k, v, pos_key, pos_query):  # training: output and LSE kept for the backward
            out = ops.attn_fwd_train_op(q, k, v, pos_key, pos_query, None, seq_lens, L, sm_scale, buckets, max_rel)[0]
        elif torch.compiler.is_compiling():
            out = ops.attn_fwd_op(q, k, v, pos_key, pos_query, None, seq_lens, L, sm_scale, buckets, max_rel)
        else:
            out = ops.disentangled_attention(q, k, v, pos_key, pos_query, seq_lens=seq_lens, max_seqlen=L,
                                             sm_scale=sm_scale, position_buckets=buckets,
                                             max_relative_positions=max_rel, prepared=self._prepared)
        out = out.view(B, L, H * D)
        if in_dtype != torch.bfloat16:
            out = out.to(in_dtype)
        return (out, None)
