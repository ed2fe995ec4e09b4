"""DeBERTa-v2/v3 backbone and task heads with the fused attention core.

Thin subclasses of transformers' DeBERTa-v2 classes, exposing the names the reference exports
(src/flashdeberta/__init__.py:1-9; classes at src/flashdeberta/model.py:259-920).  Parameter names and shapes are
those of transformers, so stock checkpoints load unchanged.  Differences from the reference's wrappers:

* the encoder hands every layer the per-sequence lengths (B,) instead of a (B, 1, L, L) mask and never builds the
  (1, L, L) int64 relative-position matrix the flash path ignores (the reference inherits both from
  transformers' encoder forward, src/flashdeberta/model.py:275-310);
* a batch with padding is packed once after the embeddings, every layer (attention, dense, LayerNorm, FFN) runs on the
  (1, T, hidden) row of valid tokens, and the result is unpacked once at the end (``config.pack_sequences``, default on;
  the reference packs and unpacks q, k, v and both bias tensors inside every layer, model.py:216-231, :249);
* ``config.attn_backend`` chooses the attention core: ``"b200"`` (default, fused kernel) or ``"eager"``
  (transformers' own module).  The reference keys the same switch on ``config._attn_implementation``
  (model.py:254-262), which transformers 5 reserves for its own back-ends.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn
from transformers.modeling_outputs import BaseModelOutput
from transformers.models.deberta_v2.configuration_deberta_v2 import DebertaV2Config
from transformers.models.deberta_v2.modeling_deberta_v2 import (
    DebertaV2Attention,
    DebertaV2Embeddings,
    DebertaV2Encoder,
    DebertaV2ForMaskedLM,
    DebertaV2ForMultipleChoice,
    DebertaV2ForQuestionAnswering,
    DebertaV2ForSequenceClassification,
    DebertaV2ForTokenClassification,
    DebertaV2Intermediate,
    DebertaV2Layer,
    DebertaV2Model,
    DebertaV2Output,
    DebertaV2SelfOutput,
    DebertaV2PreTrainedModel,
    DisentangledSelfAttention,
)

from . import ops
from .attention import FlashDisentangledSelfAttention, PackedSequences, lengths_from_mask

__all__ = [
    "DEBERTA_SELF_ATTENTION_CLASSES", "FlashDebertaV2Attention", "FlashDebertaV2Layer", "FlashDebertaV2Encoder",
    "FlashDebertaV2PreTrainedModel", "FlashDebertaV2Model", "FlashDebertaV2ForMaskedLM",
    "FlashDebertaV2ForSequenceClassification", "FlashDebertaV2ForTokenClassification",
    "FlashDebertaV2ForQuestionAnswering", "FlashDebertaV2ForMultipleChoice",
]

# same role as DEBERTA_SELF_ATTENTION_CLASSES at src/flashdeberta/model.py:254-257
DEBERTA_SELF_ATTENTION_CLASSES = {
    "eager": DisentangledSelfAttention,
    "b200": FlashDisentangledSelfAttention,
    "flash_attention_2": FlashDisentangledSelfAttention,  # the reference's name for its flash path
}


def _backend(config) -> str:
    name = getattr(config, "attn_backend", "b200")
    if name not in DEBERTA_SELF_ATTENTION_CLASSES:
        raise ValueError(f"config.attn_backend must be one of {sorted(DEBERTA_SELF_ATTENTION_CLASSES)}, got {name!r}")
    return name


def _dense_add_layernorm(block, hidden_states, input_tensor):
    """dense -> dropout -> LayerNorm(hidden + input) of transformers' DebertaV2SelfOutput / DebertaV2Output, with the add
    and the normalisation in one kernel when the case allows it (inference, CUDA, bf16)."""
    hidden_states = block.dense(hidden_states)
    ln = block.LayerNorm
    if (not block.training and ln.elementwise_affine
            and ops.can_fuse_add_layernorm(hidden_states, ln.weight, ln.bias) and input_tensor.dtype == hidden_states.dtype
            and not torch.is_grad_enabled()):
        return ops.add_layernorm(hidden_states, input_tensor, ln.weight, ln.bias, ln.eps)
    return ln(block.dropout(hidden_states) + input_tensor)


class FlashDebertaV2SelfOutput(DebertaV2SelfOutput):
    """Same parameters as transformers' block (the reference keeps it, src/flashdeberta/model.py:259-262)."""

    def forward(self, hidden_states, input_tensor):
        return _dense_add_layernorm(self, hidden_states, input_tensor)


class FlashDebertaV2Output(DebertaV2Output):
    """Same parameters as transformers' block (src/flashdeberta/model.py:265-272)."""

    def forward(self, hidden_states, input_tensor):
        return _dense_add_layernorm(self, hidden_states, input_tensor)


class FlashDebertaV2Embeddings(DebertaV2Embeddings):
    """Same parameters as transformers' module (the reference keeps it inside FlashDebertaV2Model,
    src/flashdeberta/model.py:394-428).  When the input is word embeddings alone (no position term, no token types, no
    projection: the DeBERTa-v3 configuration) and the case allows it (inference, CUDA, bf16), gather, LayerNorm and the
    multiplication by the mask are one kernel."""

    def forward(self, input_ids=None, token_type_ids=None, position_ids=None, mask=None, inputs_embeds=None):
        ln, table = self.LayerNorm, self.word_embeddings.weight
        if (input_ids is not None and inputs_embeds is None and self.position_embeddings is None
                and not self.position_biased_input and self.token_type_embeddings is None and self.embed_proj is None
                and not self.training and not torch.is_grad_enabled() and table.is_cuda and input_ids.is_cuda
                and ops.can_fuse_add_layernorm(table, ln.weight, ln.bias)
                and (mask is None or mask.numel() == input_ids.numel())):
            return ops.embed_layernorm(input_ids, table, ln.weight, ln.bias, ln.eps, row_scale=mask)
        return super().forward(input_ids=input_ids, token_type_ids=token_type_ids, position_ids=position_ids, mask=mask,
                               inputs_embeds=inputs_embeds)


class FlashDebertaV2Intermediate(DebertaV2Intermediate):
    """Same parameters as transformers' block (the reference keeps it inside FlashDebertaV2Layer,
    src/flashdeberta/model.py:265-272); dense and erf GELU run as one kernel when the case allows it (inference, CUDA,
    bf16, hidden_act "gelu")."""

    def __init__(self, config):
        super().__init__(config)
        self._erf_gelu = config.hidden_act == "gelu"

    def forward(self, hidden_states):
        d = self.dense
        if (self._erf_gelu and not self.training and not torch.is_grad_enabled()
                and ops.can_fuse_linear_gelu(hidden_states, d.weight, d.bias)):
            return ops.linear_gelu(hidden_states, d.weight, d.bias)
        return super().forward(hidden_states)


class FlashDebertaV2Attention(DebertaV2Attention):
    def __init__(self, config):
        super().__init__(config)
        self.self = DEBERTA_SELF_ATTENTION_CLASSES[_backend(config)](config)
        if _backend(config) != "eager":
            self.output = FlashDebertaV2SelfOutput(config)


class FlashDebertaV2Layer(DebertaV2Layer):
    def __init__(self, config):
        super().__init__(config)
        self.attention = FlashDebertaV2Attention(config)
        if _backend(config) != "eager":
            self.intermediate = FlashDebertaV2Intermediate(config)
            self.output = FlashDebertaV2Output(config)


class FlashDebertaV2Encoder(DebertaV2Encoder):
    def __init__(self, config):
        super().__init__(config)
        self.layer = nn.ModuleList([FlashDebertaV2Layer(config) for _ in range(config.num_hidden_layers)])
        self._fused = _backend(config) != "eager"
        self._rel_cache = None
        self._mask_cache = None
        self.config_pack = config

    def get_rel_embedding(self):
        """LayerNorm(rel_embeddings) does not depend on the input: in eval mode it is computed once and reused, which
        also lets every layer keep its projected position tables."""
        if self.training or torch.is_grad_enabled() or not self.relative_attention:
            return super().get_rel_embedding()
        w = self.rel_embeddings.weight
        key = [ops.tensor_stamp(w, held=True), w.dtype, w.device]
        if "layer_norm" in self.norm_rel_ebd:
            key += [ops.tensor_stamp(self.LayerNorm.weight, held=True), ops.tensor_stamp(self.LayerNorm.bias, held=True)]
        if self._rel_cache is None or self._rel_cache[0] != key:
            self._rel_cache = (key, super().get_rel_embedding())
        return self._rel_cache[1]

    def forward(self, hidden_states, attention_mask, output_hidden_states=True, output_attentions=False,
                query_states=None, relative_pos=None, return_dict=True, host_mask=None):
        """``host_mask``: the same mask as a host tensor, when the caller still has it there (see the model's forward)."""
        if not self._fused:
            return super().forward(hidden_states, attention_mask, output_hidden_states, output_attentions,
                                   query_states, relative_pos, return_dict)
        # What the mask says (lengths, padding or not, the packing indices) is worked out once per mask tensor: the same
        # tensor, unmodified, coming back (a serving loop with a resident mask) costs no kernels and no host read.
        stamp = ops.tensor_stamp(attention_mask)  # None for a mask without a version counter: analysed on every call
        key = (stamp, tuple(attention_mask.shape), attention_mask.dtype)
        cached = self._mask_cache
        if host_mask is not None:
            dev = hidden_states.device if torch.is_tensor(hidden_states) else attention_mask.device
            input_mask = attention_mask if attention_mask.dim() <= 2 else attention_mask.sum(-2) > 0
            packed_all, looked = None, False
            if getattr(self.config_pack, "pack_sequences", True) and self.conv is None and input_mask.dim() == 2:
                host2d = host_mask if host_mask.dim() <= 2 else host_mask.sum(-2) > 0
                packed_all, looked = PackedSequences.from_mask(host2d, device=dev), True
            # a batch that stays padded is addressed by lengths alone: its mask must be right-padded (checked here)
            seq_lens = lengths_from_mask(host_mask, check=packed_all is None).to(dev, non_blocking=True)
        elif stamp is not None and cached is not None and cached[0] == key and cached[1] is attention_mask:
            input_mask, seq_lens, packed_all, looked = cached[2]
        else:
            if attention_mask.dim() <= 2:
                input_mask = attention_mask
            else:
                input_mask = attention_mask.sum(-2) > 0
            # Ragged batch: run the whole stack on packed tokens.  (The convolution of the v2-xlarge models needs the
            # padded layout.)
            packed_all, looked = None, False
            if getattr(self.config_pack, "pack_sequences", True) and self.conv is None and input_mask.dim() == 2:
                packed_all, looked = PackedSequences.from_mask(input_mask), True
            # (B,) int32; the only form of the mask the layers see.  A batch that stays padded is addressed by lengths
            # alone: its mask must be right-padded (checked here; the packed path takes any layout)
            seq_lens = lengths_from_mask(attention_mask, check=packed_all is None)
            self._mask_cache = (key, attention_mask, (input_mask, seq_lens, packed_all, looked))
        # query_states / a list of hidden states are only used by z_steps: those stay padded
        packed = packed_all if (query_states is None and torch.is_tensor(hidden_states)) else None
        if packed is None and packed_all is not None:
            seq_lens = lengths_from_mask(attention_mask)  # stays padded after all: the mask must be right-padded
        if looked and packed_all is None:
            seq_lens = None  # no padding anywhere (from_mask has looked): the layers' tile order can be kept
        if packed is not None:
            return self._forward_packed(hidden_states, packed, output_hidden_states, return_dict)

        all_hidden_states = (hidden_states,) if output_hidden_states else None
        next_kv = hidden_states
        rel_embeddings = self.get_rel_embedding()
        output_states = hidden_states
        for i, layer_module in enumerate(self.layer):
            output_states, _ = layer_module(next_kv, seq_lens, query_states=query_states, relative_pos=None,
                                            rel_embeddings=rel_embeddings, output_attentions=output_attentions)
            if i == 0 and self.conv is not None:
                output_states = self.conv(hidden_states, output_states, input_mask)
            if output_hidden_states:
                all_hidden_states = all_hidden_states + (output_states,)
            if query_states is not None:
                query_states = output_states
                if isinstance(hidden_states, (list, tuple)):
                    next_kv = hidden_states[i + 1] if i + 1 < len(self.layer) else None
            else:
                next_kv = output_states
        if not return_dict:
            return tuple(v for v in [output_states, all_hidden_states, None] if v is not None)
        return BaseModelOutput(last_hidden_state=output_states, hidden_states=all_hidden_states, attentions=None)

    def _forward_packed(self, hidden_states, packed: PackedSequences, output_hidden_states, return_dict):
        """Every layer on the (1, T, hidden) row of valid tokens.  ``packed.indices`` None: the input already is that row
        (the caller handed the model packed ids and cu_seqlens) and so is the output."""
        already = packed.indices is None
        unpack = (lambda t: t) if already else packed.unpack
        all_hidden_states = (hidden_states,) if output_hidden_states else None
        x = hidden_states if already else packed.pack(hidden_states)  # (1, T, hidden)
        rel_embeddings = self.get_rel_embedding()
        for layer_module in self.layer:
            x, _ = layer_module(x, packed, query_states=None, relative_pos=None, rel_embeddings=rel_embeddings,
                                output_attentions=False)
            if output_hidden_states:
                all_hidden_states = all_hidden_states + (unpack(x),)
        output_states = all_hidden_states[-1] if output_hidden_states else unpack(x)
        if not return_dict:
            return tuple(v for v in [output_states, all_hidden_states, None] if v is not None)
        return BaseModelOutput(last_hidden_state=output_states, hidden_states=all_hidden_states, attentions=None)


class FlashDebertaV2PreTrainedModel(DebertaV2PreTrainedModel):
    """Same role as src/flashdeberta/model.py:312-392 (weight init and loading are transformers')."""
    config_class = DebertaV2Config


class FlashDebertaV2Model(DebertaV2Model):
    """src/flashdeberta/model.py:394-496."""

    def __init__(self, config):
        super().__init__(config)
        self.encoder = FlashDebertaV2Encoder(config)
        if self.encoder._fused:
            self.embeddings = FlashDebertaV2Embeddings(config)
        self.post_init()

    def forward(self, input_ids: Optional[torch.Tensor] = None, attention_mask: Optional[torch.Tensor] = None,
                token_type_ids: Optional[torch.Tensor] = None, position_ids: Optional[torch.Tensor] = None,
                inputs_embeds: Optional[torch.Tensor] = None, output_attentions: Optional[bool] = None,
                output_hidden_states: Optional[bool] = None, return_dict: Optional[bool] = None,
                cu_seqlens: Optional[torch.Tensor] = None, max_seqlen: Optional[int] = None, **kwargs):
        """Same arguments and outputs as src/flashdeberta/model.py:418-496; the encoder is only asked for every layer's
        hidden states when the caller wants them (the reference always collects them, model.py:463-467).

        Packed input (no counterpart in the reference's model, whose varlen path starts from a padded batch in every
        layer, model.py:206-249): ``input_ids`` (1, T) or (T,) holding the tokens of all sequences back to back,
        ``cu_seqlens`` (B+1,) int32 with sequence b at [cu_seqlens[b], cu_seqlens[b+1]) and ``max_seqlen`` >= every length.
        Nothing of size (B, L_max) is ever built; ``last_hidden_state`` comes back as (1, T, hidden).

        ``z_steps`` > 1 (set on the instance; transformers' constructor leaves it 0, src/flashdeberta/model.py:404) runs
        the last layer again z_steps - 1 times with the previous output as the queries over the keys and values of the
        layer before, which is what model.py:469-485 means to do (as written it appends to a tuple and raises)."""
        if not self.encoder._fused:
            return super().forward(input_ids=input_ids, attention_mask=attention_mask, token_type_ids=token_type_ids,
                                   position_ids=position_ids, inputs_embeds=inputs_embeds,
                                   output_attentions=output_attentions, output_hidden_states=output_hidden_states,
                                   return_dict=return_dict, **kwargs)
        if output_attentions if output_attentions is not None else self.config.output_attentions:
            raise ValueError("the fused attention never materialises attention probabilities")
        output_hidden_states = (output_hidden_states if output_hidden_states is not None
                                else self.config.output_hidden_states)
        return_dict = return_dict if return_dict is not None else self.config.return_dict
        if input_ids is not None and inputs_embeds is not None:
            raise ValueError("You cannot specify both input_ids and inputs_embeds at the same time")
        if input_ids is not None:
            input_shape, device = input_ids.size(), input_ids.device
        elif inputs_embeds is not None:
            input_shape, device = inputs_embeds.size()[:-1], inputs_embeds.device
        else:
            raise ValueError("You have to specify either input_ids or inputs_embeds")
        if cu_seqlens is not None:
            return self._forward_packed_ids(input_ids, inputs_embeds, cu_seqlens, max_seqlen, output_hidden_states,
                                            return_dict)
        host_mask = None
        if attention_mask is None:
            attention_mask = torch.ones(input_shape, device=device)
        elif attention_mask.device.type == "cpu" and device.type == "cuda":
            # A mask that is still on the host is analysed there (lengths, padded or not: a few microseconds of host work
            # and no wait for the device); the device only gets the copy the embeddings multiply by.
            host_mask = attention_mask
            attention_mask = attention_mask.to(device, non_blocking=True)
        if token_type_ids is None:
            token_type_ids = torch.zeros(input_shape, dtype=torch.long, device=device)
        embedding_output = self.embeddings(input_ids=input_ids, token_type_ids=token_type_ids,
                                           position_ids=position_ids, mask=attention_mask, inputs_embeds=inputs_embeds)
        z_extra = self.z_steps > 1
        enc = self.encoder(embedding_output, attention_mask, output_hidden_states=bool(output_hidden_states) or z_extra,
                           output_attentions=False, return_dict=True, host_mask=host_mask)
        last, hidden = enc.last_hidden_state, enc.hidden_states
        if z_extra:
            kv, query = hidden[-2], hidden[-1]
            rel_embeddings = self.encoder.get_rel_embedding()
            seq_lens = lengths_from_mask(host_mask if host_mask is not None else attention_mask)
            if seq_lens is not None:
                seq_lens = seq_lens.to(device, non_blocking=True)
            for _ in range(self.z_steps - 1):
                query, _ = self.encoder.layer[-1](kv, seq_lens, query_states=query, relative_pos=None,
                                                  rel_embeddings=rel_embeddings, output_attentions=False)
                hidden = hidden + (query,)
            last = query
        if not return_dict:
            return (last,) + ((hidden,) if output_hidden_states else ())
        return BaseModelOutput(last_hidden_state=last, hidden_states=hidden if output_hidden_states else None,
                               attentions=None)

    def _forward_packed_ids(self, input_ids, inputs_embeds, cu_seqlens, max_seqlen, output_hidden_states, return_dict):
        if self.z_steps > 1:
            raise ValueError("z_steps > 1 needs the padded form of the batch")
        if self.encoder.conv is not None:
            raise ValueError("the convolution layer of this configuration needs the padded form of the batch")
        if max_seqlen is None:
            raise ValueError("packed input needs max_seqlen (an upper bound on every sequence length) beside cu_seqlens")
        x = input_ids if input_ids is not None else inputs_embeds
        if input_ids is not None and input_ids.dim() == 1:
            input_ids = input_ids.unsqueeze(0)
        if inputs_embeds is not None and inputs_embeds.dim() == 2:
            inputs_embeds = inputs_embeds.unsqueeze(0)
        rows = (input_ids if input_ids is not None else inputs_embeds).shape[:2]
        if rows[0] != 1:
            raise ValueError("packed input is one row of tokens: input_ids (1, T) or (T,)")
        device = x.device
        cu = cu_seqlens.to(device=device, dtype=torch.int32)
        embedding_output = self.embeddings(input_ids=input_ids, token_type_ids=None, position_ids=None, mask=None,
                                           inputs_embeds=inputs_embeds)
        packed = PackedSequences(cu, int(max_seqlen), None, cu.numel() - 1, rows[1])
        return self.encoder._forward_packed(embedding_output, packed, bool(output_hidden_states), return_dict)


def _with_flash_backbone(hf_cls, doc):
    class _Head(hf_cls):
        def __init__(self, config):
            super().__init__(config)
            self.deberta = FlashDebertaV2Model(config)
            self.post_init()

    _Head.__name__ = _Head.__qualname__ = "Flash" + hf_cls.__name__
    _Head.__doc__ = doc
    return _Head


FlashDebertaV2ForMaskedLM = _with_flash_backbone(DebertaV2ForMaskedLM, "src/flashdeberta/model.py:498-606")
FlashDebertaV2ForSequenceClassification = _with_flash_backbone(
    DebertaV2ForSequenceClassification, "src/flashdeberta/model.py:608-698")
FlashDebertaV2ForTokenClassification = _with_flash_backbone(
    DebertaV2ForTokenClassification, "src/flashdeberta/model.py:700-757")
FlashDebertaV2ForQuestionAnswering = _with_flash_backbone(
    DebertaV2ForQuestionAnswering, "src/flashdeberta/model.py:759-843")
FlashDebertaV2ForMultipleChoice = _with_flash_backbone(
    DebertaV2ForMultipleChoice, "src/flashdeberta/model.py:845-920")
