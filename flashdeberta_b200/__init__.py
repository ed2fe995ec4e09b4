"""flashdeberta_b200 — DeBERTa-v2/v3 disentangled self-attention forward on NVIDIA B200 (sm_100a).

Public names follow the reference package (src/flashdeberta/__init__.py:1-9).
"""
from .attention import FlashDisentangledSelfAttention  # noqa: F401
from .model import (  # noqa: F401
    FlashDebertaV2ForMaskedLM,
    FlashDebertaV2ForMultipleChoice,
    FlashDebertaV2ForQuestionAnswering,
    FlashDebertaV2ForSequenceClassification,
    FlashDebertaV2ForTokenClassification,
    FlashDebertaV2Model,
    FlashDebertaV2PreTrainedModel,
)

__version__ = "0.1.0"
