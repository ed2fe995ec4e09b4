"""flashdeberta_b200 — DeBERTa-v2/v3 disentangled self-attention forward on NVIDIA B200 (sm_100a)."""
from .attention import FlashDisentangledSelfAttention  # noqa: F401

__version__ = "0.1.0"
