"""Loader for the fixtures under tests/golden/ (made by tests/golden/make_golden.py)."""
import glob
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def unpack_bf16(a: np.ndarray) -> torch.Tensor:
    """int16 = upper half of a float32 bit pattern -> float32 tensor (exactly bf16-representable)."""
    t = torch.from_numpy(a.astype(np.int32) << 16)
    return t.view(torch.float32)


def attn_case_names():
    return sorted(os.path.basename(p)[5:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, "attn_*.npz")))


def load_attn_case(name: str) -> dict:
    z = np.load(os.path.join(GOLDEN_DIR, f"attn_{name}.npz"))
    B, L, hid, heads, buckets, max_rel, share, rel_attn = (int(x) for x in z["meta"])
    pat = str(z["pos_att_type"])
    case = dict(
        name=name, B=B, L=L, hidden_size=hid, heads=heads, position_buckets=buckets,
        max_relative_positions=max_rel, share_att_key=bool(share), relative_attention=bool(rel_attn),
        pos_att_type=[p for p in pat.split("|") if p],
        lens=[int(x) for x in z["lens"]],
        hidden=unpack_bf16(z["hidden"]), rel_embeddings=unpack_bf16(z["rel_embeddings"]),
        out=torch.from_numpy(z["out"]),
        state={k[6:]: unpack_bf16(z[k]) for k in z.files if k.startswith("param:")},
    )
    return case


def load_bucket_golden() -> dict:
    z = np.load(os.path.join(GOLDEN_DIR, "bucket_index.npz"))
    return {k: z[k] for k in z.files}


class AttnConfig:
    """Attribute bag in the shape the reference's tests hand to the attention module
    (tests/attention.py:6-18 of the reference)."""

    def __init__(self, case: dict):
        self.hidden_size = case["hidden_size"]
        self.num_attention_heads = case["heads"]
        self.attention_probs_dropout_prob = 0.1
        self.hidden_dropout_prob = 0.1
        self.pos_att_type = case["pos_att_type"]
        self.relative_attention = case["relative_attention"]
        self.position_buckets = case["position_buckets"]
        self.max_relative_positions = case["max_relative_positions"]
        self.max_position_embeddings = 512
        self.share_att_key = case["share_att_key"]
