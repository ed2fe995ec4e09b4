"""Generate the golden fixtures in this directory from the real HuggingFace eager module.

Run once, in a container that has ``transformers`` (5.5.0 when these were made):

    python tests/golden/make_golden.py

Writes
  bucket_index.npz   relative-position table index for d in [-40000, 40000], several configs,
                     from make_log_bucket_position / build_relative_position + the clamp at
                     modeling_deberta_v2.py:318
  attn_<name>.npz    inputs, parameters and fp32 eager outputs of DisentangledSelfAttention
                     (modeling_deberta_v2.py:137-345) for small seeded cases.  Inputs and
                     parameters sit on the bfloat16 grid and are stored as the upper 16 bits of
                     their float32 pattern (int16); outputs are float32.

The tests never regenerate these; they only load them.
"""
import os

import numpy as np
import torch
import transformers
from transformers.models.deberta_v2.modeling_deberta_v2 import (
    DisentangledSelfAttention,
    build_relative_position,
    make_log_bucket_position,
)

HERE = os.path.dirname(os.path.abspath(__file__))

BUCKET_CONFIGS = [(256, 512), (64, 128), (32, 64), (128, 1024), (0, 512), (-1, 64)]
D_LO, D_HI = -40000, 40000


class Cfg:
    def __init__(self, hidden_size, heads, buckets, max_rel, pos_att_type, share, relative_attention=True):
        self.hidden_size = hidden_size
        self.num_attention_heads = heads
        self.attention_probs_dropout_prob = 0.1
        self.hidden_dropout_prob = 0.1
        self.pos_att_type = pos_att_type
        self.relative_attention = relative_attention
        self.position_buckets = buckets
        self.max_relative_positions = max_rel
        self.max_position_embeddings = 512
        self.share_att_key = share


def golden_bucket():
    out = {}
    d = torch.arange(D_LO, D_HI + 1, dtype=torch.long)
    for buckets, max_rel in BUCKET_CONFIGS:
        span = buckets if buckets > 0 else max_rel
        if buckets > 0 and max_rel > 0:
            b = make_log_bucket_position(d, buckets, max_rel).to(torch.long)
        else:
            b = d
        idx = torch.clamp(b + span, 0, 2 * span - 1)
        out[f"idx_{buckets}_{max_rel}"] = idx.numpy().astype(np.int16)
        # the matrix form the module uses, for a short sequence
        q = torch.zeros(1, 70, 1)
        rp = build_relative_position(q, q, bucket_size=buckets, max_position=max_rel)
        out[f"relpos70_{buckets}_{max_rel}"] = rp[0].numpy().astype(np.int16)
    out["d_lo"] = np.int64(D_LO)
    out["d_hi"] = np.int64(D_HI)
    np.savez_compressed(os.path.join(HERE, "bucket_index.npz"), **out)


ATTN_CASES = {
    # name: (B, L, hidden, heads, buckets, max_rel, pos_att_type, share, lens, seed)
    "v3_small_full": (2, 96, 128, 2, 256, 512, ["c2p", "p2c"], True, [96, 96], 10),
    "v3_small_padded": (3, 80, 128, 2, 256, 512, ["c2p", "p2c"], True, [80, 33, 1], 11),
    "v3_long_sat": (1, 720, 128, 2, 256, 512, ["c2p", "p2c"], True, [720], 12),
    "tiny_buckets": (2, 150, 128, 2, 32, 64, ["c2p", "p2c"], False, [150, 97], 13),
    "c2p_only": (1, 130, 128, 2, 32, 64, ["c2p"], False, [130], 14),
    "p2c_only": (1, 130, 128, 2, 32, 64, ["p2c"], False, [130], 15),
    "no_relative": (2, 70, 128, 2, 32, 64, [], False, [70, 50], 16),
    "no_buckets": (1, 200, 128, 2, -1, 64, ["c2p", "p2c"], True, [200], 17),
    "head_dim_128": (1, 64, 128, 1, 32, 64, ["c2p", "p2c"], False, [64], 18),
}


def bf16_grid(x: torch.Tensor) -> torch.Tensor:
    """Round to the nearest bfloat16-representable value (kept as float32)."""
    return x.to(torch.bfloat16).to(torch.float32)


def pack_bf16(x: torch.Tensor) -> np.ndarray:
    """Upper 16 bits of float32 values that already sit on the bfloat16 grid."""
    return (x.contiguous().view(torch.int32) >> 16).to(torch.int16).numpy()


def golden_attn():
    for name, (B, L, hid, heads, buckets, max_rel, pat, share, lens, seed) in ATTN_CASES.items():
        g = torch.Generator(device="cpu").manual_seed(seed)
        rel_attn = name != "no_relative"
        cfg = Cfg(hid, heads, buckets, max_rel, pat, share, relative_attention=rel_attn)
        mod = DisentangledSelfAttention(cfg).eval()
        with torch.no_grad():
            for p in mod.parameters():
                p.copy_(bf16_grid(torch.randn(p.shape, generator=g) * 0.05))
        span = buckets if buckets > 0 else max_rel
        hidden = bf16_grid(torch.randn(B, L, hid, generator=g))
        rel_emb = bf16_grid(torch.randn(2 * span, hid, generator=g) * 0.5)
        mask2 = torch.zeros(B, L)
        for b, n in enumerate(lens):
            mask2[b, :n] = 1
        ext = mask2.unsqueeze(1).unsqueeze(2)
        ext = ext * ext.squeeze(-2).unsqueeze(-1)  # (B,1,L,L) as tests/attention.py:34-35
        with torch.no_grad():
            out = mod(hidden, ext, rel_embeddings=rel_emb if rel_attn else None)[0]
        valid = mask2.bool().unsqueeze(-1)
        out = torch.where(valid, out, torch.zeros_like(out))  # padded rows are unspecified in eager
        blob = {
            "hidden": pack_bf16(hidden), "rel_embeddings": pack_bf16(rel_emb), "lens": np.array(lens, np.int64),
            "out": out.numpy(),
            "meta": np.array([B, L, hid, heads, buckets, max_rel, int(share), int(rel_attn)], np.int64),
            "pos_att_type": np.array("|".join(pat)),
        }
        for k, v in mod.state_dict().items():
            blob["param:" + k] = pack_bf16(v)
        np.savez_compressed(os.path.join(HERE, f"attn_{name}.npz"), **blob)
        print(name, "mean|out|", out.abs().mean().item())


if __name__ == "__main__":
    torch.set_num_threads(8)
    print("transformers", transformers.__version__, "torch", torch.__version__)
    golden_bucket()
    golden_attn()
    with open(os.path.join(HERE, "VERSIONS.txt"), "w") as f:
        f.write(f"transformers {transformers.__version__}\ntorch {torch.__version__}\n")
