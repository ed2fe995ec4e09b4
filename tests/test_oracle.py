"""The CPU oracle against the fixtures made from the real HuggingFace eager module."""
import numpy as np
import pytest
import torch

from oracle import disentangled_attention as oracle
from tests._golden import attn_case_names, load_attn_case, load_bucket_golden


def _configs(g):
    for k in g:
        if k.startswith("idx_"):
            _, b, m = k.split("_")
            yield int(b), int(m)


def test_relative_index_bit_exact_vs_hf():
    g = load_bucket_golden()
    d = np.arange(int(g["d_lo"]), int(g["d_hi"]) + 1, dtype=np.int64)
    n = 0
    for buckets, max_rel in _configs(g):
        want = g[f"idx_{buckets}_{max_rel}"].astype(np.int64)
        got = oracle.relative_index(d, buckets, max_rel)
        assert np.array_equal(got, want), (buckets, max_rel, int((got != want).sum()))
        n += 1
    assert n >= 5


def test_relative_position_matrix_vs_hf():
    g = load_bucket_golden()
    m = np.arange(70)[:, None] - np.arange(70)[None, :]
    for buckets, max_rel in _configs(g):
        want = g[f"relpos70_{buckets}_{max_rel}"].astype(np.int64)
        if buckets > 0 and max_rel > 0:
            got = oracle.log_bucket_position(m, buckets, max_rel)
        else:
            got = m
        assert np.array_equal(got, want)


def test_known_bucket_values_v3():
    # spot values for position_buckets=256, max_relative_positions=512
    b = lambda d: int(oracle.log_bucket_position(np.array([d]), 256, 512)[0])
    assert [b(127), b(128), b(129), b(255), b(256), b(510), b(511), b(512)] == [127, 128, 129, 192, 192, 255, 255, 256]
    assert b(-129) == -129 and b(-512) == -256
    idx = oracle.relative_index(np.arange(-2000, 2000), 256, 512)
    assert idx.min() == 0 and idx.max() == 511
    assert np.all(np.diff(idx) >= 0)  # monotone in d


@pytest.mark.parametrize("name", attn_case_names())
def test_module_forward_vs_hf_eager(name):
    c = load_attn_case(name)
    got = oracle.module_forward(
        c["hidden"], c["lens"], c["rel_embeddings"], c["state"], c["heads"],
        c["position_buckets"], c["max_relative_positions"], c["pos_att_type"], c["share_att_key"],
        relative_attention=c["relative_attention"],
    )
    diff = (got - c["out"]).abs()
    # fp32 against fp32: only summation order differs
    assert diff.max().item() < 2e-5, diff.max().item()
    assert diff.mean().item() < 1e-6, diff.mean().item()
    for b, n in enumerate(c["lens"]):
        assert torch.count_nonzero(got[b, n:]) == 0


def test_attention_core_blocking_is_invisible():
    g = torch.Generator().manual_seed(0)
    rows, H, D = 300, 2, 64
    q, k, v = (torch.randn(rows, H, D, generator=g) for _ in range(3))
    pk, pq = (torch.randn(H, 64, D, generator=g) for _ in range(2))
    kw = dict(seq_start=[0, 200], seq_len=[200, 100], sm_scale=0.07, position_buckets=32, max_relative_positions=64)
    a = oracle.attention_core(q, k, v, pk, pq, row_block=512, **kw)
    b, lse = oracle.attention_core(q, k, v, pk, pq, row_block=37, return_lse=True, **kw)
    assert (a - b).abs().max().item() < 1e-5
    assert torch.isfinite(lse).all()
