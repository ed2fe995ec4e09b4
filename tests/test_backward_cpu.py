"""Host logic of the attention backward (flashdeberta_b200/backward.py) on CPU: the block decomposition, the layouts and
the table-row intervals, with the two CUDA stages replaced by a few lines of torch that do what their contract says.
The reference gradients come from autograd through the fp32 oracle.  (The CUDA stages themselves are checked on the GPU
in tests/test_backward_gpu.py.)"""
import pytest
import torch

from flashdeberta_b200 import backward, bucket
from oracle import disentangled_attention as oracle


def _index_matrix(blk):
    m = torch.arange(blk["row0"], blk["row0"] + blk["rows"]).view(-1, 1)
    n = torch.arange(blk["seqlen"]).view(1, -1)
    i = (m - n - blk["lut_d_min"]).clamp(0, blk["lut_len"] - 1)
    return blk["lut"].long()[i]  # (rows, seqlen)


def _valid(blk):
    G, H, L = blk["groups"], blk["heads"], blk["seqlen"]
    lens = torch.full((G // H,), L) if blk["seq_lens"] is None else blk["seq_lens"].long()
    lens = lens.repeat_interleave(H).view(G, 1, 1)
    m = torch.arange(blk["row0"], blk["row0"] + blk["rows"]).view(1, -1, 1)
    n = torch.arange(L).view(1, 1, -1)
    return (m < lens) & (n < lens)


def fake_probs(blk):
    s = blk["scores"].clone()
    if blk["table_rows"]:
        idx = _index_matrix(blk).unsqueeze(0).expand(s.shape[0], -1, -1)
        if blk["c2p"] is not None:
            s = s + torch.gather(blk["c2p"], 2, idx)
        if blk["p2c"] is not None:
            s = s + torch.gather(blk["p2c"], 2, idx.transpose(1, 2)).transpose(1, 2)
    p = torch.exp(blk["sm_scale"] * s - blk["lse"].unsqueeze(-1))
    p = torch.where(_valid(blk), p, torch.zeros_like(p))
    g = blk["sm_scale"] * p * (blk["dprobs"] - blk["delta"].unsqueeze(-1))
    return p.bfloat16(), g.bfloat16()


def fake_sums(blk, dscores, want_c2p, p2c_sums):
    idx = _index_matrix(blk).unsqueeze(0).expand(dscores.shape[0], -1, -1)
    g = dscores.float()
    gc = None
    if want_c2p:
        gc = torch.zeros(g.shape[0], g.shape[1], blk["table_rows"]).scatter_add_(2, idx, g)
    if p2c_sums is not None:
        p2c_sums.scatter_add_(2, idx.transpose(1, 2).contiguous(), g.transpose(1, 2).contiguous())
    return gc


@pytest.fixture
def fake_stages(monkeypatch):
    monkeypatch.setattr(backward, "_stage_probs", fake_probs)
    monkeypatch.setattr(backward, "_stage_sums", fake_sums)


def _reference(q, k, v, pk, pq, starts, lens, sm, buckets, max_rel, dout):
    leaves = [t.float().clone().requires_grad_(True) if t is not None else None for t in (q, k, v, pk, pq)]
    with torch.enable_grad():
        out, lse = oracle.attention_core.__wrapped__(leaves[0], leaves[1], leaves[2], leaves[3], leaves[4], starts, lens, sm,
                                                     buckets, max_rel, return_lse=True)
        grads = torch.autograd.grad(out, [t for t in leaves if t is not None], dout.float())
    it = iter(grads)
    return out.detach(), lse.detach(), [next(it) if t is not None else None for t in leaves]


def _close(got, want, what):
    scale = want.abs().max().item() + 1e-12
    err = (got.float() - want).abs().max().item() / scale
    assert err < 2e-2, f"{what}: relative error {err:.3e}"


@pytest.mark.parametrize("buckets,max_rel,c2p,p2c", [(32, 64, True, True), (32, 64, True, False), (32, 64, False, True),
                                                     (-1, 40, True, True), (-1, -1, False, False)])
def test_dense_ragged_blocks_match_autograd(fake_stages, buckets, max_rel, c2p, p2c):
    g = torch.Generator().manual_seed(5)
    B, L, H, D = 2, 200, 2, 16
    lens = [200, 77]
    span = bucket.att_span(buckets, max_rel) if (c2p or p2c) else 0
    q, k, v, dout = (torch.randn(B, L, H, D, generator=g).bfloat16() for _ in range(4))
    pk = torch.randn(H, 2 * span, D, generator=g).bfloat16() if c2p else None
    pq = torch.randn(H, 2 * span, D, generator=g).bfloat16() if p2c else None
    sm = oracle.sm_scale_for(D, c2p, p2c)
    out, lse, want = _reference(q.view(-1, H, D), k.view(-1, H, D), v.view(-1, H, D), pk, pq, [0, L], lens, sm, buckets,
                                max_rel, dout.view(-1, H, D))
    got = backward.attention_backward(dout, q, k, v, pk, pq, out.view(B, L, H, D).bfloat16(), lse,
                                      seq_lens=torch.tensor(lens, dtype=torch.int32), max_seqlen=L, sm_scale=sm,
                                      position_buckets=buckets, max_relative_positions=max_rel,
                                      block_bytes=12 * B * H * L * 64)  # blocks of 64 rows: four of them
    names = ("dq", "dk", "dv", "dpos_key", "dpos_query")
    for name, a, b in zip(names, got, want):
        assert (a is None) == (b is None), name
        if a is not None:
            _close(a.reshape(b.shape), b, name)
    assert got[0].view(B, L, H, D)[1, 77:].abs().max().item() == 0  # rows of the padding get no gradient


def test_packed_sequences_match_autograd(fake_stages):
    g = torch.Generator().manual_seed(6)
    H, D, buckets, max_rel = 3, 16, 16, 32
    lens = [90, 1, 150]
    cu = torch.tensor([0, 90, 91, 241], dtype=torch.int32)
    T = 241
    q, k, v, dout = (torch.randn(T, H, D, generator=g).bfloat16() for _ in range(4))
    pk, pq = (torch.randn(H, 32, D, generator=g).bfloat16() for _ in range(2))
    sm = oracle.sm_scale_for(D, True, True)
    out, lse, want = _reference(q, k, v, pk, pq, [0, 90, 91], lens, sm, buckets, max_rel, dout)
    got = backward.attention_backward(dout, q, k, v, pk, pq, out.bfloat16(), lse, cu_seqlens=cu, max_seqlen=150,
                                      sm_scale=sm, position_buckets=buckets, max_relative_positions=max_rel)
    for name, a, b in zip(("dq", "dk", "dv", "dpos_key", "dpos_query"), got, want):
        _close(a, b, name)
