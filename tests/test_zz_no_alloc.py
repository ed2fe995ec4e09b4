"""fdb_attn_fwd_static — the entry point for hosts that cannot allocate device memory when they call the library
(an inference server whose arena already owns the GPU, a plug-in inside a latency-critical loop where cudaMalloc and
cudaFree would stall the device).  Its scratch is a fixed array inside the library, so the thing to prove is that it
computes exactly what fdb_attn_fwd computes with a caller workspace — on two calls in a row, because the array keeps
the first call's contents when the second one starts.

This file sorts last on purpose: a run that stops at the first failure has then already run every other test."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _inputs(seed, B, L, H, lens):
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(B, L, H, 64, generator=g).bfloat16().to(DEV) for _ in range(3))
    pk, pq = (torch.randn(H, 512, 64, generator=g).bfloat16().to(DEV) for _ in range(2))
    return q, k, v, pk, pq, torch.tensor(lens, dtype=torch.int32, device=DEV)


def test_static_scratch_entry_point_matches_workspace_entry_point_twice():
    from flashdeberta_b200 import ops
    kw = dict(position_buckets=256, max_relative_positions=512)
    # two different problems back to back: the second starts from the scratch the first one left behind
    for seed, (B, L, H, lens) in enumerate([(3, 700, 4, [700, 129, 5]), (2, 1300, 2, [1024, 1300])]):
        q, k, v, pk, pq, sl = _inputs(seed, B, L, H, lens)
        want = ops.disentangled_attention(q, k, v, pk, pq, seq_lens=sl, max_seqlen=L, **kw)
        out = torch.full_like(want, float("nan"))
        got = ops.disentangled_attention_static(q, k, v, pk, pq, out=out, seq_lens=sl, max_seqlen=L, **kw)
        torch.cuda.synchronize()
        ops.check_status()
        assert got.data_ptr() == out.data_ptr()
        # same kernels on the same inputs: identical bits (well inside the 2e-2 / 2e-3 bf16 tolerance of the other tests)
        assert torch.equal(got, want)


def test_static_entry_point_packed_position_free_and_long():
    """The forms the first test does not reach: a packed batch (cu_seqlens), a call without position terms, and a
    sequence long enough that fdb_attn_fwd would take two launches.  The static entry point is always one launch, so it
    is bit-identical to fdb_attn_fwd held to one launch, and within bf16 rounding of its default."""
    from flashdeberta_b200 import _lib, ops
    kw = dict(position_buckets=256, max_relative_positions=512)
    g = torch.Generator().manual_seed(11)

    def close(a, b):
        d = (a.float() - b.float()).abs()
        assert d.max().item() <= 2e-2 and d.mean().item() <= 2e-3

    # packed: three sequences back to back
    lens = [333, 1, 1200]
    cu = torch.tensor([0, 333, 334, 1534], dtype=torch.int32, device=DEV)
    H = 3
    q, k, v = (torch.randn(sum(lens), H, 64, generator=g).bfloat16().to(DEV) for _ in range(3))
    pk, pq = (torch.randn(H, 512, 64, generator=g).bfloat16().to(DEV) for _ in range(2))
    want = ops.disentangled_attention(q, k, v, pk, pq, cu_seqlens=cu, max_seqlen=max(lens), **kw)
    got = ops.disentangled_attention_static(q, k, v, pk, pq, out=torch.full_like(want, float("nan")), cu_seqlens=cu,
                                            max_seqlen=max(lens), **kw)
    assert torch.equal(got, want)

    # no position terms: the library's default sends these through the far kernel, the static entry point does not
    sl = torch.tensor([900, 77], dtype=torch.int32, device=DEV)
    q, k, v = (torch.randn(2, 900, H, 64, generator=g).bfloat16().to(DEV) for _ in range(3))
    one = ops.disentangled_attention(q, k, v, None, None, seq_lens=sl, max_seqlen=900, tune=_lib.TUNE_ONE_LAUNCH)
    dflt = ops.disentangled_attention(q, k, v, None, None, seq_lens=sl, max_seqlen=900)
    got = ops.disentangled_attention_static(q, k, v, None, None, out=torch.full_like(one, float("nan")), seq_lens=sl,
                                            max_seqlen=900)
    assert torch.equal(got, one)
    close(got, dflt)

    # a sequence of 4096 keys beside a short one: two launches by default, one here
    sl = torch.tensor([4096, 200], dtype=torch.int32, device=DEV)
    q, k, v = (torch.randn(2, 4096, 2, 64, generator=g).bfloat16().to(DEV) for _ in range(3))
    pk, pq = (torch.randn(2, 512, 64, generator=g).bfloat16().to(DEV) for _ in range(2))
    one = ops.disentangled_attention(q, k, v, pk, pq, seq_lens=sl, max_seqlen=4096, tune=_lib.TUNE_ONE_LAUNCH, **kw)
    dflt = ops.disentangled_attention(q, k, v, pk, pq, seq_lens=sl, max_seqlen=4096, **kw)
    got = ops.disentangled_attention_static(q, k, v, pk, pq, out=torch.full_like(one, float("nan")), seq_lens=sl,
                                            max_seqlen=4096, **kw)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(got, one)
    close(got, dflt)
    assert got[1, 200:].abs().max().item() == 0  # padding rows are zeros


def test_static_scratch_refuses_what_does_not_fit():
    from flashdeberta_b200 import _lib, ops
    H = 64  # 64 heads x 2 expanded tables x 1527 rows x 128 B > 8 MiB
    q = torch.zeros(1, 128, H, 64, dtype=torch.bfloat16, device=DEV)
    pk = torch.zeros(H, 512, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(_lib.FdbError) as e:
        ops.disentangled_attention_static(q, q, q, pk, pk, out=torch.empty_like(q), max_seqlen=128,
                                          position_buckets=256, max_relative_positions=512)
    assert e.value.code == -6 and "FDB_STATIC_SCRATCH_BYTES" in str(e.value)
