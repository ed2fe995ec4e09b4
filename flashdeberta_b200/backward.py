"""Backward pass of the disentangled attention: gradients of q, k, v and of the two projected position tables.

The reference does this in three Triton kernels (src/flashdeberta/ops/flash_attention.py:581-614 preprocess, :616-797
dK/dV with the position-bias gradients scattered by atomics :770-786, :799-940 dQ; launcher :942-1030).  Here the
contractions that are plain GEMMs go to the library GEMM in blocks of query rows, and what is specific to this
attention runs in this package's own kernels (csrc/attn_bwd.cu):

  * ``fdb_attn_bwd_probs``: rebuilds P = exp(scale * (Q.K^T + c2p + p2c) - LSE) of a block of rows from the three products
    (the two position terms gathered through the bucket table) and forms dS = scale * P * (dP - delta) in the same pass;
  * ``fdb_attn_bwd_bucket_sums``: folds dS back onto the position tables' rows without atomics on global memory — per query
    row the sum over the keys that share a table row (c2p), per key the sum over the queries that share one (p2c).

With  s[m,n] = scale * (q_m.k_n + q_m.pk[i(m-n)] + k_n.pq[i(m-n)]),  p = exp(s - lse_m),  o_m = sum_n p[m,n] v_n:

  delta_m = dO_m . O_m              dP[m,n] = dO_m . v_n            g[m,n] = scale * p[m,n] * (dP[m,n] - delta_m)
  dV_n = sum_m p[m,n] dO_m          GC[m,b] = sum_{n: i(m-n)=b} g[m,n]      GP[n,b] = sum_{m: i(m-n)=b} g[m,n]
  dQ_m = sum_n g[m,n] k_n + sum_b GC[m,b] pk_b           dK_n = sum_m g[m,n] q_m + sum_b GP[n,b] pq_b
  dpk_b = sum_m GC[m,b] q_m                              dpq_b = sum_n GP[n,b] k_n

Memory: four (sequences x heads x block rows x keys) buffers at a time (two fp32, two bf16), the block sized to
``block_bytes`` (2 GiB by default: the per-block costs — the fp32 accumulations of dK and dV, the write-back of the p2c
sums — shrink with the number of blocks).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _lib, bucket

_launches = 0  # kernels of this package launched by the functions below


class BwdBlock(C.Structure):
    """Mirror of ``fdb_bwd_block`` (include/fdb_b200.h)."""

    _fields_ = [
        ("struct_bytes", C.c_uint32), ("groups", C.c_int32), ("heads", C.c_int32), ("seqlen", C.c_int32),
        ("row0", C.c_int32), ("rows", C.c_int32), ("table_rows", C.c_int32), ("lut_d_min", C.c_int32),
        ("lut_len", C.c_int32), ("sm_scale", C.c_float),
        ("seq_lens", C.c_void_p), ("lut", C.c_void_p),
        ("scores", C.c_void_p), ("dprobs", C.c_void_p), ("c2p", C.c_void_p), ("p2c", C.c_void_p),
        ("lse", C.c_void_p), ("delta", C.c_void_p), ("probs", C.c_void_p), ("dscores", C.c_void_p),
        ("c2p_sums", C.c_void_p), ("p2c_sums", C.c_void_p), ("status", C.c_void_p),
    ]


def _bmm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Batched product of two bf16 operands with an fp32 result."""
    try:
        return torch.bmm(a, b, out_dtype=torch.float32)
    except (TypeError, RuntimeError):
        return torch.bmm(a.float(), b.float())


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stage_probs(blk: dict) -> Tuple[torch.Tensor, torch.Tensor]:
    """P and dS (bf16, (groups, rows, seqlen)) of one block: ``fdb_attn_bwd_probs``."""
    global _launches
    s = blk["scores"]
    if not s.is_cuda:
        raise RuntimeError("flashdeberta_b200 runs on CUDA devices only; there is no CPU path")
    probs = torch.empty(s.shape, dtype=torch.bfloat16, device=s.device)
    dscores = torch.empty(s.shape, dtype=torch.bfloat16, device=s.device)
    p = _block_struct(blk)
    p.scores, p.dprobs, p.c2p, p.p2c = _ptr(s), _ptr(blk["dprobs"]), _ptr(blk["c2p"]), _ptr(blk["p2c"])
    p.lse, p.delta, p.probs, p.dscores = _ptr(blk["lse"]), _ptr(blk["delta"]), _ptr(probs), _ptr(dscores)
    with torch.cuda.device(s.device):
        _lib.check(_lib.load().fdb_attn_bwd_probs(C.byref(p), C.c_void_p(torch.cuda.current_stream(s.device).cuda_stream)))
    _launches += 1
    return probs, dscores


def _stage_sums(blk: dict, dscores: torch.Tensor, want_c2p: bool, p2c_sums: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """``fdb_attn_bwd_bucket_sums``: returns GC (fp32, (groups, rows, table_rows)) when asked and adds this block's part
    to ``p2c_sums`` (fp32, (groups, seqlen, table_rows)) when given."""
    global _launches
    if not dscores.is_cuda:
        raise RuntimeError("flashdeberta_b200 runs on CUDA devices only; there is no CPU path")
    c2p_sums = None
    if want_c2p:
        c2p_sums = torch.empty(dscores.shape[0], dscores.shape[1], blk["table_rows"], dtype=torch.float32, device=dscores.device)
    p = _block_struct(blk)
    p.dscores, p.c2p_sums, p.p2c_sums = _ptr(dscores), _ptr(c2p_sums), _ptr(p2c_sums)
    with torch.cuda.device(dscores.device):
        _lib.check(_lib.load().fdb_attn_bwd_bucket_sums(C.byref(p), C.c_void_p(torch.cuda.current_stream(dscores.device).cuda_stream)))
    _launches += int(want_c2p) + int(p2c_sums is not None)
    return c2p_sums


def _block_struct(blk: dict) -> BwdBlock:
    p = BwdBlock()
    p.struct_bytes = C.sizeof(BwdBlock)
    p.groups, p.heads, p.seqlen, p.row0, p.rows = blk["groups"], blk["heads"], blk["seqlen"], blk["row0"], blk["rows"]
    p.table_rows, p.lut_d_min, p.lut_len, p.sm_scale = blk["table_rows"], blk["lut_d_min"], blk["lut_len"], blk["sm_scale"]
    p.seq_lens, p.lut, p.status = _ptr(blk["seq_lens"]), _ptr(blk["lut"]), _ptr(blk["status"])
    return p


def _heads_first(x: torch.Tensor, n_seq: int, seqlen: int) -> torch.Tensor:
    """(n_seq * seqlen, H, D) rows -> (n_seq * H, seqlen, D), contiguous."""
    H, D = x.shape[-2], x.shape[-1]
    return x.reshape(n_seq, seqlen, H, D).permute(0, 2, 1, 3).reshape(n_seq * H, seqlen, D).contiguous()


def _rows_first(x: torch.Tensor, n_seq: int, heads: int) -> torch.Tensor:
    """(n_seq * H, seqlen, D) -> (n_seq * seqlen, H, D)."""
    seqlen, D = x.shape[1], x.shape[2]
    return x.view(n_seq, heads, seqlen, D).permute(0, 2, 1, 3).reshape(n_seq * seqlen, heads, D)


def _backward_block(q, k, v, o, do, lse, pos_key, pos_query, n_seq, seqlen, seq_lens, sm_scale, position_buckets,
                    max_relative_positions, block_bytes, status):
    """One group of ``n_seq`` sequences of ``seqlen`` rows each (right-padded, lengths in ``seq_lens`` or all full).
    q, k, v, o, do: (n_seq * seqlen, H, D) bf16; lse: (n_seq * seqlen, H) fp32.  Returns dq, dk, dv in the same layout
    (fp32) and dpos_key, dpos_query as (H, table_rows, D) fp32 or None."""
    H, D = q.shape[-2], q.shape[-1]
    dev = q.device
    G = n_seq * H
    qh, kh, vh, doh = (_heads_first(t, n_seq, seqlen) for t in (q, k, v, do))
    delta = (do.float() * o.float()).sum(-1)                                   # (rows, H)
    delta = delta.view(n_seq, seqlen, H).permute(0, 2, 1).reshape(G, seqlen).contiguous()
    lse_h = lse.view(n_seq, seqlen, H).permute(0, 2, 1).reshape(G, seqlen).contiguous()
    has_c2p, has_p2c = pos_key is not None, pos_query is not None
    blk = dict(groups=G, heads=H, seqlen=seqlen, table_rows=0, lut=None, lut_d_min=0, lut_len=0,
               sm_scale=float(sm_scale), seq_lens=seq_lens, status=status, c2p=None, p2c=None)
    pkh = pqh = p2c_sums = None
    if has_c2p or has_p2c:
        lut, d_min = bucket.device_lut(position_buckets, max_relative_positions, dev)
        W = 2 * bucket.att_span(position_buckets, max_relative_positions)
        blk.update(table_rows=W, lut=lut, lut_d_min=d_min, lut_len=lut.numel())
        if has_c2p:
            pkh = pos_key.to(torch.bfloat16).unsqueeze(0).expand(n_seq, H, W, D).reshape(G, W, D)
        if has_p2c:
            pqh = pos_query.to(torch.bfloat16).unsqueeze(0).expand(n_seq, H, W, D).reshape(G, W, D)
            blk["p2c"] = _bmm(kh, pqh.transpose(1, 2))                        # (G, seqlen, W): K.pos_query^T
            p2c_sums = torch.zeros(G, seqlen, W, dtype=torch.float32, device=dev)
    dqh = torch.empty(G, seqlen, D, dtype=torch.float32, device=dev)
    dkh = torch.zeros(G, seqlen, D, dtype=torch.float32, device=dev)
    dvh = torch.zeros(G, seqlen, D, dtype=torch.float32, device=dev)
    dpk = torch.zeros(G, blk["table_rows"], D, dtype=torch.float32, device=dev) if has_c2p else None
    rows = max(1, int(block_bytes) // (12 * G * max(seqlen, 1)))
    rows = min(seqlen, max(64, rows // 64 * 64))
    for m0 in range(0, seqlen, rows):
        m1 = min(seqlen, m0 + rows)
        qc, doc = qh[:, m0:m1], doh[:, m0:m1]
        blk.update(row0=m0, rows=m1 - m0, scores=_bmm(qc, kh.transpose(1, 2)), dprobs=_bmm(doc, vh.transpose(1, 2)),
                   lse=lse_h[:, m0:m1].contiguous(), delta=delta[:, m0:m1].contiguous())
        if has_c2p:
            blk["c2p"] = _bmm(qc, pkh.transpose(1, 2))                         # (G, rows, W): Q.pos_key^T
        probs, dscores = _stage_probs(blk)
        blk["scores"] = blk["dprobs"] = None
        dvh += _bmm(probs.transpose(1, 2), doc)
        dkh += _bmm(dscores.transpose(1, 2), qc)
        dqc = _bmm(dscores, kh)
        if has_c2p or has_p2c:
            gc = _stage_sums(blk, dscores, has_c2p, p2c_sums)
            if has_c2p:
                gcb = gc.to(torch.bfloat16)
                dqc += _bmm(gcb, pkh)
                dpk += _bmm(gcb.transpose(1, 2), qc)
        dqh[:, m0:m1] = dqc
    dpq = None
    if has_p2c:
        gpb = p2c_sums.to(torch.bfloat16)
        dkh += _bmm(gpb, pqh)
        dpq = _bmm(gpb.transpose(1, 2), kh).view(n_seq, H, -1, D).sum(0)
    if has_c2p:
        dpk = dpk.view(n_seq, H, -1, D).sum(0)
    return _rows_first(dqh, n_seq, H), _rows_first(dkh, n_seq, H), _rows_first(dvh, n_seq, H), dpk, dpq


@torch.no_grad()
def attention_backward(
    dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
    pos_key: Optional[torch.Tensor], pos_query: Optional[torch.Tensor], out: torch.Tensor, lse: torch.Tensor,
    *, cu_seqlens: Optional[torch.Tensor] = None, seq_lens: Optional[torch.Tensor] = None, max_seqlen: int,
    sm_scale: float, position_buckets: int = -1, max_relative_positions: int = -1, block_bytes: int = 1 << 31,
    status: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """Gradients of ``ops.disentangled_attention`` for the bf16 path.  ``out`` and ``lse`` are what the forward returned
    (``return_lse=True``), ``dout`` the gradient of ``out``; layouts as in the forward (dense (B, L, H, D) with
    ``seq_lens``, or packed (T, H, D) with ``cu_seqlens``).  Returns (dq, dk, dv, dpos_key, dpos_query) with the shapes
    and dtypes of the inputs; rows outside every sequence get zero gradients."""
    H, D = q.shape[-2], q.shape[-1]
    shape = q.shape
    flat = lambda t: t.reshape(-1, H, D)
    q3, k3, v3, o3, do3 = flat(q), flat(k), flat(v), flat(out), flat(dout)
    lse2 = lse.reshape(-1, H)
    kw = dict(sm_scale=sm_scale, position_buckets=position_buckets, max_relative_positions=max_relative_positions,
              block_bytes=block_bytes, status=status)
    if cu_seqlens is None:
        B, L = shape[0], shape[1]
        lens = None if seq_lens is None else seq_lens.to(torch.int32).contiguous()
        dq, dk, dv, dpk, dpq = _backward_block(q3, k3, v3, o3, do3, lse2, pos_key, pos_query, B, L, lens, **kw)
    else:
        cu = [int(x) for x in cu_seqlens.tolist()]
        dq = torch.zeros(q3.shape, dtype=torch.float32, device=q.device)
        dk, dv = torch.zeros_like(dq), torch.zeros_like(dq)
        dpk = dpq = None
        for s0, s1 in zip(cu[:-1], cu[1:]):
            n = s1 - s0
            if n <= 0:
                continue
            if n > max_seqlen or s1 > q3.shape[0]:
                raise ValueError("cu_seqlens holds a length above max_seqlen or past the last row")
            r = _backward_block(q3[s0:s1], k3[s0:s1], v3[s0:s1], o3[s0:s1], do3[s0:s1], lse2[s0:s1], pos_key, pos_query,
                                1, n, None, **kw)
            dq[s0:s1], dk[s0:s1], dv[s0:s1] = r[0], r[1], r[2]
            if r[3] is not None:
                dpk = r[3] if dpk is None else dpk + r[3]
            if r[4] is not None:
                dpq = r[4] if dpq is None else dpq + r[4]
        if pos_key is not None and dpk is None:
            dpk = torch.zeros(pos_key.shape, dtype=torch.float32, device=q.device)
        if pos_query is not None and dpq is None:
            dpq = torch.zeros(pos_query.shape, dtype=torch.float32, device=q.device)
    return (dq.to(q.dtype).view(shape), dk.to(k.dtype).view(shape), dv.to(v.dtype).view(shape),
            None if dpk is None else dpk.to(pos_key.dtype).view(pos_key.shape),
            None if dpq is None else dpq.to(pos_query.dtype).view(pos_query.shape))
