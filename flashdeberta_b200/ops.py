"""Op layer: torch tensors in, one call into libfdb_b200.so, torch tensor out.

Takes the place of the reference's Triton op module (src/flashdeberta/ops/flash_attention.py:1088-1091 and
src/flashdeberta/ops/flash_attention_varlen.py:485-511).  The signature differs on purpose: the reference's ops take the
two pre-multiplied bias tensors ``q @ pos_key^T`` and ``k @ pos_query^T`` (model.py:189-192); these take the projected
position tables themselves and the products never exist in global memory.

Forward only, like the reference's packed op (flash_attention_varlen.py:481-483 raises in backward).
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Dict, Optional, Tuple

import torch

from . import _lib, bucket

__all__ = [
    "disentangled_attention", "disentangled_attention_fp8", "disentangled_attention_static", "disentangled_attention_check", "relative_index_matrix", "quantize_e4m3", "add_layernorm", "can_fuse_add_layernorm", "linear_gelu", "can_fuse_linear_gelu", "embed_layernorm",
    "check_status", "launch_count", "PreparedWorkspace",
]

_status: Dict[str, torch.Tensor] = {}
_launches = 0  # kernels this module asked the library to launch (the benchmark reports it)
event_log = None  # set to a list to have every fused-attention call append its (start, end) CUDA events


def launch_count() -> int:
    return _launches


def _status_word(device: torch.device) -> torch.Tensor:
    key = str(device)
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def check_status(device=None) -> None:
    """Read the device status word (synchronises) and raise if a kernel reported an anomaly."""
    for key, t in list(_status.items()):
        if device is not None and key != str(torch.device(device)):
            continue
        v = int(t.item())
        if v:
            t.zero_()
            what = []
            if v & _lib.FDB_DEV_TIMEOUT:
                what.append("a bounded wait inside the attention kernel ran out (output invalid)")
            if v & _lib.FDB_DEV_BAD_SEQLEN:
                what.append("cu_seqlens/seq_lens hold a length below zero or above max_seqlen")
            if v & _lib.FDB_DEV_BAD_INDEX:
                what.append("an input id lies outside the embedding table")
            if v & _lib.FDB_DEV_BAD_MASK:
                what.append("a dense attention mask was not right-padded (valid tokens must be a prefix of each row; "
                            "pack the batch to use other layouts)")
            raise RuntimeError("flashdeberta_b200 device status %d: %s" % (v, "; ".join(what)))


def tensor_stamp(t: Optional[torch.Tensor], held: bool = False):
    """(address, version counter) of a tensor: equal stamps of the same live tensor mean "not modified in place since".
    Tensors made under ``torch.inference_mode()`` keep no version counter (reading it raises).  For those the stamp is the
    object's identity when the caller keeps a reference to the tensor (``held``: the address cannot be reused, and such
    tensors cannot be written outside inference mode), else None, which callers treat as "changed"."""
    if t is None:
        return None
    if t.is_inference():
        return ("inference", id(t), t.data_ptr()) if held else None
    return (t.data_ptr(), t._version)


def flag_status(device: torch.device, condition: torch.Tensor, bit: int) -> None:
    """OR ``bit`` into the device status word where the 0-d boolean ``condition`` (on that device) is true.  No host
    synchronisation: the word is read by ``check_status``."""
    _status_word(device).bitwise_or_(condition.to(torch.int32) * bit)


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _lib.FDB_BF16
    if t.dtype == torch.float32:
        return _lib.FDB_FP32
    if t.dtype == torch.float8_e4m3fn:
        return _lib.FDB_E4M3
    raise TypeError(f"unsupported dtype {t.dtype}")


def _rows_view(x: torch.Tensor) -> Tuple[torch.Tensor, int, int]:
    """(rows, H, D) view of a (rows, H, D) or (B, L, H, D) tensor without copying when the layout allows it.
    Returns the view, its row stride and head stride in elements."""
    if x.dim() == 4:
        B, L, H, D = x.shape
        if x.stride(0) != L * x.stride(1):
            x = x.contiguous()
        x = x.as_strided((B * L, H, D), (x.stride(1), x.stride(2), x.stride(3)), x.storage_offset())
    if x.dim() != 3:
        raise ValueError("expected (rows, heads, head_dim) or (batch, seq, heads, head_dim)")
    if x.stride(2) != 1:
        x = x.contiguous()
    return x, x.stride(0), x.stride(1)


def _fill_params(q, k, v, pos_key, pos_query, cu_seqlens, seq_lens, max_seqlen, sm_scale, position_buckets,
                 max_relative_positions, out, lse, scales=None):
    dev = q.device
    q3, q_rs, q_hs = _rows_view(q)
    k3, k_rs, k_hs = _rows_view(k)
    v3, v_rs, v_hs = _rows_view(v)
    rows, H, D = q3.shape
    if k3.shape != q3.shape or v3.shape != q3.shape:
        raise ValueError("q, k and v must have the same shape")
    p = _lib.AttnParams()
    p.struct_bytes = C.sizeof(_lib.AttnParams)
    p.dtype = _dtype_code(q3)
    keep = [q3, k3, v3]
    p.q, p.k, p.v, p.out = q3.data_ptr(), k3.data_ptr(), v3.data_ptr(), out.data_ptr()
    p.q_row_stride, p.q_head_stride = q_rs, q_hs
    p.k_row_stride, p.k_head_stride = k_rs, k_hs
    p.v_row_stride, p.v_head_stride = v_rs, v_hs
    p.out_row_stride, p.out_head_stride = H * D, D
    span = bucket.att_span(position_buckets, max_relative_positions)
    for name, t in (("pos_key", pos_key), ("pos_query", pos_query)):
        if t is None:
            continue
        if t.dim() == 4 and t.shape[0] == 1:
            t = t[0]
        if t.shape != (H, 2 * span, D):
            raise ValueError(f"{name} must be (heads, 2*att_span, head_dim) = {(H, 2 * span, D)}, got {tuple(t.shape)}")
        if t.dtype != q3.dtype:
            raise TypeError(f"{name} dtype {t.dtype} differs from q dtype {q3.dtype}")
        t = t.contiguous()
        keep.append(t)
        setattr(p, name, t.data_ptr())
    if pos_key is not None or pos_query is not None:
        lut, d_min = bucket.device_lut(position_buckets, max_relative_positions, dev)
        p.bucket_lut, p.lut_d_min, p.lut_len = lut.data_ptr(), d_min, lut.numel()
    if cu_seqlens is not None:
        if cu_seqlens.dtype != torch.int32 or not cu_seqlens.is_contiguous():
            cu_seqlens = cu_seqlens.to(torch.int32).contiguous()
        keep.append(cu_seqlens)
        p.cu_seqlens = cu_seqlens.data_ptr()
        p.batch = cu_seqlens.numel() - 1
    else:
        if q.dim() != 4:
            raise ValueError("dense layout needs (batch, seq, heads, head_dim) inputs")
        p.batch = q.shape[0]
        if max_seqlen != q.shape[1]:
            raise ValueError("dense layout: max_seqlen must equal the padded length")
        if seq_lens is not None:
            if seq_lens.dtype != torch.int32 or not seq_lens.is_contiguous():
                seq_lens = seq_lens.to(torch.int32).contiguous()
            keep.append(seq_lens)
            p.seq_lens = seq_lens.data_ptr()
    p.max_seqlen, p.total_rows, p.heads, p.head_dim = int(max_seqlen), rows, H, D
    p.position_buckets, p.max_relative_positions = int(position_buckets), int(max_relative_positions)
    p.sm_scale = float(sm_scale)
    if scales is not None:
        for name, t in scales.items():
            if t is not None:
                t = t.to(torch.float32).contiguous()
                keep.append(t)
                setattr(p, name, t.data_ptr())
    if lse is not None:
        p.lse = lse.data_ptr()
    p.status = _status_word(dev).data_ptr()
    return p, keep


def _out_like(q: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    return torch.empty(q.shape, dtype=dtype, device=q.device)


class PreparedWorkspace:
    """A workspace that one caller (an attention module) keeps between calls, so that what the set-up kernels wrote into
    it can be used again (``fdb_attn_params.prepared``): the position tables gathered through the bucket index as long
    as the same table tensors come back unmodified, the order of the query tiles as long as the batch has the same shape
    and either no padding or the same, unmodified lengths tensor.  Workspaces above ``max_bytes`` (long sequences in two launches: partial results per row) are not
    kept; such calls take a fresh scratch buffer as without this object.

    "Unmodified" is judged by the tensor's address and version counter.  A write that bypasses the counter (through
    ``.data``, a DLPack alias, a raw CUDA kernel) is not seen: after such a write to a lengths or table tensor, pass a new
    tensor or drop this object (``module._prepared = ops.PreparedWorkspace()``)."""

    max_bytes = 64 << 20

    def __init__(self):
        self.buf = None
        self.layout = None     # everything the workspace layout and the schedule depend on
        self.schedule = None   # whose tile order `buf` holds: ("full",) for an unpadded batch, else (data_ptr, version) of the lengths tensor
        self.tables = None     # (data_ptr, version) of the table tensors gathered into `buf`
        self.keep = None       # those tensors, so that their addresses stay theirs
        self.stream = None     # the stream whose order protects `buf`


def disentangled_attention(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
    pos_key: Optional[torch.Tensor], pos_query: Optional[torch.Tensor],
    *, cu_seqlens: Optional[torch.Tensor] = None, seq_lens: Optional[torch.Tensor] = None,
    max_seqlen: int, sm_scale: Optional[float] = None, position_buckets: int = -1, max_relative_positions: int = -1,
    return_lse: bool = False, scales: Optional[dict] = None, prepared: Optional[PreparedWorkspace] = None,
    tune: int = 0,
):
    """softmax((Q K^T + c2p + p2c) * sm_scale) V on the fused sm_100a kernel.

    q, k, v: (B, L, H, 64) [dense, right-padded, lengths in ``seq_lens`` or all L] or (T, H, 64) [packed, with
    ``cu_seqlens``]; bf16 (or float8_e4m3fn with ``scales``).  pos_key / pos_query: (H, 2*att_span, 64) projected
    relative-position tables or None.  Returns bf16 of q's shape (and the natural-log LSE (rows, H) when asked).
    ``tune``: ``_lib.TUNE_*`` bits that force which kernels the call is split into (tests and tuning runs; 0 = the
    library chooses).
    """
    global _launches
    if not q.is_cuda:
        raise RuntimeError("flashdeberta_b200 runs on CUDA devices only; there is no CPU path")
    lib = _lib.load()
    D = q.shape[-1]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D * (1 + int(pos_key is not None) + int(pos_query is not None)))
    if wants_grad(q, k, v, pos_key, pos_query):
        # autograd is recording: the call goes through the training op (output and LSE kept), whose backward is
        # flashdeberta_b200.backward
        if scales is not None or return_lse:
            raise RuntimeError("no gradient is implemented for the e4m3 path or for the LSE output; "
                               "call under torch.no_grad() or detach the inputs")
        return attn_fwd_train_op(q, k, v, pos_key, pos_query, cu_seqlens, seq_lens, int(max_seqlen), float(sm_scale),
                                 int(position_buckets), int(max_relative_positions))[0]
    out = _out_like(q, torch.bfloat16)
    rows = out.numel() // (out.shape[-1] * out.shape[-2])
    lse = torch.empty(rows, q.shape[-2], dtype=torch.float32, device=q.device) if return_lse else None
    with torch.cuda.device(q.device):
        p, keep = _fill_params(q, k, v, pos_key, pos_query, cu_seqlens, seq_lens, max_seqlen, sm_scale,
                               position_buckets, max_relative_positions, out, lse, scales)
        p.tune = int(tune)
        need = lib.fdb_attn_workspace_bytes(C.byref(p))
        if need == 0:  # invalid parameters (raises with the library's message) or an empty batch
            _lib.check(lib.fdb_attn_fwd(C.byref(p), None))
            return (out, lse) if return_lse else out
        stream = torch.cuda.current_stream(q.device).cuda_stream
        flags = 0
        if prepared is not None and need <= prepared.max_bytes and prepared.stream in (None, stream):
            prepared.stream = stream  # the buffer stays with the first stream that used it; other streams take scratch
            layout = (q.device, stream, need, p.dtype, p.batch, p.max_seqlen, p.total_rows, p.heads, int(position_buckets),
                      int(max_relative_positions), cu_seqlens is not None)
            tables = tuple(tensor_stamp(t, held=True) for t in (pos_key, pos_query))  # kept alive in `prepared.keep`
            if any(s is None and t is not None for s, t in zip(tables, (pos_key, pos_query))):
                tables = None  # a table without a version counter: gathered again on every call
            lens_t = cu_seqlens if cu_seqlens is not None else seq_lens
            # the lengths behind the tile order: none (an unpadded batch), or this very tensor, unmodified
            full = ("full",) if lens_t is None else tensor_stamp(lens_t)
            if prepared.buf is None or prepared.layout != layout:
                prepared.buf = torch.empty(need + 256, dtype=torch.uint8, device=q.device)
            else:
                if full is not None and prepared.schedule == full:
                    flags |= _lib.PREPARED_SCHEDULE
                if tables is not None and prepared.tables == tables and tables != (None, None):
                    flags |= _lib.PREPARED_TABLES
            prepared.layout, prepared.schedule, prepared.tables, prepared.keep = None, None, None, None
            ws = prepared.buf
        else:
            ws = torch.empty(need + 256, dtype=torch.uint8, device=q.device)
        base = (ws.data_ptr() + 255) & ~255
        p.workspace, p.workspace_bytes, p.prepared = base, need, flags
        if event_log is not None:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        _lib.check(lib.fdb_attn_fwd(C.byref(p), C.c_void_p(stream)))
        if event_log is not None:
            ev1.record()
            event_log.append((ev0, ev1))
        if prepared is not None and ws is prepared.buf:  # the call went through: the workspace holds this call's set-up
            prepared.layout, prepared.schedule, prepared.tables, prepared.keep = layout, full, tables, (pos_key, pos_query, lens_t)
        _launches += 1 + int(not flags & _lib.PREPARED_SCHEDULE) + \
            int((pos_key is not None or pos_query is not None) and not flags & _lib.PREPARED_TABLES)
        # `keep` and `ws` were allocated on this stream, so the caching allocator reuses them in stream order
        del keep, ws
    return (out, lse) if return_lse else out


def disentangled_attention_fp8(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
    pos_key: Optional[torch.Tensor], pos_query: Optional[torch.Tensor],
    *, cu_seqlens: Optional[torch.Tensor] = None, seq_lens: Optional[torch.Tensor] = None,
    max_seqlen: int, sm_scale: Optional[float] = None, position_buckets: int = -1, max_relative_positions: int = -1,
):
    """FP8 attention: bf16 inputs are scaled to float8-e4m3 with one amax-derived scale per (sequence, head) for q, k, v
    and per head for the position tables, the fused kernel runs its MMAs in e4m3 with fp32 accumulation (P is stored as
    2^8 * exp2(.) in e4m3), and the scales are folded back into the softmax scale and the output.  No counterpart in the
    reference.  Returns bf16."""
    if wants_grad(q, k, v, pos_key, pos_query):
        raise RuntimeError("the e4m3 attention is forward-only; train with attn_fp8 off")
    if q.dim() == 4:
        B, L = q.shape[0], q.shape[1]
        slabs = torch.arange(0, (B + 1) * L, L, dtype=torch.int32, device=q.device)
    else:
        if cu_seqlens is None:
            raise ValueError("packed inputs need cu_seqlens")
        slabs = cu_seqlens.to(torch.int32)
    q8, sq = quantize_e4m3(q, slabs)
    k8, sk = quantize_e4m3(k, slabs)
    v8, sv = quantize_e4m3(v, slabs)
    scales = {"q_scale": sq, "k_scale": sk, "v_scale": sv}
    tabs = {}
    for name, t in (("pos_key", pos_key), ("pos_query", pos_query)):
        if t is None:
            tabs[name] = None
            continue
        H, R, D = t.shape
        rows = t.contiguous().view(H * R, 1, D)
        y, sc = quantize_e4m3(rows, torch.arange(0, (H + 1) * R, R, dtype=torch.int32, device=t.device))
        tabs[name] = y.view(H, R, D)
        scales[name + "_scale"] = sc.view(H)
    return disentangled_attention(q8, k8, v8, tabs["pos_key"], tabs["pos_query"], cu_seqlens=cu_seqlens,
                                  seq_lens=seq_lens, max_seqlen=max_seqlen, sm_scale=sm_scale,
                                  position_buckets=position_buckets, max_relative_positions=max_relative_positions,
                                  scales=scales)


def disentangled_attention_static(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
    pos_key: Optional[torch.Tensor], pos_query: Optional[torch.Tensor],
    *, out: torch.Tensor, cu_seqlens: Optional[torch.Tensor] = None, seq_lens: Optional[torch.Tensor] = None,
    max_seqlen: int, sm_scale: Optional[float] = None, position_buckets: int = -1, max_relative_positions: int = -1,
) -> torch.Tensor:
    """The fused kernel through ``fdb_attn_fwd_static``: no workspace is allocated here or in the library; the scratch
    is the library's built-in per-device array (``_lib.STATIC_SCRATCH_BYTES``).  For callers that must not allocate on
    the device at call time; ``out`` (bf16, q's shape, contiguous) is supplied by the caller for the same reason.
    Calls on one device share that array, so keep them ordered on one stream.  Larger problems raise FdbError
    (code -6)."""
    global _launches
    if not q.is_cuda:
        raise RuntimeError("flashdeberta_b200 runs on CUDA devices only; there is no CPU path")
    if out.dtype != torch.bfloat16 or out.shape != q.shape or not out.is_contiguous():
        raise ValueError("out must be a contiguous bf16 tensor of q's shape")
    lib = _lib.load()
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.shape[-1] * (1 + int(pos_key is not None) + int(pos_query is not None)))
    with torch.cuda.device(q.device):
        p, keep = _fill_params(q, k, v, pos_key, pos_query, cu_seqlens, seq_lens, max_seqlen, sm_scale,
                               position_buckets, max_relative_positions, out, None)
        stream = torch.cuda.current_stream(q.device).cuda_stream
        _lib.check(lib.fdb_attn_fwd_static(C.byref(p), C.c_void_p(stream)))
        _launches += 2 + int(pos_key is not None or pos_query is not None)
        del keep
    return out


def disentangled_attention_check(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
    pos_key: Optional[torch.Tensor], pos_query: Optional[torch.Tensor],
    *, cu_seqlens: Optional[torch.Tensor] = None, seq_lens: Optional[torch.Tensor] = None,
    max_seqlen: int, sm_scale: Optional[float] = None, position_buckets: int = -1, max_relative_positions: int = -1,
    return_lse: bool = False,
):
    """Same contract on the library's plain-fp32 check kernel (bf16 or fp32 inputs, head_dim <= 128).  Validation only."""
    global _launches
    if not q.is_cuda:
        raise RuntimeError("flashdeberta_b200 runs on CUDA devices only; there is no CPU path")
    lib = _lib.load()
    D = q.shape[-1]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D * (1 + int(pos_key is not None) + int(pos_query is not None)))
    out = _out_like(q, q.dtype)
    rows = out.numel() // (out.shape[-1] * out.shape[-2])
    lse = torch.empty(rows, q.shape[-2], dtype=torch.float32, device=q.device) if return_lse else None
    with torch.cuda.device(q.device):
        p, keep = _fill_params(q, k, v, pos_key, pos_query, cu_seqlens, seq_lens, max_seqlen, sm_scale,
                               position_buckets, max_relative_positions, out, lse)
        stream = torch.cuda.current_stream(q.device).cuda_stream
        _lib.check(lib.fdb_attn_fwd_check(C.byref(p), C.c_void_p(stream)))
        _launches += 1
    return (out, lse) if return_lse else out


def relative_index_matrix(len_q: int, len_k: int, position_buckets: int, max_relative_positions: int,
                          device) -> torch.Tensor:
    """(len_q, len_k) int32 matrix of position-table rows as the device code looks them up (for the bit-exactness test
    against transformers' build_relative_position + clamp)."""
    global _launches
    lib = _lib.load()
    device = torch.device(device)
    lut, d_min = bucket.device_lut(position_buckets, max_relative_positions, device)
    out = torch.empty(len_q, len_k, dtype=torch.int32, device=device)
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device).cuda_stream
        _lib.check(lib.fdb_relative_index_matrix(lut.data_ptr(), d_min, lut.numel(), len_q, len_k, out.data_ptr(),
                                                 C.c_void_p(stream)))
        _launches += 1
    return out


def quantize_e4m3(x: torch.Tensor, slab_start: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 (rows, H, D) -> (float8_e4m3fn (rows, H, D) contiguous, scale (n_slabs, H) fp32) with one amax-derived scale per
    (slab, head); slab s = rows [slab_start[s], slab_start[s+1])."""
    global _launches
    lib = _lib.load()
    x3, rs, hs = _rows_view(x)
    rows, H, D = x3.shape
    slab_start = slab_start.to(torch.int32).contiguous()
    n = slab_start.numel() - 1
    y = torch.empty(rows, H, D, dtype=torch.float8_e4m3fn, device=x.device)
    scale = torch.empty(n, H, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream(x.device).cuda_stream
        _lib.check(lib.fdb_quantize_e4m3(x3.data_ptr(), rows, rs, hs, slab_start.data_ptr(), n, H, D, y.data_ptr(),
                                         scale.data_ptr(), C.c_void_p(stream)))
        _launches += 1
    return y.view(x.shape), scale


def can_fuse_add_layernorm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> bool:
    """True when ``add_layernorm`` covers this case: CUDA bf16 activations and parameters, hidden a multiple of 256 up to
    2048."""
    hidden = x.shape[-1]
    return (x.is_cuda and x.dtype == torch.bfloat16 and bias is not None and weight.dtype == torch.bfloat16
            and bias.dtype == torch.bfloat16 and hidden % 256 == 0 and hidden <= 2048)


def add_layernorm(x: torch.Tensor, residual: Optional[torch.Tensor], weight: torch.Tensor, bias: torch.Tensor,
                  eps: float) -> torch.Tensor:
    """LayerNorm(x + residual) over the last dimension in one pass (``fdb_add_layernorm``): the tail of transformers'
    DebertaV2SelfOutput / DebertaV2Output, which the reference's layer classes keep (src/flashdeberta/model.py:259-272).
    bf16 in and out, fp32 statistics, the sum rounded to bf16 first as in the eager expression."""
    global _launches
    if not can_fuse_add_layernorm(x, weight, bias):
        raise ValueError("add_layernorm needs CUDA bf16 tensors with hidden a multiple of 256 up to 2048")
    lib = _lib.load()
    hidden = x.shape[-1]
    x2 = x.reshape(-1, hidden)
    x2 = x2 if x2.is_contiguous() else x2.contiguous()
    r2 = None
    if residual is not None:
        if residual.shape != x.shape or residual.dtype != x.dtype or residual.device != x.device:
            raise ValueError("residual must match x in shape, dtype and device")
        r2 = residual.reshape(-1, hidden)
        r2 = r2 if r2.is_contiguous() else r2.contiguous()
    out = torch.empty_like(x2)
    if x2.shape[0] == 0:
        return out.view(x.shape)
    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream(x.device).cuda_stream
        _lib.check(lib.fdb_add_layernorm(x2.data_ptr(), r2.data_ptr() if r2 is not None else None,
                                         weight.contiguous().data_ptr(), bias.contiguous().data_ptr(), out.data_ptr(),
                                         x2.shape[0], hidden, float(eps), C.c_void_p(stream)))
        _launches += 1
    return out.view(x.shape)


def embed_layernorm(ids: torch.Tensor, table: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float,
                    row_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """LayerNorm(table[ids]) * row_scale[..., None] in one kernel (``fdb_embed_layernorm``): transformers'
    DebertaV2Embeddings for word embeddings alone, which the reference's model keeps (src/flashdeberta/model.py:394-428).
    ids: integer tensor of any shape; table: (vocab, hidden) bf16; row_scale: ids' shape (the mask) or None.  Returns
    bf16 of shape ids.shape + (hidden,)."""
    global _launches
    hidden = table.shape[-1]
    if not (table.is_cuda and table.dim() == 2 and table.is_contiguous() and can_fuse_add_layernorm(table, weight, bias)):
        raise ValueError("embed_layernorm needs a contiguous CUDA bf16 table with hidden a multiple of 256 up to 2048")
    lib = _lib.load()
    ids1 = ids.reshape(-1).to(device=table.device, dtype=torch.int64).contiguous()
    scale1 = None
    if row_scale is not None:
        if row_scale.numel() != ids1.numel():
            raise ValueError("row_scale must have one entry per id")
        # the mask as the eager expression uses it: cast to the activation dtype first
        scale1 = row_scale.reshape(-1).to(device=table.device, dtype=torch.bfloat16).to(torch.float32).contiguous()
    out = torch.empty(ids1.numel(), hidden, dtype=torch.bfloat16, device=table.device)
    if ids1.numel() == 0:
        return out.view(*ids.shape, hidden)
    with torch.cuda.device(table.device):
        stream = torch.cuda.current_stream(table.device).cuda_stream
        _lib.check(lib.fdb_embed_layernorm(ids1.data_ptr(), table.data_ptr(), table.shape[0],
                                           weight.contiguous().data_ptr(), bias.contiguous().data_ptr(),
                                           scale1.data_ptr() if scale1 is not None else None, out.data_ptr(),
                                           ids1.numel(), hidden, float(eps), _status_word(table.device).data_ptr(),
                                           C.c_void_p(stream)))
        _launches += 1
    return out.view(*ids.shape, hidden)


def can_fuse_linear_gelu(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> bool:
    """True when ``linear_gelu`` can take the call: CUDA bf16, in_features a multiple of 64, out_features of 256."""
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.device == x.device
            and weight.dim() == 2 and x.shape[-1] == weight.shape[1] and weight.shape[1] % 64 == 0
            and weight.shape[0] % 256 == 0 and weight.is_contiguous()
            and (bias is None or (bias.dtype == torch.bfloat16 and bias.device == x.device and bias.is_contiguous()
                                  and bias.numel() == weight.shape[0])))


def linear_gelu(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """GELU(x @ weight.T + bias) in one kernel (``fdb_linear_gelu``): the intermediate block of a layer, transformers'
    DebertaV2Intermediate, which the reference's layer class keeps (src/flashdeberta/model.py:265-272).  erf GELU, the
    sum rounded to bf16 before the activation as the two separate kernels would."""
    global _launches
    if not can_fuse_linear_gelu(x, weight, bias):
        raise ValueError("linear_gelu needs CUDA bf16 tensors, in_features a multiple of 64 and out_features of 256")
    lib = _lib.load()
    k, n = weight.shape[1], weight.shape[0]
    x2 = x.reshape(-1, k)
    x2 = x2 if x2.is_contiguous() else x2.contiguous()
    out = torch.empty(x2.shape[0], n, dtype=torch.bfloat16, device=x.device)
    if x2.shape[0] == 0:
        return out.view(*x.shape[:-1], n)
    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream(x.device).cuda_stream
        _lib.check(lib.fdb_linear_gelu(x2.data_ptr(), weight.data_ptr(), bias.data_ptr() if bias is not None else None,
                                       out.data_ptr(), x2.shape[0], k, n, _status_word(x.device).data_ptr(),
                                       C.c_void_p(stream)))
        _launches += 1
    return out.view(*x.shape[:-1], n)


# --------------------------------------------------------------------------------------------------------------------
# torch custom op (so the call shows up as one node for tracing / meta tensors); thin wrapper over the function above
# --------------------------------------------------------------------------------------------------------------------
@torch.library.custom_op("flashdeberta_b200::attn_fwd", mutates_args=())
def attn_fwd_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, pos_key: Optional[torch.Tensor],
                pos_query: Optional[torch.Tensor], cu_seqlens: Optional[torch.Tensor],
                seq_lens: Optional[torch.Tensor], max_seqlen: int, sm_scale: float, position_buckets: int,
                max_relative_positions: int) -> torch.Tensor:
    return disentangled_attention(q, k, v, pos_key, pos_query, cu_seqlens=cu_seqlens, seq_lens=seq_lens,
                                  max_seqlen=max_seqlen, sm_scale=sm_scale, position_buckets=position_buckets,
                                  max_relative_positions=max_relative_positions)


@attn_fwd_op.register_fake
def _(q, k, v, pos_key, pos_query, cu_seqlens, seq_lens, max_seqlen, sm_scale, position_buckets,
      max_relative_positions):
    return torch.empty(q.shape, dtype=torch.bfloat16, device=q.device)


@torch.library.custom_op("flashdeberta_b200::attn_bwd", mutates_args=())
def attn_bwd_op(dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, pos_key: Optional[torch.Tensor],
                pos_query: Optional[torch.Tensor], out: Optional[torch.Tensor], lse: Optional[torch.Tensor],
                cu_seqlens: Optional[torch.Tensor], seq_lens: Optional[torch.Tensor], max_seqlen: int, sm_scale: float,
                position_buckets: int,
                max_relative_positions: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Gradients of the attention (dq, dk, dv, dpos_key, dpos_query; an absent table gives an empty tensor).  ``out``
    and ``lse`` are the forward's results when the caller kept them (``attn_fwd_train``); without them the fused forward
    is run again here, which costs less than a tenth of the backward and keeps nothing but the inputs alive."""
    from . import backward
    if out is None or lse is None:
        out, lse = disentangled_attention(q, k, v, pos_key, pos_query, cu_seqlens=cu_seqlens, seq_lens=seq_lens,
                                          max_seqlen=max_seqlen, sm_scale=sm_scale, position_buckets=position_buckets,
                                          max_relative_positions=max_relative_positions, return_lse=True)
    dq, dk, dv, dpk, dpq = backward.attention_backward(
        dout, q, k, v, pos_key, pos_query, out, lse, cu_seqlens=cu_seqlens, seq_lens=seq_lens, max_seqlen=max_seqlen,
        sm_scale=sm_scale, position_buckets=position_buckets, max_relative_positions=max_relative_positions,
        status=_status_word(q.device))
    return dq, dk, dv, q.new_zeros(0) if dpk is None else dpk, q.new_zeros(0) if dpq is None else dpq


@attn_bwd_op.register_fake
def _(dout, q, k, v, pos_key, pos_query, out, lse, cu_seqlens, seq_lens, max_seqlen, sm_scale, position_buckets,
      max_relative_positions):
    return (torch.empty_like(q), torch.empty_like(k), torch.empty_like(v),
            q.new_zeros(0) if pos_key is None else torch.empty_like(pos_key),
            q.new_zeros(0) if pos_query is None else torch.empty_like(pos_query))


def _attn_setup(ctx, inputs, output):
    q, k, v, pos_key, pos_query, cu_seqlens, seq_lens, max_seqlen, sm_scale, position_buckets, max_rel = inputs
    ctx.save_for_backward(q, k, v, pos_key, pos_query, cu_seqlens, seq_lens)
    ctx.fdb_args = (max_seqlen, sm_scale, position_buckets, max_rel)


def _attn_backward(ctx, grad):
    q, k, v, pos_key, pos_query, cu_seqlens, seq_lens = ctx.saved_tensors
    dq, dk, dv, dpk, dpq = attn_bwd_op(grad.contiguous(), q, k, v, pos_key, pos_query, None, None, cu_seqlens, seq_lens,
                                       *ctx.fdb_args)
    return (dq, dk, dv, None if pos_key is None else dpk, None if pos_query is None else dpq,
            None, None, None, None, None, None)


attn_fwd_op.register_autograd(_attn_backward, setup_context=_attn_setup)


@torch.library.custom_op("flashdeberta_b200::attn_fwd_train", mutates_args=())
def attn_fwd_train_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, pos_key: Optional[torch.Tensor],
                      pos_query: Optional[torch.Tensor], cu_seqlens: Optional[torch.Tensor],
                      seq_lens: Optional[torch.Tensor], max_seqlen: int, sm_scale: float, position_buckets: int,
                      max_relative_positions: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """The forward as the training path calls it: returns the output and the natural-log LSE (rows, heads), both kept
    for the backward so that it does not run the forward again.  The LSE output carries no gradient."""
    return disentangled_attention(q, k, v, pos_key, pos_query, cu_seqlens=cu_seqlens, seq_lens=seq_lens,
                                  max_seqlen=max_seqlen, sm_scale=sm_scale, position_buckets=position_buckets,
                                  max_relative_positions=max_relative_positions, return_lse=True)


@attn_fwd_train_op.register_fake
def _(q, k, v, pos_key, pos_query, cu_seqlens, seq_lens, max_seqlen, sm_scale, position_buckets,
      max_relative_positions):
    rows = q.numel() // (q.shape[-1] * q.shape[-2])
    return (torch.empty(q.shape, dtype=torch.bfloat16, device=q.device),
            torch.empty(rows, q.shape[-2], dtype=torch.float32, device=q.device))


def _train_setup(ctx, inputs, output):
    q, k, v, pos_key, pos_query, cu_seqlens, seq_lens, max_seqlen, sm_scale, position_buckets, max_rel = inputs
    out, lse = output
    ctx.save_for_backward(q, k, v, pos_key, pos_query, cu_seqlens, seq_lens, out, lse)
    ctx.fdb_args = (max_seqlen, sm_scale, position_buckets, max_rel)
    ctx.mark_non_differentiable(lse)


def _train_backward(ctx, grad, grad_lse):
    q, k, v, pos_key, pos_query, cu_seqlens, seq_lens, out, lse = ctx.saved_tensors
    dq, dk, dv, dpk, dpq = attn_bwd_op(grad.contiguous(), q, k, v, pos_key, pos_query, out, lse, cu_seqlens, seq_lens,
                                       *ctx.fdb_args)
    return (dq, dk, dv, None if pos_key is None else dpk, None if pos_query is None else dpq,
            None, None, None, None, None, None)


attn_fwd_train_op.register_autograd(_train_backward, setup_context=_train_setup)


def wants_grad(*tensors) -> bool:
    """True when autograd is recording and one of the tensors takes part in it."""
    return torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors)
