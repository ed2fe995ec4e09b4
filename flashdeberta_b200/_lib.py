"""ctypes binding of libfdb_b200.so (the C ABI declared in include/fdb_b200.h).

There is no fallback: if the library is missing this module raises, and so does every op built on it.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libfdb_b200.so")

FDB_OK = 0
FDB_BF16, FDB_FP32, FDB_E4M3 = 0, 1, 2
FDB_DEV_TIMEOUT, FDB_DEV_BAD_SEQLEN, FDB_DEV_BAD_INDEX, FDB_DEV_BAD_MASK = 1, 2, 4, 8
STATIC_SCRATCH_BYTES = 8 << 20
ABI_VERSION = 4
PREPARED_SCHEDULE, PREPARED_TABLES = 1, 2  # fdb_attn_params.prepared
TUNE_ONE_LAUNCH, TUNE_TWO_LAUNCHES = 1, 2  # fdb_attn_params.tune


class AttnParams(C.Structure):
    """Mirror of ``fdb_attn_params`` (include/fdb_b200.h); field order and types must match exactly."""

    _fields_ = [
        ("struct_bytes", C.c_uint32), ("dtype", C.c_int32),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("q_row_stride", C.c_int64), ("q_head_stride", C.c_int64),
        ("k_row_stride", C.c_int64), ("k_head_stride", C.c_int64),
        ("v_row_stride", C.c_int64), ("v_head_stride", C.c_int64),
        ("out_row_stride", C.c_int64), ("out_head_stride", C.c_int64),
        ("pos_key", C.c_void_p), ("pos_query", C.c_void_p),
        ("cu_seqlens", C.c_void_p), ("seq_lens", C.c_void_p),
        ("batch", C.c_int32), ("max_seqlen", C.c_int32), ("total_rows", C.c_int32),
        ("heads", C.c_int32), ("head_dim", C.c_int32),
        ("position_buckets", C.c_int32), ("max_relative_positions", C.c_int32),
        ("bucket_lut", C.c_void_p), ("lut_d_min", C.c_int32), ("lut_len", C.c_int32),
        ("sm_scale", C.c_float),
        ("q_scale", C.c_void_p), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
        ("pos_key_scale", C.c_void_p), ("pos_query_scale", C.c_void_p),
        ("lse", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_uint64),
        ("status", C.c_void_p),
        ("prepared", C.c_uint32), ("tune", C.c_uint32),
    ]


EXPORTS = (
    "fdb_abi_version", "fdb_last_error", "fdb_status_string", "fdb_build_bucket_lut", "fdb_relative_index",
    "fdb_attn_workspace_bytes", "fdb_attn_fwd", "fdb_attn_fwd_static", "fdb_attn_fwd_check", "fdb_relative_index_matrix",
    "fdb_quantize_e4m3", "fdb_add_layernorm", "fdb_linear_gelu", "fdb_embed_layernorm",
    "fdb_attn_bwd_probs", "fdb_attn_bwd_bucket_sums",
)

_lib = None


class FdbError(RuntimeError):
    """A call into libfdb_b200.so returned an error code."""

    def __init__(self, code: int, text: str):
        super().__init__(f"libfdb_b200: {text} (code {code})")
        self.code = code


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m flashdeberta_b200.build` (needs nvcc). "
            "flashdeberta_b200 has no fallback path."
        )
    lib = C.CDLL(LIB_PATH)
    lib.fdb_abi_version.restype = C.c_int
    lib.fdb_last_error.restype = C.c_char_p
    lib.fdb_status_string.restype = C.c_char_p
    lib.fdb_status_string.argtypes = [C.c_int]
    lib.fdb_build_bucket_lut.restype = C.c_int
    lib.fdb_build_bucket_lut.argtypes = [C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    lib.fdb_relative_index.restype = C.c_int32
    lib.fdb_relative_index.argtypes = [C.c_int32, C.c_int32, C.c_int64]
    lib.fdb_attn_workspace_bytes.restype = C.c_uint64
    lib.fdb_attn_workspace_bytes.argtypes = [C.POINTER(AttnParams)]
    lib.fdb_attn_fwd.restype = C.c_int
    lib.fdb_attn_fwd.argtypes = [C.POINTER(AttnParams), C.c_void_p]
    lib.fdb_attn_fwd_static.restype = C.c_int
    lib.fdb_attn_fwd_static.argtypes = [C.POINTER(AttnParams), C.c_void_p]
    lib.fdb_attn_fwd_check.restype = C.c_int
    lib.fdb_attn_fwd_check.argtypes = [C.POINTER(AttnParams), C.c_void_p]
    lib.fdb_relative_index_matrix.restype = C.c_int
    lib.fdb_relative_index_matrix.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
    lib.fdb_quantize_e4m3.restype = C.c_int
    lib.fdb_quantize_e4m3.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                      C.c_void_p, C.c_void_p, C.c_void_p]
    lib.fdb_add_layernorm.restype = C.c_int
    lib.fdb_add_layernorm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32,
                                      C.c_float, C.c_void_p]
    lib.fdb_embed_layernorm.restype = C.c_int
    lib.fdb_embed_layernorm.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.c_int64, C.c_int32, C.c_float, C.c_void_p, C.c_void_p]
    lib.fdb_linear_gelu.restype = C.c_int
    lib.fdb_linear_gelu.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32,
                                    C.c_void_p, C.c_void_p]
    for name in ("fdb_attn_bwd_probs", "fdb_attn_bwd_bucket_sums"):  # (const fdb_bwd_block*, stream); struct in backward.py
        getattr(lib, name).restype = C.c_int
        getattr(lib, name).argtypes = [C.c_void_p, C.c_void_p]
    if lib.fdb_abi_version() != ABI_VERSION:
        raise RuntimeError(f"libfdb_b200.so has ABI {lib.fdb_abi_version()}, this package expects {ABI_VERSION}: rebuild")
    _lib = lib
    return lib


def check(code: int) -> None:
    if code != FDB_OK:
        lib = load()
        text = lib.fdb_last_error().decode() or lib.fdb_status_string(code).decode()
        raise FdbError(code, text)
