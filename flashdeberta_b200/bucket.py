"""Relative-position bucket table: built once per (position_buckets, max_relative_positions) on the host by the
library's own integer routine and kept on each device it is used on."""
from __future__ import annotations

import ctypes as C
from typing import Dict, Tuple

import numpy as np
import torch

from . import _lib

_host_cache: Dict[Tuple[int, int], Tuple[np.ndarray, int]] = {}
_dev_cache: Dict[Tuple[int, int, str], torch.Tensor] = {}


def att_span(position_buckets: int, max_relative_positions: int) -> int:
    return position_buckets if position_buckets > 0 else max_relative_positions


def host_lut(position_buckets: int, max_relative_positions: int) -> Tuple[np.ndarray, int]:
    """(table, d_min): table[i] is the row of the position tables for relative distance d_min + i; the first and last
    entries hold for every distance beyond.  Replaces the per-element float math of the reference
    (src/flashdeberta/ops/flash_attention.py:236-254)."""
    key = (int(position_buckets), int(max_relative_positions))
    if key not in _host_cache:
        lib = _lib.load()
        d_min, n = C.c_int32(0), C.c_int32(0)
        _lib.check(lib.fdb_build_bucket_lut(key[0], key[1], None, 0, C.byref(d_min), C.byref(n)))
        buf = np.empty(n.value, dtype=np.int16)
        _lib.check(lib.fdb_build_bucket_lut(key[0], key[1], buf.ctypes.data, n.value, C.byref(d_min), C.byref(n)))
        _host_cache[key] = (buf, d_min.value)
    return _host_cache[key]


def device_lut(position_buckets: int, max_relative_positions: int, device: torch.device) -> Tuple[torch.Tensor, int]:
    tab, d_min = host_lut(position_buckets, max_relative_positions)
    key = (int(position_buckets), int(max_relative_positions), str(device))
    if key not in _dev_cache:
        _dev_cache[key] = torch.from_numpy(tab).to(device)
    return _dev_cache[key], d_min


def relative_index(distance: int, position_buckets: int, max_relative_positions: int) -> int:
    return int(_lib.load().fdb_relative_index(position_buckets, max_relative_positions, int(distance)))
