"""The kernels' size limits, read from `cm_limits.h` (the header the CUDA sources include), so that
the numbers stand in one place.  Needs neither a compiler nor a device: the configuration checks
use it on any machine.  `check_library(handle)` compares with what the loaded library was
compiled with."""
from __future__ import annotations

import os
import re

_HEADER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cm_limits.h")


def _read():
    out = {}
    with open(_HEADER) as fh:
        for line in fh:
            m = re.match(r"#define\s+CM_(\w+)\s+(\d+)\b", line)
            if m:
                out[m.group(1)] = int(m.group(2))
    return out


_LIMITS = _read()
NAMES = tuple(sorted(_LIMITS))

PAGE_TOKENS = _LIMITS["PAGE_TOKENS"]
ATTN_DECODE_CHUNK = _LIMITS["ATTN_DECODE_CHUNK"]
NORM_MAX_WIDTH = _LIMITS["NORM_MAX_WIDTH"]
MAX_HEAD_DIM = _LIMITS["MAX_HEAD_DIM"]
MAX_CONV_TAPS = _LIMITS["MAX_CONV_TAPS"]
SKINNY_MAX_ROWS = _LIMITS["SKINNY_MAX_ROWS"]
FEW_ROWS_MAX_ROWS = _LIMITS["FEW_ROWS_MAX_ROWS"]


def check_library(handle):
    """Raises if the loaded library was compiled with other limits than the header says."""
    import ctypes

    handle.cm_limit.argtypes = [ctypes.c_char_p]
    handle.cm_limit.restype = ctypes.c_longlong
    for name, value in _LIMITS.items():
        got = handle.cm_limit(name.encode())
        if got != value:
            raise RuntimeError(f"the CUDA library was built with {name} = {got}, cm_limits.h says {value}: rebuild it")
