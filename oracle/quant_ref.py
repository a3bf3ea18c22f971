"""TEST INFRASTRUCTURE ONLY — CPU oracle for the blockwise KV quantiser (numpy + C).

PARITY UNPINNED: the reference calls the un-vendored bitsandbytes 0.45.0 shared library for this
arithmetic (crates/bitsandbytes-sys/build.rs:17-19) and no reference test pins a code or a scale
(crates/hyprstream/src/runtime/kv_cache.rs:2277-2330 asserts shapes only).  The written
specification and its flagged assumptions A1-A6 are in ``oracle/quant_spec.c``.

Two independent restatements of that specification live here so they can check each other:
``quantize_c`` / ``dequantize_c`` (the C file through ctypes) and ``quantize_np`` / ``dequantize_np``
(vectorised numpy).  Only ``tests/``, ``__graft_entry__.smoke`` and ``bench.py``'s CPU-baseline leg
may import this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

INT8, NF4, FP4 = 1, 2, 3
_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libhsq_oracle.so")

# bitsandbytes-sys/src/lib.rs:131-148 / 152-169
NF4_TABLE = np.array(
    [-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
     -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
     0.24611230945587158, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
     0.7229568362236023, 1.0], dtype=np.float32)
FP4_TABLE = np.array([0.0, 0.0625, 0.125, 0.1875, 0.25, 0.3125, 0.375, 0.4375, 0.5, 0.5625, 0.625,
                      0.6875, 0.75, 0.8125, 0.875, 1.0], dtype=np.float32)


def build_c_oracle(force: bool = False) -> str:
    """Compile oracle/quant_spec.c with the committed Makefile (gcc only)."""
    src = os.path.join(_HERE, "quant_spec.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B"])
    return _LIB_PATH


_lib = None


def _c():
    global _lib
    if _lib is None:
        build_c_oracle()
        lib = ctypes.CDLL(_LIB_PATH)
        lib.hsq_quantize_blockwise.restype = ctypes.c_int
        lib.hsq_quantize_blockwise.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int,
                                               ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        lib.hsq_dequantize_blockwise.restype = ctypes.c_int
        lib.hsq_dequantize_blockwise.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int,
                                                 ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        lib.hsq_codebook.restype = ctypes.c_int
        lib.hsq_codebook.argtypes = [ctypes.c_int, ctypes.c_void_p]
        _lib = lib
    return _lib


def codebook(kind: int) -> np.ndarray:
    """f32 codebook of `kind` (lib.rs:104-181)."""
    if kind == INT8:
        return ((np.arange(256, dtype=np.float32) - np.float32(127.0)) / np.float32(127.0)).astype(np.float32)
    if kind == NF4:
        return NF4_TABLE.copy()
    if kind == FP4:
        return FP4_TABLE.copy()
    raise ValueError(f"bad kind {kind}")


def midpoints(kind: int) -> np.ndarray:
    t = codebook(kind)
    return (np.float32(0.5) * (t[:-1] + t[1:]).astype(np.float32)).astype(np.float32)


def n_code_bytes(kind: int, n: int) -> int:
    return n if kind == INT8 else (n + 1) // 2


def _f16_sat(a: np.ndarray) -> np.ndarray:
    """f32 -> f16, nearest even, saturating at 65504 (assumption A6)."""
    with np.errstate(over="ignore"):
        h = a.astype(np.float16)
    h[np.isinf(h) & np.isfinite(a)] = np.float16(65504.0)
    return h


def quantize_np(x: np.ndarray, kind: int, blocksize: int = 64, scale_f16: bool = False):
    """Vectorised numpy restatement of the spec.  `x` is any float array (flattened in C order).

    Returns (codes u8, absmax f32|f16).  Geometry follows QuantizedTensor::from_tensor
    (kv_cache.rs:741-865): block b = elements [b*blocksize, (b+1)*blocksize) of the flat tensor.
    """
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    n = x.size
    nb = (n + blocksize - 1) // blocksize
    pad = nb * blocksize - n
    xp = np.concatenate([x, np.zeros(pad, np.float32)]).reshape(nb, blocksize)
    amax = np.abs(xp).max(axis=1).astype(np.float32) if nb else np.zeros(0, np.float32)
    if scale_f16:
        stored = _f16_sat(amax)
        a = stored.astype(np.float32)
    else:
        stored = amax
        a = amax
    table = codebook(kind)
    mid = midpoints(kind)
    zero_code = int(np.nonzero(table == 0.0)[0][-1])
    with np.errstate(divide="ignore", invalid="ignore"):
        inv = (np.float32(1.0) / a).astype(np.float32)                 # A1
        y = (xp * inv[:, None]).astype(np.float32)                     # A1: single f32 rounding
    c = np.searchsorted(mid, y.reshape(-1), side="left").reshape(nb, blocksize)  # A2: #{mid < y}
    c = np.where(a[:, None] == 0.0, zero_code, c).astype(np.uint8)     # A4
    c = c.reshape(-1)[:n]
    if kind != INT8:
        if n & 1:
            c = np.concatenate([c, np.zeros(1, np.uint8)])
        c = ((c[0::2] << 4) | c[1::2]).astype(np.uint8)                # A3
    return c, stored


def dequantize_np(codes: np.ndarray, absmax: np.ndarray, kind: int, n: int, blocksize: int = 64) -> np.ndarray:
    """out[i] = table[code_i] * absmax[block(i)] in f32 (kv_cache.rs:871-957)."""
    codes = np.ascontiguousarray(codes, dtype=np.uint8).reshape(-1)
    if kind != INT8:
        idx = np.empty(codes.size * 2, np.uint8)
        idx[0::2] = codes >> 4
        idx[1::2] = codes & 0xF
        idx = idx[:n]
    else:
        idx = codes[:n]
    a = np.asarray(absmax).astype(np.float32).reshape(-1)
    blk = np.arange(n) // blocksize
    return (codebook(kind)[idx] * a[blk]).astype(np.float32)


def quantize_c(x: np.ndarray, kind: int, blocksize: int = 64, scale_f16: bool = False):
    """Same contract as `quantize_np`, computed by oracle/quant_spec.c."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    n = x.size
    nb = (n + blocksize - 1) // blocksize
    codes = np.zeros(n_code_bytes(kind, n), np.uint8)
    a32 = np.zeros(max(nb, 1), np.float32)
    a16 = np.zeros(max(nb, 1), np.uint16)
    rc = _c().hsq_quantize_blockwise(kind, x.ctypes.data, n, blocksize, int(scale_f16), codes.ctypes.data,
                                     a32.ctypes.data, a16.ctypes.data)
    if rc != 0:
        raise ValueError("hsq_quantize_blockwise rejected its arguments")
    return codes, (a16[:nb].view(np.float16) if scale_f16 else a32[:nb])


def dequantize_c(codes: np.ndarray, absmax: np.ndarray, kind: int, n: int, blocksize: int = 64) -> np.ndarray:
    codes = np.ascontiguousarray(codes, dtype=np.uint8).reshape(-1)
    out = np.zeros(n, np.float32)
    absmax = np.ascontiguousarray(absmax)
    f16 = absmax.dtype == np.float16
    a32 = absmax if not f16 else np.zeros(1, np.float32)
    a16 = absmax.view(np.uint16) if f16 else np.zeros(1, np.uint16)
    rc = _c().hsq_dequantize_blockwise(kind, codes.ctypes.data, n, blocksize, int(f16), a32.ctypes.data,
                                       a16.ctypes.data, out.ctypes.data)
    if rc != 0:
        raise ValueError("hsq_dequantize_blockwise rejected its arguments")
    return out


# Default used by the parity tests: the C restatement (fast enough for tens of millions of elements).
quantize = quantize_c
dequantize = dequantize_c
