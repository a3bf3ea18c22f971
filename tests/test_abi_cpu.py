"""CPU tests of the boundary: the C-ABI library loads and exports every symbol the header declares."""
import ctypes
import os
import re

import hyprstream_b200
from hyprstream_b200 import ffi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    names = []
    for f in sorted(os.listdir(os.path.join(ROOT, "include"))):
        text = open(os.path.join(ROOT, "include", f)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b(hs_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    declared = header_functions()
    assert len(declared) >= 10
    for name in declared:
        assert hasattr(ffi.lib, name), f"{name} is declared in include/ but not exported"
    assert sorted(ffi.exported_symbols()) == declared, "ffi.py binds a different set than the header declares"


def test_version_and_struct_layout():
    assert ffi.lib.hs_attn_version() >= 100
    assert ctypes.sizeof(ffi.KVView) == 8 * 4 + 4 * 8  # matches struct hs_kv_view


def test_no_cpu_fallback_without_device():
    """Without a usable sm_100 device every compute entry point reports HS_ERR_DEVICE instead of computing."""
    import torch

    if torch.cuda.is_available():
        return
    st = ffi.lib.hs_quantize_blockwise(ffi.KV_INT8, None, ffi.DTYPE_BF16, 64, 64, ffi.SCALE_F32, None, None, None)
    assert st == ffi.HS_ERR_DEVICE and "device" in ffi.last_error().lower()
