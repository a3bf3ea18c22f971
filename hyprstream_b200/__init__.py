"""B200-native (sm_100a) attention + quantised KV-cache kernels behind a C ABI (include/hs_attn.h).

Importing the package loads hyprstream_b200/libhs_attn.so and raises if it is missing: there is no
CPU or eager fallback.  Build the library with ``python hyprstream_b200/csrc/build.py``.
"""
from . import ffi  # noqa: F401  (raises ImportError when the library has not been built)
from .ffi import HsError, KVView  # noqa: F401

__all__ = ["ffi", "HsError", "KVView"]
