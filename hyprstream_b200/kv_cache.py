"""Python face of the host-side cache objects, which live in C++ (hyprstream_b200/csrc/kv_cache_host.cu): a mirror of
the reference's `LayerKVCache` (crates/hyprstream/src/runtime/kv_cache.rs:1029-1900) and `BlockPool`
(kv_cache.rs:477-680) over device-resident, token-granular storage.  Same names, argument meaning and error behaviour;
what differs on purpose is listed at the top of the C++ file.  This module only forwards to the C ABI
(`hs_cache_*`, `hs_pool_*`, `hs_view_*` in include/hs_attn.h) and turns status codes into exceptions.
"""
from __future__ import annotations

import ctypes
import enum
from typing import List, Optional, Sequence, Tuple

import torch

from . import ffi
from .ffi import KVView, lib

DEFAULT_CHUNK_SIZE = 1024  # kv_cache.rs:700
QUANT_BLOCKSIZE = 64       # kv_cache.rs:704
BLOCK_SIZE = 256           # kv_cache.rs:477 (tokens per page)


class KVQuantType(enum.IntEnum):
    """crates/hyprstream-rpc-std/schema/model.capnp:252-257."""
    NONE = ffi.KV_BF16
    INT8 = ffi.KV_INT8
    NF4 = ffi.KV_NF4
    FP4 = ffi.KV_FP4


class BlockPoolExhausted(RuntimeError):
    """Typed, fail-soft pool exhaustion (kv_cache.rs:482-505): a scheduler may defer admission."""


def _check(status: int) -> None:
    """Status -> the exception the reference's Result would carry."""
    if status == ffi.HS_OK:
        return
    msg = ffi.last_error()
    if status == ffi.HS_ERR_POOL_EXHAUSTED:
        raise BlockPoolExhausted(msg)
    if status in (ffi.HS_ERR_CACHE_OVERFLOW, ffi.HS_ERR_CACHE_EMPTY, ffi.HS_ERR_ARG):
        raise ValueError(msg)
    raise ffi.HsError(status, msg)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class BlockPool:
    """Pre-allocated fixed-size pages with a LIFO free list and per-page owner tags (kv_cache.rs:515-680)."""

    def __init__(self, n_blocks: int, n_kv_heads: int, head_dim: int, device, kind: int = ffi.KV_BF16,
                 block: int = QUANT_BLOCKSIZE, scale_dtype: int = ffi.SCALE_F32, page_tokens: int = BLOCK_SIZE):
        self.kind, self.block, self.scale_dtype = int(kind), block, scale_dtype
        self.n_kv_heads, self.head_dim, self.page_tokens = n_kv_heads, head_dim, page_tokens
        self.device = torch.device(device)
        self.n_blocks = n_blocks
        self._h = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _check(lib.hs_pool_create(n_blocks, page_tokens, self.kind, block, scale_dtype, n_kv_heads, head_dim, ctypes.byref(self._h)))

    def num_free(self) -> int:
        return lib.hs_pool_num_free(self._h)

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None:  # (lib is None when the interpreter is shutting down)
            lib.hs_pool_destroy(self._h)
            self._h = None


class LayerKVCache:
    """KV cache of one attention layer for one sequence (kv_cache.rs:1029-1900)."""

    def __init__(self, max_seq_len: int, quant_type: KVQuantType, n_kv_heads: int, head_dim: int, device,
                 block: int = QUANT_BLOCKSIZE, scale_dtype: int = ffi.SCALE_F32,
                 pool: Optional[BlockPool] = None, owner=None):
        self.max_seq_len = max_seq_len
        self.quant_type = KVQuantType(quant_type)
        self.kind = int(self.quant_type)
        self.n_kv_heads, self.head_dim, self.device = n_kv_heads, head_dim, torch.device(device)
        self.block, self.scale_dtype = block, scale_dtype
        self.pool, self.owner = pool, owner
        self._h = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            if pool is not None:
                if pool.kind != self.kind or pool.n_kv_heads != n_kv_heads or pool.head_dim != head_dim:
                    raise ValueError("pool geometry does not match the cache")
                owner_id = owner if isinstance(owner, int) else abs(hash(owner)) % (1 << 62)
                _check(lib.hs_cache_create_paged(max_seq_len, pool._h, owner_id, ctypes.byref(self._h)))
            else:
                _check(lib.hs_cache_create(max_seq_len, self.kind, block, scale_dtype, n_kv_heads, head_dim, ctypes.byref(self._h)))

    @classmethod
    def new_paged(cls, max_seq_len: int, pool: BlockPool, owner) -> "LayerKVCache":
        """kv_cache.rs:1111 `new_paged`; unlike the reference the pool may hold quantised pages."""
        return cls(max_seq_len, KVQuantType(pool.kind), pool.n_kv_heads, pool.head_dim, pool.device, pool.block,
                   pool.scale_dtype, pool=pool, owner=owner)

    # ---- state ----------------------------------------------------------------------------------
    @property
    def seq_pos(self) -> int:
        return lib.hs_cache_seq_pos(self._h)

    @seq_pos.setter
    def seq_pos(self, n: int) -> None:
        _check(lib.hs_cache_set_seq_pos(self._h, n))

    @property
    def allocated_capacity(self) -> int:
        return lib.hs_cache_capacity(self._h)

    @property
    def blocks(self) -> List[int]:
        return list(range(lib.hs_cache_num_pages(self._h)))

    def _ensure_capacity(self, end_pos: int) -> None:
        with torch.cuda.device(self.device):
            _check(lib.hs_cache_reserve(self._h, end_pos))

    # ---- reference API -----------------------------------------------------------------------
    def update(self, new_keys: torch.Tensor, new_values: torch.Tensor, start_pos: int) -> None:
        """Append [1, T, Hkv, D] bf16 keys/values at `start_pos` (kv_cache.rs:1275-1496)."""
        if new_keys.dim() != 4:
            raise ValueError(f"Expected 4D tensor for keys, got {list(new_keys.shape)}")
        k, v = new_keys.contiguous(), new_values.contiguous()
        with torch.cuda.device(self.device):
            _check(lib.hs_cache_update(self._h, k.data_ptr(), v.data_ptr(), k.shape[1], start_pos, None, None, 0, 0, _stream()))

    def get(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """Keys/values [1, seq_pos, Hkv, D] bf16, dequantised if need be (kv_cache.rs:1499-1643)."""
        n = self.seq_pos
        if n == 0:
            raise ValueError("Cache is empty")
        shape = (1, n, self.n_kv_heads, self.head_dim)
        k = torch.empty(shape, dtype=torch.bfloat16, device=self.device)
        v = torch.empty(shape, dtype=torch.bfloat16, device=self.device)
        with torch.cuda.device(self.device):
            _check(lib.hs_cache_get(self._h, k.data_ptr(), v.data_ptr(), _stream()))
        return k, v

    def clear(self) -> None:
        """kv_cache.rs:1646-1705: drop contents, return pages to the pool."""
        _check(lib.hs_cache_clear(self._h))

    def truncate_to(self, n: int) -> None:
        """kv_cache.rs:1707-1750; token-granular for every storage kind."""
        _check(lib.hs_cache_truncate_to(self._h, n))

    def memory_usage(self) -> int:
        """Bytes held (cf. QuantizedTensor::memory_usage, kv_cache.rs:960-962)."""
        return lib.hs_cache_memory_usage(self._h)

    def snapshot(self):
        """The stored rows as they are (hs_cache_snapshot): (k_data, v_data, k_scales, v_scales) as CPU tensors - uint8
        codes [seq_pos, Hkv, D or D/2] (bf16 values for an unquantised cache) and f32 / f16 scales [seq_pos, Hkv, D/block]
        (None for an unquantised cache).  The cache keeps its contents."""
        n = self.seq_pos
        nbytes = lib.hs_cache_offload_bytes(self._h)
        image = torch.empty(max(nbytes, 1), dtype=torch.uint8).pin_memory()
        with torch.cuda.device(self.device):
            _check(lib.hs_cache_snapshot(self._h, image.data_ptr(), nbytes, _stream()))
        h, d = self.n_kv_heads, self.head_dim
        if self.kind == ffi.KV_BF16:
            row = h * d * 2
            k, v = (image[i * n * row:(i + 1) * n * row].view(torch.bfloat16).view(n, h, d) for i in range(2))
            return k, v, None, None
        row = h * (d if self.kind == ffi.KV_INT8 else d // 2)
        sdt, sb = (torch.float16, 2) if self.scale_dtype == ffi.SCALE_F16 else (torch.float32, 4)
        srow = h * (d // self.block) * sb
        k, v = (image[i * n * row:(i + 1) * n * row].view(n, h, row // h) for i in range(2))
        off = 2 * n * row
        ks, vs = (image[off + i * n * srow:off + (i + 1) * n * srow].view(sdt).view(n, h, d // self.block) for i in range(2))
        return k, v, ks, vs

    def to_device(self, device) -> None:
        """kv_cache.rs:1838-1858 `to_device` (CPU offload / restore).  `cpu` parks the used rows - codes and scales as
        they are, or bf16 values - in pinned host memory and releases the device storage (pages go back to the pool);
        the cache's own device brings them back byte for byte.  Works for every storage kind (the reference moves
        full-precision tensors only)."""
        device = torch.device(device)
        with torch.cuda.device(self.device):
            if device.type == "cpu":
                if getattr(self, "_host_image", None) is not None:
                    return
                n = self.seq_pos
                nbytes = lib.hs_cache_offload_bytes(self._h)
                image = torch.empty(max(nbytes, 1), dtype=torch.uint8).pin_memory()
                _check(lib.hs_cache_offload(self._h, image.data_ptr(), nbytes, _stream()))
                self._host_image = (image, nbytes, n)
            else:
                if device != self.device and device.index is not None and device.index != self.device.index:
                    raise ValueError("a cache is restored to the device it was created on")
                if getattr(self, "_host_image", None) is None:
                    return
                image, nbytes, n = self._host_image
                _check(lib.hs_cache_restore(self._h, image.data_ptr(), nbytes, n, _stream()))
                self._host_image = None

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None:
            lib.hs_cache_destroy(self._h)  # pages go back to the pool on drop (kv_cache.rs:1889-1898)
            self._h = None


class _ViewHandle:
    def __init__(self, handle):
        self.handle = handle

    def __del__(self):
        if self.handle and lib is not None:
            lib.hs_view_destroy(self.handle)
            self.handle = None


def make_view(caches: Sequence[LayerKVCache]) -> Tuple[KVView, list]:
    """One hs_kv_view over the caches of a batch (one sequence each).

    Returns (view, keepalive): the view struct and its device pointer tables belong to the handle in `keepalive`,
    which must outlive the launches that use the view."""
    arr = (ctypes.c_void_p * len(caches))(*[c._h for c in caches])
    h = ctypes.c_void_p()
    with torch.cuda.device(caches[0].device):
        _check(lib.hs_view_create(arr, len(caches), ctypes.byref(h)))
    holder = _ViewHandle(h)
    view = KVView.from_address(lib.hs_view_get(h))
    return view, [holder, list(caches)]


def view_is_current(keepalive: list) -> bool:
    """False once a cache of the view released or replaced storage after the view was built (hs_view_is_current):
    the view's pointer tables are stale then and the view must be rebuilt."""
    return lib.hs_view_is_current(keepalive[0].handle) == ffi.HS_OK
