"""Host-side mirror of the reference's per-layer KV cache (crates/hyprstream/src/runtime/kv_cache.rs),
re-designed so that quantised storage is device-resident and token-granular.

Same names, argument meaning and error behaviour as `LayerKVCache` (kv_cache.rs:1029-1900) and
`BlockPool` (kv_cache.rs:477-680); what differs, on purpose:

* quantised codes and scales live in HBM (the reference keeps them in host `Vec<u8>` and copies
  across PCIe on every quantise/dequantise, kv_cache.rs:845-856,919-921);
* every token is quantised when it is written (no 64-token full-precision staging buffer and no
  whole-history re-quantisation on flush, kv_cache.rs:1204-1272): blocks never straddle a token, so
  the codes are those the reference produces at flush;
* `truncate_to` on a quantised cache is a length change (the reference clears, kv_cache.rs:1717-1720);
* paged storage may be quantised (the reference forbids the combination, kv_cache.rs:1111).

torch is used only to own device memory.
"""
from __future__ import annotations

import enum
import math
from typing import List, Optional, Sequence, Tuple

import torch

from . import ffi, ops
from .ffi import KVView

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


def _row_bytes(kind: int, n_kv_heads: int, head_dim: int) -> int:
    per = {ffi.KV_BF16: 2 * head_dim, ffi.KV_INT8: head_dim}.get(kind, head_dim // 2)
    return n_kv_heads * per


class _Storage:
    """K/V data + scale buffers for `capacity` tokens of one sequence (or one page)."""

    def __init__(self, kind: int, capacity: int, n_kv_heads: int, head_dim: int, block: int, scale_dtype: int, device):
        self.capacity = capacity
        rb = _row_bytes(kind, n_kv_heads, head_dim)
        self.k = torch.zeros(capacity * rb, dtype=torch.uint8, device=device)
        self.v = torch.zeros(capacity * rb, dtype=torch.uint8, device=device)
        if kind != ffi.KV_BF16:
            sdt = torch.float16 if scale_dtype == ffi.SCALE_F16 else torch.float32
            n = capacity * n_kv_heads * (head_dim // block)
            self.ks = torch.zeros(n, dtype=sdt, device=device)
            self.vs = torch.zeros(n, dtype=sdt, device=device)
        else:
            self.ks = self.vs = None

    def tensors(self):
        return [t for t in (self.k, self.v, self.ks, self.vs) if t is not None]


class BlockPool:
    """Pre-allocated fixed-size pages with a LIFO free list and per-page owner tags (kv_cache.rs:515-680)."""

    def __init__(self, n_blocks: int, n_kv_heads: int, head_dim: int, device, kind: int = ffi.KV_BF16,
                 block: int = QUANT_BLOCKSIZE, scale_dtype: int = ffi.SCALE_F32, page_tokens: int = BLOCK_SIZE):
        self.kind, self.block, self.scale_dtype = int(kind), block, scale_dtype
        self.n_kv_heads, self.head_dim, self.page_tokens, self.device = n_kv_heads, head_dim, page_tokens, device
        # one K page and one V page per allocation unit would double the bookkeeping; a unit here is a
        # (K, V) pair, which keeps the reference's "balanced pair" invariant (kv_cache.rs:1460-1473) by construction
        self.store = _Storage(self.kind, n_blocks * page_tokens, n_kv_heads, head_dim, block, scale_dtype, device)
        self.free_list: List[int] = list(range(n_blocks - 1, -1, -1))
        self.owner: List[Optional[object]] = [None] * n_blocks
        self.n_blocks = n_blocks

    def allocate(self, owner) -> int:
        if not self.free_list:
            raise BlockPoolExhausted(f"block pool exhausted ({self.n_blocks} blocks in use)")
        bid = self.free_list.pop()
        self.owner[bid] = owner
        return bid

    def free(self, owner, bid: int) -> None:
        if self.owner[bid] != owner:
            raise RuntimeError(f"block {bid} is not owned by {owner!r}")
        self.owner[bid] = None
        self.free_list.append(bid)

    def num_free(self) -> int:
        return len(self.free_list)

    def page_ptrs(self, bid: int) -> Tuple[int, int, int, int]:
        rb = _row_bytes(self.kind, self.n_kv_heads, self.head_dim) * self.page_tokens
        k = self.store.k.data_ptr() + bid * rb
        v = self.store.v.data_ptr() + bid * rb
        if self.store.ks is None:
            return k, v, 0, 0
        sb = self.page_tokens * self.n_kv_heads * (self.head_dim // self.block) * self.store.ks.element_size()
        return k, v, self.store.ks.data_ptr() + bid * sb, self.store.vs.data_ptr() + bid * sb


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
        self.seq_pos = 0
        self.allocated_capacity = 0
        self.pool, self.owner = pool, owner
        self.blocks: List[int] = []
        self.store: Optional[_Storage] = None
        if pool is not None and (pool.kind != self.kind or pool.n_kv_heads != n_kv_heads or pool.head_dim != head_dim):
            raise ValueError("pool geometry does not match the cache")

    @classmethod
    def new_paged(cls, max_seq_len: int, pool: BlockPool, owner) -> "LayerKVCache":
        """kv_cache.rs:1111 `new_paged`; unlike the reference the pool may hold quantised pages."""
        return cls(max_seq_len, KVQuantType(pool.kind), pool.n_kv_heads, pool.head_dim, pool.device, pool.block,
                   pool.scale_dtype, pool=pool, owner=owner)

    # ---- capacity ---------------------------------------------------------------------------
    def _ensure_capacity(self, end_pos: int) -> None:
        if self.pool is not None:
            need = (end_pos + self.pool.page_tokens - 1) // self.pool.page_tokens
            got: List[int] = []
            try:
                while len(self.blocks) + len(got) < need:
                    got.append(self.pool.allocate(self.owner))
            except BlockPoolExhausted:
                for bid in got:  # roll back so nothing leaks (kv_cache.rs:1462-1470)
                    self.pool.free(self.owner, bid)
                raise
            self.blocks.extend(got)
            self.allocated_capacity = len(self.blocks) * self.pool.page_tokens
            return
        if end_pos <= self.allocated_capacity:
            return
        # grow in 1024-token chunks, capped at max_seq_len (kv_cache.rs:1146-1200)
        new_cap = min(self.max_seq_len, (end_pos + DEFAULT_CHUNK_SIZE - 1) // DEFAULT_CHUNK_SIZE * DEFAULT_CHUNK_SIZE)
        new = _Storage(self.kind, new_cap, self.n_kv_heads, self.head_dim, self.block, self.scale_dtype, self.device)
        if self.store is not None:
            for dst, src in zip(new.tensors(), self.store.tensors()):
                dst[: src.numel()].copy_(src)
        self.store = new
        self.allocated_capacity = new_cap

    # ---- view -------------------------------------------------------------------------------
    def page_rows(self) -> Tuple[int, List[Tuple[int, int, int, int]]]:
        """(page_tokens, [(k, v, k_scale, v_scale) device pointers per page])."""
        if self.pool is not None:
            return self.pool.page_tokens, [self.pool.page_ptrs(b) for b in self.blocks]
        if self.store is None:
            return max(self.allocated_capacity, 1), []
        s = self.store
        return s.capacity, [(s.k.data_ptr(), s.v.data_ptr(), 0 if s.ks is None else s.ks.data_ptr(),
                             0 if s.vs is None else s.vs.data_ptr())]

    # ---- reference API -----------------------------------------------------------------------
    def update(self, new_keys: torch.Tensor, new_values: torch.Tensor, start_pos: int) -> None:
        """Append [1, T, Hkv, D] bf16 keys/values at `start_pos` (kv_cache.rs:1275-1496)."""
        if new_keys.dim() != 4:
            raise ValueError(f"Expected 4D tensor for keys, got {list(new_keys.shape)}")
        seq_len = new_keys.shape[1]
        end_pos = start_pos + seq_len
        if end_pos > self.max_seq_len:
            raise ValueError(f"Cache overflow: trying to cache {seq_len} tokens starting at position {start_pos}, "
                             f"but max_seq_len is {self.max_seq_len}")
        self._ensure_capacity(end_pos)
        view, keep = make_view([self])
        dst = torch.tensor([start_pos], dtype=torch.int32, device=self.device)
        ops.kv_quantize_write(view, new_keys.contiguous(), new_values.contiguous(), dst)
        del keep
        self.seq_pos = end_pos

    def get(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """Keys/values [1, seq_pos, Hkv, D] bf16, dequantised if need be (kv_cache.rs:1499-1643)."""
        if self.seq_pos == 0:
            raise ValueError("Cache is empty")
        view, keep = make_view([self])
        lens = torch.tensor([self.seq_pos], dtype=torch.int32, device=self.device)
        k, v = ops.kv_gather_dequantize(view, lens, self.seq_pos)
        del keep
        return k, v

    def clear(self) -> None:
        """kv_cache.rs:1646-1705: drop contents, return pages to the pool."""
        self.seq_pos = 0
        if self.pool is not None:
            for bid in self.blocks:
                self.pool.free(self.owner, bid)
            self.blocks = []
            self.allocated_capacity = 0

    def truncate_to(self, n: int) -> None:
        """kv_cache.rs:1707-1750; token-granular for every storage kind."""
        if n >= self.seq_pos:
            return
        self.seq_pos = n
        if self.pool is not None:
            keep = (n + self.pool.page_tokens - 1) // self.pool.page_tokens
            for bid in self.blocks[keep:]:
                self.pool.free(self.owner, bid)
            self.blocks = self.blocks[:keep]
            self.allocated_capacity = keep * self.pool.page_tokens

    def memory_usage(self) -> int:
        """Bytes held (cf. QuantizedTensor::memory_usage, kv_cache.rs:960-962)."""
        if self.pool is not None:
            rb = _row_bytes(self.kind, self.n_kv_heads, self.head_dim)
            per = 2 * rb * self.pool.page_tokens
            if self.kind != ffi.KV_BF16:
                per += 2 * self.pool.page_tokens * self.n_kv_heads * (self.head_dim // self.block) * (2 if self.scale_dtype else 4)
            return per * len(self.blocks)
        return 0 if self.store is None else sum(t.numel() * t.element_size() for t in self.store.tensors())

    def __del__(self):
        try:
            if self.pool is not None and self.blocks:
                self.clear()  # pages go back to the pool on drop (kv_cache.rs:1889-1898)
        except Exception:
            pass


def make_view(caches: Sequence[LayerKVCache]) -> Tuple[KVView, list]:
    """Builds one hs_kv_view over the caches of a batch (one sequence each).

    Returns (view, keepalive): the page-pointer tables are device tensors that must outlive the launches."""
    c0 = caches[0]
    rows = [c.page_rows() for c in caches]
    page_tokens = {pt for pt, _ in rows}
    if c0.pool is None:
        # contiguous caches of different capacities: cut each into pages of gcd(capacities) tokens
        pt = 0
        for cap in page_tokens:
            pt = math.gcd(pt, cap)
        rb = _row_bytes(c0.kind, c0.n_kv_heads, c0.head_dim)
        sb = c0.n_kv_heads * (c0.head_dim // c0.block) * (2 if c0.scale_dtype == ffi.SCALE_F16 else 4)
        cut = []
        for cap, pages in rows:
            ptrs = []
            for (k, v, ks, vs) in pages:
                for j in range(cap // pt):
                    ptrs.append((k + j * pt * rb, v + j * pt * rb, ks + j * pt * sb if ks else 0, vs + j * pt * sb if vs else 0))
            cut.append((pt, ptrs))
        rows = cut
        pps = max(1, max(len(p) for _, p in rows))
    else:
        if len(page_tokens) != 1:
            raise ValueError("paged caches of one batch must share a page size")
        pt = page_tokens.pop()
        pps = max(1, max(len(p) for _, p in rows))
    table = torch.zeros(4, len(caches), pps, dtype=torch.int64)
    for i, (_, pages) in enumerate(rows):
        for j, ptrs in enumerate(pages):
            for a in range(4):
                table[a, i, j] = ptrs[a]
    dev_table = table.to(c0.device, non_blocking=False)
    view = KVView(kind=c0.kind, scale_dtype=c0.scale_dtype, block=c0.block, n_kv_heads=c0.n_kv_heads,
                  head_dim=c0.head_dim, page_tokens=pt, pages_per_seq=pps, reserved=0,
                  k_pages=dev_table[0].data_ptr(), v_pages=dev_table[1].data_ptr(),
                  k_scale_pages=dev_table[2].data_ptr() if c0.kind != ffi.KV_BF16 else None,
                  v_scale_pages=dev_table[3].data_ptr() if c0.kind != ffi.KV_BF16 else None)
    return view, [dev_table]
