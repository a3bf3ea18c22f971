"""Python face of the continuous-batching scheduler (hyprstream_b200/csrc/scheduler.cu, `hs_sched_*` in
include/hs_attn.h): the loop around the batched decode step that the reference leaves open
(crates/hyprstream/src/runtime/torch_engine.rs:1475-1501; config/mod.rs:2146-2152; kv_cache.rs:482-505).  Forwarder only.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Sequence

from . import ffi
from .ffi import lib

DEFAULT_CONTINUOUS_BATCH_MAX = 16  # config/mod.rs:2175-2177


@dataclass
class StepPlan:
    prefill_ids: List[int]
    prefill_lens: List[int]
    prefill_caches: List[int]          # hs_cache handles (addresses)
    decode_ids: List[int]
    decode_caches: List[int]
    host_dst_pos: List[int]
    view: Optional[ffi.KVView]         # device objects: None without them or with an empty decode batch
    dst_pos: Optional[int]             # device pointers (int32 [n_decode])
    seq_lens: Optional[int]
    n_deferred: int
    n_stalled: int
    n_waiting: int
    n_running: int


class Scheduler:
    """Admission (FIFO, deferred when the pool has no pages for the prompt), decode-batch planning, retirement."""

    def __init__(self, pool_handle, continuous_batch_max: int = DEFAULT_CONTINUOUS_BATCH_MAX, max_seq_len: int = 8192):
        self._h = ctypes.c_void_p()
        self._pool = pool_handle  # keeps the pool alive
        handle = pool_handle._h if hasattr(pool_handle, "_h") else pool_handle
        ffi.check(lib.hs_sched_create(handle, continuous_batch_max, max_seq_len, ctypes.byref(self._h)))

    def submit(self, seq_id: int, prompt_len: int, max_new_tokens: int) -> None:
        ffi.check(lib.hs_sched_submit(self._h, seq_id, prompt_len, max_new_tokens))

    def plan_step(self, device_objects: bool = True, stream: int = 0) -> StepPlan:
        p = ffi.SchedPlan()
        st = lib.hs_sched_plan_step(self._h, ffi.SCHED_DEVICE_OBJECTS if device_objects else 0, ctypes.byref(p), stream)
        if st == ffi.HS_ERR_POOL_EXHAUSTED:
            from .kv_cache import BlockPoolExhausted

            raise BlockPoolExhausted(ffi.last_error())
        ffi.check(st)
        view = ffi.KVView.from_address(p.view) if p.view else None
        return StepPlan([p.prefill_ids[i] for i in range(p.n_prefill)], [p.prefill_lens[i] for i in range(p.n_prefill)],
                        [p.prefill_caches[i] for i in range(p.n_prefill)], [p.decode_ids[i] for i in range(p.n_decode)],
                        [p.decode_caches[i] for i in range(p.n_decode)], [p.host_dst_pos[i] for i in range(p.n_decode)], view,
                        p.dst_pos or None, p.seq_lens or None, p.n_deferred, p.n_stalled, p.n_waiting, p.n_running)

    def commit_step(self, finished: Sequence[int] = ()) -> None:
        arr = (ctypes.c_int64 * max(len(finished), 1))(*finished)
        ffi.check(lib.hs_sched_commit_step(self._h, arr, len(finished)))

    def cancel(self, seq_id: int) -> None:
        ffi.check(lib.hs_sched_cancel(self._h, seq_id))

    def stats(self) -> ffi.SchedStats:
        s = ffi.SchedStats()
        ffi.check(lib.hs_sched_stats(self._h, ctypes.byref(s)))
        return s

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None:
            lib.hs_sched_destroy(self._h)
            self._h = None
