"""CPU tests of the continuous-batching scheduler's host logic (hs_sched_*): FIFO admission, admission deferred on pool
exhaustion and retried once pages are released (kv_cache.rs:482-505), the decode batch in admission order, stalls,
retirement, the no-progress error.  The pool's storage comes from a host allocator installed through
hs_host_set_allocator (no GPU is touched: plans are asked for without device objects) and the "step" is a fake that
only decides which sequences end."""
import ctypes

import pytest

from hyprstream_b200 import ffi
from hyprstream_b200.ffi import lib

_libc = ctypes.CDLL(None)
_libc.malloc.restype = ctypes.c_void_p
_libc.malloc.argtypes = [ctypes.c_size_t]
_libc.free.argtypes = [ctypes.c_void_p]
ALLOC = ctypes.CFUNCTYPE(ctypes.c_void_p, ctypes.c_size_t)(lambda n: _libc.malloc(n))
FREE = ctypes.CFUNCTYPE(None, ctypes.c_void_p)(lambda p: _libc.free(p))


@pytest.fixture
def host_pool():
    """A pool of 8 pages of 16 tokens (int8, 2 kv heads x 64) in host memory."""
    ffi.check(lib.hs_host_set_allocator(ctypes.cast(ALLOC, ctypes.c_void_p), ctypes.cast(FREE, ctypes.c_void_p)))
    pool = ctypes.c_void_p()
    ffi.check(lib.hs_pool_create(8, 16, ffi.KV_INT8, 64, ffi.SCALE_F32, 2, 64, ctypes.byref(pool)))
    yield pool
    lib.hs_pool_destroy(pool)
    ffi.check(lib.hs_host_set_allocator(None, None))


def _plan(s):
    p = ffi.SchedPlan()
    st = lib.hs_sched_plan_step(s, 0, ctypes.byref(p), None)
    return st, p


def _ids(ptr, n):
    return [ptr[i] for i in range(n)]


def test_admission_defer_retry_and_retire(host_pool):
    s = ctypes.c_void_p()
    ffi.check(lib.hs_sched_create(host_pool, 4, 256, ctypes.byref(s)))
    # prompts of 40 tokens need 3 pages each (41 tokens with the first decode token): two fit into 8 pages, the third does not
    for sid in (10, 11, 12):
        ffi.check(lib.hs_sched_submit(s, sid, 40, 3 if sid != 11 else 50))
    assert lib.hs_sched_submit(s, 11, 5, 5) == ffi.HS_ERR_ARG          # queued already
    assert lib.hs_sched_submit(s, -1, 5, 5) == ffi.HS_ERR_ARG
    assert lib.hs_sched_submit(s, 13, 250, 10) == ffi.HS_ERR_CACHE_OVERFLOW
    st, p = _plan(s)
    assert st == 0 and _ids(p.prefill_ids, p.n_prefill) == [10, 11] and p.n_decode == 0
    assert p.n_deferred == 1 and p.n_waiting == 1 and p.n_running == 2   # 12 deferred: fail-soft, still queued
    assert lib.hs_pool_num_free(host_pool) == 2
    assert lib.hs_sched_plan_step(s, 0, ctypes.byref(p), None) == ffi.HS_ERR_ARG  # the plan must be committed first
    ffi.check(lib.hs_sched_commit_step(s, None, 0))
    # steps 2-4: both decode; 12 is deferred again each time; 10 finishes after 3 tokens
    for step in range(3):
        st, p = _plan(s)
        assert st == 0 and _ids(p.decode_ids, p.n_decode) == [10, 11] and p.n_prefill == 0 and p.n_deferred == 1
        assert _ids(p.host_dst_pos, 2) == [40 + step, 40 + step]
        ffi.check(lib.hs_sched_commit_step(s, None, 0))
    # 10 used its budget and was retired: its 3 pages are free and 12 gets in
    st, p = _plan(s)
    assert st == 0 and _ids(p.decode_ids, p.n_decode) == [11] and _ids(p.prefill_ids, p.n_prefill) == [12] and p.n_deferred == 0
    ffi.check(lib.hs_sched_commit_step(s, None, 0))
    st, p = _plan(s)
    assert _ids(p.decode_ids, p.n_decode) == [11, 12] and _ids(p.host_dst_pos, 2) == [44, 40]
    # the host ends 11 early (end-of-sequence)
    fin = (ctypes.c_int64 * 1)(11)
    ffi.check(lib.hs_sched_commit_step(s, fin, 1))
    stats = ffi.SchedStats()
    ffi.check(lib.hs_sched_stats(s, ctypes.byref(stats)))
    assert (stats.n_running, stats.n_waiting, stats.n_admitted, stats.n_retired) == (1, 0, 3, 2)
    assert stats.n_deferred == 4 and stats.pages_free == 8 - 3
    # run 12 to its end
    for _ in range(2):
        st, p = _plan(s)
        assert st == 0 and _ids(p.decode_ids, p.n_decode) == [12]
        ffi.check(lib.hs_sched_commit_step(s, None, 0))
    ffi.check(lib.hs_sched_stats(s, ctypes.byref(stats)))
    assert stats.n_running == 0 and stats.pages_free == 8
    lib.hs_sched_destroy(s)
    assert lib.hs_pool_num_free(host_pool) == 8


def test_batch_limit_stall_and_no_progress(host_pool):
    s = ctypes.c_void_p()
    ffi.check(lib.hs_sched_create(host_pool, 2, 256, ctypes.byref(s)))
    for sid in (1, 2, 3):
        ffi.check(lib.hs_sched_submit(s, sid, 15, 100))   # one page each (16 tokens with the first decode token)
    st, p = _plan(s)
    assert _ids(p.prefill_ids, p.n_prefill) == [1, 2] and p.n_deferred == 0 and p.n_waiting == 1  # the batch limit, not the pool
    ffi.check(lib.hs_sched_commit_step(s, None, 0))
    # both grow; each needs a second page at token 17, a third at 33, ...: 8 pages carry two sequences up to 64 tokens each
    steps = 0
    while True:
        st, p = _plan(s)
        if st != 0:
            break
        steps += 1
        assert p.n_prefill == 0
        ffi.check(lib.hs_sched_commit_step(s, None, 0))
        assert steps < 200
    # 1 and 2 hold 4 pages each (64 tokens); their next tokens need a page that does not exist: nothing can move
    assert st == ffi.HS_ERR_POOL_EXHAUSTED and "no sequence can make progress" in ffi.last_error()
    assert steps == 64 - 15
    # the host gives up on 1: its pages let 2 continue and 3 in
    st, p = _plan(s)
    assert st == ffi.HS_ERR_POOL_EXHAUSTED      # still stuck, and the failed plan left nothing to commit
    assert lib.hs_sched_commit_step(s, None, 0) == ffi.HS_ERR_ARG
    assert lib.hs_sched_cancel(s, 99) == ffi.HS_ERR_ARG
    ffi.check(lib.hs_sched_cancel(s, 1))
    st, p = _plan(s)
    assert st == 0 and _ids(p.decode_ids, p.n_decode) == [2] and _ids(p.prefill_ids, p.n_prefill) == [3]
    ffi.check(lib.hs_sched_commit_step(s, None, 0))
    ffi.check(lib.hs_sched_cancel(s, 3))
    ffi.check(lib.hs_sched_cancel(s, 2))
    assert lib.hs_pool_num_free(host_pool) == 8
    lib.hs_sched_destroy(s)
    assert lib.hs_pool_num_free(host_pool) == 8
