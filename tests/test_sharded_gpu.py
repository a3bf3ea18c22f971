"""GPU tests of hs_attn_decode_sharded: KV-length shards exchanged inside the decode kernel (one launch per rank).

On one GPU the ranks of a shard group cannot run at the same time (kernels that wait for one another must not be
separate launches on one device), so the "virtual ranks" here run one after the other: all but the last deliver their
part without waiting (HS_SHARD_PUSH_ONLY), the last one finds every part in its inbox, waits for nothing and merges.
The arithmetic, the inbox layout, the epoch / half alternation and the flags are the ones the multi-GPU path uses;
only the overlap in time is missing, and that is measured by bench.py on real GPUs.

The time-out test makes a bounded wait run out on purpose (a part that nobody delivers, a limit of 30 ms): the kernel
records HS_DEVERR_WAIT_TIMEOUT and returns, and the next step on the same context succeeds.
"""
import ctypes
import math

import pytest
import torch

from tests.util import no_device_error

pytestmark = pytest.mark.gpu


def _make(cuda, kind, block, sdt, hq, hkv, d, lens, world, seed):
    """Full caches and per-rank shard caches of the same K/V streams."""
    from hyprstream_b200 import kv_cache as kc, sharded

    g = torch.Generator(device=cuda).manual_seed(seed)
    full, shards = [], [[] for _ in range(world)]
    local_lens = [[] for _ in range(world)]
    for l in lens:
        k = torch.randn(1, l, hkv, d, device=cuda, generator=g).bfloat16()
        v = torch.randn(1, l, hkv, d, device=cuda, generator=g).bfloat16()
        c = kc.LayerKVCache(1 << 20, kc.KVQuantType(kind), hkv, d, cuda, block=block, scale_dtype=sdt)
        c.update(k, v, 0)
        full.append(c)
        for r, (a, b) in enumerate(sharded.shard_bounds(l, world)):
            s = kc.LayerKVCache(1 << 20, kc.KVQuantType(kind), hkv, d, cuda, block=block, scale_dtype=sdt)
            if b > a:
                s.update(k[:, a:b].contiguous(), v[:, a:b].contiguous(), 0)
            else:
                s._ensure_capacity(32)  # an empty shard still needs storage for its view
            shards[r].append(s)
            local_lens[r].append(b - a)
    return full, shards, local_lens


class _Groups:
    def __init__(self, cuda, world, n_seqs, hq, d):
        from hyprstream_b200 import ffi

        self.ffi, self.world = ffi, world
        self.h = []
        for r in range(world):
            h = ctypes.c_void_p()
            ffi.check(ffi.lib.hs_shard_group_create(r, world, n_seqs, hq, d, ctypes.byref(h)))
            self.h.append(h)
        arr = (ctypes.c_void_p * world)(*self.h)
        ffi.check(ffi.lib.hs_shard_group_connect_local(arr, world))

    def call(self, r, q, view, lens_t, out, ws, flags, gate=None):
        n, hq, d = q.shape
        return self.ffi.lib.hs_attn_decode_sharded(self.h[r], q.data_ptr(), ctypes.byref(view), lens_t.data_ptr(), n, hq, 1.0 / math.sqrt(d),
                                                   None if out is None else out.data_ptr(), None if gate is None else gate.data_ptr(),
                                                   ws.data_ptr(), ws.numel(), flags, torch.cuda.current_stream().cuda_stream)

    def close(self):
        for h in self.h:
            self.ffi.lib.hs_shard_group_destroy(h)
        self.h = []


@pytest.mark.parametrize("world", [3, 8])
@pytest.mark.parametrize("kind,block,sdt,hq,hkv,d", [(2, 64, 1, 32, 8, 128), (1, 128, 1, 32, 8, 128), (1, 64, 0, 16, 2, 256)])
def test_virtual_ranks_merge_to_unsplit(cuda, kind, block, sdt, hq, hkv, d, world):
    from hyprstream_b200 import ffi, kv_cache as kc, ops

    lens = [3000, 100, 2048, 5000]  # 100 tokens: one page, so the later ranks hold empty shards of that sequence
    full, shards, local_lens = _make(cuda, kind, block, sdt, hq, hkv, d, lens, world, seed=31)
    fview, fkeep = kc.make_view(full)
    views = [kc.make_view(s) for s in shards]
    lens_t = [torch.tensor(l, dtype=torch.int32, device=cuda) for l in local_lens]
    full_t = torch.tensor(lens, dtype=torch.int32, device=cuda)
    ws = ops.decode_workspace(len(lens), hq, d, cuda)
    grp = _Groups(cuda, world, len(lens), hq, d)
    try:
        for step, last in enumerate((world - 1, 0, 1, world - 1)):  # both inbox halves twice, a different rank finishing each time
            q = torch.randn(len(lens), hq, d, generator=torch.Generator().manual_seed(50 + step)).bfloat16().to(cuda)
            gate = torch.randn(len(lens), hq, d, generator=torch.Generator().manual_seed(70 + step)).bfloat16().to(cuda) if step == 1 else None
            ref = ops.decode_attention(q, fview, full_t, gate=gate)
            n0 = ffi.launch_count()
            for r in range(world):
                if r != last:
                    assert grp.call(r, q, views[r][0], lens_t[r], None, ws, ffi.SHARD_PUSH_ONLY) == 0, ffi.last_error()
            out = torch.full((len(lens), hq, d), float("nan"), dtype=torch.bfloat16, device=cuda)
            assert grp.call(last, q, views[last][0], lens_t[last], out, ws, 0, gate=gate) == 0, ffi.last_error()
            torch.cuda.synchronize()
            assert ffi.launch_count() - n0 == world  # one launch per rank and step
            assert torch.isfinite(out.float()).all()
            # merged shards == unsplit decode: 1e-3 on the fp32 result, plus half a bf16 step of the output rounding
            diff = (out.float() - ref.float()).abs()
            assert diff.max().item() <= 1e-3 + 0.004 * max(1.0, ref.float().abs().max().item()), (step, diff.max().item())
            # and == the three-call form (shard results, merge kernel) on the same shards
            parts = [ops.decode_attention(q, views[r][0], lens_t[r], shard=True) for r in range(world)]
            three = ops.merge_partials(torch.stack([p[0] for p in parts]), torch.stack([p[1] for p in parts]), gate=gate)
            assert (out.float() - three.float()).abs().max().item() <= 0.004 * max(1.0, ref.float().abs().max().item())
        assert ffi.lib.hs_shard_group_epoch(grp.h[0]) == 4
    finally:
        torch.cuda.synchronize()
        grp.close()
    no_device_error()


def test_missing_rank_times_out_and_the_next_step_succeeds(cuda):
    from hyprstream_b200 import ffi, kv_cache as kc, ops

    world, lens, hq, hkv, d = 3, [1500, 700], 32, 8, 128
    full, shards, local_lens = _make(cuda, 1, 128, 1, hq, hkv, d, lens, world, seed=33)
    fview, fkeep = kc.make_view(full)
    views = [kc.make_view(s) for s in shards]
    lens_t = [torch.tensor(l, dtype=torch.int32, device=cuda) for l in local_lens]
    ws = ops.decode_workspace(len(lens), hq, d, cuda)
    grp = _Groups(cuda, world, len(lens), hq, d)
    try:
        ffi.check(ffi.lib.hs_shard_group_set_wait_ms(grp.h[2], 30))
        q = torch.randn(len(lens), hq, d, generator=torch.Generator().manual_seed(5)).bfloat16().to(cuda)
        out = torch.zeros(len(lens), hq, d, dtype=torch.bfloat16, device=cuda)
        # step 1: rank 1 never delivers; rank 2's bounded wait runs out
        assert grp.call(0, q, views[0][0], lens_t[0], None, ws, ffi.SHARD_PUSH_ONLY) == 0
        assert grp.call(2, q, views[2][0], lens_t[2], out, ws, 0) == 0  # the launch itself is fine
        torch.cuda.synchronize()
        assert ffi.take_device_error() == ffi.DEVERR_WAIT_TIMEOUT
        assert torch.equal(out, torch.zeros_like(out))  # rows whose parts did not arrive are left unwritten
        # the straggler delivers step 1 late (every rank counts the same steps), then step 2 runs normally
        assert grp.call(1, q, views[1][0], lens_t[1], None, ws, ffi.SHARD_PUSH_ONLY) == 0
        q2 = torch.randn(len(lens), hq, d, generator=torch.Generator().manual_seed(6)).bfloat16().to(cuda)
        for r in (0, 1):
            assert grp.call(r, q2, views[r][0], lens_t[r], None, ws, ffi.SHARD_PUSH_ONLY) == 0
        assert grp.call(2, q2, views[2][0], lens_t[2], out, ws, 0) == 0
        torch.cuda.synchronize()
        ref = ops.decode_attention(q2, fview, torch.tensor(lens, dtype=torch.int32, device=cuda))
        assert (out.float() - ref.float()).abs().max().item() <= 1e-3 + 0.004 * max(1.0, ref.float().abs().max().item())
    finally:
        torch.cuda.synchronize()
        grp.close()
    no_device_error()


def test_sharded_entry_refuses_what_it_cannot_serve(cuda):
    from hyprstream_b200 import ffi, kv_cache as kc, ops

    lib = ffi.lib
    h = ctypes.c_void_p()
    assert lib.hs_shard_group_create(0, 9, 4, 32, 128, ctypes.byref(h)) == ffi.HS_ERR_ARG  # more ranks than a node has GPUs
    assert lib.hs_shard_group_create(2, 2, 4, 32, 128, ctypes.byref(h)) == ffi.HS_ERR_ARG
    ffi.check(lib.hs_shard_group_create(0, 2, 2, 32, 128, ctypes.byref(h)))
    c = kc.LayerKVCache(4096, kc.KVQuantType.INT8, 8, 128, cuda)
    c.update(torch.randn(1, 64, 8, 128).bfloat16().to(cuda), torch.randn(1, 64, 8, 128).bfloat16().to(cuda), 0)
    view, keep = kc.make_view([c])
    q = torch.randn(1, 32, 128).bfloat16().to(cuda)
    out = torch.empty_like(q)
    sl = torch.tensor([64], dtype=torch.int32, device=cuda)
    ws = ops.decode_workspace(1, 32, 128, cuda)
    args = (q.data_ptr(), ctypes.byref(view), sl.data_ptr(), 1, 32, 0.1, out.data_ptr(), None, ws.data_ptr(), ws.numel(), 0, None)
    assert lib.hs_attn_decode_sharded(h, *args) == ffi.HS_ERR_ARG and "not connected" in ffi.last_error()
    lib.hs_shard_group_destroy(h)
    # a one-rank group is connected from the start and equals the plain decode
    ffi.check(lib.hs_shard_group_create(0, 1, 2, 32, 128, ctypes.byref(h)))
    assert lib.hs_attn_decode_sharded(h, *args) == 0, ffi.last_error()
    torch.cuda.synchronize()
    assert (out.float() - ops.decode_attention(q, view, sl, softmax_scale=0.1).float()).abs().max().item() <= 0.004
    # a shape the group was not sized for; a cache kind the tensor-core kernel does not serve
    big = (q.data_ptr(), ctypes.byref(view), sl.data_ptr(), 3, 32, 0.1, out.data_ptr(), None, ws.data_ptr(), ws.numel(), 0, None)
    assert lib.hs_attn_decode_sharded(h, *big) == ffi.HS_ERR_ARG
    cb = kc.LayerKVCache(4096, kc.KVQuantType.NONE, 8, 128, cuda)
    cb.update(torch.randn(1, 64, 8, 128).bfloat16().to(cuda), torch.randn(1, 64, 8, 128).bfloat16().to(cuda), 0)
    vb, kb = kc.make_view([cb])
    bf = (q.data_ptr(), ctypes.byref(vb), sl.data_ptr(), 1, 32, 0.1, out.data_ptr(), None, ws.data_ptr(), ws.numel(), 0, None)
    e0 = lib.hs_shard_group_epoch(h)
    assert lib.hs_attn_decode_sharded(h, *bf) == ffi.HS_ERR_UNSUPPORTED
    assert lib.hs_shard_group_epoch(h) == e0  # a refused call does not count as a step
    lib.hs_shard_group_destroy(h)
    torch.cuda.synchronize()
    no_device_error()
