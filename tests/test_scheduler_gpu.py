"""GPU test of the continuous-batching scheduler driving the real batched decode step: sequences are admitted while the
pool has pages, one is deferred and gets in after another retires, every step decodes the planned batch through the
plan's cache view and position arrays, and every token of every sequence equals what that sequence produces when it is
decoded alone (batched == serial, the property of architectures/llama.rs:3658-3711)."""
import ctypes

import pytest
import torch

from tests.util import no_device_error

pytestmark = pytest.mark.gpu

HQ, HKV, D = 32, 8, 128


def _kv(seq, what, n, start):
    """Deterministic K/V/q streams per sequence: token t of sequence `seq` is the same whoever asks for it."""
    rows = []
    for t in range(start, start + n):
        g = torch.Generator().manual_seed(seq * 100003 + t * 7 + {"k": 0, "v": 1, "q": 2}[what])
        rows.append(torch.randn(HQ if what == "q" else HKV, D, generator=g))
    return torch.stack(rows).bfloat16()


def test_scheduler_drives_batched_decode_equal_to_serial(cuda):
    from hyprstream_b200 import ffi, kv_cache as kc, ops
    from hyprstream_b200.scheduler import Scheduler

    pool = kc.BlockPool(8, HKV, D, cuda, kind=ffi.KV_INT8, block=128, scale_dtype=ffi.SCALE_F16)
    sched = Scheduler(pool, continuous_batch_max=4, max_seq_len=2048)
    prompts = {0: 300, 1: 520, 2: 100, 3: 700, 4: 260}
    budget = {0: 4, 1: 6, 2: 3, 3: 3, 4: 3}
    for sid in prompts:
        sched.submit(sid, prompts[sid], budget[sid])
    outs = {sid: [] for sid in prompts}
    ws = ops.decode_workspace(4, HQ, D, cuda)
    stream = torch.cuda.current_stream().cuda_stream
    saw_deferred, max_batch, steps = 0, 0, 0
    while True:
        st = sched.stats()
        if st.n_running == 0 and st.n_waiting == 0:
            break
        plan = sched.plan_step(device_objects=True, stream=stream)
        saw_deferred += plan.n_deferred
        for sid, n, cache in zip(plan.prefill_ids, plan.prefill_lens, plan.prefill_caches):  # prompts of the newly admitted
            k, v = _kv(sid, "k", n, 0).unsqueeze(0).to(cuda), _kv(sid, "v", n, 0).unsqueeze(0).to(cuda)
            ffi.check(ffi.lib.hs_cache_update(cache, k.data_ptr(), v.data_ptr(), n, 0, None, None, 0, 0, stream))
        nd = len(plan.decode_ids)
        max_batch = max(max_batch, nd)
        if nd:
            pos = plan.host_dst_pos
            q = torch.stack([_kv(s, "q", 1, p)[0] for s, p in zip(plan.decode_ids, pos)]).to(cuda)
            kn = torch.stack([_kv(s, "k", 1, p) for s, p in zip(plan.decode_ids, pos)]).to(cuda)   # [nd, 1, Hkv, D]
            vn = torch.stack([_kv(s, "v", 1, p) for s, p in zip(plan.decode_ids, pos)]).to(cuda)
            out = torch.empty(nd, HQ, D, dtype=torch.bfloat16, device=cuda)
            ffi.check(ffi.lib.hs_kv_quantize_write(ctypes.byref(plan.view), kn.data_ptr(), vn.data_ptr(), nd, 1, plan.dst_pos, None, None, 0, 0, stream))
            ffi.check(ffi.lib.hs_attn_decode(q.data_ptr(), ctypes.byref(plan.view), plan.seq_lens, nd, HQ, D ** -0.5, out.data_ptr(), None,
                                             ws.data_ptr(), ws.numel(), None, None, stream))
            torch.cuda.synchronize()
            for i, sid in enumerate(plan.decode_ids):
                outs[sid].append(out[i].cpu())
        sched.commit_step()
        steps += 1
        assert steps < 100
    assert saw_deferred > 0 and max_batch >= 3
    st = sched.stats()
    assert st.n_retired == 5 and st.pages_free == 8
    # serial reference: each sequence alone, contiguous cache, one token at a time
    for sid in prompts:
        c = kc.LayerKVCache(2048, kc.KVQuantType.INT8, HKV, D, cuda, block=128, scale_dtype=ffi.SCALE_F16)
        n = prompts[sid]
        c.update(_kv(sid, "k", n, 0).unsqueeze(0).to(cuda), _kv(sid, "v", n, 0).unsqueeze(0).to(cuda), 0)
        assert len(outs[sid]) == budget[sid]
        for t in range(budget[sid]):
            p = n + t
            c.update(_kv(sid, "k", 1, p).unsqueeze(0).to(cuda), _kv(sid, "v", 1, p).unsqueeze(0).to(cuda), p)
            view, keep = kc.make_view([c])
            ref = ops.decode_attention(_kv(sid, "q", 1, p).to(cuda), view, torch.tensor([p + 1], dtype=torch.int32, device=cuda))
            torch.cuda.synchronize()
            assert (ref[0].cpu().float() - outs[sid][t].float()).abs().max().item() <= 8e-3, (sid, t)
    del sched
    no_device_error()
