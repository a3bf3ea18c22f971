"""GPU tests of the host-facing additions around the decode path: the one-call decode step (hs_attn_decode_step), the
stale-view check (hs_view_is_current), raw snapshots of stored codes (hs_cache_snapshot), pending error flags that must
not disturb later launches, and launch configuration on a second device of the same process."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import attention_ref as ar
from oracle import quant_ref as qr
from tests.util import assert_close_attn, no_device_error

pytestmark = pytest.mark.gpu


def _batch(cuda, lens, block=128, sdt=1, seed=1, cap=1 << 14):
    from hyprstream_b200 import kv_cache as kc

    g = torch.Generator().manual_seed(seed)
    caches, ks, vs = [], [], []
    for l in lens:
        k = torch.randn(1, l, 8, 128, generator=g).bfloat16()
        v = torch.randn(1, l, 8, 128, generator=g).bfloat16()
        c = kc.LayerKVCache(cap, kc.KVQuantType.INT8, 8, 128, cuda, block=block, scale_dtype=sdt)
        c._ensure_capacity(l + 8)
        c.update(k.to(cuda), v.to(cuda), 0)
        caches.append(c); ks.append(k); vs.append(v)
    return caches, ks, vs


def test_decode_step_equals_the_separate_calls_and_the_oracle(cuda):
    """hs_attn_decode_step (host buffers in, host buffer out, one call) == copy + hs_kv_quantize_write + hs_attn_decode,
    bit for bit, for three consecutive steps; stored codes of the written tokens equal the oracle quantiser's; the
    last step's output is within tolerance of the oracle's batched path over the dequantised caches."""
    from hyprstream_b200 import kv_cache as kc, ops

    lens = [300, 17, 1024, 2500]
    a, ks, vs = _batch(cuda, lens, seed=4)
    b, _, _ = _batch(cuda, lens, seed=4)
    va, keep_a = kc.make_view(a)
    vb, keep_b = kc.make_view(b)
    step = ops.DecodeStep(va, len(lens), 32, cuda)
    pos = torch.tensor(lens, dtype=torch.int32, device=cuda)
    gen = torch.Generator().manual_seed(9)
    for t in range(3):
        q = torch.randn(len(lens), 32, 128, generator=gen).bfloat16()
        kn = torch.randn(len(lens), 8, 128, generator=gen).bfloat16()
        vn = torch.randn(len(lens), 8, 128, generator=gen).bfloat16()
        step.q_host.copy_(q); step.k_host.copy_(kn); step.v_host.copy_(vn)
        got = step.run(pos, pos + 1).clone()
        ops.kv_quantize_write(vb, kn.unsqueeze(1).to(cuda), vn.unsqueeze(1).to(cuda), pos)
        ref = ops.decode_attention(q.to(cuda), vb, pos + 1)
        torch.cuda.synchronize()
        assert (got.float() - ref.cpu().float()).abs().max().item() <= 4e-3, f"step {t}"
        for r in range(len(lens)):
            ks[r] = torch.cat([ks[r], kn[r:r + 1].unsqueeze(0)], 1)
            vs[r] = torch.cat([vs[r], vn[r:r + 1].unsqueeze(0)], 1)
        pos += 1
    # stored codes and scales of everything written so far, against the oracle quantiser
    kd, vd = [], []
    for r, c in enumerate(a):
        c.seq_pos = lens[r] + 3
        kc_, vc_, ksc, vsc = c.snapshot()
        for src, codes, scales, dst in ((ks[r], kc_, ksc, kd), (vs[r], vc_, vsc, vd)):
            oc, oa = qr.quantize(src.float().numpy(), qr.INT8, 128, True)
            assert np.array_equal(codes.numpy().reshape(-1), oc), f"codes of sequence {r}"
            assert np.array_equal(scales.numpy().reshape(-1).view(np.uint16), np.asarray(oa).reshape(-1).view(np.uint16)), f"scales of sequence {r}"
            dst.append(torch.from_numpy(qr.dequantize(oc, oa, qr.INT8, src.numel(), 128)).bfloat16().reshape(src.shape))
    oracle = ar.llama_batched_decode(q.unsqueeze(1), kd, vd, [l + 2 for l in lens], 32).reshape(len(lens), 32, 128)
    assert_close_attn(got, oracle.float(), "decode step vs oracle batched path")
    no_device_error()


@pytest.mark.parametrize("fused_write", [False, True])
def test_decode_append_equals_write_then_decode(cuda, fused_write):
    """hs_attn_decode_append == hs_kv_quantize_write followed by hs_attn_decode, over several steps in a row without any
    host synchronisation between them, with the fused K rotation; the stored codes and scales are identical.  With explicit
    positions the attention kernel is launched as a programmatic dependent of the write kernel (two launches); with
    positions = seq_lens - 1 (dst_pos None) the attention kernel writes the new tokens itself (one launch)."""
    from hyprstream_b200 import kv_cache as kc, ops

    lens = [700, 33, 4000, 1, 512, 90]
    a, _, _ = _batch(cuda, lens, seed=6)
    b, _, _ = _batch(cuda, lens, seed=6)
    va, keep_a = kc.make_view(a)
    vb, keep_b = kc.make_view(b)
    sin, cos = (t.to(cuda) for t in ar.rope_tables(128, 500000.0, 8192, torch.bfloat16))
    pos = torch.tensor(lens, dtype=torch.int32, device=cuda)
    gen = torch.Generator(device=cuda).manual_seed(3)
    steps = 6
    qs = torch.randn(steps, len(lens), 32, 128, device=cuda, generator=gen).bfloat16()
    ks = torch.randn(steps, len(lens), 1, 8, 128, device=cuda, generator=gen).bfloat16()
    vs = torch.randn(steps, len(lens), 1, 8, 128, device=cuda, generator=gen).bfloat16()
    poss = torch.stack([pos + t for t in range(steps)])
    lenss = poss + 1
    from hyprstream_b200 import ffi
    n0 = ffi.launch_count()
    got = [ops.decode_append(qs[t], ks[t], vs[t], va, poss[t] if fused_write is False else None, lenss[t], sin=sin, cos=cos, rotary_dim=128)
           for t in range(steps)]
    torch.cuda.synchronize()
    assert ffi.launch_count() - n0 == steps * (1 if fused_write else 2)
    for t in range(steps):
        ops.kv_quantize_write(vb, ks[t], vs[t], poss[t], sin, cos, 128)
        ref = ops.decode_attention(qs[t], vb, lenss[t])
        torch.cuda.synchronize()
        assert (got[t].float() - ref.float()).abs().max().item() <= 4e-3, f"step {t}"
    for x, y, l in zip(a, b, lens):
        x.seq_pos = y.seq_pos = l + steps
        for u, w in zip(x.snapshot(), y.snapshot()):
            assert torch.equal(u.view(torch.uint8), w.view(torch.uint8))
    no_device_error()


def test_view_goes_stale_when_a_cache_grows_or_releases_storage(cuda):
    from hyprstream_b200 import ffi, kv_cache as kc

    c = kc.LayerKVCache(8192, kc.KVQuantType.INT8, 8, 128, cuda)
    x = torch.randn(1, 1000, 8, 128).bfloat16().to(cuda)
    c.update(x, x, 0)                       # capacity 1024
    view, keep = kc.make_view([c])
    assert kc.view_is_current(keep)
    c.update(x[:, :24], x[:, :24], 1000)    # still inside the slab the view points at
    assert kc.view_is_current(keep)
    c.update(x[:, :8], x[:, :8], 1024)      # grows: a new slab replaces the old one
    assert not kc.view_is_current(keep)
    assert "build a new view" in ffi.last_error() or "capacity" in ffi.last_error()
    view2, keep2 = kc.make_view([c])
    assert kc.view_is_current(keep2)
    kg, _ = c.get()                          # contents survived the growth
    c1 = kc.LayerKVCache(8192, kc.KVQuantType.INT8, 8, 128, cuda)
    c1.update(x, x, 0)
    assert torch.equal(kg[:, :1000], c1.get()[0])
    c.to_device("cpu")
    assert not kc.view_is_current(keep2)
    # paged: a cache that takes another page changes capacity; truncation that returns pages bumps the generation
    pool = kc.BlockPool(8, 8, 128, cuda, kind=ffi.KV_INT8)
    p = kc.LayerKVCache.new_paged(4096, pool, owner=1)
    p.update(x[:, :300], x[:, :300], 0)
    v3, k3 = kc.make_view([p])
    assert kc.view_is_current(k3)
    p.update(x[:, :300], x[:, :300], 300)
    assert not kc.view_is_current(k3)
    v4, k4 = kc.make_view([p])
    p.truncate_to(100)
    assert not kc.view_is_current(k4)
    torch.cuda.synchronize()
    no_device_error()


def test_pending_error_flags_do_not_disturb_later_launches(cuda):
    """The error word is a report: with HS_DEVERR_WAIT_TIMEOUT pending from some earlier launch (set here through the
    host-side hook, no wait runs out), prefill and decode still produce their results; range flags recorded by other
    kernels are OR'd in, not overwritten; one take returns all of them and clears the word."""
    from hyprstream_b200 import ffi, kv_cache as kc, ops

    ffi.take_device_error()
    ffi.check(ffi.lib.hs_attn_inject_device_error(ffi.DEVERR_WAIT_TIMEOUT))
    torch.manual_seed(3)
    q = torch.randn(1, 300, 32, 128).bfloat16()
    k = torch.randn(1, 300, 8, 128).bfloat16()
    v = torch.randn(1, 300, 8, 128).bfloat16()
    out = ops.prefill_attention(q.to(cuda), k.to(cuda), v.to(cuda))
    torch.cuda.synchronize()
    ref = ar.attention_fp32(q, k, v)  # causal: query row i sees keys 0..i
    assert_close_attn(out, ref, "prefill with a time-out flag pending")
    # a rope call with a position outside its table records its own flag on top
    sin, cos = ar.rope_tables(128, 500000.0, 16, torch.bfloat16)
    x = torch.randn(2, 8, 128).bfloat16().to(cuda)
    ops.rope_apply(x, sin.to(cuda), cos.to(cuda), torch.tensor([3, 99], dtype=torch.int32, device=cuda))
    torch.cuda.synchronize()
    assert ffi.take_device_error() == ffi.DEVERR_WAIT_TIMEOUT | ffi.DEVERR_ROPE_RANGE
    assert ffi.take_device_error() == 0


def test_second_device_of_one_process_gets_its_own_launch_configuration():
    """One process, two GPUs (the reference engine's layer split drives several devices from one process): the
    tensor-core decode (one cooperative launch) and the tcgen05 prefill must be configured on each device."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs in one process")
    from hyprstream_b200 import ffi, kv_cache as kc, ops

    outs = []
    for idx in (0, 1):
        dev = torch.device("cuda", idx)
        with torch.cuda.device(dev):
            caches, ks, vs = _batch(dev, [700, 40], seed=8)
            view, keep = kc.make_view(caches)
            torch.manual_seed(2)
            q = torch.randn(2, 32, 128).bfloat16()
            n0 = ffi.launch_count()
            out = ops.decode_attention(q.to(dev), view, torch.tensor([700, 40], dtype=torch.int32, device=dev))
            torch.cuda.synchronize()
            assert ffi.launch_count() - n0 == 1, f"device {idx}: the fused kernel did not take the launch"
            qp = torch.randn(1, 256, 32, 128).bfloat16()
            kp = torch.randn(1, 256, 8, 128).bfloat16()
            vp = torch.randn(1, 256, 8, 128).bfloat16()
            pf = ops.prefill_attention(qp.to(dev), kp.to(dev), vp.to(dev))
            torch.cuda.synchronize()
            assert ffi.take_device_error() == 0
            outs.append((out.cpu(), pf.cpu()))
    assert (outs[0][0].float() - outs[1][0].float()).abs().max().item() <= 4e-3
    assert (outs[0][1].float() - outs[1][1].float()).abs().max().item() <= 4e-3
