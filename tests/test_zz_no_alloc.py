"""GPU test of hs_attn_decode_static, the decode entry point that brings its own scratch.

It exists for hosts that cannot allocate device memory where they decode (inside a stream capture, under a
foreign allocator that owns the whole budget, or where a device-wide synchronisation is not acceptable), so
this test hands it nothing but inputs and a preallocated output, straight through the C ABI, and compares
with hs_attn_decode given an ordinary workspace.  The file name keeps it last in collection order; it must
pass both alone in a fresh process (its first call then performs the per-device address look-up) and after
every other test.
"""
import ctypes

import pytest
import torch

from tests.util import MAX_ABS_TOL, MEAN_ABS_TOL

pytestmark = pytest.mark.gpu


def _caches(cuda, lens, seed):
    from hyprstream_b200 import kv_cache as kc

    g = torch.Generator().manual_seed(seed)
    caches = []
    for l in lens:
        c = kc.LayerKVCache(1 << 16, kc.KVQuantType.INT8, 8, 128, cuda)
        c.update(torch.randn(1, l, 8, 128, generator=g).bfloat16().to(cuda),
                 torch.randn(1, l, 8, 128, generator=g).bfloat16().to(cuda), 0)
        caches.append(c)
    return caches


def test_static_scratch_decode_matches_workspace_decode_twice(cuda):
    from hyprstream_b200 import ffi, kv_cache as kc, ops

    lens = [700, 33, 2049, 1, 512]
    caches = _caches(cuda, lens, seed=21)
    view, keep = kc.make_view(caches)
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=cuda)
    stream = torch.cuda.current_stream().cuda_stream
    out = torch.empty(len(lens), 32, 128, dtype=torch.bfloat16, device=cuda)
    for call in range(2):  # the second call finds the first call's partials in the array
        q = torch.randn(len(lens), 32, 128, generator=torch.Generator().manual_seed(100 + call)).bfloat16().to(cuda)
        ref = ops.decode_attention(q, view, seq_lens)
        out.fill_(float("nan"))
        st = ffi.lib.hs_attn_decode_static(q.data_ptr(), ctypes.byref(view), seq_lens.data_ptr(), len(lens), 32,
                                           1.0 / 128 ** 0.5, out.data_ptr(), None, stream)
        assert st == 0, ffi.last_error()
        torch.cuda.synchronize()
        diff = (out.float() - ref.float()).abs()
        assert torch.isfinite(out.float()).all()
        assert diff.max().item() <= MAX_ABS_TOL and diff.mean().item() <= MEAN_ABS_TOL, (call, diff.max().item())
    assert ffi.take_device_error() == 0


def test_static_scratch_decode_refuses_shapes_beyond_its_array(cuda):
    from hyprstream_b200 import ffi, kv_cache as kc

    caches = _caches(cuda, [16], seed=3)
    view, keep = kc.make_view(caches)
    limit = ffi.lib.hs_attn_decode_static_max_bytes()
    n = 1
    while ffi.lib.hs_attn_decode_workspace_bytes(n, 32, 128) <= limit:
        n *= 2
    x = torch.zeros(8, dtype=torch.int32, device=cuda)
    st = ffi.lib.hs_attn_decode_static(x.data_ptr(), ctypes.byref(view), x.data_ptr(), n, 32, 0.1, x.data_ptr(), None, None)
    assert st == ffi.HS_ERR_WORKSPACE
    msg = ffi.last_error()
    assert str(limit) in msg and "hs_attn_decode" in msg
    torch.cuda.synchronize()
    assert ffi.take_device_error() == 0
