"""GPU test of hs_attn_decode_static, the decode entry point that brings its own scratch.

It exists for hosts that cannot allocate device memory where they decode (under a foreign allocator that owns
the whole budget, where a device-wide synchronisation is not acceptable, or in a step function that runs where
allocation is forbidden), so this test hands it nothing but inputs and a preallocated output, straight through
the C ABI, and compares with hs_attn_decode given an ordinary workspace and with an fp32 recomputation over the
dequantised cache.  It also checks the property the entry point exists for: the device's free-memory figure does
not move across a call.  The file name keeps it last in collection order; it must pass both alone in a fresh
process (its first call then performs the per-device address look-up) and after every other test.
"""
import ctypes

import pytest
import torch

from tests.util import MAX_ABS_TOL, MEAN_ABS_TOL

pytestmark = pytest.mark.gpu


def _caches(cuda, lens, seed, hkv=8, d=128):
    from hyprstream_b200 import kv_cache as kc

    g = torch.Generator().manual_seed(seed)
    caches = []
    for l in lens:
        c = kc.LayerKVCache(1 << 16, kc.KVQuantType.INT8, hkv, d, cuda)
        c.update(torch.randn(1, l, hkv, d, generator=g).bfloat16().to(cuda),
                 torch.randn(1, l, hkv, d, generator=g).bfloat16().to(cuda), 0)
        caches.append(c)
    return caches


def _fp32_over_dequantised(caches, q):
    """Attention in fp32 over what the caches hold (their dequantised contents), plain torch ops."""
    rows = []
    for r, c in enumerate(caches):
        k, v = c.get()
        g = q.shape[1] // k.shape[2]
        kf = k[0].float().repeat_interleave(g, dim=1)
        vf = v[0].float().repeat_interleave(g, dim=1)
        s = torch.einsum("hd,lhd->hl", q[r].float(), kf) / q.shape[2] ** 0.5
        rows.append(torch.einsum("hl,lhd->hd", torch.softmax(s, -1), vf))
    return torch.stack(rows)


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
        fp32 = _fp32_over_dequantised(caches, q)
        out.fill_(float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(cuda)[0]
        n0 = ffi.launch_count()
        st = ffi.lib.hs_attn_decode_static(q.data_ptr(), ctypes.byref(view), seq_lens.data_ptr(), len(lens), 32,
                                           1.0 / 128 ** 0.5, out.data_ptr(), None, stream)
        assert st == 0, ffi.last_error()
        torch.cuda.synchronize()
        if call == 1:  # (the first call of a process may load the kernel's module; from then on nothing may move)
            assert torch.cuda.mem_get_info(cuda)[0] == free_before, "hs_attn_decode_static changed the device's free memory"
        assert ffi.launch_count() - n0 == 1  # the tensor-core kernel, partials in the built-in array
        assert torch.isfinite(out.float()).all()
        assert (out.float() - ref.float()).abs().max().item() <= 4e-3, call  # same kernel and partition as the workspace form
        diff = (out.float() - fp32).abs()
        assert diff.max().item() <= MAX_ABS_TOL and diff.mean().item() <= MEAN_ABS_TOL, (call, diff.max().item())
    assert ffi.take_device_error() == 0


def test_static_scratch_serves_the_generic_kernel_and_its_merge_too(cuda):
    """A shape the tensor-core kernel does not cover (4 q / 2 kv heads, head_dim 64): the CUDA-core decode kernel and
    the separate merge kernel both run out of the built-in array; two calls in a row, no allocation."""
    from hyprstream_b200 import ffi, kv_cache as kc, ops

    lens = [300, 5, 1025]
    caches = _caches(cuda, lens, seed=23, hkv=2, d=64)
    view, keep = kc.make_view(caches)
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=cuda)
    out = torch.empty(len(lens), 4, 64, dtype=torch.bfloat16, device=cuda)
    for call in range(2):
        q = torch.randn(len(lens), 4, 64, generator=torch.Generator().manual_seed(200 + call)).bfloat16().to(cuda)
        ref = ops.decode_attention(q, view, seq_lens)
        fp32 = _fp32_over_dequantised(caches, q)
        out.fill_(float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(cuda)[0]
        n0 = ffi.launch_count()
        st = ffi.lib.hs_attn_decode_static(q.data_ptr(), ctypes.byref(view), seq_lens.data_ptr(), len(lens), 4, 1.0 / 64 ** 0.5,
                                           out.data_ptr(), None, torch.cuda.current_stream().cuda_stream)
        assert st == 0, ffi.last_error()
        torch.cuda.synchronize()
        if call == 1:
            assert torch.cuda.mem_get_info(cuda)[0] == free_before
        assert ffi.launch_count() - n0 == 2  # decode + merge
        assert (out.float() - ref.float()).abs().max().item() <= 4e-3, call
        diff = (out.float() - fp32).abs()
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
