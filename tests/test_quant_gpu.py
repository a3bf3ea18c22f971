"""GPU parity: blockwise quantiser, RoPE and quantise-on-write, bit-exact against the CPU oracle."""
import os

import numpy as np
import pytest
import torch

from oracle import attention_ref as ar
from oracle import quant_ref as qr
from tests.util import GOLD, no_device_error

pytestmark = pytest.mark.gpu

KINDS = [(qr.INT8, "int8"), (qr.NF4, "nf4"), (qr.FP4, "fp4")]


def _oracle_scale(a, f16):
    return a.view(np.uint16) if f16 else a


@pytest.mark.parametrize("kind,kn", KINDS)
@pytest.mark.parametrize("block", [64, 128])
@pytest.mark.parametrize("f16", [False, True])
def test_quantize_matches_golden_fixture(cuda, kind, kn, block, f16):
    """f32 inputs incl. zero block, +-max at block ends, exact codeword midpoints, f16 saturation/underflow."""
    from hyprstream_b200 import ops

    g = np.load(os.path.join(GOLD, "quant_spec.npz"))
    x = torch.from_numpy(g["x"]).to(cuda)
    tag = f"{kn}_b{block}_{'f16' if f16 else 'f32'}"
    codes, absmax = ops.quantize_blockwise(x, kind, block, int(f16))
    assert np.array_equal(codes.cpu().numpy(), g[f"codes_{tag}"])
    got = absmax.cpu().numpy()
    assert np.array_equal(_oracle_scale(got, f16), g[f"absmax_{tag}"])
    deq = ops.dequantize_blockwise(codes, absmax, kind, x.numel(), block, torch.float32)
    assert np.array_equal(deq.cpu().numpy(), g[f"deq_{tag}"])
    no_device_error()


@pytest.mark.parametrize("kind,kn", KINDS)
@pytest.mark.parametrize("n", [1, 63, 64, 65, 8 * 1024 + 5, 1 << 20])
def test_quantize_bf16_ragged_sizes(cuda, kind, kn, n):
    from hyprstream_b200 import ops

    torch.manual_seed(n)
    x = torch.randn(n, dtype=torch.float32).bfloat16()
    for block, f16 in ((64, False), (128, True), (256, False)):
        c_ref, a_ref = qr.quantize(x.float().numpy(), kind, block, f16)
        codes, absmax = ops.quantize_blockwise(x.to(cuda), kind, block, int(f16))
        assert np.array_equal(codes.cpu().numpy(), c_ref), (n, block, f16)
        assert np.array_equal(_oracle_scale(absmax.cpu().numpy(), f16), _oracle_scale(a_ref, f16))
        deq = ops.dequantize_blockwise(codes, absmax, kind, n, block, torch.bfloat16)
        d_ref = torch.from_numpy(qr.dequantize(c_ref, a_ref, kind, n, block)).bfloat16()
        assert torch.equal(deq.cpu(), d_ref)
    no_device_error()


def test_quantize_full_size_properties(cuda):
    """Config-4 size (8*8192*8*128 = 67.1 M elements): size-independent properties instead of a CPU oracle pass —
    |dequant - x| <= half a code step, re-quantising the dequantised tensor is idempotent, and a 4 M-element
    slice is bit-exact against the oracle."""
    from hyprstream_b200 import ops

    n = 8 * 8192 * 8 * 128
    g = torch.Generator(device=cuda).manual_seed(3)
    x = torch.randn(n, device=cuda, generator=g, dtype=torch.float32).bfloat16()
    codes, absmax = ops.quantize_blockwise(x, qr.INT8, 64, 0)
    deq = ops.dequantize_blockwise(codes, absmax, qr.INT8, n, 64, torch.float32)
    step = absmax.repeat_interleave(64) / 127.0
    assert bool(((deq - x.float()).abs() <= 0.5 * step * (1 + 1e-5)).all())
    codes2, absmax2 = ops.quantize_blockwise(deq.bfloat16(), qr.INT8, 64, 0)
    assert torch.equal(codes, codes2)
    m = 1 << 22
    c_ref, a_ref = qr.quantize(x[:m].float().cpu().numpy(), qr.INT8, 64, False)
    assert np.array_equal(codes[:m].cpu().numpy(), c_ref) and np.array_equal(absmax[: m // 64].cpu().numpy(), a_ref)
    no_device_error()


@pytest.mark.parametrize("dim,rotary", [(128, 128), (256, 64)])
def test_rope_bit_exact(cuda, dim, rotary):
    """hs_rope_apply == RoPE::apply_rotary_pos_emb in bf16 (three roundings per element), full and partial."""
    from hyprstream_b200 import ops

    torch.manual_seed(1)
    rows, heads = 37, 3
    x = torch.randn(rows, heads, dim).bfloat16()
    pos = torch.randint(0, 500, (rows,))
    sin, cos = ar.rope_tables(rotary, 500000.0, 512, torch.bfloat16)
    ref = ar.apply_partial_rope(x.unsqueeze(0), sin, cos, pos, rotary)[0]
    out = ops.rope_apply(x.to(cuda), sin.to(cuda), cos.to(cuda), pos.to(torch.int32).to(cuda), rotary)
    assert torch.equal(out.cpu(), ref)
    no_device_error()


def test_rope_out_of_table_is_recorded_not_faulted(cuda):
    from hyprstream_b200 import ffi, ops

    x = torch.randn(2, 1, 128).bfloat16().to(cuda)
    sin, cos = ar.rope_tables(128, 10000.0, 8, torch.bfloat16)
    pos = torch.tensor([3, 99], dtype=torch.int32, device=cuda)
    out = ops.rope_apply(x, sin.to(cuda), cos.to(cuda), pos)
    assert ffi.take_device_error() == ffi.DEVERR_ROPE_RANGE
    assert torch.equal(out[1], x[1])  # the bad row is copied unrotated
    assert ffi.take_device_error() == 0


@pytest.mark.parametrize("kind,kn", KINDS + [(0, "bf16")])
@pytest.mark.parametrize("paged", [False, True])
def test_kv_write_and_get_match_flat_quantiser(cuda, kind, kn, paged):
    """LayerKVCache.update/get over device-resident storage: codes equal the flat quantiser's on the same rows
    (blocks never straddle a token), for prompt + incremental appends, contiguous and paged."""
    from hyprstream_b200 import kv_cache as kc
    from hyprstream_b200 import ops

    torch.manual_seed(2)
    hkv, d = 2, 128
    if paged:
        pool = kc.BlockPool(8, hkv, d, cuda, kind=kind, page_tokens=16)
        cache = kc.LayerKVCache.new_paged(100, pool, owner="a")
    else:
        cache = kc.LayerKVCache(4096, kc.KVQuantType(kind), hkv, d, cuda)
    k = torch.randn(1, 70, hkv, d).bfloat16().to(cuda)
    v = torch.randn(1, 70, hkv, d).bfloat16().to(cuda)
    cache.update(k[:, :37], v[:, :37], 0)
    for t in range(37, 70):
        cache.update(k[:, t:t + 1], v[:, t:t + 1], t)
    assert cache.seq_pos == 70
    kg, vg = cache.get()
    assert list(kg.shape) == [1, 70, hkv, d]
    if kind == 0:
        assert torch.equal(kg, k) and torch.equal(vg, v)
    else:
        for src, got in ((k, kg), (v, vg)):
            c_ref, a_ref = qr.quantize(src.float().cpu().numpy(), kind, 64, False)
            d_ref = torch.from_numpy(qr.dequantize(c_ref, a_ref, kind, src.numel(), 64)).bfloat16().reshape(src.shape)
            assert torch.equal(got.cpu(), d_ref)
    cache.truncate_to(40)
    kg2, _ = cache.get()
    assert torch.equal(kg2, kg[:, :40])
    no_device_error()


@pytest.mark.parametrize("kind,kn", [(qr.INT8, "int8"), (qr.NF4, "nf4"), (0, "bf16")])
@pytest.mark.parametrize("paged", [False, True])
def test_cache_offload_restore_round_trip(cuda, kind, kn, paged):
    """LayerKVCache.to_device(cpu) / to_device(cuda) (kv_cache.rs:1838-1858): the used rows are parked in host memory,
    the device storage (or the pages) is released, and the restored cache returns the same values bit for bit,
    decodes to the same output and accepts further appends."""
    from hyprstream_b200 import kv_cache as kc
    from hyprstream_b200 import ops

    torch.manual_seed(7)
    hq, hkv, d, n = 32, 8, 128, 83
    pool = None
    if paged:
        pool = kc.BlockPool(8, hkv, d, cuda, kind=kind, page_tokens=32)
        cache = kc.LayerKVCache.new_paged(200, pool, owner="a")
    else:
        cache = kc.LayerKVCache(4096, kc.KVQuantType(kind), hkv, d, cuda)
    k = torch.randn(1, n + 1, hkv, d).bfloat16().to(cuda)
    v = torch.randn(1, n + 1, hkv, d).bfloat16().to(cuda)
    cache.update(k[:, :n], v[:, :n], 0)
    k0, v0 = cache.get()
    q = torch.randn(1, hq, d).bfloat16().to(cuda)
    lens = torch.tensor([n], dtype=torch.int32, device=cuda)
    view, keep = kc.make_view([cache])
    out0 = ops.decode_attention(q, view, lens).clone()
    del view, keep
    used = cache.memory_usage()
    assert used > 0

    cache.to_device("cpu")
    assert cache.seq_pos == 0 and cache.memory_usage() == 0
    if paged:
        assert pool.num_free() == 8  # the pages went back to the pool
    with pytest.raises(ValueError):
        cache.get()  # "Cache is empty", like the reference's get() on an empty cache
    cache.to_device("cpu")  # a second offload is a no-op

    cache.to_device(cuda)
    assert cache.seq_pos == n
    k1, v1 = cache.get()
    assert torch.equal(k1, k0) and torch.equal(v1, v0)
    view, keep = kc.make_view([cache])
    out1 = ops.decode_attention(q, view, lens)
    assert torch.equal(out1, out0)
    del view, keep
    cache.update(k[:, n:], v[:, n:], n)  # the restored cache keeps growing
    k2, _ = cache.get()
    assert torch.equal(k2[:, :n], k0) and k2.shape[1] == n + 1
    no_device_error()


def test_kv_write_fused_rope_equals_rope_then_quantise(cuda):
    from hyprstream_b200 import kv_cache as kc
    from hyprstream_b200 import ops

    torch.manual_seed(4)
    hkv, d, n = 8, 128, 33
    cache = kc.LayerKVCache(1024, kc.KVQuantType.INT8, hkv, d, cuda)
    cache._ensure_capacity(100)
    view, keep = kc.make_view([cache])
    k = torch.randn(1, n, hkv, d).bfloat16()
    v = torch.randn(1, n, hkv, d).bfloat16()
    sin, cos = ar.rope_tables(d, 500000.0, 256, torch.bfloat16)
    start = 50
    ops.kv_quantize_write(view, k.to(cuda), v.to(cuda), torch.tensor([start], dtype=torch.int32, device=cuda),
                          sin.to(cuda), cos.to(cuda), d)
    cache.seq_pos = start + n
    kg, vg = cache.get()
    k_rot = ar.apply_rope(k, sin, cos, torch.arange(start, start + n))
    c_ref, a_ref = qr.quantize(k_rot.float().numpy(), qr.INT8, 64, False)
    d_ref = torch.from_numpy(qr.dequantize(c_ref, a_ref, qr.INT8, k_rot.numel(), 64)).bfloat16().reshape(k_rot.shape)
    assert torch.equal(kg[:, start:].cpu(), d_ref)
    no_device_error()


def test_cache_errors_mirror_reference(cuda):
    """Overflow and shape errors are raised on the host before any launch (kv_cache.rs:1281-1294);
    pool exhaustion is typed and rolls back (kv_cache.rs:482-505,1462-1470)."""
    from hyprstream_b200 import kv_cache as kc

    cache = kc.LayerKVCache(8, kc.KVQuantType.INT8, 2, 128, cuda)
    x = torch.zeros(1, 9, 2, 128, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(ValueError, match="Cache overflow"):
        cache.update(x, x, 0)
    with pytest.raises(ValueError, match="Expected 4D"):
        cache.update(x[0], x[0], 0)
    with pytest.raises(ValueError, match="empty"):
        cache.get()
    pool = kc.BlockPool(2, 2, 128, cuda, kind=1, page_tokens=16)
    a = kc.LayerKVCache.new_paged(100, pool, "a")
    a.update(x[:, :8], x[:, :8], 0)
    b = kc.LayerKVCache.new_paged(100, pool, "b")
    big = torch.zeros(1, 40, 2, 128, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(kc.BlockPoolExhausted):
        b.update(big, big, 0)
    assert pool.num_free() == 1 and b.blocks == []
    a.clear()
    assert pool.num_free() == 2


def test_pool_outlives_its_handle_while_caches_remain(cuda):
    """A paged cache keeps its pool's storage alive (the reference's caches hold an Arc<BlockPool>, kv_cache.rs:1111-1130):
    the pool handle may be dropped first, the cache still reads its pages and returns them when it is dropped itself."""
    from hyprstream_b200 import ffi, kv_cache as kc

    pool = kc.BlockPool(4, 2, 128, cuda, kind=1, page_tokens=16)
    c = kc.LayerKVCache.new_paged(64, pool, "a")
    g = torch.Generator(device=cuda).manual_seed(3)
    k = torch.randn(1, 40, 2, 128, device=cuda, generator=g).bfloat16()
    v = torch.randn(1, 40, 2, 128, device=cuda, generator=g).bfloat16()
    c.update(k, v, 0)
    k0, v0 = c.get()
    ffi.lib.hs_pool_destroy(pool._h)  # the handle goes first
    pool._h = None
    c.pool = None
    k1, v1 = c.get()
    assert torch.equal(k0, k1) and torch.equal(v0, v1)
    c.update(k[:, :8], v[:, :8], 40)  # the remaining page of the pool is still handed out
    assert c.seq_pos == 48
    del c
    torch.cuda.synchronize()
    no_device_error()


def test_boundary_rejects_bad_arguments(cuda):
    """Null / misaligned pointers, negative sizes, unsupported geometry -> status code, no launch, no sticky CUDA error."""
    import ctypes

    from hyprstream_b200 import ffi

    lib = ffi.lib
    x = torch.zeros(256, dtype=torch.bfloat16, device=cuda)
    codes = torch.zeros(256, dtype=torch.uint8, device=cuda)
    am = torch.zeros(4, dtype=torch.float32, device=cuda)
    assert lib.hs_quantize_blockwise(1, None, 0, 256, 64, 0, codes.data_ptr(), am.data_ptr(), None) == ffi.HS_ERR_ARG
    assert lib.hs_quantize_blockwise(1, x.data_ptr(), 0, -1, 64, 0, codes.data_ptr(), am.data_ptr(), None) == ffi.HS_ERR_ARG
    assert lib.hs_quantize_blockwise(1, x.data_ptr(), 0, 256, 48, 0, codes.data_ptr(), am.data_ptr(), None) == ffi.HS_ERR_UNSUPPORTED
    assert lib.hs_quantize_blockwise(9, x.data_ptr(), 0, 256, 64, 0, codes.data_ptr(), am.data_ptr(), None) == ffi.HS_ERR_ARG
    assert lib.hs_quantize_blockwise(1, x.data_ptr() + 1, 0, 200, 64, 0, codes.data_ptr(), am.data_ptr(), None) == ffi.HS_ERR_ARG
    assert "misaligned" in ffi.last_error()
    view = ffi.KVView(kind=1, scale_dtype=0, block=64, n_kv_heads=2, head_dim=128, page_tokens=16, pages_per_seq=1)
    assert lib.hs_attn_decode(x.data_ptr(), ctypes.byref(view), x.data_ptr(), 1, 4, 0.1, x.data_ptr(), None,
                              x.data_ptr(), 1 << 20, None, None, None) == ffi.HS_ERR_ARG  # NULL page tables
    view.head_dim = 96
    assert lib.hs_attn_decode(x.data_ptr(), ctypes.byref(view), x.data_ptr(), 1, 4, 0.1, x.data_ptr(), None,
                              x.data_ptr(), 1 << 20, None, None, None) == ffi.HS_ERR_UNSUPPORTED
    assert lib.hs_attn_decode(x.data_ptr(), None, x.data_ptr(), 1, 4, 0.1, x.data_ptr(), None, x.data_ptr(), 1 << 20,
                              None, None, None) == ffi.HS_ERR_ARG
    assert lib.hs_quantize_blockwise(1, x.data_ptr(), 0, 256, 64, 0, codes.data_ptr(), am.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert ffi.take_device_error() == 0
