"""GPU parity: decode attention over bf16 / int8 / NF4 / FP4 caches against the CPU oracle
(ATen op-for-op restatement over the dequantised cache) and the fp32 recomputation."""
import math
import os

import numpy as np
import pytest
import torch

from oracle import attention_ref as ar
from oracle import quant_ref as qr
from tests.util import GOLD, assert_close_attn, bf16_from_bits, no_device_error

pytestmark = pytest.mark.gpu


def build_caches(cuda, kind, lens, hkv, d, seed, block=64, scale_dtype=0, paged=False, page_tokens=256):
    """Per-sequence caches filled through update(); returns (caches, [k_deq], [v_deq]) with the dequantised
    (what the reference's get() would hand to attention) CPU tensors [1, L, Hkv, D] bf16."""
    from hyprstream_b200 import kv_cache as kc

    g = torch.Generator().manual_seed(seed)
    caches, ks, vs = [], [], []
    pool = None
    if paged:
        n_pages = sum((l + page_tokens - 1) // page_tokens for l in lens) + 1
        pool = kc.BlockPool(n_pages, hkv, d, cuda, kind=kind, block=block, scale_dtype=scale_dtype, page_tokens=page_tokens)
    for i, l in enumerate(lens):
        k = torch.randn(1, l, hkv, d, generator=g).bfloat16()
        v = torch.randn(1, l, hkv, d, generator=g).bfloat16()
        c = (kc.LayerKVCache.new_paged(1 << 20, pool, owner=i) if paged else
             kc.LayerKVCache(1 << 20, kc.KVQuantType(kind), hkv, d, cuda, block=block, scale_dtype=scale_dtype))
        c.update(k.to(cuda), v.to(cuda), 0)
        caches.append(c)
        if kind == 0:
            ks.append(k); vs.append(v)
        else:
            for src, dst in ((k, ks), (v, vs)):
                cr, a = qr.quantize(src.float().numpy(), kind, block, bool(scale_dtype))
                dq = qr.dequantize(cr, a, kind, src.numel(), block)
                dst.append(torch.from_numpy(dq).bfloat16().reshape(src.shape))
    return caches, ks, vs


def run_decode(cuda, caches, q, lens, gate=None, shard=False):
    from hyprstream_b200 import kv_cache as kc
    from hyprstream_b200 import ops

    view, keep = kc.make_view(caches)
    sl = torch.tensor(lens, dtype=torch.int32, device=cuda)
    out = ops.decode_attention(q.to(cuda), view, sl, gate=None if gate is None else gate.to(cuda), shard=shard)
    torch.cuda.synchronize()
    return out


def test_llama_decode_golden_fixture(cuda):
    """The committed config-1-shaped case: RoPE + bf16 cache + decode, against the oracle's stored output."""
    from hyprstream_b200 import kv_cache as kc
    from hyprstream_b200 import ops

    g = np.load(os.path.join(GOLD, "attn_llama_decode.npz"))
    q, k, v = (bf16_from_bits(g[n]) for n in ("q", "k", "v"))
    sin, cos = bf16_from_bits(g["sin"]).to(cuda), bf16_from_bits(g["cos"]).to(cuda)
    L, hkv, d = k.shape[1], k.shape[2], k.shape[3]
    q_rot = ops.rope_apply(q[0].to(cuda), sin, cos, torch.tensor([L - 1], dtype=torch.int32, device=cuda))
    assert torch.equal(q_rot.cpu(), bf16_from_bits(g["q_rope"])[0])
    cache = kc.LayerKVCache(4096, kc.KVQuantType.NONE, hkv, d, cuda)
    cache._ensure_capacity(L)
    view, keep = kc.make_view([cache])
    ops.kv_quantize_write(view, k.to(cuda), v.to(cuda), torch.zeros(1, dtype=torch.int32, device=cuda), sin, cos, d)
    cache.seq_pos = L
    kg, _ = cache.get()
    assert torch.equal(kg.cpu(), bf16_from_bits(g["k_rope"]))
    out = run_decode(cuda, [cache], q_rot, [L])
    ref = bf16_from_bits(g["out"]).reshape(1, -1, d)
    assert_close_attn(out, ref.float(), "golden llama decode")
    fp32 = ar.attention_fp32(bf16_from_bits(g["q_rope"]), bf16_from_bits(g["k_rope"]), v)[0]
    assert_close_attn(out, fp32, "golden llama decode vs fp32")
    no_device_error()


def test_qwen_gated_decode_golden_fixture(cuda):
    g = np.load(os.path.join(GOLD, "attn_qwen_gated_decode.npz"))
    q, gate, k, v = (bf16_from_bits(g[n]) for n in ("q", "gate", "k", "v"))
    from hyprstream_b200 import kv_cache as kc

    cache = kc.LayerKVCache(4096, kc.KVQuantType.NONE, k.shape[2], k.shape[3], cuda)
    cache.update(k.to(cuda), v.to(cuda), 0)
    out = run_decode(cuda, [cache], q[0], [k.shape[1]], gate=gate[0])
    ref = bf16_from_bits(g["out"]).reshape(1, q.shape[2], q.shape[3])
    assert_close_attn(out, ref.float(), "golden qwen gated decode")
    no_device_error()


@pytest.mark.parametrize("kind", [0, 1, 2, 3])
@pytest.mark.parametrize("hq,hkv,d", [(32, 8, 128), (16, 2, 256), (8, 8, 128), (4, 2, 64)])
def test_decode_lengths_and_shapes(cuda, kind, hq, hkv, d):
    """L in {1, 2, 63, 64, 65, 4095}; GQA 4:1, 8:1, 1:1, 2:1; D in {64, 128, 256}; every storage kind."""
    lens = [1, 2, 63, 64, 65, 4095]
    caches, ks, vs = build_caches(cuda, kind, lens, hkv, d, seed=kind * 10 + d)
    torch.manual_seed(5)
    q = torch.randn(len(lens), hq, d).bfloat16()
    out = run_decode(cuda, caches, q, lens)
    for r, l in enumerate(lens):
        oracle = ar.llama_attention_core(q[r].reshape(1, 1, hq, d), ks[r], vs[r], hq).reshape(hq, d)
        fp32 = ar.attention_fp32(q[r].reshape(1, 1, hq, d), ks[r], vs[r]).reshape(hq, d)
        assert_close_attn(out[r], oracle.float(), f"L={l} vs oracle")
        assert_close_attn(out[r], fp32, f"L={l} vs fp32")
    no_device_error()


@pytest.mark.parametrize("kind,block,sdt", [(1, 128, 1), (2, 64, 1), (1, 64, 0)])
def test_ragged_batch_equals_serial_and_oracle(cuda, kind, block, sdt):
    """Re-expression of architectures/llama.rs:3658-3711 on the kernels: a ragged batch (B=32, config-2 geometry)
    equals per-row unbatched decode bit-for-bit in its partition-independent part, and the oracle's padded,
    masked batched path within tolerance.  Runs the BASELINE layouts (block 128 / f16 scale) too."""
    rng = np.random.default_rng(1)
    lens = [int(x) for x in rng.integers(16, 700, size=32)]
    lens[3], lens[7] = 1, 2048
    hq, hkv, d = 32, 8, 128
    caches, ks, vs = build_caches(cuda, kind, lens, hkv, d, seed=9, block=block, scale_dtype=sdt)
    torch.manual_seed(6)
    q = torch.randn(len(lens), hq, d).bfloat16()
    out = run_decode(cuda, caches, q, lens)
    oracle = ar.llama_batched_decode(q.unsqueeze(1), ks, vs, [l - 1 for l in lens], hq).reshape(len(lens), hq, d)
    assert_close_attn(out, oracle.float(), "ragged batch vs oracle batched path")
    for r in (0, 3, 7, 31):
        single = run_decode(cuda, [caches[r]], q[r:r + 1], [lens[r]])
        assert (single[0].float() - out[r].float()).abs().max().item() <= 1e-2
        fp32 = ar.attention_fp32(q[r].reshape(1, 1, hq, d), ks[r], vs[r]).reshape(hq, d)
        assert_close_attn(out[r], fp32, f"row {r} vs fp32")
    no_device_error()


@pytest.mark.parametrize("block,sdt,paged", [(128, 1, False), (128, 1, True), (64, 1, False), (128, 0, False), (64, 0, False)])
def test_qwen_shape_ragged_gated_decode(cuda, block, sdt, paged):
    """Qwen3.5 full-attention decode shape (16 q / 2 kv heads, head_dim 256, int8 cache, output gate,
    qwen3_5.rs:992-1059) on a ragged batch: the oracle's gated core and the fp32 recomputation, row by row, and one
    long row cut across many CTAs."""
    rng = np.random.default_rng(3)
    lens = [int(x) for x in rng.integers(1, 900, size=12)] + [1, 31, 32, 33, 5000]
    hq, hkv, d = 16, 2, 256
    caches, ks, vs = build_caches(cuda, 1, lens, hkv, d, seed=21, block=block, scale_dtype=sdt, paged=paged)
    torch.manual_seed(8)
    q = torch.randn(len(lens), hq, d).bfloat16()
    gate = torch.randn(len(lens), hq, d).bfloat16()
    from hyprstream_b200 import ffi
    n0 = ffi.launch_count()
    out = run_decode(cuda, caches, q, lens, gate=gate)
    # every layout of this shape is served by the tensor-core kernel, which merges its own partials: one launch (the
    # reference layout - block 64, f32 absmax - fits only one CTA per SM and runs with a grid of that size)
    assert ffi.launch_count() - n0 == 1
    plain = run_decode(cuda, caches, q, lens)
    for r, l in enumerate(lens):
        oracle = ar.qwen_gated_attention_core(q[r].reshape(1, 1, hq, d), gate[r].reshape(1, 1, hq, d), ks[r], vs[r], hq).reshape(hq, d)
        assert_close_attn(out[r], oracle.float(), f"L={l} gated vs oracle")
        fp32 = ar.attention_fp32(q[r].reshape(1, 1, hq, d), ks[r], vs[r]).reshape(hq, d)
        assert_close_attn(plain[r], fp32, f"L={l} vs fp32")
    no_device_error()


@pytest.mark.parametrize("kind", [0, 1, 2])
def test_paged_equals_contiguous(cuda, kind):
    lens = [5, 300, 1000, 257]
    hq, hkv, d = 32, 8, 128
    c1, _, _ = build_caches(cuda, kind, lens, hkv, d, seed=3)
    c2, _, _ = build_caches(cuda, kind, lens, hkv, d, seed=3, paged=True)
    torch.manual_seed(8)
    q = torch.randn(len(lens), hq, d).bfloat16()
    a = run_decode(cuda, c1, q, lens)
    b = run_decode(cuda, c2, q, lens)
    assert torch.equal(a, b)
    no_device_error()


def test_shards_merge_to_unsplit(cuda):
    """KV-length shards -> (o, lse) partials -> hs_attn_merge_partials == the unsplit result (single GPU)."""
    from hyprstream_b200 import kv_cache as kc
    from hyprstream_b200 import ops

    hq, hkv, d, L = 32, 8, 128, 3000
    torch.manual_seed(10)
    k = torch.randn(1, L, hkv, d).bfloat16().to(cuda)
    v = torch.randn(1, L, hkv, d).bfloat16().to(cuda)
    q = torch.randn(1, hq, d).bfloat16()
    full = kc.LayerKVCache(1 << 20, kc.KVQuantType.INT8, hkv, d, cuda)
    full.update(k, v, 0)
    ref = run_decode(cuda, [full], q, [L])
    bounds = [0, 700, 701, 2048, L]  # uneven shards, one of length 1
    os_, ls_ = [], []
    for a, b in zip(bounds[:-1], bounds[1:]):
        c = kc.LayerKVCache(1 << 20, kc.KVQuantType.INT8, hkv, d, cuda)
        c.update(k[:, a:b].contiguous(), v[:, a:b].contiguous(), 0)
        o, lse = run_decode(cuda, [c], q, [b - a], shard=True)
        os_.append(o); ls_.append(lse)
    merged = ops.merge_partials(torch.stack(os_), torch.stack(ls_))
    # the same parts laid out as all-gathered messages [o | lse] per part, merged where they lie
    msgs = torch.cat([torch.cat([o.reshape(-1), l.reshape(-1)]) for o, l in zip(os_, ls_)])
    in_place = ops.merge_gathered(msgs, len(os_), q.shape[0], q.shape[1], q.shape[2])
    assert torch.equal(in_place, merged)
    assert (merged.float() - ref.float()).abs().max().item() <= 1e-3 + 8e-3  # bf16 output rounding
    # an empty shard (lse = -inf) contributes nothing
    os_.append(torch.zeros_like(os_[0])); ls_.append(torch.full_like(ls_[0], float("-inf")))
    merged2 = ops.merge_partials(torch.stack(os_), torch.stack(ls_))
    assert torch.equal(merged, merged2)
    no_device_error()


@pytest.mark.parametrize("kind,block,sdt,hq,hkv,d", [(1, 128, 1, 32, 8, 128), (2, 64, 0, 32, 8, 128), (1, 64, 0, 16, 2, 256)])
def test_long_ranges_many_tiles_per_cta(cuda, kind, block, sdt, hq, hkv, d):
    """Half a million cached tokens: every CTA of the tensor-core kernel walks about a hundred tiles, so the tile
    addresses are worked out in several batches and their shared-memory slots are reused, ring stages are refilled
    dozens of times by whichever warp finishes last, and sequences are cut across many CTAs.  Checked against an fp32
    recomputation over the dequantised cache (plain torch ops on the GPU), relative to the size of the outputs, and
    paged storage against contiguous storage bit for bit."""
    from hyprstream_b200 import kv_cache as kc

    lens = [120000, 90001, 131072, 140000]
    if d == 256:
        lens = [2 * l for l in lens]  # 32-token tiles at head_dim 256
    g = torch.Generator(device=cuda).manual_seed(11)
    pt = 256
    pool = kc.BlockPool(sum((l + pt - 1) // pt for l in lens) + 1, hkv, d, cuda, kind=kind, block=block, scale_dtype=sdt, page_tokens=pt)
    flat, paged = [], []
    torch.manual_seed(12)
    q = (torch.randn(len(lens), hq, d) * 3.0).bfloat16().to(cuda)  # peaked softmax: outputs of order 0.1 - 1, not averages near 0
    refs = []
    for i, l in enumerate(lens):
        k = torch.randn(1, l, hkv, d, device=cuda, generator=g).bfloat16()
        v = torch.randn(1, l, hkv, d, device=cuda, generator=g).bfloat16()
        c = kc.LayerKVCache(1 << 20, kc.KVQuantType(kind), hkv, d, cuda, block=block, scale_dtype=sdt)
        c.update(k, v, 0)
        p = kc.LayerKVCache.new_paged(1 << 20, pool, owner=i)
        p.update(k, v, 0)
        flat.append(c); paged.append(p)
        kd, vd = c.get()  # what the reference's get() hands to attention: the dequantised history
        kf = kd[0].float().repeat_interleave(hq // hkv, dim=1)  # [L, Hq, D]
        vf = vd[0].float().repeat_interleave(hq // hkv, dim=1)
        scores = torch.einsum("hd,lhd->hl", q[i].float(), kf) / math.sqrt(d)
        refs.append(torch.einsum("hl,lhd->hd", torch.softmax(scores, dim=-1), vf))
        del k, v, kd, vd, kf, vf, scores
    ref = torch.stack(refs)
    out = run_decode(cuda, flat, q, lens)
    diff = (out.float() - ref).abs()
    assert torch.isfinite(out.float()).all()
    assert ref.abs().max().item() > 0.2, "the case must have outputs large enough for the bound to mean something"
    assert diff.max().item() <= 2e-2 and diff.mean().item() <= 2e-3, (diff.max().item(), diff.mean().item())
    assert diff.max().item() <= 0.03 * ref.abs().max().item(), (diff.max().item(), ref.abs().max().item())
    out_paged = run_decode(cuda, paged, q, lens)
    assert torch.equal(out_paged, out)
    no_device_error()


def test_config1_full_size(cuda):
    """BASELINE config 1: B=1, 32 q / 8 kv heads, d=128, L=4096 bf16 cache, RoPE base 500000, vs the oracle."""
    from hyprstream_b200 import kv_cache as kc
    from hyprstream_b200 import ops

    torch.manual_seed(0)
    hq, hkv, d, L = 32, 8, 128, 4096
    q = torch.randn(1, 1, hq, d).bfloat16()
    k = torch.randn(1, L, hkv, d).bfloat16()
    v = torch.randn(1, L, hkv, d).bfloat16()
    sin, cos = ar.rope_tables(d, 500000.0, L, torch.bfloat16)
    q_rot = ar.apply_rope(q, sin, cos, torch.tensor([L - 1]))
    k_rot = ar.apply_rope(k, sin, cos, torch.arange(L))
    oracle = ar.llama_attention_core(q_rot, k_rot, v, hq).reshape(hq, d)
    cache = kc.LayerKVCache(L, kc.KVQuantType.NONE, hkv, d, cuda)
    cache._ensure_capacity(L)
    view, keep = kc.make_view([cache])
    ops.kv_quantize_write(view, k.to(cuda), v.to(cuda), None, sin.to(cuda), cos.to(cuda), d)
    cache.seq_pos = L
    qg = ops.rope_apply(q[0].to(cuda), sin.to(cuda), cos.to(cuda), torch.tensor([L - 1], dtype=torch.int32, device=cuda))
    out = run_decode(cuda, [cache], qg, [L])
    assert_close_attn(out[0], oracle.float(), "config 1 vs oracle")
    assert_close_attn(out[0], ar.attention_fp32(q_rot, k_rot, v).reshape(hq, d), "config 1 vs fp32")
    no_device_error()


def test_seq_len_beyond_pages_is_recorded_not_faulted(cuda):
    from hyprstream_b200 import ffi

    caches, _, _ = build_caches(cuda, 1, [100], 8, 128, seed=1)
    q = torch.randn(1, 32, 128).bfloat16()
    out = run_decode(cuda, caches, q, [5000])  # capacity is 1024 tokens
    assert torch.isfinite(out.float()).all()
    assert ffi.take_device_error() == ffi.DEVERR_DECODE_RANGE
