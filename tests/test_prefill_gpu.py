"""GPU parity: causal GQA prefill against the CPU oracle (architectures/llama.rs:1023-1119 restated op for op,
including its 1024-row chunked loop) and the fp32 recomputation; fused path checks with quantise-on-write."""
import os

import numpy as np
import pytest
import torch

from oracle import attention_ref as ar
from oracle import quant_ref as qr
from tests.util import GOLD, assert_close_attn, bf16_from_bits, no_device_error

pytestmark = pytest.mark.gpu


def _rand(b, ql, kl, hq, hkv, d, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(b, ql, hq, d, generator=g).bfloat16(), torch.randn(b, kl, hkv, d, generator=g).bfloat16(),
            torch.randn(b, kl, hkv, d, generator=g).bfloat16())


@pytest.mark.parametrize("t", [1, 2, 127, 128, 129, 1024, 1025])
def test_llama_prefill_lengths(cuda, t):
    """T in {1, 2, 127, 128, 129, 1024, 1025}: 1025 crosses the reference's 1024-row query chunking (llama.rs:1094-1112)."""
    from hyprstream_b200 import ops

    hq, hkv, d = 8, 2, 128
    q, k, v = _rand(2, t, t, hq, hkv, d, seed=t)
    out = ops.prefill_attention(q.to(cuda), k.to(cuda), v.to(cuda))
    torch.cuda.synchronize()
    oracle = ar.llama_attention_core(q, k, v, hq).reshape(2, t, hq, d)
    assert_close_attn(out, oracle.float(), f"T={t} vs oracle")
    assert_close_attn(out, ar.attention_fp32(q, k, v), f"T={t} vs fp32")


@pytest.mark.parametrize("hq,hkv,d", [(4, 4, 64), (16, 2, 256), (32, 8, 128)])
def test_prefill_shapes(cuda, hq, hkv, d):
    from hyprstream_b200 import ops

    q, k, v = _rand(1, 300, 300, hq, hkv, d, seed=hq)
    out = ops.prefill_attention(q.to(cuda), k.to(cuda), v.to(cuda))
    torch.cuda.synchronize()
    assert_close_attn(out, ar.llama_attention_core(q, k, v, hq).reshape(1, 300, hq, d).float(), "vs oracle")
    assert_close_attn(out, ar.attention_fp32(q, k, v), "vs fp32")


def test_cached_prefix_offset_golden_and_serial_steps(cuda):
    """Re-expression of architectures/llama.rs:3746-3785 on the kernels: a 2-token forward at start_pos > 0 equals the
    stored oracle output and two 1-token decode steps; then a longer cached prefix (kv_len > q_len)."""
    from hyprstream_b200 import kv_cache as kc
    from hyprstream_b200 import ops

    f = np.load(os.path.join(GOLD, "attn_llama_cached2.npz"))
    q, k, v = (bf16_from_bits(f[n]) for n in ("q", "k", "v"))
    hq, d = q.shape[2], q.shape[3]
    out = ops.prefill_attention(q.to(cuda), k.to(cuda), v.to(cuda))
    torch.cuda.synchronize()
    assert_close_attn(out, bf16_from_bits(f["out"]).reshape(1, 2, hq, d).float(), "cached 2-token vs golden")
    L = k.shape[1]
    for i, kv_len in enumerate((L - 1, L)):
        cache = kc.LayerKVCache(4096, kc.KVQuantType.NONE, k.shape[2], d, cuda)
        cache.update(k[:, :kv_len].to(cuda), v[:, :kv_len].to(cuda), 0)
        view, keep = kc.make_view([cache])
        step = ops.decode_attention(q[0, i:i + 1].to(cuda), view, torch.tensor([kv_len], dtype=torch.int32, device=cuda))
        assert (step[0].float() - out[0, i].float()).abs().max().item() <= 1e-2
    q2, k2, v2 = _rand(2, 100, 777, 32, 8, 128, seed=9)
    out2 = ops.prefill_attention(q2.to(cuda), k2.to(cuda), v2.to(cuda))
    torch.cuda.synchronize()
    assert_close_attn(out2, ar.llama_attention_core(q2, k2, v2, 32).reshape(2, 100, 32, 128).float(), "prefix vs oracle")
    assert_close_attn(out2, ar.attention_fp32(q2, k2, v2), "prefix vs fp32")


def test_qwen_gated_prefill(cuda):
    """Qwen3.5 full-attention prefill: 16 q / 2 kv heads, D=256, bf16 P.V and the sigmoid output gate (qwen3_5.rs:1012-1059)."""
    from hyprstream_b200 import ops

    q, k, v = _rand(1, 200, 200, 16, 2, 256, seed=4)
    gate = torch.randn(1, 200, 16, 256, generator=torch.Generator().manual_seed(5)).bfloat16()
    out = ops.prefill_attention(q.to(cuda), k.to(cuda), v.to(cuda), gate=gate.to(cuda))
    torch.cuda.synchronize()
    oracle = ar.qwen_gated_attention_core(q, gate, k, v, 16).reshape(1, 200, 16, 256)
    assert_close_attn(out, oracle.float(), "gated prefill vs oracle")


@pytest.mark.parametrize("ql,kl", [(130, 700), (1024, 1024), (1, 64)])
def test_qwen_shape_prefix_and_long_rows(cuda, ql, kl):
    """head_dim 256 with a cached prefix (kv_len > q_len), more key tiles than score buffers and ring stages, two
    sequences, gate on: against the oracle's gated core and the fp32 recomputation of the ungated attention."""
    from hyprstream_b200 import ops

    q, k, v = _rand(2, ql, kl, 16, 2, 256, seed=ql)
    gate = torch.randn(2, ql, 16, 256, generator=torch.Generator().manual_seed(ql + 1)).bfloat16()
    out = ops.prefill_attention(q.to(cuda), k.to(cuda), v.to(cuda), gate=gate.to(cuda))
    plain = ops.prefill_attention(q.to(cuda), k.to(cuda), v.to(cuda))
    torch.cuda.synchronize()
    assert_close_attn(out, ar.qwen_gated_attention_core(q, gate, k, v, 16).reshape(2, ql, 16, 256).float(), "gated vs oracle")
    assert_close_attn(plain, ar.attention_fp32(q, k, v), "vs fp32")


def test_prefill_then_quantise_on_write_then_decode(cuda):
    """Config-4 flow at reduced size: RoPE -> prefill attention -> K/V written to the int8 cache (codes bit-exact to the
    oracle) -> the next decode step over that cache agrees with the oracle over the dequantised cache."""
    from hyprstream_b200 import kv_cache as kc
    from hyprstream_b200 import ops

    b, t, hq, hkv, d = 2, 384, 32, 8, 128
    q, k, v = _rand(b, t, t, hq, hkv, d, seed=12)
    sin, cos = ar.rope_tables(d, 500000.0, 512, torch.bfloat16)
    pos = torch.arange(t)
    q_rot = ar.apply_rope(q, sin, cos, pos)
    k_rot = ar.apply_rope(k, sin, cos, pos)
    pos_dev = pos.to(torch.int32).repeat(b).to(cuda)
    qg = ops.rope_apply(q.reshape(b * t, hq, d).to(cuda), sin.to(cuda), cos.to(cuda), pos_dev).reshape(b, t, hq, d)
    kg = ops.rope_apply(k.reshape(b * t, hkv, d).to(cuda), sin.to(cuda), cos.to(cuda), pos_dev).reshape(b, t, hkv, d)
    assert torch.equal(qg.cpu(), q_rot) and torch.equal(kg.cpu(), k_rot)
    out = ops.prefill_attention(qg, kg, v.to(cuda))
    torch.cuda.synchronize()
    assert_close_attn(out, ar.attention_fp32(q_rot, k_rot, v), "prefill vs fp32")
    caches = [kc.LayerKVCache(4096, kc.KVQuantType.INT8, hkv, d, cuda) for _ in range(b)]
    for c in caches:
        c._ensure_capacity(t + 1)
    view, keep = kc.make_view(caches)
    ops.kv_quantize_write(view, k.to(cuda), v.to(cuda), torch.zeros(b, dtype=torch.int32, device=cuda), sin.to(cuda), cos.to(cuda), d)
    ks, vs = [], []
    for i, c in enumerate(caches):
        c.seq_pos = t
        kgot, vgot = c.get()
        for src, got, dst in ((k_rot[i:i + 1], kgot, ks), (v[i:i + 1], vgot, vs)):
            cr, a = qr.quantize(src.float().numpy(), qr.INT8, 64, False)
            ref = torch.from_numpy(qr.dequantize(cr, a, qr.INT8, src.numel(), 64)).bfloat16().reshape(src.shape)
            assert torch.equal(got.cpu(), ref)
            dst.append(ref)
    qd = torch.randn(b, hq, d, generator=torch.Generator().manual_seed(3)).bfloat16()
    dec = ops.decode_attention(qd.to(cuda), view, torch.full((b,), t, dtype=torch.int32, device=cuda))
    torch.cuda.synchronize()
    oracle = ar.llama_batched_decode(qd.unsqueeze(1), ks, vs, [t - 1] * b, hq).reshape(b, hq, d)
    assert_close_attn(dec, oracle.float(), "decode after prefill")
    no_device_error()


def test_full_size_row_properties(cuda):
    """Config 4 geometry (8 x 8192, 32 q / 8 kv heads, d=128) is too large for the CPU oracle: check size-independent
    properties instead — with V = 1 every output is 1 (softmax rows sum to 1 under the causal mask), the first query row
    returns V[0], and a 64-row slice of one head matches the fp32 recomputation."""
    from hyprstream_b200 import ops

    b, t, hq, hkv, d = 8, 8192, 32, 8, 128
    g = torch.Generator(device=cuda).manual_seed(3)
    q = torch.randn(b, t, hq, d, device=cuda, generator=g).bfloat16()
    k = torch.randn(b, t, hkv, d, device=cuda, generator=g).bfloat16()
    v = torch.randn(b, t, hkv, d, device=cuda, generator=g).bfloat16()
    ones = torch.ones_like(v)
    out1 = ops.prefill_attention(q, k, ones)
    assert (out1.float() - 1.0).abs().max().item() <= 1e-2
    out = ops.prefill_attention(q, k, v)
    assert torch.equal(out[:, 0].reshape(b, hkv, hq // hkv, d), v[:, 0].unsqueeze(2).expand(b, hkv, hq // hkv, d))
    rows = slice(5000, 5064)
    qs, ks, vs = q[3:4, rows, 9:10].cpu(), k[3:4, :5064, 2:3].cpu(), v[3:4, :5064, 2:3].cpu()
    ref = ar.attention_fp32(qs, ks, vs)
    assert_close_attn(out[3:4, rows, 9:10], ref, "full-size slice vs fp32")


def test_prefill_rejects_bad_arguments(cuda):
    from hyprstream_b200 import ffi

    x = torch.zeros(64, dtype=torch.bfloat16, device=cuda)
    p = x.data_ptr()
    lib = ffi.lib
    assert lib.hs_attn_prefill_causal(p, p, p, p, None, 1, 4, 2, 8, 2, 128, 0.1, None) == ffi.HS_ERR_ARG       # kv_len < q_len
    assert lib.hs_attn_prefill_causal(p, p, p, p, None, 1, 4, 4, 8, 3, 128, 0.1, None) == ffi.HS_ERR_ARG       # heads
    assert lib.hs_attn_prefill_causal(p, p, p, p, None, 1, 4, 4, 8, 2, 96, 0.1, None) == ffi.HS_ERR_UNSUPPORTED
    assert lib.hs_attn_prefill_causal(None, p, p, p, None, 1, 4, 4, 8, 2, 128, 0.1, None) == ffi.HS_ERR_ARG
