"""CPU tests: the oracle against the committed fixtures and against itself (no GPU, no reference tree)."""
import os

import numpy as np
import pytest
import torch

from oracle import attention_ref as ar
from oracle import gdn_ref as gr
from oracle import quant_ref as qr

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def bf16_from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


KINDS = [(qr.INT8, "int8"), (qr.NF4, "nf4"), (qr.FP4, "fp4")]


@pytest.mark.parametrize("kind,kn", KINDS)
@pytest.mark.parametrize("block", [64, 128])
@pytest.mark.parametrize("f16", [False, True])
def test_quant_oracle_matches_golden(kind, kn, block, f16):
    g = np.load(os.path.join(GOLD, "quant_spec.npz"))
    x = g["x"]
    tag = f"{kn}_b{block}_{'f16' if f16 else 'f32'}"
    for fn in (qr.quantize_c, qr.quantize_np):
        c, a = fn(x, kind, block, f16)
        assert np.array_equal(c, g[f"codes_{tag}"])
        assert np.array_equal(a.view(np.uint16) if f16 else a, g[f"absmax_{tag}"])
    a = g[f"absmax_{tag}"].view(np.float16) if f16 else g[f"absmax_{tag}"]
    for fn in (qr.dequantize_c, qr.dequantize_np):
        assert np.array_equal(fn(g[f"codes_{tag}"], a, kind, x.size, block), g[f"deq_{tag}"])


def test_quant_pinned_facts():
    """What the reference does pin: codebooks, byte counts, block counts (bitsandbytes-sys/src/lib.rs:104-197,658-677)."""
    t = qr.codebook(qr.INT8)
    assert t.shape == (256,) and t[127] == 0.0 and t[0] == -1.0 and t[254] == 1.0
    assert np.array_equal(t, np.array([(np.float32(i) - np.float32(127)) / np.float32(127) for i in range(256)], np.float32))
    assert qr.codebook(qr.NF4).shape == (16,) and qr.codebook(qr.NF4)[7] == 0.0
    x = np.arange(1000, dtype=np.float32)
    c, a = qr.quantize(x, qr.INT8, 64)
    assert c.size == 1000 and a.size == 16
    c, a = qr.quantize(x[:999], qr.NF4, 64)
    assert c.size == 500 and a.size == 16


def test_quant_edge_semantics():
    # all-zero block -> code of 0.0, absmax 0 (A4); +-absmax -> end codes; midpoint tie -> lower index (A2)
    x = np.zeros(64, np.float32)
    c, a = qr.quantize(x, qr.INT8, 64)
    assert a[0] == 0.0 and (c == 127).all()
    x[0], x[63] = 2.5, -2.5
    c, a = qr.quantize(x, qr.INT8, 64)
    assert a[0] == 2.5 and c[0] == 254 and c[63] == 0 and (c[1:63] == 127).all()
    mid = qr.midpoints(qr.NF4)
    x = np.zeros(64, np.float32)
    x[0] = 1.0
    x[1:16] = mid
    c, _ = qr.quantize(x, qr.NF4, 64)
    idx = np.stack([c >> 4, c & 15], 1).reshape(-1)
    assert idx[0] == 15 and np.array_equal(idx[1:16], np.arange(15))
    x[1:16] = np.nextafter(mid, np.float32(2.0))
    c, _ = qr.quantize(x, qr.NF4, 64)
    idx = np.stack([c >> 4, c & 15], 1).reshape(-1)
    assert np.array_equal(idx[1:16], np.arange(1, 16))


def test_quant_requantise_is_idempotent():
    """Per-token quantise-on-write gives the codes the reference's flush (dequantise-all, re-quantise,
    kv_cache.rs:1234-1244) would keep: re-quantising bf16-dequantised data reproduces the codes."""
    rng = np.random.default_rng(5)
    x = torch.from_numpy(rng.standard_normal(64 * 512).astype(np.float32)).bfloat16().float().numpy()
    for kind in (qr.INT8, qr.NF4):
        c, a = qr.quantize(x, kind, 64)
        d = torch.from_numpy(qr.dequantize(c, a, kind, x.size, 64)).bfloat16().float().numpy()
        c2, a2 = qr.quantize(d, kind, 64)
        assert np.array_equal(c, c2)


def test_quant_roundtrip_error_bound():
    rng = np.random.default_rng(6)
    x = rng.standard_normal(64 * 256).astype(np.float32)
    c, a = qr.quantize(x, qr.INT8, 64)
    d = qr.dequantize(c, a, qr.INT8, x.size, 64)
    step = np.repeat(a, 64) / 127.0
    assert (np.abs(d - x) <= 0.5 * step * (1 + 1e-5)).all()


def test_attention_oracle_matches_golden():
    g = np.load(os.path.join(GOLD, "attn_llama_decode.npz"))
    q, k, v = (bf16_from_bits(g[n]) for n in ("q", "k", "v"))
    sin, cos = bf16_from_bits(g["sin"]), bf16_from_bits(g["cos"])
    L = k.shape[1]
    s2, c2 = ar.rope_tables(128, 500000.0, 128, torch.bfloat16)
    assert torch.equal(s2, sin) and torch.equal(c2, cos)
    qr_ = ar.apply_rope(q, sin, cos, torch.tensor([L - 1]))
    kr = ar.apply_rope(k, sin, cos, torch.arange(L))
    assert torch.equal(qr_, bf16_from_bits(g["q_rope"])) and torch.equal(kr, bf16_from_bits(g["k_rope"]))
    out = ar.llama_attention_core(qr_, kr, v, q.shape[2])
    ref = bf16_from_bits(g["out"])
    assert (out.float() - ref.float()).abs().max() <= 2e-2  # bf16 output; libtorch builds may differ in the last bit
    g = np.load(os.path.join(GOLD, "attn_qwen_gated_decode.npz"))
    out = ar.qwen_gated_attention_core(*(bf16_from_bits(g[n]) for n in ("q", "gate", "k", "v")), 8)
    assert (out.float() - bf16_from_bits(g["out"]).float()).abs().max() <= 2e-2


def test_attention_cached_two_tokens_equals_two_steps():
    """Re-expression of architectures/llama.rs:3746-3785: a 2-token cached forward at start_pos > 0 equals two
    1-token decode steps (pins the tril(k_len - q_len) offset)."""
    g = np.load(os.path.join(GOLD, "attn_llama_cached2.npz"))
    q, k, v = (bf16_from_bits(g[n]) for n in ("q", "k", "v"))
    both = ar.llama_attention_core(q.float(), k.float(), v.float(), q.shape[2])
    L = k.shape[1]
    first = ar.llama_attention_core(q[:, :1].float(), k[:, : L - 1].float(), v[:, : L - 1].float(), q.shape[2])
    second = ar.llama_attention_core(q[:, 1:].float(), k.float(), v.float(), q.shape[2])
    assert torch.allclose(both[:, 0], first[:, 0], rtol=1e-4, atol=1e-4)
    assert torch.allclose(both[:, 1], second[:, 0], rtol=1e-4, atol=1e-4)
    fp32 = ar.attention_fp32(q, k, v).reshape(1, 2, -1)
    assert torch.allclose(both, fp32, rtol=1e-4, atol=1e-4)


def test_attention_batched_equals_serial():
    """Re-expression of architectures/llama.rs:3658-3711: ragged batched decode == per-row serial decode."""
    torch.manual_seed(3)
    hq, hkv, d = 8, 2, 64
    lens = [5, 17, 9]
    q = torch.randn(3, 1, hq, d)
    ks = [torch.randn(1, l, hkv, d) for l in lens]
    vs = [torch.randn(1, l, hkv, d) for l in lens]
    batched = ar.llama_batched_decode(q, ks, vs, [l - 1 for l in lens], hq)
    for r in range(3):
        serial = ar.llama_attention_core(q[r:r + 1], ks[r], vs[r], hq)
        assert torch.allclose(batched[r], serial[0], rtol=1e-4, atol=1e-4)


def test_gdn_oracle_matches_independent_implementation():
    g = np.load(os.path.join(GOLD, "gdn_hf.npz"))
    q, k, v, gg, beta, s0 = (torch.from_numpy(g[n]) for n in ("q", "k", "v", "g", "beta", "s0"))
    qs = q * (q.shape[-1] ** -0.5)  # the reference scales q before the rule (qwen3_5.rs:681-682)
    o, s = gr.chunked_delta_rule(qs, k, v, gg, beta, s0)
    assert np.abs(o.numpy() - g["out_chunk"]).max() < 1e-5 and np.abs(s.numpy() - g["state_chunk"]).max() < 1e-5
    o2, s2 = gr.recurrent_sequence(qs, k, v, gg, beta, s0)
    assert np.abs(o2.numpy() - g["out_rec"]).max() < 1e-5 and np.abs(s2.numpy() - g["state_rec"]).max() < 1e-5
    assert (o - o2).abs().max() < 1e-4 and (s - s2).abs().max() < 1e-4  # chunked == recurrent


# ---- the attention oracle against `transformers` (fixtures made by tests/golden/make_golden.py::attn_hf_cases) ----
def _mostly_equal_bf16(mine: torch.Tensor, ref: torch.Tensor, what: str, frac: float = 0.97):
    """bf16 results of two implementations that differ only in fp32 operation order: nearly all elements equal bit for
    bit, none further apart than two bf16 steps of the row's scale."""
    a, b = mine.float(), ref.float()
    diff = (a - b).abs()
    scale = b.abs().amax(dim=-1, keepdim=True).clamp_min(1e-6)
    assert torch.all(diff <= 2 ** -6 * scale), f"{what}: max diff {diff.max().item():.3g}"
    assert (diff == 0).float().mean().item() >= frac, f"{what}: only {(diff == 0).float().mean().item():.4f} equal"


def test_llama_rope_and_attention_oracle_match_transformers():
    """RoPE::apply_rotary_pos_emb (rope.rs:100-248) and the Llama attention core (llama.rs:1023-1119) as restated by the
    oracle, against transformers' apply_rotary_pos_emb / repeat_kv / eager_attention_forward on the same inputs: one
    decode token and a 5-token forward over a cached prefix."""
    g = np.load(os.path.join(GOLD, "attn_hf_llama.npz"))
    k, v = bf16_from_bits(g["k"]), bf16_from_bits(g["v"])
    L, hkv, d = k.shape[1], k.shape[2], k.shape[3]
    sin, cos = ar.rope_tables(d, 500000.0, 128, torch.bfloat16)
    k_rot = ar.apply_rope(k, sin, cos, torch.arange(L))
    _mostly_equal_bf16(k_rot, bf16_from_bits(g["k_rope"]), "k rope")
    for name, ql in (("decode", 1), ("cached5", 5)):
        q = bf16_from_bits(g[f"q_{name}"])
        hq = q.shape[2]
        q_rot = ar.apply_rope(q, sin, cos, torch.arange(L - ql, L))
        _mostly_equal_bf16(q_rot, bf16_from_bits(g[f"q_rope_{name}"]), f"q rope {name}")
        # the attention core on transformers' own rotated tensors, so that only the attention arithmetic is compared
        out = ar.llama_attention_core(bf16_from_bits(g[f"q_rope_{name}"]), bf16_from_bits(g["k_rope"]), v, hq).reshape(1, ql, hq, d)
        ref = torch.from_numpy(g[f"out_{name}"])                      # fp32 [1, ql, Hq, D]
        _mostly_equal_bf16(out, ref.bfloat16(), f"attention {name}", frac=0.95)
        diff = (out.float() - ref).abs()
        assert diff.max().item() <= 2e-2 and diff.mean().item() <= 2e-3
        # and the fp32 recomputation that anchors the kernels' tolerance is the same mathematics
        fp32 = ar.attention_fp32(bf16_from_bits(g[f"q_rope_{name}"]), bf16_from_bits(g["k_rope"]), v)
        assert (fp32 - ref).abs().max().item() <= 1e-5


def test_qwen_gated_attention_oracle_matches_transformers():
    """QK-norm with (1 + w), partial RoPE, gate split and the gated attention core (qwen3_5.rs:902-1091) as restated by
    the oracle, against transformers' Qwen3_5RMSNorm, apply_rotary_pos_emb, eager_attention_forward and the gate
    arithmetic of Qwen3_5Attention.forward."""
    g = np.load(os.path.join(GOLD, "attn_hf_qwen.npz"))
    k_proj, v = bf16_from_bits(g["k_proj"]), bf16_from_bits(g["v"])
    qw, kw = torch.from_numpy(g["q_norm_w"]), torch.from_numpy(g["k_norm_w"])
    L, hkv, d = k_proj.shape[1], k_proj.shape[2], k_proj.shape[3]
    rd = 64
    sin, cos = ar.rope_tables(rd, 10000.0, 128, torch.bfloat16)
    k_rot = ar.apply_partial_rope(ar.qk_norm(k_proj, kw, 1e-6), sin, cos, torch.arange(L), rd)
    _mostly_equal_bf16(k_rot, bf16_from_bits(g["k_rope"]), "k norm + rope")
    for name, ql in (("decode", 1), ("cached4", 4)):
        q_proj = bf16_from_bits(g[f"q_proj_{name}"])                 # [1, ql, Hq, 2 D]: query | gate
        hq = q_proj.shape[2]
        query, gate = q_proj[..., :d], q_proj[..., d:]
        q_rot = ar.apply_partial_rope(ar.qk_norm(query, qw, 1e-6), sin, cos, torch.arange(L - ql, L), rd)
        _mostly_equal_bf16(q_rot, bf16_from_bits(g[f"q_rope_{name}"]), f"q norm + rope {name}")
        out = ar.qwen_gated_attention_core(bf16_from_bits(g[f"q_rope_{name}"]), gate.contiguous(), bf16_from_bits(g["k_rope"]), v, hq).reshape(1, ql, hq, d)
        ref = bf16_from_bits(g[f"out_{name}"]).float()
        # transformers forms the scores in bf16, the reference in fp32 (qwen3_5.rs:1021-1032): equal within the path's tolerance
        diff = (out.float() - ref).abs()
        assert diff.max().item() <= 2e-2 and diff.mean().item() <= 2e-3, (name, diff.max().item(), diff.mean().item())
