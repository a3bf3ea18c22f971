"""GPU parity of the kernels against fixtures computed by `transformers` (tests/golden/attn_hf_*.npz, made by
tests/golden/make_golden.py::attn_hf_cases): Llama RoPE + attention and Qwen3.5 gated attention, decode and a
multi-token forward over a cached prefix.  These expected values do not come from this repository's oracle."""
import os

import numpy as np
import pytest
import torch

from tests.util import GOLD, assert_close_attn, bf16_from_bits, no_device_error

pytestmark = pytest.mark.gpu


def test_llama_rope_decode_and_cached_prefill_match_transformers(cuda):
    from oracle import attention_ref as ar
    from hyprstream_b200 import kv_cache as kc, ops

    g = np.load(os.path.join(GOLD, "attn_hf_llama.npz"))
    k, v = bf16_from_bits(g["k"]), bf16_from_bits(g["v"])
    L, hkv, d = k.shape[1], k.shape[2], k.shape[3]
    sin, cos = (t.to(cuda) for t in ar.rope_tables(d, 500000.0, 128, torch.bfloat16))
    # cache update with the fused K rotation, then read back: the rotated keys
    cache = kc.LayerKVCache(1024, kc.KVQuantType.NONE, hkv, d, cuda)
    cache._ensure_capacity(L)
    view, keep = kc.make_view([cache])
    ops.kv_quantize_write(view, k.to(cuda), v.to(cuda), torch.zeros(1, dtype=torch.int32, device=cuda), sin, cos, d)
    cache.seq_pos = L
    k_rot, _ = cache.get()
    ref_k = bf16_from_bits(g["k_rope"])
    assert (k_rot.cpu() == ref_k).float().mean().item() >= 0.97
    assert (k_rot.cpu().float() - ref_k.float()).abs().max().item() <= 2 ** -6 * ref_k.float().abs().max().item()
    for name, ql in (("decode", 1), ("cached5", 5)):
        q = bf16_from_bits(g[f"q_{name}"])
        hq = q.shape[2]
        pos = torch.arange(L - ql, L, dtype=torch.int32, device=cuda)
        q_rot = ops.rope_apply(q[0].to(cuda), sin, cos, pos)
        assert (q_rot.cpu() == bf16_from_bits(g[f"q_rope_{name}"])[0]).float().mean().item() >= 0.97
        ref = torch.from_numpy(g[f"out_{name}"])[0]   # fp32 [ql, Hq, D]
        if ql == 1:
            out = ops.decode_attention(q_rot, view, torch.tensor([L], dtype=torch.int32, device=cuda))
        else:  # query rows at positions L - ql .. L - 1 over all L keys: the cached-prefix offset
            out = ops.prefill_attention(q_rot.unsqueeze(0), k_rot, v.to(cuda))[0]
        torch.cuda.synchronize()
        assert_close_attn(out.reshape(ql, hq, d), ref, f"llama {name} vs transformers")
    no_device_error()


def test_qwen_gated_attention_matches_transformers(cuda):
    from oracle import attention_ref as ar
    from hyprstream_b200 import kv_cache as kc, ops

    g = np.load(os.path.join(GOLD, "attn_hf_qwen.npz"))
    k_proj, v = bf16_from_bits(g["k_proj"]), bf16_from_bits(g["v"])
    qw, kw = torch.from_numpy(g["q_norm_w"]).to(cuda), torch.from_numpy(g["k_norm_w"]).to(cuda)
    L, hkv, d, rd = k_proj.shape[1], k_proj.shape[2], k_proj.shape[3], 64
    sin, cos = (t.to(cuda) for t in ar.rope_tables(rd, 10000.0, 128, torch.bfloat16))
    k_rot = ops.qk_norm_rope(k_proj[0].reshape(L, -1).contiguous().to(cuda), hkv, d, kw, 1e-6, True, sin, cos,
                             torch.arange(L, dtype=torch.int32, device=cuda), rd)
    ref_k = bf16_from_bits(g["k_rope"])[0]
    assert (k_rot.cpu() == ref_k).float().mean().item() >= 0.97
    cache = kc.LayerKVCache(1024, kc.KVQuantType.NONE, hkv, d, cuda)
    cache.update(k_rot.unsqueeze(0), v.to(cuda), 0)
    view, keep = kc.make_view([cache])
    for name, ql in (("decode", 1), ("cached4", 4)):
        q_proj = bf16_from_bits(g[f"q_proj_{name}"])   # [1, ql, Hq, 2 D]
        hq = q_proj.shape[2]
        pos = torch.arange(L - ql, L, dtype=torch.int32, device=cuda)
        query, gate = ops.qk_norm_rope(q_proj[0].reshape(ql, -1).contiguous().to(cuda), hq, d, qw, 1e-6, True, sin, cos, pos, rd, with_gate=True)
        assert (query.cpu() == bf16_from_bits(g[f"q_rope_{name}"])[0]).float().mean().item() >= 0.97
        ref = bf16_from_bits(g[f"out_{name}"])[0].float()
        if ql == 1:
            out = ops.decode_attention(query, view, torch.tensor([L], dtype=torch.int32, device=cuda), gate=gate)
        else:
            out = ops.prefill_attention(query.unsqueeze(0), k_rot.unsqueeze(0), v.to(cuda), gate=gate.unsqueeze(0))[0]
        torch.cuda.synchronize()
        assert_close_attn(out.reshape(ql, hq, d), ref, f"qwen {name} vs transformers")
    no_device_error()
