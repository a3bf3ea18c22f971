"""Generates the committed fixtures in tests/golden/ (run from the repository root:
``python tests/golden/make_golden.py``).

The reference holds no golden vectors for this path, so these fixtures are made here:
* quant_*.npz       — seeded and hand-built edge-case inputs with the codes/scales of the written
                      quantiser specification (oracle/quant_spec.c), both restatements agreeing;
* attn_*.npz        — small seeded attention cases with the outputs of the ATen op-for-op
                      restatement (oracle/attention_ref.py);
* attn_hf_*.npz     — attention cases whose expected outputs come from the independent implementation in
                      `transformers` (models/llama/modeling_llama.py: apply_rotary_pos_emb, repeat_kv,
                      eager_attention_forward; models/qwen3_5/modeling_qwen3_5.py: Qwen3_5RMSNorm, its partial-rotary
                      apply_rotary_pos_emb, eager_attention_forward, and the gate arithmetic of Qwen3_5Attention.forward):
                      the functions are imported and called, so the oracle in oracle/attention_ref.py is checked against
                      something other than itself;
* gdn_hf_*.npz      — gated-DeltaNet cases whose expected outputs come from the independent
                      implementation in `transformers` (models/qwen3_5/modeling_qwen3_5.py:
                      torch_chunk_gated_delta_rule / torch_recurrent_gated_delta_rule), the function the
                      reference says it translated (architectures/qwen3_5.rs:337).  `transformers`
                      is only needed to regenerate; the tests read the .npz.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import attention_ref as ar  # noqa: E402
from oracle import gdn_ref as gr  # noqa: E402
from oracle import quant_ref as qr  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def quant_cases():
    rng = np.random.default_rng(1234)
    x = torch.from_numpy(rng.standard_normal(64 * 40 + 37).astype(np.float32)).bfloat16().float().numpy()
    x[64:128] = 0.0                                    # an all-zero block (assumption A4)
    x[128] = 3.0; x[191] = -3.0                        # +-max at the block ends
    # values placed exactly on codeword midpoints (assumption A2): block absmax 1 so y == x
    mid8 = qr.midpoints(qr.INT8)
    x[192:256] = 0.0; x[192] = 1.0
    x[193:193 + 40] = mid8[100:140]
    x[256:320] = 0.0; x[256] = -1.0
    x[257:257 + 15] = qr.midpoints(qr.NF4)
    x[320:384] = 0.0; x[320] = 1.0
    x[321:321 + 15] = qr.midpoints(qr.FP4)
    x[384:448] = 70000.0 * np.sign(x[384:448] + 1e-9)  # beyond f16 range: saturating scale (assumption A6)
    x[448:512] *= 1e-7                                 # tiny block: f16 scale underflows towards 0
    out = {"x": x}
    for kind, kn in ((qr.INT8, "int8"), (qr.NF4, "nf4"), (qr.FP4, "fp4")):
        for block in (64, 128):
            for f16 in (False, True):
                c, a = qr.quantize_c(x, kind, block, f16)
                c2, a2 = qr.quantize_np(x, kind, block, f16)
                assert np.array_equal(c, c2) and np.array_equal(a.view(np.uint8), a2.view(np.uint8))
                tag = f"{kn}_b{block}_{'f16' if f16 else 'f32'}"
                out[f"codes_{tag}"] = c
                out[f"absmax_{tag}"] = a.view(np.uint16) if f16 else a
                out[f"deq_{tag}"] = qr.dequantize_c(c, a, kind, x.size, block)
    np.savez_compressed(os.path.join(OUT, "quant_spec.npz"), **out)


def attn_cases():
    torch.manual_seed(7)
    # Llama-shaped decode (config 1 geometry, short): 8 q heads / 2 kv heads, d=128, L=77, RoPE base 500000
    hq, hkv, d, L = 8, 2, 128, 77
    sin, cos = ar.rope_tables(d, 500000.0, 128, torch.bfloat16)
    q = torch.randn(1, 1, hq, d).bfloat16()
    k = torch.randn(1, L, hkv, d).bfloat16()
    v = torch.randn(1, L, hkv, d).bfloat16()
    qr_ = ar.apply_rope(q, sin, cos, torch.tensor([L - 1]))
    kr = ar.apply_rope(k, sin, cos, torch.arange(L))
    out = ar.llama_attention_core(qr_, kr, v, hq)
    np.savez_compressed(os.path.join(OUT, "attn_llama_decode.npz"), q=bf16_bits(q), k=bf16_bits(k), v=bf16_bits(v),
                        sin=bf16_bits(sin), cos=bf16_bits(cos), q_rope=bf16_bits(qr_), k_rope=bf16_bits(kr),
                        out=bf16_bits(out))
    # cached two-token forward at start_pos > 0 (mirrors architectures/llama.rs:3746-3785)
    q2 = torch.randn(1, 2, hq, d).bfloat16()
    out2 = ar.llama_attention_core(q2, kr, v, hq)
    np.savez_compressed(os.path.join(OUT, "attn_llama_cached2.npz"), q=bf16_bits(q2), k=bf16_bits(kr), v=bf16_bits(v),
                        out=bf16_bits(out2))
    # Qwen3.5 gated full attention decode: 8 q / 1 kv head, d=256
    hq, hkv, d, L = 8, 1, 256, 50
    q = torch.randn(1, 1, hq, d).bfloat16()
    gate = torch.randn(1, 1, hq, d).bfloat16()
    k = torch.randn(1, L, hkv, d).bfloat16()
    v = torch.randn(1, L, hkv, d).bfloat16()
    out = ar.qwen_gated_attention_core(q, gate, k, v, hq)
    np.savez_compressed(os.path.join(OUT, "attn_qwen_gated_decode.npz"), q=bf16_bits(q), gate=bf16_bits(gate),
                        k=bf16_bits(k), v=bf16_bits(v), out=bf16_bits(out))


def gdn_cases():
    from transformers.models.qwen3_5 import modeling_qwen3_5 as hf

    torch.manual_seed(11)
    b, h, t, d = 1, 2, 150, 128
    q = gr.l2_normalize(torch.randn(b, h, t, d))
    k = gr.l2_normalize(torch.randn(b, h, t, d))
    v = torch.randn(b, h, t, d)
    g = torch.nn.functional.logsigmoid(torch.randn(b, h, t))
    beta = torch.sigmoid(torch.randn(b, h, t))
    s0 = torch.randn(b, h, d, d) * 0.1
    tr = lambda x: x.transpose(1, 2).contiguous()  # HF layout is [B, T, H, *]; it scales q by d**-0.5 itself
    o_c, s_c = hf.torch_chunk_gated_delta_rule(tr(q), tr(k), tr(v), tr(g), tr(beta), chunk_size=64, initial_state=s0,
                                               output_final_state=True, use_qk_l2norm_in_kernel=False)
    o_r, s_r = hf.torch_recurrent_gated_delta_rule(tr(q), tr(k), tr(v), tr(g), tr(beta), initial_state=s0,
                                                   output_final_state=True, use_qk_l2norm_in_kernel=False)
    np.savez_compressed(os.path.join(OUT, "gdn_hf.npz"), q=q.numpy(), k=k.numpy(), v=v.numpy(), g=g.numpy(),
                        beta=beta.numpy(), s0=s0.numpy(), out_chunk=o_c.transpose(1, 2).float().numpy(),
                        state_chunk=s_c.float().numpy(), out_rec=o_r.transpose(1, 2).float().numpy(),
                        state_rec=s_r.float().numpy())


def attn_hf_cases():
    """Llama RoPE + eager attention and Qwen3.5 gated attention computed by `transformers` (imported, not restated)."""
    import types

    from transformers.models.llama import modeling_llama as ml
    from transformers.models.qwen3_5 import modeling_qwen3_5 as mq

    def hf_tables(dim, base, n_pos):
        # the inverse frequencies and angles as LlamaRotaryEmbedding forms them (fp32), cos / sin cast to the model dtype
        inv = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.int64).float() / dim))
        freqs = torch.arange(n_pos, dtype=torch.float32)[:, None] * inv[None, :]
        emb = torch.cat((freqs, freqs), dim=-1)
        return emb.cos().to(torch.bfloat16), emb.sin().to(torch.bfloat16)

    def causal_additive(q_len, kv_len):
        m = torch.zeros(q_len, kv_len)
        m.masked_fill_(torch.arange(kv_len)[None, :] > torch.arange(q_len)[:, None] + (kv_len - q_len), float("-inf"))
        return m[None, None]

    torch.manual_seed(21)
    # ---- Llama: 8 q / 2 kv heads, d = 128, 90 cached tokens; one decode token and a 5-token forward at start_pos 85
    hq, hkv, d, L = 8, 2, 128, 90
    cos, sin = hf_tables(d, 500000.0, 128)
    k = torch.randn(1, L, hkv, d).bfloat16()
    v = torch.randn(1, L, hkv, d).bfloat16()
    out = {"k": bf16_bits(k), "v": bf16_bits(v)}
    mod = types.SimpleNamespace(num_key_value_groups=hq // hkv, training=False)
    for name, ql in (("decode", 1), ("cached5", 5)):
        q = torch.randn(1, ql, hq, d).bfloat16()
        pos_q = torch.arange(L - ql, L)
        q_r, _ = ml.apply_rotary_pos_emb(q.transpose(1, 2), q.transpose(1, 2), cos[pos_q][None], sin[pos_q][None])
        k_r, _ = ml.apply_rotary_pos_emb(k.transpose(1, 2), k.transpose(1, 2), cos[:L][None], sin[:L][None])
        # fp32 operands: the reference upcasts q, K and V before the contraction (llama.rs:1044-1068)
        o, _ = ml.eager_attention_forward(mod, q_r.float(), k_r.float(), v.transpose(1, 2).float(), causal_additive(ql, L) if ql > 1 else None,
                                          scaling=d ** -0.5)
        out.update({f"q_{name}": bf16_bits(q), f"q_rope_{name}": bf16_bits(q_r.transpose(1, 2)), f"out_{name}": o.float().numpy()})
        out["k_rope"] = bf16_bits(k_r.transpose(1, 2))
    np.savez_compressed(os.path.join(OUT, "attn_hf_llama.npz"), **out)
    # ---- Qwen3.5 gated full attention: 8 q / 2 kv heads, d = 256, rotary 64, 70 cached tokens, decode and 4-token forward
    hq, hkv, d, rd, L = 8, 2, 256, 64, 70
    cos, sin = hf_tables(rd, 10000.0, 128)
    qn, kn = mq.Qwen3_5RMSNorm(d, eps=1e-6), mq.Qwen3_5RMSNorm(d, eps=1e-6)
    with torch.no_grad():
        qn.weight.copy_(0.1 * torch.randn(d)); kn.weight.copy_(0.1 * torch.randn(d))
    k_proj = torch.randn(1, L, hkv, d).bfloat16()
    v = torch.randn(1, L, hkv, d).bfloat16()
    mod = types.SimpleNamespace(num_key_value_groups=hq // hkv, training=False)
    out = {"k_proj": bf16_bits(k_proj), "v": bf16_bits(v), "q_norm_w": qn.weight.detach().numpy(), "k_norm_w": kn.weight.detach().numpy()}
    with torch.no_grad():
        for name, ql in (("decode", 1), ("cached4", 4)):
            q_proj = torch.randn(1, ql, hq, 2 * d).bfloat16()                    # per head: query | gate
            query, gate = torch.chunk(q_proj, 2, dim=-1)
            pos_q = torch.arange(L - ql, L)
            qs = qn(query).transpose(1, 2)
            ks = kn(k_proj).transpose(1, 2)
            qs_r, _ = mq.apply_rotary_pos_emb(qs, qs, cos[pos_q][None], sin[pos_q][None])
            ks_r, _ = mq.apply_rotary_pos_emb(ks, ks, cos[:L][None], sin[:L][None])
            o, _ = mq.eager_attention_forward(mod, qs_r, ks_r, v.transpose(1, 2), causal_additive(ql, L).bfloat16() if ql > 1 else None,
                                              scaling=d ** -0.5)
            o = o.reshape(1, ql, -1) * torch.sigmoid(gate.reshape(1, ql, -1))
            out.update({f"q_proj_{name}": bf16_bits(q_proj), f"q_rope_{name}": bf16_bits(qs_r.transpose(1, 2)), f"out_{name}": bf16_bits(o.reshape(1, ql, hq, d))})
            out["k_rope"] = bf16_bits(ks_r.transpose(1, 2))
    np.savez_compressed(os.path.join(OUT, "attn_hf_qwen.npz"), **out)


if __name__ == "__main__":
    quant_cases()
    attn_cases()
    attn_hf_cases()
    gdn_cases()
    for f in sorted(os.listdir(OUT)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(OUT, f)))
