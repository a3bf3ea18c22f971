"""Generates the committed fixtures in tests/golden/ (run from the repository root:
``python tests/golden/make_golden.py``).

The reference holds no golden vectors for this path, so these fixtures are made here:
* quant_*.npz       — seeded and hand-built edge-case inputs with the codes/scales of the written
                      quantiser specification (oracle/quant_spec.c), both restatements agreeing;
* attn_*.npz        — small seeded attention cases with the outputs of the ATen op-for-op
                      restatement (oracle/attention_ref.py);
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


if __name__ == "__main__":
    quant_cases()
    attn_cases()
    gdn_cases()
    for f in sorted(os.listdir(OUT)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(OUT, f)))
