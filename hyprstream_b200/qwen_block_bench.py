"""BASELINE.json configs[4] as a whole: one Qwen3.5-style block = 3 gated-DeltaNet layers + 1 gated full-attention layer,
everything between the layers' projections (the GEMMs stay with the host framework and are not timed): prefill of
4 x 32768 tokens, then decode steps at batch 64 against 32768 + t cached tokens.  Inputs are random "projection
outputs" of the right shapes and dtypes (synthetic data, random init).  Prints one JSON line.

    python -m hyprstream_b200.qwen_block_bench [--prefill-tokens 32768] [--decode-steps 256] [--decode-batch 64]

Per DeltaNet layer: hs_gdn_prologue -> hs_gdn_chunk_prefill (prefill) or hs_gdn_recurrent (decode) -> hs_gdn_epilogue.
Full-attention layer: hs_qk_norm_rope (q with gate split, k) -> hs_kv_quantize_write (int8, block 128, f16 scales) ->
hs_attn_prefill_causal (prefill) or hs_attn_decode (decode), with the output gate.
"""
import argparse
import json

import torch

from . import ffi, kv_cache as kc, ops

NK, NV, HD, KS = 16, 32, 128, 4                 # DeltaNet: 16 k/q heads, 32 v heads, d = 128, conv kernel 4
CONV_DIM = (2 * NK + NV) * HD
HQ, HKV, D, RD = 16, 2, 256, 64                 # full attention: 16 q / 2 kv heads, d = 256, rotary 64
N_GDN = 3


def ev():
    return torch.cuda.Event(enable_timing=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--prefill-batch", type=int, default=4)
    ap.add_argument("--prefill-tokens", type=int, default=32768)
    ap.add_argument("--decode-batch", type=int, default=64)
    ap.add_argument("--decode-steps", type=int, default=256)
    ap.add_argument("--context", type=int, default=32768)
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(4)
    rnd = lambda *shape: torch.randn(*shape, device=dev, generator=g)  # noqa: E731
    res = {"workload": "configs[4]: Qwen3.5-style block, 3 gated-DeltaNet layers + 1 gated full-attention layer (projections not timed)"}

    conv_w = [(rnd(CONV_DIM, 1, KS) * 0.5).bfloat16() for _ in range(N_GDN)]
    neg_a = [-torch.rand(NV, device=dev, generator=g) for _ in range(N_GDN)]
    dt_b = [rnd(NV) * 0.3 for _ in range(N_GDN)]
    norm_w = [1.0 + 0.1 * rnd(HD) for _ in range(N_GDN)]
    qn_w, kn_w = 0.1 * rnd(D), 0.1 * rnd(D)
    sin = torch.sin(torch.arange(a.context + a.decode_steps + 8, device=dev).float()[:, None] * torch.arange(RD // 2, device=dev).float()[None, :] * 1e-3).bfloat16()
    cos = torch.cos(torch.arange(a.context + a.decode_steps + 8, device=dev).float()[:, None] * torch.arange(RD // 2, device=dev).float()[None, :] * 1e-3).bfloat16()

    # ------------------------------------------------------------------ prefill
    b, t = a.prefill_batch, a.prefill_tokens
    x = rnd(b, t, CONV_DIM).bfloat16()
    z = rnd(b, t, NV, HD).bfloat16()
    a_in, b_in = rnd(b, t, NV).bfloat16(), rnd(b, t, NV).bfloat16()
    q_full = rnd(b * t, HQ * 2 * D).bfloat16()
    k_proj, v_proj = rnd(b * t, HKV * D).bfloat16(), rnd(b, t, HKV, D).bfloat16()
    pos = torch.arange(t, device=dev, dtype=torch.int32).repeat(b)
    conv = [torch.zeros(b, CONV_DIM, KS - 1, dtype=torch.bfloat16, device=dev) for _ in range(N_GDN)]
    rec = [torch.zeros(b, NV, HD, HD, device=dev) for _ in range(N_GDN)]
    caches = [kc.LayerKVCache(t, kc.KVQuantType.INT8, HKV, D, dev, block=128, scale_dtype=ffi.SCALE_F16) for _ in range(b)]
    for c in caches:
        c._ensure_capacity(t)
    view, keep = kc.make_view(caches)
    zeros = torch.zeros(b, dtype=torch.int32, device=dev)

    def gdn_layer_prefill(i):
        q, k, v, gg, beta = ops.gdn_prologue(x, conv_w[i], conv[i], False, a_in, b_in, neg_a[i], dt_b[i], NK, NV)
        o = ops.gdn_chunk_prefill(q, k, v, gg, beta, rec[i])
        return ops.gdn_epilogue(o, z, norm_w[i], 1e-6)

    def attn_layer_prefill():
        query, gate = ops.qk_norm_rope(q_full, HQ, D, qn_w, 1e-6, True, sin, cos, pos, RD, with_gate=True)
        k = ops.qk_norm_rope(k_proj, HKV, D, kn_w, 1e-6, True, sin, cos, pos, RD)
        ops.kv_quantize_write(view, k.view(b, t, HKV, D), v_proj, zeros)
        return ops.prefill_attention(query.view(b, t, HQ, D), k.view(b, t, HKV, D), v_proj, gate=gate.view(b, t, HQ, D))

    for i in range(N_GDN):   # warm-up (also builds tensor maps, sets attributes)
        gdn_layer_prefill(i)
    attn_layer_prefill()
    for r_ in rec:
        r_.zero_()
    torch.cuda.synchronize()
    e = [ev() for _ in range(3)]
    e[0].record()
    for i in range(N_GDN):
        gdn_layer_prefill(i)
    e[1].record()
    attn_layer_prefill()
    e[2].record()
    torch.cuda.synchronize()
    gdn_ms, attn_ms = e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2])
    res["prefill"] = {"batch": b, "tokens": t, "gdn_layers_ms": gdn_ms, "full_attention_layer_ms": attn_ms, "block_ms": gdn_ms + attn_ms,
                      "tokens_per_s": b * t / (gdn_ms + attn_ms) * 1e3}
    del x, z, a_in, b_in, q_full, k_proj, v_proj, caches, view, keep, conv, rec
    torch.cuda.empty_cache()

    # ------------------------------------------------------------------ decode
    b, L = a.decode_batch, a.context
    caches = []
    cap = (L + a.decode_steps + 8 + 1023) // 1024 * 1024  # whole 1024-token growth chunks (kv_cache.rs:700)
    for s in range(b):
        c = kc.LayerKVCache(cap, kc.KVQuantType.INT8, HKV, D, dev, block=128, scale_dtype=ffi.SCALE_F16)
        for t0 in range(0, L, 8192):
            n = min(8192, L - t0)
            c.update(rnd(1, n, HKV, D).bfloat16(), rnd(1, n, HKV, D).bfloat16(), t0)
        c._ensure_capacity(cap)
        caches.append(c)
    view, keep = kc.make_view(caches)
    x = rnd(b, 1, CONV_DIM).bfloat16()
    z = rnd(b, 1, NV, HD).bfloat16()
    a_in, b_in = rnd(b, 1, NV).bfloat16(), rnd(b, 1, NV).bfloat16()
    q_full = rnd(b, HQ * 2 * D).bfloat16()
    k_proj, v_proj = rnd(b, HKV * D).bfloat16(), rnd(b, 1, HKV, D).bfloat16()
    conv = [rnd(b, CONV_DIM, KS - 1).bfloat16() for _ in range(N_GDN)]
    rec = [rnd(b, NV, HD, HD) * 0.1 for _ in range(N_GDN)]
    ws = ops.decode_workspace(b, HQ, D, dev)
    lens = torch.full((b,), L, dtype=torch.int32, device=dev)

    def decode_step():
        for i in range(N_GDN):
            q, k, v, gg, beta = ops.gdn_prologue(x, conv_w[i], conv[i], True, a_in, b_in, neg_a[i], dt_b[i], NK, NV)
            o = ops.gdn_recurrent(q, k, v, gg, beta, rec[i])
            ops.gdn_epilogue(o, z, norm_w[i], 1e-6)
        query, gate = ops.qk_norm_rope(q_full, HQ, D, qn_w, 1e-6, True, sin, cos, lens, RD, with_gate=True)
        k = ops.qk_norm_rope(k_proj, HKV, D, kn_w, 1e-6, True, sin, cos, lens, RD)
        ops.kv_quantize_write(view, k.view(b, 1, HKV, D), v_proj, lens)
        lens.add_(1)
        return ops.decode_attention(query, view, lens, gate=gate, workspace=ws)

    for _ in range(3):
        decode_step()
    torch.cuda.synchronize()
    e0, e1 = ev(), ev()
    e0.record()
    for _ in range(a.decode_steps):
        decode_step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.decode_steps
    kv_bytes = b * (L + 3 + a.decode_steps / 2) * 2 * HKV * (D + (D // 128) * 2)
    state_bytes = N_GDN * 2 * b * NV * HD * HD * 4
    res["decode"] = {"batch": b, "context": L, "steps": a.decode_steps, "ms_per_step": ms, "tokens_per_s": b / ms * 1e3,
                     "algorithmic_bytes_per_step": kv_bytes + state_bytes, "hbm_gbps": (kv_bytes + state_bytes) / ms / 1e6}
    res["device_error_flags"] = ffi.take_device_error()
    print(json.dumps(res))


if __name__ == "__main__":
    main()
