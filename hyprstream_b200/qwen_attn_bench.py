"""Times the gated full-attention layer of BASELINE.json configs[4] (Qwen3.5 shape: 16 q / 2 kv heads,
head_dim 256, int8 KV cache, output gate): causal prefill of 4 x 32768 tokens with quantise-on-write,
then decode at batch 64 against 32768 cached tokens per sequence.  Prints one JSON line.

    python -m hyprstream_b200.qwen_attn_bench [--prefill-tokens 32768] [--decode-batch 64] [--context 32768]

Algorithmic figures: prefill FLOPs (causal half) 4 * B * Hq * D * T(T+1)/2; decode bytes per cached token
2 * Hkv * (D + scale bytes) (block 128, f16 absmax: 2 * 2 * (256 + 4) = 1040 B).
"""
import argparse
import json

import torch

from . import ffi, kv_cache as kc, ops

HQ, HKV, D = 16, 2, 256


def timed(fn, warmup, iters):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--prefill-batch", type=int, default=4)
    ap.add_argument("--prefill-tokens", type=int, default=32768)
    ap.add_argument("--decode-batch", type=int, default=64)
    ap.add_argument("--context", type=int, default=32768)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--decode-iters", type=int, default=50)
    ap.add_argument("--skip-prefill", action="store_true")
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    res = {"workload": "configs[4] gated full attention (16 q / 2 kv heads, d=256, int8 KV)"}

    if not a.skip_prefill:
        b, t = a.prefill_batch, a.prefill_tokens
        g = torch.Generator(device=dev).manual_seed(4)
        q = torch.randn(b, t, HQ, D, device=dev, generator=g).bfloat16()
        k = torch.randn(b, t, HKV, D, device=dev, generator=g).bfloat16()
        v = torch.randn(b, t, HKV, D, device=dev, generator=g).bfloat16()
        gate = torch.randn(b, t, HQ, D, device=dev, generator=g).bfloat16()
        caches = [kc.LayerKVCache(t, kc.KVQuantType.INT8, HKV, D, dev, block=128, scale_dtype=ffi.SCALE_F16) for _ in range(b)]
        for c in caches:
            c._ensure_capacity(t)
        view, keep = kc.make_view(caches)
        zeros = torch.zeros(b, dtype=torch.int32, device=dev)

        def pstep():
            out = ops.prefill_attention(q, k, v, gate=gate)
            ops.kv_quantize_write(view, k, v, zeros)
            return out

        ms = timed(pstep, 1, a.iters)
        flops = 4.0 * b * HQ * D * t * (t + 1) / 2
        res.update({"prefill_batch": b, "prefill_tokens": t, "prefill_ms": ms, "prefill_useful_tflops": flops / ms / 1e9})
        del q, k, v, gate, caches, view, keep
        torch.cuda.empty_cache()

    b, L = a.decode_batch, a.context
    caches = []
    for s in range(b):
        g = torch.Generator(device=dev).manual_seed(100 + s)
        c = kc.LayerKVCache(L + 256, kc.KVQuantType.INT8, HKV, D, dev, block=128, scale_dtype=ffi.SCALE_F16)
        for t0 in range(0, L, 8192):
            n = min(8192, L - t0)
            c.update(torch.randn(1, n, HKV, D, device=dev, generator=g).bfloat16(),
                     torch.randn(1, n, HKV, D, device=dev, generator=g).bfloat16(), t0)
        c._ensure_capacity(L + 1)
        caches.append(c)
    view, keep = kc.make_view(caches)
    lens = torch.full((b,), L, dtype=torch.int32, device=dev)
    g = torch.Generator(device=dev).manual_seed(9)
    q = torch.randn(b, HQ, D, device=dev, generator=g).bfloat16()
    gate = torch.randn(b, HQ, D, device=dev, generator=g).bfloat16()
    kn = torch.randn(b, 1, HKV, D, device=dev, generator=g).bfloat16()
    vn = torch.randn(b, 1, HKV, D, device=dev, generator=g).bfloat16()
    ws = ops.decode_workspace(b, HQ, D, dev)
    lens1 = lens + 1

    def dstep():
        ops.kv_quantize_write(view, kn, vn, lens)
        return ops.decode_attention(q, view, lens1, gate=gate, workspace=ws)

    ms = timed(dstep, 5, a.decode_iters)
    tok_bytes = 2 * HKV * (D + (D // 128) * 2)
    total = b * (L + 1) * tok_bytes
    res.update({"decode_batch": b, "context": L, "decode_ms": ms, "decode_gbps": total / ms / 1e6,
                "decode_tokens_per_s": b / ms * 1e3, "device_error_flags": ffi.take_device_error()})
    print(json.dumps(res))


if __name__ == "__main__":
    main()
