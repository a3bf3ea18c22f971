"""Times causal prefill (BASELINE.json configs[3]: 8 x 8192 tokens, 32 q / 8 kv heads, d=128, bf16) with
quantise-on-write of K/V into the int8 cache; prints one JSON line.  Useful FLOPs are the causal half:
4 * B * Hq * D * T(T+1)/2.

    python -m hyprstream_b200.prefill_bench [--batch 8] [--tokens 8192] [--iters 10]
"""
import argparse
import json

import torch

from . import ffi, kv_cache as kc, ops


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    hq, hkv, d = 32, 8, 128
    g = torch.Generator(device=dev).manual_seed(3)
    q = torch.randn(a.batch, a.tokens, hq, d, device=dev, generator=g).bfloat16()
    k = torch.randn(a.batch, a.tokens, hkv, d, device=dev, generator=g).bfloat16()
    v = torch.randn(a.batch, a.tokens, hkv, d, device=dev, generator=g).bfloat16()
    caches = [kc.LayerKVCache(a.tokens, kc.KVQuantType.INT8, hkv, d, dev) for _ in range(a.batch)]
    for c in caches:
        c._ensure_capacity(a.tokens)
    view, keep = kc.make_view(caches)
    zeros = torch.zeros(a.batch, dtype=torch.int32, device=dev)

    def step():
        out = ops.prefill_attention(q, k, v)
        ops.kv_quantize_write(view, k, v, zeros)
        return out

    for _ in range(a.warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.iters
    ffi.set_profiling(True)
    ops.prefill_attention(q, k, v)
    kms = ffi.last_kernel_ms()
    ffi.set_profiling(False)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(a.iters):
        ops.kv_quantize_write(view, k, v, zeros)
    e1.record()
    torch.cuda.synchronize()
    wms = e0.elapsed_time(e1) / a.iters
    wbytes = 2 * a.batch * a.tokens * hkv * (d * 2 + d + (d // 128) * 2)  # bf16 in, int8 codes + f16 scale per 128 out, K and V
    flops = 4.0 * a.batch * hq * d * a.tokens * (a.tokens + 1) / 2
    print(json.dumps({"workload": "configs[3] causal prefill + int8 quantise-on-write", "batch": a.batch, "tokens": a.tokens,
                      "ms_per_step": ms, "attn_kernel_ms": kms, "useful_tflops_step": flops / ms / 1e9,
                      "useful_tflops_kernel": flops / kms / 1e9,
                      "kv_write_ms": wms, "kv_write_gbps": wbytes / wms / 1e6, "device_error_flags": ffi.take_device_error()}))


if __name__ == "__main__":
    main()
