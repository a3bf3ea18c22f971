"""Times the gated-DeltaNet kernels on BASELINE.json configs[4] geometry (16 k/q heads, 32 v heads, d=128):
decode = one recurrent step at batch 64 (state read + written once: 2*64*32*128*128*4 = 268,435,456 B),
prefill = 4 x T tokens through the same recurrence.  Prints one JSON line.

    python -m hyprstream_b200.gdn_bench [--tokens 32768] [--iters 20]
"""
import argparse
import json

import torch

from . import ffi, ops


def _inputs(b, t, dev, seed):
    g = torch.Generator(device=dev).manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(b, t, 16, 128, device=dev, generator=g), dim=-1) * 128 ** -0.5
    k = torch.nn.functional.normalize(torch.randn(b, t, 16, 128, device=dev, generator=g), dim=-1)
    v = torch.randn(b, t, 32, 128, device=dev, generator=g)
    gl = torch.nn.functional.logsigmoid(torch.randn(b, t, 32, device=dev, generator=g))
    beta = torch.sigmoid(torch.randn(b, t, 32, device=dev, generator=g))
    return q, k, v, gl, beta


def _time(fn, iters, warmup=3):
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
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    q, k, v, g, beta = _inputs(64, 1, dev, 1)
    states = [torch.randn(64, 32, 128, 128, device=dev) * 0.1 for _ in range(2)]  # 2 x 134 MB: alternate so L2 cannot hold the state
    i = [0]

    def dec():
        i[0] ^= 1
        ops.gdn_recurrent(q, k, v, g, beta, states[i[0]])

    dec_ms = _time(dec, a.iters)
    dec_bytes = 2 * 64 * 32 * 128 * 128 * 4
    q, k, v, g, beta = _inputs(4, a.tokens, dev, 2)
    st = torch.zeros(4, 32, 128, 128, device=dev)
    pre_ms = _time(lambda: ops.gdn_recurrent(q, k, v, g, beta, st), max(2, a.iters // 10), warmup=1)
    st2 = torch.zeros(4, 32, 128, 128, device=dev)
    chunk_ms = _time(lambda: ops.gdn_chunk_prefill(q, k, v, g, beta, st2), max(2, a.iters // 5), warmup=1)
    flops_chunked = 11.7e6 * (a.tokens / 64) * 32 * 4  # the chunked algorithm's count (qwen3_5.rs:342-498), for reference
    print(json.dumps({"workload": "configs[4] gated DeltaNet", "decode_batch": 64, "decode_ms": dec_ms,
                      "decode_state_gbps": dec_bytes / dec_ms / 1e6, "prefill_tokens": a.tokens, "prefill_batch": 4,
                      "prefill_fp32_rule_ms": pre_ms, "prefill_fp32_rule_tokens_per_s": 4 * a.tokens / pre_ms * 1e3,
                      "prefill_chunked_ms": chunk_ms, "prefill_chunked_tokens_per_s": 4 * a.tokens / chunk_ms * 1e3,
                      "prefill_chunked_tflops_at_c64_count": flops_chunked / chunk_ms / 1e9, "device_error_flags": ffi.take_device_error()}))


if __name__ == "__main__":
    main()
