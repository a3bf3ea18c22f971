"""Times the DeltaNet prologue (conv1d + SiLU + split + L2 norm + gates) and epilogue (RMSNormGated) kernels at the
BASELINE.json configs[4] sizes (16 k/q heads, 32 v heads, d=128, conv kernel 4): prefill 4 x 32768 tokens and decode at
batch 64.  Prints one JSON line with time and achieved HBM bandwidth (algorithmic bytes: every input read once, every
output written once).

    python -m hyprstream_b200.gdn_edges_bench [--tokens 32768] [--iters 10]
"""
import argparse
import json

import torch

from . import ffi, ops

NK, NV, HD, KS = 16, 32, 128, 4
CONV_DIM = (2 * NK + NV) * HD


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


def case(b, t, iters, dev):
    g = torch.Generator(device=dev).manual_seed(7)
    x = torch.randn(b, t, CONV_DIM, device=dev, generator=g).bfloat16()
    w = (torch.randn(CONV_DIM, 1, KS, device=dev, generator=g) * 0.5).bfloat16()
    a = torch.randn(b, t, NV, device=dev, generator=g).bfloat16()
    bb = torch.randn(b, t, NV, device=dev, generator=g).bfloat16()
    neg_a = -torch.rand(NV, device=dev, generator=g)
    dt = torch.randn(NV, device=dev, generator=g)
    conv = torch.zeros(b, CONV_DIM, KS - 1, dtype=torch.bfloat16, device=dev)
    o = torch.randn(b, t, NV, HD, device=dev, generator=g)
    z = torch.randn(b, t, NV, HD, device=dev, generator=g).bfloat16()
    nw = torch.ones(HD, device=dev)
    pro_ms = timed(lambda: ops.gdn_prologue(x, w, conv, True, a, bb, neg_a, dt, NK, NV), 2, iters)
    epi_ms = timed(lambda: ops.gdn_epilogue(o, z, nw, 1e-6), 2, iters)
    tok = b * t
    pro_bytes = tok * (CONV_DIM * 2 + CONV_DIM * 4 + NV * (2 + 2 + 4 + 4)) + 2 * b * CONV_DIM * (KS - 1) * 2
    epi_bytes = tok * NV * HD * (4 + 2 + 2)
    return {"batch": b, "tokens": t, "prologue_ms": pro_ms, "prologue_gbps": pro_bytes / pro_ms / 1e6,
            "epilogue_ms": epi_ms, "epilogue_gbps": epi_bytes / epi_ms / 1e6}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    res = {"workload": "configs[4] gated DeltaNet prologue / epilogue", "prefill": case(4, a.tokens, a.iters, dev),
           "decode": case(64, 1, 200, dev), "device_error_flags": ffi.take_device_error()}
    print(json.dumps(res))


if __name__ == "__main__":
    main()
