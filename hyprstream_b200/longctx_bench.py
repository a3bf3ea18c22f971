"""Long-context decode over a 4-bit NF4 KV cache sharded by KV length (BASELINE.json configs[2]).

Batch 4, 32 q / 8 kv heads, d=128, context 131072 tokens per sequence, NF4 codes with an f16 absmax per
block of 64; the KV length is cut into N contiguous page-aligned shards, one per GPU; each step is
local decode -> NCCL all-gather of (o, lse) -> log-sum-exp merge.  Strong scaling (total work fixed).

    python -m hyprstream_b200.longctx_bench                      # 1 GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m hyprstream_b200.longctx_bench --steps 50
    ... --check --context 4096      # also compare with an unsharded decode of the same cache on every rank

Prints one JSON line on rank 0.  Algorithmic bytes per step: B * L * 2 * Hkv * (D/2 + (D/64)*2) = B * L * 1088.
"""
import argparse
import json
import os

import torch
import torch.distributed as dist

from . import ffi, kv_cache as kc, ops, sharded

B, HQ, HKV, D = 4, 32, 8, 128


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--context", type=int, default=131072)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--kind", default="nf4", choices=["nf4", "int8"])
    ap.add_argument("--check", action="store_true")
    a = ap.parse_args()
    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    kind = kc.KVQuantType.NF4 if a.kind == "nf4" else kc.KVQuantType.INT8
    start, end = sharded.shard_bounds(a.context, world)[rank]
    n_local = end - start
    # every rank draws the same full-length stream so that a check against the unsharded cache is possible
    caches, full = [], []
    for s in range(B):
        g = torch.Generator(device=dev).manual_seed(1000 + s)
        c = kc.LayerKVCache(max(n_local, 1), kind, HKV, D, dev, block=64, scale_dtype=ffi.SCALE_F16)
        cf = kc.LayerKVCache(a.context, kind, HKV, D, dev, block=64, scale_dtype=ffi.SCALE_F16) if a.check else None
        c._ensure_capacity(max(n_local, 1))
        for t0 in range(0, a.context, 8192):  # generate in slabs; keep only this rank's slice
            t1 = min(a.context, t0 + 8192)
            k = torch.randn(1, t1 - t0, HKV, D, device=dev, generator=g).bfloat16()
            v = torch.randn(1, t1 - t0, HKV, D, device=dev, generator=g).bfloat16()
            lo, hi = max(t0, start), min(t1, end)
            if lo < hi:
                c.update(k[:, lo - t0:hi - t0].contiguous(), v[:, lo - t0:hi - t0].contiguous(), lo - start)
            if cf is not None:
                cf.update(k, v, t0)
        caches.append(c)
        full.append(cf)
    view, keep = kc.make_view(caches)
    lens = torch.full((B,), n_local, dtype=torch.int32, device=dev)
    q = torch.randn(B, HQ, D, device=dev, generator=torch.Generator(device=dev).manual_seed(7)).bfloat16()

    dec = sharded.ShardedDecoder(B, HQ, D, dev) if world > 1 else None

    def eager_step():
        if world == 1:
            return ops.decode_attention(q, view, lens)
        return dec.step(q, view, lens)

    step = eager_step

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(a.warmup):
        out = step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        out = step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / a.steps
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    check = None
    if a.check:
        fview, fkeep = kc.make_view(full)
        ref = ops.decode_attention(q, fview, torch.full((B,), a.context, dtype=torch.int32, device=dev))
        torch.cuda.synchronize()
        diff = (out.float() - ref.float()).abs().max()
        if world > 1:
            dist.all_reduce(diff, op=dist.ReduceOp.MAX)
        check = float(diff.item())
    err = ffi.take_device_error()
    if rank == 0:
        tok_bytes = 2 * HKV * (D // 2 + (D // 64) * 2) if a.kind == "nf4" else 2 * HKV * (D + (D // 64) * 2)
        total = B * a.context * tok_bytes
        print(json.dumps({"workload": "configs[2]: long-context decode, KV-length shards + all-gather(o, lse) + LSE merge",
                          "kind": a.kind, "n_gpus": world, "context": a.context, "batch": B, "ms_per_step": ms,
                          "aggregate_gbps": total / ms / 1e6, "per_gpu_gbps": total / world / ms / 1e6,
                          "tokens_per_s": B / ms * 1e3, "collective_bytes_per_gpu": B * HQ * (D + 1) * 4,
                          "max_abs_vs_unsharded": check, "device_error_flags": err, "scaling": "strong"}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
