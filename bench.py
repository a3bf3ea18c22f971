#!/usr/bin/env python
"""Benchmark of the decode-attention hot path (BASELINE.json configs[1]).

One step = one pass of the path over one batch: quantise-on-write of one new token per sequence into
the int8 KV cache, then ragged decode attention of the batch's 32 query tokens over their caches
(split-KV + log-sum-exp merge).  Batch 32, 32 q / 8 kv heads, head_dim 128, context lengths drawn
uniformly from 512..8192 (seed 1 + rank).  Synthetic N(0,1) data.  Inputs are larger than L2
(about 290 MB of KV per GPU against 126 MB), so no flush is needed between steps.

    python bench.py --gpus 1 --steps 2000 --warmup 20
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference --steps 3 --warmup 1     # the reference's CPU op sequence

Multi-GPU: sequences are independent (each owns its cache), so every rank decodes its own batch of
32 sequences with no data-path collective — weak scaling; the time is the max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BATCH, HQ, HKV, D = 32, 32, 8, 128
# ncu capture of decode_int8_tc_kernel on this workload: 289.97 MB read + 4.34 MB written for 289.31 MB algorithmic
NCU_TRAFFIC_PER_ALGO_BYTE = (289.973248 + 4.341504) / 289.309344
LAYOUTS = {"baseline": (128, 1), "reference": (64, 0)}  # (block, scale dtype: 0 = f32, 1 = f16)


def draw_lens(rank: int) -> list[int]:
    rng = np.random.default_rng(1 + rank)
    return [int(x) for x in rng.integers(512, 8193, size=BATCH)]


def rank_lens(rank: int, world: int) -> list[int]:
    """Context lengths of this rank's 32 sequences: the world's 32 * N sequences (the N = 1 draw first) are dealt
    length-balanced, 32 per GPU; at N = 1 this is the plain draw."""
    if world == 1:
        return draw_lens(0)
    from hyprstream_b200.sharded import balance_sequences

    pool = [l for r in range(world) for l in draw_lens(r)]
    return [pool[i] for i in balance_sequences(pool, world)[rank]]


def token_bytes(block: int, scale_f16: int) -> int:
    """Algorithmic bytes of one cached token, K + V: codes plus one scale per block."""
    return 2 * HKV * (D + (D // block) * (2 if scale_f16 else 4))


def step_bytes(lens: list[int], block: int, scale_f16: int) -> int:
    """Algorithmic bytes of one step: the cache as attended (L_r + 1 tokens per row) plus, per row, the query
    (8,192 B), the output (8,192 B), the new token read in bf16 (4,096 B) and written quantised."""
    tb = token_bytes(block, scale_f16)
    return sum(l + 1 for l in lens) * tb + len(lens) * (HQ * D * 2 * 2 + 2 * HKV * D * 2 + tb)


# --------------------------------------------------------------------------------------- clocks
class ClockSampler:
    """nvidia-smi sampled every 200 ms while the timed region runs (read-only query)."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.tmp,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            pass

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        self.proc.wait()
        self.tmp.flush()
        self.tmp.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.tmp.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        self.tmp.close()
        os.unlink(self.tmp.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------- CPU reference arm
def cpu_reference(lens: list[int], block: int, scale_f16: int, steps: int, warmup: int, sample_rows: int):
    """The reference's own CPU op sequence for this step, restated by the oracle: per row, dequantise the whole
    history (QuantizedTensor::to_tensor, kv_cache.rs:871-957), append the new token, right-pad to the longest row
    and stack, GQA-expand, additive mask, fp32 attention (llama.rs:710-844,1023-1119).  Timed on the host cores
    on the first `sample_rows` sequences of the batch.  Returns (seconds per step, bytes per step, description)."""
    from oracle import attention_ref as ar
    from oracle import quant_ref as qr

    rows = lens[:sample_rows]
    rng = np.random.default_rng(7)
    stored = []
    for l in rows:
        kv = []
        for _ in range(2):
            x = torch.from_numpy(rng.standard_normal((l, HKV, D)).astype(np.float32)).bfloat16().float().numpy()
            kv.append(qr.quantize(x, qr.INT8, block, bool(scale_f16)))
        stored.append(kv)
    q = torch.randn(len(rows), 1, HQ, D).bfloat16()
    k_new = torch.randn(len(rows), 1, HKV, D).bfloat16()
    v_new = torch.randn(len(rows), 1, HKV, D).bfloat16()

    def one_step():
        ks, vs = [], []
        for r, l in enumerate(rows):
            (kc, ka), (vc, va) = stored[r]
            kd = torch.from_numpy(qr.dequantize_np(kc, ka, qr.INT8, l * HKV * D, block)).to(torch.bfloat16).reshape(1, l, HKV, D)
            vd = torch.from_numpy(qr.dequantize_np(vc, va, qr.INT8, l * HKV * D, block)).to(torch.bfloat16).reshape(1, l, HKV, D)
            ks.append(torch.cat([kd, k_new[r:r + 1]], 1))
            vs.append(torch.cat([vd, v_new[r:r + 1]], 1))
        return ar.llama_batched_decode(q, ks, vs, rows, HQ)

    for _ in range(warmup):
        one_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return dt, step_bytes(rows, block, scale_f16), f"first {len(rows)} of {BATCH} sequences (lengths {rows}), {steps} steps"


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    block, sf16 = LAYOUTS[args.layout]
    lens = draw_lens(0)
    dt, nbytes, sample = cpu_reference(lens, block, sf16, args.steps, args.warmup, sample_rows=4)
    gbs = nbytes / dt / 1e9
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": "decode_attn_hbm_gbps", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "tokens_per_s": 4 / dt,
        "config": workload_config(args.layout, lens),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference is Rust on tch-rs and cannot be built here (no cargo); this arm times its ATen "
                "operator sequence restated op-for-op in torch on the host cores (oracle port)",
    }
    print(json.dumps(line))


def workload_config(layout: str, lens: list[int]) -> dict:
    block, sf16 = LAYOUTS[layout]
    return {"workload": "configs[1]: batched ragged decode attention over an int8 KV cache with quantise-on-write",
            "batch_per_gpu": BATCH, "q_heads": HQ, "kv_heads": HKV, "head_dim": D, "context_lens": "U{512..8192}",
            "sum_context": sum(lens), "kv_layout": f"{layout}: block {block}, {'f16' if sf16 else 'f32'} absmax",
            "partition": "sequences across GPUs (32 per GPU, dealt longest-first so the cached-token sums match), no collective",
            "l2": "inputs larger than L2 (KV bytes per GPU exceed 126 MB); no flush"}


# --------------------------------------------------------------------------------------- GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layout", default="baseline", choices=sorted(LAYOUTS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        run_reference_arm(args)
        return

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    from hyprstream_b200 import ffi, kv_cache as kc, ops

    block, sf16 = LAYOUTS[args.layout]
    lens = rank_lens(rank, world)
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    caches = []
    for l in lens:
        c = kc.LayerKVCache(8192 + 1024, kc.KVQuantType.INT8, HKV, D, dev, block=block, scale_dtype=sf16)
        k = torch.randn(1, l, HKV, D, device=dev, generator=gen, dtype=torch.float32).bfloat16()
        v = torch.randn(1, l, HKV, D, device=dev, generator=gen, dtype=torch.float32).bfloat16()
        c._ensure_capacity(l + 1)
        c.update(k, v, 0)
        caches.append(c)
    view, keep = kc.make_view(caches)
    dst_pos = torch.tensor(lens, dtype=torch.int32, device=dev)
    seq_lens = dst_pos + 1
    q = torch.randn(BATCH, HQ, D, device=dev, generator=gen, dtype=torch.float32).bfloat16()
    k_new = torch.randn(BATCH, 1, HKV, D, device=dev, generator=gen, dtype=torch.float32).bfloat16()
    v_new = torch.randn(BATCH, 1, HKV, D, device=dev, generator=gen, dtype=torch.float32).bfloat16()
    out = torch.empty_like(q)
    ws = ops.decode_workspace(BATCH, HQ, D, dev)
    nbytes = step_bytes(lens, block, sf16)

    def step():
        ops.kv_quantize_write(view, k_new, v_new, dst_pos)
        ops.decode_attention(q, view, seq_lens, out=out, workspace=ws)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    # ---- device-resident timing -------------------------------------------------------------
    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = ffi.launch_count()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    launches = ffi.launch_count() - launches0  # kernels of the library inside the timed region (this rank)
    ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    total_bytes = sum_over_ranks(float(nbytes))
    clocks = sampler.stop() if sampler else None

    # ---- dominant kernel alone (the split-KV decode kernel), CUDA events on the launch stream ----
    ffi.set_profiling(True)
    kms = []
    for _ in range(min(args.steps, 20)):
        step()
        kms.append(ffi.last_kernel_ms())
    ffi.set_profiling(False)
    kernel_ms = sum(kms) / len(kms)
    kernel_bytes = sum(l + 1 for l in lens) * token_bytes(block, sf16) + BATCH * HQ * D * 2  # cache + q; partials excluded

    # ---- end to end through the public API with host buffers ----------------------------------
    # the step's inputs (q, new K, new V) sit back to back in one pinned host buffer and travel in one copy
    sizes = [q.numel(), k_new.numel(), v_new.numel()]
    host_in = torch.empty(sum(sizes), dtype=torch.bfloat16).pin_memory()
    dev_in = torch.empty(sum(sizes), dtype=torch.bfloat16, device=dev)
    q_h, k_h, v_h = (h.view_as(t) for h, t in zip(host_in.split(sizes), (q, k_new, v_new)))
    for h, t in zip((q_h, k_h, v_h), (q, k_new, v_new)):
        h.copy_(t)
    q_d, k_d, v_d = (d_.view_as(t) for d_, t in zip(dev_in.split(sizes), (q, k_new, v_new)))
    out_h = torch.empty_like(q_h).pin_memory()

    def e2e_step():
        dev_in.copy_(host_in, non_blocking=True)
        ops.kv_quantize_write(view, k_d, v_d, dst_pos)
        ops.decode_attention(q_d, view, seq_lens, out=out, workspace=ws)
        out_h.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the host consumes the result before the next step

    for _ in range(args.warmup):
        e2e_step()
    barrier()
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    h2d = q_h.numel() * 2 + k_h.numel() * 2 + v_h.numel() * 2
    d2h = out_h.numel() * 2
    torch.cuda.synchronize()
    dev_err = ffi.take_device_error()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_src = "measured (MEASURED_PEAKS.json hbm_gbs, burst copy)" if "hbm_gbs" in peaks else "fallback 6650 GB/s"
    achieved = kernel_bytes / (kernel_ms * 1e-3) / 1e9

    line = {
        "metric": "decode_attn_hbm_gbps", "value": total_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "tokens_per_s": BATCH * world / (ms * 1e-3),
        "config": workload_config(args.layout, lens),
        "e2e": {"value": total_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
                "tokens_per_s": BATCH * world / (e2e_ms * 1e-3), "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "kernel": "decode split-KV kernel (rank 0)", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src, "kernel_ms": kernel_ms,
                     "bytes_per_launch": kernel_bytes,
                     # dram__bytes_read.sum + dram__bytes_write.sum of one launch on this workload
                     # (profiles/decode_int8_tc_config2.md), scaled by this run's algorithmic bytes
                     "traffic": NCU_TRAFFIC_PER_ALGO_BYTE * kernel_bytes if args.layout == "baseline" else None},
        "clocks": clocks, "device_error_flags": dev_err,
    }
    if world == 1 and not args.no_cpu_baseline:
        dt, cb, sample = cpu_reference(lens, block, sf16, steps=2, warmup=1, sample_rows=4)
        line["cpu_baseline"] = {"value": cb / dt / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": sample, "ms_per_step": dt * 1e3}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
