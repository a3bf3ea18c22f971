#!/usr/bin/env python
"""Benchmark of the attention + quantised-KV-cache hot path.

Headline (the line's metric): batched ragged decode attention over an int8 KV cache with quantise-on-write -
batch 32, 32 q / 8 kv heads, head_dim 128, context lengths drawn uniformly from 512..8192.  One step = one pass of the
path over one batch: the new token of every sequence is quantised into its cache, then the batch's 32 query tokens are
attended over their caches (split-KV + log-sum-exp merge inside one kernel).  Synthetic N(0,1) data.  The KV bytes per
GPU (about 290 MB) exceed L2 (126 MB), so no flush is needed between steps.

The same JSON line carries, measured after the headline's timed regions:
  parity     the timed configuration's own output against an fp32 recomputation over the dequantised cache (plain torch
             ops on the GPU) and the stored codes of the written tokens against the CPU oracle quantiser;
  secondary  the other workloads the metric names: long-context NF4 decode with the KV length sharded over the run's
             GPUs (collective form and one-launch peer-store form), causal prefill 8 x 8192 with quantise-on-write
             (TFLOP/s), and the Qwen3.5-style block (3 gated-DeltaNet layers + 1 gated full-attention layer) prefill
             and decode.  These are strong-scaling: the workload is fixed and dealt over the GPUs.

    python bench.py --gpus 1 --steps 2000 --warmup 20
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference --steps 3 --warmup 1     # the reference's CPU op sequence (oracle port)
    python bench.py --config 3|4|5                            # one of the secondary workloads alone, as its own line

Multi-GPU, headline: sequences are independent (each owns its cache), so every rank decodes its own batch of 32
sequences with no data-path collective - weak scaling; the time is the max over ranks.
"""
from __future__ import annotations

import argparse
import json
import math
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
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the decode kernel on the headline workload (one ncu
# capture, --clock-control none) over that launch's algorithmic bytes
NCU_TRAFFIC_PER_ALGO_BYTE = (290.052413 + 1.588520) / 289.309344
NCU_TRAFFIC_SOURCE = ("one ncu capture of this kernel (the one-launch step: new tokens written, cache streamed, partials merged) on this "
                      "workload, averaged over 38 launches (dram__bytes_read.sum + dram__bytes_write.sum per launch: 290.05 MB + 1.59 MB "
                      "for 289.31 MB algorithmic), scaled by this run's algorithmic bytes")
LAYOUTS = {"baseline": (128, 1), "reference": (64, 0)}  # (block, scale dtype: 0 = f32, 1 = f16)
MAX_ABS_TOL, MEAN_ABS_TOL = 2e-2, 2e-3                  # acceptance: bf16 attention outputs vs an fp32 recomputation


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


def token_bytes(block: int, scale_f16: int, hkv: int = HKV, d: int = D) -> int:
    """Algorithmic bytes of one cached int8 token, K + V: codes plus one scale per block."""
    return 2 * hkv * (d + (d // block) * (2 if scale_f16 else 4))


def step_bytes(lens: list[int], block: int, scale_f16: int) -> int:
    """Algorithmic bytes of one step: the cache as attended (L_r + 1 tokens per row) plus, per row, the query
    (8,192 B), the output (8,192 B), the new token read in bf16 (4,096 B) and written quantised."""
    tb = token_bytes(block, scale_f16)
    return sum(l + 1 for l in lens) * tb + len(lens) * (HQ * D * 2 * 2 + 2 * HKV * D * 2 + tb)


def load_peaks() -> dict:
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        return {}


# --------------------------------------------------------------------------------------- clocks
class ClockSampler:
    """nvidia-smi sampled every 100 ms while the timed region runs (read-only query)."""
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


def host_threads() -> int:
    """All the host threads this process may use (the launcher of a multi-rank run sets OMP_NUM_THREADS=1, which is
    not what a CPU baseline should run with)."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(n, 1))
    return torch.get_num_threads()


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    cores = host_threads()
    block, sf16 = LAYOUTS[args.layout]
    lens = rank_lens(0, world)  # the same lengths rank 0 of the GPU arm holds at this N
    dt, nbytes, sample = cpu_reference(lens, block, sf16, args.steps, args.warmup, sample_rows=4)
    gbs = nbytes / dt / 1e9
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


# --------------------------------------------------------------------------------------- run context
class Ctx:
    """Rank, device and the few collectives the measurements need (barrier, max / sum over ranks)."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist
        self.peaks = load_peaks()

    def barrier(self):
        torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()
            torch.cuda.synchronize()

    def _reduce(self, x: float, op) -> float:
        if self.dist is None:
            return x
        t = torch.tensor([x], device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=op)
        return float(t.item())

    def max(self, x: float) -> float:
        return self._reduce(x, self.dist.ReduceOp.MAX) if self.dist else x

    def min(self, x: float) -> float:
        return self._reduce(x, self.dist.ReduceOp.MIN) if self.dist else x

    def sum(self, x: float) -> float:
        return self._reduce(x, self.dist.ReduceOp.SUM) if self.dist else x

    def timed(self, fn, warmup: int, iters: int) -> float:
        """ms per call of `fn`: `warmup` untimed calls, then `iters` calls between two CUDA events on the launch stream,
        barrier + synchronize on both sides, max over ranks."""
        for _ in range(warmup):
            fn()
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        self.barrier()
        return self.max(e0.elapsed_time(e1)) / iters

    def close(self):
        if self.dist is not None:
            self.dist.destroy_process_group()


def fp32_decode_reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """softmax(q k^T / sqrt(D)) v in fp32 with plain torch ops: q [Hq, D], k / v [L, Hkv, D] (any dtype) -> [Hq, D]."""
    g = q.shape[0] // k.shape[1]
    kf = k.float().repeat_interleave(g, dim=1)
    vf = v.float().repeat_interleave(g, dim=1)
    s = torch.einsum("hd,lhd->hl", q.float(), kf) / math.sqrt(q.shape[1])
    return torch.einsum("hl,lhd->hd", torch.softmax(s, dim=-1), vf)


def dequantise_int8_torch(codes: torch.Tensor, scales: torch.Tensor, block: int) -> torch.Tensor:
    """QuantizedTensor::to_tensor (kv_cache.rs:871-957) with plain torch ops: table[code] * absmax in f32, rounded to bf16.
    codes u8 [L, H, D], scales [L, H, D / block]."""
    table = (torch.arange(256, dtype=torch.float32, device=codes.device) - 127.0) / 127.0
    vals = table[codes.long()] * scales.float().repeat_interleave(block, dim=-1)
    return vals.bfloat16()


# --------------------------------------------------------------------------------------- headline: configs[1]
def run_headline(ctx: Ctx, args) -> dict:
    from hyprstream_b200 import ffi, kv_cache as kc, ops

    dev, rank, world = ctx.dev, ctx.rank, ctx.world
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

    def step():  # one C-ABI call, one launch: the attention kernel writes the 32 new tokens (position L_r) before it attends
        ops.decode_append(q, k_new, v_new, view, None, seq_lens, out=out, workspace=ws)

    # ---- device-resident timing -------------------------------------------------------------
    for _ in range(args.warmup):
        step()
    ctx.barrier()
    sampler = ClockSampler(ctx.local) if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = ffi.launch_count()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    ctx.barrier()
    launches = ffi.launch_count() - launches0  # kernels of the library inside the timed region (this rank)
    ms = ctx.max(e0.elapsed_time(e1)) / args.steps
    total_bytes = ctx.sum(float(nbytes))
    clocks = sampler.stop() if sampler else None

    # ---- dominant kernel alone (the split-KV decode kernel), CUDA events on the launch stream ----
    # average launch duration: the decode kernel alone, launched back to back, between one pair of events (the cache is
    # larger than L2, so every launch streams it from HBM again); and, for comparison, one pair of events around each
    # single launch inside the step (the library's tracing hook), which adds the event records' own serialisation
    n_k = max(20, min(args.steps, 200))
    for _ in range(3):
        ops.decode_attention(q, view, seq_lens, out=out, workspace=ws)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(n_k):
        ops.decode_attention(q, view, seq_lens, out=out, workspace=ws)
    e1.record()
    torch.cuda.synchronize()
    kernel_ms = e0.elapsed_time(e1) / n_k
    ffi.set_profiling(True)
    kms = []
    for _ in range(min(args.steps, 50)):
        step()
        kms.append(ffi.last_kernel_ms())
    ffi.set_profiling(False)
    kernel_bytes = sum(l + 1 for l in lens) * token_bytes(block, sf16) + BATCH * HQ * D * 2  # cache + q; partials excluded

    # ---- end to end through the public one-call step with host buffers ------------------------
    # the step's inputs (q, new K, new V) sit back to back in one pinned host buffer; hs_attn_decode_step copies them
    # in, writes the cache, attends and copies the result into a pinned host buffer, returning when it is there
    stepper = ops.DecodeStep(view, BATCH, HQ, dev)
    stepper.q_host.copy_(q); stepper.k_host.copy_(k_new[:, 0]); stepper.v_host.copy_(v_new[:, 0])

    def e2e_step():
        stepper.run(None, seq_lens, sync=True)  # the host has the result before the next step starts

    for _ in range(args.warmup):
        e2e_step()
    ctx.barrier()
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    ctx.barrier()
    e2e_ms = ctx.max(e0.elapsed_time(e1)) / args.steps
    e2e_out = stepper.out_host.clone()

    # ---- parity of the timed configuration (outside every timed region) -----------------------
    parity = None
    if rank == 0 and not args.no_parity:
        parity = headline_parity(caches, lens, q, k_new, v_new, out, e2e_out, block, sf16)
    torch.cuda.synchronize()
    dev_err = ffi.take_device_error()

    peak = float(ctx.peaks.get("hbm_gbs", 6650.0))
    peak_src = "measured (MEASURED_PEAKS.json hbm_gbs, burst copy)" if "hbm_gbs" in ctx.peaks else "fallback 6650 GB/s"
    achieved = kernel_bytes / (kernel_ms * 1e-3) / 1e9
    line = {
        "metric": "decode_attn_hbm_gbps", "value": total_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "tokens_per_s": BATCH * world / (ms * 1e-3),
        "config": workload_config(args.layout, lens),
        "e2e": {"value": total_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
                "tokens_per_s": BATCH * world / (e2e_ms * 1e-3), "h2d_bytes_per_step": stepper.h2d_bytes,
                "d2h_bytes_per_step": stepper.d2h_bytes, "api": "hs_attn_decode_step (one C-ABI call per step, pinned host buffers)"},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "kernel": "decode split-KV kernel (rank 0)", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src, "kernel_ms": kernel_ms,
                     "method": f"{n_k} launches of the decode kernel back to back between two CUDA events on the launch stream, after warm-up",
                     "kernel_ms_single_launches": {"mean": sum(kms) / len(kms), "min": min(kms),
                                                   "method": "one event pair around each launch inside the step"},
                     "bytes_per_launch": kernel_bytes,
                     "traffic": NCU_TRAFFIC_PER_ALGO_BYTE * kernel_bytes if args.layout == "baseline" else None,
                     "traffic_source": NCU_TRAFFIC_SOURCE if args.layout == "baseline" else None},
        "clocks": clocks, "device_error_flags": dev_err, "parity": parity,
    }
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        cores = host_threads()
        dt, cb, sample = cpu_reference(lens, block, sf16, steps=2, warmup=1, sample_rows=4)
        line["cpu_baseline"] = {"value": cb / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
                                "sample": sample, "ms_per_step": dt * 1e3}
    return line


def headline_parity(caches, lens, q, k_new, v_new, out, e2e_out, block, sf16) -> dict:
    """The measured configuration checked: every sequence's output of the timed step against softmax(q k^T) v in fp32
    over its dequantised cache (stored codes and scales read back raw and dequantised with plain torch ops); the codes
    and scales stored for the 32 written tokens against the CPU oracle quantiser, bit for bit."""
    from oracle import quant_ref as qr

    dev = q.device
    max_abs, sum_abs, n_el, codes_ok = 0.0, 0.0, 0, True
    for r, c in enumerate(caches):
        c.seq_pos = lens[r] + 1  # the step wrote position L_r through the view
        kc_, vc_, ks_, vs_ = c.snapshot()
        kd = dequantise_int8_torch(kc_.to(dev), ks_.to(dev), block)
        vd = dequantise_int8_torch(vc_.to(dev), vs_.to(dev), block)
        ref = fp32_decode_reference(q[r], kd, vd)
        for o in (out[r], e2e_out[r].to(dev)):
            diff = (o.float() - ref).abs()
            max_abs = max(max_abs, float(diff.max().item()))
        sum_abs += float((out[r].float() - ref).abs().sum().item())
        n_el += ref.numel()
        for new, codes, scales in ((k_new[r, 0], kc_[-1], ks_[-1]), (v_new[r, 0], vc_[-1], vs_[-1])):
            oc, oa = qr.quantize(new.float().cpu().numpy(), qr.INT8, block, bool(sf16))
            codes_ok &= bool(np.array_equal(codes.numpy().reshape(-1), oc))
            raw = scales.numpy().reshape(-1)
            codes_ok &= bool(np.array_equal(raw.view(np.uint16 if sf16 else np.uint32), np.asarray(oa).reshape(-1).view(np.uint16 if sf16 else np.uint32)))
    mean_abs = sum_abs / max(n_el, 1)
    return {"reference": "fp32 softmax(q k^T / sqrt(d)) v over the dequantised cache, plain torch ops on the GPU, all 32 sequences",
            "max_abs": max_abs, "mean_abs": mean_abs, "tolerance": {"max_abs": MAX_ABS_TOL, "mean_abs": MEAN_ABS_TOL},
            "within_tolerance": bool(max_abs <= MAX_ABS_TOL and mean_abs <= MEAN_ABS_TOL),
            "e2e_output_checked": True, "written_token_codes_bit_exact_vs_oracle": bool(codes_ok)}


# --------------------------------------------------------------------------------------- configs[2]: long context, NF4, KV-length shards
def run_longctx(ctx: Ctx, context: int = 131072, steps: int = 30, warmup: int = 5, check_context: int = 8192) -> dict:
    """Batch 4, 32 q / 8 kv heads, d = 128, `context` tokens per sequence, NF4 codes with an f16 absmax per block of 64.
    The KV length is cut into one contiguous page-aligned shard per GPU (strong scaling).  Two forms of the step are
    timed: (collective) local decode -> NCCL all-gather of (o, lse) -> merge kernel, three host calls; (fused) one
    launch per GPU: the decode kernel stores its shard result into every rank's inbox over NVLink, waits - bounded - and
    merges.  A reduced context is first checked against an unsharded decode of the same cache on every rank."""
    from hyprstream_b200 import ffi, kv_cache as kc, ops, sharded

    b, hq, hkv, d = 4, 32, 8, 128
    dev, rank, world = ctx.dev, ctx.rank, ctx.world
    res = {"workload": "configs[2]: long-context decode over an NF4 KV cache, KV length sharded across the GPUs",
           "batch": b, "context": context, "n_gpus": world, "scaling": "strong", "kv_layout": "NF4, block 64, f16 absmax",
           "collective_bytes_per_gpu": b * hq * (d + 1) * 4}

    def build(ctx_len, with_full):
        start, end = sharded.shard_bounds(ctx_len, world)[rank]
        n_local = end - start
        caches, full = [], []
        for s in range(b):
            g = torch.Generator(device=dev).manual_seed(1000 + s)  # every rank draws the same stream
            c = kc.LayerKVCache(max(n_local, 32), kc.KVQuantType.NF4, hkv, d, dev, block=64, scale_dtype=ffi.SCALE_F16)
            c._ensure_capacity(max(n_local, 32))
            cf = kc.LayerKVCache(ctx_len, kc.KVQuantType.NF4, hkv, d, dev, block=64, scale_dtype=ffi.SCALE_F16) if with_full else None
            for t0 in range(0, ctx_len, 8192):
                t1 = min(ctx_len, t0 + 8192)
                k = torch.randn(1, t1 - t0, hkv, d, device=dev, generator=g).bfloat16()
                v = torch.randn(1, t1 - t0, hkv, d, device=dev, generator=g).bfloat16()
                lo, hi = max(t0, start), min(t1, end)
                if lo < hi:
                    c.update(k[:, lo - t0:hi - t0].contiguous(), v[:, lo - t0:hi - t0].contiguous(), lo - start)
                if cf is not None:
                    cf.update(k, v, t0)
            caches.append(c)
            full.append(cf)
        view, keep = kc.make_view(caches)
        lens = torch.full((b,), n_local, dtype=torch.int32, device=dev)
        return caches, full, view, keep, lens

    q = torch.randn(b, hq, d, device=dev, generator=torch.Generator(device=dev).manual_seed(7)).bfloat16()
    coll = sharded.ShardedDecoder(b, hq, d, dev)
    fused, fused_err = None, None
    try:
        fused = sharded.FusedShardedDecoder(b, hq, d, dev)
    except Exception as e:  # e.g. the platform refuses CUDA IPC between the ranks' processes
        fused_err = f"{type(e).__name__}: {e}"
    if ctx.min(1.0 if fused is not None else 0.0) < 1.0:
        fused = None
        res["fused_unavailable"] = fused_err or "another rank could not set up its shard group"

    # ---- parity on a reduced context: sharded (both forms) == unsharded, on every rank ----
    caches, full, view, keep, lens = build(check_context, True)
    fview, fkeep = kc.make_view(full)
    ref = ops.decode_attention(q, fview, torch.full((b,), check_context, dtype=torch.int32, device=dev))
    out_c = coll.step(q, view, lens).clone()
    torch.cuda.synchronize()
    res["max_abs_vs_unsharded"] = {"context": check_context, "collective": ctx.max(float((out_c.float() - ref.float()).abs().max().item()))}
    if fused is not None:
        out_f = fused.step(q, view, lens).clone()
        torch.cuda.synchronize()
        res["max_abs_vs_unsharded"]["fused"] = ctx.max(float((out_f.float() - ref.float()).abs().max().item()))
        res["ranks_outputs_identical"] = bool(ctx.max(float((out_f.float() - out_c.float()).abs().max().item())) <= 4e-3)
    del caches, full, view, keep, fview, fkeep
    torch.cuda.empty_cache()

    # ---- timing at the full context ----
    caches, _, view, keep, lens = build(context, False)
    total = b * context * 2 * hkv * (d // 2 + (d // 64) * 2)
    peak = float(ctx.peaks.get("hbm_gbs", 6650.0))

    def report(ms):
        return {"ms_per_step": ms, "aggregate_gbps": total / ms / 1e6, "per_gpu_gbps": total / world / ms / 1e6,
                "frac_of_hbm_peak_per_gpu": total / world / ms / 1e6 / peak, "tokens_per_s": b / ms * 1e3}

    if world == 1:
        res["one_gpu"] = report(ctx.timed(lambda: ops.decode_attention(q, view, lens), warmup, steps))
    else:  # this rank's shard alone, no exchange: what the exchange adds is the difference to the forms below
        res["local_shard_decode_ms"] = ctx.timed(lambda: ops.decode_attention(q, view, lens), warmup, steps)
    res["collective"] = dict(report(ctx.timed(lambda: coll.step(q, view, lens), warmup, steps)),
                             step="decode launch + NCCL all-gather of (o, lse) + merge launch" if world > 1 else "decode launch + merge launch")
    if fused is not None:
        res["fused"] = dict(report(ctx.timed(lambda: fused.step(q, view, lens), warmup, steps)),
                            step="one launch per GPU: peer stores of (o, lse), release flags, bounded wait, merge")
    torch.cuda.synchronize()
    res["device_error_flags"] = ffi.take_device_error()
    return res


# --------------------------------------------------------------------------------------- configs[3]: causal prefill + quantise-on-write
def run_prefill(ctx: Ctx, batch: int = 8, tokens: int = 8192, iters: int = 5, warmup: int = 3) -> dict:
    """Causal GQA prefill, `batch` x `tokens` tokens, 32 q / 8 kv heads, d = 128, bf16, with the produced K/V written to
    the int8 cache (block 128, f16 absmax).  Sequences are dealt over the GPUs (independent, no collective).  Useful
    FLOPs are the causal half: 4 * B * Hq * D * T(T+1)/2."""
    from hyprstream_b200 import ffi, kv_cache as kc, ops, sharded
    from oracle import quant_ref as qr

    hq, hkv, d = 32, 8, 128
    dev, rank, world = ctx.dev, ctx.rank, ctx.world
    units = sharded.partition_units(batch, hkv, world)[rank]
    res = {"workload": "configs[3]: causal GQA prefill with int8 quantise-on-write", "batch": batch, "tokens": tokens,
           "n_gpus": world, "scaling": "strong", "partition": "sequences (then kv-head groups) dealt over the GPUs, no collective"}
    flops_total = 4.0 * batch * hq * d * tokens * (tokens + 1) / 2
    ms = kms = wms = 0.0
    parity = None
    if units:
        bl = len(units)
        h_lo, h_hi = units[0][1], units[0][2]
        hkv_l = h_hi - h_lo
        hq_l = hkv_l * (hq // hkv)
        g = torch.Generator(device=dev).manual_seed(3 + 17 * rank)
        qt = torch.randn(bl, tokens, hq_l, d, device=dev, generator=g).bfloat16()
        k = torch.randn(bl, tokens, hkv_l, d, device=dev, generator=g).bfloat16()
        v = torch.randn(bl, tokens, hkv_l, d, device=dev, generator=g).bfloat16()
        caches = [kc.LayerKVCache(tokens, kc.KVQuantType.INT8, hkv_l, d, dev, block=128, scale_dtype=ffi.SCALE_F16) for _ in range(bl)]
        for c in caches:
            c._ensure_capacity(tokens)
        view, keep = kc.make_view(caches)
        zeros = torch.zeros(bl, dtype=torch.int32, device=dev)
        outs = []

        def step():
            outs[:] = [ops.prefill_attention(qt, k, v)]
            ops.kv_quantize_write(view, k, v, zeros)
    else:
        def step():
            pass
    ms = ctx.timed(step, warmup, iters)
    if units:
        ffi.set_profiling(True)
        ks_ = []
        for _ in range(3):
            ops.prefill_attention(qt, k, v)
            ks_.append(ffi.last_kernel_ms())
        ffi.set_profiling(False)
        kms = sum(ks_) / len(ks_)
    wms_local = 0.0
    if units:
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            ops.kv_quantize_write(view, k, v, zeros)
        e1.record()
        torch.cuda.synchronize()
        wms_local = e0.elapsed_time(e1) / iters
    kms, wms = ctx.max(kms), ctx.max(wms_local)
    if units and rank == 0:
        # parity: the last 128 query rows of sequence 0 against fp32 over all keys; sequence 0's stored codes against the oracle
        out = outs[0]
        rows = slice(tokens - 128, tokens)
        g_ = hq_l // hkv_l
        kf = k[0].float().repeat_interleave(g_, dim=1)
        vf = v[0].float().repeat_interleave(g_, dim=1)
        s = torch.einsum("qhd,lhd->hql", qt[0, rows].float(), kf) / math.sqrt(d)
        mask = torch.arange(tokens, device=dev)[None, :] > torch.arange(tokens - 128, tokens, device=dev)[:, None]
        s = s.masked_fill(mask[None], float("-inf"))
        ref = torch.einsum("hql,lhd->qhd", torch.softmax(s, -1), vf)
        diff = (out[0, rows].float() - ref).abs()
        caches[0].seq_pos = tokens
        kc_, vc_, ks2, vs2 = caches[0].snapshot()
        n_chk = min(tokens, 2048)
        ok = True
        for src, codes, scales in ((k[0, :n_chk], kc_[:n_chk], ks2[:n_chk]), (v[0, :n_chk], vc_[:n_chk], vs2[:n_chk])):
            oc, oa = qr.quantize(src.float().cpu().numpy(), qr.INT8, 128, True)
            ok &= bool(np.array_equal(codes.numpy().reshape(-1), oc))
            ok &= bool(np.array_equal(scales.numpy().reshape(-1).view(np.uint16), np.asarray(oa).reshape(-1).view(np.uint16)))
        parity = {"rows_checked": "sequence 0, last 128 query rows, all heads, fp32 recomputation on the GPU",
                  "max_abs": float(diff.max().item()), "mean_abs": float(diff.mean().item()),
                  "within_tolerance": bool(diff.max().item() <= MAX_ABS_TOL and diff.mean().item() <= MEAN_ABS_TOL),
                  "cache_codes_bit_exact_vs_oracle": bool(ok), "codes_checked": f"sequence 0, first {n_chk} tokens, K and V"}
    burst = float(ctx.peaks.get("bf16_tflops", 1590.0))
    sust = float(ctx.peaks.get("bf16_tflops_sustained", 1400.0))
    tf_step = flops_total / ms / 1e9
    tf_kernel = flops_total / max(kms, 1e-9) / 1e9
    res.update({"ms_per_step": ms, "attn_kernel_ms": kms, "kv_write_ms": wms,
                "useful_tflops_with_quantise_on_write": tf_step, "useful_tflops_attention_kernel": tf_kernel,
                "per_gpu_tflops_attention_kernel": tf_kernel / world,
                "frac_of_bf16_burst_peak_per_gpu": tf_kernel / world / burst, "frac_of_bf16_sustained_peak_per_gpu": tf_kernel / world / sust,
                "kv_write_gbps_per_gpu": (2 * batch * tokens * hkv * (d * 2 + d + 2) / world) / max(wms, 1e-9) / 1e6,
                "tokens_per_s": batch * tokens / ms * 1e3, "parity": parity})
    torch.cuda.synchronize()
    res["device_error_flags"] = ffi.take_device_error()
    return res


# --------------------------------------------------------------------------------------- configs[4]: Qwen3.5-style block
def run_qwen_block(ctx: Ctx, prefill_batch: int = 4, prefill_tokens: int = 32768, decode_batch: int = 64, decode_steps: int = 64,
                   context: int = 32768) -> dict:
    """One Qwen3.5-style block = 3 gated-DeltaNet layers + 1 gated full-attention layer, everything between the layers'
    projections (the GEMMs stay with the host framework and are not timed): prefill of 4 x 32768 tokens, then decode
    steps at batch 64 against 32768 + t cached tokens.  Inputs are random "projection outputs" of the right shapes and
    dtypes.  Per DeltaNet layer: hs_gdn_prologue -> hs_gdn_chunk_prefill (prefill) / hs_gdn_recurrent (decode) ->
    hs_gdn_epilogue.  Full attention: hs_qk_norm_rope (q with gate split, k) -> hs_kv_quantize_write (int8, block 128,
    f16 scales) -> hs_attn_prefill_causal / hs_attn_decode with the output gate.  Over several GPUs the prefill is dealt
    by (sequence, head group) and the decode by sequence; no collective."""
    from hyprstream_b200 import ffi, kv_cache as kc, ops, sharded

    NK, NV, HD, KS = 16, 32, 128, 4
    HQ5, HKV5, D5, RD = 16, 2, 256, 64
    N_GDN = 3
    dev, rank, world = ctx.dev, ctx.rank, ctx.world
    g = torch.Generator(device=dev).manual_seed(4 + 31 * rank)
    rnd = lambda *shape: torch.randn(*shape, device=dev, generator=g)  # noqa: E731
    res = {"workload": "configs[4]: Qwen3.5-style block, 3 gated-DeltaNet layers + 1 gated full-attention layer (projections not timed)",
           "n_gpus": world, "scaling": "strong"}
    n_pos = context + decode_steps + 8
    ang = torch.arange(n_pos, device=dev).float()[:, None] * torch.arange(RD // 2, device=dev).float()[None, :] * 1e-3
    sin, cos = torch.sin(ang).bfloat16(), torch.cos(ang).bfloat16()

    # ------------------------------------------------------------------ prefill
    units = sharded.partition_units(prefill_batch, 2, world)[rank]  # head groups: halves (1 kv head / 8 k heads / 16 v heads each)
    b, t = len(units), prefill_tokens
    frac = (units[0][2] - units[0][1]) / 2 if units else 1
    nk, nv, hq, hkv = int(NK * frac), int(NV * frac), int(HQ5 * frac), int(HKV5 * frac)
    conv_dim = (2 * nk + nv) * HD
    if units:
        layers = [ops.GdnLayer((rnd(conv_dim, 1, KS) * 0.5).bfloat16(), torch.log(torch.rand(nv, device=dev, generator=g) + 1e-3), rnd(nv) * 0.3,
                               1.0 + 0.1 * rnd(HD), nk, nv) for _ in range(N_GDN)]
        attn = ops.QwenAttnLayer(0.1 * rnd(D5), 0.1 * rnd(D5), sin, cos, RD, hq, hkv, D5)
        x = rnd(b, t, conv_dim).bfloat16()
        z = rnd(b, t, nv, HD).bfloat16()
        a_in, b_in = rnd(b, t, nv).bfloat16(), rnd(b, t, nv).bfloat16()
        q_full = rnd(b * t, hq * 2 * D5).bfloat16()
        k_proj, v_proj = rnd(b * t, hkv * D5).bfloat16(), rnd(b, t, hkv, D5).bfloat16()
        pos = torch.arange(t, device=dev, dtype=torch.int32).repeat(b)
        states = [l.new_states(b, dev) for l in layers]
        caches = [kc.LayerKVCache(t, kc.KVQuantType.INT8, hkv, D5, dev, block=128, scale_dtype=ffi.SCALE_F16) for _ in range(b)]
        for c in caches:
            c._ensure_capacity(t)
        view, keep = kc.make_view(caches)
        zeros = torch.zeros(b, dtype=torch.int32, device=dev)
        gin = [(x, z, a_in, b_in) + states[i] for i in range(N_GDN)]
        ain = (q_full, k_proj, v_proj, view, pos, zeros, zeros + 1)
        ws = torch.empty(max(layers[0].workspace_bytes(b, t), attn.workspace_bytes(b, t)), dtype=torch.uint8, device=dev)
        # warm-up (also builds tensor maps, sets attributes): the whole block through the one block-level call
        ops.qwen_block_forward(layers, gin, attn, ain, False, b, t, dev, workspace=ws)
    # three timed passes of the block, the median pass reported (one pass is 40 ms; the DeltaNet layers' chain follows the SM clock,
    # which the power cap moves from pass to pass)
    passes = []
    for _ in range(3):
        ctx.barrier()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        if units:
            ops.qwen_block_forward(layers, gin, None, None, False, b, t, dev, workspace=ws)   # the three DeltaNet layers
        e[1].record()
        if units:
            ops.qwen_block_forward([], [], attn, ain, False, b, t, dev, workspace=ws)         # the full-attention layer
        e[2].record()
        ctx.barrier()
        passes.append((ctx.max(e[0].elapsed_time(e[2])), ctx.max(e[0].elapsed_time(e[1])), ctx.max(e[1].elapsed_time(e[2]))))
    block_ms, gdn_ms, attn_ms = sorted(passes)[1]
    attn_flops = 4.0 * prefill_batch * HQ5 * D5 * t * (t + 1) / 2
    res["prefill"] = {"batch": prefill_batch, "tokens": t, "units_per_gpu": f"{b} x ({nv} v heads, {hq} q heads)",
                      "api": "hs_qwen_block_forward", "gdn_layers_ms": gdn_ms, "full_attention_layer_ms": attn_ms, "block_ms": block_ms,
                      "block_ms_passes": [round(p[0], 3) for p in passes],
                      "tokens_per_s": prefill_batch * t / block_ms * 1e3,
                      "full_attention_useful_tflops_incl_edges": attn_flops / attn_ms / 1e9}
    if units:
        del x, z, a_in, b_in, q_full, k_proj, v_proj, caches, view, keep, states, gin, ain, ws, layers, attn
    torch.cuda.empty_cache()

    # ------------------------------------------------------------------ decode (by sequence, full heads)
    bl = len(sharded.partition_units(decode_batch, 1, world)[rank])
    L = context
    conv_dim = (2 * NK + NV) * HD
    if bl:
        layers = [ops.GdnLayer((rnd(conv_dim, 1, KS) * 0.5).bfloat16(), torch.log(torch.rand(NV, device=dev, generator=g) + 1e-3), rnd(NV) * 0.3,
                               1.0 + 0.1 * rnd(HD), NK, NV) for _ in range(N_GDN)]
        attn = ops.QwenAttnLayer(0.1 * rnd(D5), 0.1 * rnd(D5), sin, cos, RD, HQ5, HKV5, D5)
        caches = []
        cap = (L + decode_steps + 8 + 1023) // 1024 * 1024  # whole 1024-token growth chunks (kv_cache.rs:700)
        for s_ in range(bl):
            c = kc.LayerKVCache(cap, kc.KVQuantType.INT8, HKV5, D5, dev, block=128, scale_dtype=ffi.SCALE_F16)
            for t0 in range(0, L, 8192):
                n = min(8192, L - t0)
                c.update(rnd(1, n, HKV5, D5).bfloat16(), rnd(1, n, HKV5, D5).bfloat16(), t0)
            c._ensure_capacity(cap)
            caches.append(c)
        view, keep = kc.make_view(caches)
        x = rnd(bl, 1, conv_dim).bfloat16()
        z = rnd(bl, 1, NV, HD).bfloat16()
        a_in, b_in = rnd(bl, 1, NV).bfloat16(), rnd(bl, 1, NV).bfloat16()
        q_full = rnd(bl, HQ5 * 2 * D5).bfloat16()
        k_proj, v_proj = rnd(bl, HKV5 * D5).bfloat16(), rnd(bl, 1, HKV5, D5).bfloat16()
        states = [(rnd(bl, conv_dim, KS - 1).bfloat16(), rnd(bl, NV, HD, HD) * 0.1) for _ in range(N_GDN)]
        dst = torch.full((bl,), L, dtype=torch.int32, device=dev)
        lens = dst + 1
        gin = [(x, z, a_in, b_in) + states[i] for i in range(N_GDN)]
        ain = (q_full, k_proj, v_proj, view, dst, dst, lens)   # one new token per sequence: its RoPE row is its cache position
        ws = torch.empty(max(layers[0].workspace_bytes(bl, 1), attn.workspace_bytes(bl, 1)), dtype=torch.uint8, device=dev)

        def decode_step():  # one block step = one hs_qwen_block_forward call
            ops.qwen_block_forward(layers, gin, attn, ain, True, bl, 1, dev, workspace=ws)
            dst.add_(1)
            lens.add_(1)
    else:
        def decode_step():
            pass
    ms = ctx.timed(decode_step, 3, decode_steps)
    kv_bytes = decode_batch * (L + 3 + decode_steps / 2) * token_bytes(128, 1, HKV5, D5)
    state_bytes = N_GDN * 2 * decode_batch * NV * HD * HD * 4
    peak = float(ctx.peaks.get("hbm_gbs", 6650.0))
    res["decode"] = {"batch": decode_batch, "context": L, "steps": decode_steps, "api": "hs_qwen_block_forward (one call per block step)",
                     "ms_per_step": ms, "tokens_per_s": decode_batch / ms * 1e3,
                     "algorithmic_bytes_per_step": kv_bytes + state_bytes, "hbm_gbps": (kv_bytes + state_bytes) / ms / 1e6,
                     "frac_of_hbm_peak_per_gpu": (kv_bytes + state_bytes) / world / ms / 1e6 / peak}
    torch.cuda.synchronize()
    res["device_error_flags"] = ffi.take_device_error()
    return res


SECONDARY = {3: ("longctx_nf4_sharded_decode", run_longctx), 4: ("prefill_int8_write", run_prefill), 5: ("qwen_block", run_qwen_block)}


def run_secondary(ctx: Ctx, which, **kw) -> dict:
    """One secondary workload; a failure is reported in the record instead of ending the run (every rank runs the same
    code, so a refusal - an unsupported platform feature - is met by all ranks at the same point)."""
    name, fn = SECONDARY[which]
    t0 = time.perf_counter()
    try:
        rec = fn(ctx, **kw)
    except Exception as e:  # noqa: BLE001
        rec = {"error": f"{type(e).__name__}: {e}"}
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    rec["wall_s"] = round(time.perf_counter() - t0, 2)
    return rec


# --------------------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layout", default="baseline", choices=sorted(LAYOUTS))
    ap.add_argument("--config", type=int, default=2, choices=[2, 3, 4, 5],
                    help="2: the headline line with parity and the secondary record (default); 3, 4, 5: that workload alone")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--context", type=int, default=131072, help="--config 3: tokens per sequence")
    ap.add_argument("--decode-steps", type=int, default=64, help="--config 5: decode steps timed (BASELINE: 256)")
    ap.add_argument("--prefill-tokens", type=int, default=None, help="--config 4, 5: prompt tokens per sequence (default 8192, 32768)")
    ap.add_argument("--prefill-batch", type=int, default=None, help="--config 4, 5: prompt sequences (default 8, 4)")
    ap.add_argument("--decode-batch", type=int, default=64, help="--config 5: sequences of the decode steps")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        run_reference_arm(args)
        return

    ctx = Ctx()
    if args.config != 2:
        kw = {3: {"context": args.context}, 4: {"batch": args.prefill_batch or 8, "tokens": args.prefill_tokens or 8192},
              5: {"decode_steps": args.decode_steps, "prefill_tokens": args.prefill_tokens or 32768, "prefill_batch": args.prefill_batch or 4,
                  "decode_batch": args.decode_batch}}[args.config]
        rec = run_secondary(ctx, args.config, **kw)
        if ctx.rank == 0:
            print(json.dumps(rec))
        ctx.close()
        return

    line = run_headline(ctx, args)
    if not args.no_secondary:
        sec = {}
        for which in (3, 4, 5):
            sec[SECONDARY[which][0]] = run_secondary(ctx, which)
        line["secondary"] = sec
    if ctx.rank == 0:
        print(json.dumps(line))
    ctx.close()


if __name__ == "__main__":
    main()
