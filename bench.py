#!/usr/bin/env python
"""Benchmark of the quantized DiT hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N=1 and every N): the DiT projection set of one 1024x1024 image at batch 2 (CFG),
M = 2 x 4608 tokens per GPU, all W8A8 `int8-convrot` (QuantizeInt8Rows H256ConvRot +
LinearInt8Scaled + BiasAdd [+ Gelu]): fused QKV 3072->9216, out-proj 3072->3072, MLP up
3072->12288 (GELU-tanh) and MLP down 12288->3072. One step = one pass over all four. With
N > 1 every rank runs its own batch (tokens are sharded, weights replicated, no collective on
the data path): weak scaling. The metric is INT8 TOPS = 2*M*N*K summed over the projections,
divided by the step time (quantisation kernels included in the time, not in the op count).

Prints ONE JSON line on rank 0. Synthetic data: seeded N(0,1) bf16 activations with 32 outlier
channels x16, N(0,0.02) weights quantised by the same ConvRot transform, N(0,0.01) bias.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PROJECTIONS = [  # name, K, N, gelu
    ("qkv", 3072, 9216, False),
    ("out_proj", 3072, 3072, False),
    ("mlp_up", 3072, 12288, True),
    ("mlp_down", 12288, 3072, False),
]
M_TOKENS = 2 * 4608
H256_CONVROT = 2


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def recorded_traffic(kernel: str):
    """DRAM bytes per launch of `kernel` from the committed ncu capture summary, or None."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    try:
        with open(path) as f:
            return json.load(f).get(kernel)
    except Exception:
        return None


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                mhz.append(float(s[0]))
                mx = float(s[1])
            except ValueError:
                continue
            for name, val in zip(names, s[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        med = mhz[len(mhz) // 2] if mhz else None
        return {"sm_mhz": med, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(mhz)}


def synth_inputs(torch, device, seed: int):
    """Seeded synthetic activations / weights / biases of the projection set, on `device`."""
    from diffusion_compiler_b200 import ops
    g = torch.Generator(device="cpu").manual_seed(seed)
    chans = torch.randperm(3072, generator=torch.Generator().manual_seed(0))[:32]
    layers = []
    for name, K, N, gelu in PROJECTIONS:
        x = torch.randn(M_TOKENS, K, generator=g, dtype=torch.float32)
        x[:, chans] *= 16.0
        w = (torch.randn(N, K, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        b = (torch.randn(N, generator=g, dtype=torch.float32) * 0.01).to(torch.bfloat16)
        x_host = x.to(torch.bfloat16).pin_memory()
        w8, ws = ops.quantize_int8_rows([w.to(device)], H256_CONVROT)  # offline weight-side ConvRot
        layers.append({"name": name, "K": K, "N": N, "gelu": gelu, "x_host": x_host,
                       "x": x_host.to(device, non_blocking=True), "w8": w8, "ws": ws, "bias": b.to(device),
                       "codes": torch.empty(M_TOKENS, K, dtype=torch.int8, device=device),
                       "out": torch.empty(M_TOKENS, N, dtype=torch.bfloat16, device=device)})
    torch.cuda.synchronize(device)
    return layers


def run_step(ops, layers, events=None):
    for i, L in enumerate(layers):
        if events is not None:
            events[i][0].record()
        codes, scales = ops.quantize_int8_rows([L["x"]], H256_CONVROT)
        if events is not None:
            events[i][1].record()
        ops.linear_int8_scaled(codes, L["w8"], scales, L["ws"], bias=L["bias"], gelu=L["gelu"], out=L["out"])
        if events is not None:
            events[i][2].record()


def cpu_reference_sample(threads: int, rows_per_thread: int):
    """Times the reference CPU executor (oracle/_ref) -- or, where it was not built, the C
    restatement -- on a row sample of the same four projections, `threads` host threads."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import numpy as np
    import oracle_bridge as ob
    from concurrent.futures import ThreadPoolExecutor
    from diffusion_compiler_b200 import diffir
    rng = np.random.default_rng(0)
    kind = "reference" if ob.ref_available() else "port"
    jobs = []
    total_ops = 0.0
    for name, K, N, gelu in PROJECTIONS:
        w8 = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
        ws = (rng.random(N, dtype=np.float32) * 1e-3 + 1e-4).astype(np.float32)
        bias = ob.f32_to_bf16((rng.standard_normal(N) * 0.01).astype(np.float32))
        x = ob.f32_to_bf16(rng.standard_normal((rows_per_thread, K)).astype(np.float32))
        jobs.append((K, N, gelu, x, w8, ws, bias))
        total_ops += 2.0 * rows_per_thread * N * K * threads

    def work(_):
        for K, N, gelu, x, w8, ws, bias in jobs:
            if kind == "reference":
                pr = diffir.w8a8_linear_program(rows_per_thread, K, N, H256_CONVROT, bias=True, gelu=gelu)
                ids = pr["ids"]
                ob.ref().run(pr["program"], {ids["x"]: x, ids["weight"]: w8, ids["col_scales"]: ws,
                                             ids["bias"]: bias})
            else:
                c, s = ob.orc().quantize_int8_rows([x], H256_CONVROT)
                y = ob.orc().bias_add(ob.orc().linear_int8_scaled(c, w8, s, ws), bias)
                if gelu:
                    ob.orc().gelu_tanh(y)

    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=threads) as pool:
        list(pool.map(work, range(threads)))
    dt = time.perf_counter() - t0
    return {"value": total_ops / dt / 1e12, "unit": "TOPS", "cores": threads, "kind": kind,
            "sample": "%d rows per thread x %d threads of the same 4 projections (full weights), %.1f s"
                      % (rows_per_thread, threads, dt)}, dt


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    total_ops = sum(2.0 * M_TOKENS * N * K for _, K, N, _ in PROJECTIONS)
    config = {"workload": "DiT projection set (BASELINE config 1): M=2x4608 tokens per GPU, W8A8 int8-convrot "
                          "QKV 3072->9216, out 3072->3072, MLP up 3072->12288 +GELU, MLP down 12288->3072",
              "tokens_per_gpu": M_TOKENS, "quantization": "H256ConvRot activations + per-channel INT8 weights",
              "parallelism": "token-sharded x%d, weights replicated" % max(world, args.gpus),
              "l2": "inputs+weights+outputs of one step are ~1.1 GB, larger than the 126 MB L2; no flush"}

    if args.impl == "reference":
        if rank != 0:
            return
        threads = os.cpu_count() or 1
        rows = 64
        steps = max(1, min(args.steps, 3))
        vals = []
        for _ in range(min(args.warmup, 1)):
            cpu_reference_sample(threads, 8)
        for _ in range(steps):
            res, dt = cpu_reference_sample(threads, rows)
            vals.append(res)
        best = max(vals, key=lambda r: r["value"])
        ms = total_ops / (best["value"] * 1e12) * 1e3
        line = {"impl": "reference", "metric": "int8_tops_w8a8_projection_set", "value": best["value"],
                "unit": "TOPS", "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 1),
                "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "int8", "data": "synthetic", "config": config, "cpu_baseline": best,
                "e2e": {"value": best["value"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "note": "reference CPU executor on host cores; ms_per_step is the full-workload time "
                        "extrapolated from the row sample"}
        print(json.dumps(line))
        return

    import torch
    from diffusion_compiler_b200 import ops
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path for the product kernels")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    layers = synth_inputs(torch, device, seed=rank)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        run_step(ops, layers)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    # --- timed region: K steps, device-resident inputs ---
    gemm_events = [[[torch.cuda.Event(enable_timing=True) for _ in range(3)]
                    for _ in layers] for _ in range(args.steps)]
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for s in range(args.steps):
        run_step(ops, layers, gemm_events[s])
    stop.record()
    barrier()
    elapsed_ms = start.elapsed_time(stop)
    ops.poll_status()
    # --- end-to-end: host inputs -> device, compute, result -> host, every step ---
    out_host = [torch.empty_like(L["out"], device="cpu").pin_memory() for L in layers]
    h2d = sum(L["x_host"].numel() * 2 for L in layers)
    d2h = sum(o.numel() * 2 for o in out_host)

    def e2e_step():
        for L, oh in zip(layers, out_host):
            L["x"].copy_(L["x_host"], non_blocking=True)
        run_step(ops, layers)
        for L, oh in zip(layers, out_host):
            oh.copy_(L["out"], non_blocking=True)

    e2e_step()
    barrier()
    e2e_steps = max(3, min(args.steps, 10))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    clocks = sampler.stop() if rank == 0 else None

    t = torch.tensor([elapsed_ms, e2e_ms], dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms = float(t[0]), float(t[1])
    ms_per_step = elapsed_ms / args.steps
    value = world * total_ops / (ms_per_step * 1e-3) / 1e12

    if rank == 0:
        peaks = measured_peaks()
        # dominant kernel: the tcgen05 GEMM. achieved = algorithmic 2*M*N*K per launch / launch time
        gemm_ms = quant_ms_total = 0.0
        for s in range(args.steps):
            for ev in gemm_events[s]:
                quant_ms_total += ev[0].elapsed_time(ev[1])
                gemm_ms += ev[1].elapsed_time(ev[2])
        gemm_tops = args.steps * total_ops / (gemm_ms * 1e-3) / 1e12
        int8_peak = 2.0 * peaks["bf16_tflops"]
        quant_bytes = sum(3.0 * M_TOKENS * K + 4.0 * M_TOKENS for _, K, _, _ in PROJECTIONS)
        quant_ms = quant_ms_total / args.steps
        line = {
            "metric": "int8_tops_w8a8_projection_set", "value": value, "unit": "TOPS", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
            "data": "synthetic", "config": config,
            "e2e": {"value": world * total_ops / (e2e_ms * 1e-3) / 1e12, "unit": "TOPS",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                    "path": "pinned host activations -> device, 4x(quantize+linear), bf16 outputs -> pinned host"},
            "gpu_launches": args.steps * 2 * len(layers),
            "roofline": {"bound": "tensor", "kernel": "gemm_i8_kernel (tcgen05 kind::i8)",
                         "achieved": gemm_tops, "peak": int8_peak, "unit": "TOP/s", "frac": gemm_tops / int8_peak,
                         "peak_source": "2 x %s bf16 burst TFLOP/s (INT8 dense = 2x bf16 on B200); nominal 4500"
                                        % peaks["source"],
                         "frac_of_nominal_4500": gemm_tops / 4500.0,
                         "traffic": recorded_traffic("gemm_i8_kernel")},
            "roofline_quant": {"bound": "hbm", "kernel": "convrot_quant_kernel",
                               "achieved": quant_bytes / (quant_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                               "unit": "GB/s", "frac": quant_bytes / (quant_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                               "note": "CUDA events around the 4 quantize launches of every step",
                               "traffic": recorded_traffic("convrot_quant_kernel")},
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            res, _ = cpu_reference_sample(threads, 64)
            line["cpu_baseline"] = res
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
