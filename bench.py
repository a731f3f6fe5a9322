#!/usr/bin/env python
"""Benchmark of the quantized-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Default workload: MXFP8 GEMM, M = N = K = 8192 (E4M3 values, one E8M0 scale per 32 K
elements, fp32 accumulate, bf16 output), synthetic N(0,1) data quantised on the GPU
before the timed region.  One "step" = one GEMM over resident operands.  The JSON line
carries: `value` (device-timed TFLOP/s, whole job), `e2e` (same GEMM through the public
Python API from pinned HOST buffers, copies inside the timed region), `roofline` for the
GEMM kernel, `cpu_baseline` (the oracle's dequantise-then-matmul on the host cores, on a
bounded row sample), and sampled SM clocks.

With --gpus N > 1 (under torchrun) every rank runs the same GEMM on its own GPU: the GEMM
does not shard ("replicas only"), so scaling is weak and `value` is the sum over ranks.

--impl reference times the CPU restatement of the upstream torch reference path
(oracle/) on the host cores with every thread torch can use, on the same workload and
metric, each step a bounded sample of the rows.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEED = 2025 * 2024 + 2027  # upstream benchmark_mm.py:36

WORKLOADS = {
    # name: (metric, M, N, K)
    "mxfp8_gemm_8192": ("MXFP8 GEMM TFLOPS at M=N=K=8192", 8192, 8192, 8192),
    "nvfp4_gemm_8192": ("NVFP4 GEMM TFLOPS at M=N=K=8192", 8192, 8192, 8192),
    "int8_gemm_8192": ("row-scaled INT8 GEMM TOPS at M=N=K=8192", 8192, 8192, 8192),
    "int8_gemm_1024": ("row-scaled INT8 GEMM TOPS at M=N=K=1024", 1024, 1024, 1024),
    "bf16_gemm_8192": ("BF16 GEMM TFLOPS at M=N=K=8192", 8192, 8192, 8192),
}
# dense tensor-core rate of each kind relative to bf16 (B200: fp8/int8 2x, fp4 4x)
RATE_VS_BF16 = {"mxfp8": 2.0, "nvfp4": 4.0, "int8": 2.0, "bf16": 1.0}
SPEC_BF16_TFLOPS = 2250.0
# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the 2-CTA GEMM kernel
# from the committed ncu captures (profiles/gemm_*.md); None where no capture exists yet.
NCU_TRAFFIC_BYTES = {"mxfp8_gemm_8192": None, "bf16_gemm_8192": 1.098e9 + 0.160e9}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": p["hbm_gbs"], "bf16": p["bf16_tflops"], "bf16_sustained": p.get("bf16_tflops_sustained"), "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "src": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = "timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.fh = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=self.fh,
                stderr=subprocess.DEVNULL,
            )
        except Exception:
            self.proc = None

    def stop(self, t_begin: float | None = None, t_end: float | None = None) -> dict:
        """Median SM clock over the samples whose timestamp lies in [t_begin, t_end] (wall clock)."""
        import datetime

        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.fh.close()
        clocks, reasons, mx = [], set(), None
        with open(self.path) as fh:
            for line in fh:
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    clk, cmax = float(f[1]), float(f[2])
                except ValueError:
                    continue
                if t_begin is not None and not (t_begin <= ts <= t_end):
                    continue
                clocks.append(clk)
                mx = cmax
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        os.unlink(self.path)
        if clocks:
            out.update(sm_mhz=float(np.median(clocks)), sm_max_mhz=mx, reasons=sorted(reasons), samples=len(clocks))
        return out


# ------------------------------------------------------------------------------------------
# workload construction (GPU arm)
# ------------------------------------------------------------------------------------------
def build_gpu_workload(name: str, dev: torch.device):
    """Returns (step_fn(), host_step_fn or None, info) with operands resident on `dev`."""
    import gn_kernels_b200 as gk
    from gn_kernels_b200 import _lib, ops

    L = _lib.lib()
    metric, M, N, K = WORKLOADS[name]
    g = torch.Generator(device="cpu").manual_seed(SEED)
    A = torch.randn(M, K, generator=g, dtype=torch.float32).to(dev)
    Bt = torch.randn(N, K, generator=g, dtype=torch.float32).to(dev)
    P = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    stream = lambda: ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)  # noqa: E731
    C = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    kind = name.split("_")[0]

    if kind == "mxfp8":
        Aq, sfa = gk.quantize_mx(A.bfloat16(), torch.float8_e4m3fn, swizzled_scales=True)
        Bq, sfb = gk.quantize_mx(Bt.bfloat16(), torch.float8_e4m3fn, swizzled_scales=True)
        step = lambda: L.gnk_mm_mxfp8(P(Aq), K, P(Bq), K, P(sfa), P(sfb), P(C), N, M, N, K, stream())  # noqa: E731
        host_in = [Aq, Bq, sfa, sfb]
        api = lambda a, b, sa, sb: gk.cutedsl.sm100.sm100_mm_mxfp8.mm(a, b, sa, sb)  # noqa: E731
    elif kind == "nvfp4":
        tsa, tsb = ops.absmax(A, 2688.0), ops.absmax(Bt, 2688.0)
        Aq, sfa = gk.quantize_nvfp4_triton(A.bfloat16(), tsa)
        Bq, sfb = gk.quantize_nvfp4_triton(Bt.bfloat16(), tsb)
        alpha = float(tsa) * float(tsb)
        step = lambda: L.gnk_mm_nvfp4(P(Aq), K // 2, P(Bq), K // 2, P(sfa), P(sfb), alpha, P(C), N, M, N, K, stream())  # noqa: E731
        host_in = [Aq, Bq, sfa, sfb]
        api = lambda a, b, sa, sb: gk.cutedsl.sm100.sm100_mm_nvfp4.mm(a, b, sa, sb, alpha)  # noqa: E731
    elif kind == "int8":
        Aq, sA = gk.quantize_rowwise(A, torch.int8)
        Bq, sB = gk.quantize_rowwise(Bt, torch.int8)
        sA, sB = sA.view(M, 1), sB.view(1, N)
        step = lambda: L.gnk_mm_i8(P(Aq), K, P(Bq), K, P(C), N, M, N, K, P(sA), P(sB), None, 0, stream())  # noqa: E731
        host_in = [Aq, Bq, sA, sB]
        api = lambda a, b, sa, sb: gk.triton_mm(a, b.T, scale_A=sa, scale_B=sb)  # noqa: E731
    elif kind == "bf16":
        Ab, Bb = A.bfloat16(), Bt.bfloat16()
        step = lambda: L.gnk_mm_bf16(P(Ab), K, P(Bb), K, P(C), N, M, N, K, stream())  # noqa: E731
        host_in = [Ab, Bb]
        api = lambda a, b: gk.cutedsl.sm100.sm100_mm_bf16.mm(a, b.T)  # noqa: E731
    else:
        raise ValueError(name)

    pinned = [torch.empty(t.shape, dtype=t.dtype, device="cpu").pin_memory() for t in host_in]
    for p, t in zip(pinned, host_in):
        p.view(torch.uint8).copy_(t.view(torch.uint8)) if t.element_size() == 1 else p.copy_(t)
    out_host = torch.empty(M, N, dtype=torch.bfloat16).pin_memory()

    def host_step():
        dev_in = [p.to(dev, non_blocking=True) for p in pinned]
        out = api(*dev_in)
        out_host.copy_(out, non_blocking=True)

    info = {
        "metric": metric, "M": M, "N": N, "K": K, "kind": kind,
        "flops": 2.0 * M * N * K,
        "h2d": int(sum(p.numel() * p.element_size() for p in pinned)),
        "d2h": int(out_host.numel() * out_host.element_size()),
        "resident_bytes": int(sum(t.numel() * t.element_size() for t in host_in) + C.numel() * 2),
        "check": (host_in, C),
    }
    return step, host_step, info


# ------------------------------------------------------------------------------------------
# CPU arm: the oracle's dequantise-then-matmul on a bounded row sample
# ------------------------------------------------------------------------------------------
def build_cpu_workload(name: str, rows: int):
    from oracle import mm as omm
    from oracle import quant as oq

    metric, M, N, K = WORKLOADS[name]
    kind = name.split("_")[0]
    rows = min(rows, M)
    g = torch.Generator(device="cpu").manual_seed(SEED)
    A = torch.randn(M, K, generator=g, dtype=torch.float32)[:rows]
    Bt = torch.randn(N, K, generator=g, dtype=torch.float32)
    if kind == "mxfp8":
        Aq, sfa = oq.quantize_mx(A.bfloat16().float().numpy(), "e4m3")
        Bq, sfb = oq.quantize_mx(Bt.bfloat16().float().numpy(), "e4m3")
        step = lambda: omm.mm_mxfp8(Aq, Bq, sfa, sfb)  # noqa: E731
    elif kind == "nvfp4":
        Aq, sfa, tsa = oq.quantize_nvfp4(A.bfloat16().float().numpy())
        Bq, sfb, tsb = oq.quantize_nvfp4(Bt.bfloat16().float().numpy())
        step = lambda: omm.mm_nvfp4(Aq, Bq, sfa, sfb, float(tsa) * float(tsb))  # noqa: E731
    elif kind == "int8":
        Aq, sA = oq.quantize_rowwise(A.numpy(), "int8")
        Bq, sB = oq.quantize_rowwise(Bt.numpy(), "int8")
        step = lambda: omm.mm_i8_row_scaled(Aq, Bq, sA, sB)  # noqa: E731
    else:
        Ab, Bb = A.bfloat16(), Bt.bfloat16()
        step = lambda: omm.mm_bf16(Ab, Bb)  # noqa: E731
    return step, {"metric": metric, "flops": 2.0 * rows * N * K, "rows": rows, "M": M, "N": N, "K": K}


def time_cpu(step, steps: int, warmup: int):
    for _ in range(warmup):
        step()
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        ts.append(time.perf_counter() - t0)
    return float(np.sum(ts)), float(np.median(ts))


def unit_for(kind: str) -> str:
    return "TOP/s" if kind == "int8" else "TFLOP/s"


# ------------------------------------------------------------------------------------------
def run_reference(args, rank: int):
    if rank != 0:
        return
    step, info = build_cpu_workload(args.workload, args.cpu_rows)
    total, med = time_cpu(step, args.steps, max(1, min(args.warmup, 1)))
    kind = args.workload.split("_")[0]
    val = info["flops"] * args.steps / total / 1e12
    cores = torch.get_num_threads()
    sample = f"{info['rows']} of {info['M']} rows x all {info['N']} columns, K={info['K']} (dequantise + fp32 matmul + bf16 cast per step)"
    line = {
        "impl": "reference", "metric": info["metric"], "value": val, "unit": unit_for(kind), "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": kind, "data": "synthetic",
        "config": {"workload": args.workload, "M": info["M"], "N": info["N"], "K": info["K"], "sample": sample},
        "cpu_baseline": {"value": val, "unit": unit_for(kind), "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": unit_for(kind), "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "host_cpus": os.cpu_count(),
    }
    print(json.dumps(line), flush=True)


def run_gpu(args, rank: int, local_rank: int, world: int):
    import torch.distributed as dist

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from gn_kernels_b200 import _lib

    step, host_step, info = build_gpu_workload(args.workload, dev)
    kind = info["kind"]
    peaks = load_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(args.warmup, 3)):
        rc = step()
        if rc != 0:
            raise RuntimeError(f"kernel launch failed: status {rc}")
    _lib.raise_on_device_error()

    # ---- timed region: exactly K steps, per-launch events for the roofline ----
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.15)
    barrier()
    # Untimed lead-in of the same launches (about half a second) so that the 100 ms clock sampler
    # sees the GPU in the loaded state the timed steps run in; the timed region follows at once.
    t_load0 = time.time()
    lead_in = args.lead_in
    for _ in range(lead_in):
        step()
    evs[0].record()
    for i in range(args.steps):
        step()
        evs[i + 1].record()
    barrier()
    t_load1 = time.time()
    total_ms = evs[0].elapsed_time(evs[-1])
    per_launch = [evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps)]
    clocks = sampler.stop(t_load0 + 0.1, t_load1) if rank == 0 else None
    _lib.raise_on_device_error()

    # ---- end to end through the public API from pinned host buffers ----
    e2e_steps = max(2, min(args.steps, 5))
    host_step()
    barrier()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(e2e_steps):
        host_step()
    t1.record()
    barrier()
    e2e_ms = t0.elapsed_time(t1)

    t = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms = float(t[0]), float(t[1])

    if rank == 0:
        unit = unit_for(kind)
        value = world * info["flops"] * args.steps / (total_ms * 1e-3) / 1e12
        e2e_val = world * info["flops"] * e2e_steps / (e2e_ms * 1e-3) / 1e12
        avg_launch_ms = float(np.mean(per_launch))
        achieved = info["flops"] / (avg_launch_ms * 1e-3) / 1e12
        peak = peaks["bf16"] * RATE_VS_BF16[kind]
        roofline = {
            "bound": "tensor", "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
            "traffic": NCU_TRAFFIC_BYTES.get(args.workload),
            "peak_source": f"{RATE_VS_BF16[kind]:g} x cuBLAS bf16 burst {peaks['bf16']} TFLOP/s ({peaks['src']})",
            "frac_of_spec": achieved / (SPEC_BF16_TFLOPS * RATE_VS_BF16[kind]),
            "kernel_ms": avg_launch_ms,
        }
        # CPU baseline: the oracle on a bounded row sample (a few seconds of host time)
        cstep, cinfo = build_cpu_workload(args.workload, args.cpu_rows)
        ctot, _ = time_cpu(cstep, 2, 1)
        cpu_val = cinfo["flops"] * 2 / ctot / 1e12
        sample = f"{cinfo['rows']} of {cinfo['M']} rows x all {cinfo['N']} columns, K={cinfo['K']}, 2 timed passes"
        line = {
            "metric": info["metric"], "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": kind, "data": "synthetic",
            "config": {
                "workload": args.workload, "M": info["M"], "N": info["N"], "K": info["K"],
                "parallelism": "replicas only" if world > 1 else "single GPU",
                "l2": f"operands + output {info['resident_bytes'] / 2**20:.0f} MiB > 126 MB L2 (no flush needed)",
                "lead_in_steps": lead_in,
            },
            "roofline": roofline,
            "cpu_baseline": {"value": cpu_val, "unit": unit, "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": e2e_val, "unit": unit, "h2d_bytes_per_step": info["h2d"], "d2h_bytes_per_step": info["d2h"], "steps": e2e_steps},
            "gpu_launches": args.steps,
            "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"], "samples": clocks["samples"]},
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--lead-in", type=int, default=1000, help="untimed launches right before the timed region (clock sampling)")
    ap.add_argument("--workload", default="mxfp8_gemm_8192", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="gnk", choices=["gnk", "reference"])
    ap.add_argument("--cpu-rows", type=int, default=512, help="rows of A in the CPU sample (bounded host time)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product has no CPU path); use --impl reference for the CPU arm")
    run_gpu(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
