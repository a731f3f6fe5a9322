#!/usr/bin/env python
"""Benchmark of the quantized-matmul / quantizer / attention / GEMM + reduce-scatter hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference] [--kernel-only]

Default workload at EVERY N: the K-sharded BF16 GEMM + reduce-scatter, C[8192, 8192] =
A[8192, 28672] * B[28672, 8192] with K split evenly over the N ranks (strong scaling: the global
problem is fixed), every rank ending with its 8192/N rows of the reduced product.  N = 1 is the
plain GEMM the op degenerates to.  One "step" = one call of the op on resident operands.  Under
torchrun (N > 1) symmetric memory carries the exchange and every rank runs the same number of steps.

The JSON line carries: `value` (device-timed, whole job), `e2e` (the public Python API from pinned
HOST buffers, copies inside the timed region, copies of neighbouring steps overlapped with the
kernel), `roofline` (tensor and NVLink terms), `local_gemm_ms` (the same-shape GEMM without the
exchange, same run), `parity_max_rel_err` (sampled output rows of every rank against the CPU oracle,
outside the timed region), `comparators` (cuBLAS, and cuBLAS + NCCL reduce-scatter for N > 1),
`cpu_baseline` (N = 1), and the SM clocks sampled while the timed steps ran.

At N = 1 the line also has `extra`: one sub-record per remaining benchmark configuration (INT8
1024^3 and 8192^3, FP8 row-scaled, FP8 128-block-scaled, MXFP8 8192^3 and the skinny M = 16/64/128
shapes, NVFP4 8192^3, BF16 8192^3, the NVFP4 / MXFP8 / row-wise quantizers in GB/s, FP8-QK causal
attention), each with its own kernel time, roofline, clock samples and library comparators
(`torch.mm`, `torch._int_mm`, `torch._scaled_mm`, SDPA) timed interleaved in the same process.
--workload NAME makes NAME the main line instead (no extras).

--impl reference times the CPU restatement of the upstream torch reference path (oracle/) on the
host cores with every thread torch can use, same workload and metric, each step a bounded sample.
"""

from __future__ import annotations

import argparse
import ctypes
import datetime
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

SEED_MM = 2025 * 2024 + 2027  # upstream benchmark_mm.py:36
SEED_ATTN = 2025 * 2026  # upstream benchmark_attn.py:66
L2_BYTES = 126 * 2**20
SPEC_BF16_TFLOPS = 2250.0
NVLINK_GBS_MEASURED = 770.0  # peer copy per direction per GPU measured on this pool (nominal 900)
NVLINK_GBS_NOMINAL = 900.0
# dense tensor-core rate of each arithmetic kind relative to bf16 (B200: fp8/int8 2x, fp4 4x)
RATE_VS_BF16 = {"mxfp8": 2.0, "nvfp4": 4.0, "int8": 2.0, "bf16": 1.0, "fp8": 2.0}

# name -> (family, metric, shape)
WORKLOADS = {
    "bf16_gemm_rs": ("rs", "BF16 GEMM + reduce-scatter TFLOPS at M=N=8192, K=28672 sharded over the ranks", (8192, 8192, 28672)),
    "mxfp8_gemm_8192": ("gemm", "MXFP8 GEMM TFLOPS at M=N=K=8192", (8192, 8192, 8192)),
    "nvfp4_gemm_8192": ("gemm", "NVFP4 GEMM TFLOPS at M=N=K=8192", (8192, 8192, 8192)),
    "int8_gemm_8192": ("gemm", "row-scaled INT8 GEMM TOPS at M=N=K=8192", (8192, 8192, 8192)),
    "int8_gemm_1024": ("gemm", "row-scaled INT8 GEMM TOPS at M=N=K=1024", (1024, 1024, 1024)),
    "fp8_gemm_8192": ("gemm", "row-scaled FP8 GEMM TFLOPS at M=N=K=8192", (8192, 8192, 8192)),
    "fp8_block128_gemm_8192": ("gemm", "FP8 GEMM with 1x128 / 128x128 block scales, TFLOPS at M=N=K=8192", (8192, 8192, 8192)),
    "bf16_gemm_8192": ("gemm", "BF16 GEMM TFLOPS at M=N=K=8192", (8192, 8192, 8192)),
    "mxfp8_gemm_m16": ("gemm", "MXFP8 GEMM TFLOPS at M=16, N=K=8192", (16, 8192, 8192)),
    "mxfp8_gemm_m64": ("gemm", "MXFP8 GEMM TFLOPS at M=64, N=K=8192", (64, 8192, 8192)),
    "mxfp8_gemm_m128": ("gemm", "MXFP8 GEMM TFLOPS at M=128, N=K=8192", (128, 8192, 8192)),
    "nvfp4_quant_8192": ("quant", "NVFP4 quantizer GB/s at 8192x8192 bf16", (8192, 8192)),
    "mxfp8_quant_8192": ("quant", "MXFP8 quantizer GB/s at 8192x8192 bf16", (8192, 8192)),
    "rowwise_quant_attn": ("quant", "row-wise E4M3 quantizer GB/s on Q of the attention configuration (524288 rows of 128)", (4 * 4096 * 32, 128)),
    "attn_fp8_causal": ("attn", "FP8-QK causal GQA attention TFLOPS (B=4, Hq=32, Hkv=8, L=4096, D=128)", (4, 4096, 32, 8, 128)),
}
DEFAULT_WORKLOAD = "bf16_gemm_rs"
EXTRA_WORKLOADS = [
    "int8_gemm_1024", "int8_gemm_8192", "fp8_gemm_8192", "fp8_block128_gemm_8192", "mxfp8_gemm_8192", "mxfp8_gemm_m16", "mxfp8_gemm_m64",
    "mxfp8_gemm_m128", "nvfp4_gemm_8192", "bf16_gemm_8192", "nvfp4_quant_8192", "mxfp8_quant_8192", "rowwise_quant_attn", "attn_fp8_causal",
]
# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel, from the
# one-kernel ncu captures summarised under profiles/ (file named beside each figure)
NCU_TRAFFIC = {
    "bf16_gemm_rs": (6486.4e6 + 132.4e6, "profiles/ncu_counters_by_kernel.md (N = 1: the plain GEMM)"),
    "mxfp8_gemm_8192": (354.8e6 + 116.8e6, "profiles/ncu_counters_by_kernel.md"),
    "nvfp4_gemm_8192": (167.2e6 + 103.2e6, "profiles/ncu_counters_by_kernel.md"),
    "fp8_block128_gemm_8192": (698.8e6 + 127.9e6, "profiles/ncu_counters_by_kernel.md"),
    "mxfp8_gemm_m16": (69.4e6 + 1.2e6, "profiles/ncu_counters_by_kernel.md"),
    "attn_fp8_causal": (120.3e6 + 86.4e6, "profiles/ncu_counters_by_kernel.md"),
    "nvfp4_quant_8192": (134.2e6 + 20.2e6, "profiles/ncu_counters_by_kernel.md"),
    "mxfp8_quant_8192": (134.2e6 + 39.8e6, "profiles/ncu_counters_by_kernel.md"),
    "rowwise_quant_attn": (134.3e6 + 39.3e6, "profiles/ncu_counters_by_kernel.md"),
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": p["hbm_gbs"], "bf16": p["bf16_tflops"], "bf16_sustained": p.get("bf16_tflops_sustained") or p["bf16_tflops"], "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "src": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi (read-only query) while the GPU is loaded.
    One sampler runs for the whole process; window() picks the samples of a time interval."""

    Q = "timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int, period_ms: int = 50):
        self.index, self.proc, self.path, self.period_ms = index, None, None, period_ms

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.fh = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                stdout=self.fh, stderr=subprocess.DEVNULL,
            )
        except Exception:
            self.proc = None

    def _rows(self):
        rows = []
        if self.path is None or not os.path.exists(self.path):
            return rows
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
                rows.append((ts, clk, cmax, f[5:9]))
        return rows

    def window(self, t_begin: float, t_end: float) -> dict:
        """Median SM clock over the samples whose timestamp lies in [t_begin, t_end] (wall clock)."""
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        try:
            self.fh.flush()
        except Exception:
            pass
        rows = self._rows()
        inside = [r for r in rows if t_begin <= r[0] <= t_end]
        if not inside and rows:
            # a region shorter than the sampling period: the sample nearest to it, with its distance stated
            near = min(rows, key=lambda r: min(abs(r[0] - t_begin), abs(r[0] - t_end)))
            inside = [near]
            out["nearest_sample_ms_from_timed_region"] = round(1e3 * min(abs(near[0] - t_begin), abs(near[0] - t_end)), 1)
        reasons = set()
        for r in inside:
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if inside:
            out.update(sm_mhz=float(np.median([r[1] for r in inside])), sm_max_mhz=inside[-1][2], reasons=sorted(reasons),
                       samples=len(inside))
        return out

    def stop(self, t_begin: float | None = None, t_end: float | None = None) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        if t_begin is not None:
            out = self.window(t_begin, t_end)
        self.fh.close()
        if self.path and os.path.exists(self.path):
            os.unlink(self.path)
        self.proc = None
        return out


def _pin(t: torch.Tensor) -> torch.Tensor:
    p = torch.empty(t.shape, dtype=t.dtype, device="cpu").pin_memory()
    _copy(p, t)
    return p


def _copy(dst: torch.Tensor, src: torch.Tensor, non_blocking: bool = False) -> None:
    if dst.element_size() == 1:  # 8-bit float dtypes: copy the bytes
        dst.view(torch.uint8).copy_(src.view(torch.uint8), non_blocking=non_blocking)
    else:
        dst.copy_(src, non_blocking=non_blocking)


def _nbytes(ts) -> int:
    return int(sum(t.numel() * t.element_size() for t in ts))


# ------------------------------------------------------------------------------------------
# GPU arm: workloads
# ------------------------------------------------------------------------------------------
def build_gpu_workload(name: str, dev: torch.device, timeout_ms: int = 2000, rs_lagged_exit: bool = False) -> dict:
    """Operands resident on `dev`.  Returns step() (C ABI, preallocated outputs), api (the public
    Python call on device tensors), comparators (library calls of the same problem) and the accounting."""
    import gn_kernels_b200 as gk
    from gn_kernels_b200 import _lib, ops

    L = _lib.lib()
    family, metric, shape = WORKLOADS[name]
    P = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    stream = lambda: ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)  # noqa: E731
    kind = name.split("_")[0]
    w = {"name": name, "family": family, "metric": metric, "kind": kind, "config": {}, "comparators": {}, "dtype": kind}

    if family == "gemm":
        M, N, K = shape
        g = torch.Generator(device="cpu").manual_seed(SEED_MM)
        A = torch.randn(M, K, generator=g, dtype=torch.float32).to(dev)
        Bt = torch.randn(N, K, generator=g, dtype=torch.float32).to(dev)
        C = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        if name == "fp8_block128_gemm_8192":
            # DeepSeek-style operands: E4M3 codes, fp32 scale per (row, 128 K) of A and per 128 x 128 block of B
            Aq, Bq = A.to(torch.float8_e4m3fn), Bt.to(torch.float8_e4m3fn)
            sfa = (torch.rand(K // 128, M, generator=g) + 0.5).to(dev)  # M-major: element (m, kb) at kb * M + m
            sfb = (torch.rand(N // 128, K // 128, generator=g) + 0.5).to(dev)
            step = lambda: L.gnk_mm_f8_block128(P(Aq), K, P(sfa), M, P(Bq), K, P(sfb), K // 128, None, None, 0, P(C), N, M, N, K, stream())  # noqa: E731
            ins = [Aq, Bq, sfa, sfb]
            api = lambda a, b, sa, sb: gk.cutedsl.sm120.sm120_mm_fp8_1d2d.mm(a, sa.T, b, sb)  # noqa: E731
            algo_bytes = (M + N) * K + 2 * M * N
            w["kind"] = w["dtype"] = "fp8"
            sfa_mk = sfa.T.contiguous()  # [M, K/128] row-major for the library comparator

            def cublaslt_blockwise():
                from torch.nn.functional import ScalingType, SwizzleType, scaled_mm  # noqa: F401

                return scaled_mm(Aq, Bq.T, sfa_mk, ScalingType.BlockWise1x128, sfb, ScalingType.BlockWise128x128, output_dtype=torch.bfloat16)

            w["comparators"]["cuBLASLt blockwise (F.scaled_mm 1x128 / 128x128)"] = cublaslt_blockwise
        elif kind == "mxfp8":
            Aq, sfa = gk.quantize_mx(A.bfloat16(), torch.float8_e4m3fn, swizzled_scales=True)
            Bq, sfb = gk.quantize_mx(Bt.bfloat16(), torch.float8_e4m3fn, swizzled_scales=True)
            step = lambda: L.gnk_mm_mxfp8(P(Aq), K, P(Bq), K, P(sfa), P(sfb), P(C), N, M, N, K, stream())  # noqa: E731
            ins = [Aq, Bq, sfa, sfb]
            api = lambda a, b, sa, sb: gk.cutedsl.sm100.sm100_mm_mxfp8.mm(a, b, sa, sb)  # noqa: E731
            algo_bytes = N * K + N * K // 32 + M * K + M * K // 32 + 2 * M * N
            w["comparators"]["cuBLASLt MXFP8 (torch._scaled_mm)"] = lambda: torch._scaled_mm(Aq, Bq.T, sfa, sfb, out_dtype=torch.bfloat16)
            if M <= 128:
                # A decode step streams every layer's weights once: the launches rotate over four weight
                # matrices (268 MB, above twice the L2), so each one reads its 67 MB from DRAM and no
                # flush writes are needed between them.
                Ws = [(Bq, sfb)] + [(Bq.clone(), sfb.clone()) for _ in range(3)]
                turn = [0, 0]

                def step():
                    wq, ws = Ws[turn[0] & 3]
                    turn[0] += 1
                    return L.gnk_mm_mxfp8(P(Aq), K, P(wq), K, P(sfa), P(ws), P(C), N, M, N, K, stream())

                def cublaslt_rotating():
                    wq, ws = Ws[turn[1] & 3]
                    turn[1] += 1
                    return torch._scaled_mm(Aq, wq.T, sfa, ws, out_dtype=torch.bfloat16)

                w["comparators"] = {"cuBLASLt MXFP8 (torch._scaled_mm), same rotation": cublaslt_rotating}
                w["extra_resident"] = 3 * (Bq.numel() + sfb.numel())
                w["config"]["weights"] = "4 matrices of N x K in rotation, one per launch (inputs larger than L2)"
        elif kind == "nvfp4":
            tsa, tsb = ops.absmax(A, 2688.0), ops.absmax(Bt, 2688.0)
            Aq, sfa = gk.quantize_nvfp4_triton(A.bfloat16(), tsa)
            Bq, sfb = gk.quantize_nvfp4_triton(Bt.bfloat16(), tsb)
            alpha = float(tsa) * float(tsb)
            step = lambda: L.gnk_mm_nvfp4(P(Aq), K // 2, P(Bq), K // 2, P(sfa), P(sfb), alpha, P(C), N, M, N, K, stream())  # noqa: E731
            ins = [Aq, Bq, sfa, sfb]
            api = lambda a, b, sa, sb: gk.cutedsl.sm100.sm100_mm_nvfp4.mm(a, b, sa, sb, alpha)  # noqa: E731
            algo_bytes = (M + N) * (K // 2 + K // 16) + 2 * M * N
            w["comparators"]["cuBLASLt NVFP4 (torch._scaled_mm)"] = lambda: torch._scaled_mm(
                Aq.view(torch.float4_e2m1fn_x2), Bq.view(torch.float4_e2m1fn_x2).T, sfa.view(torch.float8_e4m3fn), sfb.view(torch.float8_e4m3fn),
                out_dtype=torch.bfloat16)
        elif kind == "int8":
            Aq, sA = gk.quantize_rowwise(A, torch.int8)
            Bq, sB = gk.quantize_rowwise(Bt, torch.int8)
            sA, sB = sA.view(M, 1), sB.view(1, N)
            step = lambda: L.gnk_mm_i8(P(Aq), K, P(Bq), K, P(C), N, M, N, K, P(sA), P(sB), None, 0, stream())  # noqa: E731
            ins = [Aq, Bq, sA, sB]
            api = lambda a, b, sa, sb: gk.triton_mm(a, b.T, scale_A=sa, scale_B=sb)  # noqa: E731
            algo_bytes = (M + N) * K + 2 * M * N
            Ci = torch.empty(M, N, dtype=torch.int32, device=dev)
            w["comparators"]["cuBLAS INT8 (torch._int_mm, int32 out, no scaling)"] = lambda: torch._int_mm(Aq, Bq.T, out=Ci)
            if (M + N) * K + 2 * M * N < 32 * 2**20:
                # A problem of a few MB would sit in L2 from one launch to the next: the launches rotate over
                # enough copies of the operands (and outputs) to exceed twice the L2, so no flush writes are needed
                copies = int(2.2 * L2_BYTES / ((M + N) * K + 2 * M * N)) + 1
                sets = [(Aq, Bq, C)] + [(Aq.clone(), Bq.clone(), torch.empty_like(C)) for _ in range(copies - 1)]
                turn8 = [0, 0]

                def step():
                    a, b, c = sets[turn8[0] % copies]
                    turn8[0] += 1
                    return L.gnk_mm_i8(P(a), K, P(b), K, P(c), N, M, N, K, P(sA), P(sB), None, 0, stream())

                def cublas_rotating():
                    a, b, _ = sets[turn8[1] % copies]
                    turn8[1] += 1
                    return torch._int_mm(a, b.T, out=Ci)

                w["comparators"] = {"cuBLAS INT8 (torch._int_mm, int32 out, no scaling), same rotation": cublas_rotating}
                w["extra_resident"] = (copies - 1) * ((M + N) * K + 2 * M * N)
                w["config"]["operands"] = f"{copies} copies of A, B and C in rotation, one per launch (inputs larger than L2)"
        elif kind == "fp8":
            Aq, sA = gk.quantize_rowwise(A, torch.float8_e4m3fn)
            Bq, sB = gk.quantize_rowwise(Bt, torch.float8_e4m3fn)
            sA, sB = sA.view(M, 1), sB.view(1, N)
            step = lambda: L.gnk_mm_f8(P(Aq), K, P(Bq), K, P(C), N, M, N, K, P(sA), P(sB), None, stream())  # noqa: E731
            ins = [Aq, Bq, sA, sB]
            api = lambda a, b, sa, sb: gk.triton_mm(a, b.T, scale_A=sa, scale_B=sb)  # noqa: E731
            algo_bytes = (M + N) * K + 2 * M * N
            w["comparators"]["cuBLASLt FP8 row-scaled (torch._scaled_mm)"] = lambda: torch._scaled_mm(Aq, Bq.T, sA, sB, out_dtype=torch.bfloat16)
        else:
            Ab, Bb = A.bfloat16(), Bt.bfloat16()
            step = lambda: L.gnk_mm_bf16(P(Ab), K, P(Bb), K, P(C), N, M, N, K, stream())  # noqa: E731
            ins = [Ab, Bb]
            api = lambda a, b: gk.cutedsl.sm100.sm100_mm_bf16.mm(a, b.T)  # noqa: E731
            algo_bytes = 2 * (M + N) * K + 2 * M * N
            w["comparators"]["cuBLAS BF16 (torch.mm)"] = lambda: torch.mm(Ab, Bb.T, out=C)
        del A, Bt
        w.update(work=2.0 * M * N * K, unit="TOP/s" if kind == "int8" else "TFLOP/s", scale=1e12, ins=ins, outs=[C], api=api, step=step,
                 algo_bytes=algo_bytes, bound="hbm" if M <= 128 else "tensor", config={"M": M, "N": N, "K": K, **w["config"]})
    elif family == "rs":
        # K is sharded over the ranks (strong scaling: the global problem is fixed); every rank ends
        # with its M/world rows of the reduced product.  One rank: the plain GEMM it degenerates to.
        import torch.distributed as dist

        M, N, Kt = shape
        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        Kl = Kt // world
        g = torch.Generator(device="cpu").manual_seed(SEED_MM + rank)
        x = (torch.randn(M, Kl, generator=g) / Kt**0.5).bfloat16().to(dev)
        wt = (torch.randn(N, Kl, generator=g) / Kt**0.5).bfloat16().to(dev)
        out = torch.empty(M // world, N, dtype=torch.bfloat16, device=dev)
        full = torch.empty(M, N, dtype=torch.bfloat16, device=dev)  # the local GEMM without exchange writes here
        path = "single GPU: plain GEMM"
        if world > 1:
            import torch.distributed._symmetric_memory as symm_mem

            from gn_kernels_b200.cutedsl.sm100.sm100_gemm_rs import flag_words, gemm_rs

            partial = symm_mem.empty(M, N, dtype=torch.bfloat16, device=dev)
            ph = symm_mem.rendezvous(partial, dist.group.WORLD)
            flags = symm_mem.empty(flag_words(M, N, world), dtype=torch.int32, device=dev)
            flags.zero_()
            fh = symm_mem.rendezvous(flags, dist.group.WORLD)
            torch.cuda.synchronize(dev)
            dist.barrier()
            path = "pull: multimem.ld_reduce on the NVLink multicast address" if getattr(ph, "multicast_ptr", 0) else "push: bulk stores into the owner's slots"

            def step():
                # every call ends with the exit barrier across the ranks unless --rs-lagged-exit defers it
                gemm_rs(x, wt, partial, ph, out, flags, fh, timeout_ms=timeout_ms, lagged_exit=rs_lagged_exit)
                return 0

            def api(a, b):
                o = torch.empty_like(out)
                return gemm_rs(a, b, partial, ph, o, flags, fh, timeout_ms=timeout_ms)

            def cublas_nccl():
                torch.mm(x, wt.T, out=full)
                dist.reduce_scatter_tensor(out, full)

            w["comparators"]["cuBLAS BF16 GEMM + NCCL reduce_scatter (unfused, one stream)"] = cublas_nccl
            w["extra_resident"] = partial.numel() * 2
        else:
            step = lambda: L.gnk_mm_bf16(P(x), Kl, P(wt), Kl, P(out), N, M, N, Kl, stream())  # noqa: E731
            api = lambda a, b: gk.cutedsl.sm100.sm100_mm_bf16.mm(a, b.T)  # noqa: E731
            w["comparators"]["cuBLAS BF16 (torch.mm)"] = lambda: torch.mm(x, wt.T, out=full)
        w["local_gemm"] = lambda: L.gnk_mm_bf16(P(x), Kl, P(wt), Kl, P(full), N, M, N, Kl, stream())
        w["parity_inputs"] = (x, wt, out)
        w.update(work=2.0 * M * N * Kt / world, unit="TFLOP/s", scale=1e12, ins=[x, wt], outs=[out], api=api, step=step, kind="bf16", dtype="bf16",
                 algo_bytes=2 * (M + N) * Kl + 2 * M * N, bound="tensor", scaling="strong", world=world,
                 nvlink_bytes=(world - 1) * M * N * 2 // world,
                 config={"M": M, "N": N, "K_total": Kt, "K_per_rank": Kl, "data_path": path, "timeout_ms": timeout_ms,
                         "exit_barrier": ("none (one rank)" if world == 1 else "signalled at the end of a call, waited for before the next call's first store (lagged_exit=1)"
                                          if rs_lagged_exit else "signalled and waited for at the end of every call (lagged_exit=0)"),
                         "nvlink_bytes_per_rank": (world - 1) * M * N * 2 // world})
    elif family == "quant":
        M, K = shape
        g = torch.Generator(device="cpu").manual_seed(SEED_MM)
        x = torch.randn(M, K, generator=g, dtype=torch.float32).bfloat16().to(dev)
        if kind == "nvfp4":
            ts = ops.absmax(x, 2688.0)
            q = torch.empty(M, K // 2, dtype=torch.uint8, device=dev)
            sf = torch.empty(M, K // 16, dtype=torch.uint8, device=dev)
            step = lambda: L.gnk_quant_nvfp4(P(x), 0, M, K, K, P(ts), 1e-12, P(q), P(sf), 1, stream())  # noqa: E731
            api = lambda xx: gk.quantize_nvfp4_triton(xx, ts)[0]  # noqa: E731
            nbytes = 2 * M * K + M * K // 2 + M * K // 16
            cfg = {"M": M, "K": K, "tensor_scale": "precomputed amax/(6*448), not in the timed step"}
        elif kind == "mxfp8":
            q = torch.empty(M, K, dtype=torch.uint8, device=dev)
            sf = torch.empty(M, K // 32, dtype=torch.uint8, device=dev)
            step = lambda: L.gnk_quant_mx(P(x), 0, M, K, K, 1, 0, P(q), P(sf), 1, stream())  # noqa: E731
            api = lambda xx: gk.quantize_mx(xx, torch.float8_e4m3fn, swizzled_scales=True)[0]  # noqa: E731
            nbytes = 2 * M * K + M * K + M * K // 32
            cfg = {"M": M, "K": K}
        else:
            q = torch.empty(M, K, dtype=torch.uint8, device=dev)
            sf = torch.empty(M, dtype=torch.float32, device=dev)
            step = lambda: L.gnk_quant_rowwise(P(x), 0, M, K, K, 1, P(q), P(sf), 0, 0, stream())  # noqa: E731
            api = lambda xx: gk.quantize_rowwise(xx, torch.float8_e4m3fn)[0]  # noqa: E731
            nbytes = 2 * M * K + M * K + 4 * M
            cfg = {"rows": M, "cols": K}
        dst = torch.empty(nbytes // 2, dtype=torch.uint8, device=dev)
        src = torch.empty(nbytes // 2, dtype=torch.uint8, device=dev)
        w["comparators"]["device copy moving the same number of bytes (torch copy_)"] = lambda: dst.copy_(src)
        w.update(work=float(nbytes), unit="GB/s", scale=1e9, ins=[x], outs=[q, sf], api=api, step=step, algo_bytes=nbytes, bound="hbm",
                 config=cfg, dtype="f32")
    else:
        B, Lq, Hq, Hkv, D = shape
        g = torch.Generator(device="cpu").manual_seed(SEED_ATTN)
        qf = torch.randn(B, Lq, Hq, D, generator=g).bfloat16().to(dev)
        kf = torch.randn(B, Lq, Hkv, D, generator=g).bfloat16().to(dev)
        v = torch.randn(B, Lq, Hkv, D, generator=g).bfloat16().to(dev)
        qq, sq = gk.quantize_rowwise(qf, torch.float8_e4m3fn, transpose_scales=True)
        kq, sk = gk.quantize_rowwise(kf, torch.float8_e4m3fn, transpose_scales=True)
        o = torch.empty(B, Lq, Hq, D, dtype=torch.bfloat16, device=dev)
        I3 = ctypes.c_int64 * 3
        st = [I3(*t.stride()[:3]) for t in (qq, kq, v, o)]
        step = lambda: L.gnk_attn_fwd(P(qq), P(kq), P(v), P(o), P(sq), P(sk), 1, 0, 0, B, Lq, Lq, Hq, Hkv, D, st[0], st[1], st[2], st[3], 1, stream())  # noqa: E731
        api = lambda a, b, c, d, e: gk.triton_attn(a, b, c, d, e, causal=True)  # noqa: E731
        qt, kt, vt = qf.transpose(1, 2), kf.transpose(1, 2), v.transpose(1, 2)  # [B, H, L, D] views for SDPA
        w["comparators"]["torch SDPA bf16 causal GQA (library flash attention, unquantised QK)"] = lambda: torch.nn.functional.scaled_dot_product_attention(
            qt, kt, vt, is_causal=True, enable_gqa=True)
        w.update(work=4.0 * B * Hq * Lq * Lq * D / 2, unit="TFLOP/s", scale=1e12, ins=[qq, kq, v, sq, sk], outs=[o], api=api, step=step,
                 algo_bytes=_nbytes([qq, kq, v, sq, sk, o]), bound="tensor", dtype="fp8",
                 config={"B": B, "L": Lq, "Hq": Hq, "Hkv": Hkv, "D": D, "causal": True, "flops": "causal half of 4*B*Hq*L*L*D"})

    w["resident_bytes"] = _nbytes(w["ins"]) + _nbytes(w["outs"]) + w.get("extra_resident", 0)
    return w


class HostPipeline:
    """End-to-end step through the public API from pinned host buffers: the inputs go host -> device,
    the op runs, the result comes device -> host.  Two input buffers and separate copy streams let the
    copy-in of step i+1 and the copy-out of step i-1 overlap the kernel of step i (PCIe is full duplex);
    every byte of every step is still copied inside the timed region."""

    def __init__(self, w: dict, dev: torch.device):
        self.w, self.dev = w, dev
        self.pinned = [_pin(t) for t in w["ins"]]
        out0 = w["outs"][0]
        self.out_host = [torch.empty(out0.shape, dtype=out0.dtype).pin_memory() for _ in range(2)]
        self.dev_in = [[torch.empty_like(t) for t in w["ins"]] for _ in range(2)]
        self.s_in, self.s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        self.ev_in = [torch.cuda.Event() for _ in range(2)]
        self.ev_free = [torch.cuda.Event() for _ in range(2)]
        self.ev_out = [torch.cuda.Event() for _ in range(2)]
        self.i = 0
        self.h2d = _nbytes(self.pinned)
        self.d2h = _nbytes([self.out_host[0]])

    def step(self):
        b = self.i & 1
        comp = torch.cuda.current_stream(self.dev)
        with torch.cuda.stream(self.s_in):
            if self.i >= 2:
                self.s_in.wait_event(self.ev_free[b])  # the kernel that last read this buffer has finished
            for d, p in zip(self.dev_in[b], self.pinned):
                _copy(d, p, non_blocking=True)
            self.ev_in[b].record(self.s_in)
        comp.wait_event(self.ev_in[b])
        out = self.w["api"](*self.dev_in[b])
        self.ev_free[b].record(comp)
        done = torch.cuda.Event()
        done.record(comp)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(done)
            if self.i >= 2:
                self.s_out.wait_event(self.ev_out[b])
            _copy(self.out_host[b], out, non_blocking=True)
            out.record_stream(self.s_out)
            self.ev_out[b].record(self.s_out)
        self.i += 1

    def drain(self):
        comp = torch.cuda.current_stream(self.dev)
        comp.wait_stream(self.s_in)
        comp.wait_stream(self.s_out)


# ------------------------------------------------------------------------------------------
# CPU arm: the oracle on a bounded sample of the same workload
# ------------------------------------------------------------------------------------------
def build_cpu_workload(name: str, rows: int):
    from oracle import attn as oattn
    from oracle import mm as omm
    from oracle import quant as oq

    family, metric, shape = WORKLOADS[name]
    kind = name.split("_")[0]
    if family in ("gemm", "rs"):  # the reduce-scatter's CPU arm is the global product on the row sample
        M, N, K = shape
        rows = min(rows, M)
        g = torch.Generator(device="cpu").manual_seed(SEED_MM)
        A = torch.randn(M, K, generator=g, dtype=torch.float32)[:rows]
        Bt = torch.randn(N, K, generator=g, dtype=torch.float32)
        if name == "fp8_block128_gemm_8192":
            Aq = A.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
            Bq = Bt.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
            sfa = torch.rand(rows, K // 128, generator=g) + 0.5
            sfb = torch.rand(N // 128, K // 128, generator=g) + 0.5
            step = lambda: omm.mm_f8_block128(Aq, sfa, Bq, sfb)  # noqa: E731
        elif kind == "mxfp8":
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
        elif kind == "fp8":
            Aq, sA = oq.quantize_rowwise(A.numpy(), "e4m3")
            Bq, sB = oq.quantize_rowwise(Bt.numpy(), "e4m3")
            step = lambda: omm.mm_f8_row_scaled(Aq, Bq, sA, sB)  # noqa: E731
        else:
            Ab, Bb = A.bfloat16(), Bt.bfloat16()
            step = lambda: omm.mm_bf16(Ab, Bb)  # noqa: E731
        sample = f"{rows} of {M} rows x all {N} columns, K={K} (dequantise + fp32 matmul + bf16 cast per step)"
        return step, 2.0 * rows * N * K, sample
    if family == "quant":
        M, K = shape
        rows = min(rows, M) if kind != "rowwise" else min(rows * 64, M)
        g = torch.Generator(device="cpu").manual_seed(SEED_MM)
        x = torch.randn(rows, K, generator=g, dtype=torch.float32).bfloat16().float().numpy()
        if kind == "nvfp4":
            ts = np.float32(np.abs(x).max() / 2688.0)
            step = lambda: oq.quantize_nvfp4(x, ts)  # noqa: E731
            work = float(2 * rows * K + rows * K // 2 + rows * K // 16)
        elif kind == "mxfp8":
            step = lambda: oq.quantize_mx(x, "e4m3")  # noqa: E731
            work = float(3 * rows * K + rows * K // 32)
        else:
            step = lambda: oq.quantize_rowwise(x, "e4m3")  # noqa: E731
            work = float(3 * rows * K + 4 * rows)
        return step, work, f"{rows} of {M} rows (numpy restatement of the upstream quantizer)"
    B, L, Hq, Hkv, D = shape
    g = torch.Generator(device="cpu").manual_seed(SEED_ATTN)
    heads = 2
    q = torch.randn(1, L, heads, D, generator=g).bfloat16()
    k = torch.randn(1, L, 1, D, generator=g).bfloat16()
    v = torch.randn(1, L, 1, D, generator=g).bfloat16()
    qq, sq = oq.quantize_rowwise(q.float().numpy(), "e4m3")
    kq, sk = oq.quantize_rowwise(k.float().numpy(), "e4m3")
    sq_t = torch.from_numpy(sq).permute(0, 2, 1).contiguous()
    sk_t = torch.from_numpy(sk).permute(0, 2, 1).contiguous()
    step = lambda: oattn.attention_qk_quantized(qq, kq, v, sq_t, sk_t, kind="e4m3", causal=True)  # noqa: E731
    return step, 4.0 * heads * L * L * D / 2, f"1 of {B} batches x {heads} of {Hq} query heads (dequantise + fp32 softmax attention)"


def time_cpu(step, steps: int, warmup: int) -> float:
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    return time.perf_counter() - t0


def run_reference(args, rank: int):
    if rank != 0:
        return
    family, metric, shape = WORKLOADS[args.workload]
    kind = args.workload.split("_")[0]
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        # a multi-rank launcher pins every rank to one OpenMP thread; this arm is a host benchmark on
        # rank 0 alone, so it takes every core it can get back
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    step, work, sample = build_cpu_workload(args.workload, args.cpu_rows)
    # Keep the whole run within a few minutes whatever --steps says: one probe step; if K steps would
    # take longer than about three minutes, fewer steps are executed and the line says how many.
    t_probe = time_cpu(step, 1, 0)
    executed = args.steps
    if t_probe * args.steps > 180.0:
        executed = max(2, int(180.0 / t_probe))
    total = time_cpu(step, executed, 0) * args.steps / executed
    unit, scale = ("GB/s", 1e9) if family == "quant" else (("TOP/s" if kind == "int8" else "TFLOP/s"), 1e12)
    val = work * args.steps / total / scale
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": metric, "value": val, "unit": unit, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total / args.steps * 1e3, "higher_is_better": True, "scaling": "strong" if family == "rs" else "weak", "vs_baseline": None,
        "dtype": "bf16" if family == "rs" else kind,
        "data": "synthetic", "config": {"workload": args.workload, "shape": list(shape), "sample": sample},
        "cpu_baseline": {"value": val, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "host_cpus": os.cpu_count(), "steps_executed": executed,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm: measurement
# ------------------------------------------------------------------------------------------
class Runner:
    def __init__(self, args, rank, local_rank, world):
        import torch.distributed as dist

        self.args, self.rank, self.world, self.dist = args, rank, world, dist
        self.dev = torch.device("cuda", local_rank)
        torch.cuda.set_device(self.dev)
        if world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.peaks = load_peaks()
        self.sampler = ClockSampler(local_rank)
        if rank == 0:
            self.sampler.start()
        self.flush_buf = None

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize(self.dev)

    def max_over_ranks(self, vals):
        t = torch.tensor(vals, dtype=torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t]

    def flush(self):
        if self.flush_buf is None:
            self.flush_buf = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=self.dev)
        self.flush_buf.zero_()

    def lead_in_count(self, fn, seconds: float) -> int:
        """Launch count that keeps the GPU busy for about `seconds`: the same on every rank."""
        torch.cuda.synchronize(self.dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            fn()
        e1.record()
        torch.cuda.synchronize(self.dev)
        ms = self.max_over_ranks([e0.elapsed_time(e1) / 3])[0]
        self.last_est_ms = ms
        return int(max(1, min(20000, seconds * 1e3 / max(ms, 1e-3))))

    def timed(self, fn, steps: int, flush: bool, graph: bool = False):
        """K launches.  Returns (ms of the whole region, per-launch ms list).  With an L2 flush between
        steps every launch has its own event pair (the flushes are not part of a step); otherwise ONE
        pair brackets the K back-to-back launches and the per-launch time is their mean (an event
        record between two launches keeps the second from starting as the first drains).  `graph`:
        the K launches are captured into a CUDA graph first and the timed region is one replay of it
        (for kernels of a few tens of microseconds, where the host cannot issue launches fast enough
        to keep them back to back); if the capture fails the launches are issued directly."""
        if not flush and graph:
            try:
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr):
                    for _ in range(steps):
                        fn()
                gr.replay()  # instantiation and upload happen here, untimed
                torch.cuda.synchronize(self.dev)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                gr.replay()
                e1.record()
                self.barrier()
                total = e0.elapsed_time(e1)
                self.graph_used = True
                return total, [total / steps] * steps
            except Exception:
                torch.cuda.synchronize(self.dev)
        if not flush:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            self.barrier()
            total = e0.elapsed_time(e1)
            return total, [total / steps] * steps
        ev0 = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        ev1 = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        for i in range(steps):
            self.flush()
            ev0[i].record()
            fn()
            ev1[i].record()
        self.barrier()
        per = [a.elapsed_time(b) for a, b in zip(ev0, ev1)]
        return float(np.sum(per)), per

    def measure(self, name: str, steps: int, warmup: int, main: bool) -> dict:
        from gn_kernels_b200 import _lib

        args = self.args
        w = build_gpu_workload(name, self.dev, args.timeout_ms, args.rs_lagged_exit)
        step = w["step"]
        flush = w["resident_bytes"] < 1.5 * L2_BYTES  # operands could stay in L2 between steps: flush it
        warm = max(warmup, 3)
        for _ in range(warm):
            rc = step()
            if rc != 0:
                raise RuntimeError(f"{name}: kernel launch failed: status {rc}")
        _lib.raise_on_device_error()

        # Untimed lead-in of the same launches so that the clock sampler sees the GPU in the loaded
        # state the timed steps run in; the timed region follows at once.
        lead = self.lead_in_count(step, args.lead_in_s)
        self.barrier()
        t_load0 = time.time()
        for i in range(lead):
            step()
            if (i & 63) == 63:
                torch.cuda.synchronize(self.dev)
        self.barrier()
        # short kernels (under 0.1 ms) on one GPU: the timed launches are replayed from a CUDA graph
        use_graph = self.world == 1 and not flush and self.last_est_ms < 0.1
        self.graph_used = False
        total_ms, per = self.timed(step, steps, flush, use_graph)
        launch_mode = "one CUDA graph holding the timed launches" if self.graph_used else "launches issued one by one from the host"
        t_load1 = time.time()
        _lib.raise_on_device_error()
        total_ms = self.max_over_ranks([total_ms])[0]
        clocks = self.sampler.window(t_load0 + 0.1, t_load1) if self.rank == 0 else None
        avg_ms = float(np.mean(per))
        rec = {"workload": name, "metric": w["metric"], "unit": w["unit"], "dtype": w["dtype"], "steps": steps, "ms_per_step": total_ms / steps,
               "kernel_ms": avg_ms, "value": self.world * w["work"] * steps / (total_ms * 1e-3) / w["scale"], "clocks": clocks,
               "config": {"workload": name, **w["config"], "lead_in_steps": lead, "timed_launches": launch_mode,
                          "l2": (f"operands + output {w['resident_bytes'] / 2**20:.0f} MiB > 126 MB L2 (no flush needed), back-to-back launches"
                                 if not flush else
                                 f"operands + output {w['resident_bytes'] / 2**20:.0f} MiB could stay in L2: 252 MiB written between steps, steps timed one by one")}}
        rec["roofline"] = self.roofline(w, avg_ms, sustained=lead * avg_ms > 200.0)
        if clocks and clocks.get("sm_mhz"):
            # throughput follows the SM clock on this power-capped part: time x clock compares runs on different boxes
            rec["roofline"]["achieved_per_sm_mhz"] = rec["roofline"]["achieved"] / clocks["sm_mhz"]

        # SM clock seen from inside the kernel: the same launches once more, back to back, with the
        # library's trace hook on (cycle counter and wall clock at entry and exit of CTA 0)
        if (w["family"] == "gemm" or (w["family"] == "rs" and self.world == 1)) and name != "fp8_block128_gemm_8192" and not flush:
            rec["in_kernel"] = self.in_kernel_clock(step, max(steps, lead // 2))

        # local GEMM of the same shape without the exchange (reduce-scatter workload only), same run
        if "local_gemm" in w:
            lg = w["local_gemm"]
            for _ in range(3):
                lg()
            n = self.lead_in_count(lg, min(args.lead_in_s, 0.3))
            for _ in range(n):
                lg()
            self.barrier()
            lt, _ = self.timed(lg, steps, False)
            rec["local_gemm_ms"] = self.max_over_ranks([lt / steps])[0]
            rec["frac_of_local_gemm_rate"] = rec["local_gemm_ms"] / rec["ms_per_step"]

        # library comparators, interleaved with our kernel round by round in this process
        if w["comparators"] and not args.kernel_only:
            rec["comparators"] = self.compare(w, flush, min(steps, 20), rounds=5, graph=use_graph)

        # parity of the reduce-scatter output, outside every timed region
        if "parity_inputs" in w and not args.kernel_only:
            rec.update(self.rs_parity(w))

        if main and not args.kernel_only:
            hp = HostPipeline(w, self.dev)
            e2e_steps = max(3, min(steps, 8))
            hp.step()
            hp.step()
            hp.drain()
            self.barrier()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(e2e_steps):
                hp.step()
            hp.drain()
            t1.record()
            self.barrier()
            e2e_ms = self.max_over_ranks([t0.elapsed_time(t1)])[0]
            _lib.raise_on_device_error()
            rec["e2e"] = {"value": self.world * w["work"] * e2e_steps / (e2e_ms * 1e-3) / w["scale"], "unit": w["unit"], "h2d_bytes_per_step": hp.h2d,
                          "d2h_bytes_per_step": hp.d2h, "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                          "how": "public API on pinned host buffers; copy-in of step i+1 and copy-out of step i-1 overlap the kernel of step i on separate streams"}
            del hp
        rec["_w"] = w
        return rec

    def in_kernel_clock(self, step, n: int) -> dict:
        """Cycles and nanoseconds CTA 0 of the last of `n` back-to-back launches (about as many as the
        lead-in, so the clock has settled under load again) spent in the kernel."""
        from gn_kernels_b200 import _lib

        L = _lib.lib()
        span_at = 2 * 2 * 256 * 3
        buf = torch.zeros(span_at + 4, dtype=torch.int64, device=self.dev)
        L.gnk_debug_trace(ctypes.c_void_p(buf.data_ptr()))
        try:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n):
                step()
            e1.record()
            torch.cuda.synchronize(self.dev)
        finally:
            L.gnk_debug_trace(None)
        c0, t0, c1, t1 = (int(v) for v in buf[span_at:].tolist())
        cycles, ns = c1 - c0, t1 - t0
        return {"sm_cycles": cycles, "ns": ns, "sm_mhz": cycles / ns * 1e3 if ns > 0 else None, "event_ms_per_launch": e0.elapsed_time(e1) / n,
                "what": "clock64 and globaltimer at entry and exit of CTA 0, last of the launches; globaltimer ticks in steps of up to 1 us"}

    def roofline(self, w: dict, avg_ms: float, sustained: bool) -> dict:
        peaks = self.peaks
        traffic = NCU_TRAFFIC.get(w["name"])
        if w["bound"] == "tensor":
            achieved = w["work"] / (avg_ms * 1e-3) / 1e12
            bf16_peak = peaks["bf16_sustained"] if sustained else peaks["bf16"]
            rate = 4.0 / 3.0 if w["family"] == "attn" else RATE_VS_BF16[w["kind"]]
            peak = bf16_peak * rate
            why = "FP8 QK^T at 2x + BF16 PV at 1x of equal flops -> 4/3 x" if w["family"] == "attn" else f"{rate:g} x"
            r = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                 "traffic": traffic[0] if traffic else None, "traffic_source": traffic[1] if traffic else None,
                 "peak_source": f"{why} cuBLAS bf16 {'sustained' if sustained else 'burst'} {bf16_peak} TFLOP/s ({peaks['src']})",
                 "frac_of_spec": achieved / (SPEC_BF16_TFLOPS * rate), "kernel_ms": avg_ms}
            if w["family"] == "rs":
                # a fused compute + collective kernel is bounded by the slower of the GEMM at the tensor peak and
                # the bytes that must cross NVLink at the link rate
                t_gemm = w["work"] / (peak * 1e12) * 1e3
                t_link = w["nvlink_bytes"] / (NVLINK_GBS_MEASURED * 1e9) * 1e3
                t_roof = max(t_gemm, t_link)
                r.update(terms={"gemm_ms_at_tensor_peak": t_gemm, "nvlink_ms_at_770_GBs_measured": t_link,
                                "nvlink_ms_at_900_GBs_nominal": w["nvlink_bytes"] / (NVLINK_GBS_NOMINAL * 1e9) * 1e3,
                                "roofline_ms": t_roof, "bound_by": "tensor" if t_gemm >= t_link else "nvlink"},
                         frac=t_roof / avg_ms, frac_is="max(GEMM time at the tensor peak, NVLink time at the measured link rate) / kernel time")
            return r
        achieved = w["algo_bytes"] / (avg_ms * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                "traffic": traffic[0] if traffic else None, "traffic_source": traffic[1] if traffic else None, "algorithmic_bytes": w["algo_bytes"],
                "peak_source": f"copy bandwidth {peaks['hbm_gbs']} GB/s ({peaks['src']})", "kernel_ms": avg_ms}

    def compare(self, w: dict, flush: bool, n: int, rounds: int, graph: bool = False) -> dict:
        """Median per-launch time of our kernel and of each library call, alternating round by round."""
        out = {}
        ours = w["step"]
        for cname, cfn in w["comparators"].items():
            try:
                for _ in range(3):
                    cfn()
                torch.cuda.synchronize(self.dev)
            except Exception as exc:  # the library has no kernel for this problem on this box
                out[cname] = {"unavailable": str(exc).splitlines()[0][:200]}
                continue
            mine, theirs = [], []
            for _ in range(rounds):
                self.barrier()
                tm, pm = self.timed(ours, n, flush, graph)
                tt, pt = self.timed(cfn, n, flush, graph)
                mine.append(tm / n)
                theirs.append(tt / n)
            m, t = self.max_over_ranks([float(np.median(mine)), float(np.median(theirs))])
            scale = self.world * w["work"] / w["scale"]
            out[cname] = {"ms": t, "value": scale / (t * 1e-3), "ours_ms_same_rounds": m, "ours_value_same_rounds": scale / (m * 1e-3),
                          "ours_over_theirs": t / m, "rounds": rounds, "launches_per_round": n}
        return out

    def rs_parity(self, w: dict) -> dict:
        """Sampled rows of every rank's output against the CPU oracle (bf16-rounded partials, fp32 sum)."""
        from oracle import gemm_rs as ors
        from oracle.mm import max_rel_err

        dist, world, rank = self.dist, self.world, self.rank
        x, wt, out = w["parity_inputs"]
        M = x.shape[0]
        rows_per = M // world
        per_rank = max(4, 64 // world)
        gsel = torch.Generator().manual_seed(7)
        local_rows = torch.sort(torch.randperm(rows_per, generator=gsel)[:per_rank]).values
        global_rows = torch.cat([local_rows + r * rows_per for r in range(world)]).to(self.dev)
        out.zero_()
        self.barrier()
        rc = w["step"]()
        self.barrier()
        xs_rows = x.index_select(0, global_rows).contiguous()
        mine = out.index_select(0, local_rows.to(self.dev)).contiguous()
        if world > 1:
            xs = [torch.empty_like(xs_rows) for _ in range(world)]
            ws = [torch.empty_like(wt) for _ in range(world)]
            outs = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(xs, xs_rows)
            dist.all_gather(ws, wt)
            dist.all_gather(outs, mine)
        else:
            xs, ws, outs = [xs_rows], [wt], [mine]
        res = {}
        if rank == 0:
            torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
            refs = ors.gemm_rs([t.cpu() for t in xs], [t.cpu() for t in ws])  # slices the sampled rows by owner
            errs = [max_rel_err(o.cpu(), r) for o, r in zip(outs, refs)]
            res = {"parity_max_rel_err": max(errs), "parity": {"rows_per_rank": per_rank, "ranks": world, "tolerance": 1e-2,
                                                              "ok": bool(max(errs) <= 1e-2), "rc": int(rc or 0),
                                                              "checker": "oracle.gemm_rs on the host (sum over ranks of bf16(x_r w_r^T), fp32 adds)"}}
        self.barrier()
        return res

    def cpu_baseline(self, name: str, unit: str, scale: float) -> dict:
        cstep, cwork, sample = build_cpu_workload(name, self.args.cpu_rows)
        ctot = time_cpu(cstep, 2, 1)
        return {"value": cwork * 2 / ctot / scale, "unit": unit, "cores": torch.get_num_threads(), "kind": "port", "sample": sample + ", 2 timed passes"}

    def run(self):
        args, world, rank = self.args, self.world, self.rank
        main = self.measure(args.workload, args.steps, args.warmup, main=True)
        w = main.pop("_w")
        extras = []
        if world == 1 and args.workload == DEFAULT_WORKLOAD and not args.no_extra and not args.kernel_only:
            del w
            torch.cuda.empty_cache()
            for name in EXTRA_WORKLOADS:
                try:
                    r = self.measure(name, max(20, min(args.steps, 100)), 3, main=False)
                    r.pop("_w")
                except Exception as exc:
                    r = {"workload": name, "error": str(exc)[:300]}
                extras.append(r)
                torch.cuda.empty_cache()
        cpu = None
        if world == 1 and not args.kernel_only:  # the launcher pins ranks to one host thread each
            cpu = self.cpu_baseline(args.workload, main["unit"], 1e9 if main["unit"] == "GB/s" else 1e12)
        if rank == 0:
            fam = WORKLOADS[args.workload][0]
            cfg = main["config"]
            cfg["parallelism"] = (f"K sharded over {world} ranks, reduce-scatter along M" if fam == "rs" and world > 1
                                  else "replicas only" if world > 1 else "single GPU")
            line = {
                "metric": main["metric"], "value": main["value"], "unit": main["unit"], "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
                "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "strong" if fam == "rs" else "weak", "vs_baseline": None,
                "dtype": main["dtype"], "data": "synthetic", "config": cfg, "roofline": main["roofline"], "cpu_baseline": cpu,
                "e2e": main.get("e2e"), "gpu_launches": args.steps, "clocks": main["clocks"],
            }
            for k in ("local_gemm_ms", "frac_of_local_gemm_rate", "parity_max_rel_err", "parity", "comparators", "in_kernel"):
                if k in main:
                    line[k] = main[k]
            if extras:
                line["extra"] = extras
            print(json.dumps(line), flush=True)
        self.sampler.stop()
        if world > 1:
            self.dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--lead-in-s", type=float, default=0.6, help="seconds of untimed identical launches right before the timed region (clock sampling)")
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="gnk", choices=["gnk", "reference"])
    ap.add_argument("--cpu-rows", type=int, default=512, help="rows of the CPU sample (bounded host time)")
    ap.add_argument("--rs-lagged-exit", action="store_true", help="reduce-scatter: wait for the peers before the next call's first store instead of at the end of every call")
    ap.add_argument("--timeout-ms", type=int, default=2000, help="bound of the device-side waits of the reduce-scatter")
    ap.add_argument("--no-extra", action="store_true", help="main line only")
    ap.add_argument("--kernel-only", action="store_true", help="timed kernel launches only (for profiler captures): no comparators, parity, e2e, CPU arm, extras")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product has no CPU path); use --impl reference for the CPU arm")
    Runner(args, rank, local_rank, world).run()


if __name__ == "__main__":
    main()
