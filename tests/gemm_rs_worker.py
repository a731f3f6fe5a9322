"""Multi-GPU worker for the GEMM + reduce-scatter parity test and benchmark.

    torchrun --nnodes=1 --nproc-per-node=W --master-addr 127.0.0.1 --master-port P tests/gemm_rs_worker.py [--multicast 0|1] [--trace]

Each rank holds its K shard; outputs are gathered on rank 0 and compared with the CPU oracle.
Timing lives in bench.py (--workload bf16_gemm_rs under torchrun)."""

import argparse
import ctypes
import os
import sys

import torch
import torch.distributed as dist
import torch.distributed._symmetric_memory as symm_mem

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--trace", action="store_true", help="print a per-role timeline of one full-size call instead of the parity cases")
    ap.add_argument("--k-total", type=int, default=28672, help="--trace: K summed over ranks")
    ap.add_argument("--timeout-ms", type=int, default=5000, help="bound of the device-side waits")
    ap.add_argument("--symm-backend", default="", help="torch symmetric-memory backend (empty = torch's default)")
    ap.add_argument("--multicast", type=int, default=-1, help="-1 automatic, 0 push over peer stores, 1 pull through the multicast address")
    args = ap.parse_args()
    from gn_kernels_b200 import _lib
    from gn_kernels_b200.cutedsl.sm100.sm100_gemm_rs import flag_words
    from gn_kernels_b200.cutedsl.sm100.sm100_gemm_rs import gemm_ar as _gemm_ar
    from gn_kernels_b200.cutedsl.sm100.sm100_gemm_rs import gemm_rs as _gemm_rs
    from oracle import gemm_rs as ors
    from oracle.mm import max_rel_err

    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    if args.symm_backend:  # torch's default backend offers a multicast address on NVSwitch systems
        symm_mem.set_backend(args.symm_backend)
    rank, W = dist.get_rank(), dist.get_world_size()
    if rank == 0:  # the launcher pins every rank to one host thread; rank 0 runs the CPU oracle
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    mcast = None if args.multicast < 0 else bool(args.multicast)

    def gemm_rs(*a, **k):  # every call below goes through the chosen data path
        return _gemm_rs(*a, multicast=mcast, timeout_ms=args.timeout_ms, **k)

    def alloc(M, N):
        partial = symm_mem.empty(M, N, dtype=torch.bfloat16, device=dev)
        ph = symm_mem.rendezvous(partial, dist.group.WORLD)
        flags = symm_mem.empty(flag_words(M, N, W), dtype=torch.int32, device=dev)
        flags.zero_()
        fh = symm_mem.rendezvous(flags, dist.group.WORLD)
        dist.barrier()
        if rank == 0:
            has_mc = bool(getattr(ph, "multicast_ptr", 0))
            path = "pull (multimem.ld_reduce)" if (has_mc and mcast is not False) else "push (peer stores)"
            print(f"gemm_rs data path: {path}; multicast address available: {has_mc}", flush=True)
        return partial, ph, flags, fh

    failures = 0
    # the last case has the benchmark's M and N (every CTA reduces several units) with a short K
    cases = [(256 * W, 256, 512), (512 * W, 768, 1024), (128 * W, 384, 320), (8192, 8192, 256)] if not args.trace else []
    for M, N, Kt in cases:
        Kl = Kt
        g = torch.Generator().manual_seed(1234 + rank)
        x = (torch.randn(M, Kl, generator=g) / (Kl * W) ** 0.5).bfloat16().to(dev)
        w = (torch.randn(N, Kl, generator=g) / (Kl * W) ** 0.5).bfloat16().to(dev)
        partial, ph, flags, fh = alloc(M, N)
        out = torch.empty(M // W, N, dtype=torch.bfloat16, device=dev)
        xs = [torch.empty_like(x) for _ in range(W)]
        ws = [torch.empty_like(w) for _ in range(W)]
        dist.all_gather(xs, x)
        dist.all_gather(ws, w)
        refs = ors.gemm_rs([t.cpu() for t in xs], [t.cpu() for t in ws]) if rank == 0 else None
        for it in range(3):  # repeated calls reuse flags and staging (exit barrier + flag reset)
            out.zero_()
            gemm_rs(x, w, partial, ph, out, flags, fh)
            torch.cuda.synchronize()
            _lib.raise_on_device_error()
            outs = [torch.empty_like(out) for _ in range(W)]
            dist.all_gather(outs, out)
            if rank == 0:
                errs = [max_rel_err(o.cpu(), r) for o, r in zip(outs, refs)]
                exact = all(torch.equal(o.cpu(), r) for o, r in zip(outs, refs))
                ok = max(errs) <= 1e-2
                print(f"gemm_rs W={W} M={M} N={N} K={Kl * W} call {it}: max rel err {max(errs):.2e} bit-equal-to-oracle={exact} {'OK' if ok else 'FAIL'}", flush=True)
                failures += 0 if ok else 1
            assert int(flags.abs().sum()) == 0, "flags not restored to zero"
            dist.barrier()  # a faster peer's next call may signal this rank's flags as soon as it starts
        dist.barrier()

        # E4M3 operands with tensor-wise scales: partial_r = bf16(alpha_r * (x_r w_r^T))
        if Kl % 16 == 0:
            sx, sw = x.abs().amax().float() / 448.0, w.abs().amax().float() / 448.0
            x8, w8 = (x.float() / sx).to(torch.float8_e4m3fn), (w.float() / sw).to(torch.float8_e4m3fn)
            a8 = float(sx) * float(sw)
            x8s = [torch.empty_like(x8.view(torch.uint8)) for _ in range(W)]
            w8s = [torch.empty_like(w8.view(torch.uint8)) for _ in range(W)]
            a8s = [torch.empty(1, device=dev) for _ in range(W)]
            dist.all_gather(x8s, x8.view(torch.uint8))
            dist.all_gather(w8s, w8.view(torch.uint8))
            dist.all_gather(a8s, torch.tensor([a8], device=dev))
            refs8 = None
            if rank == 0:
                refs8 = ors.gemm_rs_f8([t.view(torch.float8_e4m3fn).cpu() for t in x8s], [t.view(torch.float8_e4m3fn).cpu() for t in w8s],
                                       [float(t) for t in a8s])
            o8 = torch.zeros_like(out)
            gemm_rs(x8, w8, partial, ph, o8, flags, fh, alpha=a8)
            torch.cuda.synchronize()
            _lib.raise_on_device_error()
            assert int(flags.abs().sum()) == 0, "flags not restored to zero after the fp8 reduce-scatter"
            outs = [torch.empty_like(o8) for _ in range(W)]
            dist.all_gather(outs, o8)
            if rank == 0:
                errs = [max_rel_err(o.cpu(), r) for o, r in zip(outs, refs8)]
                ok = max(errs) <= 1e-2
                print(f"gemm_rs fp8 W={W} M={M} N={N} K={Kl * W}: max rel err {max(errs):.2e} {'OK' if ok else 'FAIL'}", flush=True)
                failures += 0 if ok else 1
            dist.barrier()

        # GEMM + all-reduce (needs the multicast path): every rank ends with all rows of the sum
        if bool(getattr(ph, "multicast_ptr", 0)) and mcast is not False:
            full = symm_mem.empty(M, N, dtype=torch.bfloat16, device=dev)
            oh = symm_mem.rendezvous(full, dist.group.WORLD)
            for it in range(2):
                full.zero_()
                torch.cuda.synchronize()
                dist.barrier()
                _gemm_ar(x, w, partial, ph, full, oh, flags, fh, timeout_ms=args.timeout_ms)
                torch.cuda.synchronize()
                _lib.raise_on_device_error()
                assert int(flags.abs().sum()) == 0, "flags not restored to zero after the all-reduce"
                fulls = [torch.empty_like(full) for _ in range(W)]
                dist.all_gather(fulls, full)
                if rank == 0:
                    want = ors.gemm_ar([t.cpu() for t in xs], [t.cpu() for t in ws])
                    errs = [max_rel_err(f.cpu(), want) for f in fulls]
                    same = all(torch.equal(f, fulls[0]) for f in fulls)
                    ok = max(errs) <= 1e-2 and same
                    print(f"gemm_ar W={W} M={M} N={N} K={Kl * W} call {it}: max rel err {max(errs):.2e} all ranks equal={same} {'OK' if ok else 'FAIL'}", flush=True)
                    failures += 0 if ok else 1
                dist.barrier()

        # A sequence with the exit wait deferred: four calls back to back with no host synchronisation in
        # between, the ranks deliberately out of step (each spins a different time first), then one
        # ordinary call that ends the sequence.  Every call's output must be right and the flags zero again.
        seq = [torch.zeros_like(out) for _ in range(5)]
        torch.cuda._sleep(200_000 * (1 + (rank * 3) % W))
        for o in seq[:4]:
            gemm_rs(x, w, partial, ph, o, flags, fh, lagged_exit=True)
        gemm_rs(x, w, partial, ph, seq[4], flags, fh)
        torch.cuda.synchronize()
        _lib.raise_on_device_error()
        assert int(flags.abs().sum()) == 0, "flags not restored to zero after the deferred-exit sequence"
        for i, o in enumerate(seq):
            outs = [torch.empty_like(o) for _ in range(W)]
            dist.all_gather(outs, o)
            if rank == 0:
                errs = [max_rel_err(t.cpu(), r) for t, r in zip(outs, refs)]
                ok = max(errs) <= 1e-2
                print(f"gemm_rs W={W} M={M} N={N} K={Kl * W} deferred-exit sequence, call {i}: max rel err {max(errs):.2e} {'OK' if ok else 'FAIL'}", flush=True)
                failures += 0 if ok else 1
        dist.barrier()

    if args.trace:
        # per-role timeline of one full-size call (M = N = 8192): the kernel writes globaltimer stamps per CTA
        # into a caller-owned buffer (gnk_debug_rs_trace); rank 0 prints a summary in microseconds
        M = N = 8192
        Kl = args.k_total // W
        g = torch.Generator().manual_seed(1234 + rank)
        x = (torch.randn(M, Kl, generator=g) / args.k_total**0.5).bfloat16().to(dev)
        w = (torch.randn(N, Kl, generator=g) / args.k_total**0.5).bfloat16().to(dev)
        out = torch.empty(M // W, N, dtype=torch.bfloat16, device=dev)
        partial, ph, flags, fh = alloc(M, N)
        for _ in range(3):
            gemm_rs(x, w, partial, ph, out, flags, fh)
        torch.cuda.synchronize()
        dist.barrier()
        buf = torch.zeros(160 * 8, dtype=torch.int64, device=dev)
        L = _lib.lib()
        L.gnk_debug_rs_trace(ctypes.c_void_p(buf.data_ptr()))
        gemm_rs(x, w, partial, ph, out, flags, fh)
        torch.cuda.synchronize()
        L.gnk_debug_rs_trace(None)
        _lib.raise_on_device_error()
        h = buf.cpu().view(160, 8)
        h = h[h[:, 0] > 0]
        t0 = int(h[:, 0].min())
        us = lambda col: (h[:, col][h[:, col] > 0] - t0).double() * 1e-3  # noqa: E731
        tot = lambda col: h[:, col].double() * 1e-3  # noqa: E731
        print(f"RS_TRACE rank {rank} W={W} K={args.k_total} CTAs {h.shape[0]} us: start max {us(0).max():.1f} | mma end mean {us(4).mean():.1f} max {us(4).max():.1f} | "
              f"epi end mean {us(1).mean():.1f} max {us(1).max():.1f} | red end mean {us(2).mean():.1f} max {us(2).max():.1f} | red wait mean {tot(3).mean():.1f} | "
              f"epi store+signal mean {tot(5).mean():.1f} | epi wait-acc mean {tot(6).mean():.1f}", flush=True)
        dist.barrier()
    dist.barrier()
    if rank == 0 and not args.trace:
        print("GEMM_RS_OK" if failures == 0 else "GEMM_RS_FAILED", flush=True)
    dist.destroy_process_group()
    sys.exit(1 if failures else 0)


if __name__ == "__main__":
    main()
