"""Multi-GPU worker for the GEMM + reduce-scatter parity test and benchmark.

    torchrun --nnodes=1 --nproc-per-node=W --master-addr 127.0.0.1 --master-port P tests/gemm_rs_worker.py [--bench]

Each rank holds its K shard; outputs are gathered on rank 0 and compared with the CPU oracle."""

import argparse
import os
import sys

import torch
import torch.distributed as dist
import torch.distributed._symmetric_memory as symm_mem

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--bench", action="store_true")
    ap.add_argument("--k-total", type=int, default=28672, help="bench: K summed over ranks")
    ap.add_argument("--symm-backend", default="", help="torch symmetric-memory backend (empty = torch's default)")
    ap.add_argument("--multicast", type=int, default=-1, help="-1 automatic, 0 push over peer stores, 1 pull through the multicast address")
    args = ap.parse_args()
    from gn_kernels_b200 import _lib
    from gn_kernels_b200.cutedsl.sm100.sm100_gemm_rs import flag_words
    from gn_kernels_b200.cutedsl.sm100.sm100_gemm_rs import gemm_rs as _gemm_rs
    from oracle import gemm_rs as ors
    from oracle.mm import max_rel_err

    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    if args.symm_backend:  # torch's default backend offers a multicast address on NVSwitch systems
        symm_mem.set_backend(args.symm_backend)
    rank, W = dist.get_rank(), dist.get_world_size()
    mcast = None if args.multicast < 0 else bool(args.multicast)

    def gemm_rs(*a, **k):  # every call below goes through the chosen data path
        return _gemm_rs(*a, multicast=mcast, **k)

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
    cases = [(256 * W, 256, 512), (512 * W, 768, 1024), (128 * W, 384, 320)] if not args.bench else []
    for M, N, Kt in cases:
        Kl = Kt
        g = torch.Generator().manual_seed(1234 + rank)
        x = (torch.randn(M, Kl, generator=g) / (Kl * W) ** 0.5).bfloat16().to(dev)
        w = (torch.randn(N, Kl, generator=g) / (Kl * W) ** 0.5).bfloat16().to(dev)
        partial, ph, flags, fh = alloc(M, N)
        out = torch.empty(M // W, N, dtype=torch.bfloat16, device=dev)
        for it in range(3):  # repeated calls reuse flags and staging (exit barrier + flag reset)
            out.zero_()
            gemm_rs(x, w, partial, ph, out, flags, fh)
            torch.cuda.synchronize()
            _lib.raise_on_device_error()
            xs = [torch.empty_like(x) for _ in range(W)]
            ws = [torch.empty_like(w) for _ in range(W)]
            outs = [torch.empty_like(out) for _ in range(W)]
            dist.all_gather(xs, x)
            dist.all_gather(ws, w)
            dist.all_gather(outs, out)
            if rank == 0:
                refs = ors.gemm_rs([t.cpu() for t in xs], [t.cpu() for t in ws])
                errs = [max_rel_err(o.cpu(), r) for o, r in zip(outs, refs)]
                exact = all(torch.equal(o.cpu(), r) for o, r in zip(outs, refs))
                ok = max(errs) <= 1e-2
                print(f"gemm_rs W={W} M={M} N={N} K={Kl * W} call {it}: max rel err {max(errs):.2e} bit-equal-to-oracle={exact} {'OK' if ok else 'FAIL'}", flush=True)
                failures += 0 if ok else 1
            assert int(flags.abs().sum()) == 0, "flags not restored to zero"
            dist.barrier()  # a faster peer's next call may signal this rank's flags as soon as it starts
        dist.barrier()

    if args.bench:
        M = N = 8192
        Kt = args.k_total
        Kl = Kt // W
        g = torch.Generator().manual_seed(1234 + rank)
        x = (torch.randn(M, Kl, generator=g) / Kt**0.5).bfloat16().to(dev)
        w = (torch.randn(N, Kl, generator=g) / Kt**0.5).bfloat16().to(dev)
        out = torch.empty(M // W, N, dtype=torch.bfloat16, device=dev)
        if W > 1:
            partial, ph, flags, fh = alloc(M, N)
        else:
            partial = ph = flags = fh = None
        for _ in range(5):
            gemm_rs(x, w, partial, ph, out, flags, fh)
        torch.cuda.synchronize()
        dist.barrier()
        steps = 20
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            gemm_rs(x, w, partial, ph, out, flags, fh)
        e1.record()
        torch.cuda.synchronize()
        _lib.raise_on_device_error()
        t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        # plain GEMM of the same local shape for the compute-only reference point
        c = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        from gn_kernels_b200 import ops

        for _ in range(3):
            ops.mm_bf16(x, w)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            ops.mm_bf16(x, w)
        e1.record()
        torch.cuda.synchronize()
        tg = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
        dist.all_reduce(tg, op=dist.ReduceOp.MAX)
        if rank == 0:
            fl = 2.0 * M * N * Kt
            print(f"GEMM_RS_BENCH W={W} M={M} N={N} K={Kt}: {float(t):.3f} ms/step, {fl / float(t) / 1e9:.0f} TFLOP/s total; "
                  f"local GEMM alone {float(tg):.3f} ms ({fl / float(tg) / 1e9:.0f} TFLOP/s total)", flush=True)
    dist.barrier()
    if rank == 0 and not args.bench:
        print("GEMM_RS_OK" if failures == 0 else "GEMM_RS_FAILED", flush=True)
    dist.destroy_process_group()
    sys.exit(1 if failures else 0)


if __name__ == "__main__":
    main()
