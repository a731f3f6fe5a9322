"""CPU tests of the reduce-scatter host logic: tile order / ownership / flag accounting (through the
C ABI's planning helper, no GPU work) and the sharding semantics on 2 gloo ranks."""

import ctypes
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _plan(L, M, N, W, rank):
    out = (ctypes.c_int32 * 5)()
    total = L.gnk_gemm_rs_plan(M, N, W, rank, 0, out)
    rows = []
    for i in range(total):
        L.gnk_gemm_rs_plan(M, N, W, rank, i, out)
        rows.append(tuple(out))
    return total, rows


@pytest.mark.parametrize("M,N,W", [(8192, 8192, 8), (2048, 7168, 4), (512, 256, 2), (384, 384, 3), (1024, 512, 1)])
def test_tile_order_covers_everything_once_and_spreads_owners(M, N, W):
    from gn_kernels_b200 import _lib

    L = _lib.lib()
    words = L.gnk_gemm_rs_flag_words(M, N, W)
    assert words > 0
    signals = {}
    for rank in range(W):
        total, rows = _plan(L, M, N, W, rank)
        seen = set()
        for i, (owner, tm, tn, unit, nunits) in enumerate(rows):
            assert (tm, tn) not in seen
            seen.add((tm, tn))
            assert 0 <= owner < W and 0 <= unit and unit + (nunits - 1) * (N // (256 if nunits == 2 else 128)) < (words - 2) // 2
            # at every step the ranks target pairwise different owners
            assert owner == (rank + 1 + i) % W
            for k in range(nunits):
                key = (owner, unit + k * (N // 256 if nunits == 2 else 0))
                signals[key] = signals.get(key, 0) + 1
        assert len(seen) == total
    # every owned unit is signalled exactly once by every rank
    assert set(signals.values()) == {W}
    # flag words: one arrival word and one finished-chunk word per unit, plus ticket and exit barrier
    assert len(signals) == W * ((words - 2) // 2)


def test_bad_shapes_rejected():
    from gn_kernels_b200 import _lib

    L = _lib.lib()
    assert L.gnk_gemm_rs_flag_words(1000, 256, 8) == -1
    assert L.gnk_gemm_rs_flag_words(1024, 200, 8) == -1
    assert L.gnk_gemm_rs_flag_words(1024, 256, 9) == -1


def _gloo_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    from oracle import gemm_rs as ors

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    M, N, Kl = 256, 128, 64
    g = torch.Generator().manual_seed(1234 + rank)
    x = torch.randn(M, Kl, generator=g).bfloat16()
    w = torch.randn(N, Kl, generator=g).bfloat16()
    # what the kernel does, spelled with collectives: bf16 partial, push row blocks to their owners, fp32 sum
    partial = (x.float() @ w.float().T).bfloat16()
    rows = M // world
    parts = [torch.empty_like(partial) for _ in range(world)]
    dist.all_gather(parts, partial)  # gloo has no all_to_all: gather, then keep the rows this rank owns
    mine = sum(t[rank * rows : (rank + 1) * rows].float() for t in parts).bfloat16()
    xs = [torch.empty_like(x) for _ in range(world)]
    ws = [torch.empty_like(w) for _ in range(world)]
    dist.all_gather(xs, x)
    dist.all_gather(ws, w)
    ref = ors.gemm_rs(xs, ws)[rank]
    q.put((rank, bool(torch.equal(mine, ref))))
    dist.destroy_process_group()


def test_sharding_semantics_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, 29541, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, True), (1, True)]


class _FakeHandle:
    """Stand-in for a torch symmetric-memory handle: allocation bases per rank and a multicast base."""

    def __init__(self, bases, size, mc=0):
        self.buffer_ptrs, self.buffer_size, self.multicast_ptr = bases, size, mc


def test_peer_addresses_apply_one_offset_to_every_mapping():
    from gn_kernels_b200.cutedsl.sm100.sm100_gemm_rs import peer_addresses

    pool = torch.zeros(1 << 16, dtype=torch.uint8)
    base = pool.data_ptr()
    bases = [0x7000_0000_0000, base, 0x7200_0000_0000]  # this rank (1) maps its own allocation at `base`
    h = _FakeHandle(bases, pool.numel(), mc=0x7F00_0000_0000)
    view = pool[4096 : 4096 + 8192].view(torch.bfloat16).view(64, 64)  # a sub-allocation 4096 bytes in
    peers, mc = peer_addresses(view, h, rank=1, world=3, need_bytes=8192)
    assert peers == [b + 4096 for b in bases] and mc == 0x7F00_0000_0000 + 4096
    whole = pool.view(torch.bfloat16)
    peers, mc = peer_addresses(whole, h, rank=1, world=3, need_bytes=1024)
    assert peers == bases and mc == 0x7F00_0000_0000
    # no multicast mapping: address 0 selects the peer-store path
    assert peer_addresses(whole, _FakeHandle(bases, pool.numel()), 1, 3, 1024)[1] == 0
    with pytest.raises(ValueError):  # a strided view cannot be addressed as one block
        peer_addresses(pool.view(torch.bfloat16).view(128, 256)[:, :64], h, 1, 3, 64)
    with pytest.raises(ValueError):  # runs past the end of the allocation
        peer_addresses(pool[65000:].view(torch.bfloat16), h, 1, 3, 4096)
    with pytest.raises(ValueError):  # too small for the problem
        peer_addresses(view, h, 1, 3, 8192 + 2)
    with pytest.raises(ValueError):  # misaligned start
        peer_addresses(pool[8 : 8 + 4096].view(torch.bfloat16), h, 1, 3, 4096)
    flags = pool[4 : 4 + 64].view(torch.int32)
    assert peer_addresses(flags, h, 1, 3, 64, align=4)[0][1] == base + 4


def test_oracle_variants_agree_with_the_reduce_scatter_statement():
    """The all-reduce statement is the reduce-scatter outputs stacked, and the E4M3 statement with
    alpha = 1 equals the bf16 statement on the same values (every E4M3 value is a bf16 value)."""
    from oracle import gemm_rs as ors

    g = torch.Generator().manual_seed(5)
    W, M, N, Kl = 4, 16, 12, 32
    xs = [torch.randn(M, Kl, generator=g).to(torch.float8_e4m3fn) for _ in range(W)]
    ws = [torch.randn(N, Kl, generator=g).to(torch.float8_e4m3fn) for _ in range(W)]
    rs = ors.gemm_rs([x.float().bfloat16() for x in xs], [w.float().bfloat16() for w in ws])
    f8 = ors.gemm_rs_f8(xs, ws, [1.0] * W)
    assert all(torch.equal(a, b) for a, b in zip(rs, f8))
    ar = ors.gemm_ar([x.float().bfloat16() for x in xs], [w.float().bfloat16() for w in ws])
    assert ar.shape == (M, N) and torch.equal(ar, torch.cat(rs, dim=0))
    # a power-of-two factor moves every rank's partial exactly
    f8s = ors.gemm_rs_f8(xs, ws, [0.25] * W)
    assert all(torch.equal(a.float() * 0.25, b.float()) for a, b in zip(f8, f8s))


def test_fp8_reduce_scatter_wrapper_refuses_missing_alpha():
    """Argument checks that need no GPU work: E4M3 operands without `alpha` are refused before any launch."""
    import torch.distributed as dist

    from gn_kernels_b200.cutedsl.sm100.sm100_gemm_rs import gemm_rs

    if not dist.is_initialized():
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29537", rank=0, world_size=1)
    try:
        x = torch.zeros(128, 64).to(torch.float8_e4m3fn)
        w = torch.zeros(128, 64).to(torch.float8_e4m3fn)
        out = torch.zeros(128, 128, dtype=torch.bfloat16)
        with pytest.raises(ValueError):
            gemm_rs(x, w, None, None, out, None, None)
        with pytest.raises(NotImplementedError):
            gemm_rs(x, w, None, None, out, None, None, alpha=1.0)
    finally:
        dist.destroy_process_group()
