"""K-sharded BF16 GEMM fused with a reduce-scatter along M (one process per GPU).
Upstream gn_kernels/cutedsl/sm100/sm100_gemm_rs.py:458-496; same call, same buffers
(example_gemm_rs.py:14-26): `partial` is a symmetric-memory [M, N] bf16 buffer, `flags` a
zero-initialised symmetric int32 buffer, both rendezvoused over the default group."""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..._lib import check, lib


def flag_words(M: int, N: int, world_size: int) -> int:
    """int32 words `flags` must hold for this problem (never more than upstream's
    (M/128)*(N/128) + SM-count allocation)."""
    n = lib().gnk_gemm_rs_flag_words(M, N, world_size)
    if n < 0:
        raise ValueError(f"gemm_rs: unsupported shape M={M} N={N} world={world_size} (need M % (128*world) == 0, N % 128 == 0)")
    return int(n)


def peer_addresses(t: torch.Tensor, handle, rank: int, world: int, need_bytes: int, align: int = 16) -> tuple[list[int], int]:
    """Addresses of `t` (a contiguous tensor inside this rank's symmetric allocation) as mapped for
    every rank, and its multicast address (0 if the handle has none).

    `handle.buffer_ptrs` are allocation bases; `t` may be a view or a sub-allocation, so ONE byte
    offset (t.data_ptr() minus this rank's base) is applied to every peer base and to the multicast
    base alike.  Using the bases for some and an offset address for others would make ranks write
    to one place and read from another."""
    if not t.is_contiguous():
        raise ValueError("gemm_rs: symmetric buffers must be contiguous")
    bases = [int(p) for p in handle.buffer_ptrs[:world]]
    if len(bases) != world:
        raise ValueError(f"gemm_rs: the symmetric-memory handle maps {len(bases)} ranks, need {world}")
    off = int(t.data_ptr()) - bases[rank]
    size = int(getattr(handle, "buffer_size", 0) or 0)
    if off < 0 or (size and off + need_bytes > size):
        raise ValueError(f"gemm_rs: tensor does not lie inside the symmetric allocation (offset {off}, need {need_bytes}, allocation {size})")
    if t.numel() * t.element_size() < need_bytes:
        raise ValueError(f"gemm_rs: symmetric buffer too small ({t.numel() * t.element_size()} bytes, need {need_bytes})")
    if off % align:
        raise ValueError(f"gemm_rs: symmetric buffer must start {align}-byte aligned inside the allocation")
    try:
        mc = int(getattr(handle, "multicast_ptr", 0) or 0)
    except Exception:
        mc = 0
    return [b + off for b in bases], (mc + off if mc else 0)


def gemm_rs(
    x: torch.Tensor,
    w: torch.Tensor,
    partial: torch.Tensor,
    partial_handle,
    output: torch.Tensor,
    flags: torch.Tensor,
    flags_handle,
    *,
    BN: int | None = None,
    timeout_ms: int = 0,
    multicast: bool | None = None,
    lagged_exit: bool = False,
    alpha: float | None = None,
) -> torch.Tensor:
    """output[M/W, N] = sum over ranks of bf16(x_r @ w_r^T)[this rank's rows], fp32 summation.

    x [M, K/W], w [N, K/W] bf16 (this rank's K shard).  Two data paths share the flag protocol:
    with an NVLink multicast address for `partial` (`partial_handle.multicast_ptr`, NVSwitch
    systems) every rank keeps its bf16 tiles in its own `partial` and the owner reads them with
    multimem.ld_reduce, as upstream does; without one, every rank stores its tiles into the owner's
    buffer over NVLink and the owner reduces from its own memory.  `multicast` = None picks the
    first when the handle offers an address, True requires it, False forces the second.
    Device-side waits are bounded by `timeout_ms` (0 = 20 s); a wait that runs out is
    reported by `gn_kernels_b200._lib.raise_on_device_error()`.
    `lagged_exit=True` is for calls issued back to back on the same buffers (one per layer, say): the
    call tells its peers that it has finished reducing and returns without waiting for them; the next
    call on the same `flags` does that wait just before its first store, under its first tiles' math.
    `output` is complete either way; `partial` and `flags` then belong to the sequence until a call
    with `lagged_exit=False` ends it (or a host barrier across the ranks, then `flags.zero_()`).
    float8_e4m3fn `x` and `w` (tensor-wise scaled; upstream's function is BF16 only) need `alpha`, this rank's
    scale_x * scale_w: the rank's partial is then bf16(alpha * (x @ w^T)).
    BN is accepted for upstream
    compatibility; the tile shape is chosen from the problem shape."""
    assert dist.is_initialized()
    rank = dist.get_rank()
    world = dist.get_world_size()
    assert world <= 8
    M, K = x.shape
    N, _ = w.shape
    fp8 = x.dtype == torch.float8_e4m3fn
    assert (fp8 or x.dtype == torch.bfloat16) and w.dtype == x.dtype and output.dtype == torch.bfloat16
    if fp8 and alpha is None:
        raise ValueError("gemm_rs: float8_e4m3fn operands need alpha = scale_x * scale_w")
    if fp8 and world == 1:
        raise NotImplementedError("gemm_rs: float8_e4m3fn operands need at least 2 ranks (one rank: triton_mm with row scales)")
    assert w.shape[1] == K and output.shape == (M // world, N)
    assert x.stride(1) == 1 and w.stride(1) == 1 and output.stride(1) == 1
    stream = ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
    mc = 0
    sp = fp = None
    if world > 1:
        assert partial.dtype == torch.bfloat16 and flags.dtype == torch.int32
        p_addr, p_mc = peer_addresses(partial, partial_handle, rank, world, M * N * 2)
        f_addr, _ = peer_addresses(flags, flags_handle, rank, world, flag_words(M, N, world) * 4, align=4)
        sp = (ctypes.c_void_p * world)(*p_addr)
        fp = (ctypes.c_void_p * world)(*f_addr)
        if multicast is not False:
            mc = p_mc
            if mc == 0 and multicast:
                raise RuntimeError("gemm_rs: multicast=True but the symmetric-memory handle has no multicast address")
    if fp8:
        with torch.cuda.device(x.device):
            check(
                lib().gnk_gemm_rs_f8(
                    ctypes.c_void_p(x.data_ptr()), x.stride(0), ctypes.c_void_p(w.data_ptr()), w.stride(0), float(alpha), sp,
                    ctypes.c_void_p(mc) if mc else None, fp, ctypes.c_void_p(output.data_ptr()), output.stride(0), M, N, K,
                    rank, world, timeout_ms, int(bool(lagged_exit)), stream,
                ),
                "gnk_gemm_rs_f8",
            )
        return output
    if mc:
        with torch.cuda.device(x.device):
            check(
                lib().gnk_gemm_rs_bf16_pull(
                    ctypes.c_void_p(x.data_ptr()), x.stride(0), ctypes.c_void_p(w.data_ptr()), w.stride(0), sp,
                    ctypes.c_void_p(mc), fp, ctypes.c_void_p(output.data_ptr()), output.stride(0), M, N, K, rank, world,
                    timeout_ms, int(bool(lagged_exit)), stream,
                ),
                "gnk_gemm_rs_bf16_pull",
            )
        return output
    with torch.cuda.device(x.device):
        check(
            lib().gnk_gemm_rs_bf16(
                ctypes.c_void_p(x.data_ptr()), x.stride(0), ctypes.c_void_p(w.data_ptr()), w.stride(0), sp, fp,
                ctypes.c_void_p(output.data_ptr()), output.stride(0), M, N, K, rank, world, timeout_ms,
                int(bool(lagged_exit)), stream,
            ),
            "gnk_gemm_rs_bf16",
        )
    return output


def gemm_ar(
    x: torch.Tensor,
    w: torch.Tensor,
    partial: torch.Tensor,
    partial_handle,
    output: torch.Tensor,
    output_handle,
    flags: torch.Tensor,
    flags_handle,
    *,
    timeout_ms: int = 0,
) -> torch.Tensor:
    """output[M, N] (on EVERY rank) = sum over ranks of bf16(x_r @ w_r^T), fp32 summation: the K-sharded GEMM
    fused with an all-reduce.  Upstream has no such function; it is `gemm_rs` whose owners store the reduced
    rows through the NVLink multicast address of the ranks' outputs instead of keeping them.

    `partial`, `flags` as for `gemm_rs`; `output` is a symmetric-memory [M, N] bf16 buffer whose handle offers
    a multicast address (NVSwitch systems), like `partial`."""
    assert dist.is_initialized()
    rank = dist.get_rank()
    world = dist.get_world_size()
    assert world <= 8
    M, K = x.shape
    N, _ = w.shape
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and output.dtype == torch.bfloat16
    assert w.shape[1] == K and output.shape == (M, N)
    assert x.stride(1) == 1 and w.stride(1) == 1 and output.is_contiguous()
    stream = ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
    sp = fp = None
    p_mc = o_mc = 0
    if world > 1:
        assert partial.dtype == torch.bfloat16 and flags.dtype == torch.int32
        p_addr, p_mc = peer_addresses(partial, partial_handle, rank, world, M * N * 2)
        _, o_mc = peer_addresses(output, output_handle, rank, world, M * N * 2)
        f_addr, _ = peer_addresses(flags, flags_handle, rank, world, flag_words(M, N, world) * 4, align=4)
        if not p_mc or not o_mc:
            raise RuntimeError("gemm_ar needs symmetric-memory handles with a multicast address for `partial` and `output`")
        sp = (ctypes.c_void_p * world)(*p_addr)
        fp = (ctypes.c_void_p * world)(*f_addr)
    with torch.cuda.device(x.device):
        check(
            lib().gnk_gemm_ar_bf16(
                ctypes.c_void_p(x.data_ptr()), x.stride(0), ctypes.c_void_p(w.data_ptr()), w.stride(0), sp,
                ctypes.c_void_p(p_mc), fp, ctypes.c_void_p(output.data_ptr()), ctypes.c_void_p(o_mc), output.stride(0),
                M, N, K, rank, world, timeout_ms, stream,
            ),
            "gnk_gemm_ar_bf16",
        )
    return output
