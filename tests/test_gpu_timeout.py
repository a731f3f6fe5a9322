"""Failure detection of the GEMM + reduce-scatter: a peer that never signals.

One GPU plays rank 0 of a world of 2; "rank 1" exists only as a second pair of local buffers and is
never launched, so rank 0's reducers wait for signals that nothing sends.  Every wait is bounded:
the call must end by itself, report GNK_ERR_TIMEOUT with the reducer's role in the detail word, cost
about one timeout (not one per work item), and leave the context usable.  Nothing here faults,
traps or hangs the GPU; there is no second process, no symmetric memory and no multicast object.
Upstream spins without a limit at these two places (sm100_gemm_rs.py:311-320, :338-346)."""

import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _call_rank0_of_2(L, x, w, staging, flags, out, timeout_ms):
    M, K = x.shape
    N = w.shape[0]
    sp = (ctypes.c_void_p * 2)(*[t.data_ptr() for t in staging])
    fp = (ctypes.c_void_p * 2)(*[t.data_ptr() for t in flags])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return L.gnk_gemm_rs_bf16(_p(x), K, _p(w), K, sp, fp, _p(out), N, M, N, K, 0, 2, timeout_ms, 0, stream)


@pytest.mark.parametrize(
    "M,N,K,timeout_ms",
    # "many-items": 1024 units = 7 reducer items per CTA; waiting for each would take 7 x 0.2 s + the exit barrier
    [(512, 256, 64, 50), (16384, 4096, 64, 200), (256, 384, 64, 50)],
    ids=["pair-tile", "many-items", "128-tile"],
)
def test_missing_peer_times_out_once_and_context_survives(M, N, K, timeout_ms):
    from gn_kernels_b200 import _lib, ops
    from oracle.mm import max_rel_err, mm_bf16

    L = _lib.lib()
    _lib.device_status(clear=True)
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(M, K, generator=g) / 8).bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) / 8).bfloat16().cuda()
    words = L.gnk_gemm_rs_flag_words(M, N, 2)
    assert words > 0
    staging = [torch.zeros(M, N, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    flags = [torch.zeros(words, dtype=torch.int32, device="cuda") for _ in range(2)]
    out = torch.full((M // 2, N), 7.0, dtype=torch.bfloat16, device="cuda")

    for attempt in range(2):  # the recovery the header prescribes makes the buffers usable again
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        assert _call_rank0_of_2(L, x, w, staging, flags, out, timeout_ms) == 0
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t0
        # one timeout per CTA in parallel (+ launch), never items x timeout
        assert elapsed < 1.0, f"give-up took {elapsed:.2f} s"
        st, detail = _lib.device_status(clear=True)
        assert st == _lib.ERR_TIMEOUT
        assert detail >> 24 == 4 and (detail >> 16) & 0xFF in (6, 7), hex(detail)  # role 4 = reducer / exit barrier
        assert _lib.device_status(clear=True) == (0, 0)  # cleared
        # the peer's half of every unit never arrived: the flag words are not zero and must be re-zeroed
        assert int(flags[0].abs().sum()) > 0
        # rank 0's own partial tiles did reach both owners' slot 0
        ref = mm_bf16(x.cpu(), w.cpu())
        assert max_rel_err(staging[0][: M // 2], ref[: M // 2]) <= 1e-2
        assert max_rel_err(staging[1][: M // 2], ref[M // 2 :]) <= 1e-2
        for f in flags:
            f.zero_()

    # while the status word is set a further call gives up at once and says so
    assert _call_rank0_of_2(L, x, w, staging, flags, out, timeout_ms) == 0
    torch.cuda.synchronize()
    assert _lib.device_status(clear=False)[0] == _lib.ERR_TIMEOUT
    for f in flags:
        f.zero_()
    t0 = time.perf_counter()
    assert _call_rank0_of_2(L, x, w, staging, flags, out, 5000) == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0
    assert _lib.device_status(clear=True)[0] == _lib.ERR_TIMEOUT

    # an ordinary GEMM afterwards is unaffected
    a = (torch.randn(384, 256, generator=g)).bfloat16().cuda()
    b = (torch.randn(512, 256, generator=g)).bfloat16().cuda()
    c = ops.mm_bf16(a, b)
    torch.cuda.synchronize()
    assert max_rel_err(c, mm_bf16(a.cpu(), b.cpu())) <= 1e-2
    assert _lib.device_status(clear=True) == (0, 0)


@pytest.mark.parametrize("M,N,K", [(512, 256, 64), (2048, 768, 512), (256, 384, 192)], ids=["pair-tile", "multi-tile", "128-tile"])
def test_two_ranks_one_after_the_other_on_one_gpu(M, N, K):
    """The whole reduce-scatter protocol (peer stores into the owner's slots, per-warp flag signals, reducers,
    flag reset, exit barrier) checked against the oracle on ONE GPU, without two kernels ever waiting
    for each other: the ranks of a world of 2 run one after the other.  The first rank to run pushes its
    tiles and signals, finds nobody answering and gives up after a short timeout (its own output is
    discarded); the second one then finds every signal it needs already there, reduces, and must end
    cleanly with the right rows and its flag words back at zero."""
    from gn_kernels_b200 import _lib
    from oracle import gemm_rs as ors
    from oracle.mm import max_rel_err

    L = _lib.lib()
    _lib.device_status(clear=True)
    W = 2
    g = torch.Generator().manual_seed(M + N + K)
    xs = [(torch.randn(M, K, generator=g) / (K * W) ** 0.5).bfloat16().cuda() for _ in range(W)]
    ws = [(torch.randn(N, K, generator=g) / (K * W) ** 0.5).bfloat16().cuda() for _ in range(W)]
    refs = ors.gemm_rs([t.cpu() for t in xs], [t.cpu() for t in ws])
    words = L.gnk_gemm_rs_flag_words(M, N, W)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call(rank, staging, flags, out, timeout_ms):
        sp = (ctypes.c_void_p * W)(*[t.data_ptr() for t in staging])
        fp = (ctypes.c_void_p * W)(*[t.data_ptr() for t in flags])
        return L.gnk_gemm_rs_bf16(_p(xs[rank]), K, _p(ws[rank]), K, sp, fp, _p(out), N, M, N, K, rank, W, timeout_ms, 0, stream)

    for second in range(W):  # the rank whose output is checked runs second
        first = 1 - second
        staging = [torch.zeros(M, N, dtype=torch.bfloat16, device="cuda") for _ in range(W)]
        flags = [torch.zeros(words, dtype=torch.int32, device="cuda") for _ in range(W)]
        scrap = torch.empty(M // W, N, dtype=torch.bfloat16, device="cuda")
        out = torch.full((M // W, N), 7.0, dtype=torch.bfloat16, device="cuda")
        assert call(first, staging, flags, scrap, 30) == 0
        torch.cuda.synchronize()
        assert _lib.device_status(clear=True)[0] == _lib.ERR_TIMEOUT  # nobody answered the first rank
        assert call(second, staging, flags, out, 2000) == 0
        torch.cuda.synchronize()
        assert _lib.device_status(clear=True) == (0, 0)  # the second rank found everything it waited for
        assert max_rel_err(out, refs[second]) <= 1e-2
        assert int(flags[second].abs().sum()) == 0, "the rank that completed must leave its flag words at zero"
