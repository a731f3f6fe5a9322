"""gnk_absmax_static: the absmax reduction for callers that have no way to hand the library scratch
memory (a host runtime whose pool owns the whole GPU, or a binding that only passes data pointers).
Its scratch is a fixed array inside the library, so the call must allocate nothing and still agree
with gnk_absmax.  Checked through the C ABI on two calls in a row (the array is reused, the second
call starts from the first one's leftovers).  Collected last on purpose."""

import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def test_static_scratch_matches_regular_entry_point_twice():
    from gn_kernels_b200 import _lib

    L = _lib.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    gen = torch.Generator().manual_seed(77)
    inputs = [
        (torch.randn(4096 * 4096 + 3, generator=gen) * 3).bfloat16().cuda(),  # many CTAs, ragged tail
        (torch.randn(1000, generator=gen) * 1e-3).cuda(),                      # fp32, a single CTA, smaller maximum than before
    ]
    scratch = torch.zeros(L.gnk_absmax_scratch_bytes(1) // 4, dtype=torch.int32, device="cuda")
    for x in inputs:  # two calls in a row on the shared array
        dt = {torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}[x.dtype]
        want = torch.empty(1, dtype=torch.float32, device="cuda")
        got = torch.full((1,), -1.0, dtype=torch.float32, device="cuda")
        assert L.gnk_absmax(_p(x), dt, x.numel(), 2688.0, _p(want), _p(scratch), stream) == 0
        # one untimed call first: loading the kernel image and looking up the array's address happen once per device
        assert L.gnk_absmax_static(_p(x), dt, x.numel(), 2688.0, _p(got), stream) == 0
        torch.cuda.synchronize()
        got.fill_(-1.0)
        torch.cuda.synchronize()
        # cudaMemGetInfo sees every allocation on the device, whoever made it; torch's own counter
        # would miss a cudaMalloc made inside the library
        free_before = torch.cuda.mem_get_info()[0]
        torch_before = torch.cuda.memory_allocated()
        assert L.gnk_absmax_static(_p(x), dt, x.numel(), 2688.0, _p(got), stream) == 0
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.cuda.memory_allocated() == torch_before
        assert float(got) == float(want)  # bit-identical: same kernel, same reduction order
        expect = np.float32(x.float().abs().max().item()) / np.float32(2688.0)  # IEEE fp32 division, as the kernel does
        assert np.float32(float(got)) == expect


def test_static_scratch_rejects_sizes_beyond_its_limit():
    from gn_kernels_b200 import _lib

    L = _lib.lib()
    x = torch.zeros(16, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(1, dtype=torch.float32, device="cuda")
    limit = L.gnk_absmax_static_max_elems()
    assert limit == 1 << 32
    rc = L.gnk_absmax_static(_p(x), _lib.BF16, limit + 1, 1.0, _p(out), None)
    assert rc == _lib.ERR_TOO_LARGE
    assert b"maximum" in L.gnk_strerror(rc)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs a second GPU")
def test_static_scratch_has_its_own_address_on_every_device():
    """The array's device address is looked up per device; a call on device 1 must not use device 0's."""
    from gn_kernels_b200 import _lib

    L = _lib.lib()
    gen = torch.Generator().manual_seed(78)
    host = (torch.randn(3 * 1024 * 1024 + 5, generator=gen) * 2).bfloat16()
    results = []
    for dev in (0, 1, 0):
        with torch.cuda.device(dev):
            x = host.to(f"cuda:{dev}")
            stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            scratch = torch.zeros(L.gnk_absmax_scratch_bytes(1) // 4, dtype=torch.int32, device=f"cuda:{dev}")
            want = torch.empty(1, dtype=torch.float32, device=f"cuda:{dev}")
            got = torch.full((1,), -1.0, dtype=torch.float32, device=f"cuda:{dev}")
            assert L.gnk_absmax(_p(x), _lib.BF16, x.numel(), 1.0, _p(want), _p(scratch), stream) == 0
            assert L.gnk_absmax_static(_p(x), _lib.BF16, x.numel(), 1.0, _p(got), stream) == 0
            torch.cuda.synchronize()
            assert float(got) == float(want) == float(host.float().abs().max())
            results.append(float(got))
    assert len(set(results)) == 1
