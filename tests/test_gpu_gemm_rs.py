"""GEMM + reduce-scatter across GPUs of one box (needs >= 2 GPUs; one process per GPU via torchrun)."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("multicast", [0, -1], ids=["push", "pull-if-multicast"])
def test_gemm_rs_all_ranks(multicast):
    """Both data paths against the oracle: peer stores into the owner's slots, and (where the
    symmetric-memory handle offers a multicast address) multimem.ld_reduce pulls."""
    world = min(torch.cuda.device_count(), 8)
    world = 1 << (world.bit_length() - 1)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", "29531", os.path.join(ROOT, "tests", "gemm_rs_worker.py"), "--multicast", str(multicast)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0 and "GEMM_RS_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_gemm_rs_single_rank_degenerates_to_gemm():
    import torch.distributed as dist

    import gn_kernels_b200 as gk
    from gn_kernels_b200.cutedsl.sm100.sm100_gemm_rs import gemm_rs
    from oracle import gemm_rs as ors
    from oracle.mm import max_rel_err

    if not dist.is_initialized():
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29533", rank=0, world_size=1)
    try:
        g = torch.Generator().manual_seed(3)
        x = (torch.randn(256, 512, generator=g) / 23).bfloat16().cuda()
        w = (torch.randn(384, 512, generator=g) / 23).bfloat16().cuda()
        out = torch.empty(256, 384, dtype=torch.bfloat16, device="cuda")
        gemm_rs(x, w, None, None, out, None, None)
        ref = ors.gemm_rs([x.cpu()], [w.cpu()])[0]
        assert max_rel_err(out, ref) <= 1e-2
        assert gk.cutedsl.sm100.sm100_gemm_rs.flag_words(2048, 7168, 4) <= (2048 // 128) * (7168 // 128) + 148
    finally:
        dist.destroy_process_group()
