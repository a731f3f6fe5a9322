"""Host-side pieces of bench.py that need no GPU: the clock-sample parser and the CPU arm."""

import datetime
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _line(t, clk, cap="Active"):
    stamp = datetime.datetime.fromtimestamp(t).strftime("%Y/%m/%d %H:%M:%S.%f")[:-3]
    return f"{stamp}, {clk}, 1965, 700.0, 0x4, Not Active, Not Active, Not Active, {cap}\n"


class _Proc:
    def terminate(self):
        pass

    def wait(self, timeout=None):
        pass


def _sampler_with(text):
    import bench

    cs = bench.ClockSampler(0)
    fd, path = tempfile.mkstemp(suffix=".csv")
    os.close(fd)
    with open(path, "w") as fh:
        fh.write(text)
    cs.proc, cs.path, cs.fh = _Proc(), path, open(os.devnull, "w")
    return cs


def test_clock_sampler_takes_samples_inside_the_timed_region():
    now = time.time()
    cs = _sampler_with(_line(now - 1.0, 1900, "Not Active") + _line(now + 0.1, 1300) + _line(now + 0.2, 1320) + _line(now + 2.0, 1950, "Not Active"))
    out = cs.stop(now, now + 0.5)
    assert out["samples"] == 2 and out["sm_mhz"] == 1310.0 and out["sm_max_mhz"] == 1965.0
    assert out["reasons"] == ["sw_power_cap"] and "nearest_sample_ms_from_timed_region" not in out


def test_clock_sampler_falls_back_to_the_nearest_sample():
    now = time.time()
    cs = _sampler_with(_line(now - 0.30, 1300) + _line(now + 0.25, 1320, "Not Active"))
    out = cs.stop(now - 0.01, now + 0.01)
    assert out["samples"] == 1 and out["sm_mhz"] == 1320.0 and out["reasons"] == []
    assert 200 < out["nearest_sample_ms_from_timed_region"] < 300


def test_every_workload_has_a_metric_and_a_cpu_arm_entry():
    import bench

    for name, (family, metric, shape) in bench.WORKLOADS.items():
        assert family in ("gemm", "quant", "attn", "rs") and metric and len(shape) >= 2, name


def test_reference_arm_prints_one_json_line_for_the_small_int8_case():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "int8_gemm_1024", "--steps", "1",
                        "--warmup", "1", "--cpu-rows", "64"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["cpu_baseline"]["kind"] == "port" and line["gpu_launches"] == 0
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["value"] > 0 and line["unit"] == "TOP/s"
