"""CPU oracle for the quantized matmul / quantizer / attention / GEMM-reduce-scatter path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this directory; the
parity tests, the smoke check and the CPU-baseline leg of the benchmark are its only
users.  Every function restates, in numpy (byte / integer arithmetic) or CPU torch
(fp32 contractions), the arithmetic of the upstream gn_kernels torch reference path and
cites the upstream file:line it follows.

Parity status: pinned.  The restatement is checked against outputs of the upstream
Python reference itself (imported on CPU by tests/golden/make_golden.py, which wrote the
committed fixtures under tests/golden/), see tests/test_oracle_golden.py.
"""

from . import attn, gemm_rs, mm, quant  # noqa: F401
