"""CPU checks of the drop-in boundary: the shared library loads without a GPU and exports every
function include/gnk.h declares; argument validation refuses bad calls before any CUDA work."""

import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "gnk.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gnk_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from gn_kernels_b200 import _lib

    L = _lib.lib()
    names = declared_functions()
    assert len(names) >= 20
    for n in names:
        assert hasattr(L, n), f"{n} declared in gnk.h but not exported by libgnk.so"
    # and the Python binding table covers them
    for n in names:
        assert n in _lib._SIGNATURES, f"{n} has no ctypes signature"


def test_version_and_error_text():
    from gn_kernels_b200 import _lib

    L = _lib.lib()
    assert L.gnk_version() == 100
    assert L.gnk_strerror(0) == b"ok"
    assert b"align" in L.gnk_strerror(-3)


def test_bad_arguments_are_refused_without_a_gpu():
    from gn_kernels_b200 import _lib

    L = _lib.lib()
    null = ctypes.c_void_p(0)
    assert L.gnk_mm_mxfp8(null, 0, null, 0, null, null, null, 0, 128, 128, 128, null) == _lib.ERR_BAD_ARG
    assert L.gnk_quant_nvfp4(null, 0, 1, 16, 16, null, 1e-12, null, null, 0, null) == _lib.ERR_BAD_ARG
    buf = (ctypes.c_char * 4096)()
    p = ctypes.c_void_p(ctypes.addressof(buf) // 16 * 16 + 16)
    assert L.gnk_quant_mx(p, 0, 4, 33, 40, 1, 0, p, p, 0, null) == _lib.ERR_BAD_SHAPE
    assert L.gnk_quant_rowwise(p, 0, 4, 12, 16, 0, p, p, 0, 0, null) == _lib.ERR_BAD_SHAPE
    assert L.gnk_gemm_rs_flag_words(1000, 256, 8) == -1


def test_cpu_tensors_raise():
    import pytest
    import torch

    import gn_kernels_b200 as gk

    with pytest.raises(RuntimeError):
        gk.quantize_nvfp4(torch.randn(16, 64).bfloat16())
    with pytest.raises(RuntimeError):
        gk.triton_mm(torch.zeros(16, 16, dtype=torch.int8), torch.zeros(16, 16, dtype=torch.int8))


def declared_prototypes():
    """name -> number of parameters, parsed from include/gnk.h (comments stripped)."""
    text = open(os.path.join(ROOT, "include", "gnk.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    protos = {}
    for name, params in re.findall(r"\b(gnk_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S):
        params = params.strip()
        protos[name] = 0 if params in ("", "void") else params.count(",") + 1
    return protos


def test_ctypes_signatures_have_the_header_parameter_counts():
    from gn_kernels_b200 import _lib

    protos = declared_prototypes()
    assert len(protos) >= 20
    for name, n in protos.items():
        restype, argtypes = _lib._SIGNATURES[name]
        assert len(argtypes) == n, f"{name}: gnk.h declares {n} parameters, the ctypes table has {len(argtypes)}"


def test_gemm_rs_pull_entry_refuses_a_missing_multicast_address():
    from gn_kernels_b200 import _lib

    L = _lib.lib()
    buf = (ctypes.c_char * 4096)()
    p = ctypes.c_void_p(ctypes.addressof(buf) // 16 * 16 + 16)
    arr = (ctypes.c_void_p * 2)(p, p)
    rc = L.gnk_gemm_rs_bf16_pull(p, 64, p, 64, arr, ctypes.c_void_p(0), arr, p, 256, 512, 256, 64, 0, 2, 0, 0, ctypes.c_void_p(0))
    assert rc == _lib.ERR_BAD_ARG


def test_pipeline_plan_keeps_the_operand_read_inside_shared_memory():
    """A problem with fewer than 128 rows keeps only `a_rows` rows of A per pipeline stage, but the MMA
    still reads 128 rows (16 KB) from the start of every A slice.  From the last stage that read must
    end inside the bytes the stages own (an out-of-range shared address faults the kernel): for every
    kind, tile and stage depth the plan the launcher uses satisfies
    (stages - 1) * stage_bytes + tail <= pool."""
    from gn_kernels_b200 import _lib

    L = _lib.lib()
    out = (ctypes.c_int32 * 4)()
    combos = [(0, 1), (1, 1), (2, 1), (3, 1), (4, 1), (3, 2), (3, 4)]
    for kind in range(5):
        for tile, kd in combos:
            for a_rows in range(8, 129, 8):
                assert L.gnk_debug_stage_plan(kind, tile, kd, a_rows, out) == 0
                stages, stage_bytes, pool, tail = list(out)
                assert stages >= 2, (kind, tile, kd, a_rows, stages)
                assert stages * stage_bytes <= pool
                assert (stages - 1) * stage_bytes + tail <= pool, (kind, tile, kd, a_rows, list(out))
                assert stage_bytes % 1024 == 0 or kind >= 3  # operand slices stay 1024-byte aligned (scale atoms follow them)
    assert L.gnk_debug_stage_plan(0, 7, 1, 16, out) != 0 and L.gnk_debug_stage_plan(0, 3, 4, 12, out) != 0
