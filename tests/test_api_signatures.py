"""The Python entry points keep upstream's names, parameter names, order and defaults
(gn_kernels/triton_mm.py:128, triton_attn.py:268 and :462, quant_utils.py:21-252,
cutedsl/sm100/*.py `mm` / `gemm_rs`), so a caller switches packages without edits.  The
expected signatures are written out here; nothing is imported from upstream."""

import inspect

import gn_kernels_b200 as gk

EXPECTED = {
    "triton_mm": (["A", "B", "bias", "scale_A", "scale_B", "out_dtype", "acc_dtype"], {"bias": None, "scale_A": None, "scale_B": None, "out_dtype": None, "acc_dtype": None}),
    "triton_attn": (["q", "k", "v", "scale_q", "scale_k", "causal", "qk_fp16_acc", "pv_fp16_acc"],
                    {"scale_q": None, "scale_k": None, "causal": False, "qk_fp16_acc": False, "pv_fp16_acc": False}),
    "triton_varlen_attn": (["q", "k", "v", "q_offsets", "kv_offsets", "max_q_len", "causal", "qk_fp16_acc", "pv_fp16_acc"],
                           {"causal": False, "qk_fp16_acc": False, "pv_fp16_acc": False}),
    "quantize_mx": (["x", "dtype", "compute_scale_method"], {"compute_scale_method": "ocp"}),
    "dequantize_mx": (["xq", "scales"], {}),
    "quantize_nvfp4": (["x", "tensor_scale", "eps"], {"tensor_scale": None, "eps": 1e-12}),
    "quantize_nvfp4_triton": (["x", "tensor_scale", "eps"], {"eps": 1e-12}),
    "permute_nv_sf": (["scales"], {}),
    "unpermute_nv_sf": (["scales"], {}),
}


def _check(fn, names, defaults, extra_ok=()):
    sig = inspect.signature(fn)
    got = [p for p in sig.parameters if p not in extra_ok]
    assert got[: len(names)] == names, (fn.__name__, got)
    for k, v in defaults.items():
        assert sig.parameters[k].default == v, (fn.__name__, k)


def test_top_level_entry_points_keep_upstream_signatures():
    for name, (names, defaults) in EXPECTED.items():
        # extensions are keyword-only and default to upstream behaviour
        _check(getattr(gk, name), names, defaults, extra_ok=("swizzled_scales",))
    kw_only = inspect.signature(gk.triton_mm).parameters
    assert all(kw_only[k].kind is inspect.Parameter.KEYWORD_ONLY for k in ("scale_A", "scale_B", "out_dtype", "acc_dtype"))
    kw_only = inspect.signature(gk.triton_attn).parameters
    assert all(kw_only[k].kind is inspect.Parameter.KEYWORD_ONLY for k in ("causal", "qk_fp16_acc", "pv_fp16_acc"))


def test_cutedsl_modules_keep_upstream_signatures():
    from gn_kernels_b200.cutedsl.sm100 import sm100_gemm_rs, sm100_mm_bf16, sm100_mm_mxfp8, sm100_mm_nvfp4
    from gn_kernels_b200.cutedsl.sm120 import sm120_mm_fp8_1d2d

    _check(sm100_mm_bf16.mm, ["A", "B"], {})
    _check(sm100_mm_mxfp8.mm, ["A", "B", "SFA", "SFB"], {})
    _check(sm100_mm_nvfp4.mm, ["A", "B", "SFA", "SFB"], {}, extra_ok=("alpha",))
    _check(sm120_mm_fp8_1d2d.mm, ["A", "SFA", "B", "SFB", "bias", "add"], {})
    _check(sm100_gemm_rs.gemm_rs, ["x", "w", "partial", "partial_handle", "output", "flags", "flags_handle", "BN"], {"BN": None},
           extra_ok=("timeout_ms", "multicast"))
    p = inspect.signature(sm100_gemm_rs.gemm_rs).parameters
    assert p["BN"].kind is inspect.Parameter.KEYWORD_ONLY
