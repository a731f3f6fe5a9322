"""Module paths of upstream gn_kernels/cutedsl kept for drop-in imports; the kernels behind
them are CUDA C++ for sm_100a, not CuteDSL."""

from . import sm100, sm120  # noqa: F401
