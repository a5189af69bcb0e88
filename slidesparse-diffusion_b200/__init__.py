"""Dynamic-token W8A8 SlideSparse projections for NVIDIA B200 (sm_100a).

Drop-in for the operator package `sdacc/w8a8_slidesparse` of SlideSparse-Diffusion
(`__init__.py:5-12` exports): packing is offline; no pruning, fitting, search or compilation in
forward.  The kernels live in a C-ABI shared library (see include/slidesparse_b200.h) that must
be built with `build_native()` (or `python build_native.py`) before first use.
"""
from .backend import build_native, load_native
from .packing import group_size, lifted_k, slide_weight
from .runtime import PackedLinear, quantize_lift
from .composite import ProtectedFFNOutput, SharedProjection
from .compilation import compile_projection

__all__ = ["PackedLinear", "quantize_lift", "slide_weight", "lifted_k", "group_size",
           "build_native", "load_native", "compile_projection", "SharedProjection",
           "ProtectedFFNOutput"]
