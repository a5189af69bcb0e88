"""Structured-sparse W8A8 projections (2:4, 4:6, 6:8) for NVIDIA B200, sm_100a only.

The public names are those of the SlideSparse-Diffusion operator package
(`sdacc/w8a8_slidesparse/__init__.py:5-12`), so code written against it imports this package
unchanged.  Everything that runs on the GPU lives in a C-ABI shared library
(`include/slidesparse_b200.h`), built in-tree by `build_native()` / `python build_native.py` and
loaded with `load_native()`; there is no second backend and no CPU fallback.

Additions that the reference package does not have are reached through their modules:
`routing` (ProjectionState / OrdinaryProxy), `banks` (mode banks), `sharding` (column shards,
tensor-parallel gather), `importer` (payloads written by the reference), `denoiser` (test models).
"""
from . import backend as _backend
from . import compilation as _compilation
from . import composite as _composite
from . import packing as _packing
from . import runtime as _runtime

# offline preparation
group_size = _packing.group_size
lifted_k = _packing.lifted_k
slide_weight = _packing.slide_weight
# operators
PackedLinear = _runtime.PackedLinear
quantize_lift = _runtime.quantize_lift
SharedProjection = _composite.SharedProjection
ProtectedFFNOutput = _composite.ProtectedFFNOutput
compile_projection = _compilation.compile_projection
# native library
build_native = _backend.build_native
load_native = _backend.load_native

__all__ = sorted(["PackedLinear", "ProtectedFFNOutput", "SharedProjection", "build_native", "compile_projection",
                  "group_size", "lifted_k", "load_native", "quantize_lift", "slide_weight"])
