"""`compile_projection` of the reference (`sdacc/w8a8_slidesparse/compilation.py:10-30`).

The reference wraps a projection in `torch.compile` with per-shape recipes tuned for its SM80
binary.  Here the hot path is two hand-written kernels behind registered operators (with fake
kernels for tracing), so compilation adds nothing to the projection itself; the function keeps
its signature, prepares the projection for the example shape and returns a callable with the
same behaviour.
"""
import math

from .composite import SharedProjection
from .runtime import PackedLinear


def compile_projection(projection, example_input):
    """Prepare offline for the example shape; returns the projection ready to call."""
    packed = projection.packed if isinstance(projection, SharedProjection) else projection
    if isinstance(packed, PackedLinear):
        rows = math.prod(example_input.shape[:-1])
        if packed.packed.is_cuda:
            packed.configure_for(rows)
    return projection
