"""Host side of the offline weight preparation: mode names, lifted widths, and the slide step.

(L-2):L sparsity (L = 4, 6, 8 for "2:4", "4:6", "6:8") is turned into hardware 2:4 by cutting every
group of L columns into L/2-1 windows of four columns that overlap by two.  The three functions
keep the names, arguments, results and exception types of the reference's
`sdacc/w8a8_slidesparse/packing.py` (group_size :8-12, lifted_k :15-20, slide_weight :23-52); the
window allocation itself is done by the native library (`ss_slide_weight_cpu`, csrc/ss_pack.cu).
"""
import ctypes

import torch

FORMATS = {"2:4": 4, "4:6": 6, "6:8": 8}
_LENGTHS = frozenset(FORMATS.values())


def _ceil_div(a, b):
    return -(-a // b)


def group_size(mode):
    """Group length L of a mode given as "2:4" / "4:6" / "6:8" or directly as 4 / 6 / 8."""
    length = FORMATS.get(mode) if isinstance(mode, str) else mode
    if isinstance(length, bool) or length not in _LENGTHS:
        raise ValueError(f"unknown sparsity mode {mode!r}: expected 2:4, 4:6 or 6:8")
    return int(length)


def lifted_k(k, mode, alignment=128):
    """(valid, padded): the width of the slid weight / activation and that width rounded up to
    `alignment` columns.  Every group of L columns becomes L/2-1 windows of 4."""
    if k <= 0:
        raise ValueError("K must be positive")
    if alignment <= 0 or alignment % 4:
        raise ValueError("the alignment must be a positive multiple of four")
    length = group_size(mode)
    windows_per_group = length // 2 - 1
    valid = _ceil_div(k, length) * windows_per_group * 4
    return valid, _ceil_div(valid, alignment) * alignment


@torch.no_grad()
def slide_weight(qweight, mode):
    """CPU INT8 [out_features, in_features] -> CPU INT8 [out_features, valid].

    Every nonzero of the input appears exactly once in the output and nothing is pruned or
    re-quantised: windows are visited left to right and lanes left to right inside a window; a
    window takes at most two nonzeros that no earlier window has taken.  A group with more than
    L-2 nonzeros cannot be represented and raises ValueError.
    """
    from . import backend
    if not isinstance(qweight, torch.Tensor) or qweight.device.type != "cpu" or qweight.dtype != torch.int8 \
            or qweight.ndim != 2:
        raise TypeError("slide_weight takes a CPU INT8 tensor of shape [out_features, in_features]")
    rows, k = qweight.shape
    if rows == 0 or k == 0:
        raise ValueError("slide_weight needs at least one row and one column")
    length = group_size(mode)
    valid, _ = lifted_k(k, length)
    dense = qweight.contiguous()
    slid = torch.empty((rows, valid), dtype=torch.int8)
    status = backend.library().ss_slide_weight_cpu(ctypes.c_void_p(dense.data_ptr()), rows, k, length,
                                                   ctypes.c_void_p(slid.data_ptr()))
    if status == backend.SS_E_FORMAT:
        raise ValueError(f"a group of {length} columns holds more than {length - 2} nonzeros")
    backend.check(status)
    return slid
