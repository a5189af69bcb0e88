"""Exact, offline conversion of (L-2):L weight sparsity into overlapping hardware 2:4 windows.

Host-side mirror of the reference's `sdacc/w8a8_slidesparse/packing.py` (group_size :8-12,
lifted_k :15-20, slide_weight :23-52): same names, arguments, return values and error types.
The per-group work itself runs in the native library (`ss_slide_weight_cpu`).
"""
import ctypes

import torch

FORMATS = {"2:4": 4, "4:6": 6, "6:8": 8}


def group_size(mode):
    """'2:4' | '4:6' | '6:8' (or 4 | 6 | 8) -> group length L."""
    if isinstance(mode, str):
        if mode in FORMATS:
            return FORMATS[mode]
    elif not isinstance(mode, bool) and mode in (4, 6, 8):
        return int(mode)
    raise ValueError("format must be 2:4, 4:6, or 6:8")


def lifted_k(k, mode, alignment=128):
    """(valid, padded) lifted width: ceil(k/L) groups x (L/2-1) windows x 4 lanes."""
    if k <= 0 or alignment <= 0 or alignment % 4:
        raise ValueError("positive K and a multiple-of-four alignment required")
    length = group_size(mode)
    valid = -(-k // length) * (length // 2 - 1) * 4
    return valid, -(-valid // alignment) * alignment


@torch.no_grad()
def slide_weight(qweight, mode):
    """Preserve every nonzero exactly once; never prune or requantise here.

    Windows are visited in increasing order and, inside a window, lanes in increasing order;
    each window keeps at most two nonzeros that no earlier window kept.  Structural zeros stay
    zero.  CPU INT8 [out_features, in_features] in, CPU INT8 [out_features, valid] out.
    Raises ValueError when a group holds more than L-2 nonzeros.
    """
    from . import backend
    if qweight.device.type != "cpu" or qweight.dtype != torch.int8 or qweight.ndim != 2:
        raise TypeError("packing requires a CPU INT8 [out_features,in_features] tensor")
    n, k = qweight.shape
    if n <= 0 or k <= 0:
        raise ValueError("empty weights are unsupported")
    length = group_size(mode)
    valid, _ = lifted_k(k, length)
    source = qweight.contiguous()
    out = torch.empty((n, valid), dtype=torch.int8)
    lib = backend.library()
    rc = lib.ss_slide_weight_cpu(ctypes.c_void_p(source.data_ptr()), n, k, length,
                                 ctypes.c_void_p(out.data_ptr()))
    if rc == backend.SS_E_FORMAT:
        raise ValueError("weight violates the frozen (L-2):L structure")
    backend.check(rc)
    return out
