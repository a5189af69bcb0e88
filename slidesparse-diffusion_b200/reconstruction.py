"""Weight preparation for the sparse projection: from a dense weight and the Hessian of its input
to the pruned INT8 `qweight` and per-channel `scales` that `PackedLinear.prepare` consumes.

Same functions, arguments, errors and result keys as the reference's
`sdacc/diffusion_research/reconstruction.py` (`factor_hessian` :18-39, `channel_scales` :41-49,
`round_signed` :52-53, `compress` :55-133).  `compress` runs on the GPU through the C-ABI kernels
(`ss_obs_block`, `ss_obs_trailing`, `ss_obs_finish`): eight lanes per output row walk a column block
in order, the block's errors reach the later columns through an fp32 GEMM with a fixed summation
order, so a result does not depend on the GPU, the grid or the run.  There is no CPU path: a CPU
weight is refused.
"""
import ctypes
from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Curvature:
    upper: torch.Tensor       # upper Cholesky factor of the damped inverse Hessian, fp32 [K,K]
    dead: torch.Tensor        # bool [K]: inputs that never fired (zero Hessian diagonal)
    damping: float            # what was added to the diagonal


@torch.inference_mode()
def factor_hessian(hessian, damping=.01):
    """Shared factor of all output rows: H + damping*mean(diag) on the diagonal, dead inputs
    decoupled, then the upper Cholesky factor of the inverse.  A Hessian that is not positive
    definite after damping fails in the factorisation; nothing is retried with more damping."""
    if hessian.ndim != 2 or hessian.shape[0] != hessian.shape[1]:
        raise ValueError(f"the Hessian must be a square matrix, got {tuple(hessian.shape)}")
    if damping < 0:
        raise ValueError("damping must not be negative")
    h = hessian.detach().to(torch.float32).clone()
    if not bool(torch.isfinite(h).all()):
        raise ValueError("the Hessian holds non-finite values")
    if not torch.allclose(h, h.T, rtol=1e-5, atol=1e-6):
        raise ValueError("the Hessian is not symmetric")
    diagonal = h.diagonal()                    # a view: the edits below land in h
    dead = diagonal == 0
    if bool(dead.any()) and int(torch.count_nonzero(h[dead])):
        raise ValueError("an input with a zero diagonal entry has non-zero cross terms")
    diagonal[dead] = 1
    amount = damping * diagonal.mean()
    diagonal += amount
    inverse = torch.cholesky_inverse(torch.linalg.cholesky(h))
    return Curvature(torch.linalg.cholesky(inverse, upper=True), dead, float(amount))


@torch.inference_mode()
def channel_scales(weight):
    """Signed symmetric 8-bit grid per output row: 2*absmax/255, 1 for a row of zeros.  The
    quotient is an IEEE division on every device (torch's CUDA division by a Python number
    multiplies by the rounded reciprocal and can differ in the last bit from the CPU result)."""
    top = weight.detach().float().abs().amax(dim=1)
    return torch.where(top > 0, (2 * top) / torch.full_like(top, 255), torch.ones_like(top))


def round_signed(value, scales):
    return torch.round(value / scales).clamp(-128, 127)


def max_blocksize():
    """Widest column block the device kernel holds in shared memory."""
    from . import backend
    return int(backend.library().ss_obs_max_blocksize())


def _check_compress_arguments(weight, curvature, group, method, blocksize, allow_tail):
    """The reference's argument contract (`reconstruction.py:66-82` there): every violation is a
    ValueError raised before any work is done.  Returns (rows, columns)."""
    if group not in (4, 6, 8):
        raise ValueError(f"sparsity group must be 4, 6 or 8, not {group!r}")
    if method != "joint" and method != "prune_then_rtn":
        raise ValueError(f"method must be 'joint' or 'prune_then_rtn', not {method!r}")
    if blocksize < 1 or blocksize % group != 0:
        raise ValueError(f"a column block of {blocksize} inputs would cut a group of {group}")
    if weight.ndim != 2 or weight.numel() == 0:
        raise ValueError("the weight must be a non-empty matrix [outputs, inputs]")
    if not bool(torch.isfinite(weight).all()):
        raise ValueError("the weight holds non-finite values")
    rows, columns = weight.shape
    if not allow_tail and columns % group != 0:
        raise ValueError(f"{columns} inputs leave an incomplete group of {group}; pass allow_tail=True to accept it")
    if tuple(curvature.upper.shape) != (columns, columns):
        raise ValueError(f"the curvature factor is {tuple(curvature.upper.shape)}, the weight has {columns} inputs")
    if curvature.upper.device != weight.device:
        raise ValueError("the curvature factor and the weight are on different devices")
    return rows, columns


def _check_scales(scales, rows, device):
    scales = scales.detach().float().clone()
    if tuple(scales.shape) != (rows,) or scales.device != device:
        raise ValueError(f"scales must be [{rows}] on the weight's device")
    if not bool(torch.isfinite(scales).all()) or not bool((scales > 0).all()):
        raise ValueError("scales must be finite and positive")
    return scales


@torch.inference_mode()
def compress(weight, curvature, group, *, method="joint", blocksize=192, scales=None, allow_tail=False,
             progress=None):
    """Prune `weight` [N,K] to two zeros per group of `group` inputs, compensating the remaining
    inputs of each row through the shared curvature, and (method "joint") round every input to the
    row's INT8 grid as it is finalised.  Returns the reference's dictionary: qweight int8, scales,
    zeros (bool), compensated (fp32), proxy_loss [N], method, group, blocksize, weight_grid,
    curvature_damping, activation_error_compensated."""
    rows, columns = _check_compress_arguments(weight, curvature, group, method, blocksize, allow_tail)
    if scales is not None:
        scales = _check_scales(scales, rows, weight.device)
    if not weight.is_cuda:
        raise ValueError("compress runs on the GPU only: move the weight and the curvature to a CUDA device")
    from . import backend
    lib = backend.library()
    if blocksize > max_blocksize():
        raise ValueError(f"column blocks wider than {max_blocksize()} do not fit the kernel's shared memory")
    device = weight.device
    if scales is None:
        scales = channel_scales(weight)
    scales = scales.contiguous()
    w = weight.detach().float().clone().contiguous()
    w[:, curvature.dead] = 0
    upper = curvature.upper.detach().float().contiguous()
    zeros = torch.zeros((rows, columns), dtype=torch.bool, device=device)
    losses = torch.zeros(rows, dtype=torch.float32, device=device)
    errors = torch.empty((rows, min(blocksize, columns)), dtype=torch.float32, device=device)
    qweight = torch.empty((rows, columns), dtype=torch.int8, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    joint = method == "joint"
    with torch.cuda.device(device):
        stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
        for start in range(0, columns, blocksize):
            width = min(blocksize, columns - start)
            backend.check(lib.ss_obs_block(p(w), rows, columns, start, width, p(upper), p(scales), group,
                                           int(joint), p(zeros), p(errors), p(losses), stream))
            backend.check(lib.ss_obs_trailing(p(w), rows, columns, start, width, p(upper), p(errors), stream))
            if progress is not None:
                progress(finalized_columns=start + width, total_columns=columns)
        zeros[:, curvature.dead] = True
        backend.check(lib.ss_obs_finish(p(w), p(scales), p(zeros), rows, columns, group, int(joint),
                                        p(qweight), p(status), stream))
    # the reference's three post-conditions, each a RuntimeError
    flags = int(status.item())
    if not bool(torch.isfinite(w).all()):
        raise RuntimeError("the compensated weight holds non-finite values")
    if flags & 1:
        raise RuntimeError("a jointly rounded weight is not on its row's INT8 grid")
    if flags & 2:
        raise RuntimeError("a complete group keeps more than group-2 non-zero weights")
    return dict(qweight=qweight, scales=scales, zeros=zeros, compensated=w, proxy_loss=losses, method=method,
                group=group, blocksize=blocksize, weight_grid="signed[-128,127]; scale=2*Dense-row-absmax/255",
                curvature_damping=curvature.damping, activation_error_compensated=False)
