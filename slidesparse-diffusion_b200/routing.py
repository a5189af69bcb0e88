"""Projection routing between the original dense members and packed sparse operators.

Mirror of the caller contract in the reference's `sdacc/diffusion_research/models/projections.py`
(`ProjectionState` :26-50, `OrdinaryProxy` :58-62): a state owns the original `nn.Linear`
members that share one input (Q|K|V, K|V, or a single FFN layer) and one packed operator per
sparsity mode; `select(mode)` switches between the dense members (mode 0) and the operator of
mode 4 / 6 / 8.  Attention cores and attention output projections are never routed.
"""
import torch
from torch.nn import functional as F


class ProjectionState:
    """members: nn.Linear modules with a common input; packed_by_mode: {4|6|8: callable(x[, output_addend=])}."""

    def __init__(self, members, packed_by_mode, protected_prefix=0):
        self.members = tuple(members)
        self.ops = dict(packed_by_mode)
        self.active = 0
        self.protected = int(protected_prefix)
        if self.protected and len(self.members) != 1:
            raise ValueError("a protected prefix belongs to a single output projection, not to fused members")
        self.widths = tuple(m.out_features for m in members)
        self.fuse = False      # run prologues inside the sparse operator's front-end kernel

    def select(self, mode):
        if type(mode) is not int or mode not in (0, 4, 6, 8):
            raise ValueError(f"mode is 0 (dense) or a group size 4 / 6 / 8, not {mode!r}")
        if mode != 0 and mode not in self.ops:
            raise ValueError(f"no packed operator was prepared for mode {mode}")
        self.active = mode

    def _sparse(self, x, prologue):
        op = self.ops[self.active]
        if prologue is None:
            return op(x)
        if self.fuse and hasattr(op, "forward_fused"):
            return op.forward_fused(x, prologue)
        return op(prologue.torch_reference(x))

    def members_output(self, x, prologue=None):
        """One output per member (dense), or the fused sparse output split by member widths.
        `prologue` (backend.Prologue) is an element-wise neighbour applied to x first: separate
        PyTorch operators on the dense path, inside the front-end kernel on the sparse path when
        `fuse` is set."""
        if self.active == 0:
            if prologue is not None:
                x = prologue.torch_reference(x)
            return tuple(module(x) for module in self.members)
        if self.protected:
            raise ValueError("a projection with a protected prefix has one output: use output()")
        return self._sparse(x, prologue).split(self.widths, dim=-1)

    def output(self, x, prologue=None, gated_residual=None):
        """Single-member projection; with a protected prefix the first columns of x stay a BF16
        dense product that the sparse operator adds in its epilogue.  `gated_residual` =
        (residual [batch, rows, n], gate [batch, n]) asks for residual + gate[b] * y: a PyTorch
        addcmul on the dense path, an in-place accumulation in the GEMM epilogue on the fused
        sparse path (rows per batch must then be a multiple of 32)."""
        if gated_residual is not None:
            residual, gate = gated_residual
            op = self.ops.get(self.active)
            fusable = (self.active != 0 and self.fuse and not self.protected and hasattr(op, "forward_fused")
                       and x.ndim == 3 and x.shape[1] % 32 == 0 and residual.is_contiguous())
            if fusable:
                return op.forward_fused(x, prologue, gate=gate, residual=residual)
            return torch.addcmul(residual, gate[:, None], self.output(x, prologue))
        if self.active == 0:
            return self.members[0](x if prologue is None else prologue.torch_reference(x))
        if not self.protected:
            return self._sparse(x, prologue)
        if prologue is not None:
            x = prologue.torch_reference(x)
        original = self.members[0]
        attention = F.linear(x[..., :self.protected], original.weight[:, :self.protected], None)
        return self.ops[self.active](x[..., self.protected:], output_addend=attention)

    def teacher(self, x):
        """Dense reference output of exactly the part the sparse operator replaces."""
        if not self.protected:
            return torch.cat([module(x) for module in self.members], dim=-1)
        original = self.members[0]
        return F.linear(x[..., self.protected:], original.weight[:, self.protected:], original.bias)


class OrdinaryProxy(torch.nn.Module):
    """Drop-in for a single routed nn.Linear."""

    def __init__(self, state):
        super().__init__()
        self.state = state
        self.original = state.members[0]
        self.in_features = self.original.in_features
        self.out_features = self.original.out_features

    def forward(self, x, prologue=None, gated_residual=None):
        return self.state.output(x, prologue, gated_residual)


def pack_members(members, mode, protected_prefix=0, curvature=None):
    """PackedLinear for the concatenation of dense members on their device, prepared entirely on
    the GPU.  With a `curvature` (reconstruction.factor_hessian of the members' shared input) the
    weight goes through the curvature-compensated pruner with joint INT8 rounding
    (`reconstruction.compress`); without one, through magnitude pruning to the (L-2):L pattern
    (the 2 smallest-|w| lanes of every aligned group of L go, ties to the lowest index; lanes
    missing from a tail group count as already pruned) and the per-channel INT8 grid
    (`ss_weight_grid_device`).  Either way slide + 2:4 packing happens on the device
    (`ss_pack_device`)."""
    import ctypes
    from . import backend
    from .packing import group_size, lifted_k
    from .runtime import PackedLinear, LAYOUT, kernel_source_sha
    length = group_size(mode)
    weight = torch.cat([m.weight for m in members]).detach()[:, protected_prefix:].float().contiguous()
    bias = None
    if all(m.bias is not None for m in members):
        bias = torch.cat([m.bias for m in members]).detach().float().contiguous()
    n, k = weight.shape
    device = weight.device
    lib = backend.library()
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    if curvature is not None:
        from .reconstruction import compress
        prepared = compress(weight, curvature, length, allow_tail=bool(k % length))
        qweight, scales = prepared["qweight"], prepared["scales"]
    else:
        pad = (-k) % length
        groups = torch.nn.functional.pad(weight.abs(), (0, pad), value=-1.0).reshape(n, -1, length)
        mask = torch.zeros_like(groups, dtype=torch.bool)
        for _ in range(2):                      # argmin returns the lowest index among ties
            first = groups.argmin(dim=-1, keepdim=True)
            mask.scatter_(-1, first, True)
            groups.scatter_(-1, first, float("inf"))
        mask = mask.reshape(n, -1)[:, :k]
        qweight = torch.empty((n, k), dtype=torch.int8, device=device)
        scales = torch.empty(n, dtype=torch.float32, device=device)
        with torch.cuda.device(device):
            weight.masked_fill_(mask, 0.0)
            backend.check(lib.ss_weight_grid_device(ctypes.c_void_p(weight.data_ptr()), n, k,
                                                    ctypes.c_void_p(qweight.data_ptr()),
                                                    ctypes.c_void_p(scales.data_ptr()), stream))
    with torch.cuda.device(device):
        _, pk = lifted_k(k, length)
        pn = -(-n // 32) * 32
        packed = torch.empty((pn, pk // 2), dtype=torch.int8, device=device)
        metadata = torch.empty(pn * pk // 32, dtype=torch.int32, device=device)
        status = torch.zeros(1, dtype=torch.int32, device=device)
        backend.check(lib.ss_pack_device(ctypes.c_void_p(qweight.data_ptr()), n, k, length,
                                         ctypes.c_void_p(packed.data_ptr()), ctypes.c_void_p(metadata.data_ptr()),
                                         ctypes.c_void_p(status.data_ptr()), stream))
    if int(status.item()):
        raise ValueError("weight violates the frozen (L-2):L structure")
    if bias is None:
        bias = torch.empty(0, dtype=torch.float32, device=device)
    identity = dict(k_physical=pk, kernel_source_sha=kernel_source_sha(), metadata_layout=LAYOUT, prepared_on="device")
    return PackedLinear(packed, metadata, scales, bias, k, n, length, identity=identity)
