"""Wrappers that present one packed operator as what a model block expects.

Two shapes of use occur in the reference's models (`sdacc/w8a8_slidesparse/composite.py:4-19`):
several projections of one input fused into a single operator whose output is cut back into the
members (Q|K|V, K|V), and an output projection whose input is the concatenation of a protected
attention part and an FFN part (FLUX single-stream blocks), where only the FFN columns are sparse.
Both keep the reference's constructor arguments, attributes and `configure()` results.
"""
import torch


def _member_slices(widths):
    """[(start, stop)] of consecutive members with the given widths."""
    bounds, start = [], 0
    for width in widths:
        width = int(width)
        if width <= 0:
            raise ValueError("member widths must be positive")
        bounds.append((start, start + width))
        start += width
    return bounds


class SharedProjection(torch.nn.Module):
    """`packed` computes all members at once; forward returns one view per member, in order."""

    def __init__(self, packed, widths):
        super().__init__()
        self.packed = packed
        self.widths = tuple(int(w) for w in widths)
        self._slices = _member_slices(self.widths)
        if not self._slices or self._slices[-1][1] != packed.n:
            raise ValueError(f"member widths {self.widths} do not add up to the operator's {packed.n} channels")

    def configure(self):
        return self.packed.configure()

    def forward(self, x):
        fused = self.packed(x)
        return tuple(fused[..., lo:hi] for lo, hi in self._slices)


class ProtectedFFNOutput(torch.nn.Module):
    """y = x[..., :p] @ attention_weight.T  (BF16, dense)  +  ffn(x[..., p:])  (sparse W8A8).

    The dense product is handed to the sparse operator as `output_addend`, so the sum is formed in
    its epilogue and no separate add kernel runs.  `attention_weight` is [n, p] BF16; the sparse
    operator reads the remaining columns of x in place (a column slice, arbitrary row stride)."""

    def __init__(self, ffn, attention_weight):
        super().__init__()
        rows, self.protected = attention_weight.shape
        if attention_weight.dtype is not torch.bfloat16:
            raise ValueError("the protected weight must be BF16")
        if rows != ffn.n:
            raise ValueError(f"the protected weight has {rows} output channels, the FFN operator {ffn.n}")
        self.ffn = ffn
        self.register_buffer("attention_weight", attention_weight)

    def configure(self):
        return {"ffn": self.ffn.configure(), "mixed": self.ffn.configure(has_addend=True)}

    def forward(self, x):
        expected = self.protected + self.ffn.k
        if x.shape[-1] != expected:
            raise ValueError(f"input width {x.shape[-1]} is not protected {self.protected} + FFN {self.ffn.k}")
        attention, rest = x[..., :self.protected], x[..., self.protected:]
        return self.ffn(rest, output_addend=torch.matmul(attention, self.attention_weight.t()))
