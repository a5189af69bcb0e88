"""`quantize_lift` and the `PackedLinear` module: the Python face of the projection.

A forward pass is two kernel launches of the native library, the quantise + slide front-end and
the sparse tcgen05 GEMM with its dequantising epilogue, reached through the `sdacc_*` torch
operators that `backend` registers.

The names, constructor and method signatures, accepted argument values, buffer names, exception
types and the save / load payload keys are those of the reference's
`sdacc/w8a8_slidesparse/runtime.py` (`quantize_lift` :72-95, `PackedLinear` :98-243), because its
callers construct the module directly, alias its buffers and pass its SM80 execution choices.
Those choices (`config` tile ids, `strategy`, Triton / native `frontend` names) select nothing
here, there is one pair of kernels, but they are validated the same way, and the `graph*` /
`direct2_*` front-ends still mean "use a prepared plan".
"""
import hashlib
from pathlib import Path

import torch

from . import backend
from .packing import group_size, lifted_k, slide_weight
from .profile import execution_profile, known_configurations

# values a caller may pass (validated, then mostly ignored: see the module docstring)
STRATEGIES = ("register", "reload")
_PLAIN_FRONTENDS = ("triton", "native", "scalar", "packed16")
_PLAN_FRONTENDS = ("graph_native", "graph_packed16", "graph1_native", "graph1_packed16",
                   "direct2_native", "direct2_packed16")
FRONTENDS = _PLAIN_FRONTENDS + _PLAN_FRONTENDS + ("auto",)
LAYOUT = "b200-v1"          # tag of this library's metadata word order, kept in identity / payloads
# `kernel_source_sha` values of payloads written by the reference's packer (the hashes its own
# `PackedLinear.load` accepts, sdacc/w8a8_slidesparse/runtime.py:236-238, plus its current
# csrc/dualscale_sm80.cu): all of them store metadata in the SM80 kernel's word order, which
# `load` converts.  A payload from any other packer is refused rather than guessed at.
REFERENCE_PACKER_SHAS = frozenset((
    "f27beddfed9f44b10a239772acc812f78cf78a999fbbeaea7ccd22f3a16c587f",
    "2787082a7feed4f7d9287578f7b7cac80857770dc4d8d704cdf888dca4a625a4",
    "e4af641f13175c73225ed6cc8e15a50c88de5d7454811151811081fa85551c61",
    "33f19700a1d9e6e01390cdc19627837ecfdeca2fffdd45e65ca1e7e7cac0c12d",
    "600cbf9ffdd7a863b9d04a0afdab6279caea70d3a705ea8cf92e26ab8c9f0b7a",
))
_TENSOR_KEYS = ("packed", "metadata", "scales", "bias")
_PAYLOAD_VERSION = 1


def kernel_source_sha():
    """Hash of the GEMM source: operators packed for another kernel generation are told apart by it."""
    return backend.sha(Path(__file__).parent / "csrc" / "ss_gemm.cu")


def quantize_lift(x, mode="2:4", strategy="register"):
    """Per-token dynamic INT8 quantisation and slide expansion of a BF16 CUDA matrix.

    x is [M, K] with unit column stride (any row stride).  Returns `(q, scale)`: q INT8
    [ceil32(M), ceil128(K')] with K' the lifted width of the mode, scale FP32 [ceil32(M)].  Rows
    beyond M are zero with scale 1.  The same scale (with its floor) is used to dequantise.
    """
    if strategy not in STRATEGIES:
        raise ValueError(f"strategy must be one of {STRATEGIES}")
    if x.ndim != 2:
        raise ValueError("quantize_lift takes a 2-D [M, K] tensor")
    return torch.ops.sdacc_mild_projection_sm80.quantize(x, group_size(mode))


def _check_execution(config, strategy, frontend):
    if config != "auto" and config not in backend.VALID_CONFIGS:
        raise ValueError(f"config must be 'auto' or one of {sorted(backend.VALID_CONFIGS)}")
    if strategy not in STRATEGIES:
        raise ValueError(f"strategy must be one of {STRATEGIES}")
    if frontend not in FRONTENDS:
        raise ValueError(f"frontend must be one of {FRONTENDS}")


def _channel_vector(values, channels, what, strictly_positive=False, optional=False):
    """A per-output-channel parameter as contiguous CPU FP32 [channels]; None -> empty if optional."""
    if values is None:
        if not optional:
            raise ValueError(f"{what} required")
        return torch.empty(0, dtype=torch.float32)
    vector = values.detach().to("cpu", torch.float32).contiguous()
    if optional and vector.numel() == 0:
        return vector
    bad = tuple(vector.shape) != (channels,) or not bool(torch.isfinite(vector).all())
    if bad or (strictly_positive and bool((vector <= 0).any())):
        kind = "finite and positive" if strictly_positive else "finite"
        raise ValueError(f"{what} must be {kind} with one value per output channel ({channels})")
    return vector


def _is_plan_frontend(frontend):
    return frontend in _PLAN_FRONTENDS


class PackedLinear(torch.nn.Module):
    """A prepared sparse W8A8 projection: y[..., n] = x[..., k] . W^T (+ bias) in BF16.

    Several projections of the same input (Q|K|V, K|V) are prepared as ONE operator from the
    row-wise concatenation of their weights, scales and biases; the caller cuts the output back
    into members (`composite.SharedProjection`).  The four buffers `packed`, `metadata`, `scales`
    and `bias` are handed to the kernels as pointers at every launch, so a caller may overwrite
    their contents in place (mode banks, per-step affine coefficients) without a new module.
    """

    def __init__(self, packed, metadata, scales, bias, k, n, mode, config="auto",
                 strategy="register", identity=None, frontend="auto"):
        super().__init__()
        for key, tensor in zip(_TENSOR_KEYS, (packed, metadata, scales, bias)):
            self.register_buffer(key, tensor)
        self.in_features = self.k = int(k)
        self.out_features = self.n = int(n)
        self.mode = group_size(mode)
        self.config = config if config == "auto" else int(config)
        self.strategy = strategy
        self.frontend = frontend
        self.identity = dict(identity) if identity else {}
        self._graphs = {}                     # rows M -> prepared-plan handle

    # ---- offline ------------------------------------------------------------------------------

    @classmethod
    def prepare(cls, qweight, scales, bias=None, mode="2:4", config="auto",
                strategy="register", frontend="auto"):
        """Pack an already pruned and quantised weight: CPU INT8 [N, K] with FP32 scales [N]
        (and optionally an FP32 bias [N]) -> operator with CPU buffers (move it with `.to`)."""
        _check_execution(config, strategy, frontend)
        channels, width = qweight.shape
        channel_scales = _channel_vector(scales, channels, "per-channel scales", strictly_positive=True)
        channel_bias = _channel_vector(bias, channels, "per-channel bias", optional=True)
        slid = slide_weight(qweight, mode)                       # raises on a structure violation
        padded_width = lifted_k(width, mode)[1]
        values, metadata = torch.ops.sdacc_dualscale_sm80.pack_cpu(slid, padded_width)
        identity = {
            "qweight_sha": hashlib.sha256(qweight.contiguous().numpy().tobytes()).hexdigest(),
            "k_lifted": slid.shape[1],
            "k_physical": padded_width,
            "metadata_layout": LAYOUT,
            "kernel_source_sha": kernel_source_sha(),
        }
        return cls(values, metadata, channel_scales, channel_bias, width, channels, mode,
                   config=config, strategy=strategy, identity=identity, frontend=frontend)

    # ---- execution choices and prepared plans ---------------------------------------------------

    def configuration_for(self, m):
        """(config, frontend) used for M rows: what the constructor fixed, else the profile's."""
        profile_config, profile_frontend = execution_profile(self.mode, m, self.k, self.n)
        config = profile_config if self.config == "auto" else self.config
        frontend = profile_frontend if self.frontend == "auto" else self.frontend
        return config, frontend

    def configure(self, has_addend=False):
        """Kernel resources `[threads, shared memory, registers, local memory, CTAs per SM]` (twice,
        as the reference reports a base and a full-tile variant): a dict per configuration when
        `config` is "auto", else the list of the fixed configuration."""
        query = torch.ops.sdacc_dualscale_sm80.configure
        if self.config != "auto":
            return query(self.packed, self.config, has_addend)
        return {c: query(self.packed, c, has_addend) for c in known_configurations(self.mode, self.k, self.n)}

    def configure_for(self, m):
        """Prepare for M rows ahead of time.  Returns the plan handle if the front-end in force is
        a prepared-plan one (resident scratch in the native library), else None."""
        config, frontend = self.configuration_for(m)
        self.configure()
        if not _is_plan_frontend(frontend):
            return None
        if m not in self._graphs:
            namespace = torch.ops.sdacc_prepared_projection_sm80
            if frontend.startswith("direct2_"):
                create = namespace.prepare_direct2
            elif frontend.startswith("graph1_"):
                create = namespace.prepare_singlepatch
            else:
                create = namespace.prepare
            self._graphs[m] = create(self.packed, self.metadata, self.scales, self.bias, self.k, m, self.n,
                                     self.mode, config, frontend.endswith("packed16"))
        return self._graphs[m]

    def close_graphs(self):
        """Release every prepared plan (their handles point at this module's current buffers)."""
        while self._graphs:
            _, handle = self._graphs.popitem()
            torch.ops.sdacc_prepared_projection_sm80.release(handle)

    def _apply(self, fn, recurse=True):
        # .to() / .cuda() replace the buffers: plans built over the old ones must go first
        if getattr(self, "_graphs", None):
            self.close_graphs()
        return super()._apply(fn, recurse)

    # ---- forward ----------------------------------------------------------------------------------

    def _check_input(self, x):
        if not (x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] == self.k):
            raise ValueError(f"expected a BF16 CUDA tensor whose last dimension is {self.k}")

    def _flat_addend(self, x, output_addend):
        expected = (*x.shape[:-1], self.n)
        if (tuple(output_addend.shape) != expected or output_addend.dtype != torch.bfloat16
                or output_addend.device != x.device):
            raise ValueError(f"output_addend must be BF16 {expected} on the input's device")
        flat = output_addend.reshape(-1, self.n)
        return flat if flat.stride(-1) == 1 else flat.contiguous()

    def forward(self, x, output_addend=None):
        """BF16 [..., k] -> new BF16 [..., n]; `output_addend` (BF16 [..., n]) is added in the epilogue."""
        self._check_input(x)
        rows = x.numel() // self.k if self.k else 0
        if rows == 0:
            return x.new_empty((*x.shape[:-1], self.n))
        config, frontend = self.configuration_for(rows)
        addend = None if output_addend is None else self._flat_addend(x, output_addend)
        if addend is None and _is_plan_frontend(frontend):
            if rows not in self._graphs:
                raise RuntimeError(f"no prepared plan for {rows} rows: call configure_for({rows}) first")
            return torch.ops.sdacc_prepared_projection_sm80.run(x, self._graphs[rows], self.n)
        operators = torch.ops.sdacc_mild_projection_sm80
        entry = {"packed16": operators.projection_packed16, "scalar": operators.projection_scalar}.get(
            frontend, operators.projection)
        return entry(x, self.packed, self.metadata, self.scales, self.bias, self.mode, self.n, config, addend)

    def forward_fused(self, x, prologue=None, output_addend=None, gate=None, residual=None):
        """forward(prologue(x)) with the element-wise neighbours inside the kernels: `prologue`
        (backend.Prologue: LayerNorm + modulation or GELU) is computed by the front-end, and with
        `gate` [batch, n] and `residual` [batch, rows, n] the epilogue accumulates
        residual += gate[b] * y in place and returns `residual`.  An extension of the reference module."""
        self._check_input(x)
        if x.numel() == 0:
            return residual if gate is not None else x.new_empty((*x.shape[:-1], self.n))
        if output_addend is not None:
            self._flat_addend(x, output_addend)            # shape / dtype check only
        return backend.projection_fused(x, prologue or backend.Prologue("none"), self.packed, self.metadata,
                                        self.scales, self.bias, self.mode, self.n, output_addend, gate, residual)

    # ---- persistence ------------------------------------------------------------------------------

    def save(self, path):
        """Write a tensors-and-scalars payload (no handles, no pickled objects) that `load` and the
        reference's own `PackedLinear.load` key set understand."""
        payload = {"version": _PAYLOAD_VERSION, "k": self.k, "n": self.n, "mode": self.mode,
                   "config": self.config, "strategy": self.strategy, "frontend": self.frontend,
                   "identity": self.identity}
        for key in _TENSOR_KEYS:
            payload[key] = getattr(self, key).detach().cpu()
        torch.save(payload, path)

    @classmethod
    def load(cls, path, device="cpu", optimized=True):
        """Rebuild an operator from a payload.  One written by the reference (no layout tag; its
        metadata is in the SM80 kernel's word order) is converted to this library's order.  With
        `optimized` the stored execution choice is kept in the identity and replaced by "auto"."""
        payload = torch.load(path, map_location="cpu", weights_only=True)
        if payload.get("version") != _PAYLOAD_VERSION:
            raise ValueError(f"payload version {payload.get('version')!r} is not supported")
        identity = dict(payload["identity"])
        metadata = payload["metadata"]
        layout, packer = identity.get("metadata_layout"), identity.get("kernel_source_sha")
        if layout == LAYOUT:
            # this library's word order; the hash is provenance only (the order is what the tag names,
            # and the tag changes whenever the packed or metadata layout does)
            if packer is None:
                raise ValueError("the payload does not say which kernel source packed it")
        elif layout is not None:
            raise ValueError(f"unknown metadata layout {layout!r}: this library reads {LAYOUT!r} and the reference's payloads")
        else:
            if packer not in REFERENCE_PACKER_SHAS:
                raise ValueError("untagged payload from an unknown packer: its metadata order cannot be assumed "
                                 f"(kernel_source_sha {packer!r})")
            from .importer import sm80_metadata_to_b200
            rows, half_width = payload["packed"].shape
            metadata = sm80_metadata_to_b200(metadata, rows, 2 * half_width)
            identity["imported_from"] = identity.get("kernel_source_sha")
            identity["kernel_source_sha"] = kernel_source_sha()
            identity["metadata_layout"] = LAYOUT
        config, frontend = payload["config"], payload.get("frontend", "triton")
        if optimized:
            identity["loaded_execution_original"] = {"config": config, "frontend": frontend}
            config = frontend = "auto"
        module = cls(payload["packed"], metadata, payload["scales"], payload["bias"], payload["k"], payload["n"],
                     payload["mode"], config=config, strategy=payload["strategy"], identity=identity,
                     frontend=frontend)
        return module.to(device)
