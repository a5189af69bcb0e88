"""One quantise+slide launch and one sparse tcgen05 GEMM launch per projection.

Host-side mirror of the reference's `sdacc/w8a8_slidesparse/runtime.py`: `quantize_lift`
(:72-95) and the `PackedLinear` module (:98-243) keep their names, constructor and method
signatures, accepted argument values, buffer names, error types and the save/load payload.  The
reference's Triton front-ends and SM80 tile configurations do not exist here: every `frontend` /
`config` / `strategy` value the reference accepts is still accepted (callers pass them), but all
of them execute the same two sm_100a kernels through the `sdacc_*` operators.
"""
import hashlib
from pathlib import Path

import torch

from . import backend
from .packing import group_size, lifted_k, slide_weight
from .profile import execution_profile, known_configurations

FRONTENDS = ("triton", "native", "scalar", "packed16", "graph_native", "graph_packed16",
             "graph1_native", "graph1_packed16", "direct2_native", "direct2_packed16", "auto")
STRATEGIES = ("register", "reload")
LAYOUT = "b200-v1"     # metadata order tag stored in identity / payloads


def kernel_source_sha():
    return backend.sha(Path(__file__).parent / "csrc" / "ss_gemm.cu")


def quantize_lift(x, mode="2:4", strategy="register"):
    """Dynamic per-token quantisation; quantise and dequantise share the same scale floor.

    x: BF16 CUDA [M,K] with unit column stride (row stride may be larger than K).  Returns
    (q int8 [ceil32(M), ceil128(K')], scale fp32 [ceil32(M)]); padding and the sliding expansion
    are produced inside the single kernel.
    """
    length = group_size(mode)
    if strategy not in STRATEGIES:
        raise ValueError("unknown Quant+Lift strategy")
    if x.ndim != 2:
        raise ValueError("[M,K] input required")
    return torch.ops.sdacc_mild_projection_sm80.quantize(x, length)


class PackedLinear(torch.nn.Module):
    """Frozen packed projection, supporting shared-input QKV/KV concatenation.

    Prepare with concatenate([q,k,v]) along output channels, using identically ordered
    scales/bias, and split the output by widths outside this module.  Buffers `packed`,
    `metadata`, `scales`, `bias` are read by the kernels at launch time, so callers may overwrite
    their contents in place between calls.
    """

    def __init__(self, packed, metadata, scales, bias, k, n, mode, config="auto",
                 strategy="register", identity=None, frontend="auto"):
        super().__init__()
        self.k, self.n = int(k), int(n)
        self.mode = group_size(mode)
        self.config, self.strategy = ("auto" if config == "auto" else int(config)), strategy
        self.frontend = frontend
        self._graphs = {}
        self.in_features, self.out_features = self.k, self.n
        self.identity = identity or {}
        for name, value in (("packed", packed), ("metadata", metadata),
                            ("scales", scales), ("bias", bias)):
            self.register_buffer(name, value)

    @classmethod
    def prepare(cls, qweight, scales, bias=None, mode="2:4", config="auto",
                strategy="register", frontend="auto"):
        """CPU int8 [N,K] (already pruned and quantised) + fp32 scales [N] -> packed operator."""
        if (config != "auto" and config not in backend.VALID_CONFIGS) or strategy not in STRATEGIES:
            raise ValueError("unsupported execution configuration")
        if frontend not in FRONTENDS:
            raise ValueError("unknown frontend")
        n, k = qweight.shape
        scales = scales.detach().cpu().float().contiguous()
        bias = torch.empty(0, dtype=torch.float32) if bias is None else bias.detach().cpu().float().contiguous()
        if scales.shape != (n,) or not torch.isfinite(scales).all() or torch.any(scales <= 0):
            raise ValueError("finite positive per-channel scales required")
        if bias.numel() and (bias.shape != (n,) or not torch.isfinite(bias).all()):
            raise ValueError("finite per-channel bias required")
        lifted = slide_weight(qweight, mode)
        _, pk = lifted_k(k, mode)
        packed, metadata = torch.ops.sdacc_dualscale_sm80.pack_cpu(lifted, pk)
        identity = dict(qweight_sha=hashlib.sha256(qweight.contiguous().numpy().tobytes()).hexdigest(),
                        k_physical=pk, k_lifted=lifted.shape[1],
                        kernel_source_sha=kernel_source_sha(), metadata_layout=LAYOUT)
        return cls(packed, metadata, scales, bias, k, n, mode, config, strategy, identity, frontend)

    # -- resources / prepared plans ------------------------------------------------------------

    def _uses_plan(self, frontend):
        return frontend.startswith(("graph", "direct2_"))

    def _prepare_plan(self, m, config, frontend):
        ops = torch.ops.sdacc_prepared_projection_sm80
        make = (ops.prepare_direct2 if frontend.startswith("direct2_")
                else ops.prepare_singlepatch if frontend.startswith("graph1_") else ops.prepare)
        return make(self.packed, self.metadata, self.scales, self.bias, self.k, m, self.n,
                    self.mode, config, frontend.endswith("packed16"))

    def configure(self, has_addend=False):
        """Inspect kernel resources before timing (and build plans for profiled plan shapes)."""
        configs = known_configurations(self.mode, self.k, self.n) if self.config == "auto" else [self.config]
        resources = {c: torch.ops.sdacc_dualscale_sm80.configure(self.packed, c, has_addend) for c in configs}
        return resources if self.config == "auto" else resources[self.config]

    def configure_for(self, m):
        """Offline preparation of a shape-specific plan (resident scratch) for M rows."""
        config, frontend = self.configuration_for(m)
        self.configure()
        if self._uses_plan(frontend) and m not in self._graphs:
            self._graphs[m] = self._prepare_plan(m, config, frontend)
        return self._graphs.get(m)

    def close_graphs(self):
        for handle in self._graphs.values():
            torch.ops.sdacc_prepared_projection_sm80.release(handle)
        self._graphs.clear()

    def _apply(self, fn, recurse=True):
        if getattr(self, "_graphs", None):
            self.close_graphs()
        return super()._apply(fn, recurse)

    def configuration_for(self, m):
        """(config, frontend) for M rows: explicit constructor values win over the profile."""
        config, frontend = execution_profile(self.mode, m, self.k, self.n)
        if self.config != "auto":
            config = self.config
        if self.frontend != "auto":
            frontend = self.frontend
        return config, frontend

    # -- forward ---------------------------------------------------------------------------------

    def forward(self, x, output_addend=None):
        if x.dtype != torch.bfloat16 or not x.is_cuda or x.shape[-1] != self.k:
            raise ValueError("BF16 CUDA input with matching last dimension required")
        rows = x.numel() // self.k if self.k else 0
        if rows == 0:
            return x.new_empty((*x.shape[:-1], self.n))
        config, frontend = self.configuration_for(rows)
        if output_addend is not None:
            if (output_addend.shape != (*x.shape[:-1], self.n) or output_addend.dtype != torch.bfloat16
                    or output_addend.device != x.device):
                raise ValueError("output_addend must match BF16 output shape/device")
            output_addend = output_addend.reshape(-1, self.n)
            if output_addend.stride(-1) != 1:
                output_addend = output_addend.contiguous()
        if self._uses_plan(frontend) and output_addend is None:
            handle = self._graphs.get(rows)
            if handle is None:
                raise RuntimeError("configure_for(M) is required before graph forward")
            return torch.ops.sdacc_prepared_projection_sm80.run(x, handle, self.n)
        op = torch.ops.sdacc_mild_projection_sm80
        run = (op.projection_packed16 if frontend == "packed16"
               else op.projection_scalar if frontend == "scalar" else op.projection)
        return run(x, self.packed, self.metadata, self.scales, self.bias, self.mode, self.n, config,
                   output_addend)

    def forward_fused(self, x, prologue=None, output_addend=None, gate=None, residual=None):
        """forward(prologue(x)) with the element-wise neighbours inside the kernels: `prologue`
        (backend.Prologue: LayerNorm + modulation or GELU) is computed by the front-end, and with
        `gate` [batch, n] and `residual` [batch, rows, n] the epilogue accumulates
        residual += gate[b] * y in place and returns `residual`.  An extension of the reference module."""
        if x.dtype != torch.bfloat16 or not x.is_cuda or x.shape[-1] != self.k:
            raise ValueError("BF16 CUDA input with matching last dimension required")
        if x.numel() == 0:
            return residual if gate is not None else x.new_empty((*x.shape[:-1], self.n))
        if output_addend is not None and (output_addend.shape != (*x.shape[:-1], self.n)
                                          or output_addend.dtype != torch.bfloat16):
            raise ValueError("output_addend must match BF16 output shape/device")
        return backend.projection_fused(x, prologue or backend.Prologue("none"), self.packed, self.metadata,
                                        self.scales, self.bias, self.mode, self.n, output_addend, gate, residual)

    # -- persistence -----------------------------------------------------------------------------

    def save(self, path):
        """Portable tensor payload; no handles, searched plans, or Python pickle."""
        torch.save(dict(version=1, k=self.k, n=self.n, mode=self.mode, config=self.config,
                        strategy=self.strategy, identity=self.identity, frontend=self.frontend,
                        **{name: tensor.detach().cpu() for name, tensor in self.named_buffers()}), path)

    @classmethod
    def load(cls, path, device="cpu", optimized=True):
        """Load a payload written by save().  A payload written by the reference implementation
        (metadata in its SM80 order, recognised by the missing layout tag) is converted."""
        blob = torch.load(path, map_location="cpu", weights_only=True)
        if blob.pop("version") != 1:
            raise ValueError("unsupported packed payload version")
        identity = dict(blob["identity"])
        if identity.get("metadata_layout") != LAYOUT:
            from .importer import sm80_metadata_to_b200
            pn, half = blob["packed"].shape
            blob["metadata"] = sm80_metadata_to_b200(blob["metadata"], pn, 2 * half)
            identity.update(metadata_layout=LAYOUT, imported_from=identity.get("kernel_source_sha"),
                            kernel_source_sha=kernel_source_sha())
        elif identity.get("kernel_source_sha") is None:
            raise ValueError("packing/kernel source identity differs")
        blob["identity"] = identity
        if optimized:
            blob["identity"] = dict(identity, loaded_execution_original=dict(
                config=blob["config"], frontend=blob.get("frontend", "triton")))
            blob["config"], blob["frontend"] = "auto", "auto"
        return cls(**blob).to(device)
