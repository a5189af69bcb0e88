"""Build and load the sm_100a native library; register the reference's torch op names on it.

Host-side mirror of `sdacc/w8a8_slidesparse/backend.py` (build_native :17-70, load_native
:73-118).  The native artefact is a thin C-ABI shared library (include/slidesparse_b200.h) built
with nvcc for sm_100a only -- no CUTLASS, no Triton, no second backend, no CPU fallback: every
operator below raises if the library is missing.

The operators keep the reference's names and schemas (csrc/dualscale_sm80.cu:400-406,
csrc/projection_sm80.cu:154-169, csrc/graph_projection.cuh:178-195) so callers that look them up
through `torch.ops.sdacc_*` keep working; `config` arguments are validated and otherwise ignored
(the SM80 tile identifiers mean nothing here, the library picks its own tile).
"""
import ctypes
import hashlib
import json
import os
import subprocess
from pathlib import Path

import torch

from .packing import group_size, lifted_k

SS_E_ARG, SS_E_CUDA, SS_E_FORMAT, SS_E_HANDLE, SS_E_DEVICE, SS_E_LIMIT = -1, -2, -3, -4, -5, -6
LIBRARY_NAME = "libslidesparse_b200.so"
SOURCES = ("ss_api.cu", "ss_gemm.cu", "ss_frontend.cu", "ss_pack.cu", "ss_noalloc.cu", "ss_micro.cu", "ss_obs.cu")
ARCH = "sm_100a"
VALID_CONFIGS = (0, 1, 2, 3, 4, 5, 6, 11, 12, 13, 14, 15, 16, 17)

_PACKAGE = Path(__file__).resolve().parent
_lib = None
_loaded_sha = None
_ops_registered = False


def sha(path):
    return hashlib.sha256(Path(path).read_bytes()).hexdigest()


def default_directory():
    """Where build_native puts, and library() looks for, the in-tree artefact."""
    return _PACKAGE / "native_sm100a"


def _source_identity():
    csrc = _PACKAGE / "csrc"
    files = sorted(p for p in csrc.iterdir() if p.suffix in (".cu", ".cuh"))
    files.append(_PACKAGE.parent / "include" / "slidesparse_b200.h")
    return {p.name: sha(p) for p in files}


def build_native(output=None, arch=ARCH, force=False):
    """Offline build, without initialising CUDA; call before measurement.

    Compiles csrc/*.cu into <output>/libslidesparse_b200.so with
    `nvcc -gencode arch=compute_100a,code=sm_100a` and writes receipt.json (source / library
    hashes, torch and CUDA versions, the command).  Returns the receipt.  An up-to-date artefact
    is kept unless force=True.
    """
    if torch.cuda.is_initialized():
        raise RuntimeError("build in a fresh CPU-only process")
    if arch != ARCH:
        raise ValueError("this library is written for sm_100a only")
    output = Path(output) if output is not None else default_directory()
    output.mkdir(parents=True, exist_ok=True)
    target, receipt_path = output / LIBRARY_NAME, output / "receipt.json"
    identity = _source_identity()
    if not force and target.exists() and receipt_path.exists():
        old = json.loads(receipt_path.read_text())
        if old.get("complete") and old.get("source_dependencies") == identity and old.get("library_sha") == sha(target):
            return old
    nvcc = str(Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "bin/nvcc")
    cmd = [nvcc, "-std=c++17", "-O3", "--shared", "-Xcompiler", "-fPIC", "-lineinfo", "-Xptxas=-v",
           "-gencode", "arch=compute_100a,code=sm_100a"]
    cmd += [str(_PACKAGE / "csrc" / name) for name in SOURCES]
    cmd += ["-o", str(target)]
    log = output / "compile.log"
    with log.open("w") as f:
        subprocess.run(cmd, check=True, stdout=f, stderr=subprocess.STDOUT)
    receipt = dict(complete=True, arch=arch, library_sha=sha(target), source_dependencies=identity,
                   torch=torch.__version__, cuda=torch.version.cuda, command=cmd,
                   compile_log_sha=sha(log), cuda_initialized=torch.cuda.is_initialized())
    receipt_path.write_text(json.dumps(receipt, indent=2) + "\n")
    return receipt


BINDING_NAME = "SOURCE_BINDING.json"


def source_binding_files(directory=None):
    """Relative paths of the files a library directory is identified by: every Python and JSON file
    of the package and the CUDA sources (build products and the binding file itself excluded)."""
    root = Path(directory) if directory is not None else _PACKAGE
    names = []
    for path in sorted(root.rglob("*")):
        rel = path.relative_to(root)
        if not path.is_file() or rel.parts[0].startswith("native_") or "__pycache__" in rel.parts:
            continue
        if path.name != BINDING_NAME and path.suffix in (".py", ".json", ".cu", ".cuh"):
            names.append(rel.as_posix())
    return names


def write_source_binding(directory=None):
    """Write <directory>/SOURCE_BINDING.json = {complete, scope, files: {relative path: sha256}}, the
    receipt `sdacc/diffusion_research/library.py:11-15` (`bind`) checks before it imports a library
    directory.  Returns the receipt."""
    root = Path(directory) if directory is not None else _PACKAGE
    receipt = dict(complete=True, scope="source snapshot of the sm_100a library; build the native artefact locally "
                                        "with build_native(<directory>/native_sm80)",
                   files={name: sha(root / name) for name in source_binding_files(root)})
    (root / BINDING_NAME).write_text(json.dumps(receipt, indent=2) + "\n")
    return receipt


def _declare(lib):
    c = ctypes
    vp, i64, i32 = c.c_void_p, c.c_int64, c.c_int
    lib.ss_last_error.restype = c.c_char_p
    sigs = {
        "ss_query": [i32, vp, i32],
        "ss_lifted_k": [i64, i32, vp, vp],
        "ss_slide_weight_cpu": [vp, i64, i64, i32, vp],
        "ss_pack_cpu": [vp, i64, i64, i64, vp, vp, vp],
        "ss_meta_convert": [vp, vp, i64, i64, i32],
        "ss_weight_grid_device": [vp, i64, i64, vp, vp, vp],
        "ss_pack_device": [vp, i64, i64, i32, vp, vp, vp, vp],
        "ss_obs_block": [vp, i64, i64, i64, i64, vp, vp, i32, i32, vp, vp, vp, vp],
        "ss_obs_trailing": [vp, i64, i64, i64, i64, vp, vp, vp],
        "ss_obs_finish": [vp, vp, vp, i64, i64, i32, i32, vp, vp, vp],
        "ss_quantize_lift": [vp, i64, i64, i64, i32, vp, vp, vp],
        "ss_gemm_run": [vp, vp, vp, vp, vp, vp, vp, i64, vp, i64, i64, i64, i64, i64, i64, vp],
        "ss_gemm_int32": [vp, vp, vp, vp, i64, i64, i64, i64, i64, vp],
        "ss_projection": [vp, i64, i64, i64, i32, vp, vp, vp, vp, vp, i64, i64, i64, vp, vp, vp, i64, vp],
        "ss_quantize_lift_fused": [vp, i64, i64, i64, i32, i32, vp, vp, i64, i64, c.c_float, vp, vp, vp],
        "ss_projection_fused": [vp, i64, i64, i64, i32, i32, vp, vp, i64, i64, c.c_float,
                                vp, vp, vp, vp, vp, i64, vp, i64, i64, i64, vp, vp, vp, i64, vp],
        "ss_projection_peers": [vp, i64, i64, i64, i32, vp, vp, vp, vp, i64, i64, vp, vp, vp, i32, i64, vp],
        "ss_projection_static": [vp, i64, i64, i64, i32, vp, vp, vp, vp, i64, i64, vp, i64, vp],
        "ss_plan_create": [vp, vp, vp, vp, i64, i64, i64, i64, i32, vp],
        "ss_plan_run": [i64, vp, i64, vp, vp, vp, i64, vp],
        "ss_plan_release": [i64],
        "ss_plan_resources": [i64, vp, i32],
        "ss_gemm_resources": [i64, i64, i64, vp, i32],
        "ss_device_status": [vp, vp],
        "ss_micro_mma_rate": [i32, i32, i32, i32, vp],
        "ss_micro_pair_rate": [i64, i64, i64, i32, i32, vp, vp],
        "ss_micro_wait_limit": [i64, vp],
        "ss_set_option": [c.c_char_p, i64],
        "ss_get_option": [c.c_char_p, vp],
    }
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = args, i32
    lib.ss_obs_max_blocksize.argtypes, lib.ss_obs_max_blocksize.restype = [], i32
    return lib


def load_native(directory=None):
    """Load once (never touching CUDA) and register the operators.  Returns the receipt.

    Refuses a binary whose receipt does not match the sources next to this file, and refuses a
    second, different binary in the same process.
    """
    global _lib, _loaded_sha
    directory = Path(directory) if directory is not None else default_directory()
    receipt_path, target = directory / "receipt.json", directory / LIBRARY_NAME
    if not receipt_path.exists() or not target.exists():
        raise FileNotFoundError(f"no native library in {directory}: run build_native() first")
    receipt = json.loads(receipt_path.read_text())
    if not receipt.get("complete") or receipt.get("arch") != ARCH:
        raise ValueError("native receipt is incomplete or for another architecture")
    if receipt.get("source_dependencies") != _source_identity():
        raise ValueError("native source dependency identity differs; rebuild this release")
    if receipt.get("library_sha") != sha(target):
        raise ValueError("native binary differs from its receipt")
    if _lib is not None:
        if _loaded_sha != receipt["library_sha"]:
            raise RuntimeError("a different native binary is already loaded in this process")
        return receipt
    _lib = _declare(ctypes.CDLL(str(target)))
    _loaded_sha = receipt["library_sha"]
    _register_ops()
    return receipt


def library():
    """The loaded C-ABI library; loads the in-tree build on first use, raises if there is none."""
    if _lib is None:
        try:
            load_native()
        except (FileNotFoundError, ValueError) as e:
            raise RuntimeError(
                "the sm_100a native library is not built/loaded (no fallback exists): " + str(e)) from e
    return _lib


def check(rc):
    if rc == 0:
        return
    message = library().ss_last_error().decode(errors="replace")
    if rc in (SS_E_ARG, SS_E_FORMAT, SS_E_LIMIT):
        raise ValueError(message)
    raise RuntimeError(message)


# ------------------------------------------------------------------------------------------
# thin typed wrappers (device pointers in, nothing allocated behind the caller's back)

def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None and t.numel() else None


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


class _on_device:
    """`with torch.cuda.device(d)` that does nothing when d is already current (the common case:
    the switch costs several microseconds of host time per call)."""

    def __init__(self, device):
        self.guard = None if device.index == torch.cuda.current_device() else torch.cuda.device(device)

    def __enter__(self):
        if self.guard is not None:
            self.guard.__enter__()

    def __exit__(self, *exc):
        if self.guard is not None:
            self.guard.__exit__(*exc)


def _scratch(pm, pk, device):
    """Front-end output handed to the GEMM inside one projection call: q [pm, pk] and sa [pm] carved
    from ONE allocation (sa first: 4*pm is a multiple of 128 bytes, so q stays 16-byte aligned).
    Returns (owner tensor, q pointer, sa pointer)."""
    owner = torch.empty(4 * pm + pm * pk, dtype=torch.uint8, device=device)
    base = owner.data_ptr()
    return owner, ctypes.c_void_p(base + 4 * pm), ctypes.c_void_p(base)


def _check_config(config):
    if config not in VALID_CONFIGS:
        raise ValueError("invalid config")


def pack_weight(lifted, padded_k, layout="b200"):
    """CPU int8 [n,kl] -> (packed int8 [pn,pk/2], metadata int32 [pn*pk/32])."""
    if lifted.device.type != "cpu" or lifted.dtype != torch.int8 or lifted.ndim != 2 or not lifted.is_contiguous():
        raise ValueError("pack needs contiguous CPU int8 weight")
    n, kl = lifted.shape
    pk = int(padded_k)
    if not (n > 0 and kl > 0 and pk >= kl and pk % 128 == 0):
        raise ValueError("invalid128-K padding")
    pn = -(-n // 32) * 32
    packed = torch.empty((pn, pk // 2), dtype=torch.int8)
    metadata = torch.empty(pn * pk // 32, dtype=torch.int32)
    raw, hw = (_ptr(metadata), None) if layout == "raw" else (None, _ptr(metadata))
    check(library().ss_pack_cpu(_ptr(lifted), n, kl, pk, _ptr(packed), raw, hw))
    return packed, metadata


def convert_metadata(metadata, pn, pk, to_b200=True):
    src = metadata.detach().cpu().contiguous().view(torch.int32)
    dst = torch.empty_like(src)
    check(library().ss_meta_convert(_ptr(src), _ptr(dst), pn, pk, 1 if to_b200 else 0))
    return dst


def quantize_lift_into(flat, group, q, sa):
    m, k = flat.shape
    with torch.cuda.device(flat.device):
        check(library().ss_quantize_lift(_ptr(flat), flat.stride(0), m, k, group, _ptr(q), _ptr(sa),
                                         _stream(flat.device)))


def _flatten_input(x, k):
    flat = x.reshape(-1, k)
    if flat.stride(-1) != 1:
        flat = flat.contiguous()
    return flat


def _quantize(input, group):
    if not input.is_cuda or input.dtype != torch.bfloat16 or input.ndim < 1:
        raise ValueError("BF16 CUDA input required")
    group = group_size(int(group))
    k = input.shape[-1]
    flat = _flatten_input(input, k)
    m = flat.shape[0]
    if m <= 0:
        raise ValueError("empty input unsupported by native frontend")
    _, pk = lifted_k(k, group)
    pm = -(-m // 32) * 32
    q = torch.empty((pm, pk), dtype=torch.int8, device=input.device)
    sa = torch.empty(pm, dtype=torch.float32, device=input.device)
    quantize_lift_into(flat, group, q, sa)
    return q, sa


def _check_weights(q_device, packed, metadata, sw, bias, pk):
    for t in (packed, metadata, sw, bias):
        if t.device != q_device or not t.is_contiguous():
            raise ValueError("buffer device/layout mismatch")
    if packed.dtype != torch.int8 or packed.ndim != 2 or metadata.dtype != torch.int32:
        raise ValueError("packed types")
    if sw.dtype != torch.float32 or bias.dtype != torch.float32:
        raise ValueError("scale/bias must be FP32")
    if packed.shape[0] % 32 or packed.shape[1] * 2 != pk:
        raise ValueError("padding mismatch")
    if metadata.numel() != packed.shape[0] * pk // 32:
        raise ValueError("metadata/token scales size")


def _check_addend(addend, device, m, n):
    if addend is None:
        return None
    if (not addend.is_cuda or addend.device != device or addend.dtype != torch.bfloat16 or addend.ndim != 2
            or addend.shape != (m, n) or addend.stride(1) != 1):
        raise ValueError("addend must be BF16 [M,N] with unit column stride")
    return addend


def _run(q, packed, metadata, sa, sw, bias, m, n, config, output_addend=None):
    if not q.is_cuda or q.dtype != torch.int8 or q.ndim != 2 or not q.is_contiguous():
        raise ValueError("q must be row-major CUDA int8")
    pm, pk = q.shape
    if pk % 128 or pm % 32:
        raise ValueError("padding mismatch")
    _check_weights(q.device, packed, metadata, sw, bias, pk)
    if sa.dtype != torch.float32 or sa.numel() != pm or sa.device != q.device:
        raise ValueError("metadata/token scales size")
    pn = packed.shape[0]
    if not (0 < m <= pm and 0 < n <= pn and sw.numel() >= n and (bias.numel() == 0 or bias.numel() >= n)):
        raise ValueError("original dimensions/channels")
    _check_config(config)
    addend = _check_addend(output_addend, q.device, m, n)
    out = torch.empty((m, n), dtype=torch.bfloat16, device=q.device)
    with torch.cuda.device(q.device):
        check(library().ss_gemm_run(_ptr(q), _ptr(packed), _ptr(metadata), _ptr(sa), _ptr(sw), _ptr(bias),
                                    _ptr(addend), addend.stride(0) if addend is not None else 0,
                                    _ptr(out), n, m, n, pm, pn, pk, _stream(q.device)))
    return out


def gemm_int32(q, packed, metadata, m, n):
    """Raw INT32 accumulators [m,n] of the sparse contraction (debug / parity epilogue)."""
    pm, pk = q.shape
    out = torch.empty((m, n), dtype=torch.int32, device=q.device)
    with torch.cuda.device(q.device):
        check(library().ss_gemm_int32(_ptr(q), _ptr(packed), _ptr(metadata), _ptr(out), m, n, pm,
                                      packed.shape[0], pk, _stream(q.device)))
    return out


def _projection(input, packed, metadata, scales, bias, group, n, config, output_addend=None):
    if not input.is_cuda or input.dtype != torch.bfloat16 or input.ndim < 1:
        raise ValueError("BF16 CUDA input required")
    group = group_size(int(group))
    _check_config(config)
    k = input.shape[-1]
    flat = _flatten_input(input, k)
    m = flat.shape[0]
    if m <= 0:
        raise ValueError("empty input unsupported by native frontend")
    _, pk = lifted_k(k, group)
    pm = -(-m // 32) * 32
    _check_weights(input.device, packed, metadata, scales, bias, pk)
    pn = packed.shape[0]
    if not (0 < n <= pn and scales.numel() >= n and (bias.numel() == 0 or bias.numel() >= n)):
        raise ValueError("original dimensions/channels")
    addend = output_addend
    if addend is not None:
        addend = _check_addend(addend.reshape(-1, n), input.device, m, n)
    owner, q_ptr, sa_ptr = _scratch(pm, pk, input.device)
    out = torch.empty((*input.shape[:-1], n), dtype=torch.bfloat16, device=input.device)
    with _on_device(input.device):
        check(library().ss_projection(_ptr(flat), flat.stride(0), m, k, group, _ptr(packed), _ptr(metadata),
                                      _ptr(scales), _ptr(bias), _ptr(addend),
                                      addend.stride(0) if addend is not None else 0, n, pn,
                                      q_ptr, sa_ptr, _ptr(out), n, _stream(input.device)))
    return out


def projection_peers(input, packed, metadata, scales, bias, group, n, destinations, out_stride):
    """Projection of this rank's column shard stored straight into every rank's gathered output.

    destinations: device addresses (ints), one per rank, of element [0, first column of this shard]
    of that rank's [m, N] BF16 buffer as mapped into this process; out_stride: its row pitch."""
    if not input.is_cuda or input.dtype != torch.bfloat16 or input.ndim != 2:
        raise ValueError("BF16 CUDA [m, k] input required")
    group = group_size(int(group))
    flat = _flatten_input(input, input.shape[-1])
    m, k = flat.shape
    _, pk = lifted_k(k, group)
    pm = -(-m // 32) * 32
    _check_weights(input.device, packed, metadata, scales, bias, pk)
    q = torch.empty((pm, pk), dtype=torch.int8, device=input.device)
    sa = torch.empty(pm, dtype=torch.float32, device=input.device)
    pointers = (ctypes.c_void_p * len(destinations))(*[int(p) for p in destinations])
    with torch.cuda.device(input.device):
        check(library().ss_projection_peers(_ptr(flat), flat.stride(0), m, k, group, _ptr(packed), _ptr(metadata),
                                            _ptr(scales), _ptr(bias), n, packed.shape[0], _ptr(q), _ptr(sa),
                                            pointers, len(destinations), int(out_stride), _stream(input.device)))


def micro_mma_rate(token_tile, sparse=True, with_metadata_copy=False, iterations=512):
    """Cycles per back-to-back 128 x token_tile INT8 tcgen05.mma of one CTA (diagnostic)."""
    value = ctypes.c_double()
    check(library().ss_micro_mma_rate(int(token_tile), int(bool(sparse)), int(bool(with_metadata_copy)),
                                      int(iterations), ctypes.byref(value)))
    return value.value


def micro_pair_rate(m, n, pk, token_tile=0, no_mma=False, no_epilogue=False, no_stores=False, loads_only=False):
    """(cycles per 256-column pipeline stage, stages) of cluster 0 of the real GEMM kernel on scratch
    operands of this size, optionally without its MMAs and / or its epilogue work (diagnostic)."""
    cycles, stages = ctypes.c_double(), ctypes.c_int64()
    check(library().ss_micro_pair_rate(int(m), int(n), int(pk), int(token_tile), int(bool(no_mma)) | 2 * int(bool(no_epilogue)) | 4 * int(bool(no_stores)) | 8 * int(bool(loads_only)),
                                       ctypes.byref(cycles), ctypes.byref(stages)))
    return cycles.value, stages.value


def micro_wait_limit(limit_ns):
    """Nanoseconds a kernel really waited on a barrier nobody signals before its bounded wait gave
    up; leaves the wait-limit bit in the device status word (diagnostic)."""
    elapsed = ctypes.c_int64()
    check(library().ss_micro_wait_limit(int(limit_ns), ctypes.byref(elapsed)))
    return elapsed.value


def set_option(name, value):
    """Change a tuning switch of the native library (see ss_set_option); returns the previous value."""
    previous = get_option(name)
    check(library().ss_set_option(name.encode(), int(value)))
    return previous


def get_option(name):
    value = ctypes.c_int64()
    check(library().ss_get_option(name.encode(), ctypes.byref(value)))
    return value.value


PROLOGUES = {"none": 0, "norm_modulate": 1, "gelu": 2}


class Prologue:
    """Element-wise neighbour fused into the front-end (an extension; the reference has none).

    Prologue.norm_modulate(shift, scale, eps): LayerNorm without affine over the last dimension,
    then x * (1 + scale[b]) + shift[b]; shift / scale are BF16 [batch, k] for an input [batch, rows, k].
    Prologue.gelu(): tanh-approximated GELU."""

    def __init__(self, kind, shift=None, scale=None, eps=1e-6):
        if kind not in PROLOGUES:
            raise ValueError("unknown prologue")
        self.kind, self.shift, self.scale, self.eps = kind, shift, scale, float(eps)

    @classmethod
    def norm_modulate(cls, shift, scale, eps=1e-6):
        return cls("norm_modulate", shift, scale, eps)

    @classmethod
    def gelu(cls):
        return cls("gelu")

    def torch_reference(self, x):
        """The same neighbour as separate PyTorch operators (what a dense path runs)."""
        if self.kind == "gelu":
            return torch.nn.functional.gelu(x, approximate="tanh")
        if self.kind == "norm_modulate":
            xn = torch.nn.functional.layer_norm(x, x.shape[-1:], eps=self.eps)
            return torch.addcmul(self.shift[:, None], xn, 1 + self.scale[:, None])
        return x

    def arguments(self, x, k):
        """(code, shift, scale, row stride of shift/scale, rows_per_batch, eps) for the C entry."""
        if self.kind != "norm_modulate":
            return PROLOGUES[self.kind], None, None, 0, (x.shape[1] if x.ndim == 3 else 1), 0.0
        if x.ndim != 3:
            raise ValueError("norm_modulate needs [batch, rows, k] input")
        batch, rows = x.shape[0], x.shape[1]
        shift, scale = self.shift, self.scale
        for t in (shift, scale):
            if t is None or t.dtype != torch.bfloat16 or t.device != x.device or tuple(t.shape) != (batch, k):
                raise ValueError("shift / scale must be BF16 [batch, k] on the input's device")
        usable = all(t.stride(1) == 1 and t.data_ptr() % 16 == 0 and t.stride(0) % 8 == 0 and t.stride(0) >= k
                     for t in (shift, scale)) and (batch == 1 or shift.stride(0) == scale.stride(0))
        if not usable:
            shift, scale = shift.contiguous(), scale.contiguous()
        return 1, shift, scale, (shift.stride(0) if batch > 1 else k), rows, self.eps


def _fused_frontend_args(input, prologue):
    k = input.shape[-1]
    code, shift, scale, mod_stride, rows, eps = prologue.arguments(input, k)
    flat = _flatten_input(input, k)
    if code and (flat.data_ptr() % 16 or flat.stride(0) % 8 or k % 8):
        flat = flat.contiguous()
        if flat.data_ptr() % 16 or k % 8:
            raise ValueError("a prologue needs k % 8 == 0")
    return flat, code, shift, scale, mod_stride, rows, eps


def quantize_lift_fused(input, group, prologue):
    """Front-end with a prologue: (q int8 [pm,pk], scales fp32 [pm])."""
    if not input.is_cuda or input.dtype != torch.bfloat16:
        raise ValueError("BF16 CUDA input required")
    group = group_size(int(group))
    flat, code, shift, scale, mod_stride, rows, eps = _fused_frontend_args(input, prologue)
    m, k = flat.shape
    _, pk = lifted_k(k, group)
    pm = -(-m // 32) * 32
    q = torch.empty((pm, pk), dtype=torch.int8, device=input.device)
    sa = torch.empty(pm, dtype=torch.float32, device=input.device)
    with torch.cuda.device(input.device):
        check(library().ss_quantize_lift_fused(_ptr(flat), flat.stride(0), m, k, group, code, _ptr(shift), _ptr(scale),
                                               mod_stride, rows, eps, _ptr(q), _ptr(sa), _stream(input.device)))
    return q, sa


def projection_fused(input, prologue, packed, metadata, scales, bias, group, n, output_addend=None,
                     gate=None, residual=None):
    """`projection` with the prologue applied to the input inside the front-end kernel.

    With `gate` (BF16 [batch, n]) and `residual` (BF16 [batch, rows, n], contiguous) the result is
    accumulated in place: residual += bf16(gate[b] * y), and `residual` is returned.

    Goes through the `slidesparse_b200::projection_fused` / `::projection_fused_accumulate_`
    operators (registered with fake kernels), so a model that uses fused neighbours still traces
    under `torch.compile(fullgraph=True)`."""
    ops = torch.ops.slidesparse_b200
    code = PROLOGUES[prologue.kind]
    if gate is not None:
        if residual is None or output_addend is not None:
            raise ValueError("gated accumulation needs [batch, rows, k] input, a residual and no addend")
        ops.projection_fused_accumulate_(residual, input, code, prologue.shift, prologue.scale, prologue.eps,
                                         packed, metadata, scales, bias, int(group), int(n), gate)
        return residual
    return ops.projection_fused(input, code, prologue.shift, prologue.scale, prologue.eps, packed, metadata, scales,
                                bias, int(group), int(n), output_addend)


def _projection_fused_impl(input, prologue, packed, metadata, scales, bias, group, n, output_addend=None,
                           gate=None, residual=None):
    """The ctypes call behind the fused-projection operators."""
    if not input.is_cuda or input.dtype != torch.bfloat16 or input.ndim < 1:
        raise ValueError("BF16 CUDA input required")
    group = group_size(int(group))
    flat, code, shift, scale, mod_stride, rows, eps = _fused_frontend_args(input, prologue)
    m, k = flat.shape
    if m <= 0:
        raise ValueError("empty input unsupported by native frontend")
    _, pk = lifted_k(k, group)
    pm = -(-m // 32) * 32
    _check_weights(input.device, packed, metadata, scales, bias, pk)
    pn = packed.shape[0]
    if not (0 < n <= pn and scales.numel() >= n and (bias.numel() == 0 or bias.numel() >= n)):
        raise ValueError("original dimensions/channels")
    addend = output_addend
    if addend is not None:
        addend = _check_addend(addend.reshape(-1, n), input.device, m, n)
    gate_stride = 0
    if gate is not None:
        if addend is not None or residual is None or input.ndim != 3:
            raise ValueError("gated accumulation needs [batch, rows, k] input, a residual and no addend")
        batch, rows = input.shape[0], input.shape[1]
        if (residual.dtype != torch.bfloat16 or residual.device != input.device or not residual.is_contiguous()
                or tuple(residual.shape) != (batch, rows, n) or residual.data_ptr() % 16 or n % 8):
            raise ValueError("residual must be contiguous, 16-byte aligned BF16 [batch, rows, n] with n % 8 == 0")
        if gate.dtype != torch.bfloat16 or gate.device != input.device or tuple(gate.shape) != (batch, n) or gate.stride(1) != 1:
            raise ValueError("gate must be BF16 [batch, n] with unit column stride")
        if rows % 32:
            raise ValueError("gated accumulation needs rows per batch to be a multiple of 32")
        gate_stride = gate.stride(0) if batch > 1 else n
        out = residual
    else:
        out = torch.empty((*input.shape[:-1], n), dtype=torch.bfloat16, device=input.device)
    owner, q_ptr, sa_ptr = _scratch(pm, pk, input.device)
    with _on_device(input.device):
        check(library().ss_projection_fused(_ptr(flat), flat.stride(0), m, k, group, code, _ptr(shift), _ptr(scale),
                                            mod_stride, rows, eps, _ptr(packed), _ptr(metadata), _ptr(scales), _ptr(bias),
                                            _ptr(addend), addend.stride(0) if addend is not None else 0,
                                            _ptr(gate), gate_stride, n, pn,
                                            q_ptr, sa_ptr, _ptr(out), n, _stream(input.device)))
    return out


def _configure(anchor, config, has_addend=False):
    if not anchor.is_cuda:
        raise ValueError("CUDA anchor required")
    _check_config(config)
    info = (ctypes.c_int64 * 8)()
    with torch.cuda.device(anchor.device):
        check(library().ss_query(anchor.device.index, info, 8))
        if info[2] != 10:
            raise RuntimeError("this library is built for sm_100a (B200) only")
        pn, half = anchor.shape
        res = (ctypes.c_int64 * 8)()
        check(library().ss_gemm_resources(4096, pn, 2 * half, res, 8))
    base = [int(v) for v in res[:5]]
    return base + base


_plan_devices = {}


def _prepare(packed, metadata, scales, bias, k, m, n, group, config, packed16):
    if not packed.is_cuda or m <= 0 or n <= 0:
        raise ValueError("prepared graph geometry")
    group = group_size(int(group))
    _check_config(config)
    _, pk = lifted_k(k, group)
    _check_weights(packed.device, packed, metadata, scales, bias, pk)
    pn = packed.shape[0]
    if not (pn >= n and scales.numel() >= n and (bias.numel() == 0 or bias.numel() >= n)):
        raise ValueError("prepared packing")
    handle = ctypes.c_int64(0)
    with torch.cuda.device(packed.device):
        check(library().ss_plan_create(_ptr(packed), _ptr(metadata), _ptr(scales), _ptr(bias), k, m, n, pn,
                                       group, ctypes.byref(handle)))
    _plan_devices[handle.value] = (packed.device, m, k, n, pk)
    return handle.value


def _prepared_run(input, handle, n):
    if handle not in _plan_devices:
        raise RuntimeError("prepared graph handle absent")
    device, m, k, plan_n, pk = _plan_devices[handle]
    if (not input.is_cuda or input.device != device or input.dtype != torch.bfloat16
            or input.shape[-1] != k):
        raise ValueError("prepared input identity")
    if input.numel() != m * k or n != plan_n:
        raise ValueError("prepared shape changed")
    flat = _flatten_input(input, k)
    out = torch.empty((*input.shape[:-1], n), dtype=torch.bfloat16, device=device)
    stream = torch.cuda.current_stream(device)
    q = sa = None
    lib = library()
    with torch.cuda.device(device):
        rc = lib.ss_plan_run(handle, _ptr(flat), flat.stride(0), None, None, _ptr(out), n,
                             ctypes.c_void_p(stream.cuda_stream))
        if rc == SS_E_ARG and b"caller scratch" in lib.ss_last_error():
            # another stream, or an outer graph capture: independent scratch from torch's allocator
            pm = -(-m // 32) * 32
            q = torch.empty((pm, pk), dtype=torch.int8, device=device)
            sa = torch.empty(pm, dtype=torch.float32, device=device)
            rc = lib.ss_plan_run(handle, _ptr(flat), flat.stride(0), _ptr(q), _ptr(sa), _ptr(out), n,
                                 ctypes.c_void_p(stream.cuda_stream))
        check(rc)
    return out


def _release(handle):
    _plan_devices.pop(handle, None)
    check(library().ss_plan_release(handle))


def _resources(handle):
    res = (ctypes.c_int64 * 8)()
    device = _plan_devices[handle][0]
    with torch.cuda.device(device):
        check(library().ss_plan_resources(handle, res, 8))
    return [int(v) for v in res[:5]]


def device_status(device=None):
    """Synchronise the current stream and return (and clear) the device's kernel status word:
    0, or the bits of the bounded waits that ran out since the last call."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    status = ctypes.c_int32(0)
    with torch.cuda.device(device):
        rc = library().ss_device_status(_stream(device), ctypes.byref(status))
    if rc != SS_E_DEVICE:
        check(rc)
    return status.value


def check_device(device=None):
    """Raise RuntimeError if a kernel gave up on a bounded wait since the last check."""
    status = device_status(device)
    if status:
        raise RuntimeError(f"a kernel gave up on a bounded wait (device status 0x{status:x})")


# ------------------------------------------------------------------------------------------
# torch operator registration under the reference's names

_libraries = []


def _register_ops():
    global _ops_registered
    if _ops_registered:
        return
    _ops_registered = True
    Library = torch.library.Library

    dual = Library("sdacc_dualscale_sm80", "DEF")
    dual.define("pack_cpu(Tensor weight,int padded_k)->(Tensor,Tensor)")
    dual.define("configure(Tensor anchor,int config,bool has_addend=False)->int[]")
    dual.define("run(Tensor q,Tensor packed,Tensor metadata,Tensor sa,Tensor sw,Tensor bias,int m,int n,"
                "int config,Tensor? output_addend=None)->Tensor")
    dual.impl("pack_cpu", lambda weight, padded_k: pack_weight(weight, padded_k), "CPU")
    dual.impl("configure", _configure, "CUDA")
    dual.impl("run", _run, "CUDA")

    mild = Library("sdacc_mild_projection_sm80", "DEF")
    proj = ("(Tensor input,Tensor packed,Tensor metadata,Tensor scales,Tensor bias,int group,int n,int config,"
            "Tensor? output_addend=None)->Tensor")
    mild.define("quantize_packed16(Tensor input,int group)->(Tensor,Tensor)")
    mild.define("projection_packed16" + proj)
    mild.define("quantize(Tensor input,int group)->(Tensor,Tensor)")
    mild.define("quantize_scalar(Tensor input)->(Tensor,Tensor)")
    mild.define("projection" + proj)
    mild.define("projection_scalar" + proj)
    # One front-end serves all three reference variants: they produce identical bits.
    mild.impl("quantize", _quantize, "CUDA")
    mild.impl("quantize_packed16", _quantize, "CUDA")
    mild.impl("quantize_scalar", lambda input: _quantize(input, 4), "CUDA")
    for name in ("projection", "projection_packed16", "projection_scalar"):
        mild.impl(name, _projection, "CUDA")

    prepared = Library("sdacc_prepared_projection_sm80", "DEF")
    prep = ("(Tensor packed,Tensor metadata,Tensor scales,Tensor bias,int k,int m,int n,int group,int config,"
            "bool packed16)->int")
    for name in ("prepare_direct2", "prepare_singlepatch", "prepare"):
        prepared.define(name + prep)
        prepared.impl(name, _prepare, "CUDA")
    prepared.define("resources(int handle)->int[]")
    prepared.define("run(Tensor input,int handle,int n)->Tensor")
    prepared.define("release(int handle)->()")
    prepared.impl("run", _prepared_run, "CUDA")
    prepared.impl("release", _release, "CompositeExplicitAutograd")
    prepared.impl("resources", _resources, "CompositeExplicitAutograd")
    _libraries.extend([dual, mild, prepared])

    @torch.library.register_fake("sdacc_dualscale_sm80::run")
    def _fake_run(q, packed, metadata, sa, sw, bias, m, n, config, output_addend=None):
        return q.new_empty((m, n), dtype=torch.bfloat16)

    def _fake_projection(x, packed, metadata, scales, bias, group, n, config, output_addend=None):
        return x.new_empty((*x.shape[:-1], n))

    for name in ("projection", "projection_scalar", "projection_packed16"):
        torch.library.register_fake("sdacc_mild_projection_sm80::" + name)(_fake_projection)

    @torch.library.register_fake("sdacc_prepared_projection_sm80::run")
    def _fake_prepared(x, handle, n):
        return x.new_empty((*x.shape[:-1], n))

    # additions of this library (no counterpart in the reference): the projection with element-wise
    # neighbours fused in, as operators so that callers using them can still be compiled
    own = Library("slidesparse_b200", "DEF")
    weights = "Tensor packed,Tensor metadata,Tensor scales,Tensor bias,int group,int n"
    pro = "int prologue,Tensor? shift,Tensor? scale,float eps"
    own.define(f"projection_fused(Tensor input,{pro},{weights},Tensor? output_addend=None)->Tensor")
    own.define(f"projection_fused_accumulate_(Tensor(a!) residual,Tensor input,{pro},{weights},Tensor gate)->()")

    def _prologue_of(code, shift, scale, eps):
        kind = {v: k for k, v in PROLOGUES.items()}[int(code)]
        return Prologue(kind, shift, scale, eps)

    def _op_fused(input, prologue, shift, scale, eps, packed, metadata, scales, bias, group, n, output_addend=None):
        return _projection_fused_impl(input, _prologue_of(prologue, shift, scale, eps), packed, metadata, scales, bias,
                                      group, n, output_addend)

    def _op_fused_accumulate(residual, input, prologue, shift, scale, eps, packed, metadata, scales, bias, group, n, gate):
        _projection_fused_impl(input, _prologue_of(prologue, shift, scale, eps), packed, metadata, scales, bias, group, n,
                               None, gate, residual)

    own.impl("projection_fused", _op_fused, "CUDA")
    own.impl("projection_fused_accumulate_", _op_fused_accumulate, "CUDA")
    _libraries.append(own)

    @torch.library.register_fake("slidesparse_b200::projection_fused")
    def _fake_fused(input, prologue, shift, scale, eps, packed, metadata, scales, bias, group, n, output_addend=None):
        return input.new_empty((*input.shape[:-1], n))

    @torch.library.register_fake("slidesparse_b200::projection_fused_accumulate_")
    def _fake_fused_accumulate(residual, input, prologue, shift, scale, eps, packed, metadata, scales, bias, group, n, gate):
        return None
