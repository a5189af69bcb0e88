"""Shape inventory of the routed projections and convenience constructors.

Mirror of `sdacc/w8a8_slidesparse/workloads/__init__.py:8-23` (`prepare_for`) and of the shape
groups in its `inventory.json`.  The reference freezes 44 shape groups in JSON together with
SM80 dispatch choices; here every group is derived from the model dimensions below (the
dispatch choices have no meaning on sm_100a), and every (workload, module) of the reference's
alias list resolves to the same (M, K, N, members, recipe).
"""
from ..composite import ProtectedFFNOutput, SharedProjection
from ..packing import group_size
from ..profile import selectable
from ..runtime import PackedLinear

# hidden width, MLP width, image tokens (CFG batch included), text tokens, family
MODELS = {
    "dit256":          dict(hidden=1152, mlp=4608, image_m=512, text_m=None, family="dit"),
    "pixart_alpha256": dict(hidden=1152, mlp=4608, image_m=512, text_m=240, family="pixart"),
    "pixart_alpha512": dict(hidden=1152, mlp=4608, image_m=2048, text_m=240, family="pixart"),
    "pixart_sigma512": dict(hidden=1152, mlp=4608, image_m=2048, text_m=600, family="pixart"),
    "flux512":         dict(hidden=3072, mlp=12288, image_m=1024, text_m=512, family="flux"),
    "flux1024":        dict(hidden=3072, mlp=12288, image_m=4096, text_m=512, family="flux"),
    "sd3_medium512":   dict(hidden=1536, mlp=6144, image_m=2048, text_m=666, family="mmdit"),
    "sd35_large512":   dict(hidden=2432, mlp=9728, image_m=2048, text_m=666, family="mmdit"),
    "glm512":          dict(hidden=4096, mlp=16384, image_m=1024, text_m=512, family="glm"),
    # configurations named by the benchmark that the reference inventory does not list
    "dit512":          dict(hidden=1152, mlp=4608, image_m=2048, text_m=None, family="dit"),
    "pixart_sigma1024": dict(hidden=1152, mlp=4608, image_m=8192, text_m=600, family="pixart"),
}


def _group(m, k, n, members=None, recipe="ordinary", row_stride=None, slice_start=0):
    return dict(m=m, k=k, n=n, members=list(members or [n]), recipe=recipe,
                row_stride=row_stride or k, slice_start=slice_start)


def shapes(workload):
    """{module name: dict(m, k, n, members, recipe, row_stride, slice_start)} for a workload."""
    spec = MODELS[workload]
    h, f, im, tm, family = spec["hidden"], spec["mlp"], spec["image_m"], spec["text_m"], spec["family"]
    out = {}

    def stream(prefix, m):
        out[prefix + ".QKV"] = _group(m, h, 3 * h, [h, h, h])
        out[prefix + ".FFN-in"] = _group(m, h, f)
        out[prefix + ".FFN-out"] = _group(m, f, h)

    if family == "dit":
        stream("image", im)
    elif family == "pixart":
        stream("image", im)
        out["image.cross-Q"] = _group(im, h, h)
        out["text.cross-KV"] = _group(tm, h, 2 * h, [h, h])
    elif family == "mmdit":
        stream("image", im)
        stream("text", tm)
    elif family == "flux":
        stream("image", im)
        stream("text", tm)
        joint = im + tm
        out["single.QKV"] = _group(joint, h, 3 * h, [h, h, h])
        out["single.FFN-in"] = _group(joint, h, f)
        out["single.QKV+FFN-in"] = _group(joint, h, 3 * h + f, [h, h, h, f], recipe="shared_qkv_ffn")
        out["single.mixed-FFN-out"] = _group(joint, f, h, recipe="protected_ffn", row_stride=h + f,
                                             slice_start=h)
    elif family == "glm":
        out["joint.QKV"] = _group(im + tm, h, 3 * h, [h, h, h])
        out["image.FFN-in"] = _group(im, h, f)
        out["image.FFN-out"] = _group(im, f, h)
        out["text.FFN-in"] = _group(tm, h, f)
        out["text.FFN-out"] = _group(tm, f, h)
    return out


def all_shapes():
    """Unique (m, k, n) triples over every workload, sorted."""
    return sorted({(g["m"], g["k"], g["n"]) for w in MODELS for g in shapes(w).values()})


def prepare_for(workload, module, qweight, scales, bias=None, mode="2:4", attention_weight=None,
                execution="default"):
    """PackedLinear / SharedProjection / ProtectedFFNOutput for one routed module of a workload."""
    if workload not in MODELS:
        raise StopIteration(f"unknown workload {workload!r}")
    table = shapes(workload)
    if module not in table:
        raise StopIteration(f"workload {workload!r} has no module {module!r}")
    group = table[module]
    length = group_size(mode)
    if execution not in ("default", "recommended"):
        raise ValueError("unknown execution recipe")
    # the reference refuses groups whose measured sparse projection did not beat dense
    # (`workloads/__init__.py:17`); here the rule is profile.selectable, from this GPU's measurements
    if not selectable(length, group["m"], group["k"], group["n"]):
        raise ValueError(f"{workload}/{module} ({group['m']}x{group['k']}->{group['n']}) is not faster than the dense "
                         "projection on this GPU; keep Dense")
    if tuple(qweight.shape) != (group["n"], group["k"]):
        raise ValueError("weight shape differs from frozen workload")
    packed = PackedLinear.prepare(qweight, scales, bias, length)
    if group["recipe"] == "protected_ffn":
        if attention_weight is None:
            raise ValueError("BF16 protected attention weight required")
        return ProtectedFFNOutput(packed, attention_weight)
    return SharedProjection(packed, group["members"]) if len(group["members"]) > 1 else packed


def _workload_module(name):
    """`workloads.<name>` with WORKLOAD and prepare(module, qweight, scales, ...) bound to it, the
    per-workload entry the reference keeps as one sub-package each
    (`sdacc/w8a8_slidesparse/workloads/<name>/__init__.py`); created here from the MODELS table."""
    import sys
    import types
    module = types.ModuleType(f"{__name__}.{name}", f"Constructors for the routed projections of the '{name}' workload.")

    def prepare(module_name, qweight, scales, bias=None, mode="2:4", attention_weight=None, execution="default"):
        return prepare_for(name, module_name, qweight, scales, bias, mode, attention_weight, execution)

    module.WORKLOAD, module.prepare, module.shapes = name, prepare, (lambda: shapes(name))
    sys.modules[module.__name__] = module
    return module


for _name in MODELS:
    globals()[_name] = _workload_module(_name)
del _name
