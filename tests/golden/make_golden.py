"""Generate golden vectors by running the reference's own CPU code.

Run where the reference tree is mounted and oracle/_ref has been built (oracle/build_ref.py):

    python tests/golden/make_golden.py [--reference /path/to/SlideSparse-Diffusion]

Imports only the reference (never this repository's package: both register the same torch
operator namespace, so they cannot share a process) and writes small .npz fixtures next to this
file.  Inputs are seeded numpy draws stored in the fixtures together with the outputs:

  slide_pack.npz   slide_weight (packing.py:23-52), pack_cpu (csrc/dualscale_sm80.cu:254-280,
                   built as oracle/_ref/dualscale_sm80.so), lifted_k (packing.py:15-20)
  lift.npz         activation_indices / lift_integer
                   (diffusion_research/integrations/cachequant/native_sparse.py:11-23)
  weight_grid.npz  channel_scales / round_signed (diffusion_research/reconstruction.py:41-53)
  reconstruction.npz  factor_hessian and compress (diffusion_research/reconstruction.py:18-39,
                   55-133) on CPU: single-block cases (bit-reproducible) and multi-block cases
                   (the trailing update goes through the BLAS the reference was run with)
"""
import argparse
import os
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent


def load_file(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


RECONSTRUCTION_CASES = (
    # rows, columns, group, blocksize, method, allow_tail, dead columns, explicit scales
    (12, 48, 4, 192, "joint", False, (), False),
    (10, 48, 6, 192, "joint", False, (7, 30), False),
    (9, 64, 8, 192, "prune_then_rtn", False, (), False),
    (8, 44, 8, 192, "joint", True, (), False),
    (7, 47, 6, 192, "joint", True, (), True),
    (16, 96, 6, 24, "joint", False, (50,), False),
    (8, 64, 4, 16, "joint", False, (), True),
    (8, 79, 8, 32, "prune_then_rtn", True, (), False),
)


def reconstruction_fixture(ref):
    recon = load_file("ref_reconstruction", ref / "sdacc/diffusion_research/reconstruction.py")
    rng = np.random.default_rng(20260)
    out = {"cases": np.array([(r, c, g, b, m == "joint", t, e) for r, c, g, b, m, t, _, e in RECONSTRUCTION_CASES],
                             dtype=np.int64)}
    for i, (rows, columns, group, blocksize, method, allow_tail, dead, explicit) in enumerate(RECONSTRUCTION_CASES):
        x = rng.normal(0, 1, size=(256, columns)).astype(np.float32)
        x[:, rng.permutation(columns)[:2]] *= 8
        x[:, list(dead)] = 0
        hessian = torch.from_numpy(x.T @ x / 256)
        hessian = (hessian + hessian.T) / 2
        weight = torch.from_numpy(rng.normal(0, 0.02, size=(rows, columns)).astype(np.float32))
        curvature = recon.factor_hessian(hessian, damping=.01)
        scales = torch.from_numpy(rng.uniform(2e-4, 6e-4, size=rows).astype(np.float32)) if explicit else None
        result = recon.compress(weight, curvature, group, method=method, blocksize=blocksize, scales=scales,
                                allow_tail=allow_tail)
        out[f"weight{i}"] = weight.numpy()
        out[f"hessian{i}"] = hessian.numpy()
        out[f"upper{i}"] = curvature.upper.numpy()
        out[f"dead{i}"] = curvature.dead.numpy()
        out[f"damping{i}"] = np.float64(curvature.damping)
        out[f"scales_in{i}"] = scales.numpy() if explicit else np.zeros(0, np.float32)
        for key in ("qweight", "scales", "zeros", "compensated", "proxy_loss"):
            out[f"{key}{i}"] = result[key].numpy()
    np.savez_compressed(HERE / "reconstruction.npz", **out)


def structured_weight(rng, n, k, l, density=0.9):
    """Random int8 [n,k] with at most l-2 nonzeros per aligned group of l (tail lanes count)."""
    w = rng.integers(-128, 128, size=(n, k), dtype=np.int64)
    w[rng.random((n, k)) > density] = 0          # extra zeros: "quantised to zero" weights
    groups = -(-k // l)
    for r in range(n):
        for g in range(groups):
            lanes = np.arange(g * l, min(k, (g + 1) * l))
            missing = l - len(lanes)
            remove = max(0, 2 - missing)
            drop = rng.choice(lanes, size=min(remove, len(lanes)), replace=False)
            w[r, drop] = 0
    return w.astype(np.int8)


def main():
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--reference", default=os.environ.get("SS_REFERENCE"), required=not os.environ.get("SS_REFERENCE"),
                        help="root of the SlideSparse-Diffusion source tree (or set SS_REFERENCE)")
    args = parser.parse_args()
    ref = Path(args.reference)
    packing = load_file("ref_packing", ref / "sdacc/w8a8_slidesparse/packing.py")
    native_sparse = load_file("ref_native_sparse",
                              ref / "sdacc/diffusion_research/integrations/cachequant/native_sparse.py")
    torch.ops.load_library(str(ROOT / "oracle/_ref/dualscale_sm80.so"))
    pack_cpu = torch.ops.sdacc_dualscale_sm80.pack_cpu

    rng = np.random.default_rng(20261125)
    out = {}
    cases = [(4, 40, 128), (4, 33, 260), (6, 32, 132), (6, 50, 38), (6, 96, 300), (8, 64, 128),
             (8, 40, 44), (8, 70, 200), (6, 35, 1152 // 4), (8, 32, 2432 // 8 + 3)]
    out["cases"] = np.array(cases, dtype=np.int64)
    for i, (l, n, k) in enumerate(cases):
        w = structured_weight(rng, n, k, l)
        lifted = packing.slide_weight(torch.from_numpy(w), l)
        valid, pk = packing.lifted_k(k, l)
        packed, metadata = pack_cpu(lifted, pk)
        out[f"w{i}"] = w
        out[f"lifted{i}"] = lifted.numpy()
        out[f"packed{i}"] = packed.numpy()
        out[f"meta_sm80_{i}"] = metadata.numpy()
        out[f"dims{i}"] = np.array([valid, pk], dtype=np.int64)
    # hand-readable window vectors (one group per row)
    small46 = np.array([[1, 0, 2, 3, 0, 4], [0, 5, 6, 0, 7, 8], [9, 10, 11, 12, 0, 0], [0, 0, 0, 0, 1, 2]], np.int8)
    small68 = np.array([[1, 2, 3, 4, 5, 6, 0, 0], [0, 0, 1, 2, 3, 4, 5, 6], [1, 0, 2, 0, 3, 4, 5, 6],
                        [1, 2, 0, 3, 4, 0, 5, 6]], np.int8)
    tail46 = np.array([[1, 2, 3, 4, 0, 0, 5]], np.int8)
    out["small46"], out["small46_lifted"] = small46, packing.slide_weight(torch.from_numpy(small46), "4:6").numpy()
    out["small68"], out["small68_lifted"] = small68, packing.slide_weight(torch.from_numpy(small68), "6:8").numpy()
    out["tail46"], out["tail46_lifted"] = tail46, packing.slide_weight(torch.from_numpy(tail46), "4:6").numpy()
    pack_in = np.array([[1, 0, 0, 2, 0, 3, 4, 0], [0, 0, 5, 0, 6, 0, 0, 0]], np.int8)
    p, m = pack_cpu(torch.from_numpy(pack_in), 128)
    out["pack_in"], out["pack_in_packed"], out["pack_in_meta_sm80"] = pack_in, p.numpy(), m.numpy()
    try:
        packing.slide_weight(torch.tensor([[1, 2, 3, 4, 5, 0]], dtype=torch.int8), "4:6")
        out["overfull_raises"] = np.array(0)
    except ValueError:
        out["overfull_raises"] = np.array(1)
    np.savez_compressed(HERE / "slide_pack.npz", **out)

    lift = {}
    pairs = [(4, 40), (6, 36), (8, 40), (6, 38), (8, 44), (6, 1152), (8, 2432), (6, 2432)]
    lift["pairs"] = np.array(pairs, dtype=np.int64)
    for i, (l, k) in enumerate(pairs):
        idx = native_sparse.activation_indices(k, l)
        lift[f"idx{i}"] = idx.numpy()
        if k <= 64:
            a = torch.from_numpy(rng.integers(-128, 128, size=(5, k), dtype=np.int64).astype(np.int8))
            lift[f"a{i}"] = a.numpy()
            lift[f"lifted{i}"] = native_sparse.lift_integer(a, idx).numpy()
    np.savez_compressed(HERE / "lift.npz", **lift)

    recon = load_file("ref_reconstruction", ref / "sdacc/diffusion_research/reconstruction.py")
    w = torch.from_numpy(rng.normal(0, 0.02, size=(12, 40)).astype(np.float32))
    w[3] = 0
    scales = recon.channel_scales(w)
    q = recon.round_signed(w, scales[:, None])
    np.savez_compressed(HERE / "weight_grid.npz", w=w.numpy(), scales=scales.numpy(), q=q.numpy().astype(np.int8))
    reconstruction_fixture(ref)
    print("wrote", [p.name for p in sorted(HERE.glob("*.npz"))])


if __name__ == "__main__":
    sys.exit(main())
