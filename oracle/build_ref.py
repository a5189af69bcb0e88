"""Compile the reference's own CPU packer (pack_cpu) from where its source lies.

TEST INFRASTRUCTURE ONLY.  Nothing here is imported by the product.

The reference keeps `pack_cpu` (2:4 compression + metadata + CUTLASS `reorder_meta`) inside
`sdacc/w8a8_slidesparse/csrc/dualscale_sm80.cu` (:254-280).  That one file compiles on its own
with nvcc against a CUTLASS header tree; the reference's build system (backend.build_native) is
not run because its hash gate wants the exact CUTLASS pin, which is not on this machine.  The
CUTLASS copy vendored with flashinfer is used instead; the four headers that define the sparse
layout and `reorder_meta` are byte-identical to the pin.

Output goes to oracle/_ref/dualscale_sm80.so only (git-ignored).  The SM80 kernels inside cannot
run on other GPUs; only the CPU op `sdacc_dualscale_sm80::pack_cpu` is used, to generate golden
vectors (tests/golden/make_golden.py) and to cross-check the restated packer.

Usage: python oracle/build_ref.py [--reference /path/to/SlideSparse-Diffusion]
"""
import argparse
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent


def cutlass_root():
    import flashinfer
    root = Path(flashinfer.__file__).parent / "data" / "cutlass"
    if not (root / "include" / "cutlass" / "cutlass.h").exists():
        raise FileNotFoundError("no CUTLASS header tree next to flashinfer")
    return root


def build(reference, force=False):
    import torch
    from torch.utils.cpp_extension import include_paths, library_paths
    source = Path(reference) / "sdacc/w8a8_slidesparse/csrc/dualscale_sm80.cu"
    if not source.exists():
        raise FileNotFoundError(source)
    out_dir = HERE / "_ref"
    out_dir.mkdir(exist_ok=True)
    target = out_dir / "dualscale_sm80.so"
    if target.exists() and not force and target.stat().st_mtime >= source.stat().st_mtime:
        return target
    cut = cutlass_root()
    nvcc = str(Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "bin/nvcc")
    cmd = [nvcc, "-std=c++17", "-O3", "--shared", "--expt-relaxed-constexpr",
           "--expt-extended-lambda", "-Xcompiler", "-fPIC", "-t", "8",
           "-gencode=arch=compute_80,code=sm_80",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           f"-I{cut}/include", f"-I{cut}/tools/util/include"]
    cmd += [f"-I{p}" for p in include_paths("cuda")]
    cmd += [f"-L{p}" for p in library_paths("cuda")]
    cmd += ["-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
            "-Xlinker", f"-rpath,{Path(torch.__file__).parent}/lib", str(source), "-o", str(target)]
    with (out_dir / "compile.log").open("w") as log:
        subprocess.run(cmd, check=True, stdout=log, stderr=subprocess.STDOUT)
    return target


def load():
    """torch.ops.sdacc_dualscale_sm80.pack_cpu from the built library (CPU only)."""
    import torch
    target = HERE / "_ref" / "dualscale_sm80.so"
    if not target.exists():
        raise FileNotFoundError(f"{target}: run oracle/build_ref.py where the reference is mounted")
    torch.ops.load_library(str(target))
    return torch.ops.sdacc_dualscale_sm80.pack_cpu


if __name__ == "__main__":
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--reference", default=os.environ.get("SS_REFERENCE"),
                        help="root of the SlideSparse-Diffusion source tree (or set SS_REFERENCE)")
    parser.add_argument("--force", action="store_true")
    args = parser.parse_args()
    if not args.reference:
        parser.error("give --reference or set SS_REFERENCE")
    print(build(args.reference, args.force))
    sys.exit(0)
