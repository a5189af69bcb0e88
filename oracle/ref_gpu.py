"""Golden vectors from the reference's own GPU code, run on whatever GPU is present.

TEST INFRASTRUCTURE ONLY.  Nothing here is imported by the product.

The reference ships its front-end (`quantize`, csrc/projection_sm80.cu:8-123) and its sparse GEMM
with the dequantising epilogue (`run`, csrc/dualscale_sm80.cu:72-398) only as CUDA code.  Its
`projection_sm80.cu` (which includes `dualscale_sm80.cu`) compiles unmodified for other
architectures: the warp-level `mma.sp` path it uses is a baseline feature of every GPU since
sm_80.  `build()` compiles that one translation unit from where it lies into
oracle/_ref/projection_sm100.so (git-ignored), `generate()` runs the reference operators on
seeded inputs in THIS process (which must not have loaded the B200 package: both define the same
torch operator namespaces) and writes the fixture that tests/test_oracle_golden.py checks the CPU
oracle against.

Only `run` configurations 14, 15 and 16 are used: the others need more than 48 KB of shared
memory, which the reference enables in `configure()`, and `configure()` refuses every GPU that is
not sm_80 (dualscale_sm80.cu:294).  All configurations share one epilogue arithmetic.

    python oracle/ref_gpu.py build    [--reference /path/to/SlideSparse-Diffusion]     (CPU box)
    python oracle/ref_gpu.py generate --out tests/golden/ref_gpu.npz                   (GPU box)
    python oracle/ref_gpu.py time                                                      (GPU box)
    python oracle/ref_gpu.py digest --out file.json                                    (GPU box)

`digest` runs the reference's projection at the FULL sizes of the benchmark configurations on
seeded inputs and writes SHA-256 digests of its INT8 activations, token scales and BF16 output;
tests/test_gpu_reference.py launches it as a child process and compares them with the digests of
this library's outputs on the same inputs.

`time` prints, for a few benchmark shapes, the device time of the reference's quantize and run
(configurations 14-16 only, see above: small tiles, not the configurations the reference's own
profiles pick on an A100) -- context for the B200 kernels, not a tuned baseline.
"""
import argparse
import hashlib
import os
import subprocess
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref" / "projection_sm100.so"

# (mode, m, k, n, config, bias, addend); k is limited to the widths the reference front-end accepts
CASES = (
    (4, 37, 1152, 40, 14, True, False),
    (6, 50, 1152, 200, 15, True, False),
    (8, 33, 1152, 96, 16, False, False),
    (6, 40, 2432, 72, 14, True, True),
    (8, 64, 1536, 130, 16, True, True),
    (6, 45, 3072, 64, 15, False, False),
)
FULL_ARRAYS = 3          # q / sa of the first cases are stored whole, the rest as SHA-256 digests


def build(reference, force=False):
    import torch
    from torch.utils.cpp_extension import include_paths, library_paths
    sys.path.insert(0, str(HERE))
    from build_ref import cutlass_root
    source = Path(reference) / "sdacc/w8a8_slidesparse/csrc/projection_sm80.cu"
    if not source.exists():
        raise FileNotFoundError(source)
    TARGET.parent.mkdir(exist_ok=True)
    if TARGET.exists() and not force and TARGET.stat().st_mtime >= source.stat().st_mtime:
        return TARGET
    cut = cutlass_root()
    nvcc = str(Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "bin/nvcc")
    cmd = [nvcc, "-std=c++17", "-O3", "--shared", "--expt-relaxed-constexpr", "--expt-extended-lambda",
           "-Xcompiler", "-fPIC", "-t", "8", "-gencode=arch=compute_100,code=sm_100",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           f"-I{cut}/include", f"-I{cut}/tools/util/include"]
    cmd += [f"-I{p}" for p in include_paths("cuda")]
    cmd += [f"-L{p}" for p in library_paths("cuda")]
    cmd += ["-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
            "-Xlinker", f"-rpath,{Path(torch.__file__).parent}/lib", str(source), "-o", str(TARGET)]
    with (TARGET.parent / "compile_sm100.log").open("w") as log:
        subprocess.run(cmd, check=True, stdout=log, stderr=subprocess.STDOUT)
    return TARGET


def case_inputs(oracle, index, mode, m, k, n, bias, addend):
    """Seeded inputs of one case; special values in the first rows pin the reference's conventions."""
    import torch
    x = oracle.make_activation(m, k, seed=100 + index).clone()
    x[0, :] = 0                                                   # all-zero row: scale floor
    x[1, :] = (x[1].float() * 1e-7).to(torch.bfloat16)             # below the scale floor
    x[2, 5] = float("inf")
    x[3, 7] = float("-inf")
    x[4, 9] = float("nan")
    x[5, 11], x[5, 13] = float("nan"), float("inf")
    qweight, scales = oracle.make_weight(n, k, mode, seed=200 + index)
    gen = torch.Generator().manual_seed(300 + index)
    b = (0.1 * torch.randn(n, generator=gen)).float().numpy() if bias else np.zeros(0, np.float32)
    a = torch.randn(m, n, generator=gen).to(torch.bfloat16) if addend else None
    return x, qweight, scales, b, a


def generate(out):
    import torch
    sys.path.insert(0, str(HERE.parent))
    from oracle import ss_oracle as oracle
    if "slidesparse_diffusion_b200" in sys.modules:
        raise RuntimeError("the B200 package is loaded: both libraries define the sdacc_* operator namespaces")
    torch.ops.load_library(str(TARGET))
    front, gemm = torch.ops.sdacc_mild_projection_sm80, torch.ops.sdacc_dualscale_sm80
    dev = torch.device("cuda", 0)
    data = {"cases": np.array(CASES, dtype=np.int64), "device": np.array(torch.cuda.get_device_name(0))}
    for index, (mode, m, k, n, config, bias, addend) in enumerate(CASES):
        x, qweight, scales, b, a = case_inputs(oracle, index, mode, m, k, n, bias, addend)
        _, pk = oracle.lifted_k(k, mode)
        lifted = torch.from_numpy(oracle.slide_weight(qweight, mode))
        packed, meta = gemm.pack_cpu(lifted, pk)                               # reference CPU packer
        q, sa = front.quantize(x.to(dev), mode)
        if k in (1152, 1536, 2432, 4608, 6144, 9728):                          # widths the packed16 front-end accepts
            q16, sa16 = front.quantize_packed16(x.to(dev), mode)
            assert torch.equal(q, q16) and torch.equal(sa.view(torch.int32), sa16.view(torch.int32)), "reference front-ends disagree"
        y = gemm.run(q, packed.to(dev), meta.to(dev), sa, torch.from_numpy(scales).to(dev), torch.from_numpy(b).to(dev),
                     m, n, config, None if a is None else a.to(dev))
        y2 = front.projection(x.to(dev), packed.to(dev), meta.to(dev), torch.from_numpy(scales).to(dev),
                              torch.from_numpy(b).to(dev), mode, n, config, None if a is None else a.to(dev))
        assert torch.equal(y.view(torch.int16), y2.view(torch.int16)), "reference projection differs from quantize + run"
        torch.cuda.synchronize()
        qn, san = q.cpu().numpy(), sa.cpu().numpy()
        if index < FULL_ARRAYS:
            data[f"q{index}"], data[f"sa{index}"] = qn, san
        data[f"q_sha{index}"] = np.array(hashlib.sha256(qn.tobytes()).hexdigest())
        data[f"sa_sha{index}"] = np.array(hashlib.sha256(san.tobytes()).hexdigest())
        data[f"y{index}"] = y.view(torch.int16).cpu().numpy().view(np.uint16)
        data[f"packed_sha{index}"] = np.array(hashlib.sha256(packed.numpy().tobytes()).hexdigest())
        data[f"meta_sha{index}"] = np.array(hashlib.sha256(meta.numpy().tobytes()).hexdigest())
    np.savez_compressed(out, **data)
    print(f"wrote {out}: {len(CASES)} cases on {torch.cuda.get_device_name(0)}")


# full-size cases of the benchmark configurations: (mode, m, k, n, config)
FULL_CASES = (
    (4, 4096, 1152, 4608, 16),        # configs[0]
    (6, 1536, 3072, 9216, 16),        # FLUX fused QKV
    (8, 1536, 12288, 3072, 15),       # FLUX MLP fc2
    (8, 4096, 3072, 12288, 16),       # FLUX MLP fc1, M swept
    (4, 2048, 4608, 1152, 14),        # DiT FFN-out
    (8, 8192, 1152, 3456, 16),        # PixArt-Sigma fused QKV
    (6, 2048, 2432, 9728, 16),        # SD3.5 image FFN-in
    (6, 666, 9728, 2432, 15),         # SD3.5 text FFN-out
)


def full_case_inputs(oracle, index, mode, m, k, n):
    import torch
    x = oracle.make_activation(m, k, seed=400 + index)
    qweight, scales = oracle.make_weight(n, k, mode, seed=500 + index)
    bias = (0.1 * torch.randn(n, generator=torch.Generator().manual_seed(600 + index))).float().numpy()
    return x, qweight, scales, bias


def digest(out):
    import json
    import torch
    sys.path.insert(0, str(HERE.parent))
    from oracle import ss_oracle as oracle
    if "slidesparse_diffusion_b200" in sys.modules:
        raise RuntimeError("the B200 package is loaded: both libraries define the sdacc_* operator namespaces")
    torch.ops.load_library(str(TARGET))
    front, gemm = torch.ops.sdacc_mild_projection_sm80, torch.ops.sdacc_dualscale_sm80
    dev = torch.device("cuda", 0)
    rows = []
    for index, (mode, m, k, n, config) in enumerate(FULL_CASES):
        x, qweight, scales, bias = full_case_inputs(oracle, index, mode, m, k, n)
        _, pk = oracle.lifted_k(k, mode)
        packed, meta = gemm.pack_cpu(torch.from_numpy(oracle.slide_weight(qweight, mode)), pk)
        q, sa = front.quantize(x.to(dev), mode)
        y = front.projection(x.to(dev), packed.to(dev), meta.to(dev), torch.from_numpy(scales).to(dev),
                             torch.from_numpy(bias).to(dev), mode, n, config, None)
        torch.cuda.synchronize()
        sha = lambda t: hashlib.sha256(t.contiguous().cpu().numpy().tobytes()).hexdigest()
        rows.append(dict(case=[mode, m, k, n, config], q=sha(q), sa=sha(sa), y=sha(y.view(torch.int16)),
                         packed=sha(packed)))
    Path(out).write_text(json.dumps({"device": torch.cuda.get_device_name(0), "rows": rows}))
    print(f"wrote {out}: {len(rows)} full-size cases")


def time_reference():
    import json
    import torch
    sys.path.insert(0, str(HERE.parent))
    from oracle import ss_oracle as oracle
    torch.ops.load_library(str(TARGET))
    front, gemm = torch.ops.sdacc_mild_projection_sm80, torch.ops.sdacc_dualscale_sm80
    dev = torch.device("cuda", 0)
    rows = []
    for (mode, m, k, n) in ((4, 4096, 1152, 4608), (6, 1536, 3072, 9216), (8, 1536, 3072, 12288),
                            (6, 4096, 3072, 9216), (4, 2048, 1152, 3456), (6, 2048, 2432, 9728)):
        _, pk = oracle.lifted_k(k, mode)
        pn, pm = -(-n // 32) * 32, -(-m // 32) * 32
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        packed = torch.randint(-127, 128, (pn, pk // 2), dtype=torch.int8, device=dev)
        meta = torch.full((pn * pk // 32,), 0x4E4E4E4E, dtype=torch.int32, device=dev)     # a valid index pair per nibble
        sw, bias = torch.rand(n, device=dev) + 0.5, torch.rand(n, device=dev)
        q, sa = front.quantize(x, mode)
        best = None
        for config in (14, 15, 16):
            for _ in range(3):
                gemm.run(q, packed, meta, sa, sw, bias, m, n, config, None)
            torch.cuda.synchronize()
            b, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            b.record()
            for _ in range(20):
                gemm.run(q, packed, meta, sa, sw, bias, m, n, config, None)
            e.record()
            torch.cuda.synchronize()
            us = b.elapsed_time(e) * 1e3 / 20
            best = (us, config) if best is None or us < best[0] else best
        b, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            front.quantize(x, mode)
        b.record()
        for _ in range(20):
            front.quantize(x, mode)
        e.record()
        torch.cuda.synchronize()
        rows.append(dict(mode=f"{mode - 2}:{mode}", m=m, k=k, n=n, run_us=best[0], run_config=best[1],
                         quantize_us=b.elapsed_time(e) * 1e3 / 20,
                         logical_tops=2.0 * m * n * k / (best[0] + b.elapsed_time(e) * 1e3 / 20) / 1e6))
    print(json.dumps({"device": torch.cuda.get_device_name(0), "rows": rows}))


if __name__ == "__main__":
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("action", choices=("build", "generate", "time", "digest"))
    parser.add_argument("--reference", default=os.environ.get("SS_REFERENCE"),
                        help="root of the SlideSparse-Diffusion source tree (or set SS_REFERENCE)")
    parser.add_argument("--out", default=str(HERE.parent / "tests" / "golden" / "ref_gpu.npz"))
    parser.add_argument("--force", action="store_true")
    args = parser.parse_args()
    if args.action == "build":
        if not args.reference:
            parser.error("build needs --reference or SS_REFERENCE")
        print(build(args.reference, args.force))
    elif args.action == "time":
        time_reference()
    elif args.action == "digest":
        digest(args.out)
    else:
        generate(args.out)
