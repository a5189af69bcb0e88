"""The library-directory contract the reference's runtime binds a projection library by
(sdacc/diffusion_research/library.py:11-28 `bind`, :53-65 `profile_for`, `read_compiler_profiles`):
SOURCE_BINDING.json with the hash of every source file, a package importable under the name
`sdacc_research_library`, `load_native(<directory>/native_sm80)` before CUDA is initialised, a
`profile` submodule and a compiler_profiles.json with `entries`.  The steps of `bind` are restated
here and run in a fresh interpreter against a snapshot of this package."""
import json
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent

BIND_STEPS = r'''
import hashlib, importlib, importlib.util, json, sys
from pathlib import Path
snapshot = Path(sys.argv[1])
def sha(path):
    return hashlib.sha256(Path(path).read_bytes()).hexdigest()
receipt = json.loads((snapshot / "SOURCE_BINDING.json").read_text())
assert receipt["complete"]
for name, digest in receipt["files"].items():
    assert sha(snapshot / name) == digest, name
name = "sdacc_research_library"
spec = importlib.util.spec_from_file_location(name, snapshot / "__init__.py", submodule_search_locations=[str(snapshot)])
module = importlib.util.module_from_spec(spec)
sys.modules[name] = module
spec.loader.exec_module(module)
import torch
assert not torch.cuda.is_initialized(), "bind the ABI before allocating CUDA tensors"
module.load_native(snapshot / "native_sm80")
assert not torch.cuda.is_initialized()
profile = importlib.import_module(module.__name__ + ".profile")
config, frontend = profile.execution_profile(6, 1536, 3072, 9216)
entries = json.loads((Path(module.__file__).parent / "compiler_profiles.json").read_text())["entries"]
ops = torch.ops.sdacc_prepared_projection_sm80
print(json.dumps(dict(files=len(receipt["files"]), config=config, frontend=frontend, entries=len(entries),
                      has_ops=all(hasattr(ops, n) for n in ("prepare", "prepare_direct2", "prepare_singlepatch", "run", "release")),
                      names=sorted(module.__all__))))
'''


def test_bind_steps_against_a_snapshot_of_the_package(sdk, backend, tmp_path):
    package = ROOT / "slidesparse-diffusion_b200"
    snapshot = tmp_path / "checkout" / "slidesparse-diffusion_b200"
    shutil.copytree(package, snapshot, ignore=shutil.ignore_patterns("native_*", "__pycache__", backend.BINDING_NAME))
    shutil.copytree(ROOT / "include", tmp_path / "checkout" / "include")
    native = snapshot / "native_sm80"                       # the name `bind` looks for
    native.mkdir()
    built = backend.default_directory()
    for name in (backend.LIBRARY_NAME, "receipt.json"):
        shutil.copy2(built / name, native / name)
    receipt = backend.write_source_binding(snapshot)
    assert receipt["complete"] and "csrc/ss_gemm.cu" in receipt["files"] and "compiler_profiles.json" in receipt["files"]
    assert not any(name.startswith("native_") for name in receipt["files"])
    script = tmp_path / "bind_steps.py"
    script.write_text(BIND_STEPS)
    done = subprocess.run([sys.executable, str(script), str(snapshot)], capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr[-2000:]
    result = json.loads(done.stdout.strip().splitlines()[-1])
    assert result["files"] == len(receipt["files"]) and result["entries"] == 0 and result["has_ops"]
    assert (result["config"], result["frontend"]) == (5, "native")
    assert {"PackedLinear", "load_native", "build_native", "quantize_lift"} <= set(result["names"])
    # a changed source file must be caught by the hash check
    (snapshot / "profile.py").write_text((snapshot / "profile.py").read_text() + "\n# edited\n")
    again = subprocess.run([sys.executable, str(script), str(snapshot)], capture_output=True, text=True, timeout=300)
    assert again.returncode != 0 and "profile.py" in again.stderr
