"""Explicit offline build of the native library; never run by package installation.

Replaces the reference's `scripts/build_native.py:6-14`: no CUTLASS checkout is needed, the only
target is sm_100a.  Usage:  python build_native.py [--output DIR] [--force]
"""
import argparse
import importlib.util
import sys
from pathlib import Path


def load_package():
    root = Path(__file__).resolve().parent
    name = "slidesparse_diffusion_b200"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, root / "__init__.py",
                                                  submodule_search_locations=[str(root)])
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    spec.loader.exec_module(module)
    return module


def main():
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--arch", default="sm_100a")
    parser.add_argument("--output", type=Path, default=None,
                        help="directory for the library and its receipt (default: <package>/native_sm100a)")
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--binding", action="store_true",
                        help="also write SOURCE_BINDING.json (file hashes) next to the package sources")
    args = parser.parse_args()
    sdk = load_package()
    receipt = sdk.build_native(args.output, arch=args.arch, force=args.force)
    print("Built native library", receipt["library_sha"][:16], "for", receipt["arch"])
    if args.binding:
        from slidesparse_diffusion_b200 import backend
        print("Wrote", backend.BINDING_NAME, "over", len(backend.write_source_binding()["files"]), "files")


if __name__ == "__main__":
    main()
