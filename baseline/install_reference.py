"""Completes the offline install of the reference under ``baseline/_ref`` for use on a B200.

Step 0 (done once by hand)::

    python -m pip install --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse \
        --target baseline/_ref <checkout of the reference>

Step 1, package data: the wheel that pip builds leaves out the package's data files (its
``MANIFEST.in`` names none), among them ``attention/zero_padded_qlen_thresholds.csv`` which
``keys_values.attention.use_eager_kernel`` reads when a model is constructed. They are copied
from the checkout as they are.

Step 2, the reference's own CUDA extension for B200, from its unchanged sources.

The reference ships ``keys_values/csrc`` (FlashInfer-template SDPA kernels) with a build
script that embeds machine code for sm_80 and sm_90 only, so the extension cannot load its
kernels on a B200. This script copies the ``csrc`` sources as they are into a scratch
folder, compiles them with the reference's own compiler flags plus one
``-gencode=arch=compute_100,code=sm_100``, and places the resulting
``_flashinfer_ops*.so`` inside the installed reference package (``baseline/_ref/keys_values``),
which is where ``keys_values.attention.flashinfer_ops`` looks for it.

    python baseline/install_reference.py [--source /path/to/reference/checkout] [--no-ext]

Not a single source line of the reference is changed; nothing of this repository is
compiled into it.
"""
from __future__ import annotations

import argparse
import os
import importlib.util
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_PKG = HERE / "_ref" / "keys_values"
SCRATCH = HERE / "_ref" / "_ext_build"


def flashinfer_includes() -> list:
    """The FlashInfer headers plus the CCCL copy that package ships for them (its headers use
    ``cuda::fast_mod_div``, which the CUDA 12.9 toolkit's own libcudacxx does not have yet)."""
    spec = importlib.util.find_spec("flashinfer")
    if spec is None or spec.origin is None:
        raise RuntimeError("the flashinfer package (for its headers) is not installed")
    data = Path(spec.origin).parent / "data"
    inc = data / "include"
    if not inc.is_dir():
        raise RuntimeError(f"flashinfer headers not found under {inc}")
    out = [str(inc)]
    for sub in ("libcudacxx/include", "cub", "thrust"):
        if (data / "cccl" / sub).is_dir():
            out.append(str(data / "cccl" / sub))
    return out


def copy_package_data(src_pkg: Path) -> None:
    for f in src_pkg.rglob("*"):
        if not f.is_file() or f.suffix in (".py", ".pyc") or "csrc" in f.parts or "__pycache__" in f.parts:
            continue
        dst = REF_PKG / f.relative_to(src_pkg)
        if dst.parent.is_dir() and not dst.exists():
            shutil.copy2(f, dst)
            print(f"copied {dst.relative_to(REF_PKG)}")


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--source", type=Path, default=Path(os.environ.get("KEYS_VALUES_REFERENCE", "reference")),
                    help="checkout of the reference that holds keys_values/csrc (default: $KEYS_VALUES_REFERENCE or ./reference)")
    ap.add_argument("--no-ext", action="store_true", help="copy the package data only")
    args = ap.parse_args()
    csrc = args.source / "keys_values" / "csrc"
    if not csrc.is_dir():
        print(f"no csrc under {args.source}", file=sys.stderr)
        return 2
    if not REF_PKG.is_dir():
        print("baseline/_ref/keys_values is missing: install the reference there first", file=sys.stderr)
        return 2
    copy_package_data(args.source / "keys_values")
    if args.no_ext:
        return 0
    if SCRATCH.exists():
        shutil.rmtree(SCRATCH)
    shutil.copytree(csrc, SCRATCH / "keys_values" / "csrc")
    (SCRATCH / "keys_values" / "__init__.py").write_text("")

    import torch.utils.cpp_extension as ext

    ext._check_cuda_version = lambda *a, **k: None
    from setuptools import setup
    from torch.utils.cpp_extension import BuildExtension, CUDAExtension

    src = SCRATCH / "keys_values" / "csrc"
    module = CUDAExtension(
        name="keys_values._flashinfer_ops",
        sources=[str(src / "bindings.cpp"), str(src / "kernels" / "sdpa_decode.cu"), str(src / "kernels" / "sdpa_prefill.cu")],
        include_dirs=[str(src), *flashinfer_includes()],
        extra_compile_args={
            "cxx": ["-O3"],
            "nvcc": [
                "-O3", "--use_fast_math", "-std=c++17", "--expt-relaxed-constexpr", "--expt-extended-lambda",
                "-Xcompiler=-fPIC", "-Xcompiler=-Wno-float-conversion",
                "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
                "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
                # the reference's own list is sm_80 + sm_90; B200 needs its own machine code
                "-gencode=arch=compute_100,code=sm_100",
            ],
        },
    )
    import os

    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    os.environ.setdefault("MAX_JOBS", "8")
    cwd = os.getcwd()
    os.chdir(SCRATCH)
    try:
        sys.argv = [sys.argv[0], "build_ext", "--inplace"]
        setup(name="keys_values_flashinfer", ext_modules=[module], cmdclass={"build_ext": BuildExtension})
    finally:
        os.chdir(cwd)
    built = sorted((SCRATCH / "keys_values").glob("_flashinfer_ops*.so"))
    if not built:
        print("build produced no _flashinfer_ops*.so", file=sys.stderr)
        return 1
    for so in built:
        shutil.copy2(so, REF_PKG / so.name)
        print(f"installed {REF_PKG / so.name}")
    shutil.rmtree(SCRATCH)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
