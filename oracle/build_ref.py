"""Builds oracle/_ref/libsharq_ref.so: the REFERENCE's own CUDA kernels for the hot path,
compiled in place from the reference checkout (no source is copied) with a short nvcc
recipe, plus the extern "C" shims of oracle/ref_wrap.cu.  TEST INFRASTRUCTURE ONLY.

    python oracle/build_ref.py [/path/to/reference] [--gemm]
    python oracle/build_ref.py [/path/to/reference] --stage-python   # see stage_python()

The reference needs NVIDIA CUTLASS, an un-vendored and unpinned submodule of its repository;
the CUTLASS 4.5.0 headers shipped inside the flashinfer wheel are used instead (the version
the reference's authors built with is unknown).  Its own build system (cmake + torch) is
not run.  Without --gemm only the quantisation kernels are built (about 2 minutes); with
--gemm also its two CUTLASS GEMM wrappers (several more minutes).  The library is
optional: tests that use it skip when it is absent.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
QUANT_SOURCES = ["fused_sparse_prepare.cu", "fused_rmsnorm_sparse_prepare.cu", "shared_weight_nvfp4.cu", "reorder.cu"]
GEMM_SOURCES = ["nvfp4.cu", "sparse_nvfp4.cu"]


def cutlass_root() -> Path:
    import flashinfer  # only to locate the vendored headers

    root = Path(flashinfer.__file__).parent / "data" / "cutlass"
    if not (root / "include" / "cutlass" / "cutlass.h").exists():
        raise SystemExit("CUTLASS headers not found; oracle/_ref not built")
    return root


def reference_dir() -> Path:
    """The reference checkout: $SHARQ_REFERENCE_DIR, else a directory named `reference` beside this repository."""
    env = os.environ.get("SHARQ_REFERENCE_DIR")
    return Path(env) if env else HERE.parent.parent / "reference"


def build(ref: Path = None, with_gemm: bool = False) -> None:
    ref = reference_dir() if ref is None else Path(ref)
    if not (ref / "kernels" / "src").exists():
        raise SystemExit(f"no reference checkout at {ref}; oracle/_ref not built")
    cut = cutlass_root()
    OUT.mkdir(exist_ok=True)
    obj = OUT / "obj"
    obj.mkdir(exist_ok=True)
    stub = OUT / "stub"
    stub.mkdir(exist_ok=True)
    # the reference includes CUTLASS's examples/common/helper.h but uses nothing from it
    (stub / "helper.h").write_text("#pragma once\n")
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "--expt-relaxed-constexpr", "-w",
             "-Xcompiler", "-fPIC", "-Xcompiler", "-fpermissive", "-DSHARQ_TARGET_SM100A",
             f"-I{ref / 'kernels' / 'include'}", f"-I{cut / 'include'}", f"-I{cut / 'tools' / 'util' / 'include'}",
             f"-I{stub}"]
    sources = [ref / "kernels" / "src" / s for s in QUANT_SOURCES + (GEMM_SOURCES if with_gemm else [])]
    sources.append(HERE / "ref_wrap.cu")
    defs = ["-DSHARQ_REF_WITH_GEMM"] if with_gemm else []

    def compile_one(src: Path) -> Path:
        o = obj / (src.name + (".gemm.o" if (with_gemm and src.name == "ref_wrap.cu") else ".o"))
        if o.exists() and o.stat().st_mtime > src.stat().st_mtime:
            return o
        subprocess.run(["nvcc", *flags, *defs, "-c", str(src), "-o", str(o)], check=True)
        return o

    with ThreadPoolExecutor(max_workers=4) as pool:
        objs = list(pool.map(compile_one, sources))
    name = "libsharq_ref_gemm.so" if with_gemm else "libsharq_ref.so"
    subprocess.run(["nvcc", "-shared", "-o", str(OUT / name), *map(str, objs)], check=True)
    print(OUT / name)


PYTHON_FILES = ["sharq_loader.py", "model/quantize.py", "model/qLinearLayer.py", "model/hif4.py",
                "benchmarks/correctness/example_fused_pairtop2_matrix_suite.py"]


def stage_python(ref: Path = None) -> Path:
    """Copies the reference's UNMODIFIED Python host code for the hot path (loader, QLinearLayer,
    quantize glue, its matrix-suite correctness script) into the git-ignored oracle/_ref/py/, keeping
    the directory layout, so that GPU tests can run it on top of this project's drop-in `sharq_ops`
    module on a machine that has no reference checkout.  Nothing of it enters the repository."""
    import shutil

    ref = reference_dir() if ref is None else Path(ref)
    out = OUT / "py"
    for rel in PYTHON_FILES:
        src = ref / rel
        if not src.exists():
            raise SystemExit(f"{src} not found; oracle/_ref/py not staged")
        dst = out / rel
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(src, dst)
    print(out)
    return out


if __name__ == "__main__":
    _args = [a for a in sys.argv[1:] if not a.startswith("--")]
    if "--stage-python" in sys.argv:
        stage_python(Path(_args[0]) if _args else None)
    else:
        build(Path(_args[0]) if _args else None, "--gemm" in sys.argv)
