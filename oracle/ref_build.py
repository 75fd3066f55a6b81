"""Compiles the REFERENCE's own CUDA op backend, unmodified and from where its sources lie, into
oracle/_ref/libaicf_ref.so for sm_100a. TEST INFRASTRUCTURE.

    python oracle/ref_build.py [--reference <reference checkout>/ai-compiler-framework]

Without --reference the tree is looked for in $AICF_REFERENCE_DIR, then in a `reference/` directory next to this
repository.

Only the reference's op launchers, registry.cpp and register_all.cpp are compiled (plain nvcc on the
files; the reference's CMake project is not run), together with oracle/ref_shim.cpp, which adds C
entry points. Nothing is copied into this repository: oracle/_ref/ holds build output only and is
git-ignored. The shared object is linked with -Bsymbolic so that its aicf::cuda symbols never mix with
the same-named symbols of libaicf_b200.so when both are loaded in one test process.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
DEFAULT_REF = Path(os.environ.get("AICF_REFERENCE_DIR") or HERE.parent.parent / "reference" / "ai-compiler-framework")
GENCODE = ["-gencode", "arch=compute_100a,code=sm_100a"]


def build(reference: Path = DEFAULT_REF, verbose: bool = True) -> Path | None:
    """Returns the library path, or None when the reference tree is not present (e.g. on a GPU
    machine that only received the prebuilt file)."""
    lib = OUT / "libaicf_ref.so"
    if not reference.exists():
        if verbose:
            print(f"[ref_build] {reference} not present; keeping {'existing' if lib.exists() else 'no'} prebuilt library")
        return lib if lib.exists() else None
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    OUT.mkdir(exist_ok=True)
    srcs = sorted((reference / "src/backends/cuda/ops").glob("*/launcher.cu"))
    srcs += [reference / "src/backends/cuda/registry/registry.cpp", reference / "src/backends/cuda/registry/register_all.cpp",
             HERE / "ref_shim.cpp"]
    newest_src = max(s.stat().st_mtime for s in srcs)
    if lib.exists() and lib.stat().st_mtime > newest_src:
        if verbose:
            print(f"[ref_build] {lib} is up to date")
        return lib
    inc = [f"-I{reference / 'include'}", f"-I{reference / 'src'}"]

    def one(src: Path) -> Path:
        obj = OUT / (src.parent.name + "__" + src.stem + ".o")
        cmd = [nvcc, *GENCODE, "-std=c++17", "-O3", "-w", "-Xcompiler", "-fPIC", *inc, "-x", "cu", "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"reference source failed to compile: {src}\n{r.stderr[-2000:]}")
        return obj

    with cf.ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(one, srcs))
    cmd = [nvcc, *GENCODE, "-shared", "-o", str(lib), *map(str, objs), "-Xlinker", "-Bsymbolic"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"reference link failed:\n{r.stderr[-2000:]}")
    for o in objs:
        o.unlink()
    if verbose:
        print(f"[ref_build] built {lib} from {len(srcs)} sources")
    return lib


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", type=Path, default=DEFAULT_REF)
    a = ap.parse_args()
    try:
        build(a.reference)
    except RuntimeError as e:
        print(e, file=sys.stderr)
        sys.exit(1)
