"""Builds libaicf_b200.so (hand-written sm_100a kernels + registry + C ABI) in-tree with nvcc, and the Python
extension module aicf_cuda/_C (pybind11 over that C ABI, no torch) with g++.

    python build.py            # incremental build into ./lib/
    python build.py --force    # rebuild everything

No GPU is needed: nvcc cross-compiles for sm_100a. The library links only the CUDA runtime
(statically) and libdl; NCCL is resolved at run time.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
REPO = ROOT.parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "build"
LIB_DIR = ROOT / "lib"
LIB = LIB_DIR / "libaicf_b200.so"

GENCODE = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC",
          f"-I{REPO / 'include'}", f"-I{CSRC}"]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build libaicf_b200.so")
    return exe


BINDINGS = CSRC / "python_bindings" / "bindings.cpp"  # the extension module, not part of the library


def sources() -> list[Path]:
    return sorted(s for s in list(CSRC.rglob("*.cu")) + list(CSRC.rglob("*.cpp")) if s != BINDINGS)


def extension_path() -> Path:
    import sysconfig
    return ROOT / "python" / "aicf_cuda" / ("_C" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_extension(force: bool = False, verbose: bool = True) -> Path:
    """aicf_cuda/_C.<abi tag>.so: pybind11 module linked against lib/libaicf_b200.so through a run path relative to
    the module's own location, so the package can be moved as a whole."""
    import sysconfig

    import pybind11
    out = extension_path()
    newest = max(BINDINGS.stat().st_mtime, (REPO / "include" / "aicf_b200.h").stat().st_mtime)
    if not force and out.exists() and out.stat().st_mtime > newest:
        if verbose:
            print(f"[build] {out} is up to date")
        return out
    gxx = shutil.which("g++")
    if gxx is None:
        raise RuntimeError("g++ not found: it is needed for the aicf_cuda._C extension module")
    cmd = [gxx, "-std=c++17", "-O2", "-shared", "-fPIC", "-fvisibility=hidden", f"-I{pybind11.get_include()}",
           f"-I{sysconfig.get_paths()['include']}", f"-I{REPO / 'include'}", str(BINDINGS), "-o", str(out),
           f"-L{LIB_DIR}", "-laicf_b200", "-Wl,-rpath,$ORIGIN/../../lib"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"g++ failed for {BINDINGS}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        print(f"[build] built {out} ({out.stat().st_size >> 10} KiB)")
    return out


def headers_mtime() -> float:
    hs = list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.hpp")) + list((REPO / "include").rglob("*.h*"))
    return max(h.stat().st_mtime for h in hs)


def compile_one(src: Path, force: bool, hdr_m: float) -> Path:
    obj = OBJ / (src.relative_to(CSRC).as_posix().replace("/", "__") + ".o")
    if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, hdr_m):
        return obj
    cmd = [nvcc(), *GENCODE, *COMMON, "-c", str(src), "-o", str(obj)]
    if src.suffix == ".cpp":
        cmd.insert(1, "-x")
        cmd.insert(2, "cu")  # host-only files still see cuda_runtime.h types
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    return obj


def build(force: bool = False, verbose: bool = True) -> Path:
    OBJ.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    srcs = sources()
    hdr_m = headers_mtime()
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(lambda s: compile_one(s, force, hdr_m), srcs))
    newest = max(o.stat().st_mtime for o in objs)
    if force or not LIB.exists() or LIB.stat().st_mtime < newest:
        cmd = [nvcc(), *GENCODE, "-shared", "-o", str(LIB), *map(str, objs), "-ldl",
               "-Xlinker", "--exclude-libs,ALL"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(f"[build] linked {LIB} ({LIB.stat().st_size >> 10} KiB) from {len(objs)} objects")
    elif verbose:
        print(f"[build] {LIB} is up to date")
    build_extension(force=force, verbose=verbose)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args()
    try:
        build(force=args.force)
    except RuntimeError as e:
        print(e, file=sys.stderr)
        sys.exit(1)
