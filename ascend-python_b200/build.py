"""In-tree build of the two native libraries.

* ``lib/libqmm_b200.so``  — the CUDA kernels behind the C ABI of
  ``include/qmm_b200.h`` (nvcc, sm_100a only).
* ``lib/libop_plugin_b200.so`` — the C++ operator host code (``op_plugin/``)
  with its generated torch-library registration, linked against the first.

Objects are rebuilt only when a source or header is newer than the object.
Run ``python build.py`` (add ``--force`` to rebuild everything).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OPP = PKG / "op_plugin"
BUILD = PKG / "build"
LIB = PKG / "lib"

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden", *NVCC_ARCH,
              f"-I{ROOT / 'include'}", f"-I{CSRC}"]

KERNEL_LIB = LIB / "libqmm_b200.so"
PLUGIN_LIB = LIB / "libop_plugin_b200.so"


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def _run(cmd, verbose=False):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError(f"command failed ({r.returncode}): {' '.join(str(c) for c in cmd)}")
    return r.stdout + r.stderr


def nccl_include_dir() -> Path | None:
    try:
        import nvidia.nccl  # type: ignore

        for base in nvidia.nccl.__path__:
            inc = Path(base) / "include"
            if (inc / "nccl.h").exists():
                return inc
    except Exception:
        pass
    for p in ("/usr/include", "/usr/local/cuda/include"):
        if (Path(p) / "nccl.h").exists():
            return Path(p)
    return None


def build_kernels(force=False, verbose=False) -> Path:
    BUILD.mkdir(exist_ok=True)
    LIB.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.inl")) + list(CSRC.glob("*.h")) + [ROOT / "include" / "qmm_b200.h"]
    sources = sorted(CSRC.glob("*.cu"))
    flags = list(NVCC_FLAGS)
    inc = nccl_include_dir()
    if inc is not None:
        flags.append(f"-I{inc}")
    jobs = []
    objs = []
    for src in sources:
        obj = BUILD / (src.stem + ".o")
        objs.append(obj)
        if force or _newer(obj, [src, *headers]):
            jobs.append([_nvcc(), *flags, "-c", src, "-o", obj])
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(lambda c: _run(c, verbose), jobs))
    if force or jobs or _newer(KERNEL_LIB, objs):
        _run([_nvcc(), "-shared", *NVCC_ARCH, "-o", KERNEL_LIB, *objs, "-ldl"], verbose)
    return KERNEL_LIB


def build_plugin(force=False, verbose=False) -> Path:
    """Generate the dispatch/registration sources from the yaml and compile the host code."""
    import torch
    from torch.utils import cpp_extension

    sys.path.insert(0, str(PKG))
    try:
        from codegen import gen_backend_stubs
    finally:
        sys.path.pop(0)
    gen_backend_stubs.run(OPP / "config" / "op_plugin_functions.yaml", OPP)

    BUILD.mkdir(exist_ok=True)
    LIB.mkdir(exist_ok=True)
    sources = sorted((OPP / "ops" / "opapi").glob("*.cpp")) + sorted((OPP / "utils").glob("*.cpp")) + \
        [OPP / "OpInterface.cpp", OPP / "TorchLibrary.cpp"]
    headers = list(OPP.rglob("*.h")) + [ROOT / "include" / "qmm_b200.h"]
    incs = [f"-I{p}" for p in cpp_extension.include_paths()] + [f"-I{ROOT / 'include'}", f"-I{PKG}",
                                                                  "-I/usr/local/cuda/include"]
    cxx = os.environ.get("CXX", "g++")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    flags = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
             "-DTORCH_API_INCLUDE_EXTENSION_H", "-Wno-deprecated-declarations", *incs]
    jobs, objs = [], []
    for src in sources:
        obj = BUILD / ("opp_" + src.stem + ".o")
        objs.append(obj)
        if force or _newer(obj, [src, *headers]):
            jobs.append([cxx, *flags, "-c", src, "-o", obj])
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(lambda c: _run(c, verbose), jobs))
    if force or jobs or _newer(PLUGIN_LIB, objs + [KERNEL_LIB]):
        tlib = Path(torch.__file__).parent / "lib"
        _run([cxx, "-shared", "-o", PLUGIN_LIB, *objs, f"-L{LIB}", "-lqmm_b200", f"-L{tlib}", "-ltorch", "-ltorch_cpu",
              "-lc10", "-ltorch_cuda", "-lc10_cuda", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tlib}"], verbose)
    return PLUGIN_LIB


def build_all(force=False, verbose=False):
    k = build_kernels(force, verbose)
    p = build_plugin(force, verbose)
    return k, p


if __name__ == "__main__":
    force = "--force" in sys.argv
    verbose = "-v" in sys.argv
    only_kernels = "--kernels" in sys.argv
    k = build_kernels(force, verbose)
    print("built", k)
    if not only_kernels:
        print("built", build_plugin(force, verbose))
