"""In-tree build of the native libraries.

Two shared objects are produced under ``zendnn-pytorch-plugin_b200/lib``:

* ``libzentorch_b200.so`` -- the CUDA kernels and the C ABI (``include/zentorch_b200.h``), compiled with
  nvcc for sm_100a only.  It does not depend on PyTorch.
* ``libzentorch_b200_torch.so`` -- the operator registrations (``csrc/torch_ops.cpp``) compiled with the
  host compiler against the installed PyTorch, linked to the first.

Run ``python -m zentorch_b200._build`` (or ``__graft_entry__.build()``) after changing sources.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys
from pathlib import Path

PKG_ROOT = Path(__file__).resolve().parent.parent
CSRC = PKG_ROOT / "csrc"
LIB_DIR = PKG_ROOT / "lib"
OBJ_DIR = LIB_DIR / "obj"
INCLUDE = PKG_ROOT.parent / "include"
KERNEL_LIB = LIB_DIR / "libzentorch_b200.so"
TORCH_LIB = LIB_DIR / "libzentorch_b200_torch.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if Path(cand).exists() else "nvcc"


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(d).stat().st_mtime <= t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(map(str, cmd)), flush=True)
    res = subprocess.run(list(map(str, cmd)), capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(map(str, cmd))}\n{res.stdout}\n{res.stderr}")
    return res.stdout + res.stderr


def build_kernels(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    jobs = []
    for src in sources:
        obj = OBJ_DIR / (src.stem + ".o")
        if force or not _newer(obj, [src, *headers]):
            # ZENTORCH_B200_NVCC_DEFINES: extra -D switches for a diagnostic build, e.g. "-DZT_TCPROF" compiles the
            # per-role cycle counters of the tcgen05 weight-only kernel (read by `bench.py --profile woq_roles`)
            extra = os.environ.get("ZENTORCH_B200_NVCC_DEFINES", "").split()
            cmd = [_nvcc(), *NVCC_FLAGS, *extra, *(["-Xptxas", "-v"] if ptxas_info else []), "-c", src, "-o", obj]
            jobs.append(cmd)
    logs = []
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            logs = list(ex.map(lambda c: _run(c, verbose), jobs))
    objs = [OBJ_DIR / (s.stem + ".o") for s in sources]
    if jobs or force or not _newer(KERNEL_LIB, objs):
        _run([_nvcc(), "-shared", "-o", KERNEL_LIB, *objs, "-cudart", "shared"], verbose)
    if ptxas_info:
        print("\n".join(logs))
    return KERNEL_LIB


def build_torch_ext(force: bool = False, verbose: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension

    src = CSRC / "torch_ops.cpp"
    deps = [src, *INCLUDE.glob("*.h"), KERNEL_LIB]
    if not force and _newer(TORCH_LIB, deps):
        return TORCH_LIB
    torch_lib = Path(torch.__file__).parent / "lib"
    inc = []
    for p in cpp_extension.include_paths(device_type="cuda"):
        inc += ["-isystem", p]
    import sysconfig
    inc += ["-isystem", sysconfig.get_paths()["include"]]
    cxx = "g++"
    cmd = [
        cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-D_GLIBCXX_USE_CXX11_ABI=1",
        "-DTORCH_API_INCLUDE_EXTENSION_H", *inc, src, "-o", TORCH_LIB,
        f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
        f"-L{LIB_DIR}", "-lzentorch_b200", "-L/usr/local/cuda/lib64", "-lcudart",
        "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}",
    ]
    _run(cmd, verbose)
    return TORCH_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force=force, verbose=verbose)
    build_torch_ext(force=force, verbose=verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
    print("built", KERNEL_LIB, TORCH_LIB)
