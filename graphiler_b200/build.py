"""In-tree build of the native libraries (sm_100a only).

  lib/libgphl.so        CUDA kernels + C ABI (include/gphl.h); no torch dependency
  lib/libgraphiler.so   TorchScript registrations (my_classes.DGLGraph, my_ops::*) over the C ABI

``python -m graphiler_b200.build [--force] [--measure]`` rebuilds whatever is out of date (``--measure`` adds
lib/libgphl_measure.so, the same kernels with their tuning knobs readable from the environment).  nvcc cross-compiles
without a GPU.  The reference builds its operator library for sm_70 with CMake
(CMakeLists.txt:12-32); nothing of that build is reused.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "lib"

KERNEL_SOURCES = ["plan.cu", "spmm.cu", "softmax.cu", "sddmm.cu", "gather.cu", "segment_mm.cu", "segment_mm_tc.cu", "gspmm.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target: Path, sources) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in sources)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError(f"build step failed: {cmd[0]} (exit {r.returncode})")
    return r.stdout + r.stderr


def kernel_sources():
    return [CSRC / s for s in KERNEL_SOURCES if (CSRC / s).exists()]


def build_kernels(force: bool = False, verbose: bool = False, ptxas_info: bool = False, measure: bool = False) -> Path:
    """Compile every .cu file to an object (in parallel) and link lib/libgphl.so.

    ``measure=True`` builds lib/libgphl_measure.so instead: the same sources with -DGPHL_MEASURE, in which the
    tuning knobs of csrc/common.cuh are read from the environment.  Only the per-kernel timer loads it."""
    LIB.mkdir(exist_ok=True)
    out = LIB / ("libgphl_measure.so" if measure else "libgphl.so")
    srcs = kernel_sources()
    deps = srcs + list(CSRC.glob("*.cuh")) + [ROOT / "include" / "gphl.h"]
    if not force and not _stale(out, deps):
        return out
    objdir = LIB / ("obj_measure" if measure else "obj")
    objdir.mkdir(exist_ok=True)
    procs = []
    for s in srcs:
        o = objdir / (s.stem + ".o")
        cmd = [_nvcc(), *NVCC_FLAGS, *(["-DGPHL_MEASURE"] if measure else []),
               *(["-Xptxas", "-v"] if ptxas_info else []), "-c", s, "-o", o]
        if verbose:
            print(" ".join(str(c) for c in cmd), flush=True)
        procs.append((s, o, subprocess.Popen([str(c) for c in cmd], stdout=subprocess.PIPE,
                                             stderr=subprocess.STDOUT, text=True)))
    objs, log = [], []
    for s, o, p in procs:
        text = p.communicate()[0]
        log.append(text)
        if p.returncode != 0:
            sys.stderr.write(text)
            raise RuntimeError(f"nvcc failed on {s.name}")
        objs.append(o)
    _run([_nvcc(), "-shared", "-o", out, *objs, "-lcudart"], verbose)
    if ptxas_info:
        (LIB / "ptxas_info.txt").write_text("\n".join(log))
    return out


def build_torch_ops(force: bool = False, verbose: bool = False) -> Path:
    """Compile the TorchScript registration library with g++ against the installed torch."""
    import torch
    from torch.utils import cpp_extension as ce

    LIB.mkdir(exist_ok=True)
    out = LIB / "libgraphiler.so"
    src = CSRC / "torch_ops.cpp"
    deps = [src, ROOT / "include" / "gphl.h", LIB / "libgphl.so"]
    if not force and not _stale(out, deps):
        return out
    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{ROOT / 'include'}", "-I/usr/local/cuda/include"]
    torch_lib = Path(torch.__file__).parent / "lib"
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DNDEBUG", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
           *inc, src, "-o", out,
           f"-L{LIB}", "-lgphl", f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
           "-L/usr/local/cuda/lib64", "-lcudart",
           "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}", "-Wl,--no-as-needed"]
    _run(cmd, verbose)
    return out


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force, verbose)
    if (CSRC / "torch_ops.cpp").exists():
        build_torch_ops(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
    if "--measure" in sys.argv:
        build_kernels(force="--force" in sys.argv, verbose=True, measure=True)
    print("built:", *(p.name for p in LIB.glob("*.so")))
