"""Build the reference's own CUDA operator library as a checker.  TEST INFRASTRUCTURE.

Output: oracle/_ref/libgraphiler_ref.so (git-ignored, never shipped, never on the product path) — the
nine translation units the reference's CMakeLists.txt:12-23 lists (src/dglgraph.cpp, src/ops/broadcast/*.cu,
src/ops/segment_softmax/*.cu, src/ops/dgl_primitives/{spmm.cu,bcast.cc,sddmm.cu}, src/ops/segment_mm/segment_mm.cu)
compiled with nvcc for sm_100 directly from where they lie in the reference tree.  No reference source is
copied or edited: the two incompatibilities with current PyTorch are bridged from outside the sources by
oracle/ref_shim/ (an empty THC/THC.h on the include path, and a force-included header that maps the
`at::optional<at::ScalarType>` arguments to `optional<int64_t>` so that the "int? t" schemas register).
The reference's CMake build is not run.

The library registers the same `my_classes.DGLGraph` / `my_ops::*` names as the product library, so one
process can load only one of the two: tests/golden/make_ref_ops_golden.py loads this one in a process of
its own, runs the reference operators on a GPU and writes the outputs that pin oracle/ops_oracle.py.

Run from the repository root:  python oracle/build_ref_cuda.py [reference_dir]
(the directory also comes from $GRAPHILER_REFERENCE_DIR; default: ../reference beside the repository).  Exits 0 with a message when the tree is absent.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
SHIM = HERE / "ref_shim"
UNITS = ["src/dglgraph.cpp", "src/ops/broadcast/broadcast.cu", "src/ops/broadcast/scatter_kernel.cu",
         "src/ops/segment_softmax/segment_softmax.cu", "src/ops/segment_softmax/segment_softmax_kernel.cu",
         "src/ops/dgl_primitives/spmm.cu", "src/ops/dgl_primitives/bcast.cc", "src/ops/dgl_primitives/sddmm.cu",
         "src/ops/segment_mm/segment_mm.cu"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def reference_dir(argv=None) -> Path:
    argv = sys.argv[1:] if argv is None else argv
    if argv:
        return Path(argv[0])
    return Path(os.environ.get("GRAPHILER_REFERENCE_DIR", HERE.parent.parent / "reference"))


def build(ref: Path, jobs: int = 0) -> int:
    if not ref.exists():
        print(f"reference tree {ref} is absent: oracle/_ref is used as already built")
        return 0
    import torch
    from torch.utils import cpp_extension as ce

    so = OUT / "libgraphiler_ref.so"
    srcs = [ref / u for u in UNITS]
    deps = srcs + list(SHIM.rglob("*.h")) + list((ref / "src" / "ops").rglob("*.h")) + list((ref / "src" / "ops").rglob("*.cuh"))
    if so.exists() and all(p.stat().st_mtime <= so.stat().st_mtime for p in deps):
        print("oracle/_ref/libgraphiler_ref.so is up to date")
        return 0
    obj = OUT / "obj_cuda"
    obj.mkdir(parents=True, exist_ok=True)
    tl = Path(torch.__file__).parent / "lib"
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    inc = [f"-I{SHIM}", *[f"-I{p}" for p in ce.include_paths()], f"-I{ref / 'include'}", f"-I{ref / 'src' / 'ops'}",
           f"-I{ref / 'src' / 'ops' / 'dgl_primitives'}"]
    flags = ["-gencode", "arch=compute_100,code=sm_100", "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-w", "-DNDEBUG",
             f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-x", "cu", "-include", str(SHIM / "ref_compat.h"), *inc]
    jobs = jobs or max(1, min(len(srcs), (os.cpu_count() or 2)))
    pending = list(srcs)
    running, objs = [], []
    failed = False
    while pending or running:
        while pending and len(running) < jobs:
            s = pending.pop(0)
            o = obj / (s.stem + ("_cc" if s.suffix == ".cc" else "") + ".o")
            objs.append(o)
            if o.exists() and all(p.stat().st_mtime <= o.stat().st_mtime for p in [s, *SHIM.rglob("*.h")]):
                continue
            running.append((s, subprocess.Popen([_nvcc(), *flags, "-c", str(s), "-o", str(o)],
                                                stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        if running:
            s, p = running.pop(0)
            text = p.communicate()[0]
            if p.returncode != 0:
                sys.stderr.write(text)
                print(f"could not compile {s}", file=sys.stderr)
                failed = True
    if failed:
        return 1
    r = subprocess.run([_nvcc(), "-shared", "-o", str(so), *[str(o) for o in objs], f"-L{tl}", "-ltorch", "-ltorch_cpu",
                        "-lc10", "-ltorch_cuda", "-lc10_cuda", "-lcusparse", "-lcublas", "-lcudart",
                        "-Xlinker", f"-rpath={tl}"], capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        return 1
    print("oracle/_ref/libgraphiler_ref.so built from", ref)
    return 0


if __name__ == "__main__":
    sys.exit(build(reference_dir()))
