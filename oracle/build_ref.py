"""Build the checker for the drop-in boundary from the reference's own sources.  TEST INFRASTRUCTURE.

Outputs, all under oracle/_ref/ (git-ignored, never shipped or timed):

  graphiler/mpdfg.so          the reference's MP-DFG builder, optimizer passes and pybind module, compiled
                              from src/pybind.cpp, src/builder/builder.cpp and src/optimizer/*.cpp where they
                              lie in the reference tree (g++ directly; -DNDEBUG because two assert bodies in
                              builder.cpp do not compile; the reference's CMake/setup.py are not run)
  graphiler/*.py              an installed copy of the reference's Python wrapper core (the five modules
                              python/graphiler/__init__.py imports; its utils package needs DGL/OGB)
  libgraphiler_cpu.so         oracle/cpu_oplib.cpp: a CPU registration of the operator set, so the compiled
                              graphs can be executed without a GPU

Run from the repository root:  python oracle/build_ref.py [reference_dir]
Skips work that is up to date; exits 0 with a message if the reference tree is absent.
"""
from __future__ import annotations

import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
CPP = ["src/pybind.cpp", "src/builder/builder.cpp", "src/optimizer/dedup.cpp", "src/optimizer/split.cpp",
       "src/optimizer/reorder.cpp", "src/optimizer/fusion.cpp"]
PY = ["__init__.py", "dgl_udf_batch.py", "mpdfg_builder.py", "mpdfg_optimizer.py", "update_all.py"]


def _flags():
    import pybind11
    import sysconfig
    import torch
    from torch.utils import cpp_extension as ce
    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}"]
    tl = Path(torch.__file__).parent / "lib"
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    common = ["-O1", "-std=c++17", "-fPIC", "-DNDEBUG", "-w", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", *inc]
    link = [f"-L{tl}", "-ltorch", "-ltorch_cpu", "-lc10", f"-Wl,-rpath,{tl}"]
    return common, link


def _stale(target: Path, sources) -> bool:
    return (not target.exists()) or any(Path(s).stat().st_mtime > target.stat().st_mtime for s in sources)


def build(ref: Path) -> int:
    if not ref.exists():
        print(f"reference tree {ref} is absent: oracle/_ref is used as already built")
        return 0
    common, link = _flags()
    pkg = OUT / "graphiler"
    obj = OUT / "obj"
    pkg.mkdir(parents=True, exist_ok=True)
    obj.mkdir(parents=True, exist_ok=True)

    so = pkg / "mpdfg.so"
    srcs = [ref / c for c in CPP]
    if _stale(so, srcs):
        procs = []
        for s in srcs:
            o = obj / (s.stem + ".o")
            procs.append((s, o, subprocess.Popen(["g++", *common, "-DTORCH_EXTENSION_NAME=mpdfg", "-DTORCH_API_INCLUDE_EXTENSION_H",
                                                  f"-I{ref}", "-c", str(s), "-o", str(o)],
                                                 stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        for s, o, p in procs:
            text = p.communicate()[0]
            if p.returncode != 0:
                sys.stderr.write(text)
                print(f"could not compile {s}", file=sys.stderr)
                return 1
        r = subprocess.run(["g++", "-shared", "-o", str(so), *[str(o) for _, o, _ in procs], *link, "-ltorch_python"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            return 1
    for name in PY:                                   # the install step of the Python wrapper
        shutil.copyfile(ref / "python" / "graphiler" / name, pkg / name)

    cpu = OUT / "libgraphiler_cpu.so"
    src = HERE / "cpu_oplib.cpp"
    if _stale(cpu, [src]):
        r = subprocess.run(["g++", *common, "-shared", str(src), "-o", str(cpu), *link], capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            return 1
    print("oracle/_ref ready:", ", ".join(sorted(p.name for p in OUT.iterdir())))
    return 0


if __name__ == "__main__":
    import os
    default = Path(os.environ.get("GRAPHILER_REFERENCE_DIR", HERE.parent.parent / "reference"))
    sys.exit(build(Path(sys.argv[1]) if len(sys.argv) > 1 else default))
