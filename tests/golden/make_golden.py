"""Regenerate the golden fixtures of this directory.

    python tests/golden/make_golden.py            (from the repository root; needs the reference's source tree for the
                                                   one-off build of oracle/_ref by oracle/build_ref.py)

ref_flow_golden.npz / ref_flow_ops.json: seeded inputs, the outputs of the reference's own compiler flow
(its MP-DFG builder and optimizer compiled from its sources, executing on the CPU operator registration
oracle/cpu_oplib.cpp) for GCN / GAT / RGCN / HGT at optimisation levels 0, 1, 2 on the reference's two debug
graphs and three seeded random graphs, and the set of my_ops operators each optimised graph calls."""
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent.parent
if __name__ == "__main__":
    subprocess.check_call([sys.executable, str(ROOT / "oracle" / "build_ref.py")])
    subprocess.check_call([sys.executable, str(ROOT / "tests" / "ref_flow.py"), "--lib",
                           str(ROOT / "oracle" / "_ref" / "libgraphiler_cpu.so"), "--device", "cpu",
                           "--golden-out", str(ROOT / "tests" / "golden")], stdout=subprocess.DEVNULL)
    print("wrote", *(p.name for p in (ROOT / "tests" / "golden").glob("ref_flow_*")))
