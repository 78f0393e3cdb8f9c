"""The added fusion patterns (graphiler_b200/fusion.py) on hand-written graphs: which targets are emitted, which
graphs are left alone, and that a rewritten graph returns what the operator-by-operator evaluation returns.  The
reference-flow tests cover the same pass on the four example models."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "oracle" / "_ref"


def run_cases(lib: Path, device: str):
    r = subprocess.run([sys.executable, str(ROOT / "tests" / "fusion_cases.py"), "--lib", str(lib), "--device", device],
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("REPORT ")][-1]
    return json.loads(line[len("REPORT "):])


def assess(rep, exact: bool):
    assert len(rep) >= 10
    for name, c in rep.items():
        assert c["emitted"] == c["expected"], (name, c)
        assert c["shapes_equal"], (name, c)
        # the CPU registration restates each target as the chain it replaces; the CUDA kernels fuse the arithmetic
        bound = 0.0 if exact else 1e-6 + 1e-5 * c["scale"]
        assert c["max_abs_diff"] <= bound, (name, c)


def test_fusion_patterns_cpu_registration():
    lib = REF / "libgraphiler_cpu.so"
    if not lib.exists():
        pytest.skip("oracle/_ref is not built (python oracle/build_ref.py needs the reference sources)")
    assess(run_cases(lib, "cpu"), exact=True)


@pytest.mark.gpu
def test_fusion_patterns_cuda_library():
    from graphiler_b200 import capi
    assert capi.TORCH_OPS_LIB.exists(), "libgraphiler.so is not built"
    assess(run_cases(capi.TORCH_OPS_LIB, "cuda"), exact=False)
