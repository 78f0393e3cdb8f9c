"""The bench's CPU arm on a small graph, without a GPU: `--impl reference` prints a well-formed line whose value is a
step measured in full (not scaled), with the user-defined-function figure beside it marked as extrapolated, and the
compiled destination-row loop it times returns what the oracle returns."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_prints_a_measured_line():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--scale", "0.002", "--steps", "2",
                        "--warmup", "1"], capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1])
    assert line["impl"] == "reference" and line["metric"] == "gcn_layer_fwd_ms" and line["unit"] == "ms"
    assert line["steps"] == 2 and line["warmup"] == 1 and line["higher_is_better"] is False
    assert line["value"] > 0 and line["value"] == line["ms_per_step"] == line["cpu_baseline"]["value"] == line["e2e"]["value"]
    cb = line["cpu_baseline"]
    assert cb["kind"] == "port" and cb["extrapolated"] is False and cb["cores"] >= 1
    assert cb["udf_path"]["extrapolated"] is True and cb["udf_path"]["scale_factor"] >= 1.0
    assert "compensated" not in line["config"]["accumulation"]           # the CPU arm adds in plain float
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["gpu_launches"] == 0


def test_cpu_layer_matches_the_oracle():
    sys.path.insert(0, str(ROOT))
    import bench
    from graphiler_b200 import synthetic
    from oracle import ops_oracle as O
    wl = synthetic.make_c5(scale=0.002, device="cpu")
    g, x, w = wl.graph, wl.feats, wl.params["gcn_w"]
    cpu = bench.CpuLayer(g, x, w, threads=2)
    sec, sec_mm = cpu.step()
    assert sec > 0 and 0 < sec_mm <= sec
    norm = g.in_degrees().clamp(min=1).double().pow(-0.5).unsqueeze(1)
    h = (x.double() @ w.double()) * norm
    want = np.maximum(O.spmm_src(h.numpy(), g.in_pointer, g.in_node_indices) * norm.numpy(), 0)
    assert np.allclose(cpu.out, want, rtol=1e-4, atol=1e-4)
    u = cpu.udf_slice(0.25)
    assert u["extrapolated"] and 3.0 < u["scale_factor"] < 5.0 and u["value"] > 0
