"""The model-level harness (graphiler_b200/harness.py): the reference's benchmark helpers restated
(python/graphiler/utils/bench.py:10-62) and the four example models on the synthetic configurations."""
import numpy as np
import pytest
import torch

from graphiler_b200 import harness


def test_log_and_check_equal_helpers():
    log = harness.init_log(["a", "b"], ["time", "mem"])
    assert list(log.index.names) == ["tag", "metric"] and log.shape == (4,) and (log == 0).all()
    log.at[("a", "time")] = 1.5
    assert log.at[("a", "time")] == 1.5
    x = torch.arange(6.0).reshape(2, 3)
    assert harness.check_equal(x, x * (1 + 1e-5))
    assert not harness.check_equal(None, x)                    # an OOM run cannot be checked
    with pytest.raises(AssertionError):
        harness.check_equal(x + 1, x + 2)
    calls = []
    wrapped = harness.empty_cache(lambda v: calls.append(v) or v * 2)
    assert wrapped(3) == 6 and calls == [3]


@pytest.mark.gpu
@pytest.mark.parametrize("name,config,scale", [("gat", "c1", 0.1), ("gcn", "c2", 0.02), ("rgcn", "c3", 0.02),
                                               ("hgt", "c4", 0.01), ("gcn", "c5", 0.001)])
def test_models_run_timed_and_replayed_from_a_cuda_graph(name, config, scale):
    net, params = harness.model(name, config, scale=scale)
    tag = f"{name}-{config}"
    log = harness.init_log([tag], ["time", "mem", "time_cuda_graph"])
    out = harness.bench(net, params, tag=tag, memory=True, repeat=3, log=log, cuda_graph=True)
    assert out is not None and out.shape[0] == params[0].shape[0] and torch.isfinite(out).all()
    assert log.at[(tag, "time")] > 0 and log.at[(tag, "time_cuda_graph")] > 0 and log.at[(tag, "mem")] >= 0
    replay_out = net(*params)
    assert torch.equal(out, replay_out)                         # deterministic from call to call


def _compiled(model, device, scale, extra=()):
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    ref = root / "oracle" / "_ref"
    if not (ref / "graphiler").exists():
        pytest.skip("the reference's compiler was not built here (oracle/build_ref.py needs its source tree once)")
    cmd = [sys.executable, "-m", "graphiler_b200.harness", "--model", model, "--compiled", "--graphiler-path", str(ref),
           "--device", device, "--scale", str(scale), "--repeat", "2", *extra]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=str(root))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("correctness check passed!") == 3, r.stdout[-2000:]
    return json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1])


@pytest.mark.parametrize("model,scale", [("gcn", 0.02), ("gat", 0.02), ("rgcn", 0.02), ("hgt", 0.004)])
def test_series_through_the_reference_compiler_on_the_cpu_registration(model, scale):
    """`--compiled`: the model's user-defined functions built by the reference's mpdfg_builder at its three
    optimisation levels plus this package's fusion patterns, run by its update_all; here against the CPU
    registration of the operators (one process per model: the reference's builder keeps static state)."""
    from pathlib import Path
    cpu_lib = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libgraphiler_cpu.so"
    if not cpu_lib.exists():
        pytest.skip("oracle/_ref/libgraphiler_cpu.so was not built")
    rep = _compiled(model, "cpu", scale, ("--ops-lib", str(cpu_lib)))
    for tag in ("1+compile", "2+reorder", "3+fusion", "4+extra-fusion"):
        assert rep[tag]["time_ms"] > 0


@pytest.mark.gpu
@pytest.mark.parametrize("model,scale", [("gcn", 0.05), ("gat", 0.2), ("rgcn", 0.05), ("hgt", 0.02)])
def test_series_through_the_reference_compiler_on_the_gpu(model, scale):
    rep = _compiled(model, "cuda:0", scale)
    for tag in harness.COMPILED_TAGS:
        assert rep[tag]["time_ms"] > 0
