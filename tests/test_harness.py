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
