"""Model-level timing harness: the counterpart of the reference's benchmark utilities
(python/graphiler/utils/bench.py:10-62 — ``check_equal``, ``bench``, ``init_log``, ``empty_cache``) and of the
``profile`` functions of its examples (examples/GAT/GAT.py:87-164 and siblings), on the seeded synthetic
configurations of ``graphiler_b200.synthetic`` instead of the DGL/OGB datasets.

Differences from the reference's ``bench``: device time is taken with CUDA events on the current stream instead of
the host clock around a synchronize; an out-of-memory ``RuntimeError`` is still reported as "OOM" and returns
``None`` (python/graphiler/utils/bench.py:43-45), every other error propagates; ``cuda_graph=True`` additionally
replays the network from a captured CUDA graph, which is what a launch-latency-bound layer costs once the
per-kernel launch overhead is amortised.

    python -m graphiler_b200.harness --model gat --config c1 [--repeat 200] [--cuda-graph] [--memory]
"""
from __future__ import annotations

import argparse
import functools
import json
from typing import Callable, Dict, Optional, Sequence

import numpy as np
import pandas as pd
import torch

from . import layers, synthetic


def check_equal(first, second, rtol: float = 1e-3) -> bool:
    """Same contract as the reference's (python/graphiler/utils/bench.py:10-16): skipped when either run hit OOM."""
    if first is None or second is None:
        print("cannot guarantee correctness because of OOM")
        return False
    np.testing.assert_allclose(first.detach().cpu().numpy(), second.detach().cpu().numpy(), rtol=rtol)
    print("correctness check passed!")
    return True


def init_log(tags: Sequence[str], metrics: Sequence[str]) -> pd.Series:
    index = pd.MultiIndex.from_product([tags, metrics], names=["tag", "metric"])
    return pd.Series(np.zeros((len(tags) * len(metrics),)), index=index)


def empty_cache(func: Callable) -> Callable:
    @functools.wraps(func)
    def wrapper(*args, **kwargs):
        torch.cuda.empty_cache()
        return func(*args, **kwargs)
    return wrapper


def _timed(fn: Callable, repeat: int) -> float:
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(repeat):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / repeat


def capture(net: Callable, net_params: Sequence) -> Callable:
    """Capture ``net(*net_params)`` into a CUDA graph and return its replay function (inputs are read from the same
    tensors on every replay)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):                              # plans, workspaces and the allocator settle before capture
            net(*net_params)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        net(*net_params)
    return graph.replay


def bench(net: Callable, net_params: Sequence, tag: str = "", nvprof: bool = False, memory: bool = False,
          repeat: int = 1000, log: Optional[pd.Series] = None, cuda_graph: bool = False):
    """Warm up five times, time ``repeat`` calls, record ms per inference (and the peak of intermediate memory) under
    ``log[tag]``; returns the network's output, or None on OOM."""
    try:
        for _ in range(5):
            out = net(*net_params)
        torch.cuda.synchronize()
        offset = torch.cuda.memory_allocated()
        torch.cuda.reset_peak_memory_stats()
        if nvprof:
            torch.cuda.profiler.start()
        elapsed = _timed(lambda: net(*net_params), repeat)
        if nvprof:
            torch.cuda.profiler.stop()
        print(f"{tag} elapsed time: {elapsed} ms/infer")
        if log is not None:
            log.at[(tag, "time")] = elapsed
        if memory:
            peak = (torch.cuda.max_memory_allocated() - offset) / 1048576
            print(f"intermediate data memory usage: {peak} MB")
            if log is not None:
                log.at[(tag, "mem")] = peak
        if cuda_graph:
            replay = capture(net, net_params)
            graphed = _timed(replay, repeat)
            print(f"{tag} replayed from a CUDA graph: {graphed} ms/infer")
            if log is not None and (tag, "time_cuda_graph") in log.index:
                log.at[(tag, "time_cuda_graph")] = graphed
    except torch.cuda.OutOfMemoryError:
        print(f"{tag} OOM")
        return None
    return out


def model(name: str, config: str, device: str = "cuda:0", scale: float = 1.0):
    """(network, parameters) of one example model on one synthetic configuration: a callable running the model's
    layers through this library and the tuple of tensors it takes."""
    gen_dev = device if config == "c5" else "cpu"
    wl = synthetic.make(config, scale=scale, device=gen_dev).to(device)
    pg = layers.PreparedGraph(wl.graph)
    p, hy = wl.params, wl.hyper
    if name == "gcn":
        nrm = layers.gcn_norms(pg)
        ws = [p[k] for k in ("w1", "w2") if k in p] or [p["gcn_w"]]

        def net(x):
            for i, w in enumerate(ws):
                x = layers.gcn_layer(pg, x, w, nrm, nrm, relu=i + 1 < len(ws))
            return x
    elif name == "gat":
        def net(x):
            return layers.gat_layer(pg, x, p["fc_weight"], p["attn_src"], p["attn_dst"], hy["slope"])
    elif name == "rgcn":
        norm = wl.edata["norm"]

        def net(x):
            return layers.rgcn_layer(pg, layers.rgcn_layer(pg, x, p["w1"], norm), p["w2"], norm)
    elif name == "hgt":
        def net(x):
            h = layers.hgt_layer(pg, x, p, int(hy["heads"]), hy["sqrt_dk"])
            return layers.hgt_layer(pg, h, p, int(hy["heads"]), hy["sqrt_dk"])
    else:
        raise ValueError(f"unknown model {name}")
    return net, (wl.feats,)


DEFAULT_CONFIG: Dict[str, str] = {"gat": "c1", "gcn": "c2", "rgcn": "c3", "hgt": "c4"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="gat", choices=list(DEFAULT_CONFIG))
    ap.add_argument("--config", default=None, choices=list(synthetic.MAKERS))
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--repeat", type=int, default=200)
    ap.add_argument("--cuda-graph", action="store_true")
    ap.add_argument("--memory", action="store_true")
    ap.add_argument("--nvprof", action="store_true", help="bracket the timed calls with cudaProfilerStart/Stop")
    a = ap.parse_args()
    config = a.config or DEFAULT_CONFIG[a.model]
    tag = f"{a.model}-{config}"
    log = init_log([tag], ["time", "mem", "time_cuda_graph"])
    net, params = model(a.model, config, scale=a.scale)
    out = bench(net, params, tag=tag, nvprof=a.nvprof, memory=a.memory, repeat=a.repeat, log=log, cuda_graph=a.cuda_graph)
    print(json.dumps({"tag": tag, "output_shape": None if out is None else list(out.shape),
                      **{m: float(log.at[(tag, m)]) for m in ("time", "mem", "time_cuda_graph")}}))


if __name__ == "__main__":
    main()
