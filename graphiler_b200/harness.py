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
    python -m graphiler_b200.harness --model hgt --compiled --graphiler-path <dir holding the reference's graphiler package>
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


def check_equal(first, second, rtol: float = 1e-3, atol: float = 0.0) -> bool:
    """Same contract as the reference's (python/graphiler/utils/bench.py:10-16): skipped when either run hit OOM.
    ``atol`` (the reference has none: its inputs are all positive) admits sums of signed terms that cancel to ~0."""
    if first is None or second is None:
        print("cannot guarantee correctness because of OOM")
        return False
    np.testing.assert_allclose(first.detach().cpu().numpy(), second.detach().cpu().numpy(), rtol=rtol, atol=atol)
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
    if not torch.cuda.is_available():                      # host-only runs (the compiled series on a CPU registration)
        import time
        t0 = time.perf_counter()
        for _ in range(repeat):
            fn()
        return (time.perf_counter() - t0) * 1e3 / repeat
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
        on_gpu = torch.cuda.is_available()
        if on_gpu:
            torch.cuda.synchronize()
            offset = torch.cuda.memory_allocated()
            torch.cuda.reset_peak_memory_stats()
        memory = memory and on_gpu
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


def model(name: str, config: str, device: str = "cuda:0", scale: float = 1.0, single_layer: bool = False):
    """(network, parameters) of one example model on one synthetic configuration: a callable running the model's
    layers through this library and the tuple of tensors it takes.  ``single_layer`` keeps only the first layer of
    the two-layer models (what one ``update_all`` of the compiled series computes)."""
    gen_dev = device if config == "c5" else "cpu"
    wl = synthetic.make(config, scale=scale, device=gen_dev).to(device)
    pg = layers.PreparedGraph(wl.graph)
    p, hy = wl.params, wl.hyper
    if name == "gcn":
        nrm = layers.gcn_norms(pg)
        ws = [p[k] for k in ("w1", "w2") if k in p] or [p["gcn_w"]]
        if single_layer:
            ws = ws[:1]

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
            h = layers.rgcn_layer(pg, x, p["w1"], norm)
            return h if single_layer else layers.rgcn_layer(pg, h, p["w2"], norm)
    elif name == "hgt":
        def net(x):
            h = layers.hgt_layer(pg, x, p, int(hy["heads"]), hy["sqrt_dk"])
            return h if single_layer else layers.hgt_layer(pg, h, p, int(hy["heads"]), hy["sqrt_dk"])
    else:
        raise ValueError(f"unknown model {name}")
    return net, (wl.feats,)


DEFAULT_CONFIG: Dict[str, str] = {"gat": "c1", "gcn": "c2", "rgcn": "c3", "hgt": "c4"}


# ---- the series through the reference's own compiler ----------------------------------------------------------------
# What a Graphiler user who changes nothing gets from this operator library: the model's user-defined functions are
# compiled by the reference's unmodified ``mpdfg_builder`` at optimisation levels 0 / 1 / 2 (the "1+compile",
# "2+reorder", "3+fusion" steps of its breakdown(), examples/GAT/GAT.py:130-164), executed by its ``update_all`` with
# this library installed where its wrapper loads the operator library from ($HOME/.dgl/libgraphiler.so,
# python/graphiler/mpdfg_builder.py:11-14), then once more after this package's additional fusion patterns
# ("4+extra-fusion").  The reference's "0-DGL-UDF" step needs DGL and is not run.  The reference's builder keeps
# static state between builds (src/builder/builder.cpp:3,9-17,344): a model without an update function must not be
# built after one that has one, so one process builds one model, and HGT's three-function build comes last.

COMPILED_TAGS = ["1+compile", "2+reorder", "3+fusion", "4+extra-fusion", "5-layers"]


def load_reference_wrapper(graphiler_path: Optional[str], home: Optional[str] = None, ops_lib: Optional[str] = None):
    """Make the reference's ``graphiler`` package importable and point it at this operator library: HOME becomes a
    scratch directory (or ``home``) whose .dgl/ holds copies of libgraphiler.so and libgphl.so."""
    import os
    import shutil
    import sys
    import tempfile
    from . import capi
    home = home or tempfile.mkdtemp(prefix="gphl_home_")
    os.environ["HOME"] = home
    dgl = os.path.join(home, ".dgl")
    os.makedirs(dgl, exist_ok=True)
    if ops_lib:                                            # another registration of the same operators (tests)
        shutil.copy(str(ops_lib), os.path.join(dgl, "libgraphiler.so"))
    else:
        for lib in (capi.TORCH_OPS_LIB, capi.KERNEL_LIB):
            shutil.copy(str(lib), os.path.join(dgl, os.path.basename(str(lib))))
    if graphiler_path:
        sys.path.insert(0, graphiler_path)
    import contextlib
    import io
    with contextlib.redirect_stdout(io.StringIO()):
        import graphiler                                   # loads $HOME/.dgl/libgraphiler.so
    return graphiler


def compiled_series(name: str, config: str, graphiler_path: Optional[str] = None, device: str = "cuda:0",
                    scale: float = 1.0, repeat: int = 50, memory: bool = True, ops_lib: Optional[str] = None) -> pd.Series:
    """Time one example model through the reference's compiler at every optimisation step (see above) and through
    ``layers.py`` directly; returns the (tag, metric) series the reference's breakdown() returns."""
    import contextlib
    import io
    from types import SimpleNamespace
    graphiler = load_reference_wrapper(graphiler_path, ops_lib=ops_lib)
    from . import compiled_udfs as udf
    from .fusion import extra_fusion
    gen_dev = device if config == "c5" else "cpu"
    wl = synthetic.make(config, scale=scale, device=gen_dev).to(device)
    g, p, hy = wl.graph, wl.params, wl.hyper
    G = torch.classes.my_classes.DGLGraph(g.in_pointer, g.in_node_indices, g.in_edge_indices, g.out_pointer,
                                          g.out_node_indices, g.out_edge_indices, g.COO_src, g.COO_dst, None, None)
    if g.ntype_pointer is not None:
        G.SetNtypePointer(g.ntype_pointer), G.SetNtypeCOO(g.ntype_COO)
    if g.etype_pointer is not None:
        G.SetEtypePointer(g.etype_pointer), G.SetEtypeCOO(g.etype_COO)
    ndata, edata, ntd, etd, msg_params, key = {}, {}, {}, {}, (), "h"
    if name == "gcn":                                      # one layer: projection outside, as examples/GCN/GCN.py:40-47
        w = p["w1"] if "w1" in p else p["gcn_w"]
        norm = g.in_degrees().clamp(min=1).float().pow(-0.5).unsqueeze(1)
        funcs = (udf.gcn_message, udf.gcn_reduce)
        ndata = {"h": torch.mm(wl.feats, w), "norm": norm}
    elif name == "gat":                                    # single head over all H * D columns
        funcs = (udf.gat_message, udf.gat_reduce)
        f = p["fc_weight"].shape[1]
        attn = torch.cat([p["attn_src"].reshape(f, 1), p["attn_dst"].reshape(f, 1)], 0).contiguous()
        ndata, msg_params = {"h": wl.feats}, (p["fc_weight"], attn)
    elif name == "rgcn":
        funcs = (udf.rgcn_message, udf.rgcn_reduce)
        ndata, edata, etd = {"h": wl.feats}, {"norm": wl.edata["norm"]}, {"weight": p["w1"]}
    elif name == "hgt":
        funcs = (udf.hgt_message, udf.hgt_reduce, udf.hgt_update)
        ndata = {"h": wl.feats}
        ntd = {k: p[k] for k in ("k_weight", "v_weight", "q_weight", "a_weight", "skip")}
        etd = {k: p[k] for k in ("relation_att", "relation_msg")}
        etd["relation_pri"] = p["relation_pri"][:, :1].contiguous()       # one head: one prior per relation
        msg_params = (float(hy["sqrt_dk"]),)
    else:
        raise ValueError(f"unknown model {name}")
    log = init_log(COMPILED_TAGS, ["time", "mem"])
    ns = SimpleNamespace(DGLGraph=G, ndata=dict(ndata), edata=edata, ntype_data=ntd, etype_data=etd)

    def run(mpdfg):
        ns.ndata = dict(ndata)
        graphiler.update_all(ns, mpdfg, msg_params=msg_params)
        return ns.ndata[key]

    outs = {}
    with torch.no_grad():
        for tag, level, extra in (("1+compile", 0, False), ("2+reorder", 1, False), ("3+fusion", 2, False),
                                  ("4+extra-fusion", 2, True)):
            with contextlib.redirect_stdout(io.StringIO()):
                mpdfg = graphiler.mpdfg_builder(*funcs, opt_level=level)
                if extra:
                    extra_fusion(mpdfg)
            outs[tag] = bench(run, (mpdfg,), tag=tag, memory=memory, repeat=repeat, log=log)
        if str(device).startswith("cuda"):
            net, params = model(name, config, device=device, scale=scale, single_layer=True)
            bench(net, params, tag="5-layers", memory=memory, repeat=repeat, log=log)
    base = outs.get("3+fusion")
    for tag, out in outs.items():
        if out is not None and base is not None and tag != "3+fusion":
            check_equal(out, base, rtol=1e-3, atol=1e-5)
    return log


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="gat", choices=list(DEFAULT_CONFIG))
    ap.add_argument("--config", default=None, choices=list(synthetic.MAKERS))
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--repeat", type=int, default=200)
    ap.add_argument("--cuda-graph", action="store_true")
    ap.add_argument("--memory", action="store_true")
    ap.add_argument("--nvprof", action="store_true", help="bracket the timed calls with cudaProfilerStart/Stop")
    ap.add_argument("--compiled", action="store_true",
                    help="time the model through the reference's mpdfg_builder + update_all at every optimisation step")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--ops-lib", default=None, help="--compiled: another operator library to install (tests)")
    ap.add_argument("--graphiler-path", default=None,
                    help="directory that holds the reference's `graphiler` Python package (default: already importable)")
    a = ap.parse_args()
    config = a.config or DEFAULT_CONFIG[a.model]
    tag = f"{a.model}-{config}"
    if a.compiled:
        log = compiled_series(a.model, config, a.graphiler_path, device=a.device, scale=a.scale, repeat=a.repeat, memory=True,
                              ops_lib=a.ops_lib)
        print(json.dumps({"model": a.model, "config": config, "scale": a.scale,
                          **{t: {"time_ms": float(log.at[(t, "time")]), "mem_mb": float(log.at[(t, "mem")])}
                             for t in COMPILED_TAGS}}))
        return
    log = init_log([tag], ["time", "mem", "time_cuda_graph"])
    net, params = model(a.model, config, scale=a.scale)
    out = bench(net, params, tag=tag, nvprof=a.nvprof, memory=a.memory, repeat=a.repeat, log=log, cuda_graph=a.cuda_graph)
    print(json.dumps({"tag": tag, "output_shape": None if out is None else list(out.shape),
                      **{m: float(log.at[(tag, m)]) for m in ("time", "mem", "time_cuda_graph")}}))


if __name__ == "__main__":
    main()
