"""Per-kernel timing on the benchmark configurations.

  python -m graphiler_b200.kernel_bench --config c2 --kernel copy_u_sum [--scale S] [--iters K]
                                        [--feat F] [--dtype fp32|bf16] [--chunk C] [--fast]
                                        [--measure] [--sweep NAME=v1,v2,...]

Times one kernel of the library with CUDA events (warm-up, then K launches) on a seeded synthetic
graph of the chosen configuration and prints one JSON line with its time, its algorithmic bytes
(every distinct input element once + every output element once + the index arrays once) and the
resulting GB/s.  It is also the command the profiler captures are taken from.

``--measure`` loads lib/libgphl_measure.so (``python -m graphiler_b200.build --measure``), the build whose tuning
knobs are read from the environment; ``--sweep NAME=v1,v2,...`` then times the kernel once per value of that knob on
the same graph and inputs (one JSON line each, with the largest difference of the output from the first value's).
"""
from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import torch

from . import capi, layers, synthetic

KERNELS = ("linear", "copy_u_sum", "copy_e_sum", "u_mul_e_sum", "u_add_v", "u_dot_v", "u_dot_v_csc", "segment_softmax", "gat_fused",
           "broadcast_src", "segment_mm_node", "segment_mm_edge")


def run(config: str, kernel: str, scale: float, iters: int, warmup: int, feat: int, heads: int, dtype: str,
        chunk: int, fast: bool = False, device: str = "cuda:0", sweep=None):
    gen_dev = device if config == "c5" else "cpu"
    wl = synthetic.make(config, scale=scale, device=gen_dev).to(device)
    g = wl.graph
    pg = layers.PreparedGraph(g, max_feat=max(feat, 256), chunk=chunk)
    n, e = g.num_nodes, g.num_edges
    td = torch.bfloat16 if dtype == "bf16" else torch.float32
    s = 2 if dtype == "bf16" else 4
    gen = torch.Generator(device=device).manual_seed(1)
    x = torch.randn(n, feat, generator=gen, device=device).to(td)
    d = feat // heads
    flops = None
    if kernel == "linear":                      # dense projection (n, feat) @ (feat, feat) with a row-scale epilogue
        w = synthetic.glorot((feat, feat), gen, device)
        sc = torch.rand(n, generator=gen, device=device) + 0.5
        xf = x.float()
        y = torch.empty(n, feat, device=device)
        fn = lambda: capi.linear(xf, w, row_scale=sc, out=y)
        b_alg = 2 * n * feat * 4 + feat * feat * 4 + n * 4
        flops = 2 * n * feat * feat
    elif kernel == "copy_u_sum":
        plan = pg.plan_in(feat)
        fn = lambda: capi.spmm_gather_sum(g.in_pointer, g.in_node_indices, x, plan, fast_accum=fast)
        b_alg = (n + 1) * 4 + e * 4 + 2 * n * feat * s
    elif kernel == "copy_e_sum":
        m = torch.randn(e, feat, generator=gen, device=device)
        plan = pg.plan_in(feat)
        fn = lambda: capi.spmm_gather_sum(g.in_pointer, g.in_edge_indices, m, plan)
        b_alg = (n + 1) * 4 + e * 4 + e * feat * 4 + n * feat * 4
    elif kernel == "u_mul_e_sum":
        w = torch.rand(e, heads, generator=gen, device=device)
        plan = pg.plan_in(feat)
        fn = lambda: capi.spmm_u_mul_e_sum(g.in_pointer, g.in_node_indices, pg.in_eid, x, w, plan)
        b_alg = (n + 1) * 4 + 2 * e * 4 + e * heads * 4 + 2 * n * feat * 4
    elif kernel == "u_add_v":
        l = torch.randn(n, heads, generator=gen, device=device)
        r = torch.randn(n, heads, generator=gen, device=device)
        fn = lambda: capi.sddmm_u_add_v(g.COO_src, g.COO_dst, l, r)
        b_alg = 2 * e * 8 + 2 * n * heads * 4 + e * heads * 4
    elif kernel == "u_dot_v":
        r = torch.randn(n, feat, generator=gen, device=device)
        fn = lambda: capi.sddmm_u_dot_v(pg.COO_src32, pg.COO_dst32, x, r, heads)
        b_alg = 2 * e * 4 + 2 * n * feat * 4 + e * heads * 4
    elif kernel == "u_dot_v_csc":               # the same dot products walked in destination-row order
        r = torch.randn(n, feat, generator=gen, device=device)
        plan = pg.plan_in(feat)
        z = torch.empty(e, heads, device=device)
        fn = lambda: capi.sddmm_u_dot_v_csc(g.in_pointer, g.in_node_indices, g.in_edge_indices, x, r, heads, plan, out=z)
        b_alg = (n + 1) * 4 + 2 * e * 4 + 2 * n * feat * 4 + e * heads * 4
    elif kernel == "segment_softmax":
        lg = torch.randn(e, heads, generator=gen, device=device)
        plan = pg.plan_in(feat)
        y = torch.empty_like(lg)
        st = torch.empty(2 * n * heads, device=device)
        fn = lambda: capi.segment_softmax(g.in_pointer, pg.in_eid, lg, plan, out=y, stats=st)
        b_alg = (n + 1) * 4 + e * 4 + 2 * e * heads * 4
    elif kernel == "gat_fused":
        el = torch.randn(n, heads, generator=gen, device=device)
        er = torch.randn(n, heads, generator=gen, device=device)
        plan = pg.plan_in(feat)
        st = torch.empty(2 * n * heads, device=device)
        fn = lambda: capi.gat_fused(g.in_pointer, g.in_node_indices, pg.in_eid, el, er, x, 0.2, plan, stats=st,
                                    fast_accum=fast)
        b_alg = (n + 1) * 4 + e * 4 + 2 * n * heads * 4 + 2 * n * feat * s
    elif kernel == "broadcast_src":
        fn = lambda: capi.gather_rows(g.COO_src, x)
        b_alg = e * 8 + n * feat * s + e * feat * s
    elif kernel in ("segment_mm_node", "segment_mm_edge"):
        node = kernel.endswith("node")
        ptr = g.ntype_pointer if node else g.etype_pointer
        if ptr is None:
            raise SystemExit(f"{config} has no type pointer for {kernel}")
        t = ptr.numel() - 1
        w = synthetic.glorot((t, feat, feat), gen, device)
        m = n if node else e
        gi = None if node else g.COO_src
        fn = lambda: capi.segment_mm(x, w, ptr, gather_idx=gi)
        b_alg = (n if not node else m) * feat * 4 + t * feat * feat * 4 + m * feat * 4 + (0 if node else e * 8)
        flops = 2 * m * feat * feat
    else:
        raise SystemExit(f"unknown kernel {kernel}")

    def timed():
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.profiler.start()           # a profiler started with --profile-from-start off sees only these launches
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        ms = a.elapsed_time(b) / iters
        out = {"config": config, "kernel": kernel, "scale": scale, "nodes": n, "edges": e, "feat": feat, "heads": heads,
               "dtype": dtype, "chunk": chunk, "fast_accum": fast, "ms": ms, "algorithmic_bytes": b_alg,
               "gbs": b_alg / ms / 1e6, "split_rows": pg.plan_in(feat).num_split_rows, "items": pg.plan_in(feat).num_items}
        if flops:
            out["tflops"] = flops / ms / 1e9
        return out

    if not sweep:
        return [timed()]
    name, values = sweep
    outs, first = [], None
    for v in values:
        os.environ[name] = v
        res = fn()
        res = res[0] if isinstance(res, tuple) else res
        o = timed()
        o["knob"] = {name: v}
        if torch.is_tensor(res):
            if first is None:
                first = res.float().clone()
            o["max_abs_diff_from_first"] = float((res.float() - first).abs().max())
        outs.append(o)
    os.environ.pop(name, None)
    return outs


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="c2", choices=list(synthetic.MAKERS))
    ap.add_argument("--kernel", default="copy_u_sum", choices=KERNELS)
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--feat", type=int, default=256)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--dtype", default="fp32", choices=["fp32", "bf16"])
    ap.add_argument("--chunk", type=int, default=capi.DEFAULT_CHUNK)
    ap.add_argument("--fast", action="store_true", help="plain fp32 accumulation instead of compensated")
    ap.add_argument("--measure", action="store_true", help="load the measurement build of the kernel library")
    ap.add_argument("--sweep", default=None, help="NAME=v1,v2,...: one timing per value of a tuning knob (needs --measure)")
    a = ap.parse_args()
    if a.measure:
        capi.load_library(Path(capi.KERNEL_LIB).with_name("libgphl_measure.so"), make_default=True)
    sweep = None
    if a.sweep:
        if not a.measure:
            raise SystemExit("--sweep needs --measure")
        name, vals = a.sweep.split("=", 1)
        sweep = (name, vals.split(","))
    for o in run(a.config, a.kernel, a.scale, a.iters, a.warmup, a.feat, a.heads, a.dtype, a.chunk, a.fast, sweep=sweep):
        print(json.dumps(o), flush=True)


if __name__ == "__main__":
    main()
