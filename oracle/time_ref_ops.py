"""TEST / MEASUREMENT INFRASTRUCTURE: device times of the reference's own CUDA operators on this machine.

    python oracle/time_ref_ops.py [--scale S] [--iters K]

Loads oracle/_ref/libgraphiler_ref.so (the reference's operator sources, unmodified, compiled for sm_100 by
oracle/build_ref_cuda.py) in this process, which must therefore not load the product's operator library (both
register `my_classes.DGLGraph` and `my_ops::*`), builds the synthetic scale-sweep graph with the package's pure-Python
generators and times, with CUDA events after warm-up, the operators the bench's layers are made of at the shapes the
reference supports:

  SpMMSrc (copy_u_sum through cuSPARSE, src/ops/dgl_primitives/spmm.cu:50-104,375-389) at F = 256,
  gspmm_src_mul_e_sum at F = 64 with one weight per edge (spmm.cu:192-356 computes only the first 64 columns),
  SegmentSoftmax on (E, 1) logits (src/ops/segment_softmax/segment_softmax_kernel.cu:4-49),
  gsddmm_u_add_v_mul_alpha at F = 8 (src/ops/dgl_primitives/sddmm.cuh:34-71), BroadcastSrcNode at F = 64.

Prints one JSON line.  bench.py runs it as a child process in its baseline leg and reports the numbers beside the
CPU baseline; nothing of the product imports it.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args()
    so = ROOT / "oracle" / "_ref" / "libgraphiler_ref.so"
    if not so.exists() or not torch.cuda.is_available():
        print(json.dumps({"unavailable": "needs oracle/_ref/libgraphiler_ref.so and a CUDA device"}))
        return 0
    torch.classes.load_library(str(so))
    torch.ops.load_library(str(so))
    from graphiler_b200 import synthetic
    dev = torch.device("cuda:0")
    wl = synthetic.make_c5(scale=a.scale, device=dev, with_params=False)
    g = wl.graph
    n, e = g.num_nodes, g.num_edges
    G = torch.classes.my_classes.DGLGraph(g.in_pointer, g.in_node_indices, g.in_edge_indices, g.out_pointer,
                                          g.out_node_indices, g.out_edge_indices, g.COO_src, g.COO_dst, None, None)
    o = torch.ops.my_ops
    gen = torch.Generator(device=dev).manual_seed(11)
    x256 = torch.randn(n, 256, device=dev, generator=gen)
    x64 = torch.randn(n, 64, device=dev, generator=gen)
    x8a, x8b = torch.randn(n, 8, device=dev, generator=gen), torch.randn(n, 8, device=dev, generator=gen)
    w = torch.rand(e, 1, device=dev, generator=gen)
    z = torch.randn(e, 1, device=dev, generator=gen).abs()          # the reference's softmax clamps its maximum at 0
    cases = {
        "SpMMSrc_f256": lambda: o.SpMMSrc(x256, [1], False, None, G),
        "gspmm_src_mul_e_sum_f64": lambda: o.gspmm_src_mul_e_sum(x64, w, [1], False, None, G),
        "SegmentSoftmax_h1": lambda: o.SegmentSoftmax(z, 1, None, G),
        "gsddmm_u_add_v_f8": lambda: o.gsddmm_u_add_v_mul_alpha(x8a, x8b, 1, G),
        "BroadcastSrcNode_f64": lambda: o.BroadcastSrcNode(x64, G),
    }
    res = {"gpu": torch.cuda.get_device_name(0), "nodes": n, "edges": e, "unit": "ms", "library": so.name}
    for name, fn in cases.items():
        try:
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(a.iters):
                fn()
            t1.record()
            torch.cuda.synchronize()
            res[name] = t0.elapsed_time(t1) / a.iters
        except Exception as ex:  # noqa: BLE001
            res[name] = f"failed: {repr(ex)[:120]}"
    print(json.dumps(res))
    return 0


if __name__ == "__main__":
    sys.exit(main())
