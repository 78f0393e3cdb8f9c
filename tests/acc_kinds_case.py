"""One pass over the gather operators with the accumulator kind forced by GPHL_ACC (1 two-sum fp32, 2 double,
3 alternating), through the measurement build of the kernel library (lib/libgphl_measure.so: the product library
compiles the choice in), also over the column-sliced kernels (GPHL_SLICE_LPR).  A script for a child process:
    GPHL_ACC=1|2|3 [GPHL_SLICE_LPR=8|16|32] python tests/acc_kinds_case.py   -> prints OK or raises."""
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

from graphiler_b200 import capi, synthetic  # noqa: E402
from oracle import ops_oracle as O  # noqa: E402

capi.load_library(Path(capi.KERNEL_LIB).with_name("libgphl_measure.so"), make_default=True)
DEV = "cuda:0"
wl = synthetic.make_c5(scale=0.002)
g, gd = wl.graph, wl.graph.to(DEV)
gen = torch.Generator().manual_seed(3)
for feat, heads in ((256, 8), (128, 4), (64, 1)):
    plan = capi.Plan(gd.in_pointer, feat, chunk=64)            # chunk 64: hub rows are cut, pieces merged from scratch
    x = torch.randn(g.num_nodes, feat, generator=gen)
    w = torch.randn(g.num_edges, heads, generator=gen)
    el, er = torch.randn(g.num_nodes, heads, generator=gen), torch.randn(g.num_nodes, heads, generator=gen)
    xd = x.to(DEV)
    checks = {
        "copy_u_sum": (capi.spmm_gather_sum(gd.in_pointer, gd.in_node_indices, xd, plan),
                       O.spmm_src(x, g.in_pointer, g.in_node_indices)),
        "u_mul_e_sum": (capi.spmm_u_mul_e_sum(gd.in_pointer, gd.in_node_indices, gd.in_edge_indices, xd, w.to(DEV), plan),
                        O.u_mul_e_sum(x, w, g.in_pointer, g.in_node_indices, g.in_edge_indices)),
        "gat_fused": (capi.gat_fused(gd.in_pointer, gd.in_node_indices, gd.in_edge_indices, el.to(DEV), er.to(DEV), xd, 0.2,
                                     plan),
                      O.gat_fused(el, er, x, 0.2, g.in_pointer, g.in_node_indices, g.in_edge_indices)),
        "copy_u_sum_bf16": (capi.spmm_gather_sum(gd.in_pointer, gd.in_node_indices, xd.bfloat16(), plan).float(),
                            None),
    }
    for name, (got, truth) in checks.items():
        if truth is None:      # bf16 storage: fp32-exact sum of the rounded inputs, rounded once to bf16
            truth = O.spmm_src(x.bfloat16().float(), g.in_pointer, g.in_node_indices)
            ok, bad, err = O.within_tolerance(got.cpu().numpy(), truth, rtol=2.0 ** -8, atol=1e-6)
        else:
            ok, bad, err = O.within_tolerance(got.cpu().numpy(), truth)
        assert ok, f"{name} F={feat}: {bad} elements outside tolerance (max abs err {err:.3e})"
print("OK")
