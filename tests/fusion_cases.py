"""Cases for graphiler_b200.fusion on hand-written TorchScript graphs.  Test helper, run as a script in a child process
(an operator library registers global TorchScript state, one library per process):

    python tests/fusion_cases.py --lib <operator library> --device cpu|cuda

Each case scripts a small function over my_ops operators, runs it, applies ``extra_fusion``, checks which targets
were emitted (none where a bypassed intermediate has a second reader or the constants do not fit) and that the
rewritten function returns the same values.  Prints one JSON report.
"""
import argparse
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
ap = argparse.ArgumentParser()
ap.add_argument("--lib", required=True)
ap.add_argument("--device", default="cpu")
args = ap.parse_args()
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import torch  # noqa: E402

torch.classes.load_library(args.lib)
torch.ops.load_library(args.lib)

from fixtures_common import hetero_graphs  # noqa: E402
from graphiler_b200.fusion import extra_fusion  # noqa: E402

G = torch.classes.my_classes.DGLGraph


def u_dot_v_case(g: G, a: torch.Tensor, b: torch.Tensor):
    s = torch.ops.my_ops.BroadcastSrcNode(a, g)
    d = torch.ops.my_ops.BroadcastDstNode(b, g)
    return torch.sum(d * s, [1], True)


def u_dot_v_three_dims(g: G, a: torch.Tensor, b: torch.Tensor):        # (N, H, D) operands: the sum runs over H only
    s = torch.ops.my_ops.BroadcastSrcNode(a, g)
    d = torch.ops.my_ops.BroadcastDstNode(b, g)
    return torch.sum(s * d, [1], True)


def u_dot_v_broadcast_width(g: G, a: torch.Tensor, b: torch.Tensor):   # (N, F) x (N, 1)
    s = torch.ops.my_ops.BroadcastSrcNode(a, g)
    d = torch.ops.my_ops.BroadcastDstNode(b, g)
    return torch.sum(s * d, [1], True)


def dot_without_keepdim(g: G, a: torch.Tensor, b: torch.Tensor):
    s = torch.ops.my_ops.BroadcastSrcNode(a, g)
    d = torch.ops.my_ops.BroadcastDstNode(b, g)
    return torch.sum(s * d, [1], False)


def dot_with_second_reader(g: G, a: torch.Tensor, b: torch.Tensor):
    s = torch.ops.my_ops.BroadcastSrcNode(a, g)
    d = torch.ops.my_ops.BroadcastDstNode(b, g)
    t = s * d
    return torch.sum(t, [1], True) + torch.sum(t)


def attention_relu(g: G, l: torch.Tensor, r: torch.Tensor, z: torch.Tensor):
    e = torch.relu(torch.ops.my_ops.gsddmm_u_add_v_mul_alpha(l, r, 1, g))
    a = torch.ops.my_ops.SegmentSoftmax(e, 1, None, g)
    return torch.ops.my_ops.gspmm_src_mul_e_sum(z, a, [1], False, None, g)


def attention_heads(g: G, l: torch.Tensor, r: torch.Tensor, z: torch.Tensor):
    e = torch.ops.aten.leaky_relu(torch.ops.my_ops.gsddmm_u_add_v_mul_alpha(l, r, 1, g), 0.2)
    a = torch.ops.my_ops.SegmentSoftmax(e, 1, None, g)
    return torch.ops.my_ops.gspmm_src_mul_e_sum(z, a, [1], False, None, g)


def attention_weights_also_returned(g: G, l: torch.Tensor, r: torch.Tensor, z: torch.Tensor):
    e = torch.ops.aten.leaky_relu(torch.ops.my_ops.gsddmm_u_add_v_mul_alpha(l, r, 1, g), 0.2)
    a = torch.ops.my_ops.SegmentSoftmax(e, 1, None, g)
    return torch.ops.my_ops.gspmm_src_mul_e_sum(z, a, [1], False, None, g), a


def weighted_sum_same_width(g: G, m: torch.Tensor, w: torch.Tensor):
    return torch.ops.my_ops.SpMMEdge(m * w, [1], False, None, g)


def weighted_sum_column_left(g: G, w: torch.Tensor, m: torch.Tensor):
    return torch.ops.my_ops.SpMMEdge(w * m, [1], False, None, g)


def weighted_sum_column_right(g: G, w: torch.Tensor, m: torch.Tensor):
    return torch.ops.my_ops.SpMMEdge(m * w, [1], False, None, g)


def gathered_linear_with_second_reader(g: G, x: torch.Tensor, w: torch.Tensor):
    s = torch.ops.my_ops.BroadcastSrcNode(x, g)
    return torch.ops.my_ops.SegmentMMEdge(s, w, g), s


def as_list(out):
    return list(out) if isinstance(out, tuple) else [out]


def main():
    dev = args.device
    arrays = hetero_graphs()["rand_hetero"].to(dev)
    g = G(arrays.in_pointer, arrays.in_node_indices, arrays.in_edge_indices, arrays.out_pointer, arrays.out_node_indices,
          arrays.out_edge_indices, arrays.COO_src, arrays.COO_dst, None, None)
    g.SetEtypePointer(arrays.etype_pointer)
    g.SetEtypeCOO(arrays.etype_COO)
    n, e, te = arrays.num_nodes, arrays.num_edges, arrays.num_etypes
    gen = torch.Generator().manual_seed(7)
    rn = lambda *s: torch.randn(*s, generator=gen).to(dev)
    cases = [
        ("u_dot_v", u_dot_v_case, (rn(n, 16), rn(n, 16)), {"gsddmm_u_dot_v": 1}),
        # shapes the fused kernel does not cover: the operator must return what the unfused chain returned
        ("u_dot_v_three_dims", u_dot_v_three_dims, (rn(n, 2, 8), rn(n, 2, 8)), {"gsddmm_u_dot_v": 1}),
        ("u_dot_v_broadcast_width", u_dot_v_broadcast_width, (rn(n, 16), rn(n, 1)), {"gsddmm_u_dot_v": 1}),
        ("dot_without_keepdim", dot_without_keepdim, (rn(n, 16), rn(n, 16)), {}),
        ("dot_with_second_reader", dot_with_second_reader, (rn(n, 16), rn(n, 16)), {}),
        ("attention_relu", attention_relu, (rn(n, 1), rn(n, 1), rn(n, 16)), {"gat_fused": 1}),
        ("attention_heads", attention_heads, (rn(n, 4), rn(n, 4), rn(n, 32)), {"gat_fused": 1}),
        ("attention_weights_also_returned", attention_weights_also_returned, (rn(n, 4), rn(n, 4), rn(n, 32)), {}),
        ("weighted_sum_same_width", weighted_sum_same_width, (rn(e, 8), rn(e, 8)), {"SpMMEdgeMul": 1}),
        ("weighted_sum_column_left", weighted_sum_column_left, (rn(e, 1), rn(e, 32)), {"SpMMEdgeMul": 1}),
        ("weighted_sum_column_right", weighted_sum_column_right, (rn(e, 1), rn(e, 20)), {"SpMMEdgeMul": 1}),
        ("gathered_linear_with_second_reader", gathered_linear_with_second_reader, (rn(n, 16), rn(te, 16, 8)),
         {"SegmentMMEdgeSrc": 1}),
    ]
    report = {}
    for name, fn, inputs, want in cases:
        before = [t.detach().cpu() for t in as_list(fn(g, *inputs))]      # eager: operator by operator
        scripted = torch.jit.script(fn)
        counts = extra_fusion(scripted)                                   # before the first run fixes an execution plan
        after = [t.detach().cpu() for t in as_list(scripted(g, *inputs))]
        emitted = {k: v for k, v in counts.items() if v}
        diff = max(float((a - b).abs().max()) if a.numel() else 0.0 for a, b in zip(before, after))
        scale = max(float(b.abs().max()) if b.numel() else 0.0 for b in before)
        report[name] = {"emitted": emitted, "expected": want, "max_abs_diff": diff, "scale": scale,
                        "shapes_equal": all(a.shape == b.shape for a, b in zip(before, after))}
    print("REPORT " + json.dumps(report))


main()
