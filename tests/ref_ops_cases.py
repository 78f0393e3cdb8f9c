"""Seeded cases on which the reference's own CUDA operators were run to pin the CPU oracle.

Shared by tests/golden/make_ref_ops_golden.py (which executes the reference's operator library on a GPU
and records its outputs), by the CPU test that checks oracle/ops_oracle.py against those outputs and by the
GPU test that checks this package's kernels against them.  Inputs are regenerated from seeds (the CPU
generator of torch is deterministic across machines); the fixture stores the outputs and a checksum of
every input.

Only shapes the reference supports are listed: one scalar weight per edge and at most 64 feature columns
for the edge-weighted sums (src/ops/dgl_primitives/spmm.cu:286-356 computes only the first 64 or 32
columns of wider rows), one logit per edge for the softmax (src/ops/segment_softmax/segment_softmax.cu:13-22),
two-dimensional inputs for the sums.  The segment sum over edge rows (SpMMEdge) is listed only on a graph
with no more edges than nodes, where the matrix size the reference declares to cuSPARSE
(src/ops/dgl_primitives/spmm.cu:369-371) covers every row it reads.
"""
from __future__ import annotations

import zlib

import numpy as np
import torch

from fixtures_common import hetero_graphs, homo_graphs
from graphiler_b200.graph import prepare_graph


def hub_graph(n=300, e=1000, hub=200, seed=21):
    """Random graph with one destination of `hub` in-edges and one source of `hub` out-edges, so that the
    32-wide batches, the remainders and a row longer than one batch are all exercised."""
    g = torch.Generator().manual_seed(seed)
    src = torch.cat([torch.randint(0, n, (e,), generator=g), torch.randint(0, n, (hub,), generator=g),
                     torch.full((hub,), 5, dtype=torch.int64), torch.arange(n)])
    dst = torch.cat([torch.randint(0, n, (e,), generator=g), torch.full((hub,), 3, dtype=torch.int64),
                     torch.randint(0, n, (hub,), generator=g), torch.arange(n)])
    perm = torch.randperm(src.numel(), generator=g)          # edge ids not sorted by destination
    return prepare_graph(src[perm], dst[perm], n)


def sparse_graph(n=120, e=90, seed=22):
    g = torch.Generator().manual_seed(seed)
    return prepare_graph(torch.randint(0, n, (e,), generator=g), torch.randint(0, n, (e,), generator=g), n)


def graphs():
    gs = dict(homo_graphs())
    gs["hub"] = hub_graph()
    gs["sparse"] = sparse_graph()
    gs.update(hetero_graphs())
    return gs


def _rn(seed, *shape, scale=1.0):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale).contiguous()


def cases():
    """Yield (case name, graph name, operator name, dict of input tensors)."""
    gs = graphs()
    out = []
    seed = 1000
    for gname, g in gs.items():
        n, e = g.num_nodes, g.num_edges
        hetero = g.ntype_pointer is not None
        for f in (1, 16, 64, 100):
            seed += 1
            out.append((f"SpMMSrc_{gname}_f{f}", gname, "SpMMSrc", {"x": _rn(seed, n, f)}))
        if e <= n:
            for f in (8, 64):
                seed += 1
                out.append((f"SpMMEdge_{gname}_f{f}", gname, "SpMMEdge", {"x": _rn(seed, e, f)}))
        for f in (8, 16, 32, 48, 64):
            for op in ("gspmm_src_mul_e_sum", "gspmm_dst_mul_e_sum"):
                seed += 1
                out.append((f"{op}_{gname}_f{f}", gname, op, {"x": _rn(seed, n, f), "w": _rn(seed + 5000, e, 1)}))
        for shape in ((e, 1), (e,)):
            seed += 1
            out.append((f"SegmentSoftmax_{gname}_{len(shape)}d", gname, "SegmentSoftmax", {"x": _rn(seed, *shape, scale=3.0)}))
        for f in (1, 8, 24):
            seed += 1
            out.append((f"gsddmm_u_add_v_mul_alpha_{gname}_f{f}", gname, "gsddmm_u_add_v_mul_alpha",
                        {"l": _rn(seed, n, f), "r": _rn(seed + 5000, n, f)}))
        for op in ("BroadcastSrcNode", "BroadcastDstNode"):
            seed += 1
            out.append((f"{op}_{gname}_f32", gname, op, {"x": _rn(seed, n, 12)}))
            out.append((f"{op}_{gname}_3d", gname, op, {"x": _rn(seed + 1, n, 3, 4)}))
            out.append((f"{op}_{gname}_i64", gname, op,
                        {"x": torch.randint(-9, 9, (n, 2), generator=torch.Generator().manual_seed(seed))}))
        if hetero:
            tn, te = g.num_ntypes, g.num_etypes
            for op, rows in (("BroadcastNodeType", tn), ("BroadcastSrcNodeType", tn), ("BroadcastDstNodeType", tn),
                             ("BroadcastEdgeType", te)):
                seed += 1
                out.append((f"{op}_{gname}_f32", gname, op, {"x": _rn(seed, rows, 6)}))
                out.append((f"{op}_{gname}_3d", gname, op, {"x": _rn(seed + 1, rows, 4, 4)}))
            for k, m in ((16, 16), (24, 40), (64, 48)):
                seed += 1
                out.append((f"SegmentMMNode_{gname}_k{k}n{m}", gname, "SegmentMMNode",
                            {"x": _rn(seed, n, k), "w": _rn(seed + 5000, tn, k, m, scale=0.3)}))
                out.append((f"SegmentMMEdge_{gname}_k{k}n{m}", gname, "SegmentMMEdge",
                            {"x": _rn(seed + 1, e, k), "w": _rn(seed + 5001, te, k, m, scale=0.3)}))
    return out


def input_checksum(inputs: dict) -> int:
    c = 0
    for k in sorted(inputs):
        c = zlib.crc32(inputs[k].numpy().tobytes(), c)
    return c


# ---- oracle evaluation of one case, with the float32 error bound of a plain summation -------------------

def oracle_eval(op, g, inp):
    """Return (truth in float64 or exact dtype, bound) where bound is None for operators that must match
    bit for bit and otherwise the element-wise allowance for a float32 implementation of the same sum:
    1e-6 + 1e-5 |truth| + 2^-23 * terms * sum |term|."""
    from oracle import ops_oracle as O
    eps = 2.0 ** -23
    if op == "SpMMSrc":
        t = O.spmm_src(inp["x"], g.in_pointer, g.in_node_indices)
        a = O.spmm_src(inp["x"].abs(), g.in_pointer, g.in_node_indices)
        d = g.in_degrees().numpy()[:, None]
        return t, 1e-6 + 1e-5 * np.abs(t) + eps * d * a
    if op == "SpMMEdge":
        t = O.spmm_edge(inp["x"], g.in_pointer, g.in_edge_indices)
        a = O.spmm_edge(inp["x"].abs(), g.in_pointer, g.in_edge_indices)
        d = g.in_degrees().numpy()[:, None]
        return t, 1e-6 + 1e-5 * np.abs(t) + eps * d * a
    if op in ("gspmm_src_mul_e_sum", "gspmm_dst_mul_e_sum"):
        if op == "gspmm_src_mul_e_sum":
            arrs, d = (g.in_pointer, g.in_node_indices, g.in_edge_indices), g.in_degrees()
        else:
            arrs, d = (g.out_pointer, g.out_node_indices, g.out_edge_indices), g.out_degrees()
        t = O.u_mul_e_sum(inp["x"], inp["w"], *arrs)
        a = O.u_mul_e_sum(inp["x"].abs(), inp["w"].abs(), *arrs)
        return t, 1e-6 + 1e-5 * np.abs(t) + eps * (d.numpy()[:, None] + 1) * a
    if op == "SegmentSoftmax":
        t = O.segment_softmax(inp["x"], g.in_pointer, g.in_edge_indices)
        # expf and the division are each good to a few ulp; the sum of positive terms adds degree * 2^-24 relative
        dmax = float(g.in_degrees().max()) if g.num_nodes else 0.0
        return t, 1e-6 + (1e-5 + eps * (dmax + 8)) * np.abs(t)
    if op == "gsddmm_u_add_v_mul_alpha":
        return O.sddmm_u_add_v(inp["l"], inp["r"], g.COO_src, g.COO_dst).astype(np.float32), None
    if op == "BroadcastSrcNode":
        return O.broadcast_src_node(inp["x"], g.COO_src), None
    if op == "BroadcastDstNode":
        return O.broadcast_dst_node(inp["x"], g.COO_dst), None
    if op == "BroadcastNodeType":
        return O.broadcast_node_type(inp["x"], g.ntype_COO), None
    if op == "BroadcastEdgeType":
        return O.broadcast_edge_type(inp["x"], g.etype_COO), None
    if op == "BroadcastSrcNodeType":
        return O.broadcast_src_node_type(inp["x"], g.ntype_COO, g.COO_src), None
    if op == "BroadcastDstNodeType":
        return O.broadcast_dst_node_type(inp["x"], g.ntype_COO, g.COO_dst), None
    if op in ("SegmentMMNode", "SegmentMMEdge"):
        ptr = g.ntype_pointer if op == "SegmentMMNode" else g.etype_pointer
        t = O.segment_mm(inp["x"], inp["w"], ptr)
        a = O.segment_mm(inp["x"].abs(), inp["w"].abs(), ptr)
        k = inp["x"].shape[1]
        # at::mm may use TF32-free fp32 FMA chains: K terms
        return t, 1e-6 + 1e-5 * np.abs(t) + eps * (k + 1) * a
    raise KeyError(op)
