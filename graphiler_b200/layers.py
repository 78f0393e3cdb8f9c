"""Layer forwards of the four example models, written against the kernel library.

Each function runs the operator sequence that the reference's optimised MP-DFG executes for
that model (python/graphiler/mpdfg_optimizer.py:4-16 applied to examples/GAT/GAT.py:25-36,
GCN/GCN.py:21-27, RGCN/RGCN.py:25-33, HGT/HGT.py:28-60), with the further fusions this
library adds: one fused attention operator for GAT; for RGCN / HGT the node->edge broadcast folded
into the edge-typed linear, which is evaluated once per distinct (relation, source) pair instead of
once per edge, the ``mul`` folded into the segment sum, and a direct row-order u_dot_v for HGT.  The GCN projection runs on this library's tensor-core kernel (fp32 accuracy, source scaling in the epilogue); the
other dense projections are plain ``torch.mm`` (cuBLAS), as in the reference.

``PreparedGraph`` is the host-side graph handle: device arrays in the reference's DGLGraph
layout plus cached row-split plans.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from . import capi
from .graph import GraphArrays


class PreparedGraph:
    def __init__(self, arrays: GraphArrays, max_feat: int = 256, chunk: int = capi.DEFAULT_CHUNK, validate: bool = True):
        if not arrays.in_pointer.is_cuda:
            raise capi.GphlError("PreparedGraph needs device arrays: call GraphArrays.to('cuda') first")
        if validate:
            # the kernels trust these arrays: check them once, here (one pass on the device), as the TorchScript
            # DGLGraph does in its constructor
            n, e = arrays.num_nodes, arrays.num_edges
            capi.validate_csr(arrays.in_pointer, arrays.in_node_indices, n, arrays.in_edge_indices, e)
            capi.validate_csr(arrays.out_pointer, arrays.out_node_indices, n, arrays.out_edge_indices, e)
            capi.validate_index(arrays.COO_src, n)
            capi.validate_index(arrays.COO_dst, n)
        self.g = arrays
        self.chunk = chunk
        self._max_feat = max_feat
        self._plan_in: Optional[capi.Plan] = None
        self._plan_out: Optional[capi.Plan] = None
        e = arrays.num_edges
        ar = torch.arange(e, dtype=torch.int32, device=arrays.device)
        # edge ids of a destination-sorted edge list equal their CSC positions: skip the indirection
        self.eid_is_position = bool(e == 0 or torch.equal(arrays.in_edge_indices, ar))
        self._arange_e = ar
        self.COO_src32 = arrays.COO_src.to(torch.int32)
        self.COO_dst32 = arrays.COO_dst.to(torch.int32)

    @property
    def device(self):
        return self.g.device

    def plan_in(self, feat: int) -> capi.Plan:
        if self._plan_in is None or feat > self._max_feat:
            self._max_feat = max(self._max_feat, feat)
            self._plan_in = capi.Plan(self.g.in_pointer, self._max_feat, self.chunk)
        return self._plan_in

    def plan_out(self, feat: int) -> capi.Plan:
        if self._plan_out is None or feat > self._max_feat:
            self._max_feat = max(self._max_feat, feat)
            self._plan_out = capi.Plan(self.g.out_pointer, self._max_feat, self.chunk)
        return self._plan_out

    @property
    def in_eid(self):
        return None if self.eid_is_position else self.g.in_edge_indices

    def source_relation_pairs(self):
        """The distinct (edge type, source node) pairs of a typed graph, grouped by edge type: an edge-typed linear
        applied to gathered source rows gives the same row for every edge of one pair, so it is computed once per
        pair (the reference's optimizer removes such repeats on the node side with its dedup pass,
        src/optimizer/dedup.cpp; this is the same idea for the (node, relation) side).  Returns (pair_src int64 (P),
        pair_type_pointer int32 (T + 1), pair row of every CSC position int32 (E)); built once per graph."""
        if getattr(self, "_pairs", None) is None:
            g = self.g
            n, t = g.num_nodes, g.num_etypes
            key = g.etype_COO.to(torch.int64) * n + g.COO_src.to(torch.int64)
            uniq, inverse = torch.unique(key, return_inverse=True)             # ascending: by type, then by node id
            pair_type = torch.div(uniq, n, rounding_mode="floor")
            ptr = torch.searchsorted(pair_type, torch.arange(t + 1, device=key.device, dtype=torch.int64)).to(torch.int32)
            pos_pair = inverse[g.in_edge_indices.to(torch.int64)].to(torch.int32).contiguous()
            self._pairs = ((uniq - pair_type * n).contiguous(), ptr.contiguous(), pos_pair)
        return self._pairs


def gcn_norms(pg: PreparedGraph):
    """(in-degree clamped at 1)^-1/2 as an (N,1) column (examples/GCN/GCN.py:22,55)."""
    deg = pg.g.in_degrees().clamp(min=1).to(torch.float32)
    return deg.pow(-0.5).unsqueeze(1)


def project(feature, weight, row_scale=None, out=None, fan=None):
    """Dense projection ``row_scale * (feature @ weight)``: the tensor-core kernel when the shape allows (the source
    scaling then rides in its epilogue), cuBLAS otherwise.  ``fan`` (a ``capi.FanOut``): the finished rows are also
    stored into the receivers' buffers from the kernel's epilogue, and ``out`` may then be None."""
    if fan is not None:
        return capi.linear_fanout(feature, weight, fan, row_scale=None if row_scale is None else row_scale.reshape(-1), out=out)
    if feature.shape[1] % 4 == 0 and feature.is_contiguous() and weight.is_contiguous():
        return capi.linear(feature, weight, row_scale=None if row_scale is None else row_scale.reshape(-1), out=out)
    h = torch.mm(feature, weight, out=out) if out is not None else torch.mm(feature, weight)
    return h if row_scale is None else h.mul_(row_scale.reshape(-1, 1))


def gcn_layer(pg: PreparedGraph, feature, weight, norm_src, norm_dst=None, relu: bool = True):
    h = project(feature, weight, norm_src)
    scale = None if norm_dst is None else norm_dst.reshape(-1)
    # destination scaling and relu ride in the aggregation kernel's epilogue
    return capi.spmm_gather_sum(pg.g.in_pointer, pg.g.in_node_indices, h, pg.plan_in(h.shape[1]), dst_scale=scale,
                                relu=relu)


def gat_projections(feature, fc_weight, attn_src, attn_dst):
    """z = h W, el[n,h] = sum_d z[n,h,d] a_src[h,d], er likewise (per-head form of the reference's
    ``mm(cat(z_s, z_d), attn_weight)`` after the optimizer's split pass)."""
    heads, dim = attn_src.shape
    z = project(feature, fc_weight)
    el, er = capi.gat_head_scores(z, attn_src.contiguous(), attn_dst.contiguous())
    return z, el, er


def gat_layer(pg: PreparedGraph, feature, fc_weight, attn_src, attn_dst, slope: float, fused: bool = True):
    z, el, er = gat_projections(feature, fc_weight, attn_src, attn_dst)
    g = pg.g
    plan = pg.plan_in(z.shape[1])
    if fused:
        return capi.gat_fused(g.in_pointer, g.in_node_indices, pg.in_eid, el, er, z, slope, plan)
    e = capi.sddmm_u_add_v(g.COO_src, g.COO_dst, el, er)
    e = torch.nn.functional.leaky_relu_(e, slope)
    a = capi.segment_softmax(g.in_pointer, pg.in_eid, e, plan)         # None: edge ids equal CSC positions
    return capi.spmm_u_mul_e_sum(g.in_pointer, g.in_node_indices, pg.in_eid, z, a, plan)


def rgcn_layer(pg: PreparedGraph, h, weight, norm):
    g = pg.g
    # one product row per distinct (relation, source) pair instead of one per edge (see source_relation_pairs);
    # BroadcastSrcNode is folded into the typed linear, mul(m, norm) into the segment sum, which reads the pair rows
    pair_src, pair_ptr, pos_pair = pg.source_relation_pairs()
    m = capi.segment_mm(h, weight, pair_ptr, gather_idx=pair_src)                # (P, out)
    plan = pg.plan_in(m.shape[1])
    return capi.spmm_u_mul_e_sum(g.in_pointer, pos_pair, pg.in_eid, m, norm, plan)


def hgt_layer(pg: PreparedGraph, h, p: Dict[str, torch.Tensor], heads: int, sqrt_dk: float):
    g = pg.g
    k = capi.segment_mm(h, p["k_weight"], g.ntype_pointer)
    v = capi.segment_mm(h, p["v_weight"], g.ntype_pointer)
    q = capi.segment_mm(h, p["q_weight"], g.ntype_pointer)
    # The relation-transformed keys and messages depend on (edge type, source node) only: one row per distinct pair
    # instead of one per edge (C4: 0.2 M pairs for 1.5 M edges), and the edge tensors are never written - the score
    # and the weighted sum read the pair rows through the pair index of each in-edge.
    pair_src, pair_ptr, pos_pair = pg.source_relation_pairs()
    k2 = capi.segment_mm(k, p["relation_att"], pair_ptr, gather_idx=pair_src)
    v2 = capi.segment_mm(v, p["relation_msg"], pair_ptr, gather_idx=pair_src)
    plan = pg.plan_in(v2.shape[1])
    s = capi.sddmm_u_dot_v_csc(g.in_pointer, pos_pair, g.in_edge_indices, k2, q, heads, plan)
    pri = capi.gather_rows(g.etype_COO, p["relation_pri"])
    s = s.mul_(pri).div_(sqrt_dk)
    a = capi.segment_softmax(g.in_pointer, pg.in_eid, s, plan)
    t = capi.spmm_u_mul_e_sum(g.in_pointer, pos_pair, pg.in_eid, v2, a, plan)
    out = capi.segment_mm(t, p["a_weight"], g.ntype_pointer)
    alpha = capi.gather_rows(g.ntype_COO, torch.sigmoid(p["skip"]).unsqueeze(1).contiguous())
    return out.mul_(alpha)
