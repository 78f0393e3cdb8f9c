"""CPU restatement of the reference's baseline path: DGL user-defined-function execution.
TEST INFRASTRUCTURE ONLY (checker and timed CPU baseline; never imported by the package).

The reference compares its compiled graphs with ``g.update_all(message_func, reduce_func)``
executed by DGL 0.6.1 (examples/GAT/GAT.py:70, GCN/GCN.py:43, RGCN/RGCN.py:57,
HGT/HGT.py:155-160; requirements.txt:1).  DGL is a third-party dependency whose source is
not part of the reference tree and which cannot be installed offline, so its published
execution model is restated here in PyTorch on CPU:

* the message function runs once over all edges in edge-id order, on an edge batch whose
  ``src[k] = ndata[k][COO_src]``, ``dst[k] = ndata[k][COO_dst]``, ``data[k] = edata[k]``,
  ``type[k] = etype_data[k][etype_COO]`` and ``srctype/dsttype[k] =
  ntype_data[k][ntype_COO][COO_src/COO_dst]`` (field names: python/graphiler/dgl_udf_batch.py:5-57);
* the reduce function runs once per distinct in-degree d > 0 on a mailbox of shape
  (n_d, d, ...) filled in in-edge order (degree bucketing); zero-in-degree nodes get zero rows;
* the update function runs once over all nodes with ``type[k] = ntype_data[k][ntype_COO]``.

The four model bodies below restate the reference's user-defined functions
(examples/GAT/GAT.py:25-36, GCN/GCN.py:21-27, RGCN/RGCN.py:25-33, HGT/HGT.py:28-60), with
the per-head reshapes of its multi-head baselines (examples/GAT/GAT_PyG.py:90-103,
examples/HGT/HGT_DGL.py:60-112) so that H > 1 is covered; with H == 1 they reduce to the
single-head bodies.  The dtype of the inputs decides the arithmetic: float32 is the timed
"reference CPU path", float64 (same float32 values, widened) is the numerical truth.

Parity pin: see oracle/ops_oracle.py.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch
import torch.nn.functional as F


class EdgeBatch:
    def __init__(self, src, dst, data, srctype, dsttype, etype):
        self.src, self.dst, self.data = src, dst, data
        self.srctype, self.dsttype, self.type = srctype, dsttype, etype


class NodeBatch:
    def __init__(self, mailbox, data, ntype):
        self.mailbox, self.data, self.type = mailbox, data, ntype


class _Lazy(dict):
    """Dict whose values are gathered on first access (a UDF only touches a few keys)."""

    def __init__(self, base: Dict[str, torch.Tensor], *index):
        super().__init__()
        self._base, self._index = base, index

    def __missing__(self, key):
        v = self._base[key]
        for ix in self._index:
            v = v[ix]
        self[key] = v
        return v


def update_all(g, ndata, edata, ntype_data, etype_data,
               message_func: Callable, reduce_func: Callable, update_func: Optional[Callable] = None,
               rows: Optional[range] = None):
    """Run one message-passing step with DGL's user-defined-function semantics.

    ``g`` is a ``GraphArrays`` on CPU.  ``rows`` restricts the destinations that are reduced
    (used to time a bounded slice of a very large graph); messages are then only created for
    the in-edges of those rows.  Returns the dict of new node data (rows x ...)."""
    src, dst = g.COO_src, g.COO_dst
    ptr = g.in_pointer.to(torch.int64)
    in_eid = g.in_edge_indices.to(torch.int64)
    if rows is None:
        r0, r1 = 0, g.num_nodes
        edge_sel = None
    else:
        r0, r1 = rows.start, rows.stop
        edge_sel = torch.sort(in_eid[ptr[r0]:ptr[r1]])[0]         # edge-id order, as DGL batches edges
        src, dst = src[edge_sel], dst[edge_sel]

    def esel(d):  # edge-indexed dict restricted to the selected edges
        return _Lazy(d, edge_sel) if edge_sel is not None else d

    ntc, etc = g.ntype_COO, g.etype_COO
    if etc is not None and edge_sel is not None:
        etc = etc[edge_sel]
    edges = EdgeBatch(_Lazy(ndata, src), _Lazy(ndata, dst), esel(edata),
                      _Lazy(ntype_data, ntc, src) if ntc is not None else {},
                      _Lazy(ntype_data, ntc, dst) if ntc is not None else {},
                      _Lazy(etype_data, etc) if etc is not None else {})
    msgs = message_func(edges)

    deg = (ptr[1:] - ptr[:-1])[r0:r1]
    out: Dict[str, torch.Tensor] = {}
    if edge_sel is not None:
        # position of every selected edge id inside the compacted message tensors
        remap = torch.empty(g.num_edges, dtype=torch.int64)
        remap[edge_sel] = torch.arange(edge_sel.numel())
    for d in torch.unique(deg).tolist():
        if d == 0:
            continue
        nodes = torch.nonzero(deg == d).squeeze(1)
        starts = ptr[nodes + r0]
        pos = starts.unsqueeze(1) + torch.arange(d).unsqueeze(0)          # (n_d, d) CSC positions
        eids = in_eid[pos]
        if edge_sel is not None:
            eids = remap[eids]
        mailbox = {k: v[eids] for k, v in msgs.items()}                   # (n_d, d, ...)
        nb = NodeBatch(mailbox, _Lazy(ndata, nodes + r0),
                       _Lazy(ntype_data, ntc, nodes + r0) if ntc is not None else {})
        red = reduce_func(nb)
        for k, v in red.items():
            if k not in out:
                out[k] = torch.zeros((r1 - r0,) + tuple(v.shape[1:]), dtype=v.dtype)
            out[k][nodes] = v
    if update_func is not None:
        all_rows = torch.arange(r0, r1)
        merged = dict(ndata)
        nd = _Lazy(merged, all_rows)
        for k, v in out.items():
            nd[k] = v
        nb = NodeBatch({}, nd, _Lazy(ntype_data, ntc, all_rows) if ntc is not None else {})
        out.update(update_func(nb))
    return out


# ------------------------------------------------------------------------------------------------
# model bodies

def gat_layer(g, h, fc_weight, attn_src, attn_dst, slope: float, rows=None):
    """GAT layer (examples/GAT/GAT.py:25-36, 44-71) with H heads of width D.

    z = h @ W viewed (., H, D); e = leaky_relu(sum_d z_src*a_src + sum_d z_dst*a_dst) per head
    (the single-head body's cat + mm with a (2F,1) vector is the H == 1 case); alpha = softmax
    over the mailbox; out = sum alpha * z_src."""
    heads, dim = attn_src.shape

    def message_func(edges):
        z_s = torch.mm(edges.src["h"], fc_weight)
        z_d = torch.mm(edges.dst["h"], fc_weight)
        a = (z_s.view(-1, heads, dim) * attn_src).sum(-1) + (z_d.view(-1, heads, dim) * attn_dst).sum(-1)
        return {"z": z_s, "e": F.leaky_relu(a, slope)}

    def reduce_func(nodes):
        alpha = torch.softmax(nodes.mailbox["e"], dim=1)                     # (n, d, H)
        z = nodes.mailbox["z"]
        zz = z.view(z.shape[0], z.shape[1], heads, dim)
        return {"h": torch.sum(alpha.unsqueeze(-1) * zz, dim=1).reshape(z.shape[0], heads * dim)}

    return update_all(g, {"h": h}, {}, {}, {}, message_func, reduce_func, rows=rows)["h"]


def gcn_layer(g, feature, weight, norm_src, norm_dst=None, relu: bool = True, rows=None):
    """GCN layer (examples/GCN/GCN.py:21-27, 33-46): h = feature @ W; message = h_src *
    norm_src; reduce = relu(sum).  The reference scales on the source side only with
    in-degree^-1/2; ``norm_dst`` adds the destination-side factor of the symmetric
    normalisation as a dense row scaling before the activation."""
    h = torch.mm(feature, weight)

    def message_func(edges):
        return {"m": edges.src["h"] * edges.src["norm"]}

    def reduce_func(nodes):
        s = torch.sum(nodes.mailbox["m"], dim=1)
        if norm_dst is not None:
            s = s * nodes.data["norm_dst"]
        return {"h": torch.relu(s) if relu else s}

    nd = {"h": h, "norm": norm_src}
    if norm_dst is not None:
        nd["norm_dst"] = norm_dst
    return update_all(g, nd, {}, {}, {}, message_func, reduce_func, rows=rows)["h"]


def rgcn_layer(g, h, weight, norm, rows=None):
    """RGCN layer (examples/RGCN/RGCN.py:25-33): msg = (h_src @ W[type]) * norm; reduce = sum."""

    def message_func(edges):
        w = edges.type["weight"]
        msg = torch.bmm(edges.src["h"].unsqueeze(1), w).squeeze(1)
        return {"m": msg * edges.data["norm"]}

    def reduce_func(nodes):
        return {"h": torch.sum(nodes.mailbox["m"], dim=1)}

    return update_all(g, {"h": h}, {"norm": norm}, {}, {"weight": weight}, message_func, reduce_func,
                      rows=rows)["h"]


def hgt_layer(g, h, p: Dict[str, torch.Tensor], heads: int, sqrt_dk: float):
    """HGT layer (examples/HGT/HGT.py:28-60) with H heads (examples/HGT/HGT_DGL.py:60-112):
    k/v/q = per-node-type projections of h at src/src/dst; k, v further multiplied by the
    per-edge-type relation matrices; score[h] = sum_d(k*q) * pri[type,h] / sqrt_dk; softmax
    per destination; t = sum alpha * v; out = (t @ a_weight[type]) * sigmoid(skip[type])."""

    def message_func(edges):
        k = torch.bmm(edges.src["h"].unsqueeze(1), edges.srctype["k_weight"]).squeeze(1)
        v = torch.bmm(edges.src["h"].unsqueeze(1), edges.srctype["v_weight"]).squeeze(1)
        q = torch.bmm(edges.dst["h"].unsqueeze(1), edges.dsttype["q_weight"]).squeeze(1)
        k = torch.bmm(k.unsqueeze(1), edges.type["relation_att"]).squeeze(1)
        v = torch.bmm(v.unsqueeze(1), edges.type["relation_msg"]).squeeze(1)
        t = (k * q).view(k.shape[0], heads, -1)
        score = torch.sum(t, dim=2) * edges.type["relation_pri"] / sqrt_dk        # (E, H)
        return {"attn": score, "v": v}

    def reduce_func(nodes):
        a = torch.softmax(nodes.mailbox["attn"], dim=1)                              # (n, d, H)
        v = nodes.mailbox["v"]
        vv = v.view(v.shape[0], v.shape[1], heads, -1)
        return {"t": torch.sum(a.unsqueeze(-1) * vv, dim=1).reshape(v.shape[0], -1)}

    def update_func(nodes):
        alpha = torch.sigmoid(nodes.type["skip"])
        out = torch.bmm(nodes.data["t"].unsqueeze(1), nodes.type["a_weight"]).squeeze(1)
        return {"h": out * alpha.unsqueeze(1)}

    ntd = {k: p[k] for k in ("k_weight", "v_weight", "q_weight", "a_weight", "skip")}
    etd = {k: p[k] for k in ("relation_att", "relation_msg", "relation_pri")}
    return update_all(g, {"h": h}, {}, ntd, etd, message_func, reduce_func, update_func)["h"]


def hgt_layer_typed(g, h, p: Dict[str, torch.Tensor], heads: int, sqrt_dk: float):
    """Same layer as ``hgt_layer`` with the per-edge weight gathers replaced by per-type
    matrix products: mathematically identical, but it avoids the (E, F, F) weight tensors
    that make the literal UDF path run out of memory on large graphs (the "OOM" bars of the
    reference's own figures).  Used where the literal path cannot be held in host memory."""
    ntp = g.ntype_pointer.tolist()
    etp = g.etype_pointer.tolist()

    def typed(x, w, ptr):
        return torch.cat([x[ptr[t]:ptr[t + 1]] @ w[t] for t in range(len(ptr) - 1)], 0)

    k = typed(h, p["k_weight"], ntp)
    v = typed(h, p["v_weight"], ntp)
    q = typed(h, p["q_weight"], ntp)
    ke = typed(k[g.COO_src], p["relation_att"], etp)
    ve = typed(v[g.COO_src], p["relation_msg"], etp)
    score = (ke * q[g.COO_dst]).view(g.num_edges, heads, -1).sum(2) * p["relation_pri"][g.etype_COO] / sqrt_dk

    def message_func(edges):
        return {"attn": score, "v": ve}

    def reduce_func(nodes):
        a = torch.softmax(nodes.mailbox["attn"], dim=1)
        vv = nodes.mailbox["v"]
        vv = vv.view(vv.shape[0], vv.shape[1], heads, -1)
        return {"t": torch.sum(a.unsqueeze(-1) * vv, dim=1).reshape(vv.shape[0], -1)}

    t = update_all(g, {"h": h}, {}, {}, {}, message_func, reduce_func)["t"]
    out = typed(t, p["a_weight"], ntp)
    return out * torch.sigmoid(p["skip"])[g.ntype_COO].unsqueeze(1)
