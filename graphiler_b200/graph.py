"""Graph preparation without DGL: edge list -> the array set every operator consumes.

Restates the layout contract of the reference's ``prepare_graph``
(python/graphiler/utils/setup.py:116-146) and of the type arrays it attaches to
heterogeneous graphs (setup.py:87-100, 149-161):

* ``in_pointer`` (N+1) int32, ``in_node_indices`` (E) int32 = source of each
  in-edge, ``in_edge_indices`` (E) int32 = edge id of each in-edge, grouped by
  destination (the reduce side, CSC);
* ``out_pointer`` / ``out_node_indices`` / ``out_edge_indices``: the same for
  out-edges (the message side, CSR);
* ``COO_src`` / ``COO_dst`` (E) int64 in edge-id order;
* ``ntype_pointer`` (Tn+1) / ``etype_pointer`` (Te+1) int32 and ``ntype_COO``
  (N) / ``etype_COO`` (E) int64 for graphs whose node / edge ids are contiguous
  per type.

The reference delegates the edge ordering inside one destination to DGL.  Here it
is part of the bit-exact contract: in-edges of a destination (and out-edges of a
source) are listed by ascending edge id, i.e. a stable sort of the edge list.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

INT32_MAX = 2**31 - 1


@dataclass
class GraphArrays:
    """The ten constructor arguments of ``my_classes.DGLGraph`` plus the type COO arrays
    (include/dglgraph.h:7-75), as plain tensors on one device."""

    num_nodes: int
    num_edges: int
    in_pointer: torch.Tensor
    in_node_indices: torch.Tensor
    in_edge_indices: torch.Tensor
    out_pointer: torch.Tensor
    out_node_indices: torch.Tensor
    out_edge_indices: torch.Tensor
    COO_src: torch.Tensor
    COO_dst: torch.Tensor
    ntype_pointer: Optional[torch.Tensor] = None
    etype_pointer: Optional[torch.Tensor] = None
    ntype_COO: Optional[torch.Tensor] = None
    etype_COO: Optional[torch.Tensor] = None
    extras: dict = field(default_factory=dict)

    _TENSORS = ("in_pointer", "in_node_indices", "in_edge_indices", "out_pointer",
                "out_node_indices", "out_edge_indices", "COO_src", "COO_dst",
                "ntype_pointer", "etype_pointer", "ntype_COO", "etype_COO")

    @property
    def device(self) -> torch.device:
        return self.in_pointer.device

    @property
    def num_ntypes(self) -> int:
        return 1 if self.ntype_pointer is None else int(self.ntype_pointer.numel()) - 1

    @property
    def num_etypes(self) -> int:
        return 1 if self.etype_pointer is None else int(self.etype_pointer.numel()) - 1

    def to(self, device) -> "GraphArrays":
        kw = {}
        for name in self._TENSORS:
            t = getattr(self, name)
            kw[name] = None if t is None else t.to(device)
        return GraphArrays(self.num_nodes, self.num_edges, extras=dict(self.extras), **kw)

    def in_degrees(self) -> torch.Tensor:
        return (self.in_pointer[1:] - self.in_pointer[:-1]).to(torch.int64)

    def out_degrees(self) -> torch.Tensor:
        return (self.out_pointer[1:] - self.out_pointer[:-1]).to(torch.int64)

    def validate(self) -> None:
        """Host-side structural checks (pointer monotone, last == E, indices in range)."""
        n, e = self.num_nodes, self.num_edges
        for ptr, idx, eid in ((self.in_pointer, self.in_node_indices, self.in_edge_indices),
                              (self.out_pointer, self.out_node_indices, self.out_edge_indices)):
            assert ptr.dtype == torch.int32 and idx.dtype == torch.int32 and eid.dtype == torch.int32
            assert ptr.numel() == n + 1 and idx.numel() == e and eid.numel() == e
            assert int(ptr[0]) == 0 and int(ptr[-1]) == e
            assert bool((ptr[1:] >= ptr[:-1]).all())
            if e:
                assert int(idx.min()) >= 0 and int(idx.max()) < n
                assert int(eid.min()) >= 0 and int(eid.max()) < e
        assert self.COO_src.dtype == torch.int64 and self.COO_dst.dtype == torch.int64
        assert self.COO_src.numel() == e and self.COO_dst.numel() == e


def _grouped(key: torch.Tensor, other: torch.Tensor, num_nodes: int):
    """Stable group-by of the edge list on ``key``: (pointer, other[perm], perm) as int32."""
    e = key.numel()
    if e == 0:
        z = torch.zeros(0, dtype=torch.int32, device=key.device)
        return torch.zeros(num_nodes + 1, dtype=torch.int32, device=key.device), z, z.clone()
    _, perm = torch.sort(key, stable=True)
    counts = torch.bincount(key, minlength=num_nodes)
    pointer = torch.zeros(num_nodes + 1, dtype=torch.int64, device=key.device)
    torch.cumsum(counts, 0, out=pointer[1:])
    return pointer.to(torch.int32), other[perm].to(torch.int32), perm.to(torch.int32)


def prepare_graph(src: torch.Tensor, dst: torch.Tensor, num_nodes: int) -> GraphArrays:
    """Edge list (edge id = position) -> ``GraphArrays`` on the edge list's device.

    Replaces the DGL calls and the Python-loop prefix sum of the reference
    (setup.py:119-141) with a stable sort and a cumulative sum.
    """
    src = src.to(torch.int64).contiguous()
    dst = dst.to(torch.int64).contiguous()
    e = src.numel()
    if dst.numel() != e:
        raise ValueError("src and dst must have the same length")
    if num_nodes > INT32_MAX or e > INT32_MAX:
        raise ValueError("node and edge counts must fit int32 (include/dglgraph.h:48-52)")
    if e and (int(src.min()) < 0 or int(dst.min()) < 0 or
              int(src.max()) >= num_nodes or int(dst.max()) >= num_nodes):
        raise ValueError("edge endpoint out of range")
    in_ptr, in_nodes, in_eids = _grouped(dst, src, num_nodes)
    out_ptr, out_nodes, out_eids = _grouped(src, dst, num_nodes)
    return GraphArrays(num_nodes, e, in_ptr, in_nodes, in_eids, out_ptr, out_nodes, out_eids,
                       src, dst)


def attach_types(g: GraphArrays, ntype_counts=None, etype_counts=None) -> GraphArrays:
    """Attach type pointers / type COO arrays for ids that are contiguous per type
    (setup.py:87-100: ``SetNtypePointer`` / ``SetEtypePointer`` / ``SetNtypeCOO`` / ``SetEtypeCOO``)."""
    dev = g.device
    if ntype_counts is not None:
        c = torch.as_tensor(list(ntype_counts), dtype=torch.int64)
        if int(c.sum()) != g.num_nodes:
            raise ValueError("node type counts must sum to num_nodes")
        g.ntype_pointer = torch.cat([torch.zeros(1, dtype=torch.int64), c.cumsum(0)]).to(torch.int32).to(dev)
        g.ntype_COO = torch.repeat_interleave(torch.arange(c.numel()), c).to(dev)
    if etype_counts is not None:
        c = torch.as_tensor(list(etype_counts), dtype=torch.int64)
        if int(c.sum()) != g.num_edges:
            raise ValueError("edge type counts must sum to num_edges")
        g.etype_pointer = torch.cat([torch.zeros(1, dtype=torch.int64), c.cumsum(0)]).to(torch.int32).to(dev)
        g.etype_COO = torch.repeat_interleave(torch.arange(c.numel()), c).to(dev)
    return g


def debug_graph() -> GraphArrays:
    """The reference's 3-node / 6-edge debug graph (setup.py:41-42)."""
    src = torch.tensor([0, 0, 0, 1, 1, 2])
    dst = torch.tensor([0, 1, 2, 1, 2, 2])
    return prepare_graph(src, dst, 3)


def debug_hetero_graph() -> GraphArrays:
    """A flattened graph with the shape of the reference's ``debug_hetero`` fixture
    (setup.py:73-81): node types user (3) and movie (2) with contiguous ids, six
    canonical edge types with contiguous edge ids in the order the fixture lists them."""
    U, M = 0, 3  # id offsets of the two node types
    blocks = [
        ([0 + U, 0 + U, 1 + U], [0 + M, 1 + M, 0 + M]),   # user +1 movie
        ([1 + U, 2 + U, 2 + U], [1 + M, 0 + M, 1 + M]),   # user -1 movie
        ([0 + U], [1 + U]),                               # user +1 user
        ([2 + U], [1 + U]),                               # user -1 user
        ([0 + M], [1 + M]),                               # movie +1 movie
        ([1 + M], [0 + M]),                               # movie -1 movie
    ]
    src = torch.tensor([s for b in blocks for s in b[0]])
    dst = torch.tensor([d for b in blocks for d in b[1]])
    g = prepare_graph(src, dst, 5)
    return attach_types(g, ntype_counts=[3, 2], etype_counts=[len(b[0]) for b in blocks])
