"""Every operator of the TorchScript registration library (libgraphiler.so), called through torch.ops.my_ops on a
GPU and checked against the CPU oracle: the reference's fifteen registrations (src/ops/**) plus this library's three
additions, on the reference's debug_hetero-shaped fixture and a seeded random graph with hub and empty rows."""
import numpy as np
import pytest
import torch

from graphiler_b200 import capi
from graphiler_b200.graph import attach_types, debug_hetero_graph, prepare_graph
from oracle import ops_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    torch.classes.load_library(str(capi.TORCH_OPS_LIB))
    torch.ops.load_library(str(capi.TORCH_OPS_LIB))
    return torch.ops.my_ops


def typed_random_graph():
    g = torch.Generator().manual_seed(5)
    n, e = 120, 900
    src = torch.cat([torch.randint(0, n, (e,), generator=g), torch.randint(0, n, (700,), generator=g)])
    dst = torch.cat([torch.randint(0, n // 2, (e,), generator=g), torch.full((700,), 11)])
    gr = prepare_graph(src, dst, n)
    return attach_types(gr, ntype_counts=[50, 40, 30], etype_counts=[400, 0, 700, 500])


def to_obj(g):
    d = g.to(DEV)
    obj = torch.classes.my_classes.DGLGraph(d.in_pointer, d.in_node_indices, d.in_edge_indices, d.out_pointer,
                                            d.out_node_indices, d.out_edge_indices, d.COO_src, d.COO_dst, None, None)
    obj.SetNtypePointer(d.ntype_pointer), obj.SetEtypePointer(d.etype_pointer)
    obj.SetNtypeCOO(d.ntype_COO), obj.SetEtypeCOO(d.etype_COO)
    return obj


def close(got, truth, rtol=1e-5, atol=1e-6):
    ok, bad, err = O.within_tolerance(got.float().cpu().numpy(), truth, rtol, atol)
    assert ok, f"{bad} elements outside tolerance (max abs err {err:.2e})"


@pytest.mark.parametrize("make", [debug_hetero_graph, typed_random_graph])
def test_all_registered_operators(ops, make):
    g = make()
    G = to_obj(g)
    n, e, tn, te = g.num_nodes, g.num_edges, g.num_ntypes, g.num_etypes
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(n, 16, generator=gen)
    xd = x.to(DEV)
    # broadcasts: bit exact, any trailing shape
    assert torch.equal(ops.BroadcastSrcNode(xd, G).cpu(), x[g.COO_src])
    assert torch.equal(ops.BroadcastDstNode(xd, G).cpu(), x[g.COO_dst])
    xt = torch.randn(tn, 4, 4, generator=gen)
    assert torch.equal(ops.BroadcastNodeType(xt.to(DEV), G).cpu(), xt[g.ntype_COO])
    assert torch.equal(ops.BroadcastSrcNodeType(xt.to(DEV), G).cpu(), xt[g.ntype_COO][g.COO_src])
    assert torch.equal(ops.BroadcastDstNodeType(xt.to(DEV), G).cpu(), xt[g.ntype_COO][g.COO_dst])
    xe = torch.randn(te, 3, generator=gen)
    assert torch.equal(ops.BroadcastEdgeType(xe.to(DEV), G).cpu(), xe[g.etype_COO])
    assert ops.get_feat_dim(torch.zeros(5, 3, 4)) == 12
    # SpMM family
    close(ops.SpMMSrc(xd, [1], False, None, G), O.spmm_src(x, g.in_pointer, g.in_node_indices))
    m = torch.randn(e, 16, generator=gen)
    close(ops.SpMMEdge(m.to(DEV), [1], False, None, G), O.spmm_edge(m, g.in_pointer, g.in_edge_indices))
    for w in (torch.randn(e, 1, generator=gen), torch.randn(e, 4, generator=gen)):      # one head / four heads
        close(ops.gspmm_src_mul_e_sum(xd, w.to(DEV), [1], False, None, G),
              O.src_mul_e_sum(x, w, g.in_pointer, g.in_node_indices, g.in_edge_indices))
        close(ops.gspmm_dst_mul_e_sum(xd, w.to(DEV), [1], False, None, G),
              O.dst_mul_e_sum(x, w, g.out_pointer, g.out_node_indices, g.out_edge_indices))
    # SDDMM
    l, r = torch.randn(n, 4, generator=gen), torch.randn(n, 4, generator=gen)
    z = ops.gsddmm_u_add_v_mul_alpha(l.to(DEV), r.to(DEV), 1, G)
    assert torch.equal(z.cpu(), l[g.COO_src] + r[g.COO_dst])
    y2 = torch.randn(n, 16, generator=gen)
    close(ops.gsddmm_u_dot_v(xd, y2.to(DEV), 4, G), O.sddmm_u_dot_v(x, y2, g.COO_src, g.COO_dst, 4))
    # segment softmax: (E,1), (E,) and multi-head
    for shape in ((e, 1), (e,), (e, 4)):
        s = torch.randn(*shape, generator=gen) * 3
        out = ops.SegmentSoftmax(s.to(DEV), 1, None, G)
        assert out.shape == s.shape
        close(out, O.segment_softmax(s, g.in_pointer, g.in_edge_indices))
    # typed linear (tensor-core path: K % 4 == 0) and the fused source gather
    wn, we = torch.randn(tn, 16, 8, generator=gen) / 4, torch.randn(te, 16, 8, generator=gen) / 4
    tol = dict(rtol=1e-5, atol=3e-6)                  # tensor-core accumulation: see tests/test_kernels_gpu.py
    close(ops.SegmentMMNode(xd, wn.to(DEV), G), O.segment_mm(x, wn, g.ntype_pointer), **tol)
    close(ops.SegmentMMEdge(m.to(DEV), we.to(DEV), G), O.segment_mm(m, we, g.etype_pointer), **tol)
    close(ops.SegmentMMEdgeSrc(xd, we.to(DEV), G), O.segment_mm(x[g.COO_src], we, g.etype_pointer), **tol)
    # fused attention
    el, er = torch.randn(n, 4, generator=gen), torch.randn(n, 4, generator=gen)
    close(ops.gat_fused(el.to(DEV), er.to(DEV), xd, 0.2, G),
          O.gat_fused(el, er, x, 0.2, g.in_pointer, g.in_node_indices, g.in_edge_indices))


def test_operators_reject_cpu_tensors_and_bad_shapes(ops):
    g = debug_hetero_graph()
    G = to_obj(g)
    with pytest.raises(RuntimeError):
        ops.SpMMSrc(torch.zeros(g.num_nodes, 4), [1], False, None, G)
    with pytest.raises(RuntimeError):
        ops.SpMMSrc(torch.zeros(g.num_nodes + 1, 4, device=DEV), [1], False, None, G)
    with pytest.raises(RuntimeError):
        ops.SegmentSoftmax(torch.zeros(g.num_edges, 2, device=DEV), 0, None, G)
    with pytest.raises(RuntimeError):
        ops.SpMMSrc(torch.zeros(g.num_nodes, 4, device=DEV, dtype=torch.float64), [1], False, None, G)
    y = ops.SpMMSrc(torch.ones(g.num_nodes, 4, device=DEV), [1], False, None, G)     # still healthy
    assert torch.equal(y.cpu()[:, 0], g.in_degrees().float())


def test_prepare_graph_on_device_matches_host():
    from graphiler_b200 import synthetic
    wl = synthetic.make_c3(scale=0.01)
    g = wl.graph
    gd = prepare_graph(g.COO_src.to(DEV), g.COO_dst.to(DEV), g.num_nodes)
    for name in ("in_pointer", "in_node_indices", "in_edge_indices", "out_pointer", "out_node_indices",
                 "out_edge_indices", "COO_src", "COO_dst"):
        assert torch.equal(getattr(gd, name).cpu(), getattr(g, name)), name


def _ctor(d, **over):
    a = {k: getattr(d, k) for k in ("in_pointer", "in_node_indices", "in_edge_indices", "out_pointer", "out_node_indices",
                                    "out_edge_indices", "COO_src", "COO_dst")}
    a.update(over)
    return torch.classes.my_classes.DGLGraph(a["in_pointer"], a["in_node_indices"], a["in_edge_indices"], a["out_pointer"],
                                             a["out_node_indices"], a["out_edge_indices"], a["COO_src"], a["COO_dst"],
                                             None, None)


def test_graph_arrays_are_validated_at_construction(ops):
    """An index out of range, a pointer array that decreases or does not end at the edge count, and a type pointer
    that does not cover its rows are refused with an error where the graph enters the library, not read out of
    bounds by a kernel later.  The context stays usable."""
    d = typed_random_graph().to(DEV)
    n, e = d.num_nodes, d.num_edges
    bad = d.in_node_indices.clone()
    bad[7] = n                                                  # one past the last node
    with pytest.raises(RuntimeError, match="neighbour index"):
        _ctor(d, in_node_indices=bad)
    bad = d.out_edge_indices.clone()
    bad[0] = -1
    with pytest.raises(RuntimeError, match="edge index"):
        _ctor(d, out_edge_indices=bad)
    bad = d.in_pointer.clone()
    bad[5], bad[6] = bad[6].item() + 1, bad[5].item()
    with pytest.raises(RuntimeError, match="pointer array"):
        _ctor(d, in_pointer=bad)
    bad = d.in_pointer.clone()
    bad[-1] = e - 1
    with pytest.raises(RuntimeError, match="pointer array"):
        _ctor(d, in_pointer=bad)
    bad = d.COO_dst.clone()
    bad[3] = n + 5
    with pytest.raises(RuntimeError, match="COO_dst"):
        _ctor(d, COO_dst=bad)
    G = _ctor(d)
    short = d.etype_pointer.clone()
    short[-1] = e - 3                                           # leaves three edges without a type
    with pytest.raises(RuntimeError, match="etype_pointer"):
        G.SetEtypePointer(short)
    G.SetEtypePointer(d.etype_pointer)
    y = ops.SpMMSrc(torch.ones(n, 4, device=DEV), [1], False, None, G)
    assert torch.equal(y.cpu()[:, 0], typed_random_graph().in_degrees().float())


def test_first_operator_call_on_a_graph_can_be_captured(ops):
    """No operator call synchronises or allocates device memory behind PyTorch's allocator: the very first calls on a
    freshly built graph (rows cut into pieces, so scratch is needed) run inside a CUDA-graph capture, which refuses
    both, and the replay gives the eager result."""
    from graphiler_b200 import synthetic
    wl = synthetic.make_c5(scale=0.002)
    d = wl.graph.to(DEV)
    assert int(d.in_degrees().max()) > 512                      # at least one row is cut
    x = torch.randn(d.num_nodes, 64, device=DEV)
    w = torch.rand(d.num_edges, 1, device=DEV)
    G = _ctor(d)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        with torch.cuda.graph(graph, stream=s):
            y = ops.SpMMSrc(x, [1], False, None, G)
            a = ops.SegmentSoftmax(w, 1, None, G)
            z = ops.gspmm_src_mul_e_sum(x, a, [1], False, None, G)
    graph.replay()
    torch.cuda.synchronize()
    G2 = _ctor(d)
    assert torch.equal(y, ops.SpMMSrc(x, [1], False, None, G2))
    assert torch.equal(z, ops.gspmm_src_mul_e_sum(x, ops.SegmentSoftmax(w, 1, None, G2), [1], False, None, G2))
    close(y, O.spmm_src(x, wl.graph.in_pointer, wl.graph.in_node_indices))


def test_typed_linear_sees_in_place_weight_updates(ops):
    g = typed_random_graph()
    G = to_obj(g)
    x = torch.randn(g.num_nodes, 64, device=DEV)
    w = torch.randn(g.num_ntypes, 64, 48, device=DEV) * 0.2
    y1 = ops.SegmentMMNode(x, w, G)
    assert torch.equal(y1, ops.SegmentMMNode(x, w, G))                      # second call: cached split weights
    w.mul_(2.0)
    assert torch.equal(ops.SegmentMMNode(x, w, G), y1 * 2.0)
    close(y1, O.segment_mm(x.cpu(), (w / 2).cpu(), g.ntype_pointer), rtol=1e-5, atol=2e-6)


def test_edge_typed_linear_on_gathered_rows_is_evaluated_per_pair(ops):
    """SegmentMMEdgeSrc on a graph with few sources per relation (every (relation, source) pair has many edges) takes
    the per-pair route inside the operator and must return, bit for bit, what the edge-typed linear returns on the
    gathered rows."""
    gen = torch.Generator().manual_seed(12)
    n, per = 60, 900
    src = torch.cat([torch.randint(0, 8, (per,), generator=gen), torch.randint(8, 20, (per,), generator=gen),
                     torch.randint(0, 60, (per,), generator=gen)])
    dst = torch.randint(0, n, (3 * per,), generator=gen)
    g = attach_types(prepare_graph(src, dst, n), ntype_counts=[20, 40], etype_counts=[per, per, per])
    G = to_obj(g)
    for k, m in ((64, 48), (16, 16)):                       # tensor-core kernel, narrow kernel
        x = torch.randn(n, k, generator=gen).to(DEV)
        w = (torch.randn(3, k, m, generator=gen) * 0.2).to(DEV)
        fused = ops.SegmentMMEdgeSrc(x, w, G)
        unfused = ops.SegmentMMEdge(ops.BroadcastSrcNode(x, G), w, G)
        assert fused.shape == (3 * per, m) and torch.equal(fused, unfused)
        close(fused, O.segment_mm(x.cpu()[g.COO_src], w.cpu(), g.etype_pointer), rtol=1e-5, atol=2e-6)
