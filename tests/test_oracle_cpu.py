"""CPU checks that pin the oracle: vectorised operator oracle vs literal loops, operator
sequences of the reference's optimised graphs vs the user-defined-function semantics, and the
array layout of the reference's debug fixtures."""
import numpy as np
import pytest
import torch

from graphiler_b200 import synthetic
from graphiler_b200.graph import attach_types, debug_graph, debug_hetero_graph, prepare_graph
from oracle import ops_oracle as O
from oracle import udf_oracle as U


def random_graph(n, e, seed, self_loops=True, empty_rows=False):
    g = torch.Generator().manual_seed(seed)
    src = torch.randint(0, n, (e,), generator=g)
    hi = n // 2 if empty_rows else n
    dst = torch.randint(0, max(1, hi), (e,), generator=g)
    if self_loops and not empty_rows:
        src = torch.cat([src, torch.arange(n)])
        dst = torch.cat([dst, torch.arange(n)])
    return prepare_graph(src, dst, n)


def test_debug_graph_layout():
    # python/graphiler/utils/setup.py:41-42 with ascending-edge-id order inside each row
    g = debug_graph()
    assert g.in_pointer.tolist() == [0, 1, 3, 6]
    assert g.in_node_indices.tolist() == [0, 0, 1, 0, 1, 2]
    assert g.in_edge_indices.tolist() == [0, 1, 3, 2, 4, 5]
    assert g.out_pointer.tolist() == [0, 3, 5, 6]
    assert g.out_node_indices.tolist() == [0, 1, 2, 1, 2, 2]
    assert g.out_edge_indices.tolist() == [0, 1, 2, 3, 4, 5]
    assert g.COO_src.dtype == torch.int64 and g.in_pointer.dtype == torch.int32
    g.validate()


def test_debug_hetero_layout():
    g = debug_hetero_graph()
    g.validate()
    assert g.num_nodes == 5 and g.num_edges == 10
    assert g.ntype_pointer.tolist() == [0, 3, 5]
    assert g.etype_pointer.tolist() == [0, 3, 6, 7, 8, 9, 10]
    assert g.ntype_COO.tolist() == [0, 0, 0, 1, 1]
    assert g.etype_COO.tolist() == [0, 0, 0, 1, 1, 1, 2, 3, 4, 5]


def test_prepare_graph_edge_cases():
    g = prepare_graph(torch.zeros(0, dtype=torch.int64), torch.zeros(0, dtype=torch.int64), 4)
    assert g.in_pointer.tolist() == [0] * 5 and g.num_edges == 0
    g = prepare_graph(torch.tensor([1, 1, 1]), torch.tensor([2, 2, 2]), 3)     # duplicate edges
    assert g.in_pointer.tolist() == [0, 0, 0, 3] and g.in_edge_indices.tolist() == [0, 1, 2]
    with pytest.raises(ValueError):
        prepare_graph(torch.tensor([0]), torch.tensor([5]), 3)


@pytest.mark.parametrize("seed", [0, 1])
def test_vectorised_ops_match_loops(seed):
    g = random_graph(40, 200, seed, empty_rows=bool(seed))
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((40, 12)).astype(np.float32)
    w = rng.standard_normal((g.num_edges, 3)).astype(np.float32)
    np.testing.assert_allclose(O.spmm_src(x, g.in_pointer, g.in_node_indices),
                               O.spmm_src_loops(x, g.in_pointer, g.in_node_indices), rtol=1e-13, atol=1e-13)
    np.testing.assert_allclose(O.u_mul_e_sum(x, w, g.in_pointer, g.in_node_indices, g.in_edge_indices),
                               O.u_mul_e_sum_loops(x, w, g.in_pointer, g.in_node_indices, g.in_edge_indices),
                               rtol=1e-13, atol=1e-13)
    np.testing.assert_allclose(O.segment_softmax(w, g.in_pointer, g.in_edge_indices),
                               O.segment_softmax_loops(w, g.in_pointer, g.in_edge_indices), rtol=1e-13, atol=1e-15)


def test_softmax_all_negative_segment_is_finite():
    # the reference's running maximum starts at 0 (segment_softmax_kernel.cu:9) and would
    # underflow here; true softmax must not
    g = debug_graph()
    x = np.full((6, 1), -200.0, dtype=np.float32)
    y = O.segment_softmax(x, g.in_pointer, g.in_edge_indices)
    assert np.isfinite(y).all()
    np.testing.assert_allclose(O._segment_sum(y[g.in_edge_indices.numpy()], g.in_pointer), 1.0)


def _f64(d):
    return {k: v.double() for k, v in d.items()}


def test_gat_op_sequence_matches_udf():
    """gsddmm_u_add_v -> leaky_relu -> SegmentSoftmax -> gspmm_src_mul_e_sum (the reference's
    optimised GAT graph) equals the user-defined-function path, multi-head."""
    wl = synthetic.make_c1(scale=0.01)
    g, p, hy = wl.graph, wl.params, wl.hyper
    h64 = wl.feats.double()
    truth = U.gat_layer(g, h64, p["fc_weight"].double(), p["attn_src"].double(), p["attn_dst"].double(), hy["slope"])
    z = (h64 @ p["fc_weight"].double()).numpy()
    H, D = p["attn_src"].shape
    el = (z.reshape(-1, H, D) * p["attn_src"].double().numpy()).sum(-1)
    er = (z.reshape(-1, H, D) * p["attn_dst"].double().numpy()).sum(-1)
    e = O.leaky_relu(O.sddmm_u_add_v(el, er, g.COO_src, g.COO_dst), hy["slope"])
    a = O.segment_softmax(e, g.in_pointer, g.in_edge_indices)
    out = O.src_mul_e_sum(z, a, g.in_pointer, g.in_node_indices, g.in_edge_indices)
    np.testing.assert_allclose(out, truth.numpy(), rtol=1e-10, atol=1e-12)
    fused = O.gat_fused(el, er, z, hy["slope"], g.in_pointer, g.in_node_indices, g.in_edge_indices)
    np.testing.assert_allclose(fused, truth.numpy(), rtol=1e-10, atol=1e-12)


def test_gcn_op_sequence_matches_udf():
    wl = synthetic.make_c2(scale=0.005)
    g = wl.graph
    deg = g.in_degrees().clamp(min=1).double().unsqueeze(1)
    norm = deg.pow(-0.5)
    x64, w64 = wl.feats.double(), wl.params["w1"].double()
    truth = U.gcn_layer(g, x64, w64, norm, norm)
    h = (x64 @ w64) * norm
    out = np.maximum(O.spmm_src(h.numpy(), g.in_pointer, g.in_node_indices) * norm.numpy(), 0)
    np.testing.assert_allclose(out, truth.numpy(), rtol=1e-10, atol=1e-12)


def test_rgcn_op_sequence_matches_udf():
    wl = synthetic.make_c3(scale=0.003)
    g = wl.graph
    x64, w64, n64 = wl.feats.double(), wl.params["w1"].double(), wl.edata["norm"].double()
    truth = U.rgcn_layer(g, x64, w64, n64)
    he = O.broadcast_src_node(x64.numpy(), g.COO_src)
    m = O.segment_mm(he, w64.numpy(), g.etype_pointer) * n64.numpy()
    out = O.spmm_edge(m, g.in_pointer, g.in_edge_indices)
    np.testing.assert_allclose(out, truth.numpy(), rtol=1e-10, atol=1e-12)


def hgt_op_sequence(g, h, p, heads, sqrt_dk):
    """The reference's optimised HGT graph restated with oracle operators (float64)."""
    k = O.segment_mm(h, p["k_weight"], g.ntype_pointer)
    v = O.segment_mm(h, p["v_weight"], g.ntype_pointer)
    q = O.segment_mm(h, p["q_weight"], g.ntype_pointer)
    k2 = O.segment_mm(O.broadcast_src_node(k, g.COO_src), p["relation_att"], g.etype_pointer)
    v2 = O.segment_mm(O.broadcast_src_node(v, g.COO_src), p["relation_msg"], g.etype_pointer)
    s = O.sddmm_u_dot_v(k2, O.broadcast_dst_node(q, g.COO_dst), np.arange(g.num_edges), np.arange(g.num_edges), heads)
    s = s * O.broadcast_edge_type(p["relation_pri"], g.etype_COO) / sqrt_dk
    a = O.segment_softmax(s, g.in_pointer, g.in_edge_indices)
    e = g.num_edges
    t = O.spmm_edge((a[:, :, None] * v2.reshape(e, heads, -1)).reshape(e, -1), g.in_pointer, g.in_edge_indices)
    al = O.broadcast_node_type(1.0 / (1.0 + np.exp(-p["skip"])), g.ntype_COO)
    return O.segment_mm(t, p["a_weight"], g.ntype_pointer) * al[:, None]


def test_hgt_op_sequence_matches_udf():
    wl = synthetic.make_c4(scale=0.002)
    g, hy = wl.graph, wl.hyper
    p64 = _f64(wl.params)
    truth = U.hgt_layer(g, wl.feats.double(), p64, hy["heads"], hy["sqrt_dk"])
    typed = U.hgt_layer_typed(g, wl.feats.double(), p64, hy["heads"], hy["sqrt_dk"])
    np.testing.assert_allclose(typed.numpy(), truth.numpy(), rtol=1e-10, atol=1e-12)
    pn = {k: v.numpy() for k, v in p64.items()}
    out = hgt_op_sequence(g, wl.feats.double().numpy(), pn, hy["heads"], hy["sqrt_dk"])
    np.testing.assert_allclose(out, truth.numpy(), rtol=1e-10, atol=1e-12)


def test_udf_oracle_row_slice_matches_full():
    wl = synthetic.make_c2(scale=0.004)
    g = wl.graph
    norm = g.in_degrees().clamp(min=1).float().pow(-0.5).unsqueeze(1)
    full = U.gcn_layer(g, wl.feats, wl.params["w1"], norm, norm)
    part = U.gcn_layer(g, wl.feats, wl.params["w1"], norm, norm, rows=range(100, 300))
    torch.testing.assert_close(part, full[100:300], rtol=0, atol=0)


def test_zero_in_degree_rows_are_zero():
    g = random_graph(30, 40, 3, empty_rows=True)
    x = torch.randn(30, 8)
    out = U.gcn_layer(g, x, torch.eye(8), torch.ones(30, 1), relu=False)
    assert (out[15:] == 0).all()
    assert (O.spmm_src(x, g.in_pointer, g.in_node_indices)[15:] == 0).all()


def test_synthetic_generators_are_seeded_and_valid():
    for name in ("c1", "c2", "c3", "c4", "c5"):
        a = synthetic.make(name, scale=0.002)
        b = synthetic.make(name, scale=0.002)
        a.graph.validate()
        assert torch.equal(a.graph.COO_src, b.graph.COO_src) and torch.equal(a.feats, b.feats)
    c3 = synthetic.make_c3(scale=0.002)
    assert bool((c3.graph.etype_COO[1:] >= c3.graph.etype_COO[:-1]).all())      # edges sorted by relation
    c1 = synthetic.make_c1(scale=0.01)
    assert torch.equal(c1.graph.in_edge_indices, torch.arange(c1.graph.num_edges, dtype=torch.int32))


def test_c_restatement_matches_numpy_oracle():
    """oracle/csr_cpu.c (the compiled checker for the full-size cases and the timed CPU baseline) against the numpy
    oracle, which is itself pinned on the reference operators' recorded outputs."""
    from oracle import csr_cpu as K
    from fixtures_common import hetero_graphs
    g = random_graph(300, 4000, 5)
    rng = np.random.default_rng(5)
    n, e = g.num_nodes, g.num_edges
    x = rng.standard_normal((n, 24)).astype(np.float32)
    sc = rng.random(n).astype(np.float32)
    t = O.spmm_src(x, g.in_pointer, g.in_node_indices)
    assert np.allclose(K.gather_sum_f64(g.in_pointer, g.in_node_indices, x), t, rtol=1e-13, atol=1e-13)
    part = K.gather_sum_f64(g.in_pointer, g.in_node_indices, x, dst_scale=sc, relu=True, rows=(17, 211))
    assert np.allclose(part, np.maximum(t * sc[:, None].astype(np.float64), 0)[17:211], rtol=1e-13, atol=1e-13)
    f32 = K.gather_sum_f32(g.in_pointer, g.in_node_indices, x)
    assert O.within_tolerance(f32, t, rtol=1e-4, atol=1e-5)[0]
    w = rng.standard_normal((e, 4)).astype(np.float32)
    t = O.u_mul_e_sum(x, w, g.in_pointer, g.in_node_indices, g.in_edge_indices)
    assert np.allclose(K.u_mul_e_sum_f64(g.in_pointer, g.in_node_indices, g.in_edge_indices, x, w), t, rtol=1e-12, atol=1e-12)
    z = (3 * rng.standard_normal((e, 4))).astype(np.float32)
    t = O.segment_softmax(z, g.in_pointer, g.in_edge_indices)
    assert np.allclose(K.segment_softmax_f64(g.in_pointer, g.in_edge_indices, z), t, rtol=1e-12, atol=1e-15)
    r = rng.standard_normal((n, 24)).astype(np.float32)
    t = O.sddmm_u_dot_v(x, r, g.COO_src, g.COO_dst, 4)
    assert np.allclose(K.u_dot_v_f64(g.COO_src, g.COO_dst, x, r, 4), t, rtol=1e-12, atol=1e-12)
    hg = hetero_graphs()["rand_hetero"]
    xe = rng.standard_normal((hg.num_edges, 12)).astype(np.float32)
    we = rng.standard_normal((hg.num_etypes, 12, 20)).astype(np.float32)
    t = O.segment_mm(xe, we, hg.etype_pointer)
    assert np.allclose(K.segment_mm_f64(xe, we, hg.etype_pointer), t, rtol=1e-12, atol=1e-12)
    xn = rng.standard_normal((hg.num_nodes, 12)).astype(np.float32)
    t = O.segment_mm(xn[hg.COO_src.numpy()], we, hg.etype_pointer)
    assert np.allclose(K.segment_mm_f64(xn, we, hg.etype_pointer, gather=hg.COO_src), t, rtol=1e-12, atol=1e-12)


def test_general_gspmm_oracle_and_broadcast_offsets():
    """The loop oracle of the general g-SpMM reproduces the pinned operators where they overlap (mul / copy with sum),
    and the broadcast offset tables restate the reference's CalcBcastOff loop (bcast.cc:34-62)."""
    from graphiler_b200.capi import broadcast_offsets
    g = random_graph(30, 150, 3, empty_rows=True)
    rng = np.random.default_rng(3)
    x = rng.standard_normal((g.num_nodes, 2, 3)).astype(np.float32)
    w = rng.standard_normal((g.num_edges, 2, 1)).astype(np.float32)
    out, _, _ = O.gspmm("mul", "sum", g.in_pointer, g.in_node_indices, g.in_edge_indices, u=x, e=w)
    want = O.u_mul_e_sum(x.reshape(g.num_nodes, 6), w.reshape(g.num_edges, 2), g.in_pointer, g.in_node_indices, g.in_edge_indices)
    assert np.allclose(out.reshape(g.num_nodes, 6), want, rtol=1e-6, atol=1e-7)
    out, _, _ = O.gspmm("copy_lhs", "sum", g.in_pointer, g.in_node_indices, g.in_edge_indices, u=x)
    assert np.allclose(out.reshape(g.num_nodes, 6), O.spmm_src(x.reshape(g.num_nodes, 6), g.in_pointer, g.in_node_indices))
    out, au, ae = O.gspmm("copy_rhs", "max", g.in_pointer, g.in_node_indices, g.in_edge_indices, e=w)
    deg = g.in_degrees().numpy()
    assert np.isneginf(out[deg == 0]).all() and (au == 0).all()
    v = int(np.argmax(deg))
    seg = g.in_edge_indices[g.in_pointer[v]:g.in_pointer[v + 1]].numpy()
    assert out[v, 0, 0] == w[seg, 0, 0].max() and ae[v, 0, 0] == seg[np.argmax(w[seg, 0, 0])]

    def calc_bcast_off(ls, rs):                      # the reference's loop, trailing shapes only
        lo, ro, out_len, sl, sr = [0], [0], 1, 1, 1
        nd = max(len(ls), len(rs))
        for j in range(nd):
            dl = ls[len(ls) - 1 - j] if len(ls) - 1 - j >= 0 else 1
            dr = rs[len(rs) - 1 - j] if len(rs) - 1 - j >= 0 else 1
            for i in range(1, max(dl, dr)):
                for k in range(out_len):
                    lo.append(lo[k] + i * (i < dl) * sl)
                    ro.append(ro[k] + i * (i < dr) * sr)
            out_len *= max(dl, dr)
            sl, sr = sl * dl, sr * dr
        return lo, ro
    for ls, rs in (((3, 4), (3, 1)), ((4,), (1,)), ((2, 1, 5), (3, 5)), ((6,), (6,)), ((1, 4), (3, 1))):
        shape, lo, ro = broadcast_offsets(ls, rs)
        wl, wr = calc_bcast_off(ls, rs)
        assert lo.tolist() == wl and ro.tolist() == wr and int(np.prod(shape)) == len(wl)
    with pytest.raises(Exception):
        broadcast_offsets((3,), (4,))
