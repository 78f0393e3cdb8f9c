"""Parity at the stated sizes: the four model configurations at scale 1.0, per operator and per layer.

Per operator the truth is the double-precision destination-row loop of oracle/csr_cpu.c (checked against the numpy
oracle, which is pinned on the reference operators' recorded outputs, in tests/test_oracle_cpu.py) on the same
float32 inputs; the bound is |gpu - truth| <= 1e-6 + 1e-5 |truth| on every element (bit-exact for u_add_v and the
row gathers; the tensor-core typed linear adds 2 ulp of sum |x||w|, as in tests/test_kernels_gpu.py).  Per layer the
protocol of tests/test_layers_gpu.py is run on the whole graph: the user-defined-function restatement in float64
is the truth, in float32 the yardstick.  The scale-sweep configuration (62 M edges) is checked at full size
inside bench.py, on every destination row.
"""
import numpy as np
import pytest
import torch

from graphiler_b200 import capi, layers, synthetic
from oracle import csr_cpu as K
from oracle import ops_oracle as O
from oracle import udf_oracle as U

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def close(got, truth, extra=None):
    got = got.float().cpu().numpy().reshape(np.asarray(truth).shape)
    err = np.abs(got.astype(np.float64) - truth)
    lim = 1e-6 + 1e-5 * np.abs(truth) + (0 if extra is None else extra)
    bad = int((err > lim).sum()) + int((~np.isfinite(got)).sum())
    assert bad == 0, f"{bad} of {err.size} elements outside the bound (max abs err {err.max():.3e})"


def rn(seed, *shape):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed))


@pytest.fixture(scope="module")
def workloads():
    cache = {}

    def get(name):
        if name not in cache:
            cache[name] = synthetic.make(name, scale=1.0)
        return cache[name]
    return get


@pytest.mark.parametrize("name,feat,heads", [("c1", 64, 8), ("c2", 256, 1), ("c2", 40, 1), ("c3", 16, 1), ("c4", 128, 8)])
def test_row_reductions_full_size(workloads, name, feat, heads):
    wl = workloads(name)
    graph = wl.graph
    g = graph.to(DEV)
    n, e = graph.num_nodes, graph.num_edges
    x, w, lg = rn(1, n, feat), torch.rand(e, heads, generator=torch.Generator().manual_seed(2)), rn(3, e, heads) * 3
    xd, wd = x.to(DEV), w.to(DEV)
    plan = capi.Plan(g.in_pointer, feat)
    ptr, nid, eid = graph.in_pointer, graph.in_node_indices, graph.in_edge_indices
    close(capi.spmm_gather_sum(g.in_pointer, g.in_node_indices, xd, plan), K.gather_sum_f64(ptr, nid, x))
    close(capi.spmm_u_mul_e_sum(g.in_pointer, g.in_node_indices, g.in_edge_indices, xd, wd, plan),
          K.u_mul_e_sum_f64(ptr, nid, eid, x, w))
    close(capi.segment_softmax(g.in_pointer, g.in_edge_indices, lg.to(DEV), plan), K.segment_softmax_f64(ptr, eid, lg))
    # copy_e_sum: one message row per edge, addressed by edge id
    m = rn(4, e, min(feat, 64))
    close(capi.spmm_gather_sum(g.in_pointer, g.in_edge_indices, m.to(DEV), capi.Plan(g.in_pointer, m.shape[1])),
          K.gather_sum_f64(ptr, eid, m))


@pytest.mark.parametrize("name,heads,dim", [("c1", 8, 8), ("c4", 8, 16)])
def test_sddmm_and_attention_full_size(workloads, name, heads, dim):
    wl = workloads(name)
    graph = wl.graph
    g = graph.to(DEV)
    n, e, f = graph.num_nodes, graph.num_edges, heads * dim
    el, er, z = rn(5, n, heads), rn(6, n, heads), rn(7, n, f)
    got = capi.sddmm_u_add_v(g.COO_src, g.COO_dst, el.to(DEV), er.to(DEV))
    assert torch.equal(got.cpu(), el[graph.COO_src] + er[graph.COO_dst])                 # one fp32 add: bit-exact
    l, r = rn(8, n, f), rn(9, n, f)
    truth = K.u_dot_v_f64(graph.COO_src, graph.COO_dst, l, r, heads)
    close(capi.sddmm_u_dot_v(g.COO_src, g.COO_dst, l.to(DEV), r.to(DEV), heads), truth)
    close(capi.sddmm_u_dot_v_csc(g.in_pointer, g.in_node_indices, g.in_edge_indices, l.to(DEV), r.to(DEV), heads,
                                 capi.Plan(g.in_pointer, f)), truth)
    out = capi.gat_fused(g.in_pointer, g.in_node_indices, g.in_edge_indices, el.to(DEV), er.to(DEV), z.to(DEV), 0.2,
                         capi.Plan(g.in_pointer, f))
    close(out, O.gat_fused(el, er, z, 0.2, graph.in_pointer, graph.in_node_indices, graph.in_edge_indices))
    # the six row gathers, bit for bit
    x = rn(10, n, 12)
    assert torch.equal(capi.gather_rows(g.COO_src, x.to(DEV)).cpu(), x[graph.COO_src])
    assert torch.equal(capi.gather_rows(g.COO_dst, x.to(DEV)).cpu(), x[graph.COO_dst])
    if graph.ntype_COO is not None:
        t = rn(11, graph.num_ntypes, 6)
        assert torch.equal(capi.gather_rows(g.ntype_COO, t.to(DEV)).cpu(), t[graph.ntype_COO])
        assert torch.equal(capi.gather_rows(g.ntype_COO, t.to(DEV), idx2=g.COO_src).cpu(), t[graph.ntype_COO[graph.COO_src]])
        assert torch.equal(capi.gather_rows(g.ntype_COO, t.to(DEV), idx2=g.COO_dst).cpu(), t[graph.ntype_COO[graph.COO_dst]])
        te = rn(12, graph.num_etypes, 6)
        assert torch.equal(capi.gather_rows(g.etype_COO, te.to(DEV)).cpu(), te[graph.etype_COO])


@pytest.mark.parametrize("name,k,nout", [("c3", 16, 16), ("c4", 128, 128)])
def test_typed_linear_full_size(workloads, name, k, nout):
    wl = workloads(name)
    graph = wl.graph
    g = graph.to(DEV)
    n, e = graph.num_nodes, graph.num_edges
    x = rn(13, n, k)
    eps2 = 2 * 2.0 ** -23
    if graph.ntype_pointer is not None:
        wn = rn(14, graph.num_ntypes, k, nout) * 0.2
        truth = K.segment_mm_f64(x, wn, graph.ntype_pointer)
        mag = K.segment_mm_f64(x.abs(), wn.abs(), graph.ntype_pointer)
        close(capi.segment_mm(x.to(DEV), wn.to(DEV), g.ntype_pointer), truth, extra=eps2 * mag)
    we = rn(15, graph.num_etypes, k, nout) * 0.2
    truth = K.segment_mm_f64(x, we, graph.etype_pointer, gather=graph.COO_src)
    mag = K.segment_mm_f64(x.abs(), we.abs(), graph.etype_pointer, gather=graph.COO_src)
    close(capi.segment_mm(x.to(DEV), we.to(DEV), g.etype_pointer, gather_idx=g.COO_src), truth, extra=eps2 * mag)
    assert capi.tc_wait_timeouts() == 0


# ---- layers, whole graphs ------------------------------------------------------------------------------------------

def assess(got, truth64, ref32):
    truth = truth64.numpy()
    _, bad_ref, _ = O.within_tolerance(ref32.numpy(), truth)
    _, bad_got, err = O.within_tolerance(got.float().cpu().numpy(), truth)
    norm_err = err / max(1e-30, float(np.abs(truth).max()))
    assert norm_err <= 1e-5, f"normalised max error {norm_err:.3e}"
    assert bad_got <= max(bad_ref, truth.size // 1000), f"{bad_got} violations vs {bad_ref} for the fp32 CPU path"


def d64(t):
    return t.double()


def test_gat_layer_full_size(workloads):
    wl = workloads("c1")
    p, hy = wl.params, wl.hyper
    truth = U.gat_layer(wl.graph, d64(wl.feats), d64(p["fc_weight"]), d64(p["attn_src"]), d64(p["attn_dst"]), hy["slope"])
    ref32 = U.gat_layer(wl.graph, wl.feats, p["fc_weight"], p["attn_src"], p["attn_dst"], hy["slope"])
    w = wl.to(DEV)
    pg = layers.PreparedGraph(w.graph)
    for fused in (True, False):
        out = layers.gat_layer(pg, w.feats, w.params["fc_weight"], w.params["attn_src"], w.params["attn_dst"], hy["slope"],
                               fused=fused)
        assess(out, truth, ref32)


def test_gcn_two_layers_full_size(workloads):
    wl = workloads("c2")
    g = wl.graph
    norm = g.in_degrees().clamp(min=1).float().pow(-0.5).unsqueeze(1)
    t1 = U.gcn_layer(g, d64(wl.feats), d64(wl.params["w1"]), d64(norm), d64(norm))
    truth = U.gcn_layer(g, t1, d64(wl.params["w2"]), d64(norm), d64(norm), relu=False)
    del t1
    r1 = U.gcn_layer(g, wl.feats, wl.params["w1"], norm, norm)
    ref32 = U.gcn_layer(g, r1, wl.params["w2"], norm, norm, relu=False)
    w = wl.to(DEV)
    pg = layers.PreparedGraph(w.graph)
    n = layers.gcn_norms(pg)
    h = layers.gcn_layer(pg, w.feats, w.params["w1"], n, n)
    out = layers.gcn_layer(pg, h, w.params["w2"], n, n, relu=False)
    assess(out, truth, ref32)


def test_rgcn_two_layers_full_size(workloads):
    wl = workloads("c3")
    g, p, norm = wl.graph, wl.params, wl.edata["norm"]
    t1 = torch.relu(U.rgcn_layer(g, d64(wl.feats), d64(p["w1"]), d64(norm)))
    truth = U.rgcn_layer(g, t1, d64(p["w2"]), d64(norm))
    r1 = torch.relu(U.rgcn_layer(g, wl.feats, p["w1"], norm))
    ref32 = U.rgcn_layer(g, r1, p["w2"], norm)
    w = wl.to(DEV)
    pg = layers.PreparedGraph(w.graph)
    h = torch.relu(layers.rgcn_layer(pg, w.feats, w.params["w1"], w.edata["norm"]))
    out = layers.rgcn_layer(pg, h, w.params["w2"], w.edata["norm"])
    assess(out, truth, ref32)


def test_hgt_layer_full_size(workloads):
    wl = workloads("c4")
    g, hy = wl.graph, wl.hyper
    p64 = {k: d64(v) for k, v in wl.params.items()}
    truth = U.hgt_layer_typed(g, d64(wl.feats), p64, hy["heads"], hy["sqrt_dk"])
    ref32 = U.hgt_layer_typed(g, wl.feats, wl.params, hy["heads"], hy["sqrt_dk"])
    w = wl.to(DEV)
    pg = layers.PreparedGraph(w.graph)
    out = layers.hgt_layer(pg, w.feats, w.params, hy["heads"], hy["sqrt_dk"])
    assess(out, truth, ref32)
