"""Parity of every CUDA kernel, called through the C ABI, with the float64 CPU oracle on the same
float32 inputs.  Tolerance: |gpu - truth| <= 1e-6 + 1e-5 |truth| element-wise for floating-point
reductions; bit-exact for gathers, index handling, zero rows and the plain fp32 add of u_add_v."""
import numpy as np
import pytest
import torch

from graphiler_b200 import capi, synthetic
from graphiler_b200.graph import debug_graph, debug_hetero_graph, prepare_graph
from oracle import ops_oracle as O

from pathlib import Path

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = Path(__file__).resolve().parent.parent
RTOL, ATOL = 1e-5, 1e-6


def close(got, truth, rtol=RTOL, atol=ATOL):
    ok, nbad, err = O.within_tolerance(got.float().cpu().numpy(), truth, rtol, atol)
    assert ok, f"{nbad} elements outside tolerance, max abs err {err:.3e}"


def hub_graph(n=300, e=4000, hub_deg=5000, seed=0, empty=True):
    """Power-law-ish graph: one hub destination far above the split threshold, many short rows, empty rows."""
    g = torch.Generator().manual_seed(seed)
    src = torch.randint(0, n, (e,), generator=g)
    dst = torch.randint(0, n // 2 if empty else n, (e,), generator=g)
    src = torch.cat([src, torch.randint(0, n, (hub_deg,), generator=g)])
    dst = torch.cat([dst, torch.full((hub_deg,), 7)])
    perm = torch.randperm(src.numel(), generator=g)            # edge ids unrelated to position
    return prepare_graph(src[perm], dst[perm], n)


GRAPHS = {
    "debug": debug_graph,
    "hub": hub_graph,
    "hub2": lambda: hub_graph(n=97, e=500, hub_deg=1100, seed=3, empty=False),
    "empty": lambda: prepare_graph(torch.zeros(0, dtype=torch.int64), torch.zeros(0, dtype=torch.int64), 5),
}


@pytest.fixture(params=list(GRAPHS))
def graph(request):
    return GRAPHS[request.param]()


@pytest.mark.parametrize("feat", [1, 3, 4, 16, 40, 64, 100, 128, 256, 516])
@pytest.mark.parametrize("use_plan", [False, True])
def test_spmm_copy_u_sum(graph, feat, use_plan):
    g = graph.to(DEV)
    x = torch.randn(g.num_nodes, feat, device=DEV)
    plan = capi.Plan(g.in_pointer, feat, chunk=64) if use_plan else None
    y = capi.spmm_gather_sum(g.in_pointer, g.in_node_indices, x, plan)
    truth = O.spmm_src(x, graph.in_pointer, graph.in_node_indices)
    close(y, truth)
    empty_rows = (graph.in_degrees() == 0).to(DEV)
    assert (y[empty_rows] == 0).all()


def test_spmm_result_independent_of_plan_when_no_row_is_cut():
    g = hub_graph(hub_deg=100).to(DEV)
    x = torch.randn(g.num_nodes, 64, device=DEV)
    a = capi.spmm_gather_sum(g.in_pointer, g.in_node_indices, x, None)
    b = capi.spmm_gather_sum(g.in_pointer, g.in_node_indices, x, capi.Plan(g.in_pointer, 64, chunk=512))
    assert torch.equal(a, b)
    c = capi.spmm_gather_sum(g.in_pointer, g.in_node_indices, x, capi.Plan(g.in_pointer, 64, chunk=512))
    assert torch.equal(b, c)              # deterministic across runs


@pytest.mark.parametrize("feat", [4, 64, 256, 30])
def test_spmm_epilogue_scale_relu(graph, feat):
    g = graph.to(DEV)
    x = torch.randn(g.num_nodes, feat, device=DEV)
    sc = torch.rand(g.num_nodes, device=DEV) + 0.5
    plan = capi.Plan(g.in_pointer, feat, chunk=64)
    base = capi.spmm_gather_sum(g.in_pointer, g.in_node_indices, x, plan)
    y = capi.spmm_gather_sum(g.in_pointer, g.in_node_indices, x, plan, dst_scale=sc, relu=True)
    assert torch.equal(y, torch.relu(base * sc.unsqueeze(1)))        # epilogue == the two separate fp32 passes
    truth = np.maximum(O.spmm_src(x, graph.in_pointer, graph.in_node_indices) * sc.cpu().numpy()[:, None].astype(np.float64), 0)
    close(y, truth)


@pytest.mark.parametrize("feat", [64, 256])
def test_spmm_fast_accumulation_is_plain_fp32(graph, feat):
    """GPHL_ACCUM_FAST: plain fp32 adds.  Checked at the accuracy plain fp32 summation has
    (error relative to the sum of magnitudes), not at the library's default tolerance."""
    g = graph.to(DEV)
    x = torch.randn(g.num_nodes, feat, device=DEV)
    plan = capi.Plan(g.in_pointer, feat, chunk=64)
    y = capi.spmm_gather_sum(g.in_pointer, g.in_node_indices, x, plan, fast_accum=True)
    truth = O.spmm_src(x, graph.in_pointer, graph.in_node_indices)
    mag = O.spmm_src(x.abs(), graph.in_pointer, graph.in_node_indices)
    err = np.abs(y.cpu().numpy().astype(np.float64) - truth)
    assert (err <= 1e-6 * (1 + mag)).all()



@pytest.mark.parametrize("feat", [16, 128])
def test_spmm_copy_e_sum(graph, feat):
    g = graph.to(DEV)
    m = torch.randn(g.num_edges, feat, device=DEV)
    plan = capi.Plan(g.in_pointer, feat, chunk=128)
    y = capi.spmm_gather_sum(g.in_pointer, g.in_edge_indices, m, plan)
    close(y, O.spmm_edge(m, graph.in_pointer, graph.in_edge_indices))


@pytest.mark.parametrize("feat", [64, 256])
def test_spmm_copy_u_sum_bf16(graph, feat):
    g = graph.to(DEV)
    x = torch.randn(g.num_nodes, feat, device=DEV).bfloat16()
    plan = capi.Plan(g.in_pointer, feat, chunk=64)
    y = capi.spmm_gather_sum(g.in_pointer, g.in_node_indices, x, plan)
    truth = O.spmm_src(x.float(), graph.in_pointer, graph.in_node_indices)    # oracle on the bf16-rounded inputs
    # fp32-accumulated sum rounded once to bf16: half an ulp = 2^-9 relative
    close(y, truth, rtol=2.0 ** -8, atol=1e-6)


@pytest.mark.parametrize("heads,dim", [(1, 64), (8, 8), (8, 32), (1, 1), (4, 3), (2, 20), (1, 256), (2, 8), (1, 32), (8, 4),
                                       (1, 4)])
@pytest.mark.parametrize("side", ["src", "dst"])
def test_spmm_u_mul_e_sum(graph, heads, dim, side):
    g = graph.to(DEV)
    x = torch.randn(g.num_nodes, heads * dim, device=DEV)
    w = torch.randn(g.num_edges, heads, device=DEV)
    if side == "src":
        arrs = (g.in_pointer, g.in_node_indices, g.in_edge_indices)
        ref = (graph.in_pointer, graph.in_node_indices, graph.in_edge_indices)
    else:
        arrs = (g.out_pointer, g.out_node_indices, g.out_edge_indices)
        ref = (graph.out_pointer, graph.out_node_indices, graph.out_edge_indices)
    plan = capi.Plan(arrs[0], heads * dim, chunk=96)
    y = capi.spmm_u_mul_e_sum(*arrs, x, w, plan)
    close(y, O.u_mul_e_sum(x, w, *ref))


@pytest.mark.parametrize("feat", [1, 8, 6, 64])
@pytest.mark.parametrize("idx_dtype", [torch.int64, torch.int32])
def test_sddmm_u_add_v(graph, feat, idx_dtype):
    g = graph.to(DEV)
    l = torch.randn(g.num_nodes, feat, device=DEV)
    r = torch.randn(g.num_nodes, feat, device=DEV)
    z = capi.sddmm_u_add_v(g.COO_src.to(idx_dtype), g.COO_dst.to(idx_dtype), l, r)
    expect = l.cpu()[graph.COO_src] + r.cpu()[graph.COO_dst]               # one fp32 add: bit-exact
    assert torch.equal(z.cpu(), expect.reshape(z.shape))
    close(z, O.sddmm_u_add_v(l, r, graph.COO_src, graph.COO_dst))


@pytest.mark.parametrize("heads,dim", [(8, 16), (1, 64), (3, 5), (8, 1), (8, 32), (4, 128), (2, 64), (64, 4), (32, 8), (16, 16)])
def test_sddmm_u_dot_v(graph, heads, dim):
    g = graph.to(DEV)
    l = torch.randn(g.num_nodes, heads * dim, device=DEV)
    r = torch.randn(g.num_nodes, heads * dim, device=DEV)
    z = capi.sddmm_u_dot_v(g.COO_src, g.COO_dst, l, r, heads)
    close(z, O.sddmm_u_dot_v(l, r, graph.COO_src, graph.COO_dst, heads))
    z32 = capi.sddmm_u_dot_v(g.COO_src.int(), g.COO_dst.int(), l, r, heads)
    assert torch.equal(z, z32)


@pytest.mark.parametrize("heads,dim", [(8, 16), (1, 64), (8, 32), (4, 128), (2, 64), (32, 8), (16, 16), (1, 4), (2, 4),
                                       (1, 8), (4, 4), (1, 128), (8, 64)])
@pytest.mark.parametrize("with_plan", [False, True])
def test_sddmm_u_dot_v_row_order(graph, heads, dim, with_plan):
    """The destination-row (CSC) walk returns the COO result for every edge: node-level operands gathered by source
    id, and edge-level left operands addressed by edge id (the HGT form), with and without the row-split plan."""
    g = graph.to(DEV)
    f = heads * dim
    l = torch.randn(g.num_nodes, f, device=DEV)
    r = torch.randn(g.num_nodes, f, device=DEV)
    plan = capi.Plan(g.in_pointer, f, chunk=32) if with_plan else None         # chunk 32: rows cut into pieces
    z = capi.sddmm_u_dot_v_csc(g.in_pointer, g.in_node_indices, g.in_edge_indices, l, r, heads, plan)
    close(z, O.sddmm_u_dot_v(l, r, graph.COO_src, graph.COO_dst, heads))
    if g.num_edges == 0:
        return
    le = torch.randn(g.num_edges, f, device=DEV)
    z = capi.sddmm_u_dot_v_csc(g.in_pointer, g.in_edge_indices, g.in_edge_indices, le, r, heads, plan)
    truth = O.sddmm_u_dot_v(le, r, torch.arange(graph.num_edges), graph.COO_dst, heads)
    close(z, truth)


def test_sddmm_u_dot_v_row_order_refuses_other_shapes(graph):
    g = graph.to(DEV)
    l = torch.randn(g.num_nodes, 15, device=DEV)
    with pytest.raises(capi.GphlError):
        capi.sddmm_u_dot_v_csc(g.in_pointer, g.in_node_indices, g.in_edge_indices, l, l, 3)
    l = torch.randn(g.num_nodes, 256, device=DEV)                       # 64 heads of 4 columns in a 1 KB row
    with pytest.raises(capi.GphlError):
        capi.sddmm_u_dot_v_csc(g.in_pointer, g.in_node_indices, g.in_edge_indices, l, l, 64)


@pytest.mark.parametrize("heads", [1, 8, 3, 40])
@pytest.mark.parametrize("use_plan", [False, True])
def test_segment_softmax(graph, heads, use_plan):
    g = graph.to(DEV)
    x = torch.randn(g.num_edges, heads, device=DEV) * 3
    plan = capi.Plan(g.in_pointer, heads, chunk=64) if use_plan else None
    y = capi.segment_softmax(g.in_pointer, g.in_edge_indices, x, plan)
    close(y, O.segment_softmax(x, graph.in_pointer, graph.in_edge_indices))


def test_segment_softmax_all_negative_and_huge_logits():
    graph = hub_graph()
    g = graph.to(DEV)
    x = torch.full((g.num_edges, 2), -300.0, device=DEV)
    x[:, 1] = torch.randn(g.num_edges, device=DEV) * 50 + 500
    y = capi.segment_softmax(g.in_pointer, g.in_edge_indices, x, capi.Plan(g.in_pointer, 2, chunk=64))
    assert torch.isfinite(y).all()
    close(y, O.segment_softmax(x, graph.in_pointer, graph.in_edge_indices))


@pytest.mark.parametrize("heads,dim", [(8, 8), (8, 32), (1, 64), (2, 3), (1, 1), (2, 8), (4, 4), (1, 16)])
@pytest.mark.parametrize("use_plan", [False, True])
def test_gat_fused(graph, heads, dim, use_plan):
    g = graph.to(DEV)
    el = torch.randn(g.num_nodes, heads, device=DEV) * 2
    er = torch.randn(g.num_nodes, heads, device=DEV) * 2
    z = torch.randn(g.num_nodes, heads * dim, device=DEV)
    plan = capi.Plan(g.in_pointer, heads * dim, chunk=64) if use_plan else None
    alpha = torch.zeros(g.num_edges, heads, device=DEV)
    out = capi.gat_fused(g.in_pointer, g.in_node_indices, g.in_edge_indices, el, er, z, 0.2, plan, alpha_out=alpha)
    truth, talpha = O.gat_fused(el, er, z, 0.2, graph.in_pointer, graph.in_node_indices, graph.in_edge_indices,
                                return_alpha=True)
    close(out, truth)
    close(alpha, talpha)
    # without the attention weights as an output (narrow rows then take the lane-group kernel)
    close(capi.gat_fused(g.in_pointer, g.in_node_indices, g.in_edge_indices, el, er, z, 0.2, plan), truth)
    # unfused sequence gives the same numbers within the same tolerance
    e = capi.sddmm_u_add_v(g.COO_src, g.COO_dst, el, er)
    e = torch.nn.functional.leaky_relu(e, 0.2)
    a = capi.segment_softmax(g.in_pointer, g.in_edge_indices, e, plan)
    out2 = capi.spmm_u_mul_e_sum(g.in_pointer, g.in_node_indices, g.in_edge_indices, z, a, plan)
    close(out2, truth)


@pytest.mark.parametrize("heads,dim", [(8, 8), (8, 32), (1, 64), (3, 5), (4, 128), (16, 4), (2, 16), (1, 4), (8, 64), (2, 256)])
def test_gat_head_scores(heads, dim):
    z = torch.randn(1003, heads * dim, device=DEV)
    a_s, a_d = torch.randn(heads, dim, device=DEV), torch.randn(heads, dim, device=DEV)
    el, er = capi.gat_head_scores(z, a_s, a_d)
    zv = z.double().cpu().view(-1, heads, dim)
    close(el, (zv * a_s.double().cpu()).sum(-1).numpy())
    close(er, (zv * a_d.double().cpu()).sum(-1).numpy())


def test_gat_fused_bf16():
    graph = hub_graph()
    g = graph.to(DEV)
    heads, dim = 8, 32
    el = torch.randn(g.num_nodes, heads, device=DEV)
    er = torch.randn(g.num_nodes, heads, device=DEV)
    z = torch.randn(g.num_nodes, heads * dim, device=DEV).bfloat16()
    out = capi.gat_fused(g.in_pointer, g.in_node_indices, None, el, er, z, 0.2, capi.Plan(g.in_pointer, heads * dim, 64))
    truth = O.gat_fused(el, er, z.float(), 0.2, graph.in_pointer, graph.in_node_indices, graph.in_edge_indices)
    close(out, truth, rtol=2.0 ** -8, atol=1e-6)


@pytest.mark.parametrize("dtype,shape", [(torch.float32, (16,)), (torch.float32, (3,)), (torch.float32, (4, 8, 8)),
                                         (torch.int8, (5,)), (torch.float64, (2,)), (torch.bfloat16, (128,)),
                                         (torch.float32, ())])
def test_broadcasts_bit_exact(dtype, shape):
    graph = debug_hetero_graph()
    g = graph.to(DEV)
    x = (torch.randn((g.num_nodes,) + shape, device=DEV) * 10).to(dtype)
    assert torch.equal(capi.gather_rows(g.COO_src, x), x[g.COO_src])
    assert torch.equal(capi.gather_rows(g.COO_dst.int(), x), x[g.COO_dst])
    xt = (torch.randn((g.num_ntypes,) + shape, device=DEV) * 10).to(dtype)
    assert torch.equal(capi.gather_rows(g.ntype_COO, xt), xt[g.ntype_COO])
    assert torch.equal(capi.gather_rows(g.ntype_COO, xt, idx2=g.COO_src), xt[g.ntype_COO][g.COO_src])
    xe = (torch.randn((g.num_etypes,) + shape, device=DEV) * 10).to(dtype)
    assert torch.equal(capi.gather_rows(g.etype_COO, xe), xe[g.etype_COO])


@pytest.mark.parametrize("k,n", [(16, 16), (128, 128), (20, 7), (1, 1), (64, 200), (256, 256), (100, 40), (64, 32), (33, 30),
                                 (65, 32)])
@pytest.mark.parametrize("tensor_cores", [False, True])
def test_segment_mm(k, n, tensor_cores):
    if tensor_cores and k % 4:
        pytest.skip("the tensor-core kernel needs k % 4 == 0")
    counts = [0, 130, 1, 0, 700, 63, 64, 65, 128, 257]
    m, t = sum(counts), len(counts)
    ptr = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32)
    x = torch.randn(m, k, device=DEV)
    w = torch.randn(t, k, n, device=DEV) / max(1, k) ** 0.5
    def check(got, truth, xin, scale=None):
        if not tensor_cores:
            return close(got, truth)                    # compensated SIMT kernel: the library's default tolerance
        # The tensor core truncates when it adds into its fp32 accumulator, so an output that cancels to ~0 from
        # partial sums of order 1 can miss atol 1e-6 by an ulp of the partial sum.  Allowed on top of the default
        # tolerance: 2 eps of sum_k |x_k||w_k| (any fp32 GEMM, the reference's cuBLAS call included, has sqrt(K) eps).
        mag = O.segment_mm(np.abs(xin.cpu().numpy()), np.abs(w.cpu().numpy()), ptr)
        if scale is not None:
            mag = mag * scale
        err = np.abs(got.cpu().numpy().astype(np.float64) - truth)
        assert (err <= ATOL + RTOL * np.abs(truth) + 2 * 2.0 ** -24 * mag).all(), float(err.max())

    y = capi.segment_mm(x, w, ptr.to(DEV), tensor_cores=tensor_cores)
    check(y, O.segment_mm(x, w, ptr), x)
    gi = torch.randint(0, m, (m,), device=DEV)
    y2 = capi.segment_mm(x, w, ptr.to(DEV), gather_idx=gi, tensor_cores=tensor_cores)
    check(y2, O.segment_mm(x.cpu()[gi.cpu()], w, ptr), x[gi])
    sc = torch.rand(m, device=DEV) + 0.5
    y3 = capi.segment_mm(x, w, ptr.to(DEV), row_scale=sc, relu=True, tensor_cores=tensor_cores)
    scn = sc.cpu().numpy().astype(np.float64)[:, None]
    check(y3, np.maximum(O.segment_mm(x, w, ptr) * scn, 0), x, scn)
    assert capi.tc_wait_timeouts() == 0


def test_segment_mm_tensor_cores_as_dense_layer_with_large_values():
    """One type covering all rows = a dense layer; inputs spanning many orders of magnitude keep fp32-level accuracy."""
    m, k, n = 1000, 256, 256
    x = torch.randn(m, k, device=DEV) * torch.logspace(-3, 3, m, device=DEV).unsqueeze(1)
    w = torch.randn(1, k, n, device=DEV) / 16
    ptr = torch.tensor([0, m], dtype=torch.int32, device=DEV)
    y = capi.segment_mm(x, w, ptr, tensor_cores=True)
    truth = x.double().cpu().numpy() @ w[0].double().cpu().numpy()
    err = np.abs(y.cpu().numpy() - truth)
    bound = 1e-6 * (np.abs(x.double().cpu().numpy()) @ np.abs(w[0].double().cpu().numpy()))   # ~16 eps of the magnitude sum
    assert (err <= bound + 1e-30).all()
    assert capi.tc_wait_timeouts() == 0


@pytest.mark.parametrize("name,scale", [("c1", 0.25), ("c2", 0.05), ("c3", 0.05), ("c4", 0.02), ("c5", 0.002)])
def test_ops_on_config_shaped_graphs(name, scale):
    wl = synthetic.make(name, scale=scale)
    graph = wl.graph
    g = graph.to(DEV)
    feat = {"c1": 64, "c2": 256, "c3": 16, "c4": 128, "c5": 256}[name]
    x = torch.randn(g.num_nodes, feat, device=DEV)
    plan = capi.Plan(g.in_pointer, feat)
    y = capi.spmm_gather_sum(g.in_pointer, g.in_node_indices, x, plan)
    close(y, O.spmm_src(x, graph.in_pointer, graph.in_node_indices))
    heads = 8
    w = torch.rand(g.num_edges, heads, device=DEV)
    y = capi.spmm_u_mul_e_sum(g.in_pointer, g.in_node_indices, g.in_edge_indices, x, w, plan)
    close(y, O.u_mul_e_sum(x, w, graph.in_pointer, graph.in_node_indices, graph.in_edge_indices))
    a = capi.segment_softmax(g.in_pointer, g.in_edge_indices, w * 5, plan)
    close(a, O.segment_softmax(w.cpu() * 5, graph.in_pointer, graph.in_edge_indices))


@pytest.mark.parametrize("kind,slice_lanes", [("1", ""), ("2", ""), ("3", ""), ("3", "16"), ("3", "32"), ("2", "8")])
def test_gather_accumulator_kinds(kind, slice_lanes):
    """The three exact accumulators of the gather kernels (compensated fp32, double, half of the column pairs each)
    meet the same tolerance, in the general kernel and in the column-sliced pair; the product library picks one per
    operator, the measurement build takes the choice from the environment."""
    import os
    import subprocess
    import sys
    from graphiler_b200 import build
    build.build_kernels(measure=True)
    env = dict(os.environ, GPHL_ACC=kind)
    if slice_lanes:
        env["GPHL_SLICE_LPR"] = slice_lanes
    r = subprocess.run([sys.executable, str(Path(__file__).resolve().parent / "acc_kinds_case.py")], env=env,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and r.stdout.strip().endswith("OK"), r.stdout[-2000:] + r.stderr[-2000:]


def test_bounded_wait_gives_up_and_reports():
    """Failure detection without a fault: a wait on a barrier that nothing completes runs out after its poll limit,
    is counted, and the context stays usable."""
    before = capi.tc_wait_timeouts()
    capi._check(capi.lib().gphl_debug_wait_selftest(2000, None), "wait selftest")
    torch.cuda.synchronize()
    assert capi.tc_wait_timeouts() == before + 1
    x = torch.randn(16, 4, device=DEV)
    assert torch.equal(capi.gather_rows(torch.arange(16, device=DEV), x), x)
    # restore the "healthy process" reading other tests assert on
    capi.lib().gphl_debug_reset_wait_timeouts()


def test_argument_errors_are_reported_not_fatal():
    g = debug_graph().to(DEV)
    x = torch.randn(3, 8, device=DEV)
    plan = capi.Plan(g.in_pointer, 8)
    with pytest.raises(capi.GphlError):
        capi.spmm_gather_sum(torch.zeros(10, dtype=torch.int32, device=DEV), g.in_node_indices, x, plan)
    with pytest.raises(capi.GphlError):
        capi.Plan(g.in_pointer, 8, chunk=33)
    y = capi.spmm_gather_sum(g.in_pointer, g.in_node_indices, x, plan)           # context still healthy
    close(y, O.spmm_src(x, g.in_pointer.cpu(), g.in_node_indices.cpu()))


def test_segment_mm_split_weights_are_cached_per_tensor_version():
    """The tensor-core path keeps the split copy of a weight tensor between calls; an in-place update of the weights
    (a new version of the same tensor) must be seen by the next call, and a view passed by `linear` must hit the
    entry of the tensor it views."""
    m, k, n = 300, 64, 48
    x = torch.randn(m, k, device=DEV)
    w = torch.randn(2, k, n, device=DEV) * 0.2
    ptr = torch.tensor([0, 120, m], dtype=torch.int32, device=DEV)
    y1 = capi.segment_mm(x, w, ptr, tensor_cores=True)
    y2 = capi.segment_mm(x, w, ptr, tensor_cores=True)                      # served from the cached split
    assert torch.equal(y1, y2)
    w.mul_(2.0)                                                             # exact in floating point
    y3 = capi.segment_mm(x, w, ptr, tensor_cores=True)
    assert torch.equal(y3, y1 * 2.0)
    wd = torch.randn(k, n, device=DEV) * 0.2
    d1 = capi.linear(x, wd)
    wd.add_(1.0)
    d2 = capi.linear(x, wd)
    truth = x.double().cpu().numpy() @ wd.double().cpu().numpy()
    mag = np.abs(x.double().cpu().numpy()) @ np.abs(wd.double().cpu().numpy())
    err = np.abs(d2.cpu().numpy() - truth)
    assert (err <= 1e-6 + 1e-5 * np.abs(truth) + 2 * 2.0 ** -23 * mag).all() and not torch.equal(d1, d2)
    assert capi.tc_wait_timeouts() == 0


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div", "copy_lhs", "copy_rhs"])
@pytest.mark.parametrize("reduce", ["sum", "max", "min"])
def test_general_gspmm(graph, op, reduce):
    """Every binary operator x reducer of the general g-SpMM against the loop oracle: sums within tolerance of the
    float64 sum of the float32 terms, max / min bit for bit with the neighbour and edge ids that produced them, with
    and without broadcasting ((N, H, D) against (E, H, 1)), on the reduce side and on the message side."""
    g = graph.to(DEV)
    n, e = graph.num_nodes, graph.num_edges
    gen = torch.Generator().manual_seed(17)
    shapes = [((n, 6), (e, 6)), ((n, 3, 4), (e, 3, 1))]
    for us, es in shapes:
        u = torch.randn(*us, generator=gen)
        ev = torch.randn(*es, generator=gen) + (3.0 if op == "div" else 0.0)      # keep quotients tame
        for side in ("in", "out"):
            arrs = ((graph.in_pointer, graph.in_node_indices, graph.in_edge_indices) if side == "in" else
                    (graph.out_pointer, graph.out_node_indices, graph.out_edge_indices))
            darrs = ((g.in_pointer, g.in_node_indices, g.in_edge_indices) if side == "in" else
                     (g.out_pointer, g.out_node_indices, g.out_edge_indices))
            want, wu, we = O.gspmm(op, reduce, *arrs, u=None if op == "copy_rhs" else u, e=None if op == "copy_lhs" else ev)
            res = capi.gspmm(op, reduce, *darrs, u=None if op == "copy_rhs" else u.to(DEV),
                             e=None if op == "copy_lhs" else ev.to(DEV), return_args=True)
            if reduce == "sum":
                close(res, want)
            else:
                out, au, ae = res
                assert np.array_equal(out.cpu().numpy(), want)
                if au is not None:
                    assert np.array_equal(au.cpu().numpy(), wu)
                if ae is not None:
                    assert np.array_equal(ae.cpu().numpy(), we)


def test_general_gspmm_agrees_with_the_tuned_kernels_and_rejects_bad_arguments(graph):
    g = graph.to(DEV)
    gen = torch.Generator().manual_seed(23)
    x = torch.randn(g.num_nodes, 16, generator=gen).to(DEV)
    w = torch.randn(g.num_edges, 1, generator=gen).to(DEV)
    a = capi.gspmm("mul", "sum", g.in_pointer, g.in_node_indices, g.in_edge_indices, u=x, e=w)
    b = capi.spmm_u_mul_e_sum(g.in_pointer, g.in_node_indices, g.in_edge_indices, x, w, capi.Plan(g.in_pointer, 16))
    # the general kernel rounds every product to fp32 before it sums (the operator is evaluated as written), the tuned
    # one keeps the products exact: they may differ by half an ulp of every term, whatever the sum cancels to
    mag = capi.gspmm("mul", "sum", g.in_pointer, g.in_node_indices, g.in_edge_indices, u=x.abs(), e=w.abs())
    assert ((a - b).abs() <= 1e-6 * b.abs() + 2.0 ** -23 * mag + 1e-30).all()
    a = capi.gspmm("copy_lhs", "sum", g.in_pointer, g.in_node_indices, g.in_edge_indices, u=x)
    assert torch.equal(a, capi.spmm_gather_sum(g.in_pointer, g.in_node_indices, x, capi.Plan(g.in_pointer, 16)))
    with pytest.raises(capi.GphlError):
        capi.gspmm("pow", "sum", g.in_pointer, g.in_node_indices, g.in_edge_indices, u=x, e=w)
    with pytest.raises(capi.GphlError):
        capi.gspmm("mul", "sum", g.in_pointer, g.in_node_indices, g.in_edge_indices, u=x)
    with pytest.raises(capi.GphlError):
        capi.gspmm("add", "sum", g.in_pointer, g.in_node_indices, g.in_edge_indices, u=x, e=torch.randn(g.num_edges, 5, device=DEV))


def test_scatter_rows_to_several_receivers():
    """The sending side of the sparse exchange on one GPU: three receive buffers, unequal counts (one empty), rows
    taken through an index list; every receiver holds exactly its rows at its offset and nothing else is touched."""
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(500, 24, generator=gen).to(DEV)
    idx = torch.randint(0, 500, (700,), generator=gen).to(DEV)
    bufs = [torch.full((400, 24), -7.0, device=DEV) for _ in range(3)]
    recv = [(bufs[0], 10, 0, 300), (bufs[1], 0, 300, 0), (bufs[2], 55, 300, 333)]
    capi.scatter_rows_peers(idx, x, recv)
    for b, first, pos, cnt in recv:
        want = torch.full((400, 24), -7.0, device=DEV)
        want[first:first + cnt] = x[idx[pos:pos + cnt]]
        assert torch.equal(b, want)
    with pytest.raises(capi.GphlError):
        capi.scatter_rows_peers(idx, x, [(torch.zeros(4, 23, device=DEV), 0, 0, 1)])


def test_projection_with_fan_out_epilogue():
    """The dense projection that also stores its finished rows into receivers' buffers (the fused sending side of
    the sparse exchange), on one GPU with local receive buffers: every receiver row named by the fan-out table holds
    the projected row bit for bit, the local output is the plain projection, rows not named are untouched, and the
    local output may be left out."""
    gen = torch.Generator().manual_seed(9)
    m, k, n = 700, 64, 96
    x = torch.randn(m, k, generator=gen).to(DEV)
    w = (torch.randn(k, n, generator=gen) * 0.2).to(DEV)
    sc = (torch.rand(m, generator=gen) + 0.5).to(DEV)
    plain = capi.linear(x, w, row_scale=sc)
    # receiver 0 takes every third row, receiver 1 a random multiset of rows (a row may go to several places), row 5 nowhere
    r0 = torch.arange(0, m, 3)
    r1 = torch.randint(0, m, (900,), generator=gen)
    r1 = r1[r1 != 5]
    rows = torch.cat([r0, r1])
    peer = torch.cat([torch.zeros_like(r0), torch.ones_like(r1)])
    dst = torch.cat([torch.arange(r0.numel()) + 4, torch.arange(r1.numel())])
    order = torch.argsort(rows, stable=True)
    entry = ((peer << 40) | dst)[order].to(DEV)
    ptr = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(torch.bincount(rows, minlength=m), 0)]).to(torch.int32).to(DEV)
    bufs = [torch.full((r0.numel() + 10, n), -3.0, device=DEV), torch.full((r1.numel() + 1, n), -3.0, device=DEV)]
    fan = capi.FanOut(bufs, ptr, entry)
    out = torch.empty(m, n, device=DEV)
    capi.linear_fanout(x, w, fan, row_scale=sc, out=out)
    assert torch.equal(out, plain)
    want0 = torch.full_like(bufs[0], -3.0)
    want0[4:4 + r0.numel()] = plain[r0.to(DEV)]
    want1 = torch.full_like(bufs[1], -3.0)
    want1[:r1.numel()] = plain[r1.to(DEV)]
    assert torch.equal(bufs[0], want0) and torch.equal(bufs[1], want1)
    for b in bufs:
        b.fill_(-3.0)
    capi.linear_fanout(x, w, fan, row_scale=sc, out=None)                 # nobody needs the rows locally
    assert torch.equal(bufs[0], want0) and torch.equal(bufs[1], want1)
    assert capi.tc_wait_timeouts() == 0


@pytest.mark.parametrize("m,n,copies", [(300, 256, 11), (129, 90, 19), (40, 16, 3)])
def test_projection_fan_out_with_many_entries_per_row(m, n, copies):
    """More (row, receiver) entries than a warp keeps in shared memory at once (32 rows x ``copies`` > 256), a width
    whose last columns leave through the scalar path, a last row tile that is not full, and rows without entries."""
    gen = torch.Generator().manual_seed(m + n)
    k = 32
    x = torch.randn(m, k, generator=gen).to(DEV)
    w = (torch.randn(k, n, generator=gen) * 0.2).to(DEV)
    plain = capi.linear(x, w)
    counts = torch.full((m,), copies, dtype=torch.int64)
    counts[::7] = 0                                                       # every seventh row goes nowhere
    counts[1::5] = 1
    rows = torch.repeat_interleave(torch.arange(m), counts)
    total = rows.numel()
    peer = torch.randint(0, 3, (total,), generator=gen)
    dst = torch.empty(total, dtype=torch.int64)
    sizes = []
    for p in range(3):
        sel = peer == p
        dst[sel] = torch.randperm(int(sel.sum()), generator=gen)
        sizes.append(int(sel.sum()))
    entry = ((peer << 40) | dst).to(DEV)
    ptr = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(counts, 0)]).to(torch.int32).to(DEV)
    bufs = [torch.full((s + 2, n), -3.0, device=DEV) for s in sizes]
    capi.linear_fanout(x, w, capi.FanOut(bufs, ptr, entry), out=None)
    for p in range(3):
        sel = peer == p
        want = torch.full_like(bufs[p], -3.0)
        want[dst[sel].to(DEV)] = plain[rows[sel].to(DEV)]
        assert torch.equal(bufs[p], want)
    assert capi.tc_wait_timeouts() == 0


def test_graph_handle_validates_its_arrays():
    """layers.PreparedGraph checks the arrays it is given once, on the device: an index out of range or a pointer array
    that does not end at the edge count is an error, not an out-of-bounds read by a kernel later."""
    import dataclasses
    from graphiler_b200 import layers
    g = hub_graph().to(DEV)
    layers.PreparedGraph(g)                                             # a valid graph passes (also the empty one)
    layers.PreparedGraph(GRAPHS["empty"]().to(DEV))
    bad = dataclasses.replace(g, in_node_indices=g.in_node_indices.clone())
    bad.in_node_indices[3] = g.num_nodes
    with pytest.raises(capi.GphlError, match="neighbour index"):
        layers.PreparedGraph(bad)
    bad = dataclasses.replace(g, COO_dst=g.COO_dst.clone())
    bad.COO_dst[0] = -1
    with pytest.raises(capi.GphlError, match="index lies outside"):
        layers.PreparedGraph(bad)
    bad = dataclasses.replace(g, out_pointer=g.out_pointer.clone())
    bad.out_pointer[-1] += 1
    with pytest.raises(capi.GphlError, match="pointer array"):
        layers.PreparedGraph(bad)
    layers.PreparedGraph(bad, validate=False)                           # opt-out for arrays already known to be valid
