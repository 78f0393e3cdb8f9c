"""Property-style parity on generated small graphs: random sizes with duplicate edges, self-loops, empty rows and a
hub row, feature widths that are not multiples of 4 or 32, one or several heads."""
import numpy as np
import pytest
import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from graphiler_b200 import capi
from graphiler_b200.graph import prepare_graph
from oracle import ops_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@st.composite
def graphs(draw):
    n = draw(st.integers(1, 60))
    e = draw(st.integers(0, 300))
    seed = draw(st.integers(0, 2 ** 16))
    hub = draw(st.sampled_from([0, 0, 150, 700]))
    g = torch.Generator().manual_seed(seed)
    src = torch.randint(0, n, (e + hub,), generator=g)
    dst = torch.cat([torch.randint(0, max(1, n - n // 3), (e,), generator=g), torch.full((hub,), n // 2)])
    return prepare_graph(src, dst, n), seed


def close(got, truth):
    ok, bad, err = O.within_tolerance(got.float().cpu().numpy(), truth)
    assert ok, f"{bad} elements outside rtol 1e-5 / atol 1e-6 (max abs err {err:.2e})"


@settings(max_examples=40, deadline=None, suppress_health_check=list(HealthCheck))
@given(graphs(), st.sampled_from([1, 2, 5, 8, 12, 33, 64, 100]), st.sampled_from([32, 64, 512]))
def test_copy_u_sum(gs, feat, chunk):
    g, seed = gs
    d = g.to(DEV)
    x = torch.randn(g.num_nodes, feat, generator=torch.Generator().manual_seed(seed))
    y = capi.spmm_gather_sum(d.in_pointer, d.in_node_indices, x.to(DEV), capi.Plan(d.in_pointer, feat, chunk=chunk))
    close(y, O.spmm_src(x, g.in_pointer, g.in_node_indices))


@settings(max_examples=40, deadline=None, suppress_health_check=list(HealthCheck))
@given(graphs(), st.sampled_from([(1, 1), (1, 8), (2, 4), (8, 4), (3, 7), (8, 16)]))
def test_softmax_and_attention(gs, hd):
    g, seed = gs
    heads, dim = hd
    d = g.to(DEV)
    gen = torch.Generator().manual_seed(seed + 1)
    logits = torch.randn(g.num_edges, heads, generator=gen) * 4
    plan = capi.Plan(d.in_pointer, heads * dim, chunk=64)
    close(capi.segment_softmax(d.in_pointer, d.in_edge_indices, logits.to(DEV), plan),
          O.segment_softmax(logits, g.in_pointer, g.in_edge_indices))
    el, er = torch.randn(g.num_nodes, heads, generator=gen), torch.randn(g.num_nodes, heads, generator=gen)
    z = torch.randn(g.num_nodes, heads * dim, generator=gen)
    out = capi.gat_fused(d.in_pointer, d.in_node_indices, d.in_edge_indices, el.to(DEV), er.to(DEV), z.to(DEV), 0.2, plan)
    close(out, O.gat_fused(el, er, z, 0.2, g.in_pointer, g.in_node_indices, g.in_edge_indices))
    w = torch.randn(g.num_edges, heads, generator=gen)
    close(capi.spmm_u_mul_e_sum(d.in_pointer, d.in_node_indices, d.in_edge_indices, z.to(DEV), w.to(DEV), plan),
          O.u_mul_e_sum(z, w, g.in_pointer, g.in_node_indices, g.in_edge_indices))
