"""Parity pinned on the reference's own operators.

tests/golden/ref_ops_golden.npz holds what the reference's CUDA operator library (its src/ops/**/*.cu and
src/dglgraph.cpp, compiled unmodified by oracle/build_ref_cuda.py) returned on a B200 for the seeded cases
of tests/ref_ops_cases.py.  Three checks:

* CPU: oracle/ops_oracle.py reproduces every recorded output — bit for bit for gathers and `u_add_v`,
  and for the float32 reductions within rtol 1e-5 / atol 1e-6 plus the rounding allowance of a plain
  float32 sum of the same terms (the reference accumulates in float32; the oracle in float64).
* GPU, through the C ABI: this package's kernels reproduce the same recorded outputs under the same bound.
* GPU, live: when oracle/_ref/libgraphiler_ref.so is present, the reference operators are run again in a
  child process on this machine's GPU and compared with the oracle, so the fixture cannot go stale.
"""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import ref_ops_cases as C

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden" / "ref_ops_golden.npz"


def _check_against(recorded, name, gname, op, inp, graphs, got=None):
    """Compare `got` (default: the recorded reference output) with the oracle for one case."""
    g = graphs[gname]
    truth, bound = C.oracle_eval(op, g, inp)
    ref = recorded[name] if got is None else got
    assert tuple(ref.shape) == tuple(np.asarray(truth).shape) or ref.size == np.asarray(truth).size, \
        f"{name}: shape {ref.shape} vs {np.asarray(truth).shape}"
    if bound is None:
        assert ref.dtype == np.asarray(truth).dtype or op == "gsddmm_u_add_v_mul_alpha", name
        assert np.array_equal(ref.reshape(-1), np.asarray(truth).reshape(-1)), f"{name}: not bit-exact"
    else:
        err = np.abs(ref.astype(np.float64).reshape(-1) - truth.reshape(-1))
        lim = np.broadcast_to(bound, truth.shape).reshape(-1)
        bad = int((err > lim).sum()) + int((~np.isfinite(ref)).sum())
        assert bad == 0, f"{name}: {bad} of {err.size} elements outside the bound (max abs err {err.max():.3e})"


@pytest.fixture(scope="module")
def recorded():
    assert GOLDEN.exists(), "tests/golden/ref_ops_golden.npz is missing"
    return np.load(GOLDEN)


def test_fixture_covers_every_case_and_inputs_reproduce(recorded):
    meta = json.loads(bytes(recorded["__meta__"]).decode())
    assert "B200" in meta["gpu"]
    cases = C.cases()
    assert meta["cases"] == len(cases)
    for name, _, _, inp in cases:
        assert name in recorded.files, name
        assert int(recorded[name + "__crc"]) == C.input_checksum(inp), f"{name}: inputs differ from the recorded run"
    ops = {op for _, _, op, _ in cases}
    assert ops >= {"SpMMSrc", "SpMMEdge", "gspmm_src_mul_e_sum", "gspmm_dst_mul_e_sum", "SegmentSoftmax",
                   "gsddmm_u_add_v_mul_alpha", "BroadcastSrcNode", "BroadcastDstNode", "BroadcastNodeType",
                   "BroadcastSrcNodeType", "BroadcastDstNodeType", "BroadcastEdgeType", "SegmentMMNode", "SegmentMMEdge"}


def test_oracle_matches_reference_operators(recorded):
    graphs = C.graphs()
    for name, gname, op, inp in C.cases():
        _check_against(recorded, name, gname, op, inp, graphs)


# ---- GPU: the product's kernels, through the C ABI, against the reference's recorded outputs -------------

def _run_product(op, g, inp):
    from graphiler_b200 import capi
    x = inp.get("x")
    if op == "SpMMSrc":
        return capi.spmm_gather_sum(g.in_pointer, g.in_node_indices, x, capi.Plan(g.in_pointer, x.shape[1]))
    if op == "SpMMEdge":
        return capi.spmm_gather_sum(g.in_pointer, g.in_edge_indices, x, capi.Plan(g.in_pointer, x.shape[1]))
    if op == "gspmm_src_mul_e_sum":
        return capi.spmm_u_mul_e_sum(g.in_pointer, g.in_node_indices, g.in_edge_indices, x, inp["w"],
                                     capi.Plan(g.in_pointer, x.shape[1]))
    if op == "gspmm_dst_mul_e_sum":
        return capi.spmm_u_mul_e_sum(g.out_pointer, g.out_node_indices, g.out_edge_indices, x, inp["w"],
                                     capi.Plan(g.out_pointer, x.shape[1]))
    if op == "SegmentSoftmax":
        return capi.segment_softmax(g.in_pointer, g.in_edge_indices, x, capi.Plan(g.in_pointer, 1))
    if op == "gsddmm_u_add_v_mul_alpha":
        return capi.sddmm_u_add_v(g.COO_src, g.COO_dst, inp["l"], inp["r"])
    if op == "BroadcastSrcNode":
        return capi.gather_rows(g.COO_src, x)
    if op == "BroadcastDstNode":
        return capi.gather_rows(g.COO_dst, x)
    if op == "BroadcastNodeType":
        return capi.gather_rows(g.ntype_COO, x)
    if op == "BroadcastEdgeType":
        return capi.gather_rows(g.etype_COO, x)
    if op == "BroadcastSrcNodeType":
        return capi.gather_rows(g.ntype_COO, x, idx2=g.COO_src)
    if op == "BroadcastDstNodeType":
        return capi.gather_rows(g.ntype_COO, x, idx2=g.COO_dst)
    if op == "SegmentMMNode":
        return capi.segment_mm(x, inp["w"], g.ntype_pointer)
    if op == "SegmentMMEdge":
        return capi.segment_mm(x, inp["w"], g.etype_pointer)
    raise KeyError(op)


@pytest.mark.gpu
def test_kernels_match_reference_operators(recorded):
    from graphiler_b200 import capi
    capi.load_library()
    dev = "cuda:0"
    graphs = C.graphs()
    dgraphs = {k: g.to(dev) for k, g in graphs.items()}
    n0 = capi.launch_count()
    for name, gname, op, inp in C.cases():
        got = _run_product(op, dgraphs[gname], {k: v.to(dev) for k, v in inp.items()})
        torch.cuda.synchronize()
        got = got.cpu().numpy()
        ref = recorded[name]
        assert got.size == ref.size, f"{name}: {got.shape} vs the reference's {ref.shape}"
        # against the oracle under the reference's own bound ...
        _check_against(recorded, name, gname, op, inp, graphs, got=got.reshape(ref.shape))
        # ... and directly against what the reference returned
        truth, bound = C.oracle_eval(op, graphs[gname], inp)
        if bound is None:
            assert np.array_equal(got.reshape(-1), ref.reshape(-1)), f"{name}: differs from the reference bit pattern"
        else:
            lim = 2 * np.broadcast_to(bound, truth.shape).reshape(-1)
            err = np.abs(got.astype(np.float64).reshape(-1) - ref.astype(np.float64).reshape(-1))
            assert not (err > lim).any(), f"{name}: max abs difference from the reference {err.max():.3e}"
    assert capi.launch_count() > n0


@pytest.mark.gpu
def test_reference_operators_live_match_oracle(tmp_path, recorded):
    so = ROOT / "oracle" / "_ref" / "libgraphiler_ref.so"
    if not so.exists():
        pytest.skip("oracle/_ref/libgraphiler_ref.so was not built (the reference's source tree is needed once)")
    r = subprocess.run([sys.executable, str(ROOT / "tests" / "golden" / "make_ref_ops_golden.py"), str(tmp_path)],
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    live = np.load(tmp_path / "ref_ops_golden.npz")
    graphs = C.graphs()
    for name, gname, op, inp in C.cases():
        assert int(live[name + "__crc"]) == int(recorded[name + "__crc"])
        _check_against(live, name, gname, op, inp, graphs)
