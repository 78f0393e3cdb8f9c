"""CPU oracle for the sparse message-passing operators.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package may import this module: it is the checker used by the
tests, by the smoke check and by the CPU-baseline leg of the benchmark.

Each function restates, in numpy with float64 accumulation on the caller's (float32)
inputs, what one operator of the reference's ``my_ops`` library computes.  Citations give
the reference file and lines the restatement follows.  Where the reference only supports
one head / a feature width of 64 (src/ops/dgl_primitives/spmm.cu:191-219,
src/ops/segment_softmax/segment_softmax.cu:19-22) the restatement follows DGL's trailing
-dimension broadcast rule instead (src/ops/dgl_primitives/bcast.h:21-35).

Parity pin: the reference ships no golden vectors or per-operator tests.  These functions
are pinned (a) against a literal loop restatement on small graphs (``*_loops`` below),
(b) against the message/reduce/update semantics of the reference's example models through
``oracle/udf_oracle.py``, and (c) against the reference's own MP-DFG builder and optimizer
compiled from its sources (``oracle/build_ref.py``), which dispatch to a CPU registration
of these operators; the fixtures under ``tests/golden/`` were produced that way.

Notation: ``seg_in(v) = [in_pointer[v], in_pointer[v+1])``; position i of the segment has
source ``in_node_indices[i]`` and edge id ``in_edge_indices[i]``.  Edge-level tensors are
always indexed by edge id.
"""
from __future__ import annotations

import numpy as np

F64 = np.float64


def _np(x, dtype=None):
    if hasattr(x, "detach"):
        x = x.detach().cpu().numpy()
    x = np.asarray(x)
    return x if dtype is None else x.astype(dtype, copy=False)


def _rows2d(x: np.ndarray) -> np.ndarray:
    """View as (rows, product of trailing dims); also valid for zero rows."""
    return x.reshape(x.shape[0], int(np.prod(x.shape[1:], dtype=np.int64)) if x.ndim > 1 else 1)


def _segment_sum(vals: np.ndarray, pointer: np.ndarray) -> np.ndarray:
    """out[v] = sum of vals[pointer[v]:pointer[v+1]] in float64; empty segments give zero rows."""
    pointer = _np(pointer, np.int64)
    n = pointer.size - 1
    out = np.zeros((n,) + vals.shape[1:], dtype=F64)
    if vals.shape[0] == 0 or n == 0:
        return out
    nonempty = pointer[1:] > pointer[:-1]
    starts = pointer[:-1][nonempty]
    out[nonempty] = np.add.reduceat(vals.astype(F64, copy=False), starts, axis=0)
    return out


def get_feat_dim(x) -> int:
    """Product of the sizes of dims >= 1 (src/ops/broadcast/broadcast.cu:3-9)."""
    s = _np(x).shape
    return int(np.prod(s[1:], dtype=np.int64)) if len(s) > 1 else 1


# ---- broadcasts: row gathers (src/ops/broadcast/broadcast.cu:58-100) -------------------

def broadcast_src_node(x, COO_src):
    return _np(x)[_np(COO_src, np.int64)]


def broadcast_dst_node(x, COO_dst):
    return _np(x)[_np(COO_dst, np.int64)]


def broadcast_node_type(x, ntype_COO):
    return _np(x)[_np(ntype_COO, np.int64)]


def broadcast_edge_type(x, etype_COO):
    return _np(x)[_np(etype_COO, np.int64)]


def broadcast_src_node_type(x, ntype_COO, COO_src):
    return _np(x)[_np(ntype_COO, np.int64)][_np(COO_src, np.int64)]


def broadcast_dst_node_type(x, ntype_COO, COO_dst):
    return _np(x)[_np(ntype_COO, np.int64)][_np(COO_dst, np.int64)]


# ---- SpMM family (src/ops/dgl_primitives/spmm.cu:286-389) ------------------------------

def spmm_src(x, in_pointer, in_node_indices):
    """copy_u_sum: y[v] = sum_{i in seg_in(v)} x[in_node_indices[i]]  (spmm.cu:375-389)."""
    x = _np(x)
    x2 = _rows2d(x)
    return _segment_sum(x2[_np(in_node_indices, np.int64)], in_pointer)


def spmm_edge(m, in_pointer, in_edge_indices):
    """copy_e_sum: y[v] = sum_{i in seg_in(v)} m[in_edge_indices[i]]  (spmm.cu:359-373)."""
    m = _np(m)
    m2 = _rows2d(m)
    return _segment_sum(m2[_np(in_edge_indices, np.int64)], in_pointer)


def u_mul_e_sum(x, w, pointer, node_indices, edge_indices):
    """y[v] = sum_i x[node_indices[i]] * w[edge_indices[i]] over the segment of v.

    With the CSC arrays this is ``gspmm_src_mul_e_sum`` (spmm.cu:286-320), with the CSR
    arrays ``gspmm_dst_mul_e_sum`` (spmm.cu:322-356).  x is (N, H*D) (or (N,H,D)); w is
    (E,), (E,1) or (E,H): one scale per edge and head, broadcast over the D columns of the
    head (bcast.h:21-35).  The reference itself handles only H == 1.
    """
    x = _np(x)
    w = _np(w)
    n_feat = int(np.prod(x.shape[1:], dtype=np.int64)) if x.ndim > 1 else 1
    x2 = x.reshape(x.shape[0], n_feat).astype(F64)
    w2 = _rows2d(w).astype(F64)
    h = w2.shape[1]
    assert n_feat % h == 0, "feature width must be a multiple of the head count"
    d = n_feat // h
    xs = x2[_np(node_indices, np.int64)].reshape(-1, h, d)
    ws = w2[_np(edge_indices, np.int64)].reshape(-1, h, 1)
    return _segment_sum((xs * ws).reshape(-1, n_feat), pointer)


def src_mul_e_sum(x, w, in_pointer, in_node_indices, in_edge_indices):
    return u_mul_e_sum(x, w, in_pointer, in_node_indices, in_edge_indices)


def dst_mul_e_sum(x, w, out_pointer, out_node_indices, out_edge_indices):
    return u_mul_e_sum(x, w, out_pointer, out_node_indices, out_edge_indices)


# ---- SDDMM family (src/ops/dgl_primitives/sddmm.cu:118-129, sddmm.cuh:34-120) -----------

def gspmm(op, reduce, pointer, node_indices, edge_indices, u=None, e=None):
    """General g-SpMM, literal loops (small inputs): SpMMCsrKernel with its functors (src/ops/dgl_primitives/
    spmm.cuh:30-75, functor.cuh:18-213) and numpy broadcasting of the trailing dimensions (bcast.cc:20-77).
    The binary operator is evaluated in float32 as the reference does; sums are returned in float64 (truth for a
    tolerance check), max / min in float32 (bit-exact), with the arguments of the first extreme position; an empty
    row gives -inf / +inf and argument 0.  Returns (out, arg_u, arg_e)."""
    ptr, nid, eid = _np(pointer, np.int64), _np(node_indices, np.int64), _np(edge_indices, np.int64)
    uu = None if u is None else _np(u, np.float32)
    ee = None if e is None else _np(e, np.float32)
    f = {"add": np.add, "sub": np.subtract, "mul": np.multiply, "div": np.divide,
         "copy_lhs": lambda a, b: a, "copy_rhs": lambda a, b: b}[op]
    n = ptr.shape[0] - 1
    if op == "copy_lhs":
        trailing = uu.shape[1:]
    elif op == "copy_rhs":
        trailing = ee.shape[1:]
    else:
        trailing = np.broadcast_shapes(uu.shape[1:], ee.shape[1:])
    out = np.zeros((n,) + tuple(trailing), dtype=np.float64 if reduce == "sum" else np.float32)
    au, ae = np.zeros(out.shape, dtype=np.int32), np.zeros(out.shape, dtype=np.int32)
    if reduce != "sum":
        out[...] = -np.inf if reduce == "max" else np.inf
    with np.errstate(divide="ignore", invalid="ignore"):
        for v in range(n):
            for i in range(ptr[v], ptr[v + 1]):
                a = None if uu is None else uu[nid[i]]
                b = None if ee is None else ee[eid[i]]
                val = np.broadcast_to(np.asarray(f(a, b), dtype=np.float32), trailing)
                if reduce == "sum":
                    out[v] += val.astype(np.float64)
                else:
                    better = out[v] < val if reduce == "max" else out[v] > val
                    out[v] = np.where(better, val, out[v])
                    if op != "copy_rhs":                      # arguments only for the operands the operator reads
                        au[v] = np.where(better, nid[i], au[v])
                    if op != "copy_lhs":
                        ae[v] = np.where(better, eid[i], ae[v])
    return out, au, ae


def sddmm_u_add_v(lhs, rhs, COO_src, COO_dst):
    """z[e] = lhs[COO_src[e]] + rhs[COO_dst[e]]; the ``alpha`` argument of the registered
    operator is ignored by the reference (sddmm.cu:116-129)."""
    l = _np(lhs)
    r = _np(rhs)
    l2 = _rows2d(l).astype(F64)
    r2 = _rows2d(r).astype(F64)
    return l2[_np(COO_src, np.int64)] + r2[_np(COO_dst, np.int64)]


def sddmm_u_dot_v(lhs, rhs, COO_src, COO_dst, heads: int):
    """z[e,h] = sum_d lhs[src,h,d] * rhs[dst,h,d] (functor ``binary::Dot``,
    functor.cuh:103-116; the tree-reduce kernel sddmm.cuh:80-120).  The reference registers
    no operator for it; its HGT flow computes the same value with mul + sum on gathered rows."""
    l = _np(lhs, F64)
    r = _np(rhs, F64)
    l3 = l.reshape(l.shape[0], heads, -1)
    r3 = r.reshape(r.shape[0], heads, -1)
    return (l3[_np(COO_src, np.int64)] * r3[_np(COO_dst, np.int64)]).sum(-1)


# ---- segment softmax (src/ops/segment_softmax/segment_softmax_kernel.cu:4-49) ------------

def segment_softmax(x, in_pointer, in_edge_indices):
    """Per destination v and per trailing column: softmax over x[in_edge_indices[seg_in(v)]],
    written back at the same edge ids.  True softmax (maximum taken over the segment, not
    clamped at zero as segment_softmax_kernel.cu:9 does; the two agree unless every logit of
    a segment is below about -87).  Edge ids outside every segment keep 0."""
    x = _np(x)
    shape = x.shape
    x2 = _rows2d(x).astype(F64)
    ptr = _np(in_pointer, np.int64)
    eid = _np(in_edge_indices, np.int64)
    y = np.zeros_like(x2)
    if eid.size == 0:
        return y.reshape(shape)
    xs = x2[eid]
    deg = ptr[1:] - ptr[:-1]
    nonempty = deg > 0
    starts = ptr[:-1][nonempty]
    mx = np.maximum.reduceat(xs, starts, axis=0)
    row_of = np.repeat(np.arange(int(nonempty.sum())), deg[nonempty])
    ex = np.exp(xs - mx[row_of])
    den = np.add.reduceat(ex, starts, axis=0)
    y[eid] = ex / den[row_of]
    return y.reshape(shape)


# ---- typed linear (src/ops/segment_mm/segment_mm.cu:4-33) ---------------------------------

def segment_mm(x, w, type_pointer):
    """y[p_t:p_{t+1}] = x[p_t:p_{t+1}] @ w[t] for every type t."""
    x = _np(x, F64)
    w = _np(w, F64)
    p = _np(type_pointer, np.int64)
    y = np.zeros((x.shape[0], w.shape[2]), dtype=F64)
    for t in range(p.size - 1):
        y[p[t]:p[t + 1]] = x[p[t]:p[t + 1]] @ w[t]
    return y


# ---- fused attention: SDDMM u_add_v -> leaky-relu -> edge softmax -> u_mul_e_sum -----------

def leaky_relu(x, slope):
    return np.where(x >= 0, x, x * slope)


def gat_fused(el, er, z, slope, in_pointer, in_node_indices, in_edge_indices, return_alpha=False):
    """out[v,h,:] = sum_i softmax_i(leaky_relu(el[u_i,h] + er[v,h])) * z[u_i,h,:].

    The composition of the three operators the reference's optimised GAT graph runs
    (gsddmm_u_add_v_mul_alpha -> aten::leaky_relu_ -> SegmentSoftmax -> gspmm_src_mul_e_sum);
    the reference has no single operator for it."""
    el = _np(el, F64)
    er = _np(er, F64)
    h = el.shape[1] if el.ndim > 1 else 1
    el = el.reshape(-1, h)
    er = er.reshape(-1, h)
    ptr = _np(in_pointer, np.int64)
    col = _np(in_node_indices, np.int64)
    eid = _np(in_edge_indices, np.int64)
    n = ptr.size - 1
    dst_of_pos = np.repeat(np.arange(n), ptr[1:] - ptr[:-1])
    logits_pos = leaky_relu(el[col] + er[dst_of_pos], slope)          # CSC position order
    logits = np.zeros((eid.size, h), dtype=F64)
    logits[eid] = logits_pos
    alpha = segment_softmax(logits, ptr, eid)
    out = u_mul_e_sum(z, alpha, ptr, col, eid)
    return (out, alpha) if return_alpha else out


# ---- literal loop restatements (small graphs only; used to pin the vectorised code) --------

def spmm_src_loops(x, in_pointer, in_node_indices):
    x = _np(x, F64)
    x = _rows2d(x)
    ptr = _np(in_pointer, np.int64)
    col = _np(in_node_indices, np.int64)
    out = np.zeros((ptr.size - 1, x.shape[1]), dtype=F64)
    for v in range(ptr.size - 1):
        for i in range(ptr[v], ptr[v + 1]):
            out[v] += x[col[i]]
    return out


def u_mul_e_sum_loops(x, w, pointer, node_indices, edge_indices):
    x = _np(x, F64)
    x = _rows2d(x)
    w = _np(w, F64)
    w = _rows2d(w)
    h = w.shape[1]
    d = x.shape[1] // h
    ptr = _np(pointer, np.int64)
    col = _np(node_indices, np.int64)
    eid = _np(edge_indices, np.int64)
    out = np.zeros((ptr.size - 1, x.shape[1]), dtype=F64)
    for v in range(ptr.size - 1):
        for i in range(ptr[v], ptr[v + 1]):
            for hh in range(h):
                out[v, hh * d:(hh + 1) * d] += x[col[i], hh * d:(hh + 1) * d] * w[eid[i], hh]
    return out


def segment_softmax_loops(x, in_pointer, in_edge_indices):
    x = _np(x, F64)
    shape = x.shape
    x = _rows2d(x)
    ptr = _np(in_pointer, np.int64)
    eid = _np(in_edge_indices, np.int64)
    y = np.zeros_like(x)
    for v in range(ptr.size - 1):
        ids = eid[ptr[v]:ptr[v + 1]]
        if ids.size == 0:
            continue
        for c in range(x.shape[1]):
            seg = x[ids, c]
            ex = np.exp(seg - seg.max())
            y[ids, c] = ex / ex.sum()
    return y.reshape(shape)


def within_tolerance(got, truth, rtol=1e-5, atol=1e-6):
    """Element-wise |got - truth| <= atol + rtol * |truth| against the float64 truth;
    returns (ok, number of violations, max abs error)."""
    got = _np(got, F64).reshape(-1)
    truth = _np(truth, F64).reshape(-1)
    err = np.abs(got - truth)
    bad = err > (atol + rtol * np.abs(truth))
    bad |= ~np.isfinite(got)
    return (not bad.any()), int(bad.sum()), float(err.max() if err.size else 0.0)
