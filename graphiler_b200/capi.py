"""ctypes binding of the C ABI in include/gphl.h, with torch tensors as device memory.

This is the Python-side mirror of the operator set the reference registers as ``my_ops::*``
(src/ops/**): same names, same argument meaning.  There is no CPU path: every function
requires CUDA tensors and raises if the native library is missing.
"""
from __future__ import annotations

import ctypes
import weakref
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_void_p, POINTER
from pathlib import Path
from typing import Optional

import torch

LIB_DIR = Path(__file__).resolve().parent / "lib"
KERNEL_LIB = LIB_DIR / "libgphl.so"
TORCH_OPS_LIB = LIB_DIR / "libgraphiler.so"
DEFAULT_CHUNK = 512
ACCUM_FAST = 1        # GPHL_ACCUM_FAST
EPILOGUE_RELU = 2     # GPHL_EPILOGUE_RELU

_lib = None

# name -> (restype, argtypes); must list every symbol include/gphl.h declares.
_P = c_void_p
SIGNATURES = {
    "gphl_last_error": (c_char_p, []),
    "gphl_version": (c_int, []),
    "gphl_launch_count": (c_int64, []),
    "gphl_plan_create": (c_int, [_P, c_int64, c_int32, c_int64, _P, POINTER(_P)]),
    "gphl_plan_bind_scratch": (c_int, [_P, _P, c_int64]),
    "gphl_plan_num_pieces": (c_int64, [_P]),
    "gphl_validate_csr": (c_int, [_P, c_int64, c_int64, _P, c_int64, _P, c_int64, _P]),
    "gphl_validate_index_i64": (c_int, [_P, c_int64, c_int64, _P]),
    "gphl_plan_destroy": (None, [_P]),
    "gphl_plan_num_items": (c_int64, [_P]),
    "gphl_plan_num_split_rows": (c_int64, [_P]),
    "gphl_plan_scratch_bytes": (c_int64, [_P]),
    "gphl_spmm_gather_sum_f32": (c_int, [_P, _P, _P, c_int64, c_int64, _P, _P, _P]),
    "gphl_spmm_gather_sum_bf16": (c_int, [_P, _P, _P, c_int64, c_int64, _P, _P, _P]),
    "gphl_spmm_gather_sum_ex_f32": (c_int, [_P, _P, _P, c_int64, c_int64, _P, _P, c_int32, _P, _P]),
    "gphl_spmm_gather_sum_ex_bf16": (c_int, [_P, _P, _P, c_int64, c_int64, _P, _P, c_int32, _P, _P]),
    "gphl_spmm_u_mul_e_sum_f32": (c_int, [_P, _P, _P, _P, c_int64, c_int64, c_int64, _P, _P, _P, _P]),
    "gphl_sddmm_u_add_v_f32_i64": (c_int, [_P, _P, c_int64, c_int64, _P, _P, _P, _P]),
    "gphl_sddmm_u_add_v_f32_i32": (c_int, [_P, _P, c_int64, c_int64, _P, _P, _P, _P]),
    "gphl_sddmm_u_dot_v_f32_i64": (c_int, [_P, _P, c_int64, c_int64, c_int64, _P, _P, _P, _P]),
    "gphl_sddmm_u_dot_v_f32_i32": (c_int, [_P, _P, c_int64, c_int64, c_int64, _P, _P, _P, _P]),
    "gphl_segment_mm_tc_prepare_weights": (c_int, [_P, c_int64, c_int64, c_int64, _P, _P]),
    "gphl_segment_mm_tc_prepared_f32": (c_int, [_P, _P, _P, c_int64, c_int64, c_int64, c_int64, _P, _P, c_int32, _P, _P]),
    "gphl_segment_mm_tc_fanout_f32": (c_int, [_P, _P, _P, c_int64, c_int64, c_int64, c_int64, _P, c_int32, _P, c_int32, _P, _P, _P, _P]),
    "gphl_scatter_rows_peers_i64": (c_int, [_P, c_int32, _P, _P, _P, _P, c_int64, _P, _P]),
    "gphl_gspmm_f32": (c_int, [c_int32, c_int32, _P, _P, _P, c_int64, c_int64, _P, c_int64, _P, c_int64, _P, _P, _P, _P, _P, _P]),
    "gphl_sddmm_u_dot_v_csc_f32": (c_int, [_P, _P, _P, _P, c_int64, c_int64, c_int64, _P, _P, _P, _P]),
    "gphl_segment_softmax_f32": (c_int, [_P, _P, _P, c_int64, c_int64, _P, _P, _P, _P]),
    "gphl_segment_softmax_noalloc_f32": (c_int, [_P, _P, c_int64, c_int64, _P, _P, _P]),
    "gphl_gat_fused_f32": (c_int, [_P, _P, _P, _P, c_int64, c_int64, c_int64, _P, _P, _P, c_float, _P, _P, _P, _P]),
    "gphl_gat_fused_bf16": (c_int, [_P, _P, _P, c_int64, c_int64, c_int64, _P, _P, _P, c_float, _P, _P, _P]),
    "gphl_gat_fused_ex_f32": (c_int, [_P, _P, _P, _P, c_int64, c_int64, c_int64, _P, _P, _P, c_float, c_int32, _P, _P, _P,
                                      _P]),
    "gphl_gat_fused_ex_bf16": (c_int, [_P, _P, _P, c_int64, c_int64, c_int64, _P, _P, _P, c_float, c_int32, _P, _P, _P]),
    "gphl_gat_head_scores_f32": (c_int, [_P, _P, _P, c_int64, c_int64, c_int64, _P, _P, _P]),
    "gphl_gather_rows_i64": (c_int, [_P, _P, c_int64, c_int64, _P, _P, _P]),
    "gphl_gather_rows_i32": (c_int, [_P, _P, c_int64, c_int64, _P, _P, _P]),
    "gphl_segment_mm_f32": (c_int, [_P, _P, _P, c_int64, c_int64, c_int64, c_int64, _P, _P, _P]),
    "gphl_segment_mm_tc_workspace_bytes": (c_int64, [c_int64, c_int64, c_int64]),
    "gphl_segment_mm_tc_f32": (c_int, [_P, _P, _P, c_int64, c_int64, c_int64, c_int64, _P, _P, c_int32, _P, _P, _P]),
    "gphl_tc_wait_timeouts": (c_int, [POINTER(c_int)]),
    "gphl_debug_wait_selftest": (c_int, [c_int32, _P]),
    "gphl_debug_reset_wait_timeouts": (c_int, []),
}


class GphlError(RuntimeError):
    pass


def load_library(path: Optional[Path] = None, make_default: bool = False):
    """dlopen libgphl.so and set the prototypes.  Raises if it has not been built.  ``make_default`` makes the
    library at ``path`` the one every wrapper of this module calls (the per-kernel timer uses it to load the
    measurement build)."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = Path(path) if path else KERNEL_LIB
    if not p.exists():
        raise GphlError(f"{p} is missing: run `python -m graphiler_b200.build` (there is no fallback path)")
    lib = ctypes.CDLL(str(p))
    for name, (res, args) in SIGNATURES.items():
        if not hasattr(lib, name):
            raise GphlError(f"{p} does not export {name}: rebuild with `python -m graphiler_b200.build --force`")
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    if path is None or make_default:
        _lib = lib
    return lib


def lib():
    return load_library()


def _check(rc: int, what: str):
    if rc != 0:
        raise GphlError(f"{what} failed ({rc}): {lib().gphl_last_error().decode()}")


def _ptr(t: Optional[torch.Tensor], empty: Optional[torch.Tensor] = None):
    """Device address of ``t``.  An empty tensor has no storage; where the C ABI wants a non-null
    array that it will never read (the index arrays of an edgeless graph), ``empty`` lends its address."""
    if t is None:
        return None
    if t.numel() == 0 and empty is not None:
        return c_void_p(empty.data_ptr())
    return c_void_p(t.data_ptr())


def _stream(t: torch.Tensor):
    return c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _dev(*ts, dtypes=None):
    """All tensors must be contiguous CUDA tensors on one device."""
    dev = None
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise GphlError("operators need CUDA tensors (there is no CPU path)")
        if not t.is_contiguous():
            raise GphlError("operators need contiguous tensors")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise GphlError("all tensors must live on one device")
    return dev


def launch_count() -> int:
    return int(lib().gphl_launch_count())


class Plan:
    """Row-split plan for one pointer array (see gphl_plan_create)."""

    def __init__(self, pointer: torch.Tensor, max_feat: int, chunk: int = DEFAULT_CHUNK):
        _dev(pointer)
        assert pointer.dtype == torch.int32
        self._h = c_void_p()
        self.n_rows = pointer.numel() - 1
        self.pointer = pointer
        with torch.cuda.device(pointer.device):
            _check(lib().gphl_plan_create(_ptr(pointer), self.n_rows, chunk, max_feat, _stream(pointer),
                                          ctypes.byref(self._h)), "gphl_plan_create")

    @property
    def handle(self):
        return self._h

    @property
    def num_items(self):
        return int(lib().gphl_plan_num_items(self._h))

    @property
    def num_split_rows(self):
        return int(lib().gphl_plan_num_split_rows(self._h))

    @property
    def scratch_bytes(self):
        return int(lib().gphl_plan_scratch_bytes(self._h))

    def __del__(self):
        try:
            if self._h:
                lib().gphl_plan_destroy(self._h)
                self._h = c_void_p()
        except Exception:
            pass


def validate_csr(pointer, idx, idx_limit: int, edge_idx=None, edge_limit: int = 0) -> None:
    """Raise GphlError unless `pointer` is a non-decreasing array from 0 to len(idx) and every index is in range
    (one pass on the device; synchronises).  The kernels themselves trust these arrays."""
    _dev(pointer, idx, edge_idx)
    with torch.cuda.device(pointer.device):
        _check(lib().gphl_validate_csr(_ptr(pointer), pointer.numel() - 1, idx.numel(), _ptr(idx), idx_limit,
                                       _ptr(edge_idx), edge_limit, _stream(pointer)), "validate_csr")


def validate_index(index, limit: int) -> None:
    """Raise GphlError unless every value of the int64 array lies in [0, limit)."""
    _dev(index)
    assert index.dtype == torch.int64
    with torch.cuda.device(index.device):
        _check(lib().gphl_validate_index_i64(_ptr(index), index.numel(), limit, _stream(index)), "validate_index")


def _h(plan: Optional[Plan]):
    return None if plan is None else plan.handle


def _feat(x: torch.Tensor) -> int:
    f = 1
    for s in x.shape[1:]:
        f *= s
    return f


def spmm_gather_sum(pointer, idx, x, plan: Optional[Plan] = None, out=None, dst_scale=None, relu: bool = False,
                    fast_accum: bool = False):
    """y[v] = sum over the segment of v of x[idx[i]] (SpMMSrc with node indices, SpMMEdge with edge ids);
    optionally followed in the same kernel by ``y[v] *= dst_scale[v]`` and ``max(y, 0)``."""
    _dev(pointer, idx, x, out, dst_scale)
    n_rows, f = pointer.numel() - 1, _feat(x)
    y = out if out is not None else torch.empty((n_rows, f), dtype=x.dtype, device=x.device)
    fn = {torch.float32: lib().gphl_spmm_gather_sum_ex_f32, torch.bfloat16: lib().gphl_spmm_gather_sum_ex_bf16}[x.dtype]
    flags = (ACCUM_FAST if fast_accum else 0) | (EPILOGUE_RELU if relu else 0)
    if dst_scale is not None and (dst_scale.dtype != torch.float32 or dst_scale.numel() != n_rows):
        raise GphlError("dst_scale must hold one float32 per output row")
    with torch.cuda.device(x.device):
        _check(fn(_h(plan), _ptr(pointer), _ptr(idx, pointer), n_rows, f, _ptr(x, pointer), _ptr(dst_scale), flags,
                  _ptr(y), _stream(x)), "spmm_gather_sum")
    return y


def spmm_u_mul_e_sum(pointer, node_idx, edge_idx, x, w, plan: Optional[Plan] = None, out=None):
    _dev(pointer, node_idx, edge_idx, x, w, out)
    n_rows, f = pointer.numel() - 1, _feat(x)
    heads = _feat(w)
    if f % heads:
        raise GphlError("feature width must be a multiple of the number of weight columns")
    y = out if out is not None else torch.empty((n_rows, f), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _check(lib().gphl_spmm_u_mul_e_sum_f32(_h(plan), _ptr(pointer), _ptr(node_idx, pointer), _ptr(edge_idx, pointer),
                                               n_rows, heads, f // heads, _ptr(x), _ptr(w, pointer), _ptr(y), _stream(x)),
               "spmm_u_mul_e_sum")
    return y


def sddmm_u_add_v(src, dst, l, r, out=None):
    _dev(src, dst, l, r, out)
    e, f = src.numel(), _feat(l)
    z = out if out is not None else torch.empty((e, f), dtype=torch.float32, device=l.device)
    fn = lib().gphl_sddmm_u_add_v_f32_i64 if src.dtype == torch.int64 else lib().gphl_sddmm_u_add_v_f32_i32
    with torch.cuda.device(l.device):
        _check(fn(_ptr(src), _ptr(dst), e, f, _ptr(l), _ptr(r), _ptr(z), _stream(l)), "sddmm_u_add_v")
    return z


def sddmm_u_dot_v(src, dst, l, r, heads: int, out=None):
    _dev(src, dst, l, r, out)
    e, f = src.numel(), _feat(l)
    z = out if out is not None else torch.empty((e, heads), dtype=torch.float32, device=l.device)
    fn = lib().gphl_sddmm_u_dot_v_f32_i64 if src.dtype == torch.int64 else lib().gphl_sddmm_u_dot_v_f32_i32
    with torch.cuda.device(l.device):
        _check(fn(_ptr(src), _ptr(dst), e, heads, f // heads, _ptr(l), _ptr(r), _ptr(z), _stream(l)), "sddmm_u_dot_v")
    return z


GSPMM_OPS = {"add": 0, "sub": 1, "mul": 2, "div": 3, "copy_lhs": 4, "copy_rhs": 5}
GSPMM_REDUCERS = {"sum": 0, "max": 1, "min": 2}


def broadcast_offsets(lhs_shape, rhs_shape):
    """Column offsets of a broadcast binary operator on the trailing dimensions of two row tensors (the reference's
    CalcBcastOff, src/ops/dgl_primitives/bcast.cc:20-77): the output's trailing shape is the right-aligned numpy
    broadcast of the two; returns (out_shape, lhs_offsets, rhs_offsets) with one flat offset per output column, last
    dimension fastest."""
    import numpy as np
    ls, rs = tuple(lhs_shape), tuple(rhs_shape)
    nd = max(len(ls), len(rs))
    ls, rs = (1,) * (nd - len(ls)) + ls, (1,) * (nd - len(rs)) + rs
    out = tuple(max(a, b) for a, b in zip(ls, rs))
    for a, b, o in zip(ls, rs, out):
        if a not in (1, o) or b not in (1, o):
            raise GphlError(f"shapes {lhs_shape} and {rhs_shape} do not broadcast")
    idx = np.indices(out).reshape(nd, -1) if nd else np.zeros((0, 1), dtype=np.int64)

    def offsets(shape):
        off, stride = np.zeros(idx.shape[1], dtype=np.int64), 1
        for d in range(nd - 1, -1, -1):
            if shape[d] != 1:
                off += idx[d] * stride
            stride *= shape[d]
        return off
    return out, offsets(ls), offsets(rs)


def gspmm(op: str, reduce: str, pointer, node_idx, edge_idx, u=None, e=None, return_args: bool = False):
    """General g-SpMM over one side of the graph: out[v] = reduce_i op(u[node_idx[i]], e[edge_idx[i]]) with numpy
    broadcasting over the trailing dimensions.  Returns out, or (out, arg_u, arg_e) for max / min with
    ``return_args`` (int32; None for an operand the operator does not read)."""
    _dev(pointer, node_idx, edge_idx, u, e)
    if op not in GSPMM_OPS or reduce not in GSPMM_REDUCERS:
        raise GphlError(f"gspmm: unknown operator {op!r} or reducer {reduce!r}")
    use_l, use_r = op != "copy_rhs", op != "copy_lhs"
    if (use_l and u is None) or (use_r and e is None):
        raise GphlError(f"gspmm: operator {op} needs " + ("u" if use_l and u is None else "e"))
    n_rows = pointer.numel() - 1
    dev = pointer.device
    if use_l and use_r:
        trailing, lo, ro = broadcast_offsets(u.shape[1:], e.shape[1:])
        same = tuple(u.shape[1:]) == tuple(e.shape[1:])
        uoff = eoff = None
        if not same:
            uoff, eoff = torch.from_numpy(lo).to(dev), torch.from_numpy(ro).to(dev)
    else:
        trailing, uoff, eoff = tuple((u if use_l else e).shape[1:]), None, None
    out_len = 1
    for d in trailing:
        out_len *= d
    out = torch.empty((n_rows,) + tuple(trailing), dtype=torch.float32, device=dev)
    want_args = return_args and reduce != "sum"
    au = torch.zeros(out.shape, dtype=torch.int32, device=dev) if want_args and use_l else None
    ae = torch.zeros(out.shape, dtype=torch.int32, device=dev) if want_args and use_r else None
    with torch.cuda.device(dev):
        _check(lib().gphl_gspmm_f32(GSPMM_OPS[op], GSPMM_REDUCERS[reduce], _ptr(pointer), _ptr(node_idx, pointer),
                                    _ptr(edge_idx), n_rows, out_len, _ptr(u, pointer) if use_l else None,
                                    _feat(u) if use_l else 0, _ptr(e, pointer) if use_r else None, _feat(e) if use_r else 0,
                                    _ptr(uoff), _ptr(eoff), _ptr(out),
                                    _ptr(au), _ptr(ae), _stream(pointer)), "gspmm")
    return (out, au, ae) if return_args and reduce != "sum" else out


def sddmm_u_dot_v_csc(pointer, idx, edge_idx, l, r, heads: int, plan: Optional[Plan] = None, out=None):
    """u_dot_v walked in destination-row order: out[edge_idx[i], h] = sum_d l[idx[i], h, d] * r[v, h, d] for every
    position i of row v (``edge_idx`` None: edge id == position).  Raises GphlError for shapes only the COO form covers."""
    _dev(pointer, idx, edge_idx, l, r, out)
    n_rows, e, f = pointer.numel() - 1, idx.numel(), _feat(l)
    z = out if out is not None else torch.empty((e, heads), dtype=torch.float32, device=l.device)
    with torch.cuda.device(l.device):
        _check(lib().gphl_sddmm_u_dot_v_csc_f32(_h(plan), _ptr(pointer), _ptr(idx, pointer), _ptr(edge_idx), n_rows, heads,
                                                f // heads, _ptr(l, pointer), _ptr(r, pointer), _ptr(z, pointer),
                                                _stream(l)), "sddmm_u_dot_v_csc")
    return z


def segment_softmax(pointer, edge_idx, x, plan: Optional[Plan] = None, out=None, stats=None):
    _dev(pointer, edge_idx, x, out, stats)
    n_rows, heads = pointer.numel() - 1, _feat(x)
    y = out if out is not None else torch.empty_like(x)     # every edge id of a valid graph lies in one segment
    if stats is None:
        stats = torch.empty(max(1, 2 * n_rows * heads), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _check(lib().gphl_segment_softmax_f32(_h(plan), _ptr(pointer), _ptr(edge_idx, pointer), n_rows, heads,
                                              _ptr(x, pointer), _ptr(y, pointer), _ptr(stats), _stream(x)), "segment_softmax")
    return y


SOFTMAX_NOALLOC_MAX_ROW_HEADS = 1 << 20


def segment_softmax_noalloc(pointer, edge_idx, x, out):
    """Segment softmax through the entry point that allocates nothing: the caller passes the output
    tensor too, and ``rows * heads`` must not exceed ``SOFTMAX_NOALLOC_MAX_ROW_HEADS``.  For callers
    that cannot obtain device memory at call time; calls on one device must not overlap."""
    _dev(pointer, edge_idx, x, out)
    if out.shape != x.shape or out.dtype != x.dtype or not out.is_contiguous():
        raise GphlError("segment_softmax_noalloc: `out` must be a contiguous tensor of x's shape and dtype")
    n_rows, heads = pointer.numel() - 1, _feat(x)
    with torch.cuda.device(x.device):
        _check(lib().gphl_segment_softmax_noalloc_f32(_ptr(pointer), _ptr(edge_idx, pointer), n_rows, heads,
                                                      _ptr(x, pointer), _ptr(out, pointer), _stream(x)),
               "segment_softmax_noalloc")
    return out


def gat_fused(pointer, node_idx, edge_idx, el, er, z, slope: float, plan: Optional[Plan] = None,
              out=None, alpha_out=None, stats=None, fast_accum: bool = False):
    _dev(pointer, node_idx, edge_idx, el, er, z, out, alpha_out, stats)
    n_rows, heads, f = pointer.numel() - 1, _feat(el), _feat(z)
    y = out if out is not None else torch.empty((n_rows, f), dtype=z.dtype, device=z.device)
    if stats is None:
        stats = torch.empty(max(1, 2 * n_rows * heads), dtype=torch.float32, device=z.device)
    flags = ACCUM_FAST if fast_accum else 0
    with torch.cuda.device(z.device):
        if z.dtype == torch.float32:
            _check(lib().gphl_gat_fused_ex_f32(_h(plan), _ptr(pointer), _ptr(node_idx, pointer), _ptr(edge_idx, pointer),
                                               n_rows, heads, f // heads, _ptr(el), _ptr(er), _ptr(z), float(slope),
                                               flags, _ptr(y), _ptr(alpha_out), _ptr(stats), _stream(z)), "gat_fused")
        else:
            _check(lib().gphl_gat_fused_ex_bf16(_h(plan), _ptr(pointer), _ptr(node_idx, pointer), n_rows, heads,
                                                f // heads, _ptr(el), _ptr(er), _ptr(z), float(slope), flags, _ptr(y),
                                                _ptr(stats), _stream(z)), "gat_fused_bf16")
    return y


def gat_head_scores(z, attn_src, attn_dst, el=None, er=None):
    """el[n,h] = sum_d z[n,h,d] attn_src[h,d], er likewise: the dense prologue of the GAT layer, one pass over z."""
    _dev(z, attn_src, attn_dst, el, er)
    heads, dim = attn_src.shape
    n = z.shape[0]
    if _feat(z) != heads * dim:
        raise GphlError("z must have heads * dim columns")
    el = el if el is not None else torch.empty((n, heads), dtype=torch.float32, device=z.device)
    er = er if er is not None else torch.empty((n, heads), dtype=torch.float32, device=z.device)
    with torch.cuda.device(z.device):
        _check(lib().gphl_gat_head_scores_f32(_ptr(z), _ptr(attn_src), _ptr(attn_dst), n, heads, dim, _ptr(el), _ptr(er),
                                              _stream(z)), "gat_head_scores")
    return el, er


def gather_rows(idx, x, idx2=None, out=None):
    """y[i] = x[idx[i]] (or x[idx[idx2[i]]]) for any dtype and trailing shape."""
    _dev(idx, idx2, x, out)
    n_out = (idx2 if idx2 is not None else idx).numel()
    row_bytes = _feat(x) * x.element_size()
    y = out if out is not None else torch.empty((n_out,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    fn = lib().gphl_gather_rows_i64 if idx.dtype == torch.int64 else lib().gphl_gather_rows_i32
    with torch.cuda.device(x.device):
        _check(fn(_ptr(idx), _ptr(idx2), n_out, row_bytes, _ptr(x), _ptr(y), _stream(x)), "gather_rows")
    return y


def scatter_rows_peers(idx, x, receivers):
    """One launch that stores rows of ``x`` into several receivers' buffers (which may be peer-mapped memory of other
    GPUs): ``receivers`` is a list of ``(buffer, first_row_in_buffer, first_position_in_idx, count)``; receiver p gets
    ``x[idx[first_position + k]]`` at row ``first_row + k`` of its buffer."""
    _dev(idx, x)
    assert idx.dtype == torch.int64
    n = len(receivers)
    row_bytes = _feat(x) * x.element_size()
    arr = lambda vals: (c_int64 * n)(*vals)
    ptrs = (c_void_p * n)(*[b.data_ptr() for b, _, _, _ in receivers])
    for b, _, _, _ in receivers:
        if b.dtype != x.dtype or _feat(b) != _feat(x) or not b.is_contiguous():
            raise GphlError("scatter_rows_peers: receiver buffers must be contiguous, of x's dtype and row width")
    with torch.cuda.device(x.device):
        _check(lib().gphl_scatter_rows_peers_i64(_ptr(idx), n, arr([r[2] for r in receivers]), arr([r[3] for r in receivers]),
                                                 ptrs, arr([r[1] for r in receivers]), row_bytes, _ptr(x), _stream(x)),
               "scatter_rows_peers")


def segment_mm(x, w, type_pointer, gather_idx=None, out=None, row_scale=None, relu: bool = False,
               tensor_cores: Optional[bool] = None, workspace=None, _weights_owner=None):
    """y[p_t:p_{t+1}] = x[p_t:p_{t+1}] @ w[t] (rows of x optionally taken through ``gather_idx``), optionally followed
    by a per-row scale and relu.  ``tensor_cores``: None = use the tcgen05 kernel whenever the shape allows
    (k % 4 == 0) and the weights are not narrow (k <= 64 and n <= 32 go to the double-accumulating narrow kernel,
    which is bound by the rows it moves), True = require it, False = the exact-fp32 SIMT kernels."""
    _dev(x, w, type_pointer, gather_idx, out, row_scale, workspace)
    m = gather_idx.numel() if gather_idx is not None else x.shape[0]
    t, k, n = w.shape
    if x.shape[1] != k:
        raise GphlError("inner dimensions differ")
    y = out if out is not None else torch.empty((m, n), dtype=torch.float32, device=x.device)
    tc_ok = (k % 4 == 0) and x.data_ptr() % 16 == 0 and y.data_ptr() % 16 == 0
    narrow = k <= 64 and n <= 32
    use_tc = (tc_ok and not narrow) if tensor_cores is None else tensor_cores
    if use_tc and not tc_ok:
        raise GphlError("the tensor-core kernel needs k % 4 == 0 and 16-byte aligned tensors")
    with torch.cuda.device(x.device):
        if use_tc:
            need = int(lib().gphl_segment_mm_tc_workspace_bytes(t, k, n))
            if workspace is not None:
                if workspace.numel() * workspace.element_size() < need:
                    raise GphlError(f"segment_mm: the workspace must hold {need} bytes")
                _check(lib().gphl_segment_mm_tc_f32(_ptr(x), _ptr(w), _ptr(type_pointer), t, m, k, n, _ptr(gather_idx),
                                                    _ptr(row_scale), 1 if relu else 0, _ptr(workspace), _ptr(y), _stream(x)),
                       "segment_mm_tc")
            else:
                ws = _prepared_weights(w if _weights_owner is None else _weights_owner, w, t, k, n, need, _stream(x))
                _check(lib().gphl_segment_mm_tc_prepared_f32(_ptr(x), _ptr(ws), _ptr(type_pointer), t, m, k, n,
                                                             _ptr(gather_idx), _ptr(row_scale), 1 if relu else 0, _ptr(y),
                                                             _stream(x)), "segment_mm_tc_prepared")
        else:
            _check(lib().gphl_segment_mm_f32(_ptr(x), _ptr(w), _ptr(type_pointer), t, m, k, n, _ptr(gather_idx), _ptr(y),
                                             _stream(x)), "segment_mm")
            if row_scale is not None:
                y.mul_(row_scale.reshape(-1, 1))
            if relu:
                torch.relu_(y)
    return y


_PREPARED = {}      # id(tensor) -> (weak reference to the tensor, key, workspace); tensors compare element-wise, so not a WeakKeyDictionary


def _prepared_weights(owner, w, t, k, n, need, stream):
    """The split, transposed copy of a weight tensor for the tensor-core kernel, made once per (tensor object, version,
    storage address, shape, stream): weights are constants of a layer.  An entry dies with its tensor.  ``owner`` is
    the tensor object the caller keeps (a view of it may be what is passed as ``w``)."""
    key = (owner._version, w.data_ptr(), tuple(w.shape), getattr(stream, "value", stream))
    oid = id(owner)
    hit = _PREPARED.get(oid)
    if hit is not None and hit[0]() is owner and hit[1] == key:
        return hit[2]
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=w.device)
    _check(lib().gphl_segment_mm_tc_prepare_weights(_ptr(w), t, k, n, _ptr(ws), stream), "segment_mm_tc_prepare_weights")
    _PREPARED[oid] = (weakref.ref(owner, lambda _r, oid=oid: _PREPARED.pop(oid, None)), key, ws)
    return ws


_ONE_TYPE = {}


def linear(x, w, row_scale=None, relu: bool = False, out=None, workspace=None):
    """Dense layer ``relu?(row_scale * (x @ w))`` on the tensor cores: the typed linear with a single type covering
    all rows.  fp32 in / out with fp32-level accuracy (three-way bf16 split, six products)."""
    key = (x.device, x.shape[0])
    ptr = _ONE_TYPE.get(key)
    if ptr is None:
        if len(_ONE_TYPE) > 64:
            _ONE_TYPE.clear()
        ptr = _ONE_TYPE[key] = torch.tensor([0, x.shape[0]], dtype=torch.int32, device=x.device)
    return segment_mm(x, w.unsqueeze(0) if w.dim() == 2 else w, ptr, out=out, row_scale=row_scale, relu=relu,
                      tensor_cores=True, workspace=workspace, _weights_owner=w)


class FanOut:
    """Where the finished rows of a projection go besides its own output: ``bases`` (one (rows, n) float32 receive
    buffer per receiver, possibly peer-mapped memory of another GPU), ``ptr`` ((m + 1) int32, device) and ``entry``
    (int64, device: receiver << 40 | row in its buffer); see gphl_segment_mm_tc_fanout_f32."""

    def __init__(self, bases, ptr, entry):
        self.bases, self.ptr, self.entry = list(bases), ptr, entry


def linear_fanout(x, w, fan: FanOut, row_scale=None, relu: bool = False, out=None):
    """``relu?(row_scale * (x @ w))`` on the tensor cores with every finished row also stored into the receivers'
    buffers from the kernel's epilogue (the sending side of the sparse exchange fused into the projection).  ``out``
    may be None when the rows are not needed locally; returns ``out``."""
    _dev(x, w, row_scale, out, fan.ptr, fan.entry)
    m, k = x.shape
    n = w.shape[-1]
    if k % 4 != 0 or x.data_ptr() % 16 or (out is not None and out.data_ptr() % 16) or x.dtype != torch.float32:
        raise GphlError("linear_fanout needs float32 rows of k % 4 == 0 columns, 16-byte aligned")
    if fan.ptr.numel() != m + 1 or fan.ptr.dtype != torch.int32 or fan.entry.dtype != torch.int64:
        raise GphlError("linear_fanout: fan.ptr must hold m + 1 int32 values, fan.entry int64")
    for b in fan.bases:
        if b.dtype != torch.float32 or _feat(b) != n or not b.is_contiguous():
            raise GphlError("linear_fanout: receive buffers must be contiguous float32 matrices of n columns")
    key = (x.device, m)
    ptr = _ONE_TYPE.get(key)
    if ptr is None:
        ptr = _ONE_TYPE[key] = torch.tensor([0, m], dtype=torch.int32, device=x.device)
    w3 = w.unsqueeze(0) if w.dim() == 2 else w
    need = int(lib().gphl_segment_mm_tc_workspace_bytes(1, k, n))
    bases = (c_void_p * len(fan.bases))(*[b.data_ptr() for b in fan.bases])
    with torch.cuda.device(x.device):
        ws = _prepared_weights(w, w3, 1, k, n, need, _stream(x))
        _check(lib().gphl_segment_mm_tc_fanout_f32(_ptr(x), _ptr(ws), _ptr(ptr), 1, m, k, n, _ptr(row_scale), 1 if relu else 0,
                                                   _ptr(out), len(fan.bases), bases, _ptr(fan.ptr), _ptr(fan.entry, fan.ptr),
                                                   _stream(x)), "segment_mm_tc_fanout")
    return out


def tc_wait_timeouts() -> int:
    c = c_int(0)
    _check(lib().gphl_tc_wait_timeouts(ctypes.byref(c)), "gphl_tc_wait_timeouts")
    return int(c.value)
