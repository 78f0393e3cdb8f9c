"""TEST INFRASTRUCTURE: builds and binds oracle/csr_cpu.c, the C restatement of the destination-row reductions.

Used by the parity tests at the stated graph sizes (double-precision truth in seconds where numpy takes minutes)
and by bench.py's CPU baseline leg (the float form, timed on all host cores).  Nothing of the product imports it.

    python oracle/csr_cpu.py        builds oracle/lib/liboracle_cpu.so with gcc -O3 -fopenmp (no -march=native:
                                    the file travels to machines with other CPUs)
"""
from __future__ import annotations

import ctypes as C
import subprocess
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
SRC = HERE / "csr_cpu.c"
LIB = HERE / "lib" / "liboracle_cpu.so"
_lib = None


def build(force: bool = False) -> Path:
    if LIB.exists() and not force and LIB.stat().st_mtime >= SRC.stat().st_mtime:
        return LIB
    LIB.parent.mkdir(exist_ok=True)
    cmd = ["gcc", "-O3", "-fopenmp", "-fPIC", "-shared", "-std=c11", "-mavx2", "-mfma", str(SRC), "-o", str(LIB), "-lm"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("gcc failed on oracle/csr_cpu.c:\n" + r.stdout + r.stderr)
    return LIB


def load():
    global _lib
    if _lib is None:
        if not LIB.exists() or LIB.stat().st_mtime < SRC.stat().st_mtime:
            build()
        _lib = C.CDLL(str(LIB))
        _lib.csr_num_threads.restype = C.c_int
    return _lib


def _p(a, ctype):
    return None if a is None else a.ctypes.data_as(C.POINTER(ctype))


def _np(t, dtype):
    """Contiguous numpy view of a torch tensor / array in the given dtype (copies only when it must)."""
    if t is None:
        return None
    if hasattr(t, "detach"):
        t = t.detach().cpu().numpy()
    return np.ascontiguousarray(t, dtype=dtype)


def num_threads() -> int:
    return int(load().csr_num_threads())


def set_threads(n: int) -> None:
    load().csr_set_threads(C.c_int(int(n)))


def gather_sum_f32(ptr, idx, x, dst_scale=None, relu=False, rows=None, out=None):
    """Float sum (the reference's arithmetic); returns the full (n_rows, feat) array, rows outside `rows` untouched."""
    ptr, idx, x = _np(ptr, np.int32), _np(idx, np.int32), _np(x, np.float32)
    n = ptr.shape[0] - 1
    r0, r1 = (0, n) if rows is None else rows
    feat = x.shape[1]
    if out is None:
        out = np.zeros((n, feat), dtype=np.float32)
    sc = _np(dst_scale, np.float32)
    load().csr_gather_sum_f32(_p(ptr, C.c_int32), _p(idx, C.c_int32), C.c_int64(r0), C.c_int64(r1), C.c_int64(feat),
                              _p(x, C.c_float), _p(sc, C.c_float), C.c_int(int(relu)), _p(out, C.c_float))
    return out


def gather_sum_f64(ptr, idx, x, dst_scale=None, relu=False, rows=None):
    """Double sum of rows [r0, r1) (default: all); returns (r1 - r0, feat) float64."""
    ptr, idx, x = _np(ptr, np.int32), _np(idx, np.int32), _np(x, np.float32)
    n = ptr.shape[0] - 1
    r0, r1 = (0, n) if rows is None else rows
    feat = x.shape[1]
    out = np.empty((r1 - r0, feat), dtype=np.float64)
    sc = _np(dst_scale, np.float32)
    load().csr_gather_sum_f64(_p(ptr, C.c_int32), _p(idx, C.c_int32), C.c_int64(r0), C.c_int64(r1), C.c_int64(feat),
                              _p(x, C.c_float), _p(sc, C.c_float), C.c_int(int(relu)), _p(out, C.c_double))
    return out


def u_mul_e_sum_f64(ptr, nid, eid, x, w, rows=None):
    ptr, nid, eid = _np(ptr, np.int32), _np(nid, np.int32), _np(eid, np.int32)
    x, w = _np(x, np.float32), _np(w, np.float32)
    w = w.reshape(w.shape[0], -1)
    n = ptr.shape[0] - 1
    r0, r1 = (0, n) if rows is None else rows
    feat, heads = x.reshape(x.shape[0], -1).shape[1], w.shape[1]
    out = np.empty((r1 - r0, feat), dtype=np.float64)
    load().csr_u_mul_e_sum_f64(_p(ptr, C.c_int32), _p(nid, C.c_int32), _p(eid, C.c_int32), C.c_int64(r0), C.c_int64(r1),
                               C.c_int64(heads), C.c_int64(feat // heads), _p(x, C.c_float), _p(w, C.c_float),
                               _p(out, C.c_double))
    return out


def segment_softmax_f64(ptr, eid, logits):
    ptr, eid, z = _np(ptr, np.int32), _np(eid, np.int32), _np(logits, np.float32)
    z2 = z.reshape(z.shape[0], -1)
    out = np.empty(z2.shape, dtype=np.float64)
    load().csr_segment_softmax_f64(_p(ptr, C.c_int32), _p(eid, C.c_int32), C.c_int64(ptr.shape[0] - 1),
                                   C.c_int64(z2.shape[1]), _p(z2, C.c_float), _p(out, C.c_double))
    return out.reshape(z.shape)


def u_dot_v_f64(src, dst, l, r, heads=1):
    src, dst = _np(src, np.int64), _np(dst, np.int64)
    l, r = _np(l, np.float32), _np(r, np.float32)
    feat = l.shape[1]
    out = np.empty((src.shape[0], heads), dtype=np.float64)
    load().coo_u_dot_v_f64(_p(src, C.c_int64), _p(dst, C.c_int64), C.c_int64(src.shape[0]), C.c_int64(heads),
                           C.c_int64(feat // heads), _p(l, C.c_float), _p(r, C.c_float), _p(out, C.c_double))
    return out


def segment_mm_f64(x, w, type_ptr, gather=None):
    x, w, tp = _np(x, np.float32), _np(w, np.float32), _np(type_ptr, np.int32)
    g = _np(gather, np.int64)
    t, k, n = w.shape
    m = int(tp[-1])
    out = np.empty((m, n), dtype=np.float64)
    load().segment_mm_f64(_p(x, C.c_float), _p(w, C.c_float), _p(tp, C.c_int32), C.c_int64(t), C.c_int64(k), C.c_int64(n),
                          _p(g, C.c_int64), _p(out, C.c_double))
    return out


if __name__ == "__main__":
    print("built", build(force="--force" in sys.argv))
