"""The C-ABI library loads here (no GPU needed) and exports every function include/gphl.h declares."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "gphl.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gphl_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_operator_set():
    names = declared_functions()
    for must in ("gphl_spmm_gather_sum_f32", "gphl_spmm_u_mul_e_sum_f32", "gphl_sddmm_u_add_v_f32_i64",
                 "gphl_sddmm_u_dot_v_f32_i64", "gphl_sddmm_u_dot_v_csc_f32", "gphl_segment_softmax_f32", "gphl_gat_fused_f32",
                 "gphl_gather_rows_i64", "gphl_segment_mm_f32", "gphl_plan_create"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from graphiler_b200 import build, capi
    build.build_kernels()
    lib = ctypes.CDLL(str(capi.KERNEL_LIB))
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, missing
    # the ctypes prototypes cover the header, nothing more and nothing less
    assert sorted(capi.SIGNATURES) == declared_functions()
    lib.gphl_version.restype = ctypes.c_int
    assert lib.gphl_version() >= 1


def test_missing_library_fails_loudly(tmp_path):
    from graphiler_b200 import capi
    with pytest.raises(capi.GphlError):
        capi.load_library(tmp_path / "libgphl.so")


def test_cpu_tensors_are_rejected():
    import torch
    from graphiler_b200 import capi
    with pytest.raises(capi.GphlError):
        capi.spmm_gather_sum(torch.zeros(2, dtype=torch.int32), torch.zeros(0, dtype=torch.int32), torch.zeros(1, 4))
