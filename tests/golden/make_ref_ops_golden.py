"""Record the outputs of the reference's own CUDA operators on the seeded cases of tests/ref_ops_cases.py.

    python oracle/build_ref_cuda.py                       (once, where the reference's source tree is present:
                                                           builds oracle/_ref/libgraphiler_ref.so from it)
    python tests/golden/make_ref_ops_golden.py OUT_DIR    (on a machine with a CUDA device)

Writes OUT_DIR/ref_ops_golden.npz: for every case `<name>` the reference operator's output, and
`<name>__crc` the CRC-32 of the case's inputs, plus `__meta__` (GPU name, CUDA and PyTorch versions).  The
committed tests/golden/ref_ops_golden.npz is that file, produced on a B200.

This script must run in a process of its own: the reference library registers `my_classes.DGLGraph` and
`my_ops::*`, the same names the product library registers, and one process can hold only one of them.
Nothing of graphiler_b200's native code is loaded here (graphiler_b200.graph is pure Python).
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import numpy as np  # noqa: E402
import torch  # noqa: E402


def load_reference_library():
    so = ROOT / "oracle" / "_ref" / "libgraphiler_ref.so"
    if not so.exists():
        raise SystemExit(f"{so} is missing: run oracle/build_ref_cuda.py where the reference tree is present")
    torch.classes.load_library(str(so))
    torch.ops.load_library(str(so))
    return so


def to_ref_graph(g, dev):
    d = g.to(dev)
    obj = torch.classes.my_classes.DGLGraph(d.in_pointer, d.in_node_indices, d.in_edge_indices, d.out_pointer,
                                            d.out_node_indices, d.out_edge_indices, d.COO_src, d.COO_dst, None, None)
    if d.ntype_pointer is not None:
        obj.SetNtypePointer(d.ntype_pointer)
        obj.SetNtypeCOO(d.ntype_COO)
    if d.etype_pointer is not None:
        obj.SetEtypePointer(d.etype_pointer)
        obj.SetEtypeCOO(d.etype_COO)
    return obj, d                                          # d keeps the device arrays alive


def run_reference_op(op, G, inp):
    o = torch.ops.my_ops
    if op in ("SpMMSrc", "SpMMEdge"):
        return getattr(o, op)(inp["x"], [1], False, None, G)
    if op in ("gspmm_src_mul_e_sum", "gspmm_dst_mul_e_sum"):
        return getattr(o, op)(inp["x"], inp["w"], [1], False, None, G)
    if op == "SegmentSoftmax":
        return o.SegmentSoftmax(inp["x"], 1, None, G)
    if op == "gsddmm_u_add_v_mul_alpha":
        return o.gsddmm_u_add_v_mul_alpha(inp["l"], inp["r"], 1, G)
    if op.startswith("Broadcast"):
        return getattr(o, op)(inp["x"], G)
    if op in ("SegmentMMNode", "SegmentMMEdge"):
        return getattr(o, op)(inp["x"], inp["w"], G)
    raise KeyError(op)


def main(out_dir: Path):
    import ref_ops_cases as C
    if not torch.cuda.is_available():
        raise SystemExit("a CUDA device is needed to run the reference's operators")
    so = load_reference_library()
    dev = torch.device("cuda:0")
    gs = C.graphs()
    handles = {k: to_ref_graph(g, dev) for k, g in gs.items()}
    rec = {}
    for name, gname, op, inp in C.cases():
        G = handles[gname][0]
        y = run_reference_op(op, G, {k: v.to(dev) for k, v in inp.items()})
        torch.cuda.synchronize()
        rec[name] = y.detach().cpu().numpy()
        rec[name + "__crc"] = np.array(C.input_checksum(inp), dtype=np.int64)
    assert int(torch.ops.my_ops.get_feat_dim(torch.zeros(3, 4, 5))) == 20
    meta = {"gpu": torch.cuda.get_device_name(0), "torch": torch.__version__, "cuda": torch.version.cuda,
            "library": so.name, "cases": len(rec) // 2}
    rec["__meta__"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    out_dir.mkdir(parents=True, exist_ok=True)
    np.savez_compressed(out_dir / "ref_ops_golden.npz", **rec)
    print(json.dumps(meta))


if __name__ == "__main__":
    main(Path(sys.argv[1]) if len(sys.argv) > 1 else ROOT / "tests" / "golden")
