"""Run the reference's own compiler flow against an operator library.  Test helper, run as a script in a
child process (the operator library registers global TorchScript state, one library per process):

    python tests/ref_flow.py --lib <libgraphiler.so> --device cpu|cuda [--golden-out DIR] [--golden-in DIR]

It installs ``--lib`` as ``$HOME/.dgl/libgraphiler.so`` in a scratch HOME (the fixed path the reference's
wrapper loads, python/graphiler/mpdfg_builder.py:11-14), imports the reference's wrapper and compiled
builder/optimizer from oracle/_ref/, compiles the four example models' user-defined functions at
optimisation levels 0/1/2 and at "level 3" (level 2 followed by this package's additional fusion patterns,
graphiler_b200/fusion.py), executes them on seeded N(0,1) inputs on the requested device and compares with
the user-defined-function oracle evaluated in float64 on the same float32 inputs.  Prints one JSON report.

The user-defined functions restate examples/GAT/GAT.py:25-36, GCN/GCN.py:21-27, RGCN/RGCN.py:25-33 and
HGT/HGT.py:28-60 (single head, as the reference's builder supports); GAT uses the compiled path's
leaky-relu slope 0.01 on both sides.
"""

import argparse
import contextlib
import io
import json
import os
import shutil
import sys
import tempfile
from pathlib import Path
from types import SimpleNamespace

ROOT = Path(__file__).resolve().parent.parent

ap = argparse.ArgumentParser()
ap.add_argument("--lib", required=True)
ap.add_argument("--device", default="cpu")
ap.add_argument("--golden-out", default=None)
ap.add_argument("--golden-in", default=None)
ap.add_argument("--levels", default="0,1,2,3")
args = ap.parse_args()

home = tempfile.mkdtemp(prefix="gphl_home_")
os.environ["HOME"] = home
dgl = Path(home) / ".dgl"
dgl.mkdir()
lib = Path(args.lib).resolve()
shutil.copy(lib, dgl / "libgraphiler.so")
if (lib.parent / "libgphl.so").exists():            # the CUDA library finds its kernels next to itself
    shutil.copy(lib.parent / "libgphl.so", dgl / "libgphl.so")
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))
sys.path.insert(0, str(ROOT / "oracle" / "_ref"))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.nn.functional as F  # noqa: E402

with contextlib.redirect_stdout(io.StringIO()):
    from graphiler import EdgeBatchDummy, NodeBatchDummy, mpdfg_builder, update_all  # noqa: E402  (reference wrapper)

from graphiler_b200.fusion import extra_fusion  # noqa: E402
from graphiler_b200.graph import GraphArrays  # noqa: E402
from fixtures_common import hetero_graphs, homo_graphs  # noqa: E402
from oracle import ops_oracle as O  # noqa: E402
from oracle import udf_oracle as U  # noqa: E402


# ---- user-defined functions (TorchScript-able, typed with the reference's batch classes) ----------------

def gcn_message(edges: EdgeBatchDummy):
    norm = torch.pow(edges.src['degree'], -0.5)
    return {'m': edges.src['h'] * norm}


def gcn_reduce(nodes: NodeBatchDummy):
    return {'h': torch.relu(torch.sum(nodes.mailbox['m'], dim=1))}


def gat_message(edges: EdgeBatchDummy, fc_weight, attn_weight):
    z_s = torch.mm(edges.src['h'], fc_weight)
    z_d = torch.mm(edges.dst['h'], fc_weight)
    z2 = torch.cat([z_s, z_d], dim=1)
    a = torch.mm(z2, attn_weight)
    return {'z': z_s, 'e': F.leaky_relu_(a)}


def gat_reduce(nodes: NodeBatchDummy):
    alpha = torch.softmax(nodes.mailbox['e'], dim=1)
    h = torch.sum(alpha * nodes.mailbox['z'], dim=1)
    return {'h': h}


def rgcn_message(edges: EdgeBatchDummy):
    relation_weight = edges.type['weight']
    msg = torch.bmm(edges.src['h'].unsqueeze(1), relation_weight).squeeze()
    msg = msg * edges.data['norm']
    return {'m': msg}


def rgcn_reduce(nodes: NodeBatchDummy):
    return {'h': torch.sum(nodes.mailbox['m'], dim=1)}


def hgt_message(edges: EdgeBatchDummy, sqrt_dk: float):
    k_weight = edges.srctype['k_weight']
    v_weight = edges.srctype['v_weight']
    q_weight = edges.dsttype['q_weight']
    k = torch.bmm(edges.src['h'].unsqueeze(1), k_weight).squeeze()
    v = torch.bmm(edges.src['h'].unsqueeze(1), v_weight).squeeze()
    q = torch.bmm(edges.dst['h'].unsqueeze(1), q_weight).squeeze()
    relation_att = edges.type['relation_att']
    relation_msg = edges.type['relation_msg']
    relation_pri = edges.type['relation_pri']
    k = torch.bmm(k.unsqueeze(1), relation_att).squeeze()
    v = torch.bmm(v.unsqueeze(1), relation_msg).squeeze()
    t = k * q
    attn_score = torch.sum(t, dim=1, keepdim=True) * relation_pri / sqrt_dk
    return {'attn': attn_score, 'v': v}


def hgt_reduce(nodes: NodeBatchDummy):
    t = torch.softmax(nodes.mailbox['attn'], dim=1)
    m = t * nodes.mailbox['v']
    return {'t': torch.sum(m, dim=1)}


def hgt_update(nodes: NodeBatchDummy):
    skip = nodes.type['skip']
    a_weight = nodes.type['a_weight']
    alpha = torch.sigmoid(skip)
    trans_out = torch.bmm(nodes.data['t'].unsqueeze(1), a_weight).squeeze()
    return {'h': trans_out * alpha.unsqueeze(1)}


# ---- graphs and inputs -----------------------------------------------------------------------------------

def to_dgl_graph(g: GraphArrays, device):
    d = g.to(device)
    obj = torch.classes.my_classes.DGLGraph(d.in_pointer, d.in_node_indices, d.in_edge_indices, d.out_pointer,
                                            d.out_node_indices, d.out_edge_indices, d.COO_src, d.COO_dst, None, None)
    if d.ntype_pointer is not None:
        obj.SetNtypePointer(d.ntype_pointer)
        obj.SetNtypeCOO(d.ntype_COO)
    if d.etype_pointer is not None:
        obj.SetEtypePointer(d.etype_pointer)
        obj.SetEtypeCOO(d.etype_COO)
    return obj


def run_compiled(mpdfg, g: GraphArrays, ndata, edata, ntd, etd, params, device, key='h'):
    mv = lambda d: {k: v.to(device) for k, v in d.items()}
    ns = SimpleNamespace(DGLGraph=to_dgl_graph(g, device), ndata=mv(ndata), edata=mv(edata), ntype_data=mv(ntd),
                         etype_data=mv(etd))
    p = tuple(x.to(device) if torch.is_tensor(x) else x for x in params)
    update_all(ns, mpdfg, msg_params=p)
    if device != "cpu":
        torch.cuda.synchronize()
    return ns.ndata[key].detach().cpu()


def f64(d):
    return {k: v.double() for k, v in d.items()}


def report(name, got, truth64, ref32, results):
    ok, bad, err = O.within_tolerance(got.double().numpy(), truth64.numpy())
    _, bad_ref, err_ref = O.within_tolerance(ref32.double().numpy(), truth64.numpy())
    scale = float(truth64.abs().max())
    results[name] = {"violations": bad, "violations_fp32_udf_path": bad_ref, "max_abs_err": err,
                     "max_abs_err_fp32_udf_path": err_ref, "norm_err": err / max(scale, 1e-30), "elements": got.numel()}


def main():
    dev = args.device
    levels = [int(x) for x in args.levels.split(",")]
    results, golden = {}, {}
    gen = torch.Generator().manual_seed(1234)
    rn = lambda *s: torch.randn(*s, generator=gen)
    quiet = contextlib.redirect_stdout(io.StringIO())

    # build order: models without an update function first, HGT (with one) last; the reference's builder keeps
    # static state across calls (src/builder/builder.cpp:3,344) and crashes in the other order
    def build(*funcs):
        out = {l: mpdfg_builder(*funcs, opt_level=min(l, 2)) for l in levels}
        if 3 in out:
            results.setdefault("extra_fusion", {})[funcs[0].__name__.split("_")[0]] = extra_fusion(out[3])
        return out

    with quiet:
        gcn, gat, rgcn = build(gcn_message, gcn_reduce), build(gat_message, gat_reduce), build(rgcn_message, rgcn_reduce)
        hgt = build(hgt_message, hgt_reduce, hgt_update)
    for l in levels:
        for nm, m in (("gcn", gcn), ("gat", gat), ("rgcn", rgcn), ("hgt", hgt)):
            ops = sorted({n.kind() for n in m[l].forward.graph.nodes() if n.kind().startswith("my_ops::")})
            results[f"ops_{nm}_opt{l}"] = ops

    homo = homo_graphs()
    for gname, g in homo.items():
        n = g.num_nodes
        h = rn(n, 24)
        deg = g.in_degrees().clamp(min=1).float().unsqueeze(1)
        w = rn(24, 16) * 0.3
        # GCN
        feat = h @ w
        truth = U.update_all(g, {"h": feat.double(), "degree": deg.double()}, {}, {}, {},
                             lambda e: {"m": e.src["h"] * torch.pow(e.src["degree"], -0.5)},
                             lambda nd: {"h": torch.relu(torch.sum(nd.mailbox["m"], dim=1))})["h"]
        ref32 = U.update_all(g, {"h": feat, "degree": deg}, {}, {}, {},
                             lambda e: {"m": e.src["h"] * torch.pow(e.src["degree"], -0.5)},
                             lambda nd: {"h": torch.relu(torch.sum(nd.mailbox["m"], dim=1))})["h"]
        for l in levels:
            got = run_compiled(gcn[l], g, {"h": feat, "degree": deg}, {}, {}, {}, (), dev)
            report(f"gcn_{gname}_opt{l}", got, truth, ref32, results)
            golden[f"gcn_{gname}_opt{l}"] = got.numpy()
        golden[f"gcn_{gname}_in_h"], golden[f"gcn_{gname}_in_degree"] = feat.numpy(), deg.numpy()
        # GAT (single head, slope 0.01 as the compiled graph uses)
        fc, aw = rn(24, 16) * 0.3, rn(32, 1) * 0.3
        a_s, a_d = aw[:16].reshape(1, 16), aw[16:].reshape(1, 16)
        truth = U.gat_layer(g, h.double(), fc.double(), a_s.double(), a_d.double(), 0.01)
        ref32 = U.gat_layer(g, h, fc, a_s, a_d, 0.01)
        for l in levels:
            got = run_compiled(gat[l], g, {"h": h}, {}, {}, {}, (fc, aw), dev)
            report(f"gat_{gname}_opt{l}", got, truth, ref32, results)
            golden[f"gat_{gname}_opt{l}"] = got.numpy()
        golden[f"gat_{gname}_in_h"], golden[f"gat_{gname}_in_fc"], golden[f"gat_{gname}_in_attn"] = h.numpy(), fc.numpy(), aw.numpy()

    hetero = hetero_graphs()
    for gname, g in hetero.items():
        n, e, tn, te = g.num_nodes, g.num_edges, g.num_ntypes, g.num_etypes
        h = rn(n, 16)
        # RGCN
        w = rn(te, 16, 16) * 0.3
        norm = (1.0 / g.in_degrees().clamp(min=1).float())[g.COO_dst].unsqueeze(1)
        truth = U.rgcn_layer(g, h.double(), w.double(), norm.double())
        ref32 = U.rgcn_layer(g, h, w, norm)
        for l in levels:
            got = run_compiled(rgcn[l], g, {"h": h}, {"norm": norm}, {}, {"weight": w}, (), dev)
            report(f"rgcn_{gname}_opt{l}", got, truth, ref32, results)
            golden[f"rgcn_{gname}_opt{l}"] = got.numpy()
        golden[f"rgcn_{gname}_in_h"], golden[f"rgcn_{gname}_in_w"], golden[f"rgcn_{gname}_in_norm"] = h.numpy(), w.numpy(), norm.numpy()
        # HGT
        p = {"k_weight": rn(tn, 16, 16) * 0.3, "v_weight": rn(tn, 16, 16) * 0.3, "q_weight": rn(tn, 16, 16) * 0.3,
             "a_weight": rn(tn, 16, 16) * 0.3, "relation_att": rn(te, 16, 16) * 0.3, "relation_msg": rn(te, 16, 16) * 0.3,
             "relation_pri": torch.ones(te, 1), "skip": torch.ones(tn)}
        truth = U.hgt_layer(g, h.double(), f64(p), 1, 4.0)
        ref32 = U.hgt_layer(g, h, p, 1, 4.0)
        ntd = {k: p[k] for k in ("k_weight", "v_weight", "q_weight", "a_weight", "skip")}
        etd = {k: p[k] for k in ("relation_att", "relation_msg", "relation_pri")}
        for l in levels:
            got = run_compiled(hgt[l], g, {"h": h}, {}, ntd, etd, (4.0,), dev)
            report(f"hgt_{gname}_opt{l}", got, truth, ref32, results)
            golden[f"hgt_{gname}_opt{l}"] = got.numpy()
        golden[f"hgt_{gname}_in_h"] = h.numpy()
        for k, v in p.items():
            golden[f"hgt_{gname}_in_{k}"] = v.numpy()

    if args.golden_out:
        out = Path(args.golden_out)
        out.mkdir(parents=True, exist_ok=True)
        np.savez_compressed(out / "ref_flow_golden.npz", **golden)
        (out / "ref_flow_ops.json").write_text(json.dumps({k: v for k, v in results.items() if k.startswith("ops_")}, indent=1))
    if args.golden_in:
        ref = np.load(Path(args.golden_in) / "ref_flow_golden.npz")
        worst = 0.0
        for k, v in golden.items():
            if "_in_" in k:
                assert np.array_equal(v, ref[k]), f"seeded input {k} differs from the golden fixture"
            else:
                # the fixture holds levels 0-2; the added fusions must not change the level-2 result
                ok, bad, err = O.within_tolerance(v, ref[k.replace("_opt3", "_opt2")].astype(np.float64), rtol=1e-4, atol=1e-5)
                worst = max(worst, err)
                results.setdefault("golden_mismatch", [])
                if not ok:
                    results["golden_mismatch"].append(k)
        results["golden_max_abs_diff"] = worst
    print("REPORT " + json.dumps(results))
    shutil.rmtree(home, ignore_errors=True)


main()
