"""Seeded synthetic workloads with the shapes of the five benchmark configurations.

The public graph datasets the reference loads through DGL/OGB
(python/graphiler/utils/setup.py:22-83) are not available offline; these generators
stand in for their shapes, degree distributions and value distributions.  Every
generator is a pure function of (sizes, seed, device); ``scale`` shrinks node and edge
counts proportionally so the same code serves small parity cases.

  c1  GAT   N=20 000, ~100 000 Zipf(2.1) out-degree edges + self-loops, in 500, 8 heads x 8
  c2  GCN   N=170 000, 1 170 000 symmetrised R-MAT edges + self-loops, 128 -> 256 -> 40
  c3  RGCN  N=100 000, E=1 000 000, 50 Zipf(1.5) relations, 16 -> 16
  c4  HGT   4 node types (60k/40k/20k/5k), 6 edge types, E=1 500 000, hidden 128 = 8 x 16
  c5  scale sweep: R-MAT N=2 400 000, E=60 000 000 + self-loops, 256-dim features
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, Optional

import numpy as np
import torch

from .graph import GraphArrays, attach_types, prepare_graph


@dataclass
class Workload:
    name: str
    graph: GraphArrays
    feats: torch.Tensor                      # (N, in_dim) float32, N(0,1)
    params: Dict[str, torch.Tensor] = field(default_factory=dict)
    edata: Dict[str, torch.Tensor] = field(default_factory=dict)
    hyper: Dict[str, float] = field(default_factory=dict)

    def to(self, device) -> "Workload":
        return Workload(self.name, self.graph.to(device), self.feats.to(device),
                        {k: v.to(device) for k, v in self.params.items()},
                        {k: v.to(device) for k, v in self.edata.items()}, dict(self.hyper))


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def glorot(shape, gen: torch.Generator, device) -> torch.Tensor:
    """Glorot/Xavier-uniform over the last two dims."""
    fan_in, fan_out = shape[-2], shape[-1]
    a = math.sqrt(6.0 / (fan_in + fan_out))
    return (torch.rand(shape, generator=gen, device=device) * 2 - 1) * a


def rmat_edges(num_nodes: int, num_edges: int, gen: torch.Generator, device,
               a=0.57, b=0.19, c=0.19) -> tuple:
    """R-MAT edge list on a 2^ceil(log2 N) grid; ids >= N are rejected and redrawn."""
    levels = max(1, math.ceil(math.log2(max(num_nodes, 2))))
    srcs, dsts, have = [], [], 0
    while have < num_edges:
        m = int((num_edges - have) * 1.35) + 1024
        s = torch.zeros(m, dtype=torch.int64, device=device)
        d = torch.zeros(m, dtype=torch.int64, device=device)
        for _ in range(levels):
            r = torch.rand(m, generator=gen, device=device)
            sbit = r >= (a + b)
            dbit = ((r >= a) & (r < a + b)) | (r >= a + b + c)
            s = (s << 1) | sbit
            d = (d << 1) | dbit
        keep = (s < num_nodes) & (d < num_nodes)
        s, d = s[keep], d[keep]
        srcs.append(s)
        dsts.append(d)
        have += s.numel()
    return torch.cat(srcs)[:num_edges], torch.cat(dsts)[:num_edges]


def _self_loops(n, device):
    ar = torch.arange(n, dtype=torch.int64, device=device)
    return ar, ar


def make_c1(scale: float = 1.0, seed: int = 43, device="cpu", heads=8, dim=8, in_dim=500) -> Workload:
    n = max(4, int(round(20_000 * scale)))
    target = max(4, int(round(100_000 * scale)))
    rng = np.random.default_rng(seed)
    k = np.minimum(rng.zipf(2.1, n), max(1, n // 10)).astype(np.int64)
    while k.sum() < target:                       # heavy tail: almost never loops
        k = k + np.minimum(rng.zipf(2.1, n), max(1, n // 10))
    src = np.repeat(np.arange(n, dtype=np.int64), k)
    src = src[rng.permutation(src.size)[:target]]  # thin uniformly down to the target count
    dst = rng.integers(0, n, size=target, dtype=np.int64)
    gen = _gen(seed, device)
    ls, ld = _self_loops(n, device)
    s = torch.cat([torch.from_numpy(src).to(device), ls])
    d = torch.cat([torch.from_numpy(dst).to(device), ld])
    # Edge ids follow the destination-sorted order, the storage format this configuration names.
    order = torch.sort(d, stable=True)[1]
    g = prepare_graph(s[order], d[order], n)
    x = torch.randn(n, in_dim, generator=gen, device=device)
    f = heads * dim
    params = {"fc_weight": glorot((in_dim, f), gen, device),
              "attn_src": glorot((heads, dim), gen, device),
              "attn_dst": glorot((heads, dim), gen, device)}
    return Workload("c1_gat", g, x, params, {}, {"heads": heads, "dim": dim, "slope": 0.2})


def make_c2(scale: float = 1.0, seed: int = 44, device="cpu", in_dim=128, hidden=256, classes=40) -> Workload:
    n = max(4, int(round(170_000 * scale)))
    pairs = max(2, int(round(585_000 * scale)))
    gen = _gen(seed, device)
    have = torch.zeros(0, dtype=torch.int64, device=device)
    while have.numel() < pairs:
        s, d = rmat_edges(n, int(pairs * 1.6) + 1024, gen, device)
        lo, hi = torch.minimum(s, d), torch.maximum(s, d)
        key = (lo * n + hi)[lo != hi]
        have = torch.unique(torch.cat([have, key]))
    have = have[torch.randperm(have.numel(), generator=gen, device=device)[:pairs]]
    lo, hi = have // n, have % n
    ls, ld = _self_loops(n, device)
    s = torch.cat([lo, hi, ls])
    d = torch.cat([hi, lo, ld])
    order = torch.sort(d, stable=True)[1]
    g = prepare_graph(s[order], d[order], n)
    x = torch.randn(n, in_dim, generator=gen, device=device)
    params = {"w1": glorot((in_dim, hidden), gen, device), "w2": glorot((hidden, classes), gen, device)}
    return Workload("c2_gcn", g, x, params, {}, {})


def make_c3(scale: float = 1.0, seed: int = 45, device="cpu", rels=50, dim=16) -> Workload:
    n = max(4, int(round(100_000 * scale)))
    e = max(rels, int(round(1_000_000 * scale)))
    gen = _gen(seed, device)
    s = torch.randint(0, n, (e,), generator=gen, device=device)
    d = torch.randint(0, n, (e,), generator=gen, device=device)
    p = torch.arange(1, rels + 1, dtype=torch.float64, device=device) ** -1.5
    rel = torch.multinomial((p / p.sum()).float(), e, replacement=True, generator=gen)
    order = torch.sort(rel, stable=True)[1]          # edge id order = relation order
    s, d, rel = s[order], d[order], rel[order]
    g = prepare_graph(s, d, n)
    attach_types(g, etype_counts=torch.bincount(rel, minlength=rels).tolist())
    x = torch.randn(n, dim, generator=gen, device=device)
    indeg = g.in_degrees().clamp(min=1).to(torch.float32)
    norm = (1.0 / indeg)[d].unsqueeze(1).contiguous()  # mean aggregation, (E,1)
    params = {"w1": glorot((rels, dim, dim), gen, device), "w2": glorot((rels, dim, dim), gen, device)}
    return Workload("c3_rgcn", g, x, params, {"norm": norm}, {})


def make_c4(scale: float = 1.0, seed: int = 46, device="cpu", heads=8, dim=16) -> Workload:
    sizes = [max(2, int(round(v * scale))) for v in (60_000, 40_000, 20_000, 5_000)]
    per_type = max(2, int(round(250_000 * scale)))
    n, f = sum(sizes), heads * dim
    offs = np.concatenate([[0], np.cumsum(sizes)])
    gen = _gen(seed, device)
    tp = torch.randint(0, 4, (6, 2), generator=_gen(seed + 1000, "cpu"))   # (src type, dst type) per edge type
    ss, dd = [], []
    for t in range(6):
        a, b = int(tp[t, 0]), int(tp[t, 1])
        ss.append(torch.randint(0, sizes[a], (per_type,), generator=gen, device=device) + int(offs[a]))
        dd.append(torch.randint(0, sizes[b], (per_type,), generator=gen, device=device) + int(offs[b]))
    g = prepare_graph(torch.cat(ss), torch.cat(dd), n)
    attach_types(g, ntype_counts=sizes, etype_counts=[per_type] * 6)
    x = torch.randn(n, f, generator=gen, device=device)

    def block_diag(t):                       # per-head (dim x dim) blocks on the diagonal of (f x f)
        w = torch.zeros(t, f, f, device=device)
        blocks = glorot((t, heads, dim, dim), gen, device)
        for h in range(heads):
            w[:, h * dim:(h + 1) * dim, h * dim:(h + 1) * dim] = blocks[:, h]
        return w

    params = {"k_weight": glorot((4, f, f), gen, device), "q_weight": glorot((4, f, f), gen, device),
              "v_weight": glorot((4, f, f), gen, device), "a_weight": glorot((4, f, f), gen, device),
              "relation_att": block_diag(6), "relation_msg": block_diag(6),
              "relation_pri": torch.ones(6, heads, device=device), "skip": torch.ones(4, device=device)}
    return Workload("c4_hgt", g, x, params, {}, {"heads": heads, "dim": dim, "sqrt_dk": math.sqrt(dim)})


def make_c5(scale: float = 1.0, seed: int = 47, device="cpu", dim=256, heads=8,
            with_params: bool = True) -> Workload:
    n = max(4, int(round(2_400_000 * scale)))
    e = max(4, int(round(60_000_000 * scale)))
    gen = _gen(seed, device)
    s, d = rmat_edges(n, e, gen, device)
    ls, ld = _self_loops(n, device)
    s, d = torch.cat([s, ls]), torch.cat([d, ld])
    order = torch.sort(d, stable=True)[1]
    s, d = s[order], d[order]
    del order
    g = prepare_graph(s, d, n)
    x = torch.randn(n, dim, generator=gen, device=device)
    params = {}
    if with_params:
        params = {"gcn_w": glorot((dim, dim), gen, device), "fc_weight": glorot((dim, dim), gen, device),
                  "attn_src": glorot((heads, dim // heads), gen, device),
                  "attn_dst": glorot((heads, dim // heads), gen, device)}
    return Workload("c5_scale", g, x, params, {}, {"heads": heads, "dim": dim // heads, "slope": 0.2})


MAKERS = {"c1": make_c1, "c2": make_c2, "c3": make_c3, "c4": make_c4, "c5": make_c5}


def make(name: str, scale: float = 1.0, device="cpu", seed: Optional[int] = None) -> Workload:
    kw = {} if seed is None else {"seed": seed}
    return MAKERS[name](scale=scale, device=device, **kw)
