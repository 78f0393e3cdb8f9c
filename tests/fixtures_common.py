"""Seeded small graphs shared by the golden-fixture generator, the reference-flow runner and the tests."""
import numpy as np
import torch

from graphiler_b200.graph import attach_types, debug_graph, debug_hetero_graph, prepare_graph


def random_homo(n, e, seed, zero_rows=False):
    g = torch.Generator().manual_seed(seed)
    src = torch.randint(0, n, (e,), generator=g)
    dst = torch.randint(0, n // 2 if zero_rows else n, (e,), generator=g)
    if not zero_rows:
        src, dst = torch.cat([src, torch.arange(n)]), torch.cat([dst, torch.arange(n)])
    return prepare_graph(src, dst, n)


def random_hetero(seed, sizes=(30, 20, 10, 5), per_type=100):
    g = torch.Generator().manual_seed(seed)
    offs = np.concatenate([[0], np.cumsum(sizes)])
    ss, dd = [], []
    pairs = [(0, 1), (1, 0), (0, 0), (2, 3), (3, 1), (1, 2)]
    for a, b in pairs:
        ss.append(torch.randint(0, sizes[a], (per_type,), generator=g) + int(offs[a]))
        dd.append(torch.randint(0, sizes[b], (per_type,), generator=g) + int(offs[b]))
    gr = prepare_graph(torch.cat(ss), torch.cat(dd), int(sum(sizes)))
    return attach_types(gr, ntype_counts=list(sizes), etype_counts=[per_type] * len(pairs))


def homo_graphs():
    return {"debug": debug_graph(), "rand200": random_homo(200, 1500, 7), "zero_rows": random_homo(50, 60, 8, True)}


def hetero_graphs():
    return {"debug_hetero": debug_hetero_graph(), "rand_hetero": random_hetero(9)}
