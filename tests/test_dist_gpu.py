"""Sharded layer on real GPUs (needs >= 2): every rank's rows must equal the single-GPU rows bit for bit."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def _worker(rank, world, port, tmp):
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from graphiler_b200 import capi, dist as gd, layers, synthetic
    wl = synthetic.make_c5(scale=0.01).to(dev)
    g, x, w = wl.graph, wl.feats, wl.params["gcn_w"]
    norm = g.in_degrees().clamp(min=1).float().pow(-0.5).unsqueeze(1)
    sl = gd.ShardedLayer(g.in_pointer, g.in_node_indices, g.num_nodes, w.shape[1], rank=rank, world=world)
    lo, hi = sl.block_range
    r0, r1 = sl.shard.row0, sl.shard.row1           # the all-gather keeps contiguous destination ranges
    y = gd.gcn_layer_sharded(sl, x[lo:hi].contiguous(), w, norm[lo:hi].contiguous(), norm[r0:r1].contiguous())
    full = sl.gather_outputs(y)
    pg = layers.PreparedGraph(g)
    single = layers.gcn_layer(pg, x, w, norm, norm)
    # the same layer with the projection / all-gather cut into four overlapped pieces
    s4 = gd.ShardedLayer(g.in_pointer, g.in_node_indices, g.num_nodes, w.shape[1], rank=rank, world=world, chunks=4)
    lo4, hi4 = s4.block_range
    y4 = gd.gcn_layer_sharded(s4, x[lo4:hi4].contiguous(), w, norm[lo4:hi4].contiguous(),
                              norm[s4.dst_rows].contiguous())
    full4 = s4.gather_outputs(y4)
    # and with the sparse (halo) exchange: only the source rows a shard reads travel, through one all-to-all
    sh = gd.ShardedLayer(g.in_pointer, g.in_node_indices, g.num_nodes, w.shape[1], rank=rank, world=world, exchange="halo")
    own = sh.owned_rows                             # source rows are dealt to the ranks by a hash of their id
    yh = gd.gcn_layer_sharded(sh, x[own].contiguous(), w, norm[own].contiguous(),
                              norm[sh.dst_rows].contiguous())
    fullh = sh.gather_outputs(yh)
    # the same exchange with the rows stored straight into the receivers' peer-mapped buffers; three steps in a row
    # exercise the alternating receive slots.  Where symmetric memory cannot be set up it is the all-to-all again.
    sp = gd.ShardedLayer(g.in_pointer, g.in_node_indices, g.num_nodes, w.shape[1], rank=rank, world=world, exchange="push")
    pushed_ok = True
    for _ in range(3):
        yp = gd.gcn_layer_sharded(sp, x[sp.owned_rows].contiguous(), w, norm[sp.owned_rows].contiguous(),
                                  norm[sp.dst_rows].contiguous())
        pushed_ok = pushed_ok and bool(torch.equal(sp.gather_outputs(yp), single))
    # and with the stores issued by the projection kernel's own epilogue (one kernel computes and sends)
    sf = gd.ShardedLayer(g.in_pointer, g.in_node_indices, g.num_nodes, w.shape[1], rank=rank, world=world, exchange="fused")
    for _ in range(3):
        yf = gd.gcn_layer_sharded(sf, x[sf.owned_rows].contiguous(), w, norm[sf.owned_rows].contiguous(),
                                  norm[sf.dst_rows].contiguous())
        pushed_ok = pushed_ok and bool(torch.equal(sf.gather_outputs(yf), single))
    # the sparse exchanges deal the destination rows by the hash that deals the source rows unless told otherwise
    # (balanced inbound traffic); contiguous edge-balanced ranges give the same bits
    pushed_ok = pushed_ok and sf.destinations == "hashed" and sp.destinations == "hashed" and sl.destinations == "ranges"
    for ex in ("fused", "push", "halo"):
        sx = gd.ShardedLayer(g.in_pointer, g.in_node_indices, g.num_nodes, w.shape[1], rank=rank, world=world, exchange=ex,
                             destinations="ranges")
        pushed_ok = pushed_ok and sx.shard.row0 is not None
        for _ in range(2):
            yx = gd.gcn_layer_sharded(sx, x[sx.owned_rows].contiguous(), w, norm[sx.owned_rows].contiguous(),
                                      norm[sx.dst_rows].contiguous())
            pushed_ok = pushed_ok and bool(torch.equal(sx.gather_outputs(yx), single))
    # two layers in a row over the fused exchange: the output rows of a rank are the rows it projects next
    w2 = (torch.randn(w.shape[1], w.shape[1], generator=torch.Generator().manual_seed(3)) * 0.1).to(dev)
    ys = gd.gcn_stack_sharded(sf, x[sf.owned_rows].contiguous(), [w, w2], norm[sf.owned_rows].contiguous())
    single2 = layers.gcn_layer(pg, single, w2, norm, norm, relu=False)
    pushed_ok = pushed_ok and bool(torch.equal(sf.gather_outputs(ys), single2))
    if rank == 0:
        print("fused exchange:", "projection epilogue stores to peers" if sf.fused else "not fused", flush=True)
    if rank == 0:
        print("push exchange:", "peer stores" if sp.push else f"fell back to all-to-all ({sp.push_unavailable})", flush=True)
    # GAT on the same graph: z, el, er gathered, fused attention on the local rows
    p = wl.params
    sg = gd.ShardedLayer(g.in_pointer, g.in_node_indices, g.num_nodes, p["fc_weight"].shape[1], rank=rank, world=world)
    lo, hi = sg.block_range
    yg = gd.gat_layer_sharded(sg, x[lo:hi].contiguous(), p["fc_weight"], p["attn_src"], p["attn_dst"], 0.2)
    full_gat = sg.gather_outputs(yg)
    single_gat = layers.gat_layer(pg, x, p["fc_weight"], p["attn_src"], p["attn_dst"], 0.2)
    # GAT over the sparse exchange (all-to-all, then peer stores for the z rows)
    gat_sparse_ok = True
    for ex, dests in (("halo", None), ("push", None), ("fused", None), ("fused", "ranges")):
        sgh = gd.ShardedLayer(g.in_pointer, g.in_node_indices, g.num_nodes, p["fc_weight"].shape[1], rank=rank, world=world,
                              exchange=ex, destinations=dests)
        for _ in range(2):
            ygh = gd.gat_layer_sharded(sgh, x[sgh.owned_rows].contiguous(), p["fc_weight"], p["attn_src"], p["attn_dst"], 0.2)
            gat_sparse_ok = gat_sparse_ok and bool(torch.equal(sgh.gather_outputs(ygh), single_gat))
    torch.cuda.synchronize()
    if rank == 0:
        # the dense projections run on different row blocks but every row's dot products are computed identically,
        # and the sparse kernels do not depend on the sharding: bit-exact
        np.save(tmp + "/ok.npy", np.array([bool(torch.equal(full, single)), full.shape[0] == g.num_nodes,
                                            bool(torch.equal(full_gat, single_gat)), bool(torch.equal(full4, single)),
                                            bool(torch.equal(fullh, single)), pushed_ok, gat_sparse_ok]))
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_gcn_layer_matches_single_gpu_bitwise(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = 29500 + os.getpid() % 2000
    mp.start_processes(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True, start_method="spawn")
    assert np.load(tmp_path / "ok.npy").all()
