"""Peer-store rates between the GPUs of one node, all ranks sending at once: what the sparse exchanges of
``dist.ShardedLayer`` can reach.  Run under torchrun with one rank per GPU (2 to 8):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 -m graphiler_b200.link_probe

Every rank moves the same 0.8 GB of 1 KiB rows: through the copy engine, through the row-scatter kernel
(gphl_scatter_rows_peers_i64) and through the fan-out epilogue of the tensor-core projection
(gphl_segment_mm_tc_fanout_f32) - to the next rank, to itself, to all other ranks round robin; times are CUDA events,
median of five, maximum over the ranks.  Rank 0 prints one JSON object.
"""
import json
import os

import torch
import torch.distributed as dist

from . import capi


def main(rows: int = 786432, feat: int = 256) -> dict:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    import torch.distributed._symmetric_memory as symm

    m, f = rows, feat
    buf = symm.empty((m, f), dtype=torch.float32, device=dev)
    hdl = symm.rendezvous(buf, dist.group.WORLD)
    peers = [hdl.get_buffer(p, (m, f), torch.float32) if p != rank else buf for p in range(world)]
    x = torch.randn(m, f, device=dev)
    w = torch.randn(f, f, device=dev) / 16
    tok = torch.zeros(1, dtype=torch.int32, device=dev)
    nxt = (rank + 1) % world
    res = {}

    def timed(name, fn, reps=5, gb=m * f * 4 / 1e9):
        for _ in range(2):
            fn()
        dist.all_reduce(tok)
        torch.cuda.synchronize()
        t = []
        for _ in range(reps):
            dist.all_reduce(tok)                                  # everybody starts together
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            t.append(a.elapsed_time(b))
        v = torch.tensor([sorted(t)[len(t) // 2]], device=dev)
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        res[name] = {"ms_max": round(float(v), 3), "GBps": round(gb / float(v) * 1e3, 1)}

    ar = torch.arange(m, device=dev, dtype=torch.int64)
    perm = torch.randperm(m, device=dev)
    timed("copy_engine_to_next", lambda: peers[nxt].copy_(x))
    timed("local_copy", lambda: buf.copy_(x))
    timed("scatter_contig_to_next", lambda: capi.scatter_rows_peers(ar, x, [(peers[nxt], 0, 0, m)]))
    timed("scatter_random_src_to_next", lambda: capi.scatter_rows_peers(perm, x, [(peers[nxt], 0, 0, m)]))
    timed("scatter_contig_local", lambda: capi.scatter_rows_peers(ar, x, [(buf, 0, 0, m)]))
    if world > 2:
        per = m // (world - 1)                                    # a piece of the rows to each of the other ranks
        recv = [(peers[(rank + 1 + k) % world], k * per, k * per, per) for k in range(world - 1)]
        timed("scatter_contig_to_all_others", lambda: capi.scatter_rows_peers(ar, x, recv), gb=per * (world - 1) * f * 4 / 1e9)

    out = torch.empty(m, f, device=dev)
    timed("projection_plain", lambda: capi.linear(x, w, out=out))
    ptr = torch.arange(m + 1, device=dev, dtype=torch.int32)
    ent_next = (torch.full((m,), nxt, device=dev, dtype=torch.int64) << 40) | ar
    ent_self = (torch.full((m,), rank, device=dev, dtype=torch.int64) << 40) | ar
    timed("projection_fan_next", lambda: capi.linear_fanout(x, w, capi.FanOut(peers, ptr, ent_next)))
    timed("projection_fan_self", lambda: capi.linear_fanout(x, w, capi.FanOut(peers, ptr, ent_self)))
    ent_perm = (torch.full((m,), nxt, device=dev, dtype=torch.int64) << 40) | perm
    timed("projection_fan_next_random_rows", lambda: capi.linear_fanout(x, w, capi.FanOut(peers, ptr, ent_perm)))
    if world > 2:
        who = (rank + 1 + (ar % (world - 1))) % world
        ent_all = (who << 40) | ar
        timed("projection_fan_all_others", lambda: capi.linear_fanout(x, w, capi.FanOut(peers, ptr, ent_all)))
    ptr2 = (torch.arange(m + 1, device=dev, dtype=torch.int64) * 2).to(torch.int32)       # every row to itself and to next
    ent2 = torch.stack([ent_self, ent_next], 1).reshape(-1).contiguous()
    timed("projection_fan_self_and_next", lambda: capi.linear_fanout(x, w, capi.FanOut(peers, ptr2, ent2)))
    line = {"world": world, "rows": m, "row_bytes": f * 4, **res}
    if rank == 0:
        print(json.dumps(line, indent=1), flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    dist.destroy_process_group()
    return line


if __name__ == "__main__":
    main()
