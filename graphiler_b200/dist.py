"""Destination-row sharding of a full-graph layer across the GPUs of one node.

The reference is single-GPU (python/graphiler/utils/setup.py:117 lists multiple devices as a
to-do); this module is new functionality.  One process per GPU:

* every operator on the path is a per-destination computation, so rank p owns a contiguous
  range of destination rows ``[rows[p], rows[p+1])`` chosen to balance the number of in-edges
  (not rows: power-law graphs put most edges in few rows);
* the dense projection is balanced by rows instead: rank p projects the equal-sized block
  ``[p*B, (p+1)*B)`` of source nodes, and one NCCL all-gather over NVLink assembles the full
  source-feature matrix in each GPU's own memory; kernels then read local memory only;
* or (``exchange="halo"``) every rank receives only the source rows its shard reads, through one all-to-all;
  source rows are then dealt to the ranks by a hash of their id (``owned_rows``), because on a power-law
  graph whose popular nodes have neighbouring ids a contiguous block would make one rank the sender of most
  of the traffic;
* with a sparse exchange the destination rows can be dealt by the same hash (``destinations="hashed"``): every
  shard then reads about the same number of distinct source rows, where the contiguous range of the many
  low-degree rows reads almost twice the rows of the range of the hubs and its inbound link sets every sender's pace;
* the row-split plan of a shard depends only on each row's own length, so putting the shards' output rows back at
  their ids (``gather_outputs``: concatenation in rank order for ranges) reproduces the single-GPU result bit for bit.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional

import torch
import torch.distributed as dist


def edge_balanced_row_ranges(pointer: torch.Tensor, world: int) -> List[int]:
    """Boundaries r_0=0 <= ... <= r_world=N such that every range holds about nnz/world entries."""
    n = pointer.numel() - 1
    nnz = int(pointer[-1])
    p64 = pointer.to(torch.int64)
    targets = torch.tensor([nnz * k // world for k in range(1, world)], dtype=torch.int64, device=pointer.device)
    cuts = torch.searchsorted(p64, targets, right=False).clamp(max=n).tolist() if world > 1 else []
    bounds = [0] + cuts + [n]
    for i in range(1, len(bounds)):              # keep monotone if many empty rows collapse cuts
        bounds[i] = max(bounds[i], bounds[i - 1])
    return bounds


def block_rows(n: int, world: int) -> int:
    """Rows per rank of the equal-sized source blocks (the last block is padded)."""
    return (n + world - 1) // world


@dataclass
class RowShard:
    """The CSC slice of one rank's destination rows: rebased pointer, global source ids.  The rows are the
    contiguous range [row0, row1), or - when ``rows`` is set - the listed rows (ascending ids; row0 / row1 are None)."""
    row0: Optional[int]
    row1: Optional[int]
    pointer: torch.Tensor          # (num_rows + 1) int32, starts at 0
    node_indices: torch.Tensor     # (nnz_local) int32, global source node ids
    edge0: Optional[int]           # first CSC position of a contiguous range (positions are global edge slots)
    rows: Optional[torch.Tensor] = None   # int64 global ids of the destination rows when they are not a range

    @property
    def num_rows(self):
        return int(self.pointer.numel()) - 1

    @property
    def nnz(self):
        return int(self.node_indices.numel())


def shard_rows(in_pointer: torch.Tensor, in_node_indices: torch.Tensor, row0: int, row1: int) -> RowShard:
    e0, e1 = int(in_pointer[row0]), int(in_pointer[row1])
    ptr = (in_pointer[row0:row1 + 1] - in_pointer[row0]).contiguous()
    return RowShard(row0, row1, ptr, in_node_indices[e0:e1].contiguous(), e0)


def shard_listed_rows(in_pointer: torch.Tensor, in_node_indices: torch.Tensor, rows: torch.Tensor) -> RowShard:
    """The CSC slice of the listed destination rows (int64, ascending), their segments copied one after the other."""
    p64 = in_pointer.to(torch.int64)
    start = p64[rows]
    deg = p64[rows + 1] - start
    ptr = torch.cat([torch.zeros(1, dtype=torch.int64, device=rows.device), torch.cumsum(deg, 0)])
    total = int(ptr[-1])
    if total >= 2 ** 31:
        raise ValueError("a shard holds at most 2^31 - 1 edges")
    pos = torch.arange(total, dtype=torch.int64, device=rows.device) + torch.repeat_interleave(start - ptr[:-1], deg)
    return RowShard(None, None, ptr.to(torch.int32).contiguous(), in_node_indices[pos].contiguous(), None, rows)


def hashed_owner(num_nodes: int, world: int, device) -> torch.Tensor:
    """Rank that owns each node id under the multiplicative hash used to deal rows to the ranks."""
    ids = torch.arange(num_nodes, dtype=torch.int64, device=device)
    return (((ids * 2654435761) & 0xFFFFFFFF) >> 13) % world


class ShardedLayer:
    """Per-rank state of one sharded layer: row shard, persistent all-gather buffer, plan.

    ``aggregate`` is the per-shard kernel call ``(shard, gathered_features, plan) -> local output``;
    it defaults to the CUDA kernels and exists as a parameter so the host logic (partition,
    all-gather, concatenation) can be exercised on CPU ranks.
    """

    def __init__(self, in_pointer, in_node_indices, num_nodes: int, feat: int, dtype=torch.float32,
                 rank: Optional[int] = None, world: Optional[int] = None, group=None, make_plan: bool = True,
                 chunks: int = 1, exchange: str = "allgather", ownership: Optional[str] = None, push_chunks: int = 4,
                 destinations: Optional[str] = None):
        self.group = group
        self.world = world if world is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)
        self.rank = rank if rank is not None else (dist.get_rank(group) if dist.is_initialized() else 0)
        self.num_nodes, self.feat = num_nodes, feat
        # Which destination rows a rank aggregates.  "ranges": contiguous, edge-balanced ranges (outputs concatenate in
        # rank order).  "hashed": the rows the rank also owns as a source under the hash - every shard then holds the
        # same mix of popular and unpopular rows, so the distinct source rows a shard reads (what it receives over
        # NVLink each step) are balanced as well as its edges; with contiguous ranges the shard of the many
        # low-degree rows reads 1.9 times the rows of the shard of the hubs, and its inbound link sets the pace of
        # every sender.  A layer's output rows are then the rows the rank projects in the next layer.
        if destinations is None:          # hashed wherever it is possible: a sparse exchange with hashed source rows
            destinations = "hashed" if exchange != "allgather" and ownership != "blocks" else "ranges"
        if destinations not in ("ranges", "hashed"):
            raise ValueError("destinations must be 'ranges' or 'hashed'")
        if destinations == "hashed" and (exchange == "allgather" or ownership == "blocks"):
            raise ValueError("destinations='hashed' goes with a sparse exchange and hashed source ownership")
        self.destinations = destinations if self.world > 1 else "ranges"
        self.bounds = edge_balanced_row_ranges(in_pointer, self.world)
        if self.destinations == "hashed":
            owner = hashed_owner(num_nodes, self.world, in_pointer.device)
            self.dst_rows = torch.nonzero(owner == self.rank).reshape(-1)                    # ascending ids
            self.shard = shard_listed_rows(in_pointer, in_node_indices, self.dst_rows)
        else:
            self.shard = shard_rows(in_pointer, in_node_indices, self.bounds[self.rank], self.bounds[self.rank + 1])
            self.dst_rows = torch.arange(self.shard.row0, self.shard.row1, dtype=torch.int64, device=in_pointer.device)
        # With chunks > 1 every rank's source block is cut into `chunks` pieces that are projected and gathered one
        # after the other, so the all-gather of piece c runs while piece c+1 is being projected.  The gather buffer
        # is then piece-major - piece c of every rank, rank-major, then piece c+1 ... - so that each collective
        # fills one contiguous slab, and the shard's source indices are renumbered to that layout once, here.
        if exchange not in ("allgather", "halo", "push", "fused"):
            raise ValueError("exchange must be 'allgather', 'halo', 'push' or 'fused'")
        # "push" is the halo exchange with the all-to-all replaced by this library's row-gather kernel storing the
        # requested rows straight into the receivers' buffers over NVLink (peer-mapped symmetric memory)
        # "fused" is "push" with the stores issued by the projection kernel's own epilogue: every finished 128-row tile
        # goes straight to the receivers that read it, and no second kernel re-reads the projected rows
        self.push = exchange in ("push", "fused") and self.world > 1
        self.fused = exchange == "fused" and self.world > 1 and feat % 4 == 0 and dtype == torch.float32
        self.push_chunks = push_chunks
        self.keep_projection = False    # fused form: also write the projected rows locally (layers that read them again)
        self.push_unavailable = None
        if exchange in ("push", "fused"):
            exchange = "halo"
        self.exchange = exchange if self.world > 1 else "allgather"
        self.phase_marks = None         # set to a list to have the halo path append (name, CUDA event) after each phase
        if self.exchange == "halo":
            chunks = 1
        self.chunks = max(1, int(chunks)) if self.world > 1 else 1
        self.block = (block_rows(num_nodes, self.world) + self.chunks - 1) // self.chunks * self.chunks
        self.chunk_rows = self.block // self.chunks
        if self.chunks > 1:
            s64 = self.shard.node_indices.to(torch.int64)
            r, o = s64 // self.block, s64 % self.block
            pos = ((o // self.chunk_rows) * self.world + r) * self.chunk_rows + o % self.chunk_rows
            self.shard.node_indices = pos.to(torch.int32)
        dev = in_pointer.device
        # which rank projects which source rows: contiguous equal blocks, or (halo default) dealt by a hash of the id
        self.ownership = ownership or ("hashed" if self.exchange == "halo" else "blocks")
        if self.ownership not in ("blocks", "hashed") or (self.ownership == "hashed" and self.exchange != "halo"):
            raise ValueError("ownership must be 'blocks', or 'hashed' together with exchange='halo'")
        lo = min(num_nodes, self.rank * self.block)
        self.owned_rows = torch.arange(lo, min(num_nodes, lo + self.block), dtype=torch.int64, device=dev)
        if self.exchange == "halo":
            self._setup_halo(feat, dtype, dev)
            self._extra = {}
            self.plan = None
            if make_plan and in_pointer.is_cuda:
                from . import capi
                self.plan = capi.Plan(self.shard.pointer, feat)
            return
        # persistent (world*block, feat) buffer; rows >= num_nodes are padding that no index refers to
        self.gathered = torch.zeros((self.world * self.block, feat), dtype=dtype, device=dev)
        self._extra = {}
        self.plan = None
        if make_plan and in_pointer.is_cuda:
            from . import capi
            self.plan = capi.Plan(self.shard.pointer, feat)

    def _setup_halo(self, feat: int, dtype, dev):
        """Sparse exchange instead of the all-gather: a shard only reads the source rows that occur in its index
        array (on a power-law graph cut 8 ways that is well under half of all rows), so every rank tells each owner
        once which of the owner's rows it needs, and each step the owners pack exactly those rows and one
        all-to-all delivers them into a compact buffer.  The shard's indices are renumbered to that buffer; the
        values and their order are unchanged, so results stay bit-identical to the single-GPU layer."""
        n, world = self.num_nodes, self.world
        ids = torch.arange(n, dtype=torch.int64, device=dev)
        if self.ownership == "hashed":
            owner_of = hashed_owner(n, world, dev)                                 # multiplicative hash of the row id
        else:
            owner_of = ids // self.block
        order = torch.argsort(owner_of, stable=True)                               # rows grouped by owner, ascending id
        counts = torch.bincount(owner_of, minlength=world)
        offsets = torch.cumsum(counts, 0) - counts
        local_of = torch.empty(n, dtype=torch.int64, device=dev)                   # position of a row in its owner's block
        local_of[order] = ids - offsets[owner_of[order]]
        o0, c0 = int(offsets[self.rank]), int(counts[self.rank])
        self.owned_rows = order[o0:o0 + c0].contiguous()
        idx64 = self.shard.node_indices.to(torch.int64)
        needed = torch.unique(idx64)
        keys, perm = torch.sort(owner_of[needed] * n + needed)                     # requests grouped by owner, then by id
        needed = needed[perm]
        need_counts = torch.bincount(owner_of[needed], minlength=world)
        self.recv_counts = need_counts.tolist()
        send_counts = torch.empty_like(need_counts)
        dist.all_to_all_single(send_counts, need_counts, group=self.group)
        self.send_counts = send_counts.tolist()
        ask = local_of[needed].contiguous()                                        # owner-relative row of each request
        asked = torch.empty(int(sum(self.send_counts)), dtype=torch.int64, device=dev)
        dist.all_to_all_single(asked, ask, output_split_sizes=self.send_counts, input_split_sizes=self.recv_counts,
                               group=self.group)
        self.send_rows = asked                                                    # rows of my block, grouped by requester
        self.shard.node_indices = torch.searchsorted(keys, owner_of[idx64] * n + idx64).to(torch.int32)
        # the destination rows of this shard, requested from their owners the same way (the GAT layer needs the
        # destination-side attention score of its own rows, which their owners compute): grouped by owner, then by id
        dst_ids = self.dst_rows
        dkeys, dperm = torch.sort(owner_of[dst_ids] * n + dst_ids)
        dst_sorted = dst_ids[dperm]
        self.dst_recv_counts = torch.bincount(owner_of[dst_sorted], minlength=world).tolist()
        dsend = torch.empty(world, dtype=torch.int64, device=dev)
        dist.all_to_all_single(dsend, torch.tensor(self.dst_recv_counts, dtype=torch.int64, device=dev), group=self.group)
        self.dst_send_counts = dsend.tolist()
        dasked = torch.empty(int(sum(self.dst_send_counts)), dtype=torch.int64, device=dev)
        dist.all_to_all_single(dasked, local_of[dst_sorted].contiguous(), output_split_sizes=self.dst_send_counts,
                               input_split_sizes=self.dst_recv_counts, group=self.group)
        self.dst_send_rows = dasked
        self.dst_position = torch.searchsorted(dkeys, owner_of[dst_ids] * n + dst_ids)     # received order -> row order
        self.proj = torch.zeros((c0, feat), dtype=dtype, device=dev)               # my projected rows
        self.send_buf = torch.empty((asked.numel(), feat), dtype=dtype, device=dev)
        self.gathered = torch.empty((needed.numel(), feat), dtype=dtype, device=dev)   # compact: only the rows this shard reads
        self.halo_rows = int(needed.numel())
        if self.push:
            self._setup_push(feat, dtype, dev)

    def _setup_push(self, feat: int, dtype, dev):
        """Peer-mapped receive buffers for the push exchange.  Every rank allocates the same (2, R, feat) tensor in
        symmetric memory (R = the largest halo of any rank; two slots used alternately, see project_and_gather) and
        learns where in each peer's buffer its own rows go: receiver p keeps the rows of sender r after those of
        senders 0..r-1, the order the all-to-all would deliver them in.  Falls back to the all-to-all, recording why,
        if symmetric memory cannot be set up on this machine."""
        world = self.world
        try:
            if not self.proj.is_cuda:
                raise RuntimeError("peer stores need CUDA tensors")
            import torch.distributed._symmetric_memory as symm
            counts = torch.tensor(self.recv_counts, dtype=torch.int64, device=dev)
            table = torch.empty((world, world), dtype=torch.int64, device=dev)         # table[p][r]: rows p receives from r
            dist.all_gather_into_tensor(table, counts, group=self.group)
            table = table.cpu()
            self.push_offset = [int(table[p, :self.rank].sum()) for p in range(world)]  # my first row in p's buffer
            rmax = max(1, int(table.sum(1).max()))
            buf = symm.empty((2, rmax, feat), dtype=dtype, device=dev)
            hdl = symm.rendezvous(buf, self.group if self.group is not None else dist.group.WORLD)
            self._symm_handle, self._symm_local = hdl, buf
            self.peer_bufs = [hdl.get_buffer(p, (2, rmax, feat), dtype) if p != self.rank else buf for p in range(world)]
            self.push_slot = 0
            self.send_offsets = [0]
            for c in self.send_counts:
                self.send_offsets.append(self.send_offsets[-1] + c)
            self._push_token = torch.zeros(1, dtype=torch.int32, device=dev)
            # The projection and the stores overlap piece by piece: the owned rows are cut into `push_chunks` ranges;
            # every requester's list is in ascending row order, so a range of rows is a range of each list.
            self.push_chunks = max(1, min(int(self.push_chunks), max(1, self.num_owned)))
            nm = self.num_owned
            self.push_bounds = [nm * c // self.push_chunks for c in range(self.push_chunks + 1)]
            cuts = []
            bvec = torch.tensor(self.push_bounds, dtype=torch.int64, device=dev)
            for peer in range(world):
                a, b = self.send_offsets[peer], self.send_offsets[peer + 1]
                cuts.append((torch.searchsorted(self.send_rows[a:b].contiguous(), bvec) + a).tolist())
            self.push_cuts = cuts                                    # push_cuts[peer][c]: first list position of piece c
            self._push_stream = torch.cuda.Stream(device=dev)
            # fan-out table of the fused form: for every owned row, the (receiver, row in its buffer) pairs that read it
            peer_of = torch.repeat_interleave(torch.arange(world, device=dev), torch.tensor(self.send_counts, device=dev))
            pos = torch.arange(self.send_rows.numel(), device=dev)
            first = torch.tensor(self.send_offsets[:-1], device=dev)[peer_of]
            dst_row = torch.tensor(self.push_offset, device=dev)[peer_of] + (pos - first)
            order = torch.argsort(self.send_rows, stable=True)
            self.fan_entry = ((peer_of << 40) | dst_row)[order].contiguous()
            counts = torch.bincount(self.send_rows, minlength=nm)
            self.fan_ptr = torch.cat([torch.zeros(1, dtype=torch.int64, device=dev), torch.cumsum(counts, 0)]).to(torch.int32)
        except Exception as ex:  # noqa: BLE001 - any failure means "use the all-to-all"
            self.push = self.fused = False
            self.push_unavailable = repr(ex)[:300]

    def exchange_rows(self, owned: torch.Tensor, which: str = "sources") -> torch.Tensor:
        """All-to-all of rows of a (num_owned, width) tensor this rank computed: ``which="sources"`` returns the rows
        this shard reads, in the compact order its renumbered indices refer to; ``which="destinations"`` returns the
        rows of this shard's own destination range, in row order.  Halo exchanges only."""
        assert self.exchange == "halo"
        if which == "destinations" and self.destinations == "hashed":
            return owned                                   # a rank's destination rows are the rows it owns, in this order
        if which == "sources":
            rows, sc, rc = self.send_rows, self.send_counts, self.recv_counts
        else:
            rows, sc, rc = self.dst_send_rows, self.dst_send_counts, self.dst_recv_counts
        if owned.is_cuda:
            from . import capi
            packed = capi.gather_rows(rows, owned)
        else:
            packed = owned.index_select(0, rows)
        got = torch.empty((int(sum(rc)),) + tuple(owned.shape[1:]), dtype=owned.dtype, device=owned.device)
        dist.all_to_all_single(got, packed, output_split_sizes=rc, input_split_sizes=sc, group=self.group)
        return got if which == "sources" else got.index_select(0, self.dst_position)

    @property
    def block_range(self):
        """(lo, hi) of this rank's contiguous source block (``ownership == 'blocks'``); see ``owned_rows``."""
        if self.ownership != "blocks":
            raise ValueError("source rows are dealt by hash: use owned_rows")
        lo = self.rank * self.block
        return lo, min(self.num_nodes, lo + self.block)

    @property
    def num_owned(self) -> int:
        return int(self.owned_rows.numel())

    def my_block(self) -> torch.Tensor:
        """View of this rank's slot in the gather buffer: write the projected rows here (chunks == 1 only)."""
        assert self.chunks == 1, "with chunks > 1 use project_and_gather"
        lo = self.rank * self.block
        return self.gathered[lo:lo + self.block]

    def all_gather(self):
        assert self.chunks == 1, "with chunks > 1 use project_and_gather"
        if self.world > 1:
            dist.all_gather_into_tensor(self.gathered, self.my_block(), group=self.group)
        return self.gathered

    def project_and_gather(self, fill: Callable) -> torch.Tensor:
        """Produce this rank's source rows and assemble everyone's.  ``fill(row_lo, row_hi, out)`` writes rows
        [row_lo, row_hi) of this rank's block (block-relative) into ``out``.  Piece by piece: the collective of a
        piece is issued asynchronously right after its rows were produced and overlaps the next piece's ``fill``."""
        n_mine = self.num_owned
        if self.exchange == "halo" and self.push:
            # One launch of the multi-receiver row-scatter kernel per piece: it reads the projected rows from local
            # memory and stores them through NVLink into every receiver's slot, dealing the rows so that concurrent
            # stores go to different receivers; it runs on a second stream while the next piece is projected.  Slots alternate between steps, so a sender that is one step ahead never overwrites rows a
            # receiver is still aggregating: between two writes to the same slot lies the other slot's barrier, which
            # a receiver enters only after that aggregation was launched on the same stream.  The barrier is a
            # one-word NCCL all-reduce: stream-ordered, and it completes on a rank only when every rank's stores of
            # this step were finished before it.
            from . import capi
            self._mark("start")
            slot, self.push_slot = self.push_slot, 1 - self.push_slot
            if self.fused:
                # the projection kernel stores every finished tile into the receivers' slots itself
                fan = capi.FanOut([b[slot] for b in self.peer_bufs], self.fan_ptr, self.fan_entry)
                fill(0, n_mine, self.proj[:n_mine] if self.keep_projection else None, fan)
                self._mark("project")
                self._mark("pack")
                dist.all_reduce(self._push_token, group=self.group)
                self._mark("exchange")
                return self._symm_local[slot, :self.halo_rows]
            main, side = torch.cuda.current_stream(), self._push_stream
            for c in range(self.push_chunks):
                r0, r1 = self.push_bounds[c], self.push_bounds[c + 1]
                if r1 > r0:
                    fill(r0, r1, self.proj[r0:r1])
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    recv = []
                    for k in range(self.world):
                        peer = (self.rank + k) % self.world
                        a, b = self.push_cuts[peer][c], self.push_cuts[peer][c + 1]
                        if b > a:
                            recv.append((self.peer_bufs[peer][slot], self.push_offset[peer] + (a - self.send_offsets[peer]), a, b - a))
                    if recv:
                        capi.scatter_rows_peers(self.send_rows, self.proj, recv)
            self._mark("project")
            main.wait_stream(side)
            self._mark("pack")
            dist.all_reduce(self._push_token, group=self.group)
            self._mark("exchange")
            return self._symm_local[slot, :self.halo_rows]
        if self.exchange == "halo":
            self._mark("start")
            fill(0, n_mine, self.proj[:n_mine])
            self._mark("project")
            if self.proj.is_cuda:
                from . import capi
                capi.gather_rows(self.send_rows, self.proj, out=self.send_buf)    # pack the requested rows
            else:
                torch.index_select(self.proj, 0, self.send_rows, out=self.send_buf)
            self._mark("pack")
            dist.all_to_all_single(self.gathered, self.send_buf, output_split_sizes=self.recv_counts,
                                   input_split_sizes=self.send_counts, group=self.group)
            self._mark("exchange")
            return self.gathered
        works = []
        for c in range(self.chunks):
            slab = self.gathered[c * self.world * self.chunk_rows:(c + 1) * self.world * self.chunk_rows]
            mine = slab[self.rank * self.chunk_rows:(self.rank + 1) * self.chunk_rows]
            r0, r1 = c * self.chunk_rows, min((c + 1) * self.chunk_rows, n_mine)
            if r1 > r0:
                fill(r0, r1, mine[:r1 - r0])
            if self.world > 1:
                works.append(dist.all_gather_into_tensor(slab, mine, group=self.group, async_op=True))
        for w in works:
            w.wait()
        return self.gathered

    def _mark(self, name: str):
        if self.phase_marks is not None and self.proj.is_cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.phase_marks.append((name, ev))

    def extra_buffer(self, name: str, width: int, dtype=None) -> torch.Tensor:
        """A further persistent (world*block, width) gather buffer (attention logits of the GAT layer); float32
        unless it was created with another dtype."""
        buf = self._extra.get(name)
        if dtype is None:
            dtype = buf.dtype if buf is not None else torch.float32
        if buf is None or buf.shape[1] != width or buf.dtype != dtype:
            buf = self._extra[name] = torch.zeros((self.world * self.block, width), dtype=dtype, device=self.gathered.device)
        return buf

    def all_gather_extra(self, name: str) -> torch.Tensor:
        buf = self._extra[name]
        if self.world > 1:
            lo = self.rank * self.block
            dist.all_gather_into_tensor(buf, buf[lo:lo + self.block], group=self.group)
        return buf

    def gather_outputs(self, local_out: torch.Tensor) -> torch.Tensor:
        """Every rank's output rows assembled in node-id order (testing / export helper): the ranges concatenated in
        rank order, or the hashed rows put back at their ids."""
        if self.world == 1:
            return local_out
        owner = order = None
        if self.destinations == "hashed":
            owner = hashed_owner(self.num_nodes, self.world, local_out.device)
            sizes = torch.bincount(owner, minlength=self.world).tolist()
            order = torch.argsort(owner, stable=True)                      # rank-major, ascending id within a rank
        else:
            sizes = [self.bounds[i + 1] - self.bounds[i] for i in range(self.world)]
        pad = max(sizes)                      # ranges differ in length: exchange equal-sized padded blocks, then trim
        mine = torch.zeros((pad,) + tuple(local_out.shape[1:]), dtype=local_out.dtype, device=local_out.device)
        mine[:local_out.shape[0]] = local_out
        outs = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(outs, mine, group=self.group)
        cat = torch.cat([o[:s] for o, s in zip(outs, sizes)], 0)
        if order is None:
            return cat
        full = torch.empty_like(cat)
        full[order] = cat
        return full


def gcn_layer_sharded(sl: ShardedLayer, feature_block: torch.Tensor, weight, norm_src_block, norm_dst_local,
                      relu: bool = True, aggregate: Optional[Callable] = None):
    """One GCN layer on this rank: project the local source block, all-gather, aggregate the local
    destination rows.  ``feature_block`` holds rows ``sl.owned_rows`` of the node features."""
    def fill(r0, r1, out, fan=None):
        if fan is not None:                                             # fused: the epilogue sends the rows itself
            from .layers import project
            project(feature_block[r0:r1], weight, norm_src_block[r0:r1], out=out, fan=fan)
        elif feature_block.is_cuda:
            from .layers import project
            if out.dtype == feature_block.dtype:
                project(feature_block[r0:r1], weight, norm_src_block[r0:r1], out=out)   # straight into the gather slot
            else:                                                       # bf16 storage: fp32 product, one rounding
                out.copy_(project(feature_block[r0:r1], weight, norm_src_block[r0:r1]))
        else:
            out.copy_(torch.mm(feature_block[r0:r1], weight).mul_(norm_src_block[r0:r1]))

    full = sl.project_and_gather(fill)
    if aggregate is None:
        from . import capi
        # destination scaling and relu ride in the aggregation kernel's epilogue
        scale = None if norm_dst_local is None else norm_dst_local.reshape(-1).float().contiguous()
        return capi.spmm_gather_sum(sl.shard.pointer, sl.shard.node_indices, full, sl.plan, dst_scale=scale, relu=relu)
    y = aggregate(sl.shard, full)
    if norm_dst_local is not None:
        y.mul_(norm_dst_local.to(y.dtype))
    return torch.relu_(y) if relu else y


def gcn_stack_sharded(sl: ShardedLayer, feature_block: torch.Tensor, weights, norm_block, aggregate: Optional[Callable] = None):
    """Several GCN layers in a row on one sharded graph (relu between the layers, none after the last; every layer
    ``sl.feat`` wide).  Needs ``destinations="hashed"``: a rank's output rows are then the rows it owns as a source, in
    the same order, so a layer's output is the next layer's ``feature_block`` as it stands and nothing is
    redistributed between the layers.  ``norm_block`` holds the normaliser of the owned rows, used on both sides."""
    if sl.world > 1 and sl.destinations != "hashed":
        raise ValueError("stacked layers need destinations='hashed' (the output rows of a range are not the rows the rank projects)")
    h = feature_block
    for i, w in enumerate(weights):
        h = gcn_layer_sharded(sl, h, w, norm_block, norm_block, relu=i + 1 < len(weights), aggregate=aggregate)
    return h


def gat_layer_sharded(sl: ShardedLayer, feature_block: torch.Tensor, fc_weight, attn_src, attn_dst, slope: float,
                      aggregate: Optional[Callable] = None):
    """One GAT layer on this rank: project the local source block (z, el, er), all-gather the three, then run the
    fused attention operator over the local destination rows.  er is needed for the local *destination* rows, whose
    edge-balanced range differs from the equal source block, so it is gathered too (N x H floats)."""
    if sl.exchange == "halo":
        # sparse form: every rank projects the rows it owns and computes their two attention scores; the rows this
        # shard reads travel as in the GCN layer (z through project_and_gather, which may store them straight into the
        # receivers' buffers; the 8-float score rows through a small all-to-all), and the destination-side scores of
        # this shard's own rows come from their owners the same way
        heads, dim = attn_src.shape
        sdt = torch.float32 if feature_block.is_cuda else feature_block.dtype
        scores = {k: torch.empty((sl.num_owned, heads), dtype=sdt, device=feature_block.device) for k in ("el", "er")}
        a_s, a_d = attn_src.contiguous(), attn_dst.contiguous()

        sl.keep_projection = True                   # the head scores read the projected rows again

        def fill(r0, r1, out, fan=None):             # called once, or once per piece of the owned rows
            if feature_block.is_cuda:
                from . import capi
                from .layers import project
                z = project(feature_block[r0:r1], fc_weight, out=out, fan=fan)
                capi.gat_head_scores(z, a_s, a_d, el=scores["el"][r0:r1], er=scores["er"][r0:r1])
            else:
                z = torch.mm(feature_block[r0:r1], fc_weight)
                zv = z.view(-1, heads, dim)
                scores["el"][r0:r1], scores["er"][r0:r1] = (zv * attn_src).sum(-1), (zv * attn_dst).sum(-1)
                out.copy_(z)

        full_z = sl.project_and_gather(fill)
        full_el = sl.exchange_rows(scores["el"], "sources")
        er_local = sl.exchange_rows(scores["er"], "destinations")
        if aggregate is None:
            from . import capi
            return capi.gat_fused(sl.shard.pointer, sl.shard.node_indices, None, full_el, er_local, full_z, slope, sl.plan)
        return aggregate(sl.shard, full_el, er_local, full_z)
    assert sl.chunks == 1 and sl.exchange == "allgather", \
        "the dense GAT layer gathers three tensors in one step: build its ShardedLayer with chunks=1"
    lo, hi = sl.block_range
    heads, dim = attn_src.shape
    mine = sl.my_block()
    el_buf, er_buf = sl.extra_buffer("el", heads), sl.extra_buffer("er", heads)
    b0 = sl.rank * sl.block
    if feature_block.is_cuda:
        from . import capi
        from .layers import project
        z = project(feature_block, fc_weight, out=mine[:hi - lo])         # straight into the gather slot
        capi.gat_head_scores(z, attn_src.contiguous(), attn_dst.contiguous(), el=el_buf[b0:b0 + hi - lo],
                             er=er_buf[b0:b0 + hi - lo])
    else:
        z = torch.mm(feature_block, fc_weight)
        zv = z.view(-1, heads, dim)
        el_buf[b0:b0 + hi - lo] = (zv * attn_src).sum(-1)
        er_buf[b0:b0 + hi - lo] = (zv * attn_dst).sum(-1)
        mine[:hi - lo].copy_(z)
    full_z = sl.all_gather()
    full_el, full_er = sl.all_gather_extra("el"), sl.all_gather_extra("er")
    er_local = full_er[sl.shard.row0:sl.shard.row1]
    if aggregate is None:
        from . import capi
        return capi.gat_fused(sl.shard.pointer, sl.shard.node_indices, None, full_el, er_local, full_z, slope, sl.plan)
    return aggregate(sl.shard, full_el, er_local, full_z)
