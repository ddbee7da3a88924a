"""Row-partitioned SpMM / SDDMM / attention / AutoSAGEConv over the GPUs of one node (one process per GPU).

The reference is single-GPU.  For graphs that should be spread over 2/4/8 B200s the destination
rows are cut into contiguous ranges balanced by nnz; rank r owns rows [b_r, b_{r+1}), the matching
slice of col/val (row pointers rebased to 0), the X rows of the same range and the output rows.
Every output row needs X rows of arbitrary columns, so X is gathered over NVLink into a full-height
local buffer.  On CUDA the buffer lives in symmetric memory and each rank pulls the other P-1 shards
with plain device-to-device copies on a side stream (copy engines, no SMs), in the order rank+1,
rank+2, ...; with NCCL (or gloo on CPU) the same transfer is P-1 grouped send/recv steps, step s
moving rank r's shard to rank (r - s) mod P while the shard of rank (r + s) mod P arrives.  To overlap,
the local CSR is pre-split into column blocks by owner (optionally several consecutive arrivals per
block); the block of the rank's own columns is multiplied first (no wait) and each further block as
soon as its last shard has landed, accumulating into the same output rows.  Summation order therefore
differs from the single-GPU kernel (block by block) but stays inside the float32 tolerance; all
integer outputs (bounds, block CSRs) are deterministic.

Remote data is always landed in local memory before a kernel reads it; ordering is by stream events
and the symmetric-memory barriers only.  CPU tensors with the gloo backend run the same
orchestration with torch's CPU SpMM, which is how the logic is tested without GPUs.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.distributed as dist

from . import _native
from .conv import apply_linear
from .ops import DEFAULT_HUB_THRESHOLD, DEFAULT_WARPS, load_native


def partition_rows(crow: torch.Tensor, parts: int) -> torch.Tensor:
    """Boundaries b_0..b_parts of contiguous row ranges with ~nnz/parts edges each:
    b_k = first row whose pointer is >= k*nnz/parts (int64, on the CPU)."""
    crow = crow.to(torch.long)
    n = crow.numel() - 1
    base = int(crow[0])
    nnz = int(crow[-1]) - base
    targets = torch.tensor([base + (k * nnz) // parts for k in range(parts + 1)], dtype=torch.long,
                           device=crow.device)
    bounds = torch.searchsorted(crow.contiguous(), targets, right=False).clamp_(0, n).cpu()
    bounds[0], bounds[-1] = 0, n
    return torch.cummax(bounds, 0).values


@dataclass
class ColumnBlock:
    """The edges of a shard whose columns belong to one owner rank, as a CSR over the shard's rows.
    Column ids stay global (they index the gathered X)."""

    owner: int
    crow: torch.Tensor
    col: torch.Tensor
    val: Optional[torch.Tensor]
    workspace: Optional[torch.Tensor] = None
    plan_ready: bool = False
    pack_short: bool = False   # rows hold a fraction of their edges: run short rows one per lane group


@dataclass
class RowShard:
    rank: int
    world: int
    bounds: torch.Tensor          # int64[world + 1], CPU
    crow: torch.Tensor            # local row pointers, rebased to 0
    col: torch.Tensor             # global column ids
    val: Optional[torch.Tensor]
    blocks: list[ColumnBlock] = field(default_factory=list)   # one per column group, in arrival order
    groups: list[list[int]] = field(default_factory=list)     # owners of each block

    @property
    def row_begin(self) -> int:
        return int(self.bounds[self.rank])

    @property
    def row_end(self) -> int:
        return int(self.bounds[self.rank + 1])

    @property
    def n_local(self) -> int:
        return self.row_end - self.row_begin

    @property
    def n_global(self) -> int:
        return int(self.bounds[-1])


def arrival_order(rank: int, world: int) -> list[int]:
    """Owners in the order their X shards become available on ``rank``: its own, then rank+1, ..."""
    return [(rank + s) % world for s in range(world)]


def column_groups(rank: int, world: int, groups=None) -> list[list[int]]:
    """The arrival order cut into runs of consecutive arrivals: ``groups`` equal runs when it is an
    int (all singletons when None), or runs of the given sizes when it is a sequence summing to
    ``world`` (e.g. (1, 3, 3, 1): the rank's own columns alone, so the first product needs no
    transfer, and a one-owner last group, so little work is left after the last arrival).
    The SpMM of a group can start once its last member has arrived."""
    order = arrival_order(rank, world)
    if groups is not None and not isinstance(groups, int):
        sizes = [int(v) for v in groups]
        if any(v < 1 for v in sizes) or sum(sizes) != world:
            raise ValueError(f"group sizes {sizes} must be positive and sum to the world size {world}")
    else:
        k = world if groups is None else max(1, min(int(groups), world))
        base, extra = divmod(world, k)
        sizes = [base + (1 if g < extra else 0) for g in range(k)]
    out, start = [], 0
    for size in sizes:
        out.append(order[start:start + size])
        start += size
    return out


def split_edges_by_group(crow: torch.Tensor, col: torch.Tensor, val: Optional[torch.Tensor], group: torch.Tensor,
                         n_groups: int, labels: Optional[list[int]] = None) -> list[ColumnBlock]:
    """Stable partition of a CSR's edges by ``group[e]`` (int64, one entry per edge): block g is a CSR
    over the same rows holding the edges of group g in their original order.  ``labels[g]`` becomes the
    block's ``owner`` field (default g)."""
    n_local = crow.numel() - 1
    device = col.device
    degrees = crow[1:] - crow[:-1]
    rows = torch.repeat_interleave(torch.arange(n_local, device=device, dtype=torch.long), degrees)
    order = torch.argsort(group * max(n_local, 1) + rows, stable=True)
    per_group = torch.bincount(group[order], minlength=n_groups).cpu().tolist()
    blocks: list[ColumnBlock] = []
    start = 0
    for g in range(n_groups):
        stop = start + per_group[g]
        picked = order[start:stop]
        counts = torch.bincount(rows[picked], minlength=n_local)
        block_crow = torch.zeros(n_local + 1, dtype=torch.long, device=device)
        torch.cumsum(counts, 0, out=block_crow[1:])
        blocks.append(ColumnBlock(g if labels is None else labels[g], block_crow, col[picked].contiguous(),
                                  None if val is None else val[picked].contiguous()))
        start = stop
    return blocks


def split_columns_by_owner(crow: torch.Tensor, col: torch.Tensor, val: Optional[torch.Tensor],
                           bounds: torch.Tensor, groups: Optional[list[list[int]]] = None) -> list[ColumnBlock]:
    """Stable partition of a CSR's edges by the group of owner(col), owner k holding columns
    bounds[k] <= col < bounds[k+1]; edge order inside a (row, group) pair is preserved.  Without
    ``groups`` every owner is its own group, in owner order.  Block g covers groups[g]; its
    ``owner`` field is the LAST owner of the group (the one whose arrival releases the block)."""
    world = bounds.numel() - 1
    if groups is None:
        groups = [[k] for k in range(world)]
    device = col.device
    cuts = bounds[1:-1].to(device)
    owner = torch.bucketize(col, cuts, right=True) if world > 1 else torch.zeros_like(col)
    group_of = torch.empty(world, dtype=torch.long)
    for g, members in enumerate(groups):
        for k in members:
            group_of[k] = g
    return split_edges_by_group(crow, col, val, group_of.to(device)[owner], len(groups),
                                labels=[members[-1] for members in groups])


class GatherLayout:
    """Where row g of the gathered operand lives in a rank's buffer when the exchange moves CHUNKS of
    every shard at once (one collective, or one push, per chunk) instead of one owner's shard at a time.

    Shards are cut into ``chunks`` pieces of ``chunk_rows`` rows (the last piece of a shard may be
    shorter or empty; shards are padded to ``chunks * chunk_rows`` rows).  The buffer holds, chunk after
    chunk, that chunk of every owner in owner order:
        position(owner k, local row i) = (i // chunk_rows) * world * chunk_rows + k * chunk_rows + i % chunk_rows
    so chunk c of all owners is the contiguous slice ``chunk_view(buffer, c)`` - the output of one
    all-gather whose per-rank input is ``own_view(buffer, c, rank)``, a slice of that output."""

    def __init__(self, bounds: torch.Tensor, chunks: int) -> None:
        self.bounds = bounds.to(torch.long).cpu()
        self.world = self.bounds.numel() - 1
        self.chunks = max(1, int(chunks))
        longest = int((self.bounds[1:] - self.bounds[:-1]).max()) if self.world else 0
        self.chunk_rows = max(1, -(-longest // self.chunks))
        self.rows_total = self.chunks * self.world * self.chunk_rows

    def owner_and_local(self, rows: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        cuts = self.bounds[1:-1].to(rows.device)
        owner = torch.bucketize(rows, cuts, right=True) if self.world > 1 else torch.zeros_like(rows)
        return owner, rows - self.bounds.to(rows.device)[owner]

    def position(self, rows: torch.Tensor) -> torch.Tensor:
        """Buffer positions of the global row ids ``rows`` (any device)."""
        owner, local = self.owner_and_local(rows)
        chunk = torch.div(local, self.chunk_rows, rounding_mode="floor")
        return chunk * (self.world * self.chunk_rows) + owner * self.chunk_rows + (local - chunk * self.chunk_rows)

    def chunk_of(self, rows: torch.Tensor) -> torch.Tensor:
        return torch.div(self.owner_and_local(rows)[1], self.chunk_rows, rounding_mode="floor")

    def chunk_view(self, buffer: torch.Tensor, chunk: int) -> torch.Tensor:
        span = self.world * self.chunk_rows
        return buffer[chunk * span:(chunk + 1) * span]

    def own_view(self, buffer: torch.Tensor, chunk: int, rank: int) -> torch.Tensor:
        begin = chunk * self.world * self.chunk_rows + rank * self.chunk_rows
        return buffer[begin:begin + self.chunk_rows]

    def local_pieces(self, rank: int) -> list[tuple[int, int, int]]:
        """(first local row, number of rows, buffer position) of the pieces of rank's own shard."""
        n_local = int(self.bounds[rank + 1] - self.bounds[rank])
        pieces = []
        for chunk in range(self.chunks):
            first = chunk * self.chunk_rows
            count = min(self.chunk_rows, n_local - first)
            if count > 0:
                pieces.append((first, count, chunk * self.world * self.chunk_rows + rank * self.chunk_rows))
        return pieces


def shard_csr(crow: torch.Tensor, col: torch.Tensor, val: Optional[torch.Tensor], rank: int, world: int,
              bounds: Optional[torch.Tensor] = None, device: Optional[torch.device] = None,
              groups: Optional[int] = None) -> RowShard:
    """Cut rank ``rank``'s rows out of a full CSR (on any device) and build its column blocks, one per
    group of ``column_groups(rank, world, groups)`` in arrival order."""
    bounds = partition_rows(crow, world) if bounds is None else bounds
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    first, last = int(crow[lo]), int(crow[hi])
    local_crow = (crow[lo:hi + 1] - crow[lo]).to(torch.long)
    local_col = col[first:last]
    local_val = None if val is None else val[first:last]
    if device is not None:
        local_crow, local_col = local_crow.to(device), local_col.to(device)
        local_val = None if local_val is None else local_val.to(device)
    local_crow, local_col = local_crow.contiguous(), local_col.contiguous()
    local_val = None if local_val is None else local_val.contiguous()
    shard = RowShard(rank, world, bounds, local_crow, local_col, local_val)
    shard.groups = column_groups(rank, world, groups)
    shard.blocks = split_columns_by_owner(local_crow, local_col, local_val, bounds, shard.groups)
    return shard


def exchange_schedule(rank: int, world: int) -> list[tuple[int, int]]:
    """(send_to, receive_from) for steps 1..world-1: every rank sends and receives exactly one shard
    per step and all links of the switch are busy at once."""
    return [((rank - s) % world, (rank + s) % world) for s in range(1, world)]


def _block_spmm(block: ColumnBlock, x_full: torch.Tensor, y: torch.Tensor, accumulate: bool, *, feature_tile: int,
                warps: int, threshold: int) -> None:
    if y.is_cuda:
        if block.workspace is None:
            block.workspace = torch.empty(_native.workspace_bytes(y.size(0)), dtype=torch.uint8, device=y.device)
            block.plan_ready = False
        flags = (_native.FLAG_ACCUMULATE if accumulate else 0) | (_native.FLAG_PLAN_READY if block.plan_ready else 0)
        if block.pack_short:
            flags |= _native.FLAG_PACK_SHORT_ROWS
        _native.spmm(block.crow, block.col, block.val, x_full, y, feature_tile=feature_tile, warps=warps,
                     threshold=threshold, flags=flags, workspace=block.workspace)
        block.plan_ready = True
        return
    weights = torch.ones(block.col.numel(), dtype=x_full.dtype) if block.val is None else block.val.to(x_full.dtype)
    matrix = torch.sparse_csr_tensor(block.crow, block.col, weights, size=(y.size(0), x_full.size(0)), dtype=x_full.dtype)
    product = torch.sparse.mm(matrix, x_full)
    if accumulate:
        y.add_(product)
    else:
        y.copy_(product)


class ShardedSpmm:
    """Holds the gathered-X buffer, the exchange machinery and the per-block plans of one shard.

    Exchange modes
      "peer"  (default on CUDA) X lives in symmetric memory (torch.distributed._symmetric_memory);
              every rank PULLS the other shards with plain device-to-device copies on a side
              stream, which the driver runs on the copy engines: NVLink traffic without occupying
              SMs, so the column-block SpMMs keep the whole GPU.  One barrier before the pulls (all
              shards written) and one after (all pulls done, shards may be overwritten).
      "nccl"  P-1 grouped isend/irecv steps; also the path of the CPU/gloo tests.
      "allgather"  the collective itself: ``chunks`` calls of all_gather_into_tensor (NCCL picks its own
              algorithm, NVLS included), chunk c of every shard at once, in the padded chunk-major layout
              of ``GatherLayout``.  Column blocks are then "own columns" (no wait) plus one per chunk.
      "push"  SM-driven: every rank stores chunk c of its own shard into all peers' buffers with plain
              128-bit stores (``asg_push_to_peers``, ``push_ctas`` CTAs), a symmetric-memory barrier after
              every chunk; same layout and column blocks as "allgather".
    """

    def __init__(self, shard: RowShard, features: int, *, group=None, dtype=torch.float32, feature_tile: int = 128,
                 warps: int = DEFAULT_WARPS, threshold: int = DEFAULT_HUB_THRESHOLD,
                 exchange: Optional[str] = None, copy_streams: int = 1, slabs: int = 0, chunks: int = 2,
                 push_ctas: int = 32, pack_short_rows: bool = False) -> None:
        self.shard = shard
        self.group = group
        self.features = features
        self.feature_tile, self.warps, self.threshold = feature_tile, warps, threshold
        device = shard.crow.device
        self.device = device
        if device.type == "cuda" and not load_native():
            raise RuntimeError("libautosage_b200.so is required for the CUDA path")
        self.comm_stream = torch.cuda.Stream(device=device) if device.type == "cuda" else None
        # further streams for the pulls (peer mode): consecutive sources alternate between them
        self.copy_streams = ([torch.cuda.Stream(device=device) for _ in range(max(0, int(copy_streams) - 1))]
                             if device.type == "cuda" else [])
        self.handle = None
        self.x_full = None
        self.layout: Optional[GatherLayout] = None
        self.push_ctas = int(push_ctas)
        wanted = exchange or os.getenv("AUTOSAGE_EXCHANGE", "peer" if device.type == "cuda" else "nccl")
        if wanted in ("allgather", "push") and shard.world > 1:
            self.layout = GatherLayout(shard.bounds, chunks)
            if wanted == "push" and device.type == "cuda":
                self._try_symmetric(dtype, rows=self.layout.rows_total)
            if self.x_full is None:
                self.x_full = torch.empty(self.layout.rows_total, features, dtype=dtype, device=device)
            self.exchange = "push" if self.handle is not None else "allgather"
            self._chunk_blocks = self._build_chunk_blocks()
            self._chunk_events = [torch.cuda.Event() for _ in range(self.layout.chunks)] if device.type == "cuda" else []
        else:
            if wanted == "peer" and device.type == "cuda" and shard.world > 1:
                self._try_symmetric(dtype)
            if self.x_full is None:
                self.x_full = torch.empty(shard.n_global, features, dtype=dtype, device=device)
            self.exchange = "peer" if self.handle is not None else "nccl"
        if not shard.groups:
            shard.groups = [[k] for k in arrival_order(shard.rank, shard.world)]
        # A row of a column block holds 1/P .. 1/groups of its edges; running such short rows one per
        # lane group (ASG_FLAG_PACK_SHORT_ROWS) was measured on 4 GPUs and did not pay (2.92 ms per step
        # against 2.87 ms): off unless asked for.
        for block in (self._chunk_blocks if self.layout is not None else shard.blocks):
            block.pack_short = bool(pack_short_rows) and shard.world > 1
        # Feature-slab mode (peer exchange only): X is pulled in `slabs` bands of feature columns, band s
        # of every remote shard before band s+1, and each band is multiplied over the WHOLE local CSR
        # as soon as it is complete.  No column blocks, so rows keep their full degree and nothing is
        # accumulated into Y twice; the price is that no product can start before the first band is in.
        self.slabs = 0
        if self.exchange == "peer" and slabs and slabs > 1 and features % (32 * slabs) == 0:
            self.slabs = int(slabs)
            self._whole = ColumnBlock(shard.rank, shard.crow, shard.col, shard.val)
            self._slab_events = [torch.cuda.Event() for _ in range(self.slabs)]
        self._events = [torch.cuda.Event() for _ in range(shard.world)] if device.type == "cuda" else []
        self._opened = torch.cuda.Event() if device.type == "cuda" else None
        # Optional timeline: set ``trace`` to a list and every forward appends {name: timing event};
        # ``timeline_ms`` turns the collected steps into mean offsets from the step's start.
        self.trace: Optional[list] = None
        self._marks: Optional[dict] = None

    def _mark(self, name: str, stream=None) -> None:
        if self._marks is not None:
            event = torch.cuda.Event(enable_timing=True)
            event.record(stream if stream is not None else torch.cuda.current_stream(self.device))
            self._marks[name] = event

    def timeline_ms(self) -> dict:
        """Mean offset (ms) of every recorded mark from "start", over the traced steps (synchronises)."""
        torch.cuda.synchronize(self.device)
        sums: dict = {}
        for marks in self.trace or []:
            for name, event in marks.items():
                if name != "start":
                    sums.setdefault(name, []).append(marks["start"].elapsed_time(event))
        return {name: round(sum(v) / len(v), 4) for name, v in sums.items()}

    def _try_symmetric(self, dtype, rows: Optional[int] = None) -> None:
        """Allocate X in symmetric memory and map the peers' copies; all ranks agree on the outcome.
        With ``rows`` (chunked layouts) each peer's WHOLE buffer is mapped, else only the peer's own shard."""
        ok = 1
        try:
            import torch.distributed._symmetric_memory as symm

            pg = self.group if self.group is not None else dist.group.WORLD
            total = self.shard.n_global if rows is None else rows
            buffer = symm.empty((total, self.features), dtype=dtype, device=self.device)
            handle = symm.rendezvous(buffer, pg)
            peers = {}
            b = self.shard.bounds
            for owner in range(self.shard.world):
                if owner != self.shard.rank:
                    if rows is None:
                        count = int(b[owner + 1]) - int(b[owner])
                        peers[owner] = handle.get_buffer(owner, (count, self.features), dtype, int(b[owner]) * self.features)
                    else:
                        peers[owner] = handle.get_buffer(owner, (total, self.features), dtype, 0)
        except Exception as exc:  # noqa: BLE001 - any failure means "use NCCL send/recv instead"
            self._symmetric_error = exc
            ok = 0
        flag = torch.tensor([ok], device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 1:
            self.x_full, self.handle, self._peers = buffer, handle, peers

    @property
    def x_local(self) -> torch.Tensor:
        """View of the rank's own rows inside the gathered buffer: write the shard's features here.
        (Chunked layouts keep the shard in several pieces: use ``load_local`` there.)"""
        if self.layout is not None:
            raise RuntimeError("the chunked layout has no single view of the local rows; use load_local()")
        return self.x_full[self.shard.row_begin:self.shard.row_end]

    def load_local(self, features: torch.Tensor, non_blocking: bool = False) -> None:
        """Copy this rank's feature rows (``[n_local, F]``, any device) into the gathered buffer."""
        if self.layout is None:
            if features.data_ptr() != self.x_local.data_ptr():
                self.x_local.copy_(features, non_blocking=non_blocking)
            return
        for first, count, position in self.layout.local_pieces(self.shard.rank):
            self.x_full[position:position + count].copy_(features[first:first + count], non_blocking=non_blocking)

    def _build_chunk_blocks(self) -> list[ColumnBlock]:
        """Chunked layouts: block 0 holds the edges into this rank's own columns, block 1 + c the edges
        into the other ranks' columns of chunk c; column ids become positions in the gathered buffer."""
        shard, layout = self.shard, self.layout
        owner, local = layout.owner_and_local(shard.col)
        chunk = torch.div(local, layout.chunk_rows, rounding_mode="floor")
        group = torch.where(owner == shard.rank, torch.zeros_like(chunk), chunk + 1)
        return split_edges_by_group(shard.crow, layout.position(shard.col), shard.val, group, layout.chunks + 1)

    def _start_chunk_exchange(self) -> None:
        """Chunked layouts, on the communication stream (CPU: inline): chunk after chunk of every shard,
        an event after each."""
        shard, layout = self.shard, self.layout
        if self.exchange == "push":
            main = self.comm_stream
            self.handle.barrier(channel=0)  # every rank is done reading the previous contents
            self._mark("pulls_begin", main)
            others = [owner for owner in arrival_order(shard.rank, shard.world)[1:]]
            for c in range(layout.chunks):
                own = layout.own_view(self.x_full, c, shard.rank)
                _native.push_to_peers(own, [layout.own_view(self._peers[o], c, shard.rank) for o in others], self.push_ctas)
                self.handle.barrier(channel=0)  # all ranks' stores of this chunk have completed
                self._chunk_events[c].record(main)
            self._mark("pulls_end", main)
            return
        for c in range(layout.chunks):
            whole, own = layout.chunk_view(self.x_full, c), layout.own_view(self.x_full, c, shard.rank)
            if self.comm_stream is None:
                dist.all_gather_into_tensor(whole.view(-1), own.reshape(-1), group=self.group)
                continue
            if c == 0:
                self._mark("pulls_begin", self.comm_stream)
            work = dist.all_gather_into_tensor(whole.view(-1), own.view(-1), group=self.group, async_op=True)
            work.wait()  # the communication stream (current here) waits for the collective; the host does not
            self._chunk_events[c].record(self.comm_stream)
        if self.comm_stream is not None:
            self._mark("pulls_end", self.comm_stream)

    def _shard_view(self, owner: int) -> torch.Tensor:
        b = self.shard.bounds
        return self.x_full[int(b[owner]):int(b[owner + 1])]

    def _start_exchange(self) -> list[tuple[int, list]]:
        """NCCL/gloo mode: one grouped send+recv per step; returns (source rank, works) per step."""
        shard = self.shard
        steps: list[tuple[int, list]] = []
        for send_to, recv_from in exchange_schedule(shard.rank, shard.world):
            ops = [dist.P2POp(dist.isend, self.x_local, send_to, group=self.group),
                   dist.P2POp(dist.irecv, self._shard_view(recv_from), recv_from, group=self.group)]
            steps.append((recv_from, dist.batch_isend_irecv(ops)))
        return steps

    def _start_pulls(self) -> None:
        """Peer mode, on the communication stream: barrier, one copy-engine pull per source in
        arrival order (an event after each), barrier."""
        shard = self.shard
        main = self.comm_stream
        self.handle.barrier(channel=0)
        self._mark("pulls_begin", main)
        streams = [main] + self.copy_streams
        if self.copy_streams:
            self._opened.record(main)
            for extra in self.copy_streams:
                extra.wait_event(self._opened)
        sources = arrival_order(shard.rank, shard.world)[1:]
        for i, owner in enumerate(sources):
            stream = streams[i % len(streams)]
            with torch.cuda.stream(stream):
                self._shard_view(owner).copy_(self._peers[owner], non_blocking=True)
                self._events[owner].record(stream)
        if self.copy_streams:
            for owner in sources:
                main.wait_event(self._events[owner])
        self._mark("pulls_end", main)
        self.handle.barrier(channel=1)
        self._mark("closing_barrier", main)

    def _start_slab_pulls(self) -> None:
        """Slab mode, on the communication stream: barrier, then band after band of feature columns
        from every source (pitched copy-engine copies), an event after each band, barrier."""
        shard = self.shard
        main = self.comm_stream
        width = self.features // self.slabs
        self.handle.barrier(channel=0)
        streams = [main] + self.copy_streams
        if self.copy_streams:
            self._opened.record(main)
            for extra in self.copy_streams:
                extra.wait_event(self._opened)
        sources = arrival_order(shard.rank, shard.world)[1:]
        for band in range(self.slabs):
            for i, owner in enumerate(sources):
                stream = streams[i % len(streams)]
                with torch.cuda.stream(stream):
                    _native.copy_columns(self._shard_view(owner), self._peers[owner], band * width, width)
            for extra in self.copy_streams:  # the band is complete when every stream has finished its share
                self._opened.record(extra)
                main.wait_event(self._opened)
            self._slab_events[band].record(main)
        self.handle.barrier(channel=1)

    def _slab_products(self, y: torch.Tensor, current, after_band=None) -> None:
        """One SpMM per band over the whole local CSR; with ``current`` given, each waits for its band.
        ``after_band(band, first_column, width)`` runs after each band's product is enqueued."""
        width = self.features // self.slabs
        tile = min(self.feature_tile, width)
        block = self._whole
        if block.workspace is None:
            block.workspace = torch.empty(_native.workspace_bytes(y.size(0)), dtype=torch.uint8, device=y.device)
            block.plan_ready = False
        for band in range(self.slabs):
            if current is not None:
                current.wait_event(self._slab_events[band])
            _native.spmm_range(block.crow, block.col, block.val, self.x_full, y, feature_begin=band * width,
                               feature_count=width, feature_tile=tile, warps=self.warps, threshold=self.threshold,
                               flags=_native.FLAG_PLAN_READY if block.plan_ready else 0, workspace=block.workspace)
            block.plan_ready = True
            if after_band is not None:
                after_band(band, band * width, width)

    def exchange_only(self) -> None:
        """Runs just the gather of X (for measurements); the current stream waits for its end."""
        if self.shard.world == 1:
            return
        if self.layout is not None:
            if self.comm_stream is None:
                self._start_chunk_exchange()
                return
            current = torch.cuda.current_stream(self.device)
            self.comm_stream.wait_stream(current)
            with torch.cuda.stream(self.comm_stream):
                self._start_chunk_exchange()
            current.wait_stream(self.comm_stream)
            return
        if self.exchange == "peer":
            current = torch.cuda.current_stream(self.device)
            self.comm_stream.wait_stream(current)
            with torch.cuda.stream(self.comm_stream):
                if self.slabs:
                    self._start_slab_pulls()
                else:
                    self._start_pulls()
            current.wait_stream(self.comm_stream)
            return
        for _, works in self._start_exchange():
            for work in works:
                work.wait()

    def forward(self, out: Optional[torch.Tensor] = None, overlap: bool = True, *, before_products=None,
                after_band=None) -> torch.Tensor:
        """y_local = A_local @ gather(X).  ``x_local`` must already hold this rank's features.

        Slab mode only: ``before_products()`` runs on the current stream once the pulls are enqueued,
        ``after_band(band, first_column, width)`` after each band's product (the layer uses them to
        run its Linear band by band, under the transfer of the following band)."""
        shard = self.shard
        y = out if out is not None else torch.empty(shard.n_local, self.features, dtype=self.x_full.dtype,
                                                    device=self.device)
        kw = dict(feature_tile=self.feature_tile, warps=self.warps, threshold=self.threshold)
        self._marks = {} if self.trace is not None else None
        if self._marks is not None:
            self.trace.append(self._marks)
        self._mark("start")
        if shard.world == 1:
            _block_spmm(shard.blocks[0], self.x_full, y, False, **kw)
            self._mark("spmm_end")
            return y

        if self.layout is not None:
            blocks = self._chunk_blocks
            if self.comm_stream is None:  # CPU ranks: exchange first, then the products
                self._start_chunk_exchange()
                for g, block in enumerate(blocks):
                    _block_spmm(block, self.x_full, y, g > 0, **kw)
                return y
            current = torch.cuda.current_stream(self.device)
            self.comm_stream.wait_stream(current)
            with torch.cuda.stream(self.comm_stream):
                self._start_chunk_exchange()
            if not overlap:
                current.wait_stream(self.comm_stream)
            for g, block in enumerate(blocks):
                if overlap and g > 0:
                    current.wait_event(self._chunk_events[g - 1])
                _block_spmm(block, self.x_full, y, g > 0, **kw)
                self._mark(f"block{g}_end")
            current.wait_stream(self.comm_stream)
            return y

        if self.exchange == "peer" and self.slabs:
            current = torch.cuda.current_stream(self.device)
            self.comm_stream.wait_stream(current)
            with torch.cuda.stream(self.comm_stream):
                self._start_slab_pulls()
            if not overlap:
                current.wait_stream(self.comm_stream)
            if before_products is not None:
                before_products()
            self._slab_products(y, current if overlap else None, after_band)
            current.wait_stream(self.comm_stream)
            return y

        if self.exchange == "peer":
            current = torch.cuda.current_stream(self.device)
            self.comm_stream.wait_stream(current)
            with torch.cuda.stream(self.comm_stream):
                self._start_pulls()
            if not overlap:
                current.wait_stream(self.comm_stream)
            for g, (block, members) in enumerate(zip(shard.blocks, shard.groups)):
                if overlap:
                    for member in members:
                        if member != shard.rank:
                            current.wait_event(self._events[member])
                _block_spmm(block, self.x_full, y, g > 0, **kw)
                self._mark(f"block{g}_end")
            # the closing barrier of the exchange must be part of this step's stream order
            current.wait_stream(self.comm_stream)
            return y

        if self.comm_stream is not None:
            current = torch.cuda.current_stream(self.device)
            self.comm_stream.wait_stream(current)
            with torch.cuda.stream(self.comm_stream):
                steps = self._start_exchange()
        else:
            steps = self._start_exchange()
        arrived = {shard.rank}
        pending = list(steps)
        for g, (block, members) in enumerate(zip(shard.blocks, shard.groups)):
            need = set(members) if overlap else set(range(shard.world))
            while not need <= arrived:
                source, works = pending.pop(0)
                for work in works:
                    work.wait()  # CUDA: the current stream waits for the collective, the host does not
                arrived.add(source)
            _block_spmm(block, self.x_full, y, g > 0, **kw)
        for _, works in pending:
            for work in works:
                work.wait()
        return y


class _GatheredOperand:
    """A dense operand indexed by COLUMN (K or V), gathered like X: the exchange half of a
    ``ShardedSpmm`` without its products."""

    def __init__(self, shard: RowShard, features: int, group, exchange: Optional[str]) -> None:
        self._engine = ShardedSpmm(shard, features, group=group, exchange=exchange)

    @property
    def local(self) -> torch.Tensor:
        return self._engine.x_local

    @property
    def full(self) -> torch.Tensor:
        return self._engine.x_full

    @property
    def exchange(self) -> str:
        return self._engine.exchange

    def gather(self, local: Optional[torch.Tensor]) -> torch.Tensor:
        if local is not None:
            self._engine.load_local(local)
        self._engine.exchange_only()
        return self.full


def _cpu_sddmm(crow, col, query, key) -> torch.Tensor:
    rows = torch.repeat_interleave(torch.arange(crow.numel() - 1, device=crow.device), crow[1:] - crow[:-1])
    return (query.index_select(0, rows) * key.index_select(0, col)).sum(dim=1)


def _cpu_row_softmax(crow, scores) -> torch.Tensor:
    if scores.numel() == 0:
        return scores.clone()
    rows = torch.repeat_interleave(torch.arange(crow.numel() - 1, device=crow.device), crow[1:] - crow[:-1])
    peak = torch.full((crow.numel() - 1,), -torch.inf, dtype=scores.dtype, device=scores.device)
    peak.scatter_reduce_(0, rows, scores, reduce="amax", include_self=True)
    shifted = (scores - peak.index_select(0, rows)).exp()
    total = torch.zeros_like(peak).scatter_add_(0, rows, shifted)
    return shifted / total.index_select(0, rows)


class ShardedSddmm:
    """SDDMM over a row shard: ``out[e] = <Q[row(e)], K[col[e]]>`` for the shard's edges.  Q is
    row-local; K is gathered over NVLink exactly like X (every shard's rows into a full-height
    buffer), then the SDDMM kernels run over the local rows against the gathered K."""

    def __init__(self, shard: RowShard, features: int, *, group=None, warps: int = 8, threshold: int = 8192,
                 exchange: Optional[str] = None) -> None:
        self.shard, self.warps, self.threshold = shard, warps, threshold
        self.keys = _GatheredOperand(shard, features, group, exchange)
        self._workspace = None
        self._plan_ready = False

    def forward(self, query_local: torch.Tensor, key_local: Optional[torch.Tensor] = None) -> torch.Tensor:
        shard = self.shard
        key_full = self.keys.gather(key_local)
        if not query_local.is_cuda:
            return _cpu_sddmm(shard.crow, shard.col, query_local, key_full)
        query = query_local.contiguous()
        out = torch.empty(shard.col.numel(), dtype=query.dtype, device=query.device)
        if out.numel() == 0:
            return out
        if self._workspace is None:
            self._workspace = torch.empty(_native.workspace_bytes(shard.n_local), dtype=torch.uint8, device=query.device)
        _native.sddmm(shard.crow, shard.col, query, key_full, out, warps=self.warps, threshold=self.threshold,
                      flags=_native.FLAG_PLAN_READY if self._plan_ready else 0, workspace=self._workspace)
        self._plan_ready = True
        return out


class ShardedAttention:
    """softmax_row(scale * Q K^T on the shard's CSR pattern) V for the shard's rows.  Q is row-local;
    K and V are gathered like X; the fused one-pass kernel then runs over the local rows."""

    def __init__(self, shard: RowShard, features: int, *, group=None, warps: int = 4, threshold: int = 1024,
                 exchange: Optional[str] = None) -> None:
        if features > 512:
            raise ValueError("the fused attention kernel takes at most 512 features")
        self.shard, self.warps, self.threshold = shard, warps, threshold
        self.keys = _GatheredOperand(shard, features, group, exchange)
        self.values = _GatheredOperand(shard, features, group, exchange)
        self._workspace = None
        self._plan_ready = False

    def forward(self, query_local: torch.Tensor, key_local: Optional[torch.Tensor] = None,
                value_local: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
        shard = self.shard
        key_full = self.keys.gather(key_local)
        value_full = self.values.gather(value_local)
        if not query_local.is_cuda:
            scores = _cpu_sddmm(shard.crow, shard.col, query_local * scale, key_full)
            weights = _cpu_row_softmax(shard.crow, scores)
            matrix = torch.sparse_csr_tensor(shard.crow, shard.col, weights, size=(shard.n_local, shard.n_global))
            return torch.sparse.mm(matrix, value_full)
        query = query_local.contiguous()
        out = torch.empty_like(query)
        if out.numel() == 0:
            return out
        if self._workspace is None:
            self._workspace = torch.empty(_native.workspace_bytes(shard.n_local) + _native.attention_extra_bytes(shard.n_local),
                                          dtype=torch.uint8, device=query.device)
        _native.attention(shard.crow, shard.col, query, key_full, value_full, out, scale=float(scale), warps=self.warps,
                          threshold=self.threshold, flags=_native.FLAG_PLAN_READY if self._plan_ready else 0,
                          workspace=self._workspace)
        self._plan_ready = True
        return out


class ShardedAutoSAGEConv(torch.nn.Module):
    """AutoSAGEConv over a row shard: gathered aggregation, then the layer's Linear on local rows."""

    def __init__(self, shard: RowShard, in_channels: int, out_channels: int, *, bias: bool = True, group=None,
                 feature_tile: int = 128, warps: int = DEFAULT_WARPS, threshold: int = DEFAULT_HUB_THRESHOLD,
                 exchange: Optional[str] = None, copy_streams: int = 1, slabs: int = 0, chunks: int = 2,
                 push_ctas: int = 32, pack_short_rows: bool = False) -> None:
        super().__init__()
        self.linear = torch.nn.Linear(in_channels, out_channels, bias=bias)
        self.spmm = ShardedSpmm(shard, in_channels, group=group, feature_tile=feature_tile, warps=warps,
                                threshold=threshold, exchange=exchange, copy_streams=copy_streams, slabs=slabs,
                                chunks=chunks, push_ctas=push_ctas, pack_short_rows=pack_short_rows)

    def capture(self, warmup: int = 2):
        """Captures one inference forward (features already in ``spmm.x_local``) into a CUDA graph and
        returns ``replay() -> out``; ``out`` is the same tensor on every replay.

        The pulls, both symmetric-memory barriers, every column-block SpMM and the Linear become one
        graph launch, so a step costs the host one call instead of a few dozen - at 4 and 8 GPUs a step
        is 2-3 ms of GPU work and the eager launch sequence does not always stay ahead of it.  All
        ranks must call this together; if any rank fails to capture, all return None (run eagerly)."""
        spmm = self.spmm
        if spmm.device.type != "cuda" or (spmm.shard.world > 1 and spmm.exchange == "nccl"):
            return None  # the send/recv exchange is driven from the host (work.wait()), step by step
        ok = 1
        graph, out = None, None
        try:
            with torch.no_grad():
                for _ in range(max(warmup, 1)):  # builds the plans and fills the allocator's pools
                    self.forward()
                torch.cuda.synchronize(spmm.device)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    out = self.forward()
        except Exception as exc:  # noqa: BLE001 - any failure means "stay eager"
            self._capture_error = exc
            ok = 0
        if spmm.shard.world > 1:
            flag = torch.tensor([ok], device=spmm.device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=spmm.group)
            ok = int(flag.item())
        if not ok:
            return None

        def replay() -> torch.Tensor:
            graph.replay()
            return out

        replay.graph = graph
        return replay

    def forward(self, x_local: Optional[torch.Tensor] = None, overlap: bool = True) -> torch.Tensor:
        if x_local is not None:
            self.spmm.load_local(x_local)
        spmm = self.spmm
        differentiating = torch.is_grad_enabled() and any(p.requires_grad for p in self.linear.parameters())
        if not spmm.slabs or spmm.shard.world == 1 or differentiating:
            out = apply_linear(self.linear, spmm.forward(overlap=overlap))
            spmm._mark("linear_end")
            return out
        # Slab mode: out = bias + sum over bands of Y[:, band] @ W[:, band]^T.  The partial product of
        # band s runs while band s+1 is still crossing NVLink, so only the last band's SpMM and its
        # partial GEMM remain after the transfer.
        linear = self.linear
        out = torch.empty(spmm.shard.n_local, linear.out_features, dtype=spmm.x_full.dtype, device=spmm.device)
        y = torch.empty(spmm.shard.n_local, spmm.features, dtype=spmm.x_full.dtype, device=spmm.device)
        weight_t = linear.weight.t()

        def before_products():
            if linear.bias is not None:
                out.copy_(linear.bias.expand_as(out))

        def after_band(band, first, width):
            part, w = y[:, first:first + width], weight_t[first:first + width]
            if band == 0 and linear.bias is None:
                torch.mm(part, w, out=out)
            else:
                out.addmm_(part, w)

        spmm.forward(out=y, overlap=overlap, before_products=before_products, after_band=after_band)
        return out
