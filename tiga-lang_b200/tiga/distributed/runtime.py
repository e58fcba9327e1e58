"""Halo-exchange runtime for destination-partitioned message passing.

What it keeps from the reference (python/tiga/distributed/transport.py:692-1403
and nccl.py:209-284 of walkerchi/TIGA-lang): one process per rank, contiguous
destination ranges, ghosts = sorted unique remote sources, ghost rows numbered
after the owned rows in ascending global id, one grouped send/recv per source
field per call, reverse exchange of ghost cotangents summed into owned rows in
the backward, and the ``with DistributedRuntime(transport):`` calling
convention.

What is different by design: everything is built with tensor ops on the
graph's device (the reference walks Python lists of the whole CSR,
transport.py:969-983), peers' rows are received straight into their slice of
the ghost buffer (ghost ids are sorted, so each owner's rows are contiguous: no
unpack copies), and communication overlaps compute on every call: the relation
is split by EDGE into the part whose sources are owned and the part whose
sources are ghosts; the owned part runs while the halo is in flight and the
ghost part is accumulated onto it afterwards (the reference's public policy is
communication-then-compute, transport.py:702-705).

The local compute is a backend object so that the host logic can be exercised
on CPU ranks (gloo) in tests with a checker backend; the product backend is the
native CUDA library and nothing else.
"""
from __future__ import annotations

import contextvars
from dataclasses import dataclass

import torch
import torch.distributed as dist

from .. import capture as cap
from ..graph import Graph
from ..reducer import SumReducer
from .model import HaloMap, partition_bounds

_ACTIVE = contextvars.ContextVar("tiga_distributed_runtime", default=None)
DEFAULT_WAVES = 3


def current_distributed_runtime():
    return _ACTIVE.get()


class ProcessGroupTransport:
    """Neighbour exchange over a ``torch.distributed`` process group (NCCL
    send/recv over NVLink on GPUs, gloo on CPU ranks)."""

    def __init__(self, group=None):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.group = group
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)

    def _peer(self, rank: int) -> int:
        return rank if self.group is None else dist.get_global_rank(self.group, rank)

    def exchange(self, sends, receives):
        """Start one grouped exchange; ``sends``/``receives`` are lists of
        (peer, contiguous tensor).  Returns the outstanding work handles."""
        ops = [dist.P2POp(dist.irecv, tensor, self._peer(peer), self.group) for peer, tensor in receives
               if tensor.numel()]
        ops += [dist.P2POp(dist.isend, tensor, self._peer(peer), self.group) for peer, tensor in sends
                if tensor.numel()]
        return dist.batch_isend_irecv(ops) if ops else []

    @staticmethod
    def wait(works) -> None:
        for work in works:
            work.wait()

    def all_gather_counts(self, counts: torch.Tensor) -> torch.Tensor:
        gathered = [torch.empty_like(counts) for _ in range(self.world_size)]
        dist.all_gather(gathered, counts, group=self.group)
        return torch.stack(gathered)

    def all_reduce_sum(self, tensor: torch.Tensor) -> torch.Tensor:
        dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=self.group)
        return tensor


class NCCLTransport(ProcessGroupTransport):
    """``NCCLTransport(rank, world_size, device=...)``: initialises the default
    NCCL process group from the launcher's environment when none exists."""

    def __init__(self, rank: int | None = None, world_size: int | None = None, unique_id=None, *,
                 device=None, group=None):
        if not dist.is_initialized():
            kwargs = {}
            if rank is not None and world_size is not None:
                kwargs = {"rank": rank, "world_size": world_size}
            if device is not None:
                kwargs["device_id"] = torch.device(device)
            dist.init_process_group("nccl", **kwargs)
        super().__init__(group)


class NativeBackend:
    """Local compute through the CUDA library (the only product backend)."""

    @staticmethod
    def forward(graph, x, w, accumulate_into=None):
        from .. import ops

        out, _ = ops.csr_reduce_forward(graph.native_plan(transpose=False), "sum", x, w, 0.0,
                                        accumulate_into=accumulate_into)
        return out

    @staticmethod
    def begin_forward(shard):
        """A new forward over the shard: weights kept in transposed order by the last backward go."""
        from .. import ops

        for relation in (shard.graph_own, shard.graph_ghost):
            for plan in relation._plans.values():
                ops.forget_transposed_weights(plan)

    @staticmethod
    def backward_dx(graph, dy, w):
        from .. import ops

        return ops.csr_reduce_backward_dx(graph.native_plan(transpose=True), "sum", dy, w)

    @staticmethod
    def pack_rows(rows, ids):
        from .. import ops

        return ops.rows_gather(rows, ids)

    @staticmethod
    def add_rows(rows, ids, packed):
        from .. import ops

        ops.rows_scatter_add(rows, ids, packed)

    @staticmethod
    def backward_dw(graph, dy, x, out):
        from .. import ops

        return ops.csr_reduce_backward_dw(graph.native_plan(transpose=False), "sum", dy, x, out=out)


class DistributedRuntime:
    """``with DistributedRuntime(transport): kernel(graph=g.halo(mesh), ...)``.

    ``trace=True`` records a CUDA event on the compute stream at every phase boundary of a sharded call
    (pack + start exchange, owned-source part, exposed wait for the halo, ghost-source part, ...);
    ``phase_times()`` turns the marks of the calls since the last ``reset_trace()`` into milliseconds
    per phase.  Device timestamps, not host clocks, so an exposed wait is what the stream really waited
    (the reference's ``last_execution_trace`` keeps host nanoseconds and declines to claim overlap,
    python/tiga/distributed/transport.py:1311-1370)."""

    def __init__(self, transport: ProcessGroupTransport, *, backend=None, trace: bool = False,
                 waves: int | None = None, push: bool = False, window_slots: int = 4):
        self.transport = transport
        self.backend = backend or NativeBackend()
        self._token = None
        self.trace = bool(trace)
        self.last_execution_trace = []
        # push=True (one node, CUDA): halo rows are stored straight into the receivers' ghost buffers
        # through peer windows (see peer.py) instead of pack + send / recv; off by default
        self.push = bool(push)
        self.window_slots = max(int(window_slots), 2)
        self._windows = {}
        self._signals = None
        self._comm_stream = None
        # the forward halo arrives in `waves` grouped exchanges; the ghost-source edges of a wave
        # are reduced as soon as that wave has landed, while the later waves are still in flight
        self.waves = DEFAULT_WAVES if waves is None else max(int(waves), 1)

    def reset_trace(self) -> None:
        self.last_execution_trace = []

    # ---------------------------------------------------------------- peer windows (push=True)
    def comm_stream(self, device):
        if self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=device)
        return self._comm_stream

    def signals(self, device):
        from .peer import PushSignals

        if self._signals is None:
            self._signals = PushSignals(self.transport, device)
        return self._signals

    def halo_windows(self, shard: "ShardPlan", F: int, device):
        """(ghost window, cotangent window) of a shard for rows of F floats; created collectively on
        first use.  A slot of the ghost window is this rank's ghost buffer [G, F]; a slot of the
        cotangent window holds, peer after peer, the cotangent rows the peers return."""
        from .peer import PeerWindow

        key = (id(shard), int(F))
        if key not in self._windows:
            row_bytes = 4 * int(F)
            ghost_layout = {"recv_offsets": [o for o, _ in shard.recv_offsets]}
            ghost = PeerWindow(self.transport, device, int(shard.ghosts.numel()) * row_bytes, self.window_slots,
                               ghost_layout)
            starts, total = [], 0
            for ids in shard.send_ids:
                starts.append(total)
                total += int(ids.numel())
            landing = PeerWindow(self.transport, device, total * row_bytes, 2, {"starts": starts})
            self._windows[key] = (ghost, landing, starts)
        return self._windows[key]

    def mark(self, name: str, device) -> None:
        if self.trace and torch.device(device).type == "cuda":
            event = torch.cuda.Event(enable_timing=True)
            event.record(torch.cuda.current_stream(device))
            self.last_execution_trace.append((name, event))

    def phase_times(self) -> dict:
        """Milliseconds between consecutive marks, summed per phase name (the name of a mark is the
        phase that ENDS there).  Synchronises."""
        totals = {}
        marks = self.last_execution_trace
        if marks:
            marks[-1][1].synchronize()
        for (_, before), (name, after) in zip(marks[:-1], marks[1:]):
            if name.endswith(":begin"):
                continue
            totals[name] = totals.get(name, 0.0) + before.elapsed_time(after)
        return totals

    def __enter__(self):
        self._token = _ACTIVE.set(self)
        return self

    def __exit__(self, *exc):
        _ACTIVE.reset(self._token)
        self._token = None
        return False


@dataclass
class ShardPlan:
    """Everything one rank needs to run its destination rows of a graph."""

    rank: int
    world_size: int
    bounds: list            # partition begin offsets + end, len world_size + 1
    begin: int
    end: int
    ghosts: torch.Tensor    # [G] ascending global ids of remote sources
    recv_offsets: list      # per peer: (offset, count) into the ghost buffer
    send_ids: list          # per peer: local row indices (tensor) that peer needs
    graph_own: Graph        # local rows x owned sources
    graph_ghost: Graph      # local rows x ghost sources (all of them: the backward uses this one)
    edges_own: torch.Tensor    # positions of the owned-source edges in the local edge list
    edges_ghost: torch.Tensor  # positions of the ghost-source edges
    num_local_edges: int
    waves: list             # per wave: (peers received from, Graph of the ghost-source edges they own)

    @property
    def owned(self) -> int:
        return self.end - self.begin

    def halo_map(self) -> HaloMap:
        """The reference's HaloMap of this rank (same ids, same grouping)."""
        ghosts = self.ghosts.tolist()
        receives, sends = [], []
        for peer, (offset, count) in enumerate(self.recv_offsets):
            if count:
                receives.append((peer, tuple(ghosts[offset:offset + count])))
        for peer, ids in enumerate(self.send_ids):
            if ids.numel():
                sends.append((peer, tuple((ids + self.begin).tolist())))
        return HaloMap(rank=self.rank, world_size=self.world_size, owned_begin=self.begin, owned_end=self.end,
                       ghost_ids=tuple(ghosts), receive_from=tuple(receives), send_to=tuple(sends))


def exchange_waves(rank: int, world: int, waves: int) -> list:
    """Peers in the order their rows are received, cut into at most `waves` consecutive groups.
    Ring order: at step s (1 .. world-1) a rank receives from rank - s and sends to rank + s, so
    every step pairs all ranks up at once and the groups of all ranks line up."""
    steps = list(range(1, world))
    if not steps:
        return []
    waves = min(max(waves, 1), len(steps))
    cuts = [(len(steps) * k) // waves for k in range(waves + 1)]
    return [[((rank - s) % world, (rank + s) % world) for s in steps[cuts[k]:cuts[k + 1]]] for k in range(waves)]


def _local_rows(graph: Graph, transport: ProcessGroupTransport):
    """(bounds, local row_ptr starting at 0 as int64, local col_idx with global ids)."""
    world, rank = transport.world_size, transport.rank
    n = graph.num_dst
    if graph._shard is not None:
        first_row, _ = graph._shard
        row_ptr, col_idx = graph._row_ptr, graph._col_idx
        mine = torch.tensor([first_row, row_ptr.numel() - 1], dtype=torch.int64, device=row_ptr.device)
        blocks = transport.all_gather_counts(mine).tolist()
        bounds = [int(b[0]) for b in blocks] + [n]
        for r, (first, rows) in enumerate(blocks):
            if first + rows != bounds[r + 1] or (r == 0 and first != 0):
                raise ValueError("the ranks' blocks of rows do not tile [0, num_nodes) in rank order: "
                                 f"rank {r} holds rows [{first}, {first + rows}), the next block starts at "
                                 f"{bounds[r + 1]}")
        return bounds, row_ptr.to(torch.int64), col_idx
    row_ptr, col_idx = graph.resolve_csr()
    placement = graph.placement
    balance = placement.partition.balance if placement is not None else "auto"
    bounds = partition_bounds(n, world, row_ptr=row_ptr, balance=balance)
    begin, end = bounds[rank], bounds[rank + 1]
    first, last = int(row_ptr[begin].item()), int(row_ptr[end].item())
    return bounds, (row_ptr[begin:end + 1] - first).to(torch.int64), col_idx[first:last]


def build_shard_plan(graph: Graph, transport: ProcessGroupTransport, waves: int = 1) -> ShardPlan:
    """Partition, ghost lists, request exchange and the local relations."""
    if graph.num_src != graph.num_dst:
        raise NotImplementedError("halo partitions need a homogeneous relation (num_src == num_dst)")
    world, rank = transport.world_size, transport.rank
    placement = graph.placement
    if placement is not None and placement.mesh.size != world:
        raise ValueError(f"graph was placed on a mesh of {placement.mesh.size} ranks, the runtime has {world}")
    bounds, local_ptr, local_col = _local_rows(graph, transport)
    begin, end = bounds[rank], bounds[rank + 1]
    owned = end - begin
    device, index_dtype = local_ptr.device, graph.schema.index_dtype
    if local_col.numel() >= 1 << 31:
        raise NotImplementedError("more than 2^31 local edges per rank")
    local_col = local_col.to(torch.int64)
    degree = local_ptr[1:] - local_ptr[:-1]
    local_dst = torch.repeat_interleave(torch.arange(owned, device=device), degree)
    is_own = (local_col >= begin) & (local_col < end)

    def sub_relation(positions, columns, num_src):
        """CSR over the owned rows of the edges at `positions` (ascending) of the local edge list;
        it reads the caller's per-edge arrays through those positions."""
        counts = torch.bincount(local_dst[positions], minlength=owned)
        ptr = torch.zeros(owned + 1, dtype=torch.int64, device=device)
        torch.cumsum(counts, 0, out=ptr[1:])
        relation = Graph.from_csr(ptr.to(index_dtype), columns.to(index_dtype).contiguous(), num_src=num_src)
        relation._edge_map = positions.to(torch.int32)
        return relation

    edges_own = torch.nonzero(is_own).reshape(-1)
    edges_ghost = torch.nonzero(~is_own).reshape(-1)
    del is_own
    ghost_cols = local_col[edges_ghost]
    ghosts = torch.unique(ghost_cols, sorted=True)
    num_ghosts = int(ghosts.numel())
    graph_own = sub_relation(edges_own, local_col[edges_own] - begin, owned)
    ghost_slot = torch.searchsorted(ghosts, ghost_cols)           # position in the ghost buffer
    graph_ghost = sub_relation(edges_ghost, ghost_slot, num_ghosts)

    # ghosts are sorted, owners are contiguous ranges => each owner's ids are one slice
    bound_t = torch.tensor(bounds, dtype=torch.int64, device=device)
    cuts = torch.searchsorted(ghosts, bound_t).tolist()
    recv_offsets = [(cuts[p], cuts[p + 1] - cuts[p]) for p in range(world)]

    # the forward reduces the ghost-source edges wave by wave: one sub-relation per wave of peers
    wave_plans = []
    schedule = exchange_waves(rank, world, waves)
    if len(schedule) <= 1:
        wave_plans = [([pair for pair in schedule[0]] if schedule else [], graph_ghost)]
    else:
        wave_of_peer = torch.full((world,), -1, dtype=torch.int64, device=device)
        for k, pairs in enumerate(schedule):
            for source, _ in pairs:
                wave_of_peer[source] = k
        owner = torch.searchsorted(bound_t, ghost_cols, right=True) - 1
        wave_of_edge = wave_of_peer[owner]
        for k, pairs in enumerate(schedule):
            chosen = torch.nonzero(wave_of_edge == k).reshape(-1)
            wave_plans.append((pairs, sub_relation(edges_ghost[chosen], ghost_slot[chosen], num_ghosts)))
        del owner, wave_of_edge
    del ghost_cols, ghost_slot, local_dst

    # tell every owner which of its rows this rank needs
    counts = torch.tensor([c for _, c in recv_offsets], dtype=torch.int64, device=device)
    matrix = transport.all_gather_counts(counts)      # matrix[r, p] = rows rank r needs from p
    incoming = matrix[:, rank].tolist()
    requests = [torch.empty(incoming[p], dtype=torch.int64, device=device) for p in range(world)]
    works = transport.exchange(
        sends=[(p, ghosts[o:o + c].contiguous()) for p, (o, c) in enumerate(recv_offsets) if p != rank],
        receives=[(p, requests[p]) for p in range(world) if p != rank])
    transport.wait(works)
    send_ids = [(requests[p] - begin) if p != rank else requests[p][:0] for p in range(world)]
    for ids in send_ids:
        if ids.numel() and (int(ids.min()) < 0 or int(ids.max()) >= owned):
            raise RuntimeError("a peer requested a row this rank does not own")
    return ShardPlan(rank=rank, world_size=world, bounds=bounds, begin=begin, end=end, ghosts=ghosts,
                     recv_offsets=recv_offsets, send_ids=send_ids, graph_own=graph_own, graph_ghost=graph_ghost,
                     edges_own=edges_own, edges_ghost=edges_ghost, num_local_edges=int(local_col.numel()),
                     waves=wave_plans)


def shard_plan_for(graph: Graph, runtime: DistributedRuntime) -> ShardPlan:
    cache = graph.__dict__.setdefault("_shard_plans", {})
    key = (id(runtime.transport), runtime.transport.rank, runtime.transport.world_size, runtime.waves)
    if key not in cache:
        cache[key] = build_shard_plan(graph, runtime.transport, runtime.waves)
    return cache[key]


def _push_forward(runtime, shard: ShardPlan, window, slot: int, rows, w_own, w_ghost, F: int):
    """Forward halo through peer windows: every wave's rows are gathered straight into the
    receivers' ghost buffers by the row mover, on the communication stream, and a one-element
    all-reduce after the wave tells every rank that the wave has landed everywhere."""
    from .peer import push_rows

    backend = runtime.backend
    device = rows.device
    compute = torch.cuda.current_stream(device)
    comm = runtime.comm_stream(device)
    signals = runtime.signals(device)
    ghost_x = window.view(slot, (int(shard.ghosts.numel()), F))
    row_bytes = 4 * F
    comm.wait_stream(compute)                              # the rows to send are final
    if window.released[slot] is not None:
        comm.wait_event(window.released[slot])             # this rank's last read of the slot
    landed = []
    with torch.cuda.stream(comm):
        signals.barrier()                                  # ... and every other rank's: the slot is free everywhere
        for pairs, _ in shard.waves:
            for _, target in pairs:
                ids = shard.send_ids[target]
                if ids.numel():
                    where = window.peer_layout[target]["recv_offsets"][shard.rank] * row_bytes
                    push_rows(rows, ids, window.address(target, slot, where))
            signals.barrier()
            landed.append(comm.record_event())
    rows.record_stream(comm)
    runtime.mark("forward pack + start exchange", device)
    out = backend.forward(shard.graph_own, rows, w_own)
    runtime.mark("forward owned-source part", device)
    for (_, relation), event in zip(shard.waves, landed):
        compute.wait_event(event)
        runtime.mark("forward exposed halo wait", device)
        if relation.resolve_csr()[1].numel():
            out = backend.forward(relation, ghost_x, w_ghost, accumulate_into=out)
        runtime.mark("forward ghost-source part", device)
    return out, ghost_x


def _push_cotangents(runtime, shard: ShardPlan, d_ghost, F: int):
    """Reverse halo through peer windows: each owner's slice of the ghost cotangents is copied into
    that owner's landing window; returns (landed, (event, window, slot))."""
    from .peer import push_block

    device = d_ghost.device
    _, landing, starts = runtime.halo_windows(shard, F, device)
    slot = landing.acquire()
    if slot is None:
        raise RuntimeError("the cotangent window is still in use: backward calls must not overlap")
    compute = torch.cuda.current_stream(device)
    comm = runtime.comm_stream(device)
    signals = runtime.signals(device)
    row_bytes = 4 * F
    comm.wait_stream(compute)                              # d_ghost is final
    if landing.released[slot] is not None:
        comm.wait_event(landing.released[slot])
    with torch.cuda.stream(comm):
        signals.barrier()                                  # the landing slot is free on every rank
        for owner, (offset, count) in enumerate(shard.recv_offsets):
            if count and owner != shard.rank:
                where = landing.peer_layout[owner]["starts"][shard.rank] * row_bytes
                push_block(d_ghost[offset:offset + count], landing.address(owner, slot, where))
        signals.barrier()
        done = comm.record_event()
    d_ghost.record_stream(comm)
    total_rows = starts[-1] + int(shard.send_ids[-1].numel()) if starts else 0
    buffer = landing.view(slot, (max(total_rows, 1), F))
    landed = [(p, ids, buffer[starts[p]:starts[p] + ids.numel()]) for p, ids in enumerate(shard.send_ids)
              if ids.numel()]
    return landed, (done, landing, slot)


class _HaloWeightedSum(torch.autograd.Function):
    """out[owned rows] = sum over local edges of w * x[source], sources owned or ghost."""

    @staticmethod
    def forward(ctx, x, w, shard: ShardPlan, runtime: DistributedRuntime):
        transport, backend = runtime.transport, runtime.backend
        rows = x.contiguous().reshape(shard.owned, -1)
        F = rows.shape[1]
        w_flat = None if w is None else w.contiguous().reshape(-1)
        w_own = w_ghost = w_flat        # the sub-relations read it through their edge maps
        device = rows.device
        runtime.mark("forward:begin", device)
        if hasattr(backend, "begin_forward"):
            backend.begin_forward(shard)
        slot = window = None
        if runtime.push and rows.is_cuda and rows.dtype == torch.float32:
            window, _, _ = runtime.halo_windows(shard, F, device)
            slot = window.acquire()                     # None: every slot is still held by a forward
        if slot is not None:
            out, ghost_x = _push_forward(runtime, shard, window, slot, rows, w_own, w_ghost, F)
        else:
            ghost_x = torch.empty((int(shard.ghosts.numel()), F), dtype=rows.dtype, device=rows.device)
            packed = {p: backend.pack_rows(rows, ids) for p, ids in enumerate(shard.send_ids) if ids.numel()}
            in_flight = []
            for pairs, relation in shard.waves:             # every wave is one grouped exchange
                receives = [(source, ghost_x[o:o + c]) for source, _ in pairs
                            for o, c in (shard.recv_offsets[source],) if c]
                sends = [(target, packed[target]) for _, target in pairs if target in packed]
                in_flight.append((transport.exchange(sends=sends, receives=receives), relation))
            runtime.mark("forward pack + start exchange", device)
            out = backend.forward(shard.graph_own, rows, w_own)              # ... while owned-source edges reduce
            runtime.mark("forward owned-source part", device)
            for works, relation in in_flight:               # a wave's edges reduce while later waves are in flight
                transport.wait(works)
                runtime.mark("forward exposed halo wait", device)
                if relation.resolve_csr()[1].numel():
                    out = backend.forward(relation, ghost_x, w_ghost, accumulate_into=out)
                runtime.mark("forward ghost-source part", device)
        ctx.window, ctx.slot = window, slot
        if slot is not None and not (torch.is_grad_enabled() and (x.requires_grad or (w is not None and w.requires_grad))):
            window.release(slot, torch.cuda.current_stream(device))      # no backward will read the slot
            ctx.slot = None
        ctx.shard, ctx.runtime = shard, runtime
        ctx.x_shape, ctx.w_shape = x.shape, None if w is None else w.shape
        ctx.save_for_backward(rows, w_flat, ghost_x)
        ctx.halo_bytes = ghost_x.numel() * ghost_x.element_size()
        return out.reshape((shard.owned,) + tuple(x.shape[1:]))

    @staticmethod
    def backward(ctx, grad_output):
        rows, w_flat, ghost_x = ctx.saved_tensors
        w_own = w_ghost = w_flat
        shard, runtime = ctx.shard, ctx.runtime
        transport, backend = runtime.transport, runtime.backend
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dy = grad_output.contiguous().reshape(shard.owned, -1)
        F = dy.shape[1]
        dx = dw = None
        works, landed, pushed = [], [], None
        device = dy.device
        runtime.mark("backward:begin", device)
        if need_x:
            # ghost cotangents go back to their owners while everything else of the backward runs
            use_push = runtime.push and dy.is_cuda and dy.dtype == torch.float32
            # the pushed exchange is collective (its signals are all-reduces): every rank takes part,
            # also one without ghosts or requests
            if use_push or shard.edges_ghost.numel() or any(ids.numel() for ids in shard.send_ids):
                d_ghost = (backend.backward_dx(shard.graph_ghost, dy, w_ghost) if shard.ghosts.numel()
                           else dy.new_zeros((0, F)))
                if use_push:
                    landed, pushed = _push_cotangents(runtime, shard, d_ghost, F)
                else:
                    landed = [(p, ids, torch.empty((ids.numel(), F), dtype=dy.dtype, device=dy.device))
                              for p, ids in enumerate(shard.send_ids) if ids.numel()]
                    works = transport.exchange(
                        sends=[(p, d_ghost[o:o + c]) for p, (o, c) in enumerate(shard.recv_offsets)
                               if c and p != shard.rank],
                        receives=[(p, buffer) for p, _, buffer in landed])
            runtime.mark("backward ghost cotangents + start exchange", device)
            dx = backend.backward_dx(shard.graph_own, dy, w_own)
            runtime.mark("backward dx owned part", device)
        if need_w and ctx.w_shape is not None:
            dw = torch.empty(shard.num_local_edges, dtype=dy.dtype, device=dy.device)
            if shard.edges_own.numel():      # each part writes its own entries of dw through its edge map
                backend.backward_dw(shard.graph_own, dy, rows, dw)
            if shard.edges_ghost.numel():
                backend.backward_dw(shard.graph_ghost, dy, ghost_x, dw)
            dw = dw.reshape(ctx.w_shape)
            runtime.mark("backward dw", device)
        if need_x:
            if pushed is not None:
                torch.cuda.current_stream(device).wait_event(pushed[0])   # every peer's rows have landed
            else:
                transport.wait(works)
            runtime.mark("backward exposed cotangent wait", device)
            for _, ids, buffer in landed:            # fixed peer order: deterministic
                backend.add_rows(dx, ids, buffer)
            if pushed is not None:
                pushed[1].release(pushed[2], torch.cuda.current_stream(device))
            dx = dx.reshape(ctx.x_shape)
            runtime.mark("backward add received cotangents", device)
        if ctx.slot is not None:                     # the ghost rows of this call have been read for the last time
            ctx.window.release(ctx.slot, torch.cuda.current_stream(device))
            ctx.slot = None
        return dx, dw, None, None


def halo_weighted_sum(graph: Graph, x: torch.Tensor, w: torch.Tensor | None, runtime=None) -> torch.Tensor:
    runtime = runtime or current_distributed_runtime()
    if runtime is None:
        raise RuntimeError("a Graph.halo() snapshot needs an active DistributedRuntime")
    shard = shard_plan_for(graph, runtime)
    if x.shape[0] != shard.owned:
        raise ValueError(f"src field leading dimension must be the {shard.owned} rows this rank owns, "
                         f"got {tuple(x.shape)}")
    if w is not None and w.numel() != shard.num_local_edges:
        raise ValueError(f"edge field must have one value per local edge ({shard.num_local_edges})")
    return _HaloWeightedSum.apply(x, w, shard, runtime)


def specialise_sharded_message_passing(kernel, *, graph, src, dst, edge, params):
    """Stage a MessagePassing kernel for a ``Graph.halo()`` snapshot: returns
    (bindings, tensors, constants, runner) for the dispatcher's guarded warm path.  ``runner``
    executes the sharded call under whichever DistributedRuntime is active when it is invoked:
    every rank passes the fields of the rows it owns and gets its rows of the aggregate
    (execute_sharded_message_passing, python/tiga/distributed/transport.py:898-1403 of the
    reference)."""
    if not isinstance(kernel.reducer, SumReducer) or kernel.reducer.identity() != 0:
        raise NotImplementedError("sharded execution is implemented for the sum reducer")
    pattern = cap.recognize_weighted_sum(cap.capture_edge(kernel.edge, params))
    if pattern is None:
        raise NotImplementedError("sharded execution needs an `edge.w * src.x` or `src.x` message")
    bindings, tensors = [("src", pattern.src_field)], [src[pattern.src_field]]
    if pattern.edge_field is not None:
        bindings.append(("edge", pattern.edge_field))
        tensors.append(edge[pattern.edge_field])
    constants = {name: value for name, value in cap.selected_params(kernel.edge, params).items()
                 if not isinstance(value, torch.Tensor)}

    def runner(x, w=None):
        return halo_weighted_sum(graph, x, w, current_distributed_runtime())

    kernel._record(graph, "b200-halo-csr-weighted-sum", ("partition-by-destination", "derive-halo",
                                                          "split-owned-ghost-edges", "overlap-exchange"),
                   ("halo rows land in their slice of the ghost buffer; owned-source edges reduce while the "
                    "exchange is in flight",))
    return bindings, tensors, constants, runner


def execute_sharded_message_passing(kernel, *, graph, src, dst, edge, params):
    """One sharded call (aggregate plus the kernel's ``node`` epilogue)."""
    if current_distributed_runtime() is None:
        raise RuntimeError("a Graph.halo() snapshot needs an active DistributedRuntime")
    _, tensors, _, runner = specialise_sharded_message_passing(kernel, graph=graph, src=src, dst=dst, edge=edge,
                                                               params=params)
    aggregate = runner(*tensors)
    from types import SimpleNamespace

    from ..message_passing import MessagePassing

    if type(kernel).node is MessagePassing.node:
        return aggregate
    return cap.call_region(kernel.node, (SimpleNamespace(**dst), aggregate), params)


__all__ = ["DistributedRuntime", "NCCLTransport", "NativeBackend", "ProcessGroupTransport", "ShardPlan",
           "build_shard_plan", "current_distributed_runtime", "execute_sharded_message_passing",
           "halo_weighted_sum", "shard_plan_for", "specialise_sharded_message_passing"]
