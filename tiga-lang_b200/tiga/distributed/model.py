"""Destination partitioning and halo maps.

Same public objects as python/tiga/distributed/model.py:8-194 of the reference
(``DeviceMesh``, ``ByDestination``, ``GraphPlacement``, ``HaloMap``,
``destination_owner``, ``owned_range``, ``derive_halo_map``) with identical
results; the halo derivation here is vectorised over torch tensors so that it
also runs on the device for graphs with billions of edges, where the
reference walks Python lists.

Partition rule (model.py:124-130): with ``base, extra = divmod(N, W)`` rank r
owns ``[r*base + min(r, extra), ... + base + (r < extra))``.  ``ByDestination
(balance="edges")`` is honoured here as contiguous ranges that balance the
edge count instead of the row count (the reference declares the option,
model.py:55-65, but its ``owned_range`` ignores it); ``"entities"`` and
``"auto"`` keep the reference's rule.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Sequence


class DeviceMesh:
    """Declarative device mesh; it never initialises a process group."""

    __slots__ = ("device_type", "shape", "names")

    def __init__(self, device_type: str, shape, *, names: tuple[str, ...] = ()) -> None:
        extents = (shape,) if isinstance(shape, int) else tuple(shape)
        if not device_type:
            raise ValueError("device_type must be non-empty")
        if not extents or any(not isinstance(e, int) or e <= 0 for e in extents):
            raise ValueError("mesh shape must contain positive integers")
        if names and len(names) != len(extents):
            raise ValueError("mesh names must match the mesh rank")
        if len(set(names)) != len(names):
            raise ValueError("mesh names must be unique")
        object.__setattr__(self, "device_type", device_type)
        object.__setattr__(self, "shape", extents)
        object.__setattr__(self, "names", tuple(names))

    def __setattr__(self, name, value):
        raise AttributeError("DeviceMesh is immutable")

    def __eq__(self, other):
        return isinstance(other, DeviceMesh) and self.specialization_key() == other.specialization_key()

    def __hash__(self):
        return hash(self.specialization_key())

    def __repr__(self):
        return f"DeviceMesh({self.device_type!r}, {self.shape!r}, names={self.names!r})"

    @property
    def size(self) -> int:
        return math.prod(self.shape)

    def specialization_key(self) -> tuple[object, ...]:
        return self.device_type, self.shape, self.names


@dataclass(frozen=True)
class ByDestination:
    mesh_axis: int | str = 0
    balance: str = "auto"

    def __post_init__(self) -> None:
        if not isinstance(self.mesh_axis, (int, str)):
            raise TypeError("mesh_axis must be an integer or a named mesh axis")
        if self.balance not in {"edges", "entities", "auto", "cost"}:
            raise ValueError("balance must be 'edges', 'entities', 'auto' or 'cost'")

    def specialization_key(self) -> tuple[object, ...]:
        return "by_destination", self.mesh_axis, self.balance


@dataclass(frozen=True)
class GraphPlacement:
    mesh: DeviceMesh
    partition: ByDestination
    halo_depth: object

    def __post_init__(self) -> None:
        depth = self.halo_depth
        if depth != "auto" and (not isinstance(depth, int) or depth < 0):
            raise ValueError("halo depth must be a non-negative integer or 'auto'")
        axis = self.partition.mesh_axis
        rank = len(self.mesh.shape)
        if isinstance(axis, int) and not -rank <= axis < rank:
            raise ValueError("partition mesh_axis is outside the device mesh rank")
        if isinstance(axis, str) and axis not in self.mesh.names:
            raise ValueError(f"unknown named mesh axis {axis!r}")

    def specialization_key(self) -> tuple[object, ...]:
        return (*self.mesh.specialization_key(), *self.partition.specialization_key(), self.halo_depth)


@dataclass(frozen=True)
class HaloMap:
    rank: int
    world_size: int
    owned_begin: int
    owned_end: int
    ghost_ids: tuple[int, ...]
    receive_from: tuple[tuple[int, tuple[int, ...]], ...]
    send_to: tuple[tuple[int, tuple[int, ...]], ...] = field(default=())

    @property
    def owned_entities(self) -> int:
        return self.owned_end - self.owned_begin

    @property
    def ghost_entities(self) -> int:
        return len(self.ghost_ids)

    def bytes_for(self, itemsize: int, trailing_elements: int = 1) -> int:
        if itemsize <= 0 or trailing_elements <= 0:
            raise ValueError("itemsize and trailing_elements must be positive")
        return self.ghost_entities * itemsize * trailing_elements


def owned_range(entities: int, world_size: int, rank: int) -> tuple[int, int]:
    if entities < 0 or world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError("invalid destination partition")
    base, extra = divmod(entities, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def destination_owner(entity: int, entities: int, world_size: int) -> int:
    if not 0 <= entity < entities or world_size <= 0:
        raise ValueError("entity/world_size is outside the partition domain")
    base, extra = divmod(entities, world_size)
    boundary = (base + 1) * extra  # the first `extra` ranks own one more row
    if entity < boundary:
        return entity // (base + 1)
    return extra + (entity - boundary) // base if base else extra


import os

# balance="cost": one destination row weighs as much as this many edges.  Measured on 4 B200s with the
# GCN layer (R-MAT, 2^20 nodes per GPU), ms per step for 8 / 16 / 24 / 32 / 64: 22.6 / 21.2 / 20.2 /
# 19.0 / 21.2 -- a row costs its pointer reads, two output-row passes (owned and ghost part), its
# share of the dense linear and of the halo traffic.
ROW_COST_IN_EDGES = int(os.environ.get("TIGA_B200_ROW_COST", "32"))


def partition_bounds(entities: int, world_size: int, *, row_ptr=None, balance: str = "auto"):
    """Begin offsets of every rank plus the end: ``bounds[r]..bounds[r+1]``.

    ``balance='edges'`` needs ``row_ptr`` (a torch tensor) and places the cut
    for rank r at the first row whose prefix edge count reaches r*E/W.
    ``balance='cost'`` (an addition of this package) balances edges plus
    ROW_COST_IN_EDGES per row: a destination row costs a pointer read, an
    output row and its share of the node epilogue whatever its degree, which on
    power-law graphs is what an edge-only balance gets wrong."""
    if balance in ("edges", "cost") and row_ptr is not None and entities > 0:
        import torch

        prefix = row_ptr[:-1].to(torch.int64)
        total = int(row_ptr[-1].item())
        if balance == "cost":
            prefix = prefix + ROW_COST_IN_EDGES * torch.arange(entities, device=row_ptr.device, dtype=torch.int64)
            total += ROW_COST_IN_EDGES * entities
        targets = torch.tensor([(total * r) // world_size for r in range(1, world_size)],
                               dtype=torch.int64, device=row_ptr.device)
        cuts = torch.searchsorted(prefix.contiguous(), targets, right=False).tolist()
        bounds = [0]
        for cut in cuts:
            bounds.append(min(max(int(cut), bounds[-1]), entities))
        bounds.append(entities)
        return bounds
    return [owned_range(entities, world_size, r)[0] for r in range(world_size)] + [entities]


def derive_halo_map(row_ptr: Sequence[int], col_idx: Sequence[int], *, num_entities: int, world_size: int,
                    rank: int, peer_requests: Sequence[Sequence[int]] | None = None) -> HaloMap:
    """Exact ghosts of one rank's owned rows (sorted unique remote sources),
    grouped by owner; ``peer_requests[p]`` (ids this rank owns that peer p
    asked for) fills ``send_to``."""
    import torch

    rows = row_ptr.to(torch.int64) if isinstance(row_ptr, torch.Tensor) else torch.as_tensor(row_ptr, dtype=torch.int64)
    cols = col_idx.to(torch.int64) if isinstance(col_idx, torch.Tensor) else torch.as_tensor(col_idx, dtype=torch.int64)
    if rows.numel() != num_entities + 1 or int(rows[0]) != 0 or int(rows[-1]) != cols.numel():
        raise ValueError("row_ptr does not describe num_entities CSR rows")
    if bool((rows[1:] < rows[:-1]).any()):
        raise ValueError("row_ptr must be monotonic")
    if cols.numel() and (int(cols.min()) < 0 or int(cols.max()) >= num_entities):
        raise ValueError("col_idx contains an out-of-range entity")
    begin, end = owned_range(num_entities, world_size, rank)
    mine = cols[int(rows[begin]):int(rows[end])]
    ghosts = torch.unique(mine[(mine < begin) | (mine >= end)], sorted=True)
    bounds = torch.tensor(partition_bounds(num_entities, world_size), dtype=torch.int64, device=ghosts.device)
    owner = torch.searchsorted(bounds, ghosts, right=True) - 1
    receives = []
    for peer in range(world_size):
        ids = ghosts[owner == peer]
        if ids.numel():
            receives.append((peer, tuple(ids.tolist())))
    sends = []
    if peer_requests is not None:
        if len(peer_requests) != world_size:
            raise ValueError("peer_requests must contain one entry per rank")
        for peer, requested in enumerate(peer_requests):
            unique = tuple(sorted({int(v) for v in requested}))
            if any(not begin <= v < end for v in unique):
                raise ValueError("peer requested an entity not owned by this rank")
            if unique:
                sends.append((peer, unique))
    return HaloMap(rank=rank, world_size=world_size, owned_begin=begin, owned_end=end,
                   ghost_ids=tuple(ghosts.tolist()), receive_from=tuple(receives), send_to=tuple(sends))


__all__ = ["ByDestination", "DeviceMesh", "GraphPlacement", "HaloMap", "derive_halo_map",
           "destination_owner", "owned_range", "partition_bounds"]
