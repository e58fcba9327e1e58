"""Rebuildable geometric relations behind ``Graph.radius`` and ``Graph.knn``.

Behaviour follows the Torch twin of the reference's Graph
(python/tiga/interop/torch/graph.py of walkerchi/TIGA-lang: constructors :391-534, ``resolve_csr``
:851-1003, cell-list candidates :1023-1125, pair selection :1127-1176, pairwise cutoff :1178-1194,
minimum image :1203-1210, implicit edge fields :1403-1444, ``explain`` :1444-1478):

* a relation is *dynamic*: positions may be changed in place between calls, and the CSR is rebuilt
  whenever the physical snapshot (storage address + tensor version of positions, cutoff, lattice and
  builder fields) differs from the one the cached CSR was built from;
* edge order is destination-major; inside a row the cell list yields the 3^D neighbour cells in
  meshgrid order (first axis slowest) with the points of a cell in ascending index, the all-pairs
  path yields sources in ascending index; kNN rows are ascending by (distance, source index);
* ``metric`` replaces the Euclidean distance (all-pairs only), ``select`` is an additional boolean
  filter, the cutoff may be a scalar, one value per destination or a full [N, N] matrix.

float32 CUDA positions with the default metric, a scalar cutoff and 1-3 dimensions build on the
device with the kernels of ``geometry``; every other combination (CPU tensors, float64, callables that
must see all pairs) is evaluated with Torch tensor operations, as the reference itself does.
"""
from __future__ import annotations

import itertools
from types import SimpleNamespace
from typing import Callable, Mapping

import torch

from . import geometry


def _version(tensor: torch.Tensor) -> int:
    return int(tensor._version)


def _pair_values(name: str, value, pairs: int, device, dtype=None) -> torch.Tensor:
    """One value per candidate pair from a metric / select callable."""
    if not isinstance(value, torch.Tensor):
        raise TypeError(f"{name} must return a torch.Tensor")
    if value.device != device:
        raise ValueError(f"{name} returned a tensor on {value.device}, expected {device}")
    if value.ndim == 2 and value.shape[1] == 1:
        value = value[:, 0]
    if value.ndim != 1 or value.shape[0] != pairs:
        raise ValueError(f"{name} must return one value per candidate pair ({pairs}), got {tuple(value.shape)}")
    if dtype is not None and value.is_floating_point() and value.dtype != dtype:
        value = value.to(dtype)
    return value


class GeometricRelation:
    """Positions, search parameters and the caches of one dynamic relation."""

    def __init__(self, kind: str, positions: torch.Tensor, *, cutoff=None, k: int | None = None,
                 source_positions: torch.Tensor | None = None, periodic: torch.Tensor | None = None,
                 exclude_self: bool = True, fields: Mapping[str, torch.Tensor] | None = None,
                 metric: Callable | None = None, select: Callable | None = None):
        self.kind = kind                       # "radius" | "knn"
        self.positions = positions
        self.source_positions = source_positions
        self.cutoff = cutoff
        self.k = k
        self.periodic = periodic
        self.exclude_self = exclude_self
        self.fields = dict(fields or {})
        self.metric = metric
        self.select = select
        self.builder = "unresolved"
        self.build_info: dict | None = None
        self._csr = None            # (key, row_ptr, col, info, distance | None, displacement | None)
        self._directory = None      # (key, CellDirectory)
        self._knn_row_ptr = None

    # ------------------------------------------------------------------ identity of a snapshot
    def snapshot_key(self):
        cutoff = self.cutoff
        cutoff_key = ((cutoff.data_ptr(), _version(cutoff)) if isinstance(cutoff, torch.Tensor)
                      else (None if cutoff is None else float(cutoff)))
        periodic_key = None if self.periodic is None else (self.periodic.data_ptr(), _version(self.periodic))
        sources = self.source_positions
        return (self.positions.data_ptr(), _version(self.positions),
                None if sources is None else (sources.data_ptr(), _version(sources)),
                cutoff_key, periodic_key, self.k, self.exclude_self,
                tuple((name, value.data_ptr(), _version(value)) for name, value in sorted(self.fields.items())),
                None if self.metric is None else id(self.metric),
                None if self.select is None else id(self.select))

    def signature(self):
        """What a specialised launch depends on besides the tensors it is handed: a new Graph over a
        new snapshot with the same signature reuses the launch."""
        cutoff = self.cutoff
        # the cutoff VALUE is a runtime scalar (the runner reads it from the graph of the call); only
        # what selects the code path is part of the signature
        return (self.kind, tuple(self.positions.shape[1:]), self.positions.dtype, self.positions.device,
                None if cutoff is None else (isinstance(cutoff, torch.Tensor), self.scalar_cutoff() is not None),
                self.k, self.exclude_self, self.source_positions is None,
                None if self.periodic is None else tuple(self.periodic.shape),
                self.metric is None, self.select is None, tuple(sorted(self.fields)))

    # ------------------------------------------------------------------ helpers
    def scalar_cutoff(self) -> float | None:
        """The cell size when the Euclidean cell list applies (scalar positive cutoff, default
        metric, one to three dimensions), else None."""
        if self.metric is not None or self.positions.shape[1] not in (1, 2, 3):
            return None
        cutoff = self.cutoff
        if isinstance(cutoff, torch.Tensor):
            if cutoff.numel() != 1:
                return None
            value = float(cutoff.detach().item())
        else:
            value = float(cutoff)
        return value if value > 0.0 else None

    def _lattice(self) -> torch.Tensor:
        return geometry.periodic_lattice(self.periodic)

    def minimum_image(self, displacement: torch.Tensor) -> torch.Tensor:
        if self.periodic is None:
            return displacement
        lattice = self._lattice()
        fractional = displacement @ torch.linalg.inv(lattice)
        fractional = fractional - torch.round(fractional)
        return fractional @ lattice

    def native_cells(self) -> bool:
        p = self.positions
        return (self.kind == "radius" and p.is_cuda and p.dtype == torch.float32
                and self.scalar_cutoff() is not None
                and (self.periodic is None or self.periodic.dtype == torch.float32))

    def fusable(self) -> bool:
        """The fused consumer needs the symmetric relation of a plain scalar-cutoff search."""
        return self.native_cells() and self.select is None and not self.fields

    # ------------------------------------------------------------------ directory (device)
    def directory(self) -> geometry.CellDirectory:
        key = self.snapshot_key()
        if self._directory is None or self._directory[0] != key:
            space = geometry.make_cell_space(self.positions.shape[1], self.scalar_cutoff(), self.periodic)
            self._directory = (key, geometry.CellDirectory(self.positions, space))
            self.builder = "b200_hash_cell_list"
        return self._directory[1]

    # ------------------------------------------------------------------ CSR
    def resolve(self, num_dst: int):
        key = self.snapshot_key()
        if self._csr is not None and self._csr[0] == key:
            self.build_info = {**self._csr[3], "cache_hit": True}
            self.builder = str(self._csr[3]["builder"])
            return self._csr[1], self._csr[2], False
        if self.kind == "knn":
            row_ptr, col, info, distance, displacement = self._resolve_knn()
        elif self.native_cells():
            row_ptr, col, info, distance, displacement = self._resolve_radius_native()
        else:
            row_ptr, col, info, distance, displacement = self._resolve_radius_torch(num_dst)
        self.builder = str(info["builder"])
        self.build_info = dict(info)
        self._csr = (key, row_ptr, col, dict(info), distance, displacement)
        return row_ptr, col, True

    def _resolve_knn(self):
        queries = self.positions
        candidates = queries if self.source_positions is None else self.source_positions
        k = int(self.k)
        if queries.is_cuda and queries.dtype == torch.float32 and queries.shape[1] <= 64 and k <= 128:
            col, builder = geometry.knn_indices(queries, candidates, k, self.exclude_self,
                                                self_search=self.source_positions is None)
        else:
            distances = torch.cdist(queries.detach(), candidates.detach(),
                                    compute_mode="donot_use_mm_for_euclid_dist")
            if self.exclude_self:
                distances.fill_diagonal_(float("inf"))
            col = torch.argsort(distances, dim=1, stable=True)[:, :k].reshape(-1).to(torch.int64)
            builder = "torch-cdist-stable-argsort"
        if self._knn_row_ptr is None or self._knn_row_ptr.numel() != queries.shape[0] + 1:
            self._knn_row_ptr = torch.arange(0, col.numel() + 1, k, device=queries.device, dtype=torch.int64)
        info = {"builder": builder, "candidate_pairs": queries.shape[0] * candidates.shape[0],
                "accepted_edges": int(col.numel()), "materialized": True, "cache_hit": False}
        return self._knn_row_ptr, col, info, None, None

    def _resolve_radius_native(self):
        directory = self.directory()
        cutoff = self.scalar_cutoff()
        row_ptr, col, distance, displacement, pairs = directory.radius_csr(
            cutoff, self.exclude_self, with_fields=True)
        if self.select is not None:
            destination = torch.repeat_interleave(
                torch.arange(row_ptr.numel() - 1, device=row_ptr.device), row_ptr.diff())
            keep = self._selected(destination, col, displacement, distance,
                                  torch.full_like(distance, cutoff))
            destination, col = destination[keep], col[keep]
            distance, displacement = distance[keep], displacement[keep]
            row_ptr = _row_ptr_of(destination, row_ptr.numel() - 1)
        info = {"builder": "b200_hash_cell_list", "candidate_pairs": pairs, "accepted_edges": int(col.numel()),
                "materialized": True, "cache_hit": False}
        return row_ptr, col, info, distance, displacement

    def _selected(self, destination, source, displacement, distance, cutoff):
        src_view, dst_view = self._endpoint_views(source, destination)
        selected = _pair_values(
            "select", self.select(src_view, dst_view,
                                  SimpleNamespace(displacement=displacement, distance=distance, cutoff=cutoff)),
            int(source.numel()), self.positions.device)
        if selected.dtype is not torch.bool:
            raise TypeError("select must return a boolean tensor")
        return selected

    def _endpoint_views(self, source, destination):
        p = self.positions
        src_view = SimpleNamespace(position=p[source], **{n: v[source] for n, v in self.fields.items()})
        dst_view = SimpleNamespace(position=p[destination], **{n: v[destination] for n, v in self.fields.items()})
        return src_view, dst_view

    def _pair_cutoff(self, destination, source, num_dst):
        cutoff, p = self.cutoff, self.positions
        if not isinstance(cutoff, torch.Tensor):
            return torch.full((source.numel(),), float(cutoff), device=p.device, dtype=p.dtype)
        if cutoff.device != p.device:
            raise ValueError(f"cutoff is on {cutoff.device}, expected {p.device}")
        if cutoff.ndim == 0 or cutoff.numel() == 1:
            return cutoff.reshape(()).expand(source.numel())
        if cutoff.shape == (num_dst,):
            return cutoff[destination]
        if cutoff.shape == (num_dst, num_dst):
            return cutoff[destination, source]
        raise ValueError("cutoff must be scalar, per-destination [N], or pairwise [N, N]; "
                         f"got {tuple(cutoff.shape)}")

    def _resolve_radius_torch(self, num_dst: int):
        p = self.positions.detach()
        count = p.shape[0]
        cell = self.scalar_cutoff()
        if cell is None:
            index = torch.arange(count, device=p.device)
            destination, source = index.repeat_interleave(count), index.repeat(count)
            builder = "all_pairs"
        else:
            destination, source = self._cell_candidates(p, cell)
            builder = "uniform_cell_list"
        candidates = int(source.numel())
        src_view, dst_view = self._endpoint_views(source, destination)
        displacement = self.minimum_image(src_view.position - dst_view.position)
        if self.metric is None:
            distance = torch.linalg.vector_norm(displacement, dim=-1)
        else:
            distance = _pair_values("metric",
                                    self.metric(src_view, dst_view, SimpleNamespace(displacement=displacement)),
                                    candidates, p.device, p.dtype)
            if not distance.is_floating_point():
                raise TypeError("metric must return a floating-point tensor")
        cutoff = self._pair_cutoff(destination, source, num_dst)
        keep = distance <= cutoff
        if self.select is not None:
            selected = _pair_values(
                "select", self.select(src_view, dst_view, SimpleNamespace(
                    displacement=displacement, distance=distance, cutoff=cutoff)), candidates, p.device)
            if selected.dtype is not torch.bool:
                raise TypeError("select must return a boolean tensor")
            keep = keep & selected
        if self.exclude_self:
            keep = keep & (source != destination)
        destination, source = destination[keep], source[keep]
        info = {"builder": builder, "candidate_pairs": candidates, "accepted_edges": int(source.numel()),
                "materialized": True, "cache_hit": False}
        return _row_ptr_of(destination, num_dst), source.to(torch.int64), info, None, None

    def _cell_candidates(self, p: torch.Tensor, cell: float):
        """(destination, source) of every pair of points in adjacent cells, destination-major, the
        neighbour cells of a destination in meshgrid order and the members of a cell in ascending
        index.  One pass per neighbour offset (at most 27): the pairs of an offset come out grouped by
        destination, and a stable sort of the concatenation by destination restores the row order."""
        count, dims = p.shape
        device = p.device
        empty = torch.empty(0, device=device, dtype=torch.int64)
        if count == 0:
            return empty, empty
        if self.periodic is not None:
            inverse = torch.linalg.inv(self._lattice())
            fractional = p @ inverse
            fractional = fractional - torch.floor(fractional)
            extents = geometry.periodic_extents(inverse, cell).to(device)
            cells = torch.minimum(torch.floor(fractional * extents).to(torch.int64), extents - 1)
            lower = torch.zeros_like(extents)
            axes = [(0,) if e == 1 else ((0, 1) if e == 2 else (-1, 0, 1)) for e in extents.tolist()]
        else:
            cells = torch.floor(p / cell).to(torch.int64)
            lower, upper = cells.amin(dim=0), cells.amax(dim=0)
            extents = upper - lower + 1
            axes = [(-1, 0, 1)] * dims
        strides = torch.ones(dims, device=device, dtype=torch.int64)
        if dims > 1:
            strides[1:] = torch.cumprod(extents[:-1], dim=0)
        keys = ((cells - lower) * strides).sum(dim=-1)
        sorted_keys, order = torch.sort(keys, stable=True)
        occupied, occupancy = torch.unique_consecutive(sorted_keys, return_counts=True)
        first = torch.cumsum(occupancy, dim=0) - occupancy
        everyone = torch.arange(count, device=device)
        destinations, sources = [], []
        for offset in itertools.product(*axes):
            neighbour = cells + torch.tensor(offset, device=device, dtype=torch.int64)
            if self.periodic is not None:
                neighbour = torch.remainder(neighbour, extents)
                inside = torch.ones(count, dtype=torch.bool, device=device)
            else:
                inside = ((neighbour >= lower) & (neighbour <= upper)).all(dim=-1)
            wanted = ((neighbour - lower) * strides).sum(dim=-1)
            slot = torch.searchsorted(occupied, wanted).clamp_max(occupied.numel() - 1)
            found = inside & (occupied[slot] == wanted)
            members = torch.where(found, occupancy[slot], torch.zeros_like(slot))
            owner = torch.repeat_interleave(everyone, members)
            if owner.numel() == 0:
                continue
            start = torch.cumsum(members, dim=0) - members
            within = torch.arange(owner.numel(), device=device) - start[owner]
            destinations.append(owner)
            sources.append(order[first[slot[owner]] + within])
        if not destinations:
            return empty, empty
        destination, source = torch.cat(destinations), torch.cat(sources)
        by_row = torch.sort(destination, stable=True).indices
        return destination[by_row], source[by_row]

    # ------------------------------------------------------------------ implicit edge fields
    def edge_fields(self, row_ptr: torch.Tensor, col: torch.Tensor, destination: torch.Tensor):
        p = self.positions
        sources = p if self.source_positions is None else self.source_positions
        cached = self._csr
        if (self.metric is None and cached is not None and cached[1] is row_ptr and cached[4] is not None
                and cached[0] == self.snapshot_key() and not p.requires_grad):
            return {"displacement": cached[5], "distance": cached[4]}
        native = (p.is_cuda and p.dtype == torch.float32 and self.metric is None
                  and not (p.requires_grad or sources.requires_grad)
                  and p.shape[1] <= (3 if self.periodic is not None else 8)
                  and (self.periodic is None or self.periodic.dtype == torch.float32))
        if native:
            space = geometry.make_cell_space(p.shape[1], 1.0, self.periodic)
            displacement, distance = geometry.edge_geometry(p, sources, space, row_ptr, col)
            return {"displacement": displacement, "distance": distance}
        displacement = self.minimum_image(sources[col] - p[destination])
        if self.metric is None:
            distance = torch.linalg.vector_norm(displacement, dim=-1)
        else:
            src_view = SimpleNamespace(position=sources[col], **{n: v[col] for n, v in self.fields.items()})
            dst_view = SimpleNamespace(position=p[destination],
                                       **{n: v[destination] for n, v in self.fields.items()})
            distance = _pair_values("metric",
                                    self.metric(src_view, dst_view, SimpleNamespace(displacement=displacement)),
                                    int(col.numel()), p.device, p.dtype)
        return {"displacement": displacement, "distance": distance}

    # ------------------------------------------------------------------ reporting
    def describe(self) -> str:
        if self.kind == "knn":
            search = "self" if self.source_positions is None else "bipartite"
            text = f", k={self.k}, search={search}, metric=euclidean, builder={self.builder}"
        else:
            broad = "euclidean-cell-list-eligible" if self.metric is None else "all-pairs-only"
            text = (f", metric={'custom' if self.metric else 'euclidean'}, "
                    f"select={'custom' if self.select else 'cutoff-only'}, "
                    f"periodic={'none' if self.periodic is None else tuple(self.periodic.shape)}, "
                    f"broad_phase={broad}, builder={self.builder}")
        if self.build_info is not None:
            text += (f", candidates={self.build_info['candidate_pairs']:,}, "
                     f"accepted={self.build_info['accepted_edges']:,}")
        return text


def _row_ptr_of(destination: torch.Tensor, num_dst: int) -> torch.Tensor:
    counts = torch.bincount(destination, minlength=num_dst)
    row_ptr = torch.zeros(num_dst + 1, device=destination.device, dtype=torch.int64)
    torch.cumsum(counts, dim=0, out=row_ptr[1:])
    return row_ptr


# ---------------------------------------------------------------------- argument checks
def check_radius_arguments(positions, cutoff, fields, metric, select, periodic):
    """Validation of ``Graph.radius`` (graph.py:414-457 of the reference); returns the lattice tensor."""
    if not isinstance(positions, torch.Tensor) or positions.ndim != 2:
        raise ValueError("positions must have shape [particles, dimensions]")
    if not positions.is_floating_point():
        raise TypeError("positions must use a floating-point dtype")
    if metric is not None and not callable(metric):
        raise TypeError("metric must be callable")
    if select is not None and not callable(select):
        raise TypeError("select must be callable")
    count, dims = positions.shape
    if periodic is not None:
        if not isinstance(periodic, torch.Tensor):
            periodic = torch.as_tensor(periodic, dtype=positions.dtype, device=positions.device)
        if tuple(periodic.shape) not in {(dims,), (dims, dims)}:
            raise ValueError("periodic must contain box lengths [D] or lattice vectors [D,D]")
        if periodic.dtype != positions.dtype or periodic.device != positions.device:
            raise ValueError("periodic must share the positions dtype and device")
        if not bool(torch.isfinite(periodic).all().item()):
            raise ValueError("periodic lattice must be finite")
        determinant = torch.linalg.det(geometry.periodic_lattice(periodic))
        if not bool(torch.isfinite(determinant).item()) or determinant.abs().item() == 0:
            raise ValueError("periodic lattice must be nonsingular")
    fields = dict(fields or {})
    if "position" in fields:
        raise ValueError("fields cannot redefine the reserved 'position' field")
    for name, value in fields.items():
        if not isinstance(value, torch.Tensor):
            raise TypeError(f"fields[{name!r}] must be a torch.Tensor")
        if value.ndim == 0 or value.shape[0] != count:
            raise ValueError(f"fields[{name!r}] leading dimension must be {count}, got {tuple(value.shape)}")
        if value.device != positions.device:
            raise ValueError(f"fields[{name!r}] is on {value.device}, expected {positions.device}")
    return periodic, fields


def check_knn_arguments(positions, k, candidates, exclude_self):
    """Validation of ``Graph.knn`` (graph.py:487-515 of the reference); returns (sources, exclude_self)."""
    if not isinstance(positions, torch.Tensor):
        raise TypeError("positions must be a torch.Tensor")
    if positions.ndim != 2 or not positions.dtype.is_floating_point:
        raise TypeError("positions must be a rank-two floating Tensor")
    self_search = candidates is None
    sources = positions if self_search else candidates
    if not isinstance(sources, torch.Tensor):
        raise TypeError("candidates must be a torch.Tensor")
    if sources.ndim != 2 or not sources.dtype.is_floating_point:
        raise TypeError("candidates must be a rank-two floating Tensor")
    if sources.shape[1] != positions.shape[1]:
        raise ValueError("positions and candidates must share feature width")
    if sources.dtype != positions.dtype:
        raise TypeError("positions and candidates must share dtype")
    if sources.device != positions.device:
        raise ValueError("positions and candidates must share device")
    if exclude_self is None:
        exclude_self = self_search
    if not isinstance(exclude_self, bool):
        raise TypeError("exclude_self must be bool or None")
    if exclude_self and not self_search:
        raise ValueError("exclude_self is only defined for self-kNN; omit candidates")
    maximum = sources.shape[0] - 1 if exclude_self else sources.shape[0]
    if not isinstance(k, int) or k <= 0 or k > maximum:
        raise ValueError(f"k must be in [1, {maximum}] for {sources.shape[0]} candidates")
    return (None if self_search else sources), exclude_self


__all__ = ["GeometricRelation", "check_knn_arguments", "check_radius_arguments"]
