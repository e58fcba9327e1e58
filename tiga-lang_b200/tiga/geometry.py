"""Device builders of the dynamic relations (``Graph.radius`` / ``Graph.knn``) and the fused radius
consumer, over the C ABI of the CUDA library.

What the reference evaluates with Torch tensor programs
(python/tiga/interop/torch/graph.py:851-1003 ``resolve_csr``, :1023-1125 cell-list candidates,
:1127-1176 pair selection, :1403-1444 implicit edge fields of walkerchi/TIGA-lang) and, for the default
Euclidean radius, with a hash-grid directory plus a generated kernel
(python/tiga/interop/torch/radius_grid.py, lowering ``gf-kernel-to-ttir-generated-radius-distance-sum``)
runs here as hand-written kernels: a stable bucket sort of the points, a count / scan / fill pass in
the reference's edge order, an exact brute-force k-nearest search, and a fused walk that folds
``weight(i, j) * x[j]`` without writing the relation.  Everything in this module needs CUDA tensors;
the Torch restatement used for CPU tensors lives with the Graph class.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _native

PAIR_WEIGHT_ONE, PAIR_WEIGHT_DISTANCE = 0, 1


class CellSpaceStruct(ctypes.Structure):
    """``tgb_cell_space`` of include/tiga_b200.h."""

    _fields_ = [("dims", ctypes.c_int32), ("periodic", ctypes.c_int32), ("cell_size", ctypes.c_float),
                ("lattice", ctypes.c_float * 9), ("inverse", ctypes.c_float * 9), ("extents", ctypes.c_int32 * 3)]


@dataclass
class CellSpace:
    """Broad-phase geometry: cell edge, optional periodic lattice with its inverse and cells per axis."""

    dims: int
    cell_size: float
    lattice: torch.Tensor | None     # [D, D] on the CPU, float32
    inverse: torch.Tensor | None
    extents: tuple[int, ...] | None
    struct: CellSpaceStruct

    @property
    def periodic(self) -> bool:
        return self.lattice is not None


def periodic_lattice(periodic: torch.Tensor) -> torch.Tensor:
    return torch.diag(periodic) if periodic.ndim == 1 else periodic


def periodic_extents(inverse: torch.Tensor, cell_size: float) -> torch.Tensor:
    """Cells per periodic axis: a bin at least ``cutoff * ||inverse[:, a]||`` wide in fractional
    coordinates keeps one wrapped neighbour step a safe broad phase, skew lattices included
    (graph.py:1044-1054 of the reference)."""
    bound = cell_size * torch.linalg.vector_norm(inverse, dim=0)
    return torch.floor(1.0 / bound.clamp_min(1.0e-12)).clamp(min=1).to(torch.int64)


def make_cell_space(dims: int, cell_size: float, periodic: torch.Tensor | None) -> CellSpace:
    struct = CellSpaceStruct()
    struct.dims = int(dims)
    struct.cell_size = float(cell_size)
    lattice = inverse = extents = None
    if periodic is not None:
        lattice = periodic_lattice(periodic.detach()).to("cpu", torch.float32).contiguous()
        inverse = torch.linalg.inv(lattice).contiguous()
        extents = tuple(int(v) for v in periodic_extents(inverse, float(cell_size)).tolist())
        struct.periodic = 1
        for i, value in enumerate(lattice.reshape(-1).tolist()):
            struct.lattice[i] = value
        for i, value in enumerate(inverse.reshape(-1).tolist()):
            struct.inverse[i] = value
        for i, value in enumerate(extents):
            struct.extents[i] = value
    return CellSpace(int(dims), float(cell_size), lattice, inverse, extents, struct)


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _check_positions(positions: torch.Tensor) -> torch.Tensor:
    if not positions.is_cuda:
        raise RuntimeError("the native geometry builders need CUDA tensors")
    if positions.dtype != torch.float32:
        raise NotImplementedError(f"the native geometry builders take float32 positions, got {positions.dtype}")
    return positions.detach().contiguous()


class CellDirectory:
    """Points sorted into the modular hash buckets of their cells (one device allocation)."""

    def __init__(self, positions: torch.Tensor, space: CellSpace):
        lib = _native.lib()
        self.positions = _check_positions(positions)
        self.space = space
        self.count = int(self.positions.shape[0])
        persistent, temp = ctypes.c_uint64(), ctypes.c_uint64()
        _native.check(lib.tgb_cell_directory_sizes(self.count, space.dims, ctypes.byref(persistent),
                                                   ctypes.byref(temp)), "tgb_cell_directory_sizes")
        device = self.positions.device
        self.temp_bytes = int(temp.value)
        self.buffer = torch.empty(int(persistent.value), dtype=torch.uint8, device=device)
        self.scratch = torch.empty(self.temp_bytes, dtype=torch.uint8, device=device)
        with torch.cuda.device(device):
            _native.check(lib.tgb_cell_directory_build(
                self.positions.data_ptr(), self.count, ctypes.byref(space.struct), self.buffer.data_ptr(),
                self.buffer.numel(), self.scratch.data_ptr(), self.temp_bytes, _stream(device)),
                "tgb_cell_directory_build")

    # -- CSR in the reference's edge order ---------------------------------------------------------
    def radius_csr(self, cutoff: float, exclude_self: bool, *, with_fields: bool = False):
        """(row_ptr, col, distance | None, displacement | None, candidate_pairs)."""
        lib = _native.lib()
        device = self.positions.device
        n, dims = self.count, self.space.dims
        row_ptr = torch.empty(n + 1, dtype=torch.int64, device=device)
        pairs = torch.zeros(1, dtype=torch.int64, device=device)
        with torch.cuda.device(device):
            _native.check(lib.tgb_radius_row_ptr(
                self.positions.data_ptr(), n, ctypes.byref(self.space.struct), self.buffer.data_ptr(),
                float(cutoff), int(bool(exclude_self)), row_ptr.data_ptr(), pairs.data_ptr(),
                self.scratch.data_ptr(), self.temp_bytes, _stream(device)), "tgb_radius_row_ptr")
            totals = torch.stack((row_ptr[-1], pairs[0])).tolist()      # the one synchronisation: sizes col
            edges, candidate_pairs = int(totals[0]), int(totals[1])
            col = torch.empty(edges, dtype=torch.int64, device=device)
            distance = torch.empty(edges, dtype=torch.float32, device=device) if with_fields else None
            displacement = torch.empty((edges, dims), dtype=torch.float32, device=device) if with_fields else None
            if edges > 0:
                _native.check(lib.tgb_radius_fill(
                    self.positions.data_ptr(), n, ctypes.byref(self.space.struct), self.buffer.data_ptr(),
                    float(cutoff), int(bool(exclude_self)), row_ptr.data_ptr(), col.data_ptr(),
                    0 if distance is None else distance.data_ptr(),
                    0 if displacement is None else displacement.data_ptr(), _stream(device)), "tgb_radius_fill")
        return row_ptr, col, distance, displacement, candidate_pairs

    # -- fused consumer ----------------------------------------------------------------------------
    def weighted_sum(self, cutoff: float, exclude_self: bool, weight: int, x: torch.Tensor) -> torch.Tensor:
        lib = _native.lib()
        rows = x.detach().contiguous().reshape(self.count, -1)
        if rows.dtype != torch.float32:
            raise NotImplementedError(f"the fused radius consumer takes float32 features, got {rows.dtype}")
        out = torch.empty_like(rows)
        with torch.cuda.device(rows.device):
            _native.check(lib.tgb_radius_wsum_fwd(
                self.positions.data_ptr(), self.count, ctypes.byref(self.space.struct), self.buffer.data_ptr(),
                float(cutoff), int(bool(exclude_self)), int(weight), rows.data_ptr(), rows.shape[1],
                out.data_ptr(), _stream(rows.device)), "tgb_radius_wsum_fwd")
        return out.reshape(x.shape)

    def weighted_sum_position_grad(self, cutoff: float, exclude_self: bool, x: torch.Tensor,
                                   dy: torch.Tensor) -> torch.Tensor:
        lib = _native.lib()
        rows = x.detach().contiguous().reshape(self.count, -1)
        grads = dy.detach().contiguous().reshape(self.count, -1)
        dpos = torch.empty_like(self.positions)
        with torch.cuda.device(rows.device):
            _native.check(lib.tgb_radius_wsum_bwd_pos(
                self.positions.data_ptr(), self.count, ctypes.byref(self.space.struct), self.buffer.data_ptr(),
                float(cutoff), int(bool(exclude_self)), rows.data_ptr(), grads.data_ptr(), rows.shape[1],
                dpos.data_ptr(), _stream(rows.device)), "tgb_radius_wsum_bwd_pos")
        return dpos


class RadiusWeightedSumFunction(torch.autograd.Function):
    """out[i] = sum_j weight(i, j) * x[j] over a scalar-cutoff radius relation that is never written.

    The relation is symmetric, so the source cotangent is the same fold applied to ``dy``; the
    position cotangent (distance weight only) has its own kernel."""

    @staticmethod
    def forward(ctx, positions, x, directory: CellDirectory, cutoff: float, exclude_self: bool, weight: int):
        ctx.directory, ctx.cutoff, ctx.exclude_self, ctx.weight = directory, cutoff, exclude_self, weight
        ctx.save_for_backward(x)
        return directory.weighted_sum(cutoff, exclude_self, weight, x)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        d = ctx.directory
        dx = d.weighted_sum(ctx.cutoff, ctx.exclude_self, ctx.weight, dy) if ctx.needs_input_grad[1] else None
        dpos = None
        if ctx.needs_input_grad[0] and ctx.weight == PAIR_WEIGHT_DISTANCE:
            dpos = d.weighted_sum_position_grad(ctx.cutoff, ctx.exclude_self, x, dy)
        return dpos, dx, None, None, None, None


_UNIT_BALL = {1: 2.0, 2: 3.141592653589793, 3: 4.1887902047863905}
KNN_GRID_MIN_CANDIDATES = 4096      # below this the tiled scan over all candidates is as fast


def _knn_cell_size(lower, upper, count: int, k: int, dims: int) -> float:
    """Cell edge for the shell search: the radius of a ball that holds about k points at the mean
    density of the candidates' bounding box, plus a fifth.  Axes along which the points do not
    spread (a plane or a line embedded in space) do not count as dimensions of that density."""
    extents = [float(h) - float(l) for l, h in zip(lower, upper)]
    widest = max(extents)
    if widest <= 0.0:
        return 1.0
    spread = [extent for extent in extents if extent >= 1.0e-3 * widest]
    volume = 1.0
    for extent in spread:
        volume *= extent
    radius = (k * volume / (count * _UNIT_BALL[len(spread)])) ** (1.0 / len(spread))
    return 1.2 * radius


def knn_indices(queries: torch.Tensor, candidates: torch.Tensor, k: int, exclude_self: bool, *,
                self_search: bool | None = None) -> tuple[torch.Tensor, str]:
    """(col [nq * k] int64, builder name): the k nearest candidates of every query, ascending by
    (squared distance, candidate index).  Up to three dimensions and enough candidates: the shell
    search over a cell directory of the candidates; otherwise the tiled scan over all candidates.
    Both are exact and give identical results."""
    lib = _native.lib()
    q, c = _check_positions(queries), _check_positions(candidates)
    if self_search is None:
        self_search = queries is candidates
    col = torch.empty(q.shape[0] * int(k), dtype=torch.int64, device=q.device)
    dims = int(q.shape[1])
    if dims <= 3 and c.shape[0] >= KNN_GRID_MIN_CANDIDATES and q.shape[0] > 0:
        # one small read-back: the bounding boxes size the cells and bound the rounding of a coordinate
        box = torch.stack((*c.aminmax(dim=0), *q.aminmax(dim=0))).tolist()
        lower, upper = box[0], box[1]
        largest = max(max(abs(v) for v in row) for row in box)
        cell = _knn_cell_size(lower, upper, int(c.shape[0]), int(k), dims)
        if all(v == v and abs(v) != float("inf") for row in box for v in row) and largest / cell < 2.0 ** 30:
            space = make_cell_space(dims, cell, None)
            directory = CellDirectory(c, space)
            unsettled = torch.empty(q.shape[0], dtype=torch.int32, device=q.device)
            margin = 4.0e-7 * largest
            with torch.cuda.device(q.device):
                _native.check(lib.tgb_knn_grid(
                    q.data_ptr(), q.shape[0], c.data_ptr(), c.shape[0], ctypes.byref(space.struct),
                    directory.buffer.data_ptr(), int(k), int(bool(exclude_self)), int(bool(self_search)),
                    float(margin), col.data_ptr(), 0, unsettled.data_ptr(), _stream(q.device)), "tgb_knn_grid")
            return col, "b200-exact-knn-cell-shells"
    with torch.cuda.device(q.device):
        _native.check(lib.tgb_knn(q.data_ptr(), q.shape[0], c.data_ptr(), c.shape[0], q.shape[1], int(k),
                                  int(bool(exclude_self)), col.data_ptr(), 0, _stream(q.device)), "tgb_knn")
    return col, "b200-exact-knn-tiled-scan"


def edge_geometry(dst_positions: torch.Tensor, src_positions: torch.Tensor, space: CellSpace,
                  row_ptr: torch.Tensor, col: torch.Tensor):
    """(displacement [E, D], distance [E]) of a stored relation, minimum image under a lattice."""
    lib = _native.lib()
    d, s = _check_positions(dst_positions), _check_positions(src_positions)
    edges = int(col.numel())
    displacement = torch.empty((edges, d.shape[1]), dtype=torch.float32, device=d.device)
    distance = torch.empty(edges, dtype=torch.float32, device=d.device)
    with torch.cuda.device(d.device):
        _native.check(lib.tgb_edge_geometry(
            d.data_ptr(), s.data_ptr(), ctypes.byref(space.struct), row_ptr.data_ptr(), col.data_ptr(),
            d.shape[0], edges, displacement.data_ptr(), distance.data_ptr(), _stream(d.device)),
            "tgb_edge_geometry")
    return displacement, distance


__all__ = ["CellDirectory", "CellSpace", "RadiusWeightedSumFunction", "edge_geometry", "knn_indices",
           "make_cell_space", "periodic_extents", "periodic_lattice", "PAIR_WEIGHT_ONE", "PAIR_WEIGHT_DISTANCE"]
