"""Logical relation object over torch tensors: ``tg.Graph``.

Mirrors the Torch-facing behaviour of the reference's ``Graph``
(python/tiga/graph/core.py:157-709,1271-1299 and its Torch twin
python/tiga/interop/torch/graph.py:152-340,1212-1245 of walkerchi/TIGA-lang):
the constructors ``from_csr / from_coo / regular / cu_seqlens / cat /
triangular / dense``, ``transpose()``, ``halo()``, ``resolve_csr()``,
``destination_index()``, the degree statistics and ``planning_key()``.

CSR construction is integer work done with the same stable-sort / bincount /
cumsum recipe as the reference, so results are bit-identical.  The per-graph
launch plan of the CUDA library (degree buckets, split rows, transposed
relation) is built lazily and cached on the graph.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Literal

import torch

from .distributed.model import ByDestination, DeviceMesh, GraphPlacement

_INDEX_DTYPES = (torch.int32, torch.int64)
_DENSE_EDGE_LIMIT = 1 << 22  # resolve_csr guard of the reference (interop/torch/graph.py:899-904)


@dataclass(frozen=True)
class GraphSchema:
    num_src: int
    num_dst: int
    origin: str
    lifecycle: str
    realization: str
    index_dtype: torch.dtype
    sorted_by_dst: bool

    def specialization_key(self) -> tuple[object, ...]:
        return (self.num_src, self.num_dst, self.origin, self.lifecycle, self.realization,
                str(self.index_dtype), self.sorted_by_dst)


class Graph:
    """Immutable relation; static CSR owns two index tensors, dense/triangular
    and packed-sequence relations stay implicit."""

    _tiga_graph = True

    def __init__(self, schema: GraphSchema, *, row_ptr=None, col_idx=None, dense_boundary: str = "full",
                 device=None, placement: GraphPlacement | None = None, cu_seqlens=None, causal: bool = True):
        self._schema = schema
        self._row_ptr = row_ptr
        self._col_idx = col_idx
        self._dense_boundary = dense_boundary
        self._device = torch.device(device) if device is not None else (
            row_ptr.device if row_ptr is not None else torch.device("cpu"))
        if self._device.type == "cuda" and self._device.index is None and torch.cuda.is_available():
            # tensors report "cuda:<index>"
            self._device = torch.device("cuda", torch.cuda.current_device())
        self._placement = placement
        self._cu_seqlens = cu_seqlens  # packed block-diagonal relation kept implicit
        self._causal = causal
        self._degree_bounds_cache = None
        self._destination_cache = None
        self._plans = {}
        self._transpose_cache = None
        self._edge_map = None   # set for sub-relations whose weights live in a larger edge list
        self._shard = None      # (first_row, num_nodes) when the tensors hold one rank's block of rows only
        self._paged_store = None   # PagedCSRStore of a graph opened from a .gfg directory
        self._geometry = None      # GeometricRelation of a Graph.radius / Graph.knn relation
        self.page_rows = int(os.environ.get("TIGA_PAGE_ROWS", 1 << 20))   # destination rows per page

    # ------------------------------------------------------------ properties
    @property
    def schema(self) -> GraphSchema:
        return self._schema

    @property
    def device(self) -> torch.device:
        return self._device

    @property
    def placement(self):
        return self._placement

    @property
    def is_distributed(self) -> bool:
        return self._placement is not None

    @property
    def num_src(self) -> int:
        return self._schema.num_src

    @property
    def num_dst(self) -> int:
        return self._schema.num_dst

    @property
    def cu_seqlens_tensor(self):
        return self._cu_seqlens

    @property
    def causal(self) -> bool:
        return self._causal

    # ---------------------------------------------------------- constructors
    @staticmethod
    def _validate_index_tensor(name: str, value) -> None:
        if not isinstance(value, torch.Tensor):
            raise TypeError(f"{name} must be a torch.Tensor")
        if value.dtype not in _INDEX_DTYPES:
            raise TypeError(f"{name} must have dtype int32 or int64")
        if value.ndim != 1:
            raise ValueError(f"{name} must be one-dimensional")

    @staticmethod
    def _validate_csr_values(row_ptr, col_idx, num_src: int) -> None:
        if int(row_ptr[0].item()) != 0:
            raise ValueError("row_ptr must start at zero")
        if int(row_ptr[-1].item()) != col_idx.numel():
            raise ValueError("row_ptr[-1] must equal the number of edges")
        if bool(torch.any(row_ptr[1:] < row_ptr[:-1]).item()):
            raise ValueError("row_ptr must be monotonic")
        if col_idx.numel() and (int(col_idx.min().item()) < 0 or int(col_idx.max().item()) >= num_src):
            raise ValueError("col_idx contains an out-of-range source index")

    @classmethod
    def from_csr(cls, row_ptr, col_idx, *, num_src: int | None = None, sorted_by_dst: bool = True,
                 validate: Literal["basic", "full"] = "basic") -> "Graph":
        cls._validate_index_tensor("row_ptr", row_ptr)
        cls._validate_index_tensor("col_idx", col_idx)
        if row_ptr.device != col_idx.device:
            raise ValueError("row_ptr and col_idx must be on the same device")
        if row_ptr.numel() == 0:
            raise ValueError("row_ptr must contain at least the initial zero")
        num_dst = row_ptr.numel() - 1
        if num_src is None:
            num_src = num_dst if col_idx.numel() == 0 else int(col_idx.max().item()) + 1
        if num_src < 0:
            raise ValueError("num_src must be non-negative")
        if validate == "full":
            cls._validate_csr_values(row_ptr, col_idx, num_src)
        elif validate != "basic":
            raise ValueError("validate must be 'basic' or 'full'")
        schema = GraphSchema(num_src=num_src, num_dst=num_dst, origin="explicit", lifecycle="static",
                             realization="materialized_csr", index_dtype=col_idx.dtype,
                             sorted_by_dst=sorted_by_dst)
        return cls(schema, row_ptr=row_ptr, col_idx=col_idx)

    @classmethod
    def from_csr_shard(cls, row_ptr, col_idx, *, num_nodes: int, first_row: int) -> "Graph":
        """One rank's block of destination rows of a homogeneous relation over ``num_nodes`` nodes:
        ``row_ptr`` (starting at 0) and ``col_idx`` (GLOBAL source ids) describe rows
        ``[first_row, first_row + len(row_ptr) - 1)``.  Only ``.halo(mesh)`` snapshots of such a
        graph can be executed; every rank of the mesh passes its own block and the blocks must tile
        ``[0, num_nodes)`` in rank order.  An addition to the reference's constructors for graphs
        that are too large to hold whole on every rank (its ``halo()`` starts from the full CSR,
        python/tiga/distributed/transport.py:969-983)."""
        cls._validate_index_tensor("row_ptr", row_ptr)
        cls._validate_index_tensor("col_idx", col_idx)
        if row_ptr.device != col_idx.device:
            raise ValueError("row_ptr and col_idx must be on the same device")
        if row_ptr.numel() == 0:
            raise ValueError("row_ptr must contain at least the initial zero")
        rows = row_ptr.numel() - 1
        if not (0 <= first_row and first_row + rows <= num_nodes):
            raise ValueError("the block of rows must lie inside [0, num_nodes)")
        schema = GraphSchema(num_src=int(num_nodes), num_dst=int(num_nodes), origin="explicit", lifecycle="static",
                             realization="materialized_csr", index_dtype=col_idx.dtype, sorted_by_dst=True)
        graph = cls(schema, row_ptr=row_ptr, col_idx=col_idx)
        graph._shard = (int(first_row), int(num_nodes))
        return graph

    @classmethod
    def open(cls, path, *, device="cpu") -> "Graph":
        """Open a persistent ``.gfg`` graph without loading its CSR arrays
        (python/tiga/graph/core.py:413-426 of the reference).  The topology stays on disk
        (``schema.realization == "paged_csr"``); MessagePassing calls run page by page over blocks
        of ``page_rows`` destination rows, ``resolve_csr()`` materialises it on the graph's device."""
        from .storage import PagedCSRStore

        store = PagedCSRStore(path)
        schema = GraphSchema(num_src=store.num_src, num_dst=store.num_dst, origin="persistent", lifecycle="static",
                             realization="paged_csr", index_dtype=store.index_dtype,
                             sorted_by_dst=store.sorted_by_dst)
        graph = cls(schema, device=device)
        graph._paged_store = store
        return graph

    # ------------------------------------------------------ dynamic relations
    @classmethod
    def radius(cls, positions, cutoff, *, exclude_self: bool = True, fields=None, metric=None, select=None,
               periodic=None) -> "Graph":
        """Rebuildable radius relation over ``positions`` [N, D]: j is a neighbour of i when the
        (minimum-image) distance is at most ``cutoff`` (a scalar, one value per destination or an
        [N, N] matrix).  ``metric(src, dst, edge)`` replaces the Euclidean distance,
        ``select(src, dst, edge)`` is an additional boolean filter; the endpoint namespaces hold
        ``position`` plus ``fields``, the edge namespace ``displacement``, ``distance``, ``cutoff``
        (Graph.radius of the reference, python/tiga/interop/torch/graph.py:391-478)."""
        from .dynamic_graph import GeometricRelation, check_radius_arguments

        periodic, fields = check_radius_arguments(positions, cutoff, fields, metric, select, periodic)
        count = positions.shape[0]
        schema = GraphSchema(num_src=count, num_dst=count, origin="geometric_radius", lifecycle="dynamic",
                             realization="procedural_radius", index_dtype=torch.int64, sorted_by_dst=True)
        graph = cls(schema, device=positions.device)
        graph._geometry = GeometricRelation("radius", positions, cutoff=cutoff, periodic=periodic,
                                            exclude_self=exclude_self, fields=fields, metric=metric, select=select)
        return graph

    @classmethod
    def knn(cls, positions, k: int, *, candidates=None, exclude_self: bool | None = None) -> "Graph":
        """Exact k-nearest-neighbour relation: row i holds the k candidates nearest to query i,
        ascending by (distance, candidate index); ``candidates=None`` searches the queries themselves
        and then skips i (Graph.knn of the reference, graph.py:481-534)."""
        from .dynamic_graph import GeometricRelation, check_knn_arguments

        sources, exclude_self = check_knn_arguments(positions, k, candidates, exclude_self)
        schema = GraphSchema(num_src=(positions if sources is None else sources).shape[0],
                             num_dst=positions.shape[0], origin="geometric_knn", lifecycle="dynamic",
                             realization="procedural_knn", index_dtype=torch.int64, sorted_by_dst=True)
        graph = cls(schema, device=positions.device)
        graph._geometry = GeometricRelation("knn", positions, k=k, source_positions=sources,
                                            exclude_self=exclude_self)
        return graph

    @property
    def build_info(self) -> dict:
        """How the last resolve of a dynamic relation ran: builder, candidate_pairs, accepted_edges,
        materialized, cache_hit."""
        if self._geometry is None or self._geometry.build_info is None:
            raise RuntimeError("dynamic graph has not been resolved yet")
        return dict(self._geometry.build_info)

    def dynamic_signature(self):
        """Hashable description of a dynamic relation's search (None for stored relations): two graphs
        with equal signatures differ only in the tensors they were handed."""
        return None if self._geometry is None else (self._schema.specialization_key(), self._geometry.signature())

    @property
    def num_edges(self) -> int | None:
        if self._paged_store is not None:
            return self._paged_store.num_edges
        if self._geometry is not None:          # a dynamic relation has no edge count of its own
            return None
        return None if self._col_idx is None else int(self._col_idx.numel())

    def paged_rows(self, begin: int, end: int):
        """(row_ptr from 0, col_idx) of destination rows [begin, end) of a persistent graph."""
        if self._paged_store is None:
            raise TypeError("paged_rows requires a graph opened from a .gfg directory")
        return self._paged_store.read_rows(begin, end)

    def paged_page(self, begin: int, end: int):
        """paged_rows plus the global position of the page's first edge."""
        if self._paged_store is None:
            raise TypeError("paged_page requires a graph opened from a .gfg directory")
        return self._paged_store.read_page(begin, end)

    def fields(self, role: str):
        """Node / edge fields stored inside the .gfg, loaded onto the graph's device."""
        if self._paged_store is None:
            raise TypeError("fields() requires a graph opened from a .gfg directory")
        return self._paged_store.fields(role, self._device)

    def explain(self) -> str:
        backing = f" backing=nvme:{self._paged_store.path}" if self._paged_store is not None else ""
        dynamic = "" if self._geometry is None else self._geometry.describe()
        return (f"Graph num_src={self.num_src} num_dst={self.num_dst} origin={self._schema.origin} "
                f"lifecycle={self._schema.lifecycle} realization={self._schema.realization} "
                f"device={self._device}{backing}{dynamic}")

    @classmethod
    def from_coo(cls, src, dst, *, num_src: int | None = None, num_dst: int | None = None) -> "Graph":
        cls._validate_index_tensor("src", src)
        cls._validate_index_tensor("dst", dst)
        if src.shape != dst.shape:
            raise ValueError("src and dst must have identical shapes")
        if src.device != dst.device:
            raise ValueError("src and dst must be on the same device")
        if num_src is None:
            num_src = int(src.max().item()) + 1 if src.numel() else 0
        if num_dst is None:
            num_dst = int(dst.max().item()) + 1 if dst.numel() else 0
        if not isinstance(num_src, int) or num_src < 0:
            raise ValueError("num_src must be a non-negative integer")
        if not isinstance(num_dst, int) or num_dst < 0:
            raise ValueError("num_dst must be a non-negative integer")
        if src.numel():
            if int(src.min().item()) < 0 or int(src.max().item()) >= num_src:
                raise ValueError("src contains an out-of-range source index")
            if int(dst.min().item()) < 0 or int(dst.max().item()) >= num_dst:
                raise ValueError("dst contains an out-of-range destination index")
        order = torch.argsort(dst, stable=True)
        sorted_dst = dst[order]
        col_idx = src[order]
        counts = torch.bincount(sorted_dst.to(torch.int64), minlength=num_dst)
        row_ptr = torch.empty(num_dst + 1, device=dst.device, dtype=dst.dtype)
        row_ptr[0] = 0
        torch.cumsum(counts, dim=0, out=row_ptr[1:])
        return cls.from_csr(row_ptr, col_idx, num_src=num_src, sorted_by_dst=True, validate="basic")

    @classmethod
    def regular(cls, num_nodes: int, degree: int, *, device="cpu") -> "Graph":
        if not isinstance(num_nodes, int) or num_nodes < 1:
            raise ValueError("num_nodes must be a positive integer")
        if not isinstance(degree, int) or degree < 0:
            raise ValueError("degree must be a non-negative integer")
        row_ptr = torch.arange(num_nodes + 1, device=device, dtype=torch.int64) * degree
        col_idx = torch.arange(num_nodes * degree, device=device, dtype=torch.int64) % num_nodes
        return cls.from_csr(row_ptr, col_idx, num_src=num_nodes)

    @classmethod
    def cu_seqlens(cls, cu_seqlens, *, causal: bool = True) -> "Graph":
        """Block-diagonal packed variable-length relation (flash-attn varlen
        style).  Position i of sequence k gathers from [s_k, i] (causal) or its
        whole sequence.  Kept implicit; ``resolve_csr()`` materialises it."""
        cls._validate_index_tensor("cu_seqlens", cu_seqlens)
        if not isinstance(causal, bool):
            raise TypeError("causal must be bool")
        if cu_seqlens.numel() == 0 or int(cu_seqlens[0].item()) != 0:
            raise ValueError("cu_seqlens must start at zero")
        if bool(torch.any(cu_seqlens[1:] < cu_seqlens[:-1]).item()):
            raise ValueError("cu_seqlens must be monotonic")
        total = int(cu_seqlens[-1].item())
        schema = GraphSchema(num_src=total, num_dst=total, origin="packed_sequences", lifecycle="static",
                             realization="implicit_block_dense", index_dtype=cu_seqlens.dtype,
                             sorted_by_dst=True)
        return cls(schema, device=cu_seqlens.device, cu_seqlens=cu_seqlens, causal=causal,
                   dense_boundary="lower_inclusive" if causal else "full")

    @classmethod
    def dense(cls, num_src: int, num_dst: int | None = None, *, device=None, index_dtype=torch.int64) -> "Graph":
        if num_dst is None:
            num_dst = num_src
        if not isinstance(num_src, int) or num_src < 0:
            raise ValueError("num_src must be non-negative")
        if not isinstance(num_dst, int) or num_dst < 0:
            raise ValueError("num_dst must be non-negative")
        if index_dtype not in _INDEX_DTYPES:
            raise TypeError("index_dtype must be int32 or int64")
        schema = GraphSchema(num_src=num_src, num_dst=num_dst, origin="cartesian", lifecycle="static",
                             realization="implicit_dense", index_dtype=index_dtype, sorted_by_dst=True)
        return cls(schema, device=device or "cpu")

    @classmethod
    def triangular(cls, num_entities: int, *, device=None, index_dtype=torch.int64) -> "Graph":
        graph = cls.dense(num_entities, num_entities, device=device, index_dtype=index_dtype)
        graph._schema = GraphSchema(num_src=num_entities, num_dst=num_entities, origin="lower_triangular",
                                    lifecycle="static", realization="implicit_dense", index_dtype=index_dtype,
                                    sorted_by_dst=True)
        graph._dense_boundary = "lower_inclusive"
        return graph

    @classmethod
    def cat(cls, graphs) -> "Graph":
        """Block-diagonal composition.  A list of square triangular (or square
        dense) blocks stays implicit as a packed-sequence relation, which is
        what ``cat([triangular(n) for n in lengths])`` means in the reference
        (python/tiga/graph/core.py:650-709); anything else is assembled as CSR."""
        blocks = list(graphs)
        if not blocks:
            raise ValueError("graphs must be a non-empty sequence")
        for block in blocks:
            if not isinstance(block, Graph):
                raise TypeError("graphs must contain only Graph instances")
        device = blocks[0].device
        if any(str(block.device) != str(device) for block in blocks):
            raise ValueError("all blocks must share a device")
        dtype = (torch.int64 if any(block.schema.index_dtype == torch.int64 for block in blocks)
                 else torch.int32)
        implicit = all(block.schema.realization == "implicit_dense" and block.num_src == block.num_dst
                       for block in blocks)
        boundaries = {block._dense_boundary for block in blocks}
        if implicit and len(boundaries) == 1:
            lengths = torch.tensor([0] + [block.num_dst for block in blocks], dtype=dtype)
            cu = torch.cumsum(lengths, 0).to(dtype).to(device)
            return cls.cu_seqlens(cu, causal=boundaries == {"lower_inclusive"})
        row_parts = [torch.zeros(1, device=device, dtype=dtype)]
        col_parts = []
        edge_offset = 0
        src_offset = 0
        for block in blocks:
            block_rows, block_cols = block.resolve_csr()
            block_rows = block_rows.to(dtype)
            col_parts.append(block_cols.to(dtype) + src_offset)
            row_parts.append(block_rows[1:] + edge_offset)
            edge_offset += int(block_rows[-1].item())
            src_offset += block.schema.num_src
        row_ptr = torch.cat(row_parts)
        col_idx = (torch.cat(col_parts) if any(part.numel() for part in col_parts)
                   else torch.empty(0, device=device, dtype=dtype))
        return cls.from_csr(row_ptr, col_idx, num_src=src_offset)

    # --------------------------------------------------------------- queries
    def sequence_boundaries(self):
        """cu_seqlens of an implicit dense / triangular / packed relation, or
        None for a stored CSR."""
        if self._cu_seqlens is not None:
            return self._cu_seqlens
        if self._schema.realization == "implicit_dense" and self.num_src == self.num_dst:
            return torch.tensor([0, self.num_dst], dtype=self._schema.index_dtype, device=self._device)
        return None

    def resolve_csr(self):
        if self._shard is not None and self._placement is None:
            raise RuntimeError("a Graph.from_csr_shard block is executable only as a .halo(mesh) snapshot "
                               "under a DistributedRuntime")
        if self._geometry is not None:
            row_ptr, col_idx, rebuilt = self._geometry.resolve(self._schema.num_dst)
            if rebuilt or self._row_ptr is not row_ptr:
                # a new physical snapshot: everything derived from the previous CSR is stale
                self._plans, self._transpose_cache = {}, None
                self._destination_cache = self._degree_bounds_cache = None
                self.__dict__.pop("_span_ratio_cache", None)
            self._row_ptr, self._col_idx = row_ptr, col_idx
            return row_ptr, col_idx
        if self._row_ptr is not None:
            return self._row_ptr, self._col_idx
        if self._paged_store is not None:      # a persistent graph: load the whole topology onto the device
            self._row_ptr, self._col_idx = self._paged_store.materialize(device=self._device)
            return self._row_ptr, self._col_idx
        dtype = self._schema.index_dtype
        device = self._device
        if self._cu_seqlens is not None:
            # Graph.cu_seqlens of the reference (interop/torch/graph.py:259-294)
            cu = self._cu_seqlens
            lengths = cu.diff()
            total = int(cu[-1].item())
            positions = torch.arange(total, device=device, dtype=dtype)
            sequence = torch.repeat_interleave(
                torch.arange(lengths.numel(), device=device, dtype=dtype), lengths.to(torch.int64))
            start = cu[:-1][sequence]
            degree = positions - start + 1 if self._causal else lengths[sequence]
            if int(degree.sum().item()) > _DENSE_EDGE_LIMIT:
                raise RuntimeError("refusing to materialise more than 2^22 edges of an implicit relation")
            row_ptr = torch.cat([cu.new_zeros(1), degree.cumsum(0, dtype=dtype)])
            repeats = degree.to(torch.int64)
            offset = torch.arange(int(row_ptr[-1].item()), device=device, dtype=dtype)
            col_idx = start.repeat_interleave(repeats) + (offset - row_ptr[:-1].repeat_interleave(repeats))
        else:
            n_src, n_dst = self.num_src, self.num_dst
            if self._dense_boundary == "lower_inclusive":
                degree = torch.arange(1, n_dst + 1, device=device, dtype=dtype).clamp(max=n_src)
            else:
                degree = torch.full((n_dst,), n_src, device=device, dtype=dtype)
            if int(degree.sum().item()) > _DENSE_EDGE_LIMIT:
                raise RuntimeError("refusing to materialise more than 2^22 edges of an implicit relation")
            row_ptr = torch.cat([degree.new_zeros(1), degree.cumsum(0, dtype=dtype)])
            offset = torch.arange(int(row_ptr[-1].item()), device=device, dtype=dtype)
            col_idx = offset - row_ptr[:-1].repeat_interleave(degree.to(torch.int64))
        self._row_ptr, self._col_idx = row_ptr, col_idx
        return row_ptr, col_idx

    def destination_index(self, row_ptr=None):
        if row_ptr is None:
            row_ptr = self.resolve_csr()[0]
        if self._destination_cache is None or self._destination_cache[0] is not row_ptr:
            rows = row_ptr.numel() - 1
            destination = torch.repeat_interleave(
                torch.arange(rows, device=row_ptr.device, dtype=row_ptr.dtype),
                (row_ptr[1:] - row_ptr[:-1]).to(torch.int64))
            self._destination_cache = (row_ptr, destination)
        return self._destination_cache[1]

    def implicit_edge_fields(self, row_ptr, col_idx):
        """Edge fields the relation provides by itself: ``displacement`` (source - destination,
        minimum image) and ``distance`` of geometric relations, nothing for stored ones."""
        if self._geometry is None:
            return {}
        return self._geometry.edge_fields(row_ptr, col_idx, self.destination_index(row_ptr))

    def degree_bounds(self) -> tuple[int, int]:
        if self._degree_bounds_cache is None:
            row_ptr = self.resolve_csr()[0]
            if row_ptr.numel() <= 1:
                self._degree_bounds_cache = (0, 0)
            else:
                degree = row_ptr[1:] - row_ptr[:-1]
                self._degree_bounds_cache = (int(degree.min().item()), int(degree.max().item()))
        return self._degree_bounds_cache

    def degree_statistics(self) -> tuple[int, int, int]:
        lo, hi = self.degree_bounds()
        row_ptr = self.resolve_csr()[0]
        return lo, hi, int(row_ptr[-1].item()) if row_ptr.numel() else 0

    def fixed_degree(self) -> int | None:
        lo, hi = self.degree_bounds()
        return lo if lo == hi else None

    _HISTOGRAM_DEGREE_LIMIT = 4096

    def degree_histogram(self) -> tuple[int, ...]:
        """``counts[d]`` = number of destination rows with exactly ``d`` edges, for ``d`` up to the
        largest degree; exact, integer work on the graph's device.  Like the reference's
        (python/tiga/interop/torch/graph.py:1258-1277) it refuses graphs whose largest degree
        exceeds 4096: the table is a planning aid for bounded-degree graphs."""
        _, largest, _ = self.degree_statistics()
        if largest > self._HISTOGRAM_DEGREE_LIMIT:
            raise ValueError("exact degree histogram is limited to degree_max <= 4096")
        if self._row_ptr is None and self._schema.realization == "implicit_dense":
            if self._dense_boundary == "lower_inclusive":     # row i sees i + 1 sources
                return (0,) + (1,) * largest
            return (0,) * largest + (self.num_dst,)
        row_ptr = self.resolve_csr()[0]
        lengths = (row_ptr[1:] - row_ptr[:-1]).to(torch.int64)
        return tuple(torch.bincount(lengths, minlength=largest + 1).cpu().tolist())

    def source_index_span_ratio(self, samples: int = 4096) -> float:
        """Locality signal for planning: mean ``|source id - destination id|`` over up to
        ``samples`` evenly spaced edge slots, divided by the larger endpoint count.  Near 0 for
        index-local gathers, about 1/3 for random numbering (the reference's definition,
        python/tiga/interop/torch/graph.py:1279-1311); cached on the immutable snapshot."""
        cached = self.__dict__.get("_span_ratio_cache")
        if cached is not None:
            return cached
        if self._row_ptr is None and self._schema.realization in ("implicit_dense", "implicit_block_dense"):
            return 1.0 / 3.0
        row_ptr, col_idx = self.resolve_csr()
        edges = int(col_idx.numel())
        ratio = 0.0
        if edges:
            picked = torch.linspace(0, edges - 1, min(int(samples), edges), dtype=torch.float64,
                                    device=col_idx.device).to(row_ptr.dtype)
            owner = torch.searchsorted(row_ptr[1:].contiguous(), picked, right=True)
            distance = (col_idx[picked.long()].to(torch.int64) - owner).abs().double().mean()
            ratio = float(distance.item()) / max(1, self.num_src, self.num_dst)
        ratio = min(max(ratio, 0.0), 1.0)
        self.__dict__["_span_ratio_cache"] = ratio
        return ratio

    def specialization_key(self) -> tuple[object, ...]:
        placement = self._placement.specialization_key() if self._placement is not None else ()
        return (*self._schema.specialization_key(), self._dense_boundary, placement)

    def planning_key(self) -> tuple[object, ...]:
        if self._row_ptr is None:
            return (*self.specialization_key(), "implicit")
        return (*self.specialization_key(), self.degree_statistics())

    def transpose(self) -> "Graph":
        """Materialised snapshot with endpoint roles swapped (stable order)."""
        if self._transpose_cache is None:
            row_ptr, col_idx = self.resolve_csr()
            destination = self.destination_index(row_ptr)
            self._transpose_cache = type(self).from_coo(
                destination, col_idx, num_src=self._schema.num_dst, num_dst=self._schema.num_src)
        return self._transpose_cache

    def halo(self, mesh: DeviceMesh, *, partition: ByDestination | None = None, depth="auto") -> "Graph":
        placement = GraphPlacement(mesh, partition or ByDestination(), depth)
        clone = object.__new__(Graph)
        clone.__dict__ = self.__dict__.copy()
        clone._placement = placement
        clone._plans = {}
        return clone

    # ------------------------------------------------------------ native plan
    def native_plan(self, *, transpose: bool):
        """Launch plan of the CUDA library for this CSR, cached per graph."""
        from .plan import CSRPlan

        if self._geometry is not None:
            self.resolve_csr()           # drops the cached plans when the positions have changed
        plan = self._plans.get(True) or (None if transpose else self._plans.get(False))
        if plan is None:
            row_ptr, col_idx = self.resolve_csr()
            plan = CSRPlan(row_ptr, col_idx, self.num_src, transpose=transpose, edge_map=self._edge_map)
            self._plans[transpose] = plan
        return plan


__all__ = ["Graph", "GraphSchema"]
