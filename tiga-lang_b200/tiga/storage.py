"""Persistent CSR graphs (``.gfg`` directories) and their row-paged access.

On-disk format of the reference (python/tiga/graph/storage.py:20-24, 352-635 of
walkerchi/TIGA-lang), read and written here bit for bit:

    <name>.gfg/
        manifest.json   {"format": "tiga.gfg.csr.v1" | "tiga.gfg.csr.v2", "num_src", "num_dst",
                         "num_edges", "index_dtype": "int32" | "int64", "sorted_by_dst",
                         "fields": [{"role", "name", "shape", "dtype", "file"}, ...]   (v2 only)}
                        written as json.dumps(indent=2, sort_keys=True) + "\\n"
        row_ptr.bin     little-endian indices, num_dst + 1 of them
        col_idx.bin     little-endian indices, num_edges of them
        fields/<role>.<name>.bin    fixed-row-width little-endian payload per node / edge field

``tg.save(graph, path, fields=)`` writes one, ``tg.load(path, device=)`` opens one as a Graph whose
topology stays on disk (``schema.realization == "paged_csr"``).  A MessagePassing call on such a
graph runs page by page over blocks of destination rows: each page's rows are read from the
memory-mapped files, moved to the GPU and reduced by the same native kernels as a resident graph
(tiga/message_passing.py), so a relation larger than device memory can be processed; the reference
does the same on its host evaluator (python/tiga/message_passing/paged.py:434-583).
"""
from __future__ import annotations

import json
import math
import os
import shutil
import tempfile
from pathlib import Path
from typing import Iterator, Mapping

import numpy as np
import torch

FORMAT_V1 = "tiga.gfg.csr.v1"
FORMAT_V2 = "tiga.gfg.csr.v2"          # v1 + a "fields" section
ROLES = ("src", "dst", "edge")
_INDEX = {"int32": np.dtype("<i4"), "int64": np.dtype("<i8")}
_FIELD = {"float16": np.dtype("<f2"), "float32": np.dtype("<f4"), "float64": np.dtype("<f8"),
          "int32": np.dtype("<i4"), "int64": np.dtype("<i8"), "bool": np.dtype("?"),
          "complex64": np.dtype("<c8"), "complex128": np.dtype("<c16")}
_TORCH_NAME = {torch.float16: "float16", torch.float32: "float32", torch.float64: "float64",
               torch.int32: "int32", torch.int64: "int64", torch.bool: "bool",
               torch.complex64: "complex64", torch.complex128: "complex128"}


class PagedCSRStore:
    """Manifest handle over CSR indices (and fields) that live in files; reads are explicit
    destination-row ranges through memory maps, the whole ``col_idx`` is never required in RAM."""

    def __init__(self, path) -> None:
        root = Path(path).expanduser().resolve()
        manifest_path = root / "manifest.json"
        try:
            manifest = json.loads(manifest_path.read_text(encoding="utf-8"))
        except FileNotFoundError as error:
            raise FileNotFoundError(f"not a Tiga graph: {root}") from error
        if manifest.get("format") not in (FORMAT_V1, FORMAT_V2):
            raise ValueError(f"unsupported Tiga graph format in {manifest_path}")
        if not {"num_src", "num_dst", "num_edges", "index_dtype"} <= manifest.keys():
            raise ValueError("Tiga graph manifest is incomplete")
        if manifest["index_dtype"] not in _INDEX:
            raise ValueError("persistent CSR index_dtype must be int32 or int64")
        self.path = root
        self.num_src, self.num_dst, self.num_edges = (int(manifest[k]) for k in ("num_src", "num_dst", "num_edges"))
        if min(self.num_src, self.num_dst, self.num_edges) < 0:
            raise ValueError("persistent CSR extents must be non-negative")
        self.index_name = manifest["index_dtype"]
        self.index_dtype = torch.int32 if self.index_name == "int32" else torch.int64
        self.sorted_by_dst = bool(manifest.get("sorted_by_dst", True))
        item = _INDEX[self.index_name]
        row_file, col_file = root / "row_ptr.bin", root / "col_idx.bin"
        if row_file.stat().st_size != (self.num_dst + 1) * item.itemsize:
            raise ValueError("persistent row_ptr size disagrees with manifest")
        if col_file.stat().st_size != self.num_edges * item.itemsize:
            raise ValueError("persistent col_idx size disagrees with manifest")
        self._rows = np.memmap(row_file, dtype=item, mode="r", shape=(self.num_dst + 1,))
        self._cols = (np.memmap(col_file, dtype=item, mode="r", shape=(self.num_edges,)) if self.num_edges
                      else np.zeros(0, dtype=item))
        if [int(self._rows[0]), int(self._rows[-1])] != [0, self.num_edges]:
            raise ValueError("persistent CSR row pointer endpoints are invalid")
        self._fields: dict[tuple[str, str], tuple[tuple[int, ...], str, Path]] = {}
        leading = {"src": self.num_src, "dst": self.num_dst, "edge": self.num_edges}
        for entry in manifest.get("fields", []):
            role, name = entry.get("role"), entry.get("name")
            if role not in ROLES or not isinstance(name, str) or not name:
                raise ValueError("persistent field entry has an invalid role/name")
            if (role, name) in self._fields:
                raise ValueError(f"duplicate persistent field {role}.{name}")
            dtype = entry.get("dtype")
            if dtype not in _FIELD:
                raise ValueError(f"persistent field {role}.{name} has unknown dtype")
            shape = tuple(int(extent) for extent in entry.get("shape", ()))
            if not shape or any(extent < 0 for extent in shape):
                raise ValueError(f"persistent field {role}.{name} shape is invalid")
            if shape[0] != leading[role]:
                raise ValueError(f"persistent field {role}.{name} leading dimension must be {leading[role]}")
            relative = Path(entry.get("file", ""))
            if relative.is_absolute() or ".." in relative.parts:
                raise ValueError(f"persistent field {role}.{name} path is unsafe")
            if (root / relative).stat().st_size != math.prod(shape) * _FIELD[dtype].itemsize:
                raise ValueError(f"persistent field {role}.{name} size disagrees with manifest")
            self._fields[(role, name)] = (shape, dtype, root / relative)

    # ------------------------------------------------------------------ topology
    def _page(self, begin: int, end: int):
        if not 0 <= begin <= end <= self.num_dst:
            raise ValueError("paged CSR row range is outside the graph")
        rows = np.asarray(self._rows[begin:end + 1])
        first, last = int(rows[0]), int(rows[-1])
        cols = np.asarray(self._cols[first:last])
        if rows.size > 1 and bool(np.any(rows[1:] < rows[:-1])):
            raise ValueError("persistent row_ptr must be monotonic")
        if cols.size and (int(cols.min()) < 0 or int(cols.max()) >= self.num_src):
            raise ValueError("persistent col_idx contains an out-of-range source index")
        return rows - rows[0], cols, first

    def read_rows(self, begin: int, end: int):
        """(row_ptr starting at 0, col_idx) of destination rows [begin, end) as tuples of ints."""
        rows, cols, _ = self._page(begin, end)
        return tuple(rows.tolist()), tuple(cols.tolist())

    def read_page(self, begin: int, end: int):
        """read_rows plus the position of the page's first edge in the global edge list."""
        rows, cols, first = self._page(begin, end)
        return tuple(rows.tolist()), tuple(cols.tolist()), first

    def page_tensors(self, begin: int, end: int, device):
        """The page as index tensors on `device` plus its first edge (what paged execution uses)."""
        rows, cols, first = self._page(begin, end)
        to = lambda a: torch.from_numpy(np.array(a)).to(device)       # noqa: E731  (a copy: the map is read-only)
        return to(rows), to(cols), first

    def iter_pages(self, *, rows_per_page: int) -> Iterator[tuple[int, int, tuple, tuple]]:
        if rows_per_page <= 0:
            raise ValueError("rows_per_page must be positive")
        for begin in range(0, self.num_dst, rows_per_page):
            end = min(self.num_dst, begin + rows_per_page)
            yield (begin, end, *self.read_rows(begin, end))

    def materialize(self, *, device="cpu"):
        rows, cols, _ = self.page_tensors(0, self.num_dst, device)
        return rows, cols

    # -------------------------------------------------------------------- fields
    def field_names(self, role: str) -> tuple[str, ...]:
        if role not in ROLES:
            raise ValueError("field role must be 'src', 'dst' or 'edge'")
        return tuple(name for r, name in self._fields if r == role)

    def field_shape_dtype(self, role: str, name: str):
        if (role, name) not in self._fields:
            raise KeyError(f"no persistent field {role}.{name}")
        shape, dtype, _ = self._fields[(role, name)]
        return shape, dtype

    def field_rows(self, role: str, name: str, begin: int, end: int, device="cpu") -> torch.Tensor:
        """Rows [begin, end) of a stored field, read through a memory map."""
        if (role, name) not in self._fields:
            raise KeyError(f"no persistent field {role}.{name}")
        shape, dtype, file = self._fields[(role, name)]
        if not 0 <= begin <= end <= shape[0]:
            raise ValueError("field row range is outside the field")
        mapped = np.memmap(file, dtype=_FIELD[dtype], mode="r", shape=shape) if math.prod(shape) else \
            np.zeros(shape, dtype=_FIELD[dtype])
        return torch.from_numpy(np.array(mapped[begin:end])).to(device)

    def fields(self, role: str, device="cpu") -> dict[str, torch.Tensor]:
        return {name: self.field_rows(role, name, 0, self._fields[(role, name)][0][0], device)
                for name in self.field_names(role)}


def _index_bytes(values: torch.Tensor, name: str) -> bytes:
    return values.detach().cpu().numpy().astype(_INDEX[name], copy=False).tobytes()


def save_graph(graph, path, *, fields: Mapping[str, Mapping[str, torch.Tensor]] | None = None) -> None:
    """Write a static CSR Graph (resident or paged) as a ``.gfg`` directory; refuses to overwrite."""
    destination = Path(path).expanduser().resolve()
    if destination.exists():
        raise FileExistsError(f"refusing to overwrite existing Tiga graph: {destination}")
    schema = graph.schema
    if schema.lifecycle != "static" or schema.realization not in ("materialized_csr", "paged_csr"):
        raise TypeError("only a static CSR Graph can be saved as .gfg")
    fields = {role: dict(group) for role, group in (fields or {}).items() if group}
    store = getattr(graph, "_paged_store", None)
    num_edges = store.num_edges if store is not None else int(graph.resolve_csr()[1].numel())
    leading = {"src": schema.num_src, "dst": schema.num_dst, "edge": num_edges}
    for role, group in fields.items():
        if role not in ROLES:
            raise ValueError("field role must be 'src', 'dst' or 'edge'")
        for name, value in group.items():
            if not isinstance(value, torch.Tensor) or value.ndim == 0 or value.shape[0] != leading[role]:
                raise ValueError(f"{role}.{name} leading dimension must be {leading[role]}")
            if value.dtype not in _TORCH_NAME:
                raise ValueError(f"unsupported persistent field dtype {value.dtype}")
    destination.parent.mkdir(parents=True, exist_ok=True)
    temporary = Path(tempfile.mkdtemp(prefix=f".{destination.name}.", dir=destination.parent))
    try:
        if store is not None:       # a paged graph is copied file by file: its topology is never materialised
            shutil.copytree(store.path, temporary, dirs_exist_ok=True)
            manifest = json.loads((temporary / "manifest.json").read_text(encoding="utf-8"))
        else:
            row_ptr, col_idx = graph.resolve_csr()
            name = "int32" if schema.index_dtype == torch.int32 else "int64"
            rows = row_ptr.detach().cpu()
            if rows.numel() == 0 or int(rows[0]) != 0 or int(rows[-1]) != col_idx.numel():
                raise ValueError("invalid CSR row pointer endpoints")
            if bool((rows[1:] < rows[:-1]).any()):
                raise ValueError("row_ptr must be monotonic")
            if col_idx.numel() and (int(col_idx.min()) < 0 or int(col_idx.max()) >= schema.num_src):
                raise ValueError("col_idx contains an out-of-range source index")
            (temporary / "row_ptr.bin").write_bytes(_index_bytes(row_ptr, name))
            (temporary / "col_idx.bin").write_bytes(_index_bytes(col_idx, name))
            manifest = {"format": FORMAT_V1, "num_src": schema.num_src, "num_dst": schema.num_dst,
                        "num_edges": int(col_idx.numel()), "index_dtype": name,
                        "sorted_by_dst": schema.sorted_by_dst}
        if fields:
            (temporary / "fields").mkdir(exist_ok=True)
            merged = {(item["role"], item["name"]): item for item in manifest.get("fields", [])}
            for role in ROLES:
                for name, value in fields.get(role, {}).items():
                    relative = f"fields/{role}.{name}.bin"
                    dtype = _TORCH_NAME[value.dtype]
                    payload = value.detach().cpu().contiguous().numpy().astype(_FIELD[dtype], copy=False).tobytes()
                    (temporary / relative).write_bytes(payload)
                    merged[(role, name)] = {"role": role, "name": name, "shape": list(value.shape),
                                            "dtype": dtype, "file": relative}
            manifest["format"] = FORMAT_V2
            manifest["fields"] = list(merged.values())
        (temporary / "manifest.json").write_text(json.dumps(manifest, indent=2, sort_keys=True) + "\n",
                                                 encoding="utf-8")
        os.replace(temporary, destination)
    except BaseException:
        shutil.rmtree(temporary, ignore_errors=True)
        raise


def save(graph, path, *, fields=None, overwrite: bool = False) -> None:
    """``tg.save``: persist a static CSR Graph (python/tiga/__init__.py:84-105 of the reference).
    Graph overwriting is unsupported; save to a new directory."""
    if overwrite:
        raise ValueError("Graph overwrite is not supported; save to a new directory")
    save_graph(graph, path, fields=fields)


def load(path, *, device="cpu"):
    """``tg.load``: open a persistent graph without loading its CSR arrays."""
    from .graph import Graph

    return Graph.open(path, device=device)


__all__ = ["FORMAT_V1", "FORMAT_V2", "PagedCSRStore", "load", "save", "save_graph"]
