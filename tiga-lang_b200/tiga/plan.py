"""Python owner of one native CSR plan (device buffers + opaque handle)."""
from __future__ import annotations

import ctypes

import torch

from . import _native


class CSRPlan:
    """Degree-bucket launch plan (and, optionally, the stable transposed
    relation) of one CSR graph, built by ``tgb_csr_plan_create``.  The plan's
    device memory is a torch uint8 tensor owned by this object; the library
    only holds pointers into it."""

    def __init__(self, row_ptr: torch.Tensor, col_idx: torch.Tensor, num_src: int, *, transpose: bool,
                 edge_map: torch.Tensor | None = None):
        if not row_ptr.is_cuda:
            raise RuntimeError("native plans exist for CUDA graphs only")
        if row_ptr.dtype != col_idx.dtype:
            raise TypeError("row_ptr and col_idx must share one index dtype")
        lib = _native.lib()
        self.row_ptr = row_ptr.contiguous()
        self.col_idx = col_idx.contiguous()
        self.num_dst = self.row_ptr.numel() - 1
        self.num_src = int(num_src)
        self.num_edges = self.col_idx.numel()
        self.index_bits = 32 if row_ptr.dtype == torch.int32 else 64
        self.transposed = bool(transpose)
        self.device = row_ptr.device
        flags = _native.PLAN_FORWARD | (_native.PLAN_TRANSPOSE if transpose else 0)
        persistent = ctypes.c_uint64()
        temp = ctypes.c_uint64()
        with torch.cuda.device(self.device):
            _native.check(lib.tgb_csr_plan_sizes(self.num_dst, self.num_src, self.num_edges, self.index_bits,
                                                 flags, ctypes.byref(persistent), ctypes.byref(temp)),
                          "tgb_csr_plan_sizes")
            self._persistent = torch.empty(max(int(persistent.value), 256), dtype=torch.uint8, device=self.device)
            scratch = torch.empty(max(int(temp.value), 256), dtype=torch.uint8, device=self.device)
            handle = ctypes.c_void_p()
            stream = torch.cuda.current_stream(self.device).cuda_stream
            _native.check(lib.tgb_csr_plan_create(
                self.row_ptr.data_ptr(), self.col_idx.data_ptr(), self.num_dst, self.num_src, self.num_edges,
                self.index_bits, flags, self._persistent.data_ptr(), self._persistent.numel(),
                scratch.data_ptr(), scratch.numel(), stream, ctypes.byref(handle)), "tgb_csr_plan_create")
        self._handle = handle
        self.edge_map = None
        if edge_map is not None:
            # edge e of this CSR is entry edge_map[e] of the caller's weight / dw arrays
            self.edge_map = edge_map.to(device=self.device, dtype=torch.int32).contiguous()
            with torch.cuda.device(self.device):
                _native.check(lib.tgb_csr_plan_set_edge_map(self._handle, self.edge_map.data_ptr(), stream),
                              "tgb_csr_plan_set_edge_map")
        info = (ctypes.c_int64 * 16)()
        _native.check(lib.tgb_csr_plan_info(self._handle, info), "tgb_csr_plan_info")
        self.info = {
            "num_dst": info[0], "num_src": info[1], "num_edges": info[2], "min_degree": info[3],
            "max_degree": info[4], "long_rows": info[5], "segments": info[6], "long_rows_t": info[7],
            "segments_t": info[8], "split_threshold": info[9], "segment_edges": info[10],
            "min_in_degree": info[11], "max_in_degree": info[12],
        }
        self._scratch_sizes = {}

    @property
    def handle(self):
        return self._handle

    def __del__(self):
        handle = getattr(self, "_handle", None)
        if handle:
            try:
                _native.lib().tgb_csr_plan_destroy(handle)
            except Exception:
                pass
            self._handle = None

    def scratch_bytes(self, direction: int, reducer: int, features: int) -> int:
        key = (direction, reducer, features)
        if key not in self._scratch_sizes:
            size = ctypes.c_uint64()
            _native.check(_native.lib().tgb_csr_plan_scratch_bytes(
                self._handle, direction, reducer, features, _native.DTYPE_F32, ctypes.byref(size)),
                "tgb_csr_plan_scratch_bytes")
            self._scratch_sizes[key] = int(size.value)
        return self._scratch_sizes[key]

    def scratch(self, direction: int, reducer: int, features: int):
        size = self.scratch_bytes(direction, reducer, features)
        if size == 0:
            return None, 0, 0
        buffer = torch.empty(size, dtype=torch.uint8, device=self.device)
        return buffer, buffer.data_ptr(), size

    def array(self, which: int) -> torch.Tensor:
        """Copy of one plan array as a tensor (0 row order, 1 transposed
        row_ptr, 2 transposed destinations, 3 transposed edge ids, 4 transposed
        row order)."""
        pointer = ctypes.c_uint64()
        count = ctypes.c_int64()
        _native.check(_native.lib().tgb_csr_plan_array(self._handle, which, ctypes.byref(pointer),
                                                       ctypes.byref(count)), "tgb_csr_plan_array")
        dtype = torch.int64 if which == 1 else torch.int32
        width = 8 if which == 1 else 4
        if count.value == 0:
            return torch.empty(0, dtype=dtype, device=self.device)
        offset = pointer.value - self._persistent.data_ptr()
        view = self._persistent[offset:offset + count.value * width].view(dtype)
        return view.clone()
