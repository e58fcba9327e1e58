"""ctypes binding of libtiga_b200.so (the C ABI declared in include/tiga_b200.h).

The reference binds its native runtime the same way: a ctypes ``CDLL`` of a
C-ABI shared library located through an environment variable or next to the
package (python/tiga/runtime/__init__.py:104-168 of walkerchi/TIGA-lang), and
turns every non-zero status into ``RuntimeError(f"{op} failed: {message}")``
(python/tiga/runtime/__init__.py:279-284).

There is no fallback: if the library is missing the import of this module's
``lib()`` raises, and every GPU entry point of the package fails with it.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_DEFAULT = os.path.join(_HERE, "_native", "libtiga_b200.so")
_lib = None

OK, INVALID_ARGUMENT, UNSUPPORTED, OUT_OF_MEMORY, INTERNAL = range(5)
DTYPE_F32, DTYPE_BF16 = 0, 1
REDUCER_SUM, REDUCER_MEAN, REDUCER_MAX = 0, 1, 2
PLAN_FORWARD, PLAN_TRANSPOSE = 1, 2
REDUCE_ACCUMULATE = 1

_u64 = ctypes.c_uint64
_i64 = ctypes.c_int64
_i32 = ctypes.c_int32
_f32 = ctypes.c_float
_vp = ctypes.c_void_p

# name -> (restype, argtypes); mirrors include/tiga_b200.h one to one
_SIGNATURES = {
    "tgb_status_string": (ctypes.c_char_p, [_i32]),
    "tgb_last_error": (ctypes.c_char_p, []),
    "tgb_version": (ctypes.c_char_p, []),
    "tgb_launch_count": (_i64, []),
    "tgb_mirror_word": (_i32, [_vp, _vp, _u64]),
    "tgb_csr_plan_sizes": (_i32, [_i64, _i64, _i64, _i32, _i32, ctypes.POINTER(_u64), ctypes.POINTER(_u64)]),
    "tgb_csr_plan_create": (_i32, [_vp, _vp, _i64, _i64, _i64, _i32, _i32, _vp, _u64, _vp, _u64, _u64,
                                   ctypes.POINTER(_vp)]),
    "tgb_csr_plan_destroy": (_i32, [_vp]),
    "tgb_csr_plan_set_edge_map": (_i32, [_vp, _vp, _u64]),
    "tgb_csr_plan_info": (_i32, [_vp, ctypes.POINTER(_i64)]),
    "tgb_csr_plan_array": (_i32, [_vp, _i32, ctypes.POINTER(_u64), ctypes.POINTER(_i64)]),
    "tgb_csr_plan_scratch_bytes": (_i32, [_vp, _i32, _i32, _i64, _i32, ctypes.POINTER(_u64)]),
    "tgb_csr_reduce_fwd": (_i32, [_vp, _i32, _vp, _vp, _vp, _vp, _i64, _i32, _f32, _i32, _vp, _u64, _u64]),
    "tgb_csr_reduce_bwd_dx": (_i32, [_vp, _i32, _vp, _vp, _vp, _vp, _i64, _i32, _vp, _u64, _u64]),
    "tgb_csr_reduce_bwd_dw": (_i32, [_vp, _i32, _vp, _vp, _vp, _vp, _i64, _i32, _vp, _u64, _u64]),
    "tgb_csr_transposed_weights": (_i32, [_vp, _vp, _vp, _u64]),
    "tgb_csr_wsum_fwd_noalloc": (_i32, [_vp, _vp, _vp, _vp, _i64, _f32, _u64]),
    "tgb_rows_gather": (_i32, [_vp, _vp, _vp, _i64, _i64, _u64]),
    "tgb_rows_scatter_add": (_i32, [_vp, _vp, _vp, _i64, _i64, _u64]),
    "tgb_varlen_attn_fwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _i32, _f32, _i32, _vp, _u64]),
    "tgb_varlen_attn_bwd": (_i32, [_vp] * 12 + [_i64, _i64, _i64, _i32, _i32, _i32, _f32, _i32, _vp, _u64]),
    "tgb_linear_f32": (_i32, [_vp, _vp, _vp, _i64, _i32, _i32, _vp, _u64]),
    "tgb_linear_dw_f32": (_i32, [_vp, _vp, _vp, _vp, _u64, _i64, _i32, _i32, _vp, _u64]),
    "tgb_linear_dw_partials": (_i32, [_i64, ctypes.POINTER(_i32)]),
    "tgb_gat_node_scores": (_i32, [_vp, _vp, _i64, _i32, _i32, _vp, _u64]),
    "tgb_gat_scratch_bytes": (_i32, [_vp, _i32, _i32, _i32, ctypes.POINTER(_u64)]),
    "tgb_gat_fwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _f32, _vp, _u64, _u64]),
    "tgb_gat_bwd": (_i32, [_vp] * 11 + [_i32, _i32, _f32, _vp, _vp, _vp, _vp, _vp, _u64, _u64]),
    "tgb_selftest_bounded_wait": (_i32, [_vp, ctypes.c_uint32, _vp, _u64]),
    "tgb_softmax_field_fwd": (_i32, [_vp, _vp, _vp, _i32, _vp, _vp, _vp, _i32, _i32, _u64]),
    "tgb_softmax_field_bwd": (_i32, [_vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _vp, _vp, _vp, _u64]),
    "tgb_peer_export": (_i32, [_vp, _vp, ctypes.POINTER(_u64)]),
    "tgb_peer_open": (_i32, [_vp, ctypes.POINTER(_u64)]),
    "tgb_peer_close": (_i32, [_u64]),
    "tgb_peer_copy": (_i32, [_u64, _vp, _u64, _u64]),
    "tgb_cell_directory_sizes": (_i32, [_i64, _i32, ctypes.POINTER(_u64), ctypes.POINTER(_u64)]),
    "tgb_cell_directory_build": (_i32, [_vp, _i64, _vp, _vp, _u64, _vp, _u64, _u64]),
    "tgb_radius_row_ptr": (_i32, [_vp, _i64, _vp, _vp, _f32, _i32, _vp, _vp, _vp, _u64, _u64]),
    "tgb_radius_fill": (_i32, [_vp, _i64, _vp, _vp, _f32, _i32, _vp, _vp, _vp, _vp, _u64]),
    "tgb_radius_wsum_fwd": (_i32, [_vp, _i64, _vp, _vp, _f32, _i32, _i32, _vp, _i64, _vp, _u64]),
    "tgb_radius_wsum_bwd_pos": (_i32, [_vp, _i64, _vp, _vp, _f32, _i32, _vp, _vp, _i64, _vp, _u64]),
    "tgb_knn": (_i32, [_vp, _i64, _vp, _i64, _i32, _i32, _i32, _vp, _vp, _u64]),
    "tgb_knn_grid": (_i32, [_vp, _i64, _vp, _i64, _vp, _vp, _i32, _i32, _i32, _f32, _vp, _vp, _vp, _u64]),
    "tgb_edge_geometry": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp, _vp, _u64]),
    "tgb_edge_program_fwd": (_i32, [_vp, _vp, _vp, _i32, _f32, _vp, _vp, _vp, _u64]),
    "tgb_edge_program_bwd_rows": (_i32, [_vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _u64]),
    "tgb_edge_program_bwd_sources": (_i32, [_vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _u64]),
    "tgb_edge_algebra_fwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _u64]),
    "tgb_edge_algebra_bwd_messages": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _u64]),
    "tgb_edge_algebra_bwd_rows": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _u64]),
    "tgb_edge_algebra_bwd_sources": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _u64]),
    "tgb_column_sum": (_i32, [_vp, _i64, _i64, _vp, _u64]),
    "tgb_jit_build": (_i32, [ctypes.c_char_p, ctypes.POINTER(_vp), ctypes.c_char_p, _i64]),
    "tgb_jit_image_bytes": (_i32, [_vp, ctypes.POINTER(_i64)]),
    "tgb_jit_launch": (_i32, [_vp, ctypes.c_char_p, ctypes.c_uint32, ctypes.c_uint32, _vp, _u64]),
    "tgb_jit_destroy": (None, [_vp]),
    "tgb_edge_program_jit_fwd": (_i32, [_vp, _vp, _vp, _vp, _i32, _f32, _vp, _vp, _vp, _u64]),
    "tgb_edge_program_jit_bwd": (_i32, [_vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _u64]),
    "tgb_edge_algebra_jit_fwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _u64]),
    "tgb_edge_algebra_jit_bwd_messages": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _u64]),
    "tgb_edge_algebra_jit_bwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _u64]),
}


def library_path() -> str:
    return os.environ.get("TIGA_B200_LIBRARY", _DEFAULT)


def exported_symbols() -> tuple[str, ...]:
    return tuple(_SIGNATURES)


def lib() -> ctypes.CDLL:
    """Load the CUDA extension; raises if it has not been built."""
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"tiga-b200 CUDA extension not found at {path}; build it with "
                "`python tiga-lang_b200/build.py` (there is no fallback path)")
        handle = ctypes.CDLL(path)
        for name, (restype, argtypes) in _SIGNATURES.items():
            function = getattr(handle, name)  # AttributeError if a symbol is missing
            function.restype = restype
            function.argtypes = argtypes
        _lib = handle
    return _lib


def check(status: int, operation: str) -> None:
    if status:
        handle = lib()
        message = handle.tgb_last_error().decode() or handle.tgb_status_string(status).decode()
        if status == UNSUPPORTED:
            raise NotImplementedError(f"{operation} failed: {message}")
        if status == OUT_OF_MEMORY:
            raise MemoryError(f"{operation} failed: {message}")
        if status == INVALID_ARGUMENT:
            raise ValueError(f"{operation} failed: {message}")
        raise RuntimeError(f"{operation} failed: {message}")


def launch_count() -> int:
    return int(lib().tgb_launch_count())
