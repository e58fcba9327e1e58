"""ctypes/numpy front end of the CPU oracle (TEST INFRASTRUCTURE, not product).

Loads ``oracle/libtiga_oracle.so`` (built from ``oracle/tiga_oracle.c`` by
``make -C oracle``) and exposes each restated reference algorithm on numpy
arrays.  Only tests, the smoke check and the CPU-baseline legs of the
benchmark import this module; the product package never does.

The citations of the reference files each function follows live next to the C
code.  ``build()`` compiles the library when it is missing.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libtiga_oracle.so")
_lib = None

_i64p = ctypes.POINTER(ctypes.c_int64)
_f32p = ctypes.POINTER(ctypes.c_float)
_u16p = ctypes.POINTER(ctypes.c_uint16)


def build(force: bool = False) -> str:
    """Compile the C oracle (and the reference runtime when it is present)."""
    if force or not os.path.exists(_LIB_PATH) or (
            os.path.getmtime(_LIB_PATH)
            < max(os.path.getmtime(os.path.join(_HERE, name))
                  for name in ("tiga_oracle.c", "tiga_geometry_oracle.c"))):
        subprocess.run(["make", "-C", _HERE], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.orc_destination_owner.restype = ctypes.c_int64
        _lib.orc_derive_ghosts.restype = ctypes.c_int64
        _lib.orc_num_threads.restype = ctypes.c_int
        _lib.orc_radius_build.restype = ctypes.c_int64
        _lib.orc_knn_build.restype = ctypes.c_int32
    return _lib


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(ctypes.c_int(int(n)))


def _i64(a):
    a = np.ascontiguousarray(a, dtype=np.int64)
    return a, a.ctypes.data_as(_i64p)


def _f32(a):
    if a is None:
        return None, None
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_f32p)


def _u16(a):
    a = np.ascontiguousarray(a, dtype=np.uint16)
    return a, a.ctypes.data_as(_u16p)


def _c64(v):
    return ctypes.c_int64(int(v))


# ----------------------------------------------------------------- CSR build
def coo_to_csr(src, dst, num_dst):
    src, psrc = _i64(src)
    dst, pdst = _i64(dst)
    E = src.size
    row_ptr = np.zeros(num_dst + 1, np.int64)
    col = np.zeros(E, np.int64)
    order = np.zeros(E, np.int64)
    rc = lib().orc_coo_to_csr(psrc, pdst, _c64(E), _c64(num_dst),
                              row_ptr.ctypes.data_as(_i64p),
                              col.ctypes.data_as(_i64p),
                              order.ctypes.data_as(_i64p))
    if rc:
        raise ValueError("dst contains an out-of-range destination index")
    return row_ptr, col, order


def destination_index(row_ptr):
    row_ptr, p = _i64(row_ptr)
    N = row_ptr.size - 1
    out = np.zeros(int(row_ptr[-1]), np.int64)
    lib().orc_destination_index(p, _c64(N), out.ctypes.data_as(_i64p))
    return out


def csr_transpose(row_ptr, col_idx, num_src):
    row_ptr, prow = _i64(row_ptr)
    col_idx, pcol = _i64(col_idx)
    N = row_ptr.size - 1
    E = col_idx.size
    t_ptr = np.zeros(num_src + 1, np.int64)
    t_col = np.zeros(E, np.int64)
    order = np.zeros(E, np.int64)
    rc = lib().orc_csr_transpose(prow, pcol, _c64(N), _c64(num_src),
                                 t_ptr.ctypes.data_as(_i64p),
                                 t_col.ctypes.data_as(_i64p),
                                 order.ctypes.data_as(_i64p))
    if rc:
        raise ValueError("col_idx contains an out-of-range source index")
    return t_ptr, t_col, order


def degree_stats(row_ptr):
    row_ptr, p = _i64(row_ptr)
    stats = np.zeros(3, np.int64)
    lib().orc_degree_stats(p, _c64(row_ptr.size - 1),
                           stats.ctypes.data_as(_i64p))
    return int(stats[0]), int(stats[1]), int(stats[2])


# --------------------------------------------------------------- sum / mean
def _as_2d(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    return x.reshape(x.shape[0], -1), x.shape


def wsum_fwd(row_ptr, col_idx, x, w=None, identity=0.0, mean=False):
    row_ptr, prow = _i64(row_ptr)
    col_idx, pcol = _i64(col_idx)
    x2, shape = _as_2d(x)
    N, F = row_ptr.size - 1, x2.shape[1]
    w, pw = _f32(None if w is None else np.asarray(w).reshape(-1))
    out = np.zeros((N, F), np.float32)
    lib().orc_csr_wsum_fwd_f32(prow, pcol, _c64(N), x2.ctypes.data_as(_f32p),
                               _c64(F), pw, ctypes.c_float(identity),
                               ctypes.c_int(int(mean)),
                               out.ctypes.data_as(_f32p))
    return out.reshape((N,) + tuple(shape[1:]))


def wsum_bwd_dx(row_ptr, col_idx, num_src, dy, w=None, mean=False):
    row_ptr, prow = _i64(row_ptr)
    col_idx, pcol = _i64(col_idx)
    dy2, shape = _as_2d(dy)
    N, F = row_ptr.size - 1, dy2.shape[1]
    w, pw = _f32(None if w is None else np.asarray(w).reshape(-1))
    dx = np.zeros((num_src, F), np.float32)
    rc = lib().orc_csr_wsum_bwd_dx_f32(prow, pcol, _c64(N), _c64(num_src),
                                       dy2.ctypes.data_as(_f32p), _c64(F), pw,
                                       ctypes.c_int(int(mean)),
                                       dx.ctypes.data_as(_f32p))
    if rc:
        raise ValueError("invalid CSR")
    return dx.reshape((num_src,) + tuple(shape[1:]))


def wsum_bwd_dx_pre(row_ptr, t_ptr, t_col, order, num_src, dy, w=None, mean=False):
    """dx with a transposed relation built beforehand by csr_transpose."""
    row_ptr, prow = _i64(row_ptr)
    t_ptr, ptp = _i64(t_ptr)
    t_col, ptc = _i64(t_col)
    order, por = _i64(order)
    dy2, shape = _as_2d(dy)
    F = dy2.shape[1]
    w, pw = _f32(None if w is None else np.asarray(w).reshape(-1))
    dx = np.zeros((num_src, F), np.float32)
    lib().orc_csr_wsum_bwd_dx_pre_f32(prow, ptp, ptc, por, _c64(num_src), dy2.ctypes.data_as(_f32p), _c64(F), pw,
                                      ctypes.c_int(int(mean)), dx.ctypes.data_as(_f32p))
    return dx.reshape((num_src,) + tuple(shape[1:]))


def wsum_bwd_dw(row_ptr, col_idx, dy, x, mean=False):
    row_ptr, prow = _i64(row_ptr)
    col_idx, pcol = _i64(col_idx)
    dy2, _ = _as_2d(dy)
    x2, _ = _as_2d(x)
    N, F = row_ptr.size - 1, x2.shape[1]
    dw = np.zeros(col_idx.size, np.float32)
    lib().orc_csr_wsum_bwd_dw_f32(prow, pcol, _c64(N),
                                  dy2.ctypes.data_as(_f32p),
                                  x2.ctypes.data_as(_f32p), _c64(F),
                                  ctypes.c_int(int(mean)),
                                  dw.ctypes.data_as(_f32p))
    return dw


# ------------------------------------------------------------------ product
def product_fwd(row_ptr, message):
    """out[i] = product of the rows ``message[row_ptr[i]:row_ptr[i+1]]`` (1 for a row without edges)."""
    row_ptr, prow = _i64(row_ptr)
    m2, shape = _as_2d(message)
    N, F = row_ptr.size - 1, m2.shape[1]
    out = np.zeros((N, F), np.float32)
    lib().orc_csr_product_fwd_f32(prow, _c64(N), m2.ctypes.data_as(_f32p), _c64(F), out.ctypes.data_as(_f32p))
    return out.reshape((N,) + tuple(shape[1:]))


def product_vjp(row_ptr, message, dy):
    """Cotangent of every message: dy[row] times the product of the row's other messages."""
    row_ptr, prow = _i64(row_ptr)
    m2, shape = _as_2d(message)
    dy2, _ = _as_2d(dy)
    N, F = row_ptr.size - 1, m2.shape[1]
    grad = np.zeros_like(m2)
    lib().orc_csr_product_vjp_f32(prow, _c64(N), m2.ctypes.data_as(_f32p), _c64(F), dy2.ctypes.data_as(_f32p),
                                  grad.ctypes.data_as(_f32p))
    return grad.reshape(shape)


# ---------------------------------------------------------------------- max
def max_fwd(row_ptr, col_idx, x, w=None, identity=-np.inf):
    row_ptr, prow = _i64(row_ptr)
    col_idx, pcol = _i64(col_idx)
    x2, shape = _as_2d(x)
    N, F = row_ptr.size - 1, x2.shape[1]
    w, pw = _f32(None if w is None else np.asarray(w).reshape(-1))
    out = np.zeros((N, F), np.float32)
    arg = np.zeros((N, F), np.int64)
    lib().orc_csr_max_fwd_f32(prow, pcol, _c64(N), x2.ctypes.data_as(_f32p),
                              _c64(F), pw, ctypes.c_float(identity),
                              out.ctypes.data_as(_f32p),
                              arg.ctypes.data_as(_i64p))
    tail = tuple(shape[1:])
    return out.reshape((N,) + tail), arg.reshape((N,) + tail)


def max_bwd(row_ptr, col_idx, num_src, dy, x, argmax, w=None):
    row_ptr, prow = _i64(row_ptr)
    col_idx, pcol = _i64(col_idx)
    dy2, _ = _as_2d(dy)
    x2, shape = _as_2d(x)
    N, F = row_ptr.size - 1, x2.shape[1]
    w, pw = _f32(None if w is None else np.asarray(w).reshape(-1))
    arg, parg = _i64(np.asarray(argmax).reshape(N, F))
    dx = np.zeros((num_src, F), np.float32)
    dw = np.zeros(col_idx.size, np.float32)
    lib().orc_csr_max_bwd_f32(prow, pcol, _c64(N), _c64(num_src),
                              dy2.ctypes.data_as(_f32p),
                              x2.ctypes.data_as(_f32p), _c64(F), pw, parg,
                              dx.ctypes.data_as(_f32p),
                              dw.ctypes.data_as(_f32p))
    return dx.reshape((num_src,) + tuple(shape[1:])), dw


# ----------------------------------------------------------- online softmax
def online_softmax_fwd(row_ptr, score, value):
    """score [E,H] (or [E]), value [E,H,D] (or [E,D] / [E]) float32."""
    row_ptr, prow = _i64(row_ptr)
    score = np.ascontiguousarray(score, dtype=np.float32)
    value = np.ascontiguousarray(value, dtype=np.float32)
    E = score.shape[0]
    H = int(np.prod(score.shape[1:])) if score.ndim > 1 else 1
    D = int(value.size // max(E * H, 1)) if E else int(
        np.prod(value.shape[score.ndim:]))
    N = row_ptr.size - 1
    out = np.zeros((N, H, D), np.float32)
    m = np.zeros((N, H), np.float32)
    l = np.zeros((N, H), np.float32)
    lib().orc_online_softmax_fwd_f32(prow, _c64(N),
                                     score.ctypes.data_as(_f32p),
                                     value.ctypes.data_as(_f32p), _c64(H),
                                     _c64(D), out.ctypes.data_as(_f32p),
                                     m.ctypes.data_as(_f32p),
                                     l.ctypes.data_as(_f32p))
    return out.reshape((N,) + tuple(value.shape[1:])), m, l


def online_softmax_bwd(row_ptr, score, value, out, dout):
    row_ptr, prow = _i64(row_ptr)
    score = np.ascontiguousarray(score, dtype=np.float32)
    value = np.ascontiguousarray(value, dtype=np.float32)
    out = np.ascontiguousarray(out, dtype=np.float32)
    dout = np.ascontiguousarray(dout, dtype=np.float32)
    E = score.shape[0]
    H = int(np.prod(score.shape[1:])) if score.ndim > 1 else 1
    D = int(value.size // max(E * H, 1))
    N = row_ptr.size - 1
    dscore = np.zeros_like(score)
    dvalue = np.zeros_like(value)
    lib().orc_online_softmax_bwd_f32(prow, _c64(N),
                                     score.ctypes.data_as(_f32p),
                                     value.ctypes.data_as(_f32p),
                                     out.ctypes.data_as(_f32p),
                                     dout.ctypes.data_as(_f32p), _c64(H),
                                     _c64(D), dscore.ctypes.data_as(_f32p),
                                     dvalue.ctypes.data_as(_f32p))
    return dscore, dvalue


def f32_to_bf16(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.zeros(a.shape, np.uint16)
    lib().orc_f32_to_bf16_array(a.ctypes.data_as(_f32p),
                                out.ctypes.data_as(_u16p), _c64(a.size))
    return out


def bf16_to_f32(a):
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.zeros(a.shape, np.float32)
    lib().orc_bf16_to_f32_array(a.ctypes.data_as(_u16p),
                                out.ctypes.data_as(_f32p), _c64(a.size))
    return out


def gat_fwd(row_ptr, col_idx, x_src, x_dst, a_src, a_dst, slope=0.2):
    """All feature arguments are uint16 bit patterns of bfloat16."""
    row_ptr, prow = _i64(row_ptr)
    col_idx, pcol = _i64(col_idx)
    x_src, pxs = _u16(x_src)
    x_dst, pxd = _u16(x_dst)
    a_src, pas = _u16(a_src)
    a_dst, pad = _u16(a_dst)
    N = row_ptr.size - 1
    H, D = x_src.shape[1], x_src.shape[2]
    out = np.zeros((N, H, D), np.uint16)
    m = np.zeros((N, H), np.float32)
    l = np.zeros((N, H), np.float32)
    score = np.zeros((col_idx.size, H), np.float32)
    lib().orc_gat_fwd_bf16(prow, pcol, _c64(N), pxs, pxd, pas, pad, _c64(H),
                           _c64(D), ctypes.c_float(slope),
                           out.ctypes.data_as(_u16p), m.ctypes.data_as(_f32p),
                           l.ctypes.data_as(_f32p),
                           score.ctypes.data_as(_f32p))
    return out, m, l, score


def gat_bwd(row_ptr, col_idx, x_src, x_dst, a_src, a_dst, dout, slope=0.2):
    row_ptr, prow = _i64(row_ptr)
    col_idx, pcol = _i64(col_idx)
    x_src, pxs = _u16(x_src)
    x_dst, pxd = _u16(x_dst)
    a_src, pas = _u16(a_src)
    a_dst, pad = _u16(a_dst)
    dout, pdo = _u16(dout)
    N = row_ptr.size - 1
    num_src, H, D = x_src.shape
    dxs = np.zeros((num_src, H, D), np.float32)
    dxd = np.zeros((N, H, D), np.float32)
    das = np.zeros((H, D), np.float32)
    dad = np.zeros((H, D), np.float32)
    lib().orc_gat_bwd_bf16(prow, pcol, _c64(N), _c64(num_src), pxs, pxd, pas,
                           pad, _c64(H), _c64(D), ctypes.c_float(slope), pdo,
                           dxs.ctypes.data_as(_f32p),
                           dxd.ctypes.data_as(_f32p),
                           das.ctypes.data_as(_f32p),
                           dad.ctypes.data_as(_f32p))
    return dxs, dxd, das, dad


# ------------------------------------------------------ dense varlen relation
def varlen_attn_fwd(cu_seqlens, q, k, v, scale, causal=True):
    cu, pcu = _i64(cu_seqlens)
    q, pq = _f32(q)
    k, pk = _f32(k)
    v, pv = _f32(v)
    T, H, D = q.shape
    out = np.zeros((T, H, D), np.float32)
    lse = np.zeros((T, H), np.float32)
    lib().orc_varlen_attn_fwd(pcu, _c64(cu.size - 1), pq, pk, pv, _c64(H),
                              _c64(D), ctypes.c_float(scale),
                              ctypes.c_int(int(causal)),
                              out.ctypes.data_as(_f32p),
                              lse.ctypes.data_as(_f32p))
    return out, lse


def varlen_attn_bwd(cu_seqlens, q, k, v, out, dout, scale, causal=True):
    cu, pcu = _i64(cu_seqlens)
    q, pq = _f32(q)
    k, pk = _f32(k)
    v, pv = _f32(v)
    out, po = _f32(out)
    dout, pdo = _f32(dout)
    T, H, D = q.shape
    dq = np.zeros_like(q)
    dk = np.zeros_like(k)
    dv = np.zeros_like(v)
    lib().orc_varlen_attn_bwd(pcu, _c64(cu.size - 1), pq, pk, pv, po, pdo,
                              _c64(H), _c64(D), ctypes.c_float(scale),
                              ctypes.c_int(int(causal)),
                              dq.ctypes.data_as(_f32p),
                              dk.ctypes.data_as(_f32p),
                              dv.ctypes.data_as(_f32p))
    return dq, dk, dv


def linear(a, W):
    a, pa = _f32(a)
    W, pW = _f32(W)
    N, K = a.shape
    J = W.shape[1]
    out = np.zeros((N, J), np.float32)
    lib().orc_linear_f32(pa, pW, _c64(N), _c64(K), _c64(J),
                         out.ctypes.data_as(_f32p))
    return out


# ------------------------------------------------------------- distribution
def owned_range(entities, world, rank):
    b = ctypes.c_int64()
    e = ctypes.c_int64()
    lib().orc_owned_range(_c64(entities), _c64(world), _c64(rank),
                          ctypes.byref(b), ctypes.byref(e))
    return int(b.value), int(e.value)


def destination_owner(entity, entities, world):
    return int(lib().orc_destination_owner(_c64(entity), _c64(entities),
                                           _c64(world)))


def derive_ghosts(row_ptr, col_idx, num_entities, world, rank):
    row_ptr, prow = _i64(row_ptr)
    col_idx, pcol = _i64(col_idx)
    buf = np.zeros(max(col_idx.size, 1), np.int64)
    n = lib().orc_derive_ghosts(prow, pcol, _c64(num_entities), _c64(world),
                                _c64(rank), buf.ctypes.data_as(_i64p))
    return buf[:int(n)].copy()


def local_csr(row_ptr, col_idx, num_entities, world, rank, ghost_ids):
    row_ptr, prow = _i64(row_ptr)
    col_idx, pcol = _i64(col_idx)
    ghosts, pg = _i64(ghost_ids)
    b, e = owned_range(num_entities, world, rank)
    local_ptr = np.zeros(e - b + 1, np.int64)
    local_col = np.zeros(int(row_ptr[e] - row_ptr[b]), np.int64)
    lib().orc_local_csr(prow, pcol, _c64(num_entities), _c64(world),
                        _c64(rank), pg, _c64(ghosts.size),
                        local_ptr.ctypes.data_as(_i64p),
                        local_col.ctypes.data_as(_i64p))
    return local_ptr, local_col


# ------------------------------------------------------- dynamic relations
def _lattice_arguments(lattice, inverse, dims):
    if lattice is None:
        return None, None, None, None
    lattice, pl = _f32(np.asarray(lattice, np.float32).reshape(dims, dims))
    inverse, pi = _f32(np.asarray(inverse, np.float32).reshape(dims, dims))
    return lattice, pl, inverse, pi


def radius_build(positions, cutoff, *, exclude_self=True, lattice=None, inverse=None, extents=None,
                 use_cells=True):
    """Graph.radius -> (row_ptr, col, distance, displacement, candidate_pairs).  `lattice`/`inverse`
    are the [D, D] periodic lattice and its inverse, `extents` the periodic cells per axis."""
    positions, pp = _f32(np.asarray(positions, np.float32))
    n, dims = positions.shape
    cutoff, pc = _f32(np.atleast_1d(np.asarray(cutoff, np.float32)))
    lattice, pl, inverse, pi = _lattice_arguments(lattice, inverse, dims)
    ext, pe = _i64(np.zeros(dims, np.int64) if extents is None else extents)
    row_ptr = np.zeros(n + 1, np.int64)
    pairs = ctypes.c_int64()
    args = (pp, _c64(n), ctypes.c_int32(dims), pc, _c64(cutoff.size), ctypes.c_int32(bool(exclude_self)),
            pl, pi, pe, ctypes.c_int32(bool(use_cells)), row_ptr.ctypes.data_as(_i64p))
    edges = lib().orc_radius_build(*args, None, None, None, ctypes.byref(pairs))
    if edges < 0:
        raise ValueError("orc_radius_build rejected its arguments")
    col = np.zeros(edges, np.int64)
    distance = np.zeros(edges, np.float32)
    displacement = np.zeros((edges, dims), np.float32)
    lib().orc_radius_build(*args, col.ctypes.data_as(_i64p), distance.ctypes.data_as(_f32p),
                           displacement.ctypes.data_as(_f32p), ctypes.byref(pairs))
    return row_ptr, col, distance, displacement, int(pairs.value)


def knn_build(queries, candidates, k, *, exclude_self):
    """Graph.knn -> col [nq, k], ascending by (squared distance, candidate index)."""
    queries, pq = _f32(np.asarray(queries, np.float32))
    candidates, pc = _f32(np.asarray(candidates, np.float32))
    col = np.zeros((queries.shape[0], int(k)), np.int64)
    status = lib().orc_knn_build(pq, _c64(queries.shape[0]), pc, _c64(candidates.shape[0]),
                                 ctypes.c_int32(queries.shape[1]), ctypes.c_int32(int(k)),
                                 ctypes.c_int32(bool(exclude_self)), col.ctypes.data_as(_i64p))
    if status != 0:
        raise ValueError("k out of range for the candidate set")
    return col


def edge_geometry(dst_positions, src_positions, destination, col, *, lattice=None, inverse=None):
    """Graph.implicit_edge_fields -> (displacement [E, D], distance [E])."""
    dst_positions, pd = _f32(np.asarray(dst_positions, np.float32))
    src_positions, ps = _f32(np.asarray(src_positions, np.float32))
    dims = dst_positions.shape[1]
    destination, pdst = _i64(destination)
    col, pcol = _i64(col)
    lattice, pl, inverse, pi = _lattice_arguments(lattice, inverse, dims)
    displacement = np.zeros((col.size, dims), np.float32)
    distance = np.zeros(col.size, np.float32)
    lib().orc_edge_geometry(pd, ps, ctypes.c_int32(dims), pdst, pcol, _c64(col.size), pl, pi,
                            displacement.ctypes.data_as(_f32p), distance.ctypes.data_as(_f32p))
    return displacement, distance
