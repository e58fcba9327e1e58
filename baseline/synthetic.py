"""Seeded synthetic inputs with the shapes of the benchmark configurations.

Everything is generated with integer torch ops from a counter-based hash, so
the CPU and the GPU produce bit-identical graphs for the same seed.  The
R-MAT generator follows the published recursive-quadrant definition
(probabilities a, b, c, d for the (0,0), (0,1), (1,0), (1,1) quadrants of the
(source, destination) bit pair at every level); by default no vertex
relabelling, so hubs sit at low ids (`relabel=True` permutes the ids).  These graphs stand in for the Graph500-style cases the
reference only plans (benchmarks/large_graphs/suite.json of the reference);
no external generator or data set is used.
"""
from __future__ import annotations

import torch

_MASK63 = (1 << 63) - 1


def _mix(x: torch.Tensor) -> torch.Tensor:
    """splitmix64-style finaliser on int64 tensors (wrapping arithmetic)."""
    def lsr(v, s):
        return (v >> s) & ((1 << (64 - s)) - 1)

    x = x + (-7046029254386353131)            # 0x9E3779B97F4A7C15 as signed
    x = (x ^ lsr(x, 30)) * (-4658895280553007687)   # 0xBF58476D1CE4E5B9
    x = (x ^ lsr(x, 27)) * (-7723592293110705685)   # 0x94D049BB133111EB
    return x ^ lsr(x, 31)


def uniform_u16(seed: int, counter: torch.Tensor, stream: int) -> torch.Tensor:
    """Four 16-bit uniform integers per counter value: returns [4, n] int64."""
    salt = ((seed * 1000003 + stream) * 2654435761) & _MASK63
    h = _mix(_mix(counter + salt))
    return torch.stack([(h >> (16 * k)) & 0xFFFF for k in range(4)])


def rmat_edges(scale: int, num_edges: int, *, seed: int = 1, a=0.57, b=0.19, c=0.19, d=0.05, device="cpu",
               chunk: int = 1 << 24):
    """Directed R-MAT edge list (src, dst) as int64 tensors of length num_edges."""
    srcs, dsts = [], []
    for start in range(0, num_edges, chunk):
        src, dst = _rmat_chunk(scale, start, min(chunk, num_edges - start), seed, device, a=a, b=b, c=c)
        srcs.append(src)
        dsts.append(dst)
    return torch.cat(srcs), torch.cat(dsts)


def _rmat_chunk(scale: int, start: int, n: int, seed: int, device, *, a=0.57, b=0.19, c=0.19):
    """Edges start .. start+n-1 of the stream (each edge has its own counter, so any slice of the
    stream can be generated alone)."""
    ta = int(round(a * 65536))
    tb = ta + int(round(b * 65536))
    tc = tb + int(round(c * 65536))
    counter = torch.arange(start, start + n, dtype=torch.int64, device=device)
    src = torch.zeros(n, dtype=torch.int64, device=device)
    dst = torch.zeros(n, dtype=torch.int64, device=device)
    for level in range(scale):
        if level % 4 == 0:
            draws = uniform_u16(seed, counter, level // 4)
        r = draws[level % 4]
        src_bit = (r >= tb).to(torch.int64)                      # quadrants c, d
        dst_bit = (((r >= ta) & (r < tb)) | (r >= tc)).to(torch.int64)  # quadrants b, d
        src = (src << 1) | src_bit
        dst = (dst << 1) | dst_bit
    return src, dst


def csr_from_pairs(src: torch.Tensor, dst: torch.Tensor, num_nodes: int, *, symmetrize: bool, dedup: bool = True):
    """CSR by destination, sources ascending inside a row.  Self loops are kept
    as generated."""
    if symmetrize:
        src, dst = torch.cat((src, dst)), torch.cat((dst, src))
    key = dst * num_nodes + src
    key = torch.unique(key) if dedup else torch.sort(key).values
    dst = key // num_nodes
    src = key - dst * num_nodes
    counts = torch.bincount(dst, minlength=num_nodes)
    row_ptr = torch.zeros(num_nodes + 1, dtype=torch.int64, device=key.device)
    torch.cumsum(counts, 0, out=row_ptr[1:])
    return row_ptr, src


def random_relabelling(num_nodes: int, *, seed: int, device="cpu") -> torch.Tensor:
    """A seeded random permutation of the vertex ids (new id of old id i is
    perm[i]): the order of a 63-bit hash of the ids, ties broken by id."""
    ids = torch.arange(num_nodes, dtype=torch.int64, device=device)
    key = _mix(ids + ((seed * 2862933555777941757 + 3037000493) & _MASK63)) & _MASK63
    order = torch.argsort(key, stable=True)
    perm = torch.empty_like(order)
    perm[order] = ids
    return perm


def rmat_csr(scale: int, edge_factor: int, *, seed: int = 1, symmetrize: bool = True, device="cpu",
             relabel: bool = False):
    """R-MAT graph as CSR by destination.  `relabel=True` applies the random
    vertex relabelling that Graph500-style generators prescribe, which spreads
    the hubs over the whole id range (contiguous id ranges then hold the same
    mix of degrees); the default keeps the generator's natural ids."""
    n = 1 << scale
    src, dst = rmat_edges(scale, n * edge_factor, seed=seed, device=device)
    if relabel:
        perm = random_relabelling(n, seed=seed, device=device)
        src, dst = perm[src], perm[dst]
    return csr_from_pairs(src, dst, n, symmetrize=symmetrize)


def rmat_csr_rows(scale: int, edge_factor: int, first_row: int, last_row: int, *, seed: int = 1,
                  symmetrize: bool = True, relabel: bool = False, device="cpu", chunk: int = 1 << 24,
                  fold_limit: int = 1_300_000_000):
    """Rows [first_row, last_row) of the graph `rmat_csr` builds for the same arguments, without
    ever holding the whole graph: the edge stream is generated chunk by chunk, every chunk is
    symmetrised and filtered to destinations in the range, and the survivors are sorted and
    de-duplicated at the end.  Returns (row_ptr of the range starting at 0, global source ids)."""
    n = 1 << scale
    perm = random_relabelling(n, seed=seed, device=device) if relabel else None
    rows = last_row - first_row
    kept, pending = [], 0
    total = n * edge_factor
    for start in range(0, total, chunk):
        count = min(chunk, total - start)
        src, dst = _rmat_chunk(scale, start, count, seed, device)
        if perm is not None:
            src, dst = perm[src], perm[dst]
        pairs = ((src, dst), (dst, src)) if symmetrize else ((src, dst),)
        for s, d in pairs:
            mask = (d >= first_row) & (d < last_row)
            kept.append((d[mask] - first_row) * n + s[mask])
        pending += sum(int(piece.numel()) for piece in kept[-len(pairs):])
        if pending > fold_limit:     # bound the memory of the pending pieces: fold them into one unique list
            kept = [torch.unique(torch.cat(kept))]
            pending = int(kept[0].numel())
    key = torch.unique(torch.cat(kept)) if kept else torch.zeros(0, dtype=torch.int64, device=device)
    del kept
    dst = key // n
    src = key - dst * n
    counts = torch.bincount(dst, minlength=rows)
    row_ptr = torch.zeros(rows + 1, dtype=torch.int64, device=key.device)
    torch.cumsum(counts, 0, out=row_ptr[1:])
    return row_ptr, src


def gcn_norm_weights_rows(row_ptr: torch.Tensor, col_idx: torch.Tensor, degree: torch.Tensor,
                          first_row: int) -> torch.Tensor:
    """`gcn_norm_weights` for a block of rows: `degree` holds the row lengths of the WHOLE graph
    (global ids), `row_ptr` / `col_idx` the block starting at global row `first_row`."""
    lengths = row_ptr[1:] - row_ptr[:-1]
    deg = degree.to(torch.float32)
    dst = torch.repeat_interleave(torch.arange(lengths.numel(), device=row_ptr.device), lengths) + first_row
    return torch.rsqrt(deg[dst] * deg[col_idx])


def normal_rows(first_row: int, last_row: int, width: int, *, seed: int, device="cpu", std: float = 1.0,
                ids: torch.Tensor | None = None) -> torch.Tensor:
    """Rows of a conceptually unbounded N(0, std^2) feature matrix addressed by GLOBAL row id:
    row i is the same on every rank and every device (Box-Muller on the counter hash), so a rank
    can produce the features of its own rows, and a checker those of any remote row, without the
    others.  `ids` (int64) selects arbitrary rows instead of the range."""
    if ids is None:
        ids = torch.arange(first_row, last_row, dtype=torch.int64, device=device)
    ids = ids.to(device)
    out = torch.empty((ids.numel(), width), dtype=torch.float32, device=device)
    salt = ((seed * 1000003 + 77) * 2654435761) & _MASK63
    columns = torch.arange(width, dtype=torch.int64, device=device)[None, :]
    block = max((1 << 24) // max(width, 1), 1)          # bounds the float64 temporaries
    for start in range(0, ids.numel(), block):
        part = ids[start:start + block]
        h = _mix(_mix(part[:, None] * width + columns + salt))
        u1 = (((h >> 11) & ((1 << 24) - 1)).to(torch.float64) + 1.0) / float(1 << 24)     # (0, 1]
        u2 = ((h >> 35) & ((1 << 24) - 1)).to(torch.float64) / float(1 << 24)             # [0, 1)
        z = torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(2.0 * torch.pi * u2)
        out[start:start + block] = (z * std).to(torch.float32)
    return out


def gcn_norm_weights(row_ptr: torch.Tensor, col_idx: torch.Tensor) -> torch.Tensor:
    """Symmetric GCN normalisation 1/sqrt(deg_i * deg_j), deg = CSR row length."""
    deg = (row_ptr[1:] - row_ptr[:-1]).to(torch.float32)
    dst = torch.repeat_interleave(torch.arange(deg.numel(), device=row_ptr.device), (row_ptr[1:] - row_ptr[:-1]))
    return torch.rsqrt(deg[dst] * deg[col_idx])


def normal(shape, *, seed: int, device="cpu", dtype=torch.float32, std: float = 1.0):
    """N(0, std^2) values from a seeded CPU-or-GPU generator of that device."""
    gen = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std).to(dtype)


def fixed_degree_graph(num_nodes: int, degree: int, *, seed: int = 1234, device="cpu"):
    """Config-1 shape: exactly `degree` in-edges per row, uniform random sources."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    row_ptr = torch.arange(0, num_nodes * degree + 1, degree, dtype=torch.int64)
    col_idx = torch.randint(0, num_nodes, (num_nodes * degree,), generator=gen, dtype=torch.int64)
    return row_ptr.to(device), col_idx.to(device)
