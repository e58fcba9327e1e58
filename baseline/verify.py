"""In-run verification of the 2-layer halo GCN against the CPU oracle.

Before bench.py times the multi-GPU workload it runs one step whose results
are compared, on every rank, with the CPU oracle on a compacted sub-problem:
a sample of owned rows (ordinary rows, empty rows, split hub rows) with all of
their edges.  The checked quantities are exactly those that depend on rows
that crossed the halo exchange:

  layer 1 aggregate  rows of  A x        x of ghost sources comes from the seeded generator
  layer 2 aggregate  rows of  A h1       h1 of ghost sources is fetched from its owner
  dx of both layers  rows of  A^T d_agg  the graph and its weights are symmetric, so row j of
                                          A^T is row j of A; d_agg of remote rows is fetched
  dw                 per edge of the sampled rows, both layers added (the layers share w)
  the two linears    sampled rows against float64 products; dW against a float64 product
                     reduced over all ranks

Remote rows are fetched through an independent channel (index_select on the
owner, one all-reduce of a zero-padded answer table), never through the halo
runtime or the library's row movers, so an error in those cannot cancel out.

This module is measurement infrastructure: only bench.py imports it, and it is
the one place besides the tests where the oracle is called as a checker.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

EPS32 = float(np.finfo(np.float32).eps)
SPLIT_ROW_DEGREE = 512      # rows above this degree are reduced in segments by the kernels


def excess(got, want, magnitude, *, rtol=1e-5, atol=1e-6, ulps=8) -> float:
    """max(|got - want| - bound) with the float32-sum bound of the parity tests: rel 1e-5 / abs 1e-6
    plus `ulps` float32 ulps of the sum of absolute values of the terms.  <= 0 passes."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    if got.size == 0:
        return -1.0
    bound = rtol * np.abs(want) + atol + ulps * EPS32 * np.asarray(magnitude, np.float64)
    worst = float(np.max(np.abs(got - want) - bound))
    return worst if np.isfinite(worst) else float("inf")


def fetch_rows(owned: torch.Tensor, first_row: int, ids: torch.Tensor, world: int) -> torch.Tensor:
    """Rows `ids` (global, int64, any owner) of a row-partitioned matrix whose block `owned`
    starts at global row `first_row` on this rank."""
    width = owned.shape[1]
    if world == 1:
        return owned.index_select(0, ids - first_row)
    device = owned.device
    count = torch.tensor([ids.numel()], dtype=torch.int64, device=device)
    counts = [torch.empty_like(count) for _ in range(world)]
    dist.all_gather(counts, count)
    most = max(int(c.item()) for c in counts)
    padded = torch.full((most,), -1, dtype=torch.int64, device=device)
    padded[:ids.numel()] = ids
    requests = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(requests, padded)
    answers = torch.zeros((world, most, width), dtype=owned.dtype, device=device)
    for r, wanted in enumerate(requests):
        mine = (wanted >= first_row) & (wanted < first_row + owned.shape[0])
        slots = torch.nonzero(mine).reshape(-1)
        answers[r, slots] = owned.index_select(0, wanted[slots] - first_row)
    dist.all_reduce(answers)          # every row has exactly one owner: the sum adds zeros only
    return answers[dist.get_rank(), :ids.numel()].clone()


def sample_rows(row_ptr: torch.Tensor, *, seed: int, ordinary: int = 40, max_neighbours: int = 200_000):
    """Local row numbers to check: random rows, a few empty rows, and the longest rows that keep the
    sample's neighbour count under `max_neighbours` (split rows included where they fit)."""
    degree = (row_ptr[1:] - row_ptr[:-1]).cpu()
    rows = degree.numel()
    gen = torch.Generator().manual_seed(seed)
    picks = [torch.randint(0, rows, (ordinary,), generator=gen)]
    empty = torch.nonzero(degree == 0).reshape(-1)
    picks.append(empty[:3])
    order = torch.argsort(degree, descending=True)
    budget = max_neighbours - int(degree[picks[0]].clamp(max=4096).sum())
    hubs = []
    for r in order[:64].tolist():
        d = int(degree[r])
        if d <= budget // 2 and len(hubs) < 3:
            hubs.append(r)
            budget -= d
    picks.append(torch.tensor(hubs, dtype=torch.int64))
    chosen = torch.unique(torch.cat(picks))
    chosen = chosen[degree[chosen] <= max(max_neighbours // 4, 4096)]
    return chosen


def check_two_layer_gcn(oracle, *, row_ptr, col_idx, first_row, num_nodes, weight, feature_of, tensors,
                        linears, world, seed=7) -> dict:
    """Compare one step's results with the oracle on sampled owned rows.

    row_ptr, col_idx   this rank's rows (row_ptr from 0, global source ids), on the device
    weight             per-edge weights of those rows
    feature_of(ids)    input features of arbitrary global rows (seeded generator), float32 on CPU
    tensors            dict of this rank's device results: agg1, h1, agg2, out, d_agg1, d_h1, d_agg2,
                       dx, dw, dW1, dW2 (dW already summed over ranks)
    linears            (W1, W2)
    Returns {"rows", "edges", "max_excess", "worst", "ok"}; every rank must call it (collectives inside)."""
    device = row_ptr.device
    rows_local = sample_rows(row_ptr, seed=seed + 13 * (first_row % 9973))
    rp = row_ptr.cpu()
    begins, ends = rp[rows_local], rp[rows_local + 1]
    degree = ends - begins
    sub_ptr = torch.cat((torch.zeros(1, dtype=torch.int64), degree.cumsum(0)))
    if int(sub_ptr[-1]):
        edges = torch.cat([torch.arange(int(b), int(e)) for b, e in zip(begins.tolist(), ends.tolist())])
    else:
        edges = torch.zeros(0, dtype=torch.int64)
    edges_dev = edges.to(device)
    cols = col_idx[edges_dev].to(torch.int64)
    sub_w = weight.detach()[edges_dev].cpu().numpy()
    unique_cols, compact = torch.unique(cols, return_inverse=True)
    sub_col = compact.cpu().numpy()
    sub_ptr_np = sub_ptr.numpy()
    n_compact = int(unique_cols.numel())
    rows_dev = rows_local.to(device)
    W1, W2 = (w.detach() for w in linears)

    def rows_of(name):
        return tensors[name].detach().index_select(0, rows_dev).cpu().numpy()

    results = {}
    abs_w = np.abs(sub_w)

    split = (degree > SPLIT_ROW_DEGREE).numpy()
    starts = sub_ptr_np[:-1][degree.numpy() > 0]

    def aggregate_check(name, table):
        """rows of A @ table against the oracle; `table` holds the compacted neighbour rows.
        Rows the kernels split into segments (hubs) are compared with the float64 sum of the same
        float32 products instead: the oracle adds a row's terms one after the other in float32, and
        over 10^4..10^6 same-signed terms that order alone carries about sqrt(n) ulps of rounding,
        more than the tolerance; the kernel's segment tree does not follow it."""
        want = oracle.wsum_fwd(sub_ptr_np, sub_col, table, sub_w).astype(np.float64)
        magnitude = oracle.wsum_fwd(sub_ptr_np, sub_col, np.abs(table), abs_w)
        if split.any():
            products = (sub_w[:, None] * table[sub_col]).astype(np.float64)     # float32 products, as the kernel forms them
            sums = np.zeros_like(want)
            sums[degree.numpy() > 0] = np.add.reduceat(products, starts, axis=0)
            want[split] = sums[split]
        results[name] = excess(rows_of(name), want, magnitude)

    # forward, layer 1: neighbours' input features come from the generator, owned or not
    x_table = feature_of(unique_cols.cpu()).numpy()
    aggregate_check("agg1", x_table)
    # forward, layer 2: neighbours' hidden rows are fetched from their owners
    h1_table = fetch_rows(tensors["h1"].detach(), first_row, unique_cols, world).cpu().numpy()
    aggregate_check("agg2", h1_table)
    # backward: A is symmetric with symmetric weights, so (A^T g)[j] = sum over row j of w * g[col]
    d_agg2_table = fetch_rows(tensors["d_agg2"].detach(), first_row, unique_cols, world).cpu().numpy()
    d_agg1_table = fetch_rows(tensors["d_agg1"].detach(), first_row, unique_cols, world).cpu().numpy()
    for name, table in (("d_h1", d_agg2_table), ("dx", d_agg1_table)):
        aggregate_check(name, table)
    # dw of the sampled rows' edges: <d_agg1[i], x[j]> + <d_agg2[i], h1[j]>
    d1_rows, d2_rows = rows_of("d_agg1"), rows_of("d_agg2")
    want_dw = (oracle.wsum_bwd_dw(sub_ptr_np, sub_col, d1_rows, x_table)
               + oracle.wsum_bwd_dw(sub_ptr_np, sub_col, d2_rows, h1_table))
    magnitude = (oracle.wsum_bwd_dw(sub_ptr_np, sub_col, np.abs(d1_rows), np.abs(x_table))
                 + oracle.wsum_bwd_dw(sub_ptr_np, sub_col, np.abs(d2_rows), np.abs(h1_table)))
    results["dw"] = excess(tensors["dw"].detach()[edges_dev].cpu().numpy(), want_dw, magnitude)
    # the linears on the sampled rows, in float64 (tensor-core 3xTF32 products: 4 more ulps of sum |a w|)
    for out_name, in_name, matrix in (("h1", "agg1", W1), ("out", "agg2", W2)):
        a = rows_of(in_name).astype(np.float64)
        m = matrix.cpu().numpy().astype(np.float64)
        results[f"linear {out_name}"] = excess(rows_of(out_name), a @ m, np.abs(a) @ np.abs(m), ulps=12)
    for out_name, in_name, matrix in (("d_agg1", "d_h1", W1),):
        g = rows_of(in_name).astype(np.float64)
        m = matrix.cpu().numpy().astype(np.float64).T
        results[f"linear {out_name}"] = excess(rows_of(out_name), g @ m, np.abs(g) @ np.abs(m), ulps=12)
    # dW = a^T @ g over all rows of all ranks, against float64 on the device
    for name, a_name, g_name in (("dW1", "agg1", "d_h1"), ("dW2", "agg2", None)):
        a = tensors[a_name].detach().double()
        g = tensors[g_name].detach().double() if g_name else torch.ones(
            (a.shape[0], W2.shape[1]), dtype=torch.float64, device=device)
        want = a.t() @ g
        magnitude = a.abs().t() @ g.abs()
        if world > 1:
            dist.all_reduce(want)
            dist.all_reduce(magnitude)
        results[name] = excess(tensors[name].detach().cpu().numpy(), want.cpu().numpy(), magnitude.cpu().numpy(),
                               ulps=64)
    worst = max(results, key=results.get)
    return {"rows": int(rows_local.numel()), "edges": int(edges.numel()), "neighbour_rows": n_compact,
            "max_excess": float(results[worst]), "worst": worst, "ok": bool(results[worst] <= 0.0),
            "excess": {k: float(f"{v:.3e}") for k, v in results.items()}}
