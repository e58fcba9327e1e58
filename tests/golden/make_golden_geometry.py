"""Generate tests/golden/geometry_cases.npz by running the UNMODIFIED reference on the CPU.

    make -C oracle
    python tests/golden/make_golden_geometry.py [--reference /path/to/TIGA-lang]

Covers the dynamic relations that feed the CSR kernels: ``tg.Graph.radius`` (uniform cell list,
all-pairs, periodic boxes, per-destination cutoffs, metric / select callables, exclude_self) and
``tg.Graph.knn`` (self search, bipartite candidates, ties), through the reference's public API:
``resolve_csr()``, ``implicit_edge_fields()``, ``build_info`` and ``kernel.reference(...)`` with
``torch.autograd.grad``.  Inputs and outputs are saved together so that the fixtures replay
without the reference.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def binary_grid_points(n, d, gen, case="uniform"):
    """Coordinates on a 1/64 grid in [-0.5, 0.5): squared distances are exact in float32, so the
    cutoff comparison has no rounding ambiguity, ties at the cutoff included
    (the reference's own protocol, tests/python/test_radius_hash_grid.py:20-28)."""
    p = (torch.rand(n, d, generator=gen) * 64).floor() / 64 - 0.5
    if case == "collisions":
        p[::2] += 64
    if case == "duplicates":
        p[1::2] = p[::2]
    return p


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", default=os.environ.get("TIGA_REFERENCE"))
    args = parser.parse_args()
    if not args.reference:
        sibling = os.path.join(os.path.dirname(ROOT), "reference")
        if not os.path.isdir(sibling):
            raise SystemExit("pass --reference /path/to/TIGA-lang (or set TIGA_REFERENCE)")
        args.reference = sibling
    runtime = os.path.join(ROOT, "oracle", "_ref", "libtiga_runtime.so")
    if not os.path.exists(runtime):
        raise SystemExit("build oracle/_ref first: make -C oracle")
    os.environ["TIGA_RUNTIME_LIBRARY"] = runtime
    sys.dont_write_bytecode = True
    sys.path.insert(0, os.path.join(args.reference, "python"))
    import tiga as tg

    assert os.path.realpath(tg.__file__).startswith(os.path.realpath(args.reference))
    torch.manual_seed(0)
    torch.set_num_threads(1)

    class DistanceSum(tg.MessagePassing):
        reducer = tg.sum()

        def edge(self, src, dst, edge):
            return edge.distance * src.x

    class NeighborSum(tg.MessagePassing):
        reducer = tg.sum()

        def edge(self, src, dst, edge):
            return src.x

    gen = torch.Generator().manual_seed(4321)
    saved = {}

    def save_radius(key, positions, cutoff, **kwargs):
        graph = tg.Graph.radius(positions, cutoff, **kwargs)
        row_ptr, col = graph.resolve_csr()
        fields = graph.implicit_edge_fields(row_ptr, col)
        saved[key + "_pos"] = positions.numpy()
        saved[key + "_cutoff"] = (cutoff.numpy() if isinstance(cutoff, torch.Tensor)
                                  else np.float64(cutoff))
        saved[key + "_row_ptr"] = row_ptr.numpy()
        saved[key + "_col"] = col.numpy()
        saved[key + "_distance"] = fields["distance"].numpy()
        saved[key + "_displacement"] = fields["displacement"].numpy()
        saved[key + "_builder"] = np.array(graph.build_info["builder"])
        saved[key + "_candidate_pairs"] = np.int64(graph.build_info["candidate_pairs"])
        if "periodic" in kwargs and kwargs["periodic"] is not None:
            saved[key + "_periodic"] = kwargs["periodic"].numpy()
        return graph

    # ------------------------------------------------------------- radius, open boundary
    for d in (1, 2, 3):
        for case in ("uniform", "collisions", "duplicates"):
            p = binary_grid_points(160, d, gen, case)
            save_radius(f"radius_grid_d{d}_{case}", p, 0.25)
    p = torch.rand(300, 3, generator=gen)
    save_radius("radius_random_d3", p, 0.2)
    save_radius("radius_random_d3_self", p, 0.2, exclude_self=False)
    p = torch.randn(257, 2, generator=gen)
    save_radius("radius_normal_d2", p, 0.35)
    # degenerate inputs: empty, one point, no pair within the cutoff
    save_radius("radius_empty", torch.empty(0, 3), 0.25)
    save_radius("radius_single", torch.zeros(1, 3), 0.25)
    save_radius("radius_isolated", torch.arange(12, dtype=torch.float32).reshape(4, 3) * 10, 0.25)
    # four dimensions: the reference falls back to all pairs
    save_radius("radius_d4_all_pairs", torch.rand(90, 4, generator=gen), 0.5)
    # per-destination cutoff tensor: all pairs, asymmetric relation
    p = torch.rand(120, 3, generator=gen)
    save_radius("radius_per_dst_cutoff", p, torch.rand(120, generator=gen) * 0.3 + 0.05)

    # ------------------------------------------------------------- radius, periodic boxes
    p = binary_grid_points(200, 3, gen) + 0.5
    save_radius("radius_periodic_box", p, 0.25, periodic=torch.ones(3))
    save_radius("radius_periodic_box_2cells", p, 0.4, periodic=torch.ones(3))
    save_radius("radius_periodic_box_1cell", p * 0.5, 0.3, periodic=torch.full((3,), 0.5))
    p2 = torch.rand(150, 2, generator=gen) * torch.tensor([2.0, 1.0])
    save_radius("radius_periodic_rect_d2", p2, 0.3, periodic=torch.tensor([2.0, 1.0]))
    lattice = torch.tensor([[1.0, 0.0, 0.0], [0.25, 1.0, 0.0], [0.0, 0.5, 1.5]])
    p3 = torch.rand(180, 3, generator=gen) @ lattice
    save_radius("radius_periodic_skew", p3, 0.3, periodic=lattice)

    # ------------------------------------------------------------- radius, metric / select
    def anisotropic(src, dst, edge):
        del src, dst
        return torch.linalg.vector_norm(edge.displacement * torch.tensor([2.0, 1.0, 1.0]), dim=-1)

    def other_type(src, dst, edge):
        return (src.kind != dst.kind) & (edge.distance > 0)

    p = torch.rand(100, 3, generator=gen)
    kind = torch.randint(0, 2, (100,), generator=gen)
    saved["radius_select_kind"] = kind.numpy()
    save_radius("radius_metric", p, 0.3, metric=anisotropic)
    save_radius("radius_select", p, 0.3, fields={"kind": kind}, select=other_type)

    # ------------------------------------------------------------- radius consumers + gradients
    for key, p in (("radius_consumer_grid", binary_grid_points(96, 3, gen, "duplicates")),
                   ("radius_consumer_random", torch.rand(200, 3, generator=gen))):
        p = p.clone().requires_grad_()
        for F in (1,):      # the implicit distance is one scalar per edge: scalar features broadcast against it
            x = torch.rand(p.shape[0], generator=gen).requires_grad_()
            dy = torch.randn(x.shape, generator=gen)
            graph = tg.Graph.radius(p, 0.25)
            out = DistanceSum().reference(graph=graph, src={"x": x}, dst={})
            dp, dx = torch.autograd.grad(out, (p, x), dy)
            tag = f"{key}_f{F}"
            saved[tag + "_pos"] = p.detach().numpy()
            saved[tag + "_x"] = x.detach().numpy()
            saved[tag + "_dy"] = dy.numpy()
            saved[tag + "_out"] = out.detach().numpy()
            saved[tag + "_dpos"] = dp.numpy()
            saved[tag + "_dx"] = dx.numpy()

    # ------------------------------------------------------------- kNN
    def save_knn(key, positions, k, **kwargs):
        graph = tg.Graph.knn(positions, k, **kwargs)
        row_ptr, col = graph.resolve_csr()
        fields = graph.implicit_edge_fields(row_ptr, col)
        saved[key + "_pos"] = positions.numpy()
        saved[key + "_k"] = np.int64(k)
        if kwargs.get("candidates") is not None:
            saved[key + "_candidates"] = kwargs["candidates"].numpy()
        saved[key + "_row_ptr"] = row_ptr.numpy()
        saved[key + "_col"] = col.numpy()
        saved[key + "_distance"] = fields["distance"].numpy()
        saved[key + "_displacement"] = fields["displacement"].numpy()
        saved[key + "_builder"] = np.array(graph.build_info["builder"])
        x = torch.randn(graph.schema.num_src, 3, generator=gen)
        out = NeighborSum().reference(graph=graph, src={"x": x}, dst={})
        saved[key + "_x"] = x.numpy()
        saved[key + "_out"] = out.numpy()

    p = torch.rand(200, 3, generator=gen)
    for k in (1, 5, 13, 64):
        save_knn(f"knn_self_d3_k{k}", p, k)
    save_knn("knn_self_keep_d3_k4", p, 4, exclude_self=False)
    save_knn("knn_self_d2_k7", torch.randn(150, 2, generator=gen), 7)
    save_knn("knn_self_d8_k6", torch.randn(130, 8, generator=gen), 6)
    save_knn("knn_bipartite_d3_k9", torch.rand(70, 3, generator=gen), 9,
             candidates=torch.rand(310, 3, generator=gen))
    save_knn("knn_all_candidates", torch.rand(12, 3, generator=gen), 20,
             candidates=torch.rand(20, 3, generator=gen))

    out_path = os.path.join(HERE, "geometry_cases.npz")
    np.savez_compressed(out_path, **saved)
    print(f"wrote {out_path}: {len(saved)} arrays, {os.path.getsize(out_path) / 1024:.1f} KiB")


if __name__ == "__main__":
    main()
