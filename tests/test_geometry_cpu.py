"""Dynamic relations without a GPU: the C oracle against the reference-generated fixtures, the Torch
path of Graph.radius / Graph.knn (CPU tensors) against the same fixtures, argument checks, snapshot
semantics.  Everything here is bit-exact (integer indices; float32 geometry in the reference's
operation order) unless a tolerance is written next to the comparison."""
import os

import numpy as np
import pytest
import torch

import tiga as tg

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def geo():
    return dict(np.load(os.path.join(ROOT, "tests", "golden", "geometry_cases.npz")))


def radius_keys(geo):
    return sorted(k[:-4] for k in geo if k.startswith("radius") and k.endswith("_pos") and "consumer" not in k)


def knn_keys(geo):
    return sorted(k[:-4] for k in geo if k.startswith("knn") and k.endswith("_pos"))


def lattice_arguments(geo, key):
    if key + "_periodic" not in geo:
        return {}
    periodic = torch.from_numpy(geo[key + "_periodic"])
    lattice = torch.diag(periodic) if periodic.ndim == 1 else periodic
    inverse = torch.linalg.inv(lattice)
    bound = float(geo[key + "_cutoff"]) * torch.linalg.vector_norm(inverse, dim=0)
    extents = torch.floor(1.0 / bound.clamp_min(1.0e-12)).clamp(min=1).to(torch.int64)
    return dict(lattice=lattice.numpy(), inverse=inverse.numpy(), extents=extents.numpy())


def radius_arguments(geo, key):
    kwargs = {}
    if key + "_periodic" in geo:
        kwargs["periodic"] = torch.from_numpy(geo[key + "_periodic"])
    if key.endswith("_self"):
        kwargs["exclude_self"] = False
    if key == "radius_metric":
        kwargs["metric"] = lambda src, dst, edge: torch.linalg.vector_norm(
            edge.displacement * torch.tensor([2.0, 1.0, 1.0], device=edge.displacement.device), dim=-1)
    if key == "radius_select":
        kwargs["fields"] = {"kind": torch.from_numpy(geo["radius_select_kind"])}
        kwargs["select"] = lambda src, dst, edge: (src.kind != dst.kind) & (edge.distance > 0)
    cutoff = geo[key + "_cutoff"]
    return (float(cutoff) if cutoff.ndim == 0 else torch.from_numpy(cutoff)), kwargs


# ------------------------------------------------------------------ the oracle is pinned by the reference
def test_oracle_radius_matches_reference_fixtures(oracle, geo):
    checked = 0
    for key in radius_keys(geo):
        if key in ("radius_metric", "radius_select"):      # callables: covered through the Graph below
            continue
        cutoff = geo[key + "_cutoff"]
        kwargs = lattice_arguments(geo, key) if cutoff.ndim == 0 else {}
        row_ptr, col, distance, displacement, pairs = oracle.radius_build(
            geo[key + "_pos"], cutoff, exclude_self=not key.endswith("_self"),
            use_cells=str(geo[key + "_builder"]) == "uniform_cell_list", **kwargs)
        np.testing.assert_array_equal(row_ptr, geo[key + "_row_ptr"], err_msg=key)
        np.testing.assert_array_equal(col, geo[key + "_col"], err_msg=key)
        np.testing.assert_array_equal(displacement, geo[key + "_displacement"], err_msg=key)
        if geo[key + "_pos"].shape[1] <= 3:
            np.testing.assert_array_equal(distance, geo[key + "_distance"], err_msg=key)
        else:       # four terms: Torch's vectorised norm adds them in another order; one ulp
            np.testing.assert_allclose(distance, geo[key + "_distance"], rtol=2e-7)
        assert pairs == int(geo[key + "_candidate_pairs"]), key
        checked += 1
    assert checked >= 20


def test_oracle_knn_matches_reference_fixtures(oracle, geo):
    for key in knn_keys(geo):
        pos, k = geo[key + "_pos"], int(geo[key + "_k"])
        self_search = key + "_candidates" not in geo
        candidates = pos if self_search else geo[key + "_candidates"]
        col = oracle.knn_build(pos, candidates, k, exclude_self=self_search and "keep" not in key)
        want = geo[key + "_col"].reshape(-1, k)
        # the reference ranks by a matmul-form distance whose rounding may swap two neighbours that
        # are equal to ~1e-7: rows must hold the same set, and all but a handful the same order
        assert all(set(a) == set(b) for a, b in zip(col, want)), key
        assert (col != want).any(axis=1).sum() <= 1, key


def test_oracle_knn_ties_rank_by_candidate_index(oracle):
    # three distinct coordinates repeated: the (distance, index) key decides
    # (the case of tests/python/test_ranked_rebinding.py:88-104 of the reference)
    p = (np.arange(1031, dtype=np.float32) % 3)[:, None]
    query = np.array([[0.0], [350.0]], np.float32)
    for k in (1, 13, 16, 63):
        col = oracle.knn_build(query, p, k, exclude_self=False)
        d = (query - p.T) ** 2
        want = np.argsort(d, axis=1, kind="stable")[:, :k]
        np.testing.assert_array_equal(col, want)


# ------------------------------------------------------------------ Graph.radius / Graph.knn on CPU tensors
def test_graph_radius_cpu_matches_reference_fixtures(geo):
    for key in radius_keys(geo):
        cutoff, kwargs = radius_arguments(geo, key)
        graph = tg.Graph.radius(torch.from_numpy(geo[key + "_pos"]), cutoff, **kwargs)
        row_ptr, col = graph.resolve_csr()
        fields = graph.implicit_edge_fields(row_ptr, col)
        np.testing.assert_array_equal(row_ptr.numpy(), geo[key + "_row_ptr"], err_msg=key)
        np.testing.assert_array_equal(col.numpy(), geo[key + "_col"], err_msg=key)
        np.testing.assert_array_equal(fields["distance"].numpy(), geo[key + "_distance"], err_msg=key)
        np.testing.assert_array_equal(fields["displacement"].numpy(), geo[key + "_displacement"], err_msg=key)
        assert graph.build_info["builder"] == str(geo[key + "_builder"])
        assert graph.build_info["candidate_pairs"] == int(geo[key + "_candidate_pairs"])
        assert graph.build_info["accepted_edges"] == col.numel()


def test_graph_knn_cpu_matches_reference_fixtures(geo):
    for key in knn_keys(geo):
        kwargs = {}
        if key + "_candidates" in geo:
            kwargs["candidates"] = torch.from_numpy(geo[key + "_candidates"])
        if "keep" in key:
            kwargs["exclude_self"] = False
        k = int(geo[key + "_k"])
        graph = tg.Graph.knn(torch.from_numpy(geo[key + "_pos"]), k, **kwargs)
        row_ptr, col = graph.resolve_csr()
        np.testing.assert_array_equal(row_ptr.numpy(), geo[key + "_row_ptr"])
        got, want = col.numpy().reshape(-1, k), geo[key + "_col"].reshape(-1, k)
        assert all(set(a) == set(b) for a, b in zip(got, want)), key
        assert graph.schema.origin == "geometric_knn" and graph.schema.lifecycle == "dynamic"


def test_reference_known_answers():
    # tests/python/test_reference.py:485-497, 543-560, 562-584 of the reference
    positions = torch.tensor([[0.0, 0.0], [0.5, 0.0], [2.0, 0.0]])
    graph = tg.Graph.radius(positions, 0.75)
    row_ptr, col = graph.resolve_csr()
    assert row_ptr.tolist() == [0, 1, 2, 2] and col.tolist() == [1, 0]
    assert "lifecycle=dynamic" in graph.explain()
    assert graph.build_info["builder"] == "uniform_cell_list"
    assert graph.num_edges is None

    positions = torch.tensor([[0.0, 0.0], [0.6, 0.0], [0.0, 0.6]])
    graph = tg.Graph.radius(positions, cutoff=0.75, metric=lambda src, dst, edge: torch.linalg.vector_norm(
        edge.displacement * torch.tensor([2.0, 1.0]), dim=-1))
    row_ptr, col = graph.resolve_csr()
    assert row_ptr.tolist() == [0, 1, 1, 2] and col.tolist() == [2, 0]
    assert "metric=custom" in graph.explain() and "broad_phase=all-pairs-only" in graph.explain()
    assert graph.build_info["builder"] == "all_pairs"

    positions = torch.tensor([[0.0, 0.0], [0.4, 0.0], [0.8, 0.0]])
    graph = tg.Graph.radius(positions, cutoff=0.5, fields={"particle_type": torch.tensor([0, 0, 1])},
                            select=lambda src, dst, edge: (src.particle_type != dst.particle_type)
                            & (edge.distance > 0))
    row_ptr, col = graph.resolve_csr()
    assert row_ptr.tolist() == [0, 0, 1, 2] and col.tolist() == [2, 1]
    assert "select=custom" in graph.explain() and "broad_phase=euclidean-cell-list-eligible" in graph.explain()


def test_cell_list_equals_all_pairs():
    gen = torch.Generator().manual_seed(17)
    positions = torch.rand(97, 3, generator=gen)
    graph = tg.Graph.radius(positions, 0.23)
    row_ptr, col = graph.resolve_csr()
    adjacency = torch.zeros(97, 97, dtype=torch.bool)
    adjacency[graph.destination_index(row_ptr), col] = True
    expected = torch.cdist(positions, positions) <= 0.23
    expected.fill_diagonal_(False)
    assert torch.equal(adjacency, expected)
    assert graph.build_info["candidate_pairs"] < 97 ** 2


def test_snapshot_is_rebuilt_after_an_in_place_change():
    positions = torch.tensor([[0.0, 0.0], [0.5, 0.0], [0.0, 0.5], [0.5, 0.5]])
    graph = tg.Graph.radius(positions, 0.75)
    first = graph.resolve_csr()
    assert graph.resolve_csr()[1] is first[1] and graph.build_info["cache_hit"]
    positions[3] += 5.0                      # bumps the tensor version: a new physical snapshot
    row_ptr, col = graph.resolve_csr()
    assert not graph.build_info["cache_hit"]
    assert row_ptr.tolist() == [0, 2, 4, 6, 6] and sorted(col.tolist()) == [0, 0, 1, 1, 2, 2]
    with pytest.raises(RuntimeError):
        tg.Graph.radius(positions, 0.75).build_info


def test_argument_checks():
    p = torch.rand(8, 3)
    with pytest.raises(ValueError, match="shape"):
        tg.Graph.radius(torch.rand(8), 0.1)
    with pytest.raises(TypeError, match="floating"):
        tg.Graph.radius(torch.zeros(8, 3, dtype=torch.int64), 0.1)
    with pytest.raises(TypeError, match="callable"):
        tg.Graph.radius(p, 0.1, metric=3)
    with pytest.raises(ValueError, match="box lengths"):
        tg.Graph.radius(p, 0.1, periodic=torch.ones(2))
    with pytest.raises(ValueError, match="nonsingular"):
        tg.Graph.radius(p, 0.1, periodic=torch.zeros(3, 3))
    with pytest.raises(ValueError, match="reserved"):
        tg.Graph.radius(p, 0.1, fields={"position": p})
    with pytest.raises(ValueError, match="leading dimension"):
        tg.Graph.radius(p, 0.1, fields={"kind": torch.zeros(5)})
    with pytest.raises(ValueError, match=r"k must be in \[1, 7\] for 8 candidates"):
        tg.Graph.knn(p, 8)
    with pytest.raises(ValueError, match="only defined for self-kNN"):
        tg.Graph.knn(p, 2, candidates=torch.rand(9, 3), exclude_self=True)
    with pytest.raises(ValueError, match="share feature width"):
        tg.Graph.knn(p, 2, candidates=torch.rand(9, 2))
    with pytest.raises(ValueError, match="scalar, per-destination"):
        tg.Graph.radius(p, torch.ones(3)).resolve_csr()


def test_eager_reference_reads_the_implicit_fields(geo):
    class DistanceSum(tg.MessagePassing):
        reducer = tg.sum()

        def edge(self, src, dst, edge):
            return edge.distance * src.x

    for tag in ("radius_consumer_grid_f1", "radius_consumer_random_f1"):
        p = torch.from_numpy(geo[tag + "_pos"]).requires_grad_()
        x = torch.from_numpy(geo[tag + "_x"]).requires_grad_()
        graph = tg.Graph.radius(p, 0.25)
        out = DistanceSum().reference(graph=graph, src={"x": x}, dst={})
        np.testing.assert_array_equal(out.detach().numpy(), geo[tag + "_out"])
        dp, dx = torch.autograd.grad(out, (p, x), torch.from_numpy(geo[tag + "_dy"]))
        np.testing.assert_allclose(dp.numpy(), geo[tag + "_dpos"], rtol=1e-6, atol=1e-7)
        np.testing.assert_allclose(dx.numpy(), geo[tag + "_dx"], rtol=1e-6, atol=1e-7)
    with pytest.raises(ValueError, match="shadow graph-provided fields: distance"):
        DistanceSum().reference(graph=graph, src={"x": x}, dst={},
                                edge={"distance": torch.zeros(graph.resolve_csr()[1].numel())})
