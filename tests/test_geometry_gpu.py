"""GPU parity of the dynamic-relation builders and the fused radius consumer.

Indices (row_ptr, col) and the float32 geometry (distance, displacement) must equal the reference's
fixtures and the CPU oracle BIT FOR BIT: the kernels evaluate the reference's float32 operation
order.  Sums are compared bit for bit where the summation order is the relation's edge order
(forward), and within float32 sum tolerance where it is not (cotangents)."""
import os

import numpy as np
import pytest
import torch

import tiga as tg
from conftest import assert_sum_close
from test_geometry_cpu import knn_keys, radius_arguments, radius_keys

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def geo():
    return dict(np.load(os.path.join(ROOT, "tests", "golden", "geometry_cases.npz")))


class DistanceSum(tg.MessagePassing):
    reducer = tg.sum()

    def edge(self, src, dst, edge):
        return edge.distance * src.x


class NeighborSum(tg.MessagePassing):
    reducer = tg.sum()

    def edge(self, src, dst, edge):
        return src.x


class NeighborMean(tg.MessagePassing):
    reducer = tg.mean()

    def edge(self, src, dst, edge):
        return edge.distance * src.x


def cuda_kwargs(kwargs):
    out = dict(kwargs)
    if "periodic" in out:
        out["periodic"] = out["periodic"].cuda()
    if "fields" in out:
        out["fields"] = {k: v.cuda() for k, v in out["fields"].items()}
    return out


def test_radius_matches_reference_fixtures_bit_for_bit(geo):
    native = 0
    for key in radius_keys(geo):
        cutoff, kwargs = radius_arguments(geo, key)
        if isinstance(cutoff, torch.Tensor):
            cutoff = cutoff.cuda()
        graph = tg.Graph.radius(torch.from_numpy(geo[key + "_pos"]).cuda(), cutoff, **cuda_kwargs(kwargs))
        row_ptr, col = graph.resolve_csr()
        fields = graph.implicit_edge_fields(row_ptr, col)
        np.testing.assert_array_equal(row_ptr.cpu().numpy(), geo[key + "_row_ptr"], err_msg=key)
        np.testing.assert_array_equal(col.cpu().numpy(), geo[key + "_col"], err_msg=key)
        np.testing.assert_array_equal(fields["displacement"].cpu().numpy(), geo[key + "_displacement"], err_msg=key)
        if geo[key + "_pos"].shape[1] <= 3 and key != "radius_metric":
            np.testing.assert_array_equal(fields["distance"].cpu().numpy(), geo[key + "_distance"], err_msg=key)
        else:   # four columns / a Torch callable evaluated on the device: one ulp
            np.testing.assert_allclose(fields["distance"].cpu().numpy(), geo[key + "_distance"], rtol=3e-7)
        info = graph.build_info
        assert info["accepted_edges"] == col.numel()
        if info["builder"] == "b200_hash_cell_list":
            native += 1
            assert str(geo[key + "_builder"]) == "uniform_cell_list"
            assert info["candidate_pairs"] == int(geo[key + "_candidate_pairs"]), key
    assert native >= 18          # everything except the all-pairs and callable-metric cases


def test_radius_large_against_oracle(oracle):
    # hash buckets shared by far-apart cells, a dense cluster, hubs; sizes the oracle finishes in seconds
    gen = torch.Generator().manual_seed(5)
    cloud = torch.rand(20000, 3, generator=gen) * 4.0
    cluster = torch.rand(3000, 3, generator=gen) * 0.15 + 100.0           # ~3000 points in two cells
    far = torch.rand(2000, 3, generator=gen) * 4.0 - 5000.0
    positions = torch.cat((cloud, cluster, far))[torch.randperm(25000, generator=gen)]
    for cutoff, periodic in ((0.11, None), (0.3, torch.tensor([4.0, 4.0, 4.0]))):
        kwargs = {}
        lattice = {}
        if periodic is not None:
            kwargs["periodic"] = periodic.cuda()
            inverse = torch.linalg.inv(torch.diag(periodic))
            bound = cutoff * torch.linalg.vector_norm(inverse, dim=0)
            lattice = dict(lattice=torch.diag(periodic).numpy(), inverse=inverse.numpy(),
                           extents=torch.floor(1.0 / bound.clamp_min(1e-12)).clamp(min=1).to(torch.int64).numpy())
        graph = tg.Graph.radius(positions.cuda(), cutoff, **kwargs)
        row_ptr, col = graph.resolve_csr()
        fields = graph.implicit_edge_fields(row_ptr, col)
        want_ptr, want_col, want_dist, want_disp, pairs = oracle.radius_build(
            positions.numpy(), np.float32(cutoff), exclude_self=True, use_cells=True, **lattice)
        np.testing.assert_array_equal(row_ptr.cpu().numpy(), want_ptr)
        np.testing.assert_array_equal(col.cpu().numpy(), want_col)
        np.testing.assert_array_equal(fields["distance"].cpu().numpy(), want_dist)
        np.testing.assert_array_equal(fields["displacement"].cpu().numpy(), want_disp)
        assert graph.build_info["candidate_pairs"] == pairs
        assert col.numel() > 100000


@pytest.mark.parametrize("dims", (1, 2))
def test_radius_low_dimensions_against_oracle(oracle, dims):
    gen = torch.Generator().manual_seed(dims)
    positions = torch.randn(6000, dims, generator=gen)
    cutoff = 0.002 if dims == 1 else 0.03
    graph = tg.Graph.radius(positions.cuda(), cutoff, exclude_self=False)
    row_ptr, col = graph.resolve_csr()
    want_ptr, want_col, want_dist, _, _ = oracle.radius_build(positions.numpy(), np.float32(cutoff),
                                                             exclude_self=False, use_cells=True)
    np.testing.assert_array_equal(row_ptr.cpu().numpy(), want_ptr)
    np.testing.assert_array_equal(col.cpu().numpy(), want_col)
    np.testing.assert_array_equal(graph.implicit_edge_fields(row_ptr, col)["distance"].cpu().numpy(), want_dist)


def test_fused_consumer_matches_reference_fixture(geo):
    for tag in ("radius_consumer_grid_f1", "radius_consumer_random_f1"):
        p = torch.from_numpy(geo[tag + "_pos"]).cuda().requires_grad_()
        x = torch.from_numpy(geo[tag + "_x"]).cuda().requires_grad_()
        kernel = DistanceSum()
        graph = tg.Graph.radius(p, 0.25)
        out = kernel(graph=graph, src={"x": x}, dst={})
        assert "generated-radius" in kernel.last_variant.lowering
        assert graph._row_ptr is None and graph.num_edges is None        # nothing was materialised
        # forward: same terms in the same order as the reference's index_add over its edge list
        np.testing.assert_array_equal(out.detach().cpu().numpy(), geo[tag + "_out"])
        dp, dx = torch.autograd.grad(out, (p, x), torch.from_numpy(geo[tag + "_dy"]).cuda())
        magnitude = np.abs(geo[tag + "_dx"]).max() * 30
        assert_sum_close(dx.cpu().numpy(), geo[tag + "_dx"], magnitude)
        assert_sum_close(dp.cpu().numpy(), geo[tag + "_dpos"], np.abs(geo[tag + "_dpos"]).max() * 30, rtol=1e-4)


@pytest.mark.parametrize("features", ((), (1,), (5,), (32,), (4, 8), (128,)))
@pytest.mark.parametrize("periodic", (False, True))
def test_fused_consumer_equals_the_materialised_relation(features, periodic):
    gen = torch.Generator().manual_seed(len(features) + 10 * periodic)
    n = 3000
    positions = torch.rand(n, 3, generator=gen).cuda()
    kwargs = {"periodic": torch.ones(3, device="cuda")} if periodic else {}
    x = torch.randn((n,) + features, generator=gen).cuda()
    dy = torch.randn((n,) + features, generator=gen).cuda()
    p1, x1 = positions.clone().requires_grad_(), x.clone().requires_grad_()
    fused = DistanceSum() if len(features) == 0 else None
    if len(features) == 0:
        out = fused(graph=tg.Graph.radius(p1, 0.12, **kwargs), src={"x": x1}, dst={})
        dp, dx = torch.autograd.grad(out, (p1, x1), dy)
    else:       # vector features take the unweighted fold (distance broadcasts against scalars only)
        fused = NeighborSum()
        out = fused(graph=tg.Graph.radius(p1, 0.12, **kwargs), src={"x": x1}, dst={})
        (dx,) = torch.autograd.grad(out, (x1,), dy)
    assert "generated-radius" in fused.last_variant.lowering
    # the same program over the stored CSR of the same relation
    graph = tg.Graph.radius(positions, 0.12, **kwargs)
    row_ptr, col = graph.resolve_csr()
    stored = tg.Graph.from_csr(row_ptr, col, num_src=n)
    x2 = x.clone().requires_grad_()
    if len(features) == 0:
        class Weighted(tg.MessagePassing):
            reducer = tg.sum()

            def edge(self, src, dst, edge):
                return edge.w * src.x

        p2 = positions.clone().requires_grad_()
        destination = stored.destination_index(row_ptr)
        distance = torch.linalg.vector_norm(
            tg.Graph.radius(p2, 0.12, **kwargs)._geometry.minimum_image(p2[col] - p2[destination]), dim=-1)
        want = Weighted()(graph=stored, src={"x": x2}, dst={}, edge={"w": distance})
        want_dp, want_dx = torch.autograd.grad(want, (p2, x2), dy)
        torch.testing.assert_close(dp, want_dp, rtol=2e-4, atol=2e-5)
        # the bit-for-bit statement needs the distances in the kernels' own rounding (Torch's norm on
        # the device may differ by an ulp): the relation's implicit field
        own = graph.implicit_edge_fields(row_ptr, col)["distance"]
        want = Weighted()(graph=stored, src={"x": x}, dst={}, edge={"w": own})
    else:
        want = NeighborSum()(graph=stored, src={"x": x2}, dst={})
        (want_dx,) = torch.autograd.grad(want, (x2,), dy)
    assert torch.equal(out, want)                       # same fold order: bit for bit
    torch.testing.assert_close(dx, want_dx, rtol=1e-4, atol=1e-5)


def test_positions_changed_in_place_rebuild_without_respecialising():
    gen = torch.Generator(device="cuda").manual_seed(519)
    p = (torch.rand(480, 3, generator=gen, device="cuda") * 64).floor() / 64 - 0.5
    x = torch.ones(480, device="cuda")
    graph, kernel = tg.Graph.radius(p, 0.25), DistanceSum()
    first = kernel(graph=graph, src={"x": x}, dst={}).clone()
    p.mul_(0.5)
    second = kernel(graph=graph, src={"x": x}, dst={})
    distances = torch.cdist(p, p, compute_mode="donot_use_mm_for_euclid_dist")
    expected = (distances * (distances <= 0.25)).sum(-1)
    torch.testing.assert_close(second, expected, atol=2e-5, rtol=2e-5)
    assert not torch.allclose(first, second)
    assert kernel.cache_info["misses"] == 1
    # a new Graph over new coordinates with the same search signature reuses the launch
    q = torch.rand(480, 3, generator=gen, device="cuda")
    third = kernel(graph=tg.Graph.radius(q, 0.25), src={"x": x}, dst={})
    distances = torch.cdist(q, q, compute_mode="donot_use_mm_for_euclid_dist")
    torch.testing.assert_close(third, (distances * (distances <= 0.25)).sum(-1), atol=2e-5, rtol=2e-5)
    assert kernel.cache_info["misses"] == 1 and kernel.cache_info["hits"] >= 2
    # the cutoff is a runtime scalar: another value reuses the launch and is honoured
    wider = kernel(graph=tg.Graph.radius(q, 0.3), src={"x": x}, dst={})
    torch.testing.assert_close(wider, (distances * (distances <= 0.3)).sum(-1), atol=2e-5, rtol=2e-5)
    assert kernel.cache_info["misses"] == 1
    # a different search (self pairs kept) is another signature
    kernel(graph=tg.Graph.radius(q, 0.3, exclude_self=False), src={"x": x}, dst={})
    assert kernel.cache_info["misses"] == 1 and len(kernel._launches) == 2


def test_other_reducers_and_select_run_over_the_built_csr(geo):
    gen = torch.Generator().manual_seed(8)
    positions = torch.rand(2000, 3, generator=gen)
    kind = torch.randint(0, 2, (2000,), generator=gen)
    x = torch.randn(2000, 16, generator=gen)
    select = lambda src, dst, edge: (src.kind != dst.kind) & (edge.distance > 0.02)     # noqa: E731
    graph = tg.Graph.radius(positions.cuda(), 0.15, fields={"kind": kind.cuda()}, select=select)
    cpu_graph = tg.Graph.radius(positions, 0.15, fields={"kind": kind}, select=select)
    row_ptr, col = graph.resolve_csr()
    want_ptr, want_col = cpu_graph.resolve_csr()
    assert torch.equal(row_ptr.cpu(), want_ptr) and torch.equal(col.cpu(), want_col)
    kernel = NeighborSum()
    out = kernel(graph=graph, src={"x": x.cuda()}, dst={})
    assert "csr-weighted-sum" in kernel.last_variant.lowering           # select: the relation is not symmetric-safe
    want = NeighborSum().reference(graph=cpu_graph, src={"x": x}, dst={})
    torch.testing.assert_close(out.cpu(), want, rtol=1e-5, atol=1e-5)
    # mean of distance-weighted messages: implicit weight on the CSR kernels
    plain = tg.Graph.radius(positions.cuda(), 0.15)
    xs = x[:, 0].contiguous()
    got = NeighborMean()(graph=plain, src={"x": xs.cuda()}, dst={})
    want = NeighborMean().reference(graph=tg.Graph.radius(positions, 0.15), src={"x": xs}, dst={})
    torch.testing.assert_close(got.cpu(), want, rtol=1e-5, atol=1e-6, equal_nan=True)


def test_knn_matches_reference_fixtures(geo, oracle):
    for key in knn_keys(geo):
        kwargs = {}
        pos = torch.from_numpy(geo[key + "_pos"]).cuda()
        self_search = key + "_candidates" not in geo
        if not self_search:
            kwargs["candidates"] = torch.from_numpy(geo[key + "_candidates"]).cuda()
        if "keep" in key:
            kwargs["exclude_self"] = False
        k = int(geo[key + "_k"])
        graph = tg.Graph.knn(pos, k, **kwargs)
        row_ptr, col = graph.resolve_csr()
        assert graph.build_info["builder"].startswith("b200-exact-knn-")
        np.testing.assert_array_equal(row_ptr.cpu().numpy(), geo[key + "_row_ptr"])
        candidates = geo[key + "_pos"] if self_search else geo[key + "_candidates"]
        want = oracle.knn_build(geo[key + "_pos"], candidates, k, exclude_self=self_search and "keep" not in key)
        np.testing.assert_array_equal(col.cpu().numpy().reshape(-1, k), want, err_msg=key)    # oracle: bit exact
        reference = geo[key + "_col"].reshape(-1, k)
        assert all(set(a) == set(b) for a, b in zip(want, reference)), key
        # consumer over the relation, against the reference's output
        x = torch.from_numpy(geo[key + "_x"]).cuda()
        out = NeighborSum()(graph=graph, src={"x": x}, dst={})
        np.testing.assert_allclose(out.cpu().numpy(), geo[key + "_out"], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("search", ("scan", "shells"))
def test_knn_searches_agree_on_hard_inputs(oracle, monkeypatch, search):
    """The shell search over the cell directory and the scan over all candidates are both exact:
    fixtures with few points, duplicated points, a dense cluster beside far outliers (unsettled
    queries finish by the scan), collinear points, bipartite queries outside the candidates' box."""
    from tiga import geometry

    monkeypatch.setattr(geometry, "KNN_GRID_MIN_CANDIDATES", 1 if search == "shells" else 1 << 60)
    gen = torch.Generator().manual_seed(77)
    cluster = torch.rand(3000, 3, generator=gen) * 0.05
    outliers = torch.rand(40, 3, generator=gen) * 500.0 - 250.0
    duplicated = torch.rand(500, 3, generator=gen).repeat(2, 1)
    line = torch.cat((torch.rand(2000, 1, generator=gen), torch.zeros(2000, 2)), dim=1)
    cases = {"cluster+outliers": torch.cat((cluster, outliers))[torch.randperm(3040, generator=gen)],
             "duplicates": duplicated, "line": line, "grid": (torch.rand(4000, 2, generator=gen) * 16).floor() / 16}
    for name, points in cases.items():
        for k in (1, 7, 32):
            graph = tg.Graph.knn(points.cuda(), k)
            col = graph.resolve_csr()[1].cpu().numpy().reshape(-1, k)
            want = oracle.knn_build(points.numpy(), points.numpy(), k, exclude_self=True)
            np.testing.assert_array_equal(col, want, err_msg=f"{name} k={k} {search}")
            expected = "b200-exact-knn-cell-shells" if search == "shells" else "b200-exact-knn-tiled-scan"
            assert graph.build_info["builder"] == expected
    queries = torch.rand(300, 3, generator=gen) * 3.0 - 1.0          # partly outside the unit cube
    candidates = torch.rand(5000, 3, generator=gen)
    graph = tg.Graph.knn(queries.cuda(), 9, candidates=candidates.cuda())
    want = oracle.knn_build(queries.numpy(), candidates.numpy(), 9, exclude_self=False)
    np.testing.assert_array_equal(graph.resolve_csr()[1].cpu().numpy().reshape(-1, 9), want)


@pytest.mark.parametrize("k", (1, 13, 16, 63, 128))
@pytest.mark.parametrize("order", ("ascending", "descending", "ties"))
def test_knn_selection_is_exact_under_ordered_input_and_ties(k, order):
    # several tiles plus a tail; ordered input exercises late replacement, ties the index part of the key
    # (tests/python/test_ranked_rebinding.py:88-104 of the reference)
    p = torch.arange(2531, device="cuda", dtype=torch.float32)[:, None]
    if order == "descending":
        p = p.flip(0)
    if order == "ties":
        p = (p % 3).contiguous()
    query = torch.tensor([[0.0], [350.0]], device="cuda")
    x = torch.arange(len(p), device="cuda", dtype=torch.float32)
    graph = tg.Graph.knn(query, k, candidates=p)
    col = graph.resolve_csr()[1].reshape(2, k)
    selected = (query - p.T).square().argsort(dim=1, stable=True)[:, :k]
    assert torch.equal(col, selected)
    actual = NeighborSum()(graph=graph, src={"x": x}, dst={})
    torch.testing.assert_close(actual, x[selected].sum(1))


@pytest.mark.parametrize("dims", (2, 3, 8, 33, 64))
def test_knn_large_against_oracle(oracle, dims):
    gen = torch.Generator().manual_seed(dims)
    n = 5000 if dims <= 8 else 1500
    positions = torch.randn(n, dims, generator=gen)
    graph = tg.Graph.knn(positions.cuda(), 10)
    col = graph.resolve_csr()[1].cpu().numpy().reshape(n, 10)
    want = oracle.knn_build(positions.numpy(), positions.numpy(), 10, exclude_self=True)
    np.testing.assert_array_equal(col, want)
    fields = graph.implicit_edge_fields(*graph.resolve_csr())
    assert fields["distance"].shape == (n * 10,) and fields["displacement"].shape == (n * 10, dims)
    if dims <= 8:
        displacement, distance = oracle.edge_geometry(positions.numpy(), positions.numpy(),
                                                      np.repeat(np.arange(n), 10), want.reshape(-1))
        np.testing.assert_array_equal(fields["displacement"].cpu().numpy(), displacement)
        np.testing.assert_array_equal(fields["distance"].cpu().numpy(), distance)


def test_empty_and_degenerate_inputs():
    empty = tg.Graph.radius(torch.empty(0, 3, device="cuda"), 0.25)
    row_ptr, col = empty.resolve_csr()
    assert row_ptr.tolist() == [0] and col.numel() == 0
    single = tg.Graph.radius(torch.zeros(1, 3, device="cuda"), 0.25)
    assert single.resolve_csr()[0].tolist() == [0, 0]
    kept = tg.Graph.radius(torch.zeros(4, 2, device="cuda"), 0.25, exclude_self=False)     # coincident points
    assert kept.resolve_csr()[0].tolist() == [0, 4, 8, 12, 16]
    out = DistanceSum()(graph=tg.Graph.radius(torch.zeros(4, 2, device="cuda"), 0.25),
                        src={"x": torch.ones(4, device="cuda")}, dst={})
    assert out.tolist() == [0.0] * 4
    with pytest.raises(ValueError, match="shadow graph-provided fields: distance"):
        DistanceSum()(graph=single, src={"x": torch.ones(1, device="cuda")}, dst={},
                      edge={"distance": torch.zeros(0, device="cuda")})
