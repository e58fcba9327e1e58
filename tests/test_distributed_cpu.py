"""Multi-rank host logic on CPU: partition, halo derivation, request exchange,
forward halo exchange and the reverse (cotangent) exchange, run as real
processes over the gloo backend (world sizes 2 and 3).  The local compute of
each rank is done by a checker backend built on the CPU oracle, so these tests
exercise exactly the host-side code the GPU ranks run, without a GPU."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class OracleBackend:
    """Local compute of one rank through the CPU oracle (test checker)."""

    @staticmethod
    def _csr(graph):
        row_ptr, col = graph.resolve_csr()
        return row_ptr.numpy().astype(np.int64), col.numpy().astype(np.int64)

    def forward(self, graph, x, w, accumulate_into=None):
        from oracle import oracle

        row_ptr, col = self._csr(graph)
        if w is not None and graph._edge_map is not None:
            w = w[graph._edge_map.long()]
        out = torch.from_numpy(oracle.wsum_fwd(row_ptr, col, x.numpy(), None if w is None else w.numpy()))
        if accumulate_into is not None:
            accumulate_into += out
            return accumulate_into
        return out

    @staticmethod
    def pack_rows(rows, ids):
        return rows.index_select(0, ids)

    @staticmethod
    def add_rows(rows, ids, packed):
        rows.index_add_(0, ids, packed)

    def backward_dx(self, graph, dy, w):
        from oracle import oracle

        row_ptr, col = self._csr(graph)
        if w is not None and graph._edge_map is not None:
            w = w[graph._edge_map.long()]
        return torch.from_numpy(oracle.wsum_bwd_dx(row_ptr, col, graph.num_src, dy.numpy(),
                                                   None if w is None else w.numpy()))

    def backward_dw(self, graph, dy, x, out):
        from oracle import oracle

        row_ptr, col = self._csr(graph)
        dw = torch.from_numpy(oracle.wsum_bwd_dw(row_ptr, col, dy.numpy(), x.numpy()))
        if graph._edge_map is not None:
            out[graph._edge_map.long()] = dw
        else:
            out.copy_(dw)
        return out


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, balance, result_dir, shard_only=False, waves=1):
    for path in (ROOT, os.path.join(ROOT, "tiga-lang_b200")):
        sys.path.insert(0, path)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import tiga as tg
        from baseline import synthetic as syn
        from tiga.distributed import model
        from tiga.distributed.runtime import DistributedRuntime, ProcessGroupTransport, shard_plan_for

        class WeightedSum(tg.MessagePassing):
            reducer = tg.sum()

            def edge(self, src, dst, edge):
                return edge.weight * src.x

        row_ptr, col = syn.rmat_csr(7, 6, seed=13)           # 128 nodes, every rank builds the same graph
        n, F = row_ptr.numel() - 1, 8
        gen = torch.Generator().manual_seed(99)
        x = torch.randn(n, F, generator=gen)
        w = torch.rand(col.numel(), generator=gen)
        dy = torch.randn(n, F, generator=gen)
        if shard_only:
            # every rank holds nothing but its own block of rows, generated without the whole graph
            first, last = model.owned_range(n, world, rank)
            block_ptr, block_col = syn.rmat_csr_rows(7, 6, first, last, seed=13, chunk=256)
            assert torch.equal(block_col, col[int(row_ptr[first]):int(row_ptr[last])])
            graph = tg.Graph.from_csr_shard(block_ptr, block_col, num_nodes=n, first_row=first).halo(
                tg.DeviceMesh("cpu", world))
            with pytest.raises(RuntimeError):
                tg.Graph.from_csr_shard(block_ptr, block_col, num_nodes=n, first_row=first).resolve_csr()
        else:
            graph = tg.Graph.from_csr(row_ptr, col, num_src=n).halo(
                tg.DeviceMesh("cpu", world), partition=tg.ByDestination(balance=balance))
        runtime = DistributedRuntime(ProcessGroupTransport(), backend=OracleBackend(), waves=waves)
        with runtime:
            shard = shard_plan_for(graph, runtime)
            assert len(shard.waves) == min(waves, world - 1)
            assert sorted(p for pairs, _ in shard.waves for p, _ in pairs) == [p for p in range(world) if p != rank]
            b, e = shard.begin, shard.end
            lo, hi = int(row_ptr[b]), int(row_ptr[e])
            xs = x[b:e].clone().requires_grad_()
            ws = w[lo:hi].clone().requires_grad_()
            out = WeightedSum()(graph=graph, src={"x": xs}, dst={}, edge={"weight": ws})
            dx, dw = torch.autograd.grad(out, (xs, ws), dy[b:e])
            # only one gradient wanted: the backward runs per sub-relation instead of over the whole
            # local relation; every rank takes part in both exchanges
            xs1 = x[b:e].clone().requires_grad_()
            out1 = WeightedSum()(graph=graph, src={"x": xs1}, dst={}, edge={"weight": w[lo:hi].clone()})
            (dx_only,) = torch.autograd.grad(out1, (xs1,), dy[b:e])
            ws1 = w[lo:hi].clone().requires_grad_()
            out2 = WeightedSum()(graph=graph, src={"x": x[b:e].clone()}, dst={}, edge={"weight": ws1})
            (dw_only,) = torch.autograd.grad(out2, (ws1,), dy[b:e])
        np.testing.assert_allclose(dx_only.numpy(), dx.numpy(), rtol=1e-5, atol=2e-6)
        np.testing.assert_allclose(dw_only.numpy(), dw.numpy(), rtol=1e-5, atol=2e-6)
        halo = shard.halo_map()
        if balance == "auto":
            peers = [model.derive_halo_map(row_ptr, col, num_entities=n, world_size=world, rank=r)
                     for r in range(world)]
            requests = [[i for i in peers[p].ghost_ids if b <= i < e] for p in range(world)]
            expect = model.derive_halo_map(row_ptr, col, num_entities=n, world_size=world, rank=rank,
                                           peer_requests=requests)
            assert halo == expect, "halo map differs from derive_halo_map"
        np.savez(os.path.join(result_dir, f"rank{rank}.npz"), begin=b, end=e, lo=lo, hi=hi,
                 out=out.detach().numpy(), dx=dx.numpy(), dw=dw.numpy(), ghosts=shard.ghosts.numpy())
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,balance,shard_only,waves", (
    (2, "auto", False, 1), (3, "auto", False, 2), (2, "edges", False, 1), (3, "cost", False, 1),
    (4, "auto", True, 2), (4, "auto", False, 3)))
def test_sharded_weighted_sum_matches_single_process(tmp_path, oracle, world, balance, shard_only, waves):
    port = _free_port()
    mp.start_processes(_worker, args=(world, port, balance, str(tmp_path), shard_only, waves), nprocs=world,
                       join=True, start_method="spawn")
    sys.path.insert(0, os.path.join(ROOT, "tiga-lang_b200"))
    from baseline import synthetic as syn

    row_ptr, col = syn.rmat_csr(7, 6, seed=13)
    n, F = row_ptr.numel() - 1, 8
    gen = torch.Generator().manual_seed(99)
    x = torch.randn(n, F, generator=gen)
    w = torch.rand(col.numel(), generator=gen)
    dy = torch.randn(n, F, generator=gen)
    ref_out = oracle.wsum_fwd(row_ptr.numpy(), col.numpy(), x.numpy(), w.numpy())
    ref_dx = oracle.wsum_bwd_dx(row_ptr.numpy(), col.numpy(), n, dy.numpy(), w.numpy())
    ref_dw = oracle.wsum_bwd_dw(row_ptr.numpy(), col.numpy(), dy.numpy(), x.numpy())
    covered = 0
    for rank in range(world):
        data = np.load(tmp_path / f"rank{rank}.npz")
        b, e, lo, hi = int(data["begin"]), int(data["end"]), int(data["lo"]), int(data["hi"])
        covered += e - b
        np.testing.assert_allclose(data["out"], ref_out[b:e], rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(data["dx"], ref_dx[b:e], rtol=1e-5, atol=2e-6)
        np.testing.assert_allclose(data["dw"], ref_dw[lo:hi], rtol=1e-5, atol=2e-6)
        expect_ghosts = oracle.derive_ghosts(row_ptr.numpy(), col.numpy(), n, world, rank)
        if balance == "auto":
            np.testing.assert_array_equal(data["ghosts"], expect_ghosts)
    assert covered == n


def _failing_worker(rank, world, port, result_dir):
    """Rank 1 leaves before the halo exchange (a host-side failure between steps);
    rank 0 must get an exception from its exchange instead of waiting forever."""
    import datetime

    for path in (ROOT, os.path.join(ROOT, "tiga-lang_b200")):
        sys.path.insert(0, path)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    import tiga as tg
    from baseline import synthetic as syn
    from tiga.distributed.runtime import DistributedRuntime, ProcessGroupTransport, halo_weighted_sum, shard_plan_for

    row_ptr, col = syn.rmat_csr(7, 6, seed=13)
    n = row_ptr.numel() - 1
    graph = tg.Graph.from_csr(row_ptr, col, num_src=n).halo(tg.DeviceMesh("cpu", world))
    runtime = DistributedRuntime(ProcessGroupTransport(), backend=OracleBackend())
    with runtime:
        shard = shard_plan_for(graph, runtime)          # both ranks take part in the plan
        dist.barrier()
        if rank == 1:
            os._exit(0)                                  # leaves between steps, nothing in flight
        x = torch.randn(shard.owned, 4)
        try:
            halo_weighted_sum(graph, x, None, runtime)
            outcome = "no error"
        except Exception as error:                       # the exchange must fail, not hang
            outcome = f"raised {type(error).__name__}"
    with open(os.path.join(result_dir, "rank0.txt"), "w") as handle:
        handle.write(outcome)
    os._exit(0)


def test_peer_leaving_between_steps_surfaces_as_an_error(tmp_path):
    port = _free_port()
    context = mp.start_processes(_failing_worker, args=(2, port, str(tmp_path)), nprocs=2, join=False,
                                 start_method="spawn")
    for process in context.processes:
        process.join(90)
        assert not process.is_alive(), "a rank is still waiting: the failure did not surface"
    assert (tmp_path / "rank0.txt").read_text().startswith("raised")


def _verify_worker(rank, world, port, result_dir, corrupt):
    """Two-layer GCN over shard-only graphs with the oracle backend, then the bench's in-run
    verification; with `corrupt` the hidden rows one rank sends to its peers arrive damaged."""
    for path in (ROOT, os.path.join(ROOT, "tiga-lang_b200")):
        sys.path.insert(0, path)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import tiga as tg
        from baseline import synthetic as syn
        from baseline import verify
        from oracle import oracle
        from tiga.distributed import model
        from tiga.distributed.runtime import DistributedRuntime, ProcessGroupTransport

        class WeightedSum(tg.MessagePassing):
            reducer = tg.sum()

            def edge(self, src, dst, edge):
                return edge.weight * src.x

        scale, factor, F, seed = 9, 8, 8, 21
        n = 1 << scale
        first, last = model.owned_range(n, world, rank)
        row_ptr, col = syn.rmat_csr_rows(scale, factor, first, last, seed=seed, relabel=True)
        pieces = [torch.zeros(n // world, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(pieces, row_ptr.diff())
        degree = torch.cat(pieces)
        weight = syn.gcn_norm_weights_rows(row_ptr, col, degree, first).requires_grad_()
        x = syn.normal_rows(first, last, F, seed=seed + 1).requires_grad_()
        W1 = syn.normal((F, F), seed=3, std=F ** -0.5).requires_grad_()
        W2 = syn.normal((F, F), seed=4, std=F ** -0.5).requires_grad_()
        graph = tg.Graph.from_csr_shard(row_ptr, col, num_nodes=n, first_row=first).halo(tg.DeviceMesh("cpu", world))
        layer = WeightedSum()
        ones = torch.ones(last - first, F)
        class LossyBackend(OracleBackend):
            """Damages the rows rank 1 sends in the second exchange: a stand-in for a transport fault."""
            calls = 0

            def pack_rows(self, rows, ids):
                packed = rows.index_select(0, ids)
                type(self).calls += 1
                if corrupt and rank == 1 and type(self).calls > world - 1:
                    packed = packed + 1e-3
                return packed

        with DistributedRuntime(ProcessGroupTransport(), backend=LossyBackend(), waves=2):
            agg1 = layer(graph=graph, src={"x": x}, dst={}, edge={"weight": weight})
            h1 = agg1 @ W1
            agg2 = layer(graph=graph, src={"x": h1}, dst={}, edge={"weight": weight})
            out = agg2 @ W2
            dx, dw, dW1, dW2, d_agg1, d_h1, d_agg2 = torch.autograd.grad(
                out, (x, weight, W1, W2, agg1, h1, agg2), ones)
        dist.all_reduce(dW1)
        dist.all_reduce(dW2)
        tensors = {"agg1": agg1, "h1": h1, "agg2": agg2, "out": out, "d_agg1": d_agg1, "d_h1": d_h1,
                   "d_agg2": d_agg2, "dx": dx, "dw": dw, "dW1": dW1, "dW2": dW2}
        report = verify.check_two_layer_gcn(
            oracle, row_ptr=row_ptr, col_idx=col, first_row=first, num_nodes=n, weight=weight,
            feature_of=lambda ids: syn.normal_rows(0, 0, F, seed=seed + 1, ids=ids), tensors=tensors,
            linears=(W1, W2), world=world)
        with open(os.path.join(result_dir, f"rank{rank}.txt"), "w") as handle:
            handle.write(f"{int(report['ok'])} {report['worst']} {report['rows']} {report['edges']}")
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("corrupt", (False, True))
def test_in_run_verification_passes_and_detects_a_wrong_ghost_row(tmp_path, oracle, corrupt):
    world = 2
    mp.start_processes(_verify_worker, args=(world, _free_port(), str(tmp_path), corrupt), nprocs=world, join=True,
                       start_method="spawn")
    reports = [(tmp_path / f"rank{r}.txt").read_text().split(" ", 1) for r in range(world)]
    if corrupt:
        assert reports[0][0] == "0" and reports[0][1].startswith("agg2"), reports   # rank 0 read the damaged rows
    else:
        assert all(ok == "1" for ok, _ in reports), reports
