"""Two ranks on two GPUs over NCCL: the halo-exchange path with the native CUDA
backend against the single-process CPU oracle.  Skipped on a one-GPU box."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir, shard_only=False, waves=1, index_dtype=torch.int64, F=64, push=False):
    for path in (ROOT, os.path.join(ROOT, "tiga-lang_b200")):
        sys.path.insert(0, path)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        import tiga as tg
        from baseline import synthetic as syn
        from tiga.distributed.runtime import DistributedRuntime, NCCLTransport, shard_plan_for

        class WeightedSum(tg.MessagePassing):
            reducer = tg.sum()

            def edge(self, src, dst, edge):
                return edge.weight * src.x

        row_ptr, col = syn.rmat_csr(11, 12, seed=13, device=device)   # integer generator: same on CPU and GPU
        n = row_ptr.numel() - 1
        x = syn.normal((n, F), seed=5).to(device)                      # CPU generator, so the test can replay it
        w = syn.gcn_norm_weights(row_ptr.cpu(), col.cpu()).to(device)
        dy = syn.normal((n, F), seed=6).to(device)
        if shard_only:       # every rank holds its own block of rows only
            from tiga.distributed.model import owned_range

            first, last = owned_range(n, world, rank)
            block_ptr, block_col = syn.rmat_csr_rows(11, 12, first, last, seed=13, device=device)
            graph = tg.Graph.from_csr_shard(block_ptr.to(index_dtype), block_col.to(index_dtype), num_nodes=n,
                                            first_row=first).halo(tg.DeviceMesh("cuda", world))
        else:
            graph = tg.Graph.from_csr(row_ptr.to(index_dtype), col.to(index_dtype), num_src=n).halo(
                tg.DeviceMesh("cuda", world))
        runtime = DistributedRuntime(NCCLTransport(device=device), waves=waves, push=push)
        with runtime:
            shard = shard_plan_for(graph, runtime)
            b, e = shard.begin, shard.end
            lo, hi = int(row_ptr[b]), int(row_ptr[e])
            xs = x[b:e].clone().requires_grad_()
            ws = w[lo:hi].clone().requires_grad_()
            for _ in range(3 if push else 2):     # later calls reuse the cached shard plan (and window slots)
                out = WeightedSum()(graph=graph, src={"x": xs}, dst={}, edge={"weight": ws})
                dx, dw = torch.autograd.grad(out, (xs, ws), dy[b:e])
        torch.cuda.synchronize()
        np.savez(os.path.join(result_dir, f"rank{rank}.npz"), begin=b, end=e, lo=lo, hi=hi,
                 out=out.detach().cpu().numpy(), dx=dx.cpu().numpy(), dw=dw.cpu().numpy())
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _run_and_compare(tmp_path, oracle, world, shard_only, waves, index_dtype, F, push=False):
    from conftest import assert_sum_close

    mp.start_processes(_worker, args=(world, _free_port(), str(tmp_path), shard_only, waves, index_dtype, F, push),
                       nprocs=world, join=True, start_method="spawn")
    from baseline import synthetic as syn

    row_ptr, col = syn.rmat_csr(11, 12, seed=13)
    n = row_ptr.numel() - 1
    x = syn.normal((n, F), seed=5).numpy()
    w = syn.gcn_norm_weights(row_ptr, col).numpy()
    dy = syn.normal((n, F), seed=6).numpy()
    rp, ci = row_ptr.numpy(), col.numpy()
    ref_out = oracle.wsum_fwd(rp, ci, x, w)
    ref_dx = oracle.wsum_bwd_dx(rp, ci, n, dy, w)
    ref_dw = oracle.wsum_bwd_dw(rp, ci, dy, x)
    # magnitudes (sum of |terms|) for the float32 tolerance of the single-GPU tests
    mag_out = oracle.wsum_fwd(rp, ci, np.abs(x), np.abs(w))
    mag_dx = oracle.wsum_bwd_dx(rp, ci, n, np.abs(dy), np.abs(w))
    mag_dw = oracle.wsum_bwd_dw(rp, ci, np.abs(dy), np.abs(x))
    covered = 0
    for rank in range(world):
        data = np.load(tmp_path / f"rank{rank}.npz")
        b, e, lo, hi = int(data["begin"]), int(data["end"]), int(data["lo"]), int(data["hi"])
        covered += e - b
        assert_sum_close(data["out"], ref_out[b:e], mag_out[b:e])
        assert_sum_close(data["dx"], ref_dx[b:e], mag_dx[b:e])
        assert_sum_close(data["dw"], ref_dw[lo:hi], mag_dw[lo:hi])
    assert covered == n


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("shard_only,index_dtype,F", ((False, torch.int64, 64), (True, torch.int32, 64),
                                                      (True, torch.int64, 6)))
def test_two_gpu_halo_matches_oracle(tmp_path, oracle, shard_only, index_dtype, F):
    _run_and_compare(tmp_path, oracle, 2, shard_only, 1, index_dtype, F)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs four GPUs")
def test_four_gpu_halo_in_waves_matches_oracle(tmp_path, oracle):
    _run_and_compare(tmp_path, oracle, 4, True, 3, torch.int64, 64)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("F", (64, 6))
def test_two_gpu_halo_through_peer_windows_matches_oracle(tmp_path, oracle, F):
    """push=True: halo rows are stored straight into the peer's ghost buffer (CUDA IPC window), the
    cotangents straight into the owner's landing window; signals are one-element all-reduces."""
    _run_and_compare(tmp_path, oracle, 2, True, 1, torch.int64, F, push=True)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs four GPUs")
def test_four_gpu_halo_through_peer_windows_in_waves_matches_oracle(tmp_path, oracle):
    _run_and_compare(tmp_path, oracle, 4, True, 3, torch.int64, 64, push=True)
