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


def _worker(rank, world, port, result_dir):
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
        n, F = row_ptr.numel() - 1, 64
        x = syn.normal((n, F), seed=5).to(device)                      # CPU generator, so the test can replay it
        w = syn.gcn_norm_weights(row_ptr.cpu(), col.cpu()).to(device)
        dy = syn.normal((n, F), seed=6).to(device)
        graph = tg.Graph.from_csr(row_ptr, col, num_src=n).halo(tg.DeviceMesh("cuda", world))
        runtime = DistributedRuntime(NCCLTransport(device=device))
        with runtime:
            shard = shard_plan_for(graph, runtime)
            b, e = shard.begin, shard.end
            lo, hi = int(row_ptr[b]), int(row_ptr[e])
            xs = x[b:e].clone().requires_grad_()
            ws = w[lo:hi].clone().requires_grad_()
            for _ in range(2):     # second call reuses the cached shard plan
                out = WeightedSum()(graph=graph, src={"x": xs}, dst={}, edge={"weight": ws})
                dx, dw = torch.autograd.grad(out, (xs, ws), dy[b:e])
        torch.cuda.synchronize()
        np.savez(os.path.join(result_dir, f"rank{rank}.npz"), begin=b, end=e, lo=lo, hi=hi,
                 out=out.detach().cpu().numpy(), dx=dx.cpu().numpy(), dw=dw.cpu().numpy())
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_halo_matches_oracle(tmp_path, oracle):
    world = 2
    mp.start_processes(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True,
                       start_method="spawn")
    from baseline import synthetic as syn

    row_ptr, col = syn.rmat_csr(11, 12, seed=13)
    n, F = row_ptr.numel() - 1, 64
    x = syn.normal((n, F), seed=5).numpy()
    w = syn.gcn_norm_weights(row_ptr, col).numpy()
    dy = syn.normal((n, F), seed=6).numpy()
    ref_out = oracle.wsum_fwd(row_ptr.numpy(), col.numpy(), x, w)
    ref_dx = oracle.wsum_bwd_dx(row_ptr.numpy(), col.numpy(), n, dy, w)
    ref_dw = oracle.wsum_bwd_dw(row_ptr.numpy(), col.numpy(), dy, x)
    covered = 0
    for rank in range(world):
        data = np.load(tmp_path / f"rank{rank}.npz")
        b, e, lo, hi = int(data["begin"]), int(data["end"]), int(data["lo"]), int(data["hi"])
        covered += e - b
        np.testing.assert_allclose(data["out"], ref_out[b:e], rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(data["dx"], ref_dx[b:e], rtol=1e-5, atol=2e-6)
        np.testing.assert_allclose(data["dw"], ref_dw[lo:hi], rtol=1e-4, atol=1e-5)
    assert covered == n
