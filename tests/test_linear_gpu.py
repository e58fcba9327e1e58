"""Tensor-core (tcgen05, 3xTF32) dense linear against the float64-accumulating
CPU oracle.  Tolerance: rel 1e-5 / abs 1e-6 plus 4 ulp of sum_k |a_k * w_k| -- the
rounding any float32 summation order may introduce (the tensor core adds its
K = 8 partial products into the float32 accumulator with round-toward-zero)."""
import numpy as np
import pytest
import torch

from tiga import ops
from baseline import synthetic as syn

pytestmark = pytest.mark.gpu


def assert_gemm_close(got, a, w, ref):
    magnitude = np.abs(a).astype(np.float64) @ np.abs(w).astype(np.float64)
    bound = 1e-5 * np.abs(ref) + 1e-6 + 4 * np.finfo(np.float32).eps * magnitude
    error = np.abs(got.astype(np.float64) - ref)
    assert np.all(error <= bound), f"max excess {np.max(error - bound)} at {np.argmax(error - bound)}"


@pytest.mark.parametrize("M", (1, 127, 128, 129, 1000, 40000))
@pytest.mark.parametrize("K,N", ((128, 128), (64, 64), (32, 128), (96, 64)))
def test_forward_matches_oracle(oracle, M, K, N):
    a = syn.normal((M, K), seed=M + K)
    w = syn.normal((K, N), seed=N, std=K ** -0.5)
    out = ops.dense_linear(a.cuda(), w.cuda())
    ops.check_async_errors()
    ref = oracle.linear(a.numpy(), w.numpy())
    assert_gemm_close(out.cpu().numpy(), a.numpy(), w.numpy(), ref)


def test_values_that_stress_the_split(oracle):
    # large dynamic range and exact small integers: a plain tf32 product would lose these
    M, K, N = 300, 128, 128
    gen = torch.Generator().manual_seed(3)
    a = torch.randn(M, K, generator=gen) * torch.logspace(-3, 3, K)
    w = torch.randn(K, N, generator=gen)
    out = ops.dense_linear(a.cuda(), w.cuda())
    ref = oracle.linear(a.numpy(), w.numpy())
    scale = np.abs(a.numpy()) @ np.abs(w.numpy())
    assert np.all(np.abs(out.cpu().numpy() - ref) <= 1e-6 * scale + 1e-6)
    a = torch.randint(-2048, 2048, (M, K), generator=gen).float() + 0.5     # needs > 10 mantissa bits
    out = ops.dense_linear(a.cuda(), torch.eye(K).cuda())
    np.testing.assert_array_equal(out.cpu().numpy(), a.numpy())
    ops.check_async_errors()


@pytest.mark.parametrize("K,N", ((128, 128), (64, 64), (64, 128), (128, 64)))
def test_backward_matches_oracle(oracle, K, N):
    M = 5000
    a = syn.normal((M, K), seed=1)
    w = syn.normal((K, N), seed=2, std=K ** -0.5)
    dy = syn.normal((M, N), seed=3)
    ag, wg = a.cuda().requires_grad_(), w.cuda().requires_grad_()
    out = ops.dense_linear(ag, wg)
    da, dw = torch.autograd.grad(out, (ag, wg), dy.cuda())
    ops.check_async_errors()
    wt = w.t().contiguous().numpy()
    assert_gemm_close(da.cpu().numpy(), dy.numpy(), wt, oracle.linear(dy.numpy(), wt))
    ref_dw = oracle.linear(a.t().contiguous().numpy(), dy.numpy())
    assert_gemm_close(dw.cpu().numpy(), a.t().contiguous().numpy(), dy.numpy(), ref_dw)


@pytest.mark.parametrize("M", (1, 31, 32, 33, 4777, 200000))
@pytest.mark.parametrize("K,N", ((128, 64), (128, 128), (64, 64), (32, 128), (96, 64)))
def test_weight_gradient_kernel(oracle, M, K, N):
    a = syn.normal((M, K), seed=M)
    dy = syn.normal((M, N), seed=M + 1)
    dw = ops._linear_dw_raw(a.cuda(), dy.cuda())
    again = ops._linear_dw_raw(a.cuda(), dy.cuda())
    ops.check_async_errors()
    assert torch.equal(dw, again)                      # deterministic split-K
    ref = oracle.linear(a.t().contiguous().numpy(), dy.numpy())
    assert_gemm_close(dw.cpu().numpy(), a.t().contiguous().numpy(), dy.numpy(), ref)


def test_unsupported_shapes_raise():
    with pytest.raises(NotImplementedError):
        ops.dense_linear(torch.zeros(4, 100, device="cuda"), torch.zeros(100, 128, device="cuda"))
    with pytest.raises(NotImplementedError):     # K = 32 has no d(a) kernel: refused up front, never a library fallback
        ops.dense_linear(torch.zeros(4, 32, device="cuda", requires_grad=True), torch.zeros(32, 128, device="cuda"))


def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable(oracle):
    """A bounded wait that gives up must end the kernel with an error code, not hang: the self-test
    kernel waits 4096 polls on a barrier nothing signals.  The code then surfaces through the error
    word (here by the explicit check, in product use at the next tensor-core call), and the next
    real kernel on the same context is correct."""
    import ctypes

    from tiga import _native

    device = torch.device("cuda", torch.cuda.current_device())
    ops.check_async_errors()
    word = ops.error_flag(device)
    fell_through = torch.zeros(1, dtype=torch.int32, device=device)
    status = _native.lib().tgb_selftest_bounded_wait(word.data_ptr(), ctypes.c_uint32(4096), fell_through.data_ptr(),
                                                     torch.cuda.current_stream().cuda_stream)
    assert status == _native.OK
    ops.launched(device)
    torch.cuda.synchronize()
    assert int(fell_through.item()) == 1                   # the second wait returned at once
    with pytest.raises(RuntimeError, match="code 99"):
        ops.error_flag(device)                             # what the next launch would do first
    ops.check_async_errors()                               # the word was cleared when it was reported
    a = syn.normal((1000, 64), seed=1)
    w = syn.normal((64, 64), seed=2, std=0.125)
    out = ops.dense_linear(a.cuda(), w.cuda())
    ops.check_async_errors()
    assert_gemm_close(out.cpu().numpy(), a.numpy(), w.numpy(), oracle.linear(a.numpy(), w.numpy()))
    assert _native.lib().tgb_selftest_bounded_wait(word.data_ptr(), ctypes.c_uint32(0), fell_through.data_ptr(),
                                                   0) == _native.INVALID_ARGUMENT


def test_matmul_written_in_node_runs_on_the_tensor_core_kernels(oracle):
    """`aggregate @ W` inside node() (the reference's GCN example) launches this library's linear
    kernels, forward and backward, not a library GEMM; other shapes fall through to Torch."""
    import tiga as tg
    from baseline import synthetic as syn
    from tiga import _native

    class Layer(tg.MessagePassing):
        reducer = tg.sum()

        def edge(self, src, dst, edge):
            return edge.weight * src.x

        def node(self, dst, aggregate, W):
            return aggregate @ W

    row_ptr, col = syn.rmat_csr(10, 8, seed=3)
    n = row_ptr.numel() - 1
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(n, 64, generator=gen).cuda().requires_grad_()
    w = torch.rand(col.numel(), generator=gen).cuda()
    W = (torch.randn(64, 128, generator=gen) / 8).cuda().requires_grad_()
    graph = tg.Graph.from_csr(row_ptr.cuda(), col.cuda(), num_src=n)
    layer = Layer()
    layer(graph=graph, src={"x": x}, dst={}, edge={"weight": w}, W=W)          # specialise
    before = _native.launch_count()
    out = layer(graph=graph, src={"x": x}, dst={}, edge={"weight": w}, W=W)
    forward_launches = _native.launch_count() - before
    assert type(out) is torch.Tensor and out.shape == (n, 128)
    assert forward_launches >= 2                      # the gather and the linear are both this library's
    agg = oracle.wsum_fwd(row_ptr.numpy(), col.numpy(), x.detach().cpu().numpy(), w.cpu().numpy())
    want = oracle.linear(agg, W.detach().cpu().numpy())
    np.testing.assert_allclose(out.detach().cpu().numpy(), want, rtol=2e-5, atol=2e-5 * np.abs(want).max())
    before = _native.launch_count()
    dx, dW = torch.autograd.grad(out, (x, W), torch.ones_like(out))
    assert _native.launch_count() - before >= 4       # d(aggregate), dW (+ its partial sum), dx gather
    ref_x, ref_W = x.detach().clone().requires_grad_(), W.detach().clone().requires_grad_()
    ref = Layer().reference(graph=graph, src={"x": ref_x}, dst={}, edge={"weight": w[:, None]}, W=ref_W)
    want_dx, want_dW = torch.autograd.grad(ref, (ref_x, ref_W), torch.ones_like(ref))
    torch.testing.assert_close(dx, want_dx, rtol=1e-4, atol=1e-4 * float(want_dx.abs().max()))
    torch.testing.assert_close(dW, want_dW, rtol=1e-4, atol=1e-4 * float(want_dW.abs().max()))
    # a width the kernels do not take: plain Torch, same answer as Torch
    W3 = torch.randn(64, 3, device="cuda")
    out3 = layer(graph=graph, src={"x": x}, dst={}, edge={"weight": w}, W=W3)
    torch.testing.assert_close(out3, layer.reference(graph=graph, src={"x": x}, dst={}, edge={"weight": w[:, None]}, W=W3),
                               rtol=1e-4, atol=1e-4)
