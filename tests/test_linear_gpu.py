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
