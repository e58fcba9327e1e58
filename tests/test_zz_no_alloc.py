"""The allocation-free forward entry point against the regular one.

`tgb_csr_wsum_fwd_noalloc` serves callers that cannot allocate device memory
where they need the aggregation (no cudaMalloc allowed in that region, or no
allocator handed to a plug-in): its scratch for split rows is a fixed array
inside the library.  The test drives it through the C ABI exactly as such a
caller would -- raw pointers, no scratch argument -- and requires the same bits
as `tgb_csr_reduce_fwd` on two calls in a row (the second with other inputs, so
stale scratch contents would show), then checks that a graph beyond the fixed
capacity is refused with a clear message.  This file is collected last on
purpose."""
import ctypes

import numpy as np
import pytest
import torch

import tiga as tg
from tiga import _native, ops
from baseline import synthetic as syn

pytestmark = pytest.mark.gpu


def _call_noalloc(plan, x, w, identity=0.0):
    out = torch.full((plan.num_dst, x.shape[1]), float("nan"), dtype=torch.float32, device=x.device)
    status = _native.lib().tgb_csr_wsum_fwd_noalloc(
        plan.handle, x.data_ptr(), 0 if w is None else w.data_ptr(), out.data_ptr(), x.shape[1], identity,
        torch.cuda.current_stream().cuda_stream)
    return status, out


def test_noalloc_matches_regular_entry_point_twice():
    row_ptr, col = syn.rmat_csr(12, 16, seed=31)               # hubs well above the split threshold
    n = row_ptr.numel() - 1
    g = tg.Graph.from_csr(row_ptr.cuda(), col.cuda(), num_src=n)
    plan = g.native_plan(transpose=False)
    assert plan.info["segments"] > 0, "the case must exercise the scratch array"
    for seed, F in ((1, 128), (2, 128), (3, 64), (4, 5)):
        x = syn.normal((n, F), seed=seed).cuda()
        w = torch.rand(col.numel(), generator=torch.Generator().manual_seed(seed)).cuda()
        expect, _ = ops.csr_reduce_forward(plan, "sum", x, w, 0.25)
        status, got = _call_noalloc(plan, x, w, 0.25)
        assert status == _native.OK, _native.lib().tgb_last_error()
        torch.cuda.synchronize()
        np.testing.assert_array_equal(got.cpu().numpy(), expect.cpu().numpy())
    # unweighted message, int32 indices
    g32 = tg.Graph.from_csr(row_ptr.int().cuda(), col.int().cuda(), num_src=n)
    plan32 = g32.native_plan(transpose=False)
    x = syn.normal((n, 32), seed=9).cuda()
    expect, _ = ops.csr_reduce_forward(plan32, "sum", x, None, 0.0)
    status, got = _call_noalloc(plan32, x, None)
    assert status == _native.OK
    np.testing.assert_array_equal(got.cpu().numpy(), expect.cpu().numpy())


def test_noalloc_refuses_graphs_beyond_its_capacity():
    rows, degree, F = 2048, 1024, 512                          # 8192 segments x 512 floats > 2 Mi floats
    row_ptr, col = syn.fixed_degree_graph(rows, degree, seed=3)
    g = tg.Graph.from_csr(row_ptr.cuda(), col.cuda(), num_src=rows)
    plan = g.native_plan(transpose=False)
    assert plan.info["segments"] * F > (2 << 20)
    x = torch.zeros((rows, F), device="cuda")
    status, _ = _call_noalloc(plan, x, None)
    assert status == _native.UNSUPPORTED
    message = _native.lib().tgb_last_error().decode()
    assert "built-in scratch" in message and str(plan.info["segments"]) in message
    # the same graph is fine with a narrower feature row
    x = syn.normal((rows, 64), seed=1).cuda()
    expect, _ = ops.csr_reduce_forward(plan, "sum", x, None, 0.0)
    status, got = _call_noalloc(plan, x, None)
    assert status == _native.OK
    np.testing.assert_array_equal(got.cpu().numpy(), expect.cpu().numpy())


def test_noalloc_honours_a_plan_edge_map():
    """A plan whose edges address the caller's weight array through an edge map (the halo runtime's
    sub-relations do) must read w[map[e]] in the allocation-free entry point too."""
    from tiga.plan import CSRPlan

    row_ptr, col = syn.rmat_csr(11, 16, seed=7)
    n, E = row_ptr.numel() - 1, col.numel()
    perm = torch.randperm(E, generator=torch.Generator().manual_seed(1)).to(torch.int32)
    plan = CSRPlan(row_ptr.cuda(), col.cuda(), n, transpose=False, edge_map=perm)
    assert plan.info["segments"] > 0
    x = syn.normal((n, 64), seed=2).cuda()
    w = torch.rand(E, generator=torch.Generator().manual_seed(3)).cuda()
    expect, _ = ops.csr_reduce_forward(plan, "sum", x, w, 0.0)
    status, got = _call_noalloc(plan, x, w)
    assert status == _native.OK, _native.lib().tgb_last_error()
    torch.cuda.synchronize()
    np.testing.assert_array_equal(got.cpu().numpy(), expect.cpu().numpy())
    # and that really is the mapped weight: the same sums from a plan without a map and w gathered by hand
    plain = CSRPlan(row_ptr.cuda(), col.cuda(), n, transpose=False)
    by_hand, _ = ops.csr_reduce_forward(plain, "sum", x, w[perm.long().cuda()], 0.0)
    np.testing.assert_array_equal(got.cpu().numpy(), by_hand.cpu().numpy())
