"""The torch.library operator facade: dispatcher op, fake tensor, autograd."""
import numpy as np
import pytest
import torch

import tiga as tg
from baseline import synthetic as syn
from tiga.library import register_message_passing

pytestmark = pytest.mark.gpu


class WeightedSum(tg.MessagePassing):
    reducer = tg.sum()

    def edge(self, src, dst, edge):
        return edge.weight * src.x


def test_registered_operator_matches_direct_call_and_differentiates(oracle):
    row_ptr, col = syn.rmat_csr(9, 8, seed=4)
    n = row_ptr.numel() - 1
    graph = tg.Graph.from_csr(row_ptr.cuda(), col.cuda(), num_src=n)
    x = syn.normal((n, 64), seed=1).cuda().requires_grad_()
    w = torch.rand(col.numel(), generator=torch.Generator().manual_seed(2)).cuda().requires_grad_()
    kernel = WeightedSum()
    op = register_message_passing(kernel, graph=graph, src={"x": x}, dst={}, edge={"weight": w}, name="wsum_test")
    assert op.qualified_name == "tiga::wsum_test" and op.bindings == (("src", "x"), ("edge", "weight"))
    assert register_message_passing(kernel, graph=graph, src={"x": x}, dst={}, edge={"weight": w},
                                    name="wsum_test") is op
    out = op(src={"x": x}, dst={}, edge={"weight": w})
    direct = kernel(graph=graph, src={"x": x}, dst={}, edge={"weight": w})
    assert torch.equal(out, direct)
    via_ops = torch.ops.tiga.wsum_test(graph.resolve_csr()[0], graph.resolve_csr()[1], x, w)
    assert torch.equal(via_ops, direct)
    dy = syn.normal((n, 64), seed=3).cuda()
    got = torch.autograd.grad(out, (x, w), dy)
    want = torch.autograd.grad(direct, (x, w), dy)
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    ref = oracle.wsum_fwd(row_ptr.numpy(), col.numpy(), x.detach().cpu().numpy(), w.detach().cpu().numpy())
    np.testing.assert_allclose(out.detach().cpu().numpy(), ref, rtol=1e-5, atol=1e-6)
    with pytest.raises(ValueError):
        op(src={"y": x}, dst={}, edge={"weight": w})


def test_fake_tensor_and_schema_checks():
    row_ptr, col = syn.fixed_degree_graph(64, 4, seed=5)
    graph = tg.Graph.from_csr(row_ptr.cuda(), col.cuda(), num_src=64)
    x = torch.randn(64, 16, device="cuda", requires_grad=True)
    w = torch.rand(256, device="cuda", requires_grad=True)
    op = register_message_passing(WeightedSum(), graph=graph, src={"x": x}, dst={}, edge={"weight": w},
                                  name="wsum_opcheck")
    results = op.opcheck(x, w)
    assert all(status == "SUCCESS" for status in results.values()), results
