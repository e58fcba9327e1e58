"""Row-paged execution of a persistent (.gfg) graph on the GPU: page by page through the native
kernels, same results as the resident graph, gradients included."""
import numpy as np
import pytest
import torch

import tiga as tg
from baseline import synthetic as syn

pytestmark = pytest.mark.gpu


class Biased(tg.MessagePassing):
    reducer = tg.sum()

    def edge(self, src, dst, edge):
        return edge.weight * src.x

    def node(self, dst, aggregate):
        return aggregate + dst.bias


class Softmax(tg.MessagePassing):
    reducer = tg.online_softmax()

    def edge(self, src, dst, edge):
        return self.reducer(edge.score, src.value)


@pytest.mark.parametrize("page_rows", (100, 1024, 1 << 20))
def test_paged_weighted_sum_equals_resident(tmp_path, oracle, page_rows):
    row_ptr, col = syn.rmat_csr(11, 12, seed=17)                    # hubs longer than a page of 100 rows' edges
    n, E, F = row_ptr.numel() - 1, col.numel(), 32
    gen = torch.Generator().manual_seed(2)
    x, w, bias = torch.randn(n, F, generator=gen), torch.rand(E, generator=gen), torch.randn(n, F, generator=gen)
    resident = tg.Graph.from_csr(row_ptr.cuda(), col.cuda(), num_src=n)
    tg.save(resident, tmp_path / "g.gfg", fields={"edge": {"weight": w}})
    paged = tg.load(tmp_path / "g.gfg", device="cuda")
    paged.page_rows = page_rows
    assert paged.schema.realization == "paged_csr" and paged.num_edges == E
    xg, wg = x.cuda().requires_grad_(), paged.fields("edge")["weight"].requires_grad_()
    assert torch.equal(wg.detach().cpu(), w)
    kernel = Biased()
    out = kernel(graph=paged, src={"x": xg}, dst={"bias": bias.cuda()}, edge={"weight": wg})
    x2, w2 = x.cuda().requires_grad_(), w.cuda().requires_grad_()
    want = Biased()(graph=resident, src={"x": x2}, dst={"bias": bias.cuda()}, edge={"weight": w2})
    assert torch.equal(out, want)                                    # same kernels, same row order: same bits
    ref = oracle.wsum_fwd(row_ptr.numpy(), col.numpy(), x.numpy(), w.numpy()) + bias.numpy()
    np.testing.assert_allclose(out.detach().cpu().numpy(), ref, rtol=1e-5, atol=1e-5)
    dy = torch.randn(n, F, generator=gen).cuda()
    got = torch.autograd.grad(out, (xg, wg), dy)
    expect = torch.autograd.grad(want, (x2, w2), dy)
    torch.testing.assert_close(got[0], expect[0], rtol=1e-5, atol=1e-5)     # dx: pages add in another order
    assert torch.equal(got[1], expect[1])                                   # dw: per edge, page-local
    assert paged._row_ptr is None                                           # the topology was never materialised


def test_paged_field_softmax_equals_resident(tmp_path):
    row_ptr, col = syn.rmat_csr(9, 8, seed=5, symmetrize=False)
    n, E = row_ptr.numel() - 1, col.numel()
    gen = torch.Generator().manual_seed(4)
    score, value = torch.randn(E, 2, generator=gen).cuda(), torch.randn(n, 2, 8, generator=gen).cuda()
    resident = tg.Graph.from_csr(row_ptr.cuda(), col.cuda(), num_src=n)
    tg.save(resident, tmp_path / "s.gfg")
    paged = tg.load(tmp_path / "s.gfg", device="cuda")
    paged.page_rows = 64
    out = Softmax()(graph=paged, src={"value": value}, dst={}, edge={"score": score})
    want = Softmax()(graph=resident, src={"value": value}, dst={}, edge={"score": score})
    assert torch.equal(out, want)


def test_paged_graph_needs_a_cuda_device(tmp_path):
    resident = tg.Graph.from_csr(torch.tensor([0, 1, 2]), torch.tensor([1, 0]), num_src=2)
    tg.save(resident, tmp_path / "c.gfg")
    with pytest.raises(NotImplementedError):
        Biased()(graph=tg.load(tmp_path / "c.gfg"), src={"x": torch.zeros(2, 4)}, dst={"bias": torch.zeros(2, 4)},
                 edge={"weight": torch.zeros(2)})
