"""GPU parity of the online-softmax reducer with per-edge scores and per-source values
(``edge(): return self.reducer(edge.score, src.value)``) against the fixture generated from the
unmodified reference and against the CPU oracle.

Tolerances: float32 state, so forward rel 1e-5 / abs 1e-6; gradients rel 1e-4 / abs 1e-6 (the
tolerance the oracle itself is pinned with on this fixture); bf16 values rel 2e-2."""
import numpy as np
import pytest
import torch

import tiga as tg
from baseline import synthetic as syn

pytestmark = pytest.mark.gpu


class Softmax(tg.MessagePassing):
    reducer = tg.online_softmax()

    def edge(self, src, dst, edge):
        return self.reducer(edge.score, src.value)


def test_reference_fixture_with_extreme_scores_and_an_empty_row(golden):
    # scores of +-1000 in two rows, 2 heads x 3 payload values, row 1 has no edges
    row_ptr = torch.from_numpy(golden["softmax_row_ptr"]).cuda()
    col = torch.from_numpy(golden["softmax_col"]).cuda()
    score = torch.from_numpy(golden["softmax_score"]).cuda().requires_grad_()
    value = torch.from_numpy(golden["softmax_value"]).cuda().requires_grad_()
    graph = tg.Graph.from_csr(row_ptr, col, num_src=value.shape[0])
    kernel = Softmax()
    out = kernel(graph=graph, src={"value": value}, dst={}, edge={"score": score})
    assert out.shape == (4, 2, 3) and out.dtype == torch.float32
    np.testing.assert_allclose(out.detach().cpu().numpy(), golden["softmax_out"], rtol=1e-5, atol=1e-6)
    assert torch.all(out[1] == 0)                      # a row without edges is exactly zero
    assert "stable-weighted" in kernel.last_variant.lowering
    d_score, d_value = torch.autograd.grad(out, (score, value), torch.from_numpy(golden["softmax_dy"]).cuda())
    np.testing.assert_allclose(d_score.cpu().numpy(), golden["softmax_dscore"], rtol=1e-4, atol=1e-6)
    np.testing.assert_allclose(d_value.cpu().numpy(), golden["softmax_dvalue"], rtol=1e-4, atol=1e-6)
    # the second call takes the guarded warm path and must give the same bits
    again = kernel(graph=graph, src={"value": value}, dst={}, edge={"score": score})
    assert torch.equal(again, out) and kernel.cache_info["hits"] >= 1


@pytest.mark.parametrize("lanes,payload,index_dtype", (((4,), (16,), torch.int64), ((), (), torch.int32),
                                                       ((2,), (3,), torch.int64), ((3,), (100,), torch.int32),
                                                       ((40,), (9,), torch.int64)))
def test_rmat_against_oracle(oracle, lanes, payload, index_dtype):
    row_ptr, col = syn.rmat_csr(10, 12, seed=23, symmetrize=False)       # hubs, empty rows, duplicates removed
    n, E = row_ptr.numel() - 1, col.numel()
    gen = torch.Generator().manual_seed(5)
    score = torch.randn((E, *lanes), generator=gen) * 3.0
    value = torch.randn((n, *lanes, *payload), generator=gen)
    dy = torch.randn((n, *lanes, *payload), generator=gen)
    graph = tg.Graph.from_csr(row_ptr.to(index_dtype).cuda(), col.to(index_dtype).cuda(), num_src=n)
    sg, vg = score.cuda().requires_grad_(), value.cuda().requires_grad_()
    out = Softmax()(graph=graph, src={"value": vg}, dst={}, edge={"score": sg})
    d_score, d_value = torch.autograd.grad(out, (sg, vg), dy.cuda())
    H = int(np.prod(lanes)) if lanes else 1
    D = int(np.prod(payload)) if payload else 1
    s2, v2 = score.reshape(E, H).numpy(), value.reshape(n, H, D).numpy()
    ref, _, _ = oracle.online_softmax_fwd(row_ptr.numpy(), s2, v2[col.numpy()])
    ref_ds, ref_dv_edge = oracle.online_softmax_bwd(row_ptr.numpy(), s2, v2[col.numpy()], ref,
                                                    dy.reshape(n, H, D).numpy())
    ref_dv = np.zeros_like(v2)
    np.add.at(ref_dv, col.numpy(), ref_dv_edge)
    np.testing.assert_allclose(out.detach().cpu().numpy().reshape(n, H, D), ref, rtol=1e-5, atol=2e-6)
    np.testing.assert_allclose(d_score.cpu().numpy().reshape(E, H), ref_ds, rtol=1e-4, atol=2e-5)
    np.testing.assert_allclose(d_value.cpu().numpy().reshape(n, H, D), ref_dv, rtol=1e-4, atol=2e-5)
    empty = (row_ptr.diff() == 0).numpy()
    assert empty.any() and np.all(out.detach().cpu().numpy().reshape(n, -1)[empty] == 0)


def test_bf16_values_and_trailing_singleton_scores(oracle):
    row_ptr, col = syn.rmat_csr(9, 8, seed=3, symmetrize=False)
    n, E, H, D = row_ptr.numel() - 1, col.numel(), 4, 32
    gen = torch.Generator().manual_seed(11)
    score = torch.randn((E, H, 1), generator=gen)                 # the trailing 1 is squeezed away
    value = torch.randn((n, H, D), generator=gen).to(torch.bfloat16)
    graph = tg.Graph.from_csr(row_ptr.cuda(), col.cuda(), num_src=n)
    sg, vg = score.cuda().requires_grad_(), value.cuda().requires_grad_()
    out = Softmax()(graph=graph, src={"value": vg}, dst={}, edge={"score": sg})
    assert out.dtype == torch.bfloat16 and out.shape == (n, H, D)
    ref, _, _ = oracle.online_softmax_fwd(row_ptr.numpy(), score.reshape(E, H).numpy(),
                                          value.float().numpy()[col.numpy()])
    np.testing.assert_allclose(out.detach().float().cpu().numpy(), ref, rtol=2e-2, atol=2e-2)
    d_score, d_value = torch.autograd.grad(out, (sg, vg), torch.ones_like(out))
    assert d_score.shape == score.shape and d_value.dtype == torch.bfloat16
    # softmax weights of a row sum to one, so the score cotangents of every (row, head) sum to ~0
    destination = torch.repeat_interleave(torch.arange(n), row_ptr.diff()).cuda()
    per_row = torch.zeros((n, H), device="cuda").index_add_(0, destination, d_score.reshape(E, H).float())
    scale = torch.zeros((n, H), device="cuda").index_add_(0, destination, d_score.reshape(E, H).float().abs())
    assert torch.all(per_row.abs() <= 2e-2 * scale + 1e-3)


def test_other_online_softmax_programs_take_the_algebra_kernels_or_raise():
    """A score EXPRESSION (not a stored field) with one score per edge runs through the interpreting
    algebra kernels; several score lanes per edge against a payload have no kernel and raise."""
    class Scaled(tg.MessagePassing):
        reducer = tg.online_softmax()

        def edge(self, src, dst, edge):
            return self.reducer(edge.score * 2.0, src.value)

    row_ptr = torch.tensor([0, 2, 3]).cuda()
    col = torch.tensor([1, 0, 0]).cuda()
    graph = tg.Graph.from_csr(row_ptr, col, num_src=2)
    value = torch.randn(2, 4, device="cuda", generator=torch.Generator("cuda").manual_seed(3))
    score = torch.tensor([0.3, -0.2, 0.9], device="cuda")
    kernel = Scaled()
    got = kernel(graph=graph, src={"value": value}, dst={}, edge={"score": score})
    assert kernel.last_variant.lowering == "b200-csr-algebra-tile"
    want = Scaled().reference(graph=tg.Graph.from_csr(row_ptr.cpu(), col.cpu(), num_src=2), src={"value": value.cpu()},
                              dst={}, edge={"score": score.cpu()})
    torch.testing.assert_close(got.cpu(), want, rtol=1e-5, atol=1e-6)
    with pytest.raises(NotImplementedError):
        Scaled()(graph=graph, src={"value": torch.zeros(2, 2, 4, device="cuda")}, dst={},
                 edge={"score": torch.zeros(3, 2, device="cuda")})
