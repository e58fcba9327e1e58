"""Dense-relation (varlen causal / full) attention on the tensor cores against
the float64 CPU oracle.  Tolerance: bf16 attention within rel 2e-2 (abs 2e-2)."""
import numpy as np
import pytest
import torch

import tiga as tg
from tiga import ops

pytestmark = pytest.mark.gpu


class Attention(tg.MessagePassing):
    reducer = tg.online_softmax()

    def edge(self, src, dst, edge, scale):
        score = (src.key * dst.query).sum(dim=-1) * scale
        return self.reducer(score, src.value)


def make_inputs(lengths, H, D, seed):
    gen = torch.Generator().manual_seed(seed)
    T = sum(lengths)
    q, k, v = (torch.randn(T, H, D, generator=gen).to(torch.bfloat16) for _ in range(3))
    cu = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int64)
    return q, k, v, cu


@pytest.mark.parametrize("lengths,H,D", (
    ([5, 1, 9, 16], 2, 128),            # shorter than one tile
    ([128], 1, 128),                    # exactly one tile
    ([300, 129, 127, 513], 2, 128),     # several key blocks, ragged ends
    ([700, 40], 3, 64),
))
@pytest.mark.parametrize("causal", (True, False))
def test_forward_matches_oracle(oracle, lengths, H, D, causal):
    q, k, v, cu = make_inputs(lengths, H, D, seed=len(lengths) + D)
    scale = D ** -0.5
    graph = tg.Graph.cu_seqlens(cu.cuda(), causal=causal)
    kernel = Attention()
    out = kernel(graph=graph, src={"key": k.cuda(), "value": v.cuda()}, dst={"query": q.cuda()}, scale=scale)
    ops.check_async_errors()
    assert out.dtype == torch.bfloat16 and out.shape == q.shape
    assert "tcgen05" in kernel.last_variant.lowering
    ref, lse = oracle.varlen_attn_fwd(cu.numpy(), q.float().numpy(), k.float().numpy(), v.float().numpy(), scale,
                                      causal=causal)
    np.testing.assert_allclose(out.float().cpu().numpy(), ref, rtol=2e-2, atol=2e-2)


def test_cat_of_triangular_blocks_is_the_same_relation(oracle):
    lengths = [70, 200]
    q, k, v, cu = make_inputs(lengths, 2, 128, seed=4)
    graph = tg.Graph.cat([tg.Graph.triangular(n, device="cuda") for n in lengths])
    out = Attention()(graph=graph, src={"key": k.cuda(), "value": v.cuda()}, dst={"query": q.cuda()}, scale=0.1)
    ref, _ = oracle.varlen_attn_fwd(cu.numpy(), q.float().numpy(), k.float().numpy(), v.float().numpy(), 0.1)
    np.testing.assert_allclose(out.float().cpu().numpy(), ref, rtol=2e-2, atol=2e-2)
    ops.check_async_errors()


@pytest.mark.parametrize("lengths,H,D", (
    ([5, 1, 9, 16], 2, 128),
    ([300, 129, 127, 513], 2, 128),
    ([700, 40], 3, 64),
))
@pytest.mark.parametrize("causal", (True, False))
def test_backward_matches_oracle(oracle, lengths, H, D, causal):
    q, k, v, cu = make_inputs(lengths, H, D, seed=7 + D)
    gen = torch.Generator().manual_seed(11)
    dy = torch.randn(q.shape, generator=gen).to(torch.bfloat16)
    scale = D ** -0.5
    graph = tg.Graph.cu_seqlens(cu.cuda(), causal=causal)
    qg, kg, vg = (t.cuda().requires_grad_() for t in (q, k, v))
    out = Attention()(graph=graph, src={"key": kg, "value": vg}, dst={"query": qg}, scale=scale)
    dq, dk, dv = torch.autograd.grad(out, (qg, kg, vg), dy.cuda())
    ops.check_async_errors()
    qf, kf, vf = q.float().numpy(), k.float().numpy(), v.float().numpy()
    ref_out, _ = oracle.varlen_attn_fwd(cu.numpy(), qf, kf, vf, scale, causal=causal)
    rq, rk, rv = oracle.varlen_attn_bwd(cu.numpy(), qf, kf, vf, ref_out, dy.float().numpy(), scale, causal=causal)
    for got, ref in ((dq, rq), (dk, rk), (dv, rv)):
        np.testing.assert_allclose(got.float().cpu().numpy(), ref, rtol=2e-2, atol=2e-2 * np.abs(ref).max())
