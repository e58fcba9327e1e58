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


@pytest.mark.parametrize("lengths,H,H_kv,D,causal", (
    ([128], 8, 2, 64, True),                 # the reference's grouped-query case: 8 query lanes on 2 source lanes
    ([300, 129, 513], 4, 1, 128, True),
    ([200, 77], 6, 3, 64, False),
))
def test_grouped_queries_match_oracle(oracle, lengths, H, H_kv, D, causal):
    """Fewer key/value heads than query heads: query head h reads head h // (H / H_kv), the map of
    the reference's dense kernel (tests/python/test_mlir_bridge.py:441-467 checks it against SDPA
    with enable_gqa).  The oracle has one head count, so K and V are repeated per group for it and
    its dK, dV are summed over each group."""
    gen = torch.Generator().manual_seed(H * 10 + D)
    T, group = sum(lengths), H // H_kv
    q = torch.randn(T, H, D, generator=gen).to(torch.bfloat16)
    k, v = (torch.randn(T, H_kv, D, generator=gen).to(torch.bfloat16) for _ in range(2))
    dy = torch.randn(T, H, D, generator=gen).to(torch.bfloat16)
    cu = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int64)
    scale = D ** -0.5
    graph = tg.Graph.cu_seqlens(cu.cuda(), causal=causal)
    qg, kg, vg = (t.cuda().requires_grad_() for t in (q, k, v))
    out = Attention()(graph=graph, src={"key": kg, "value": vg}, dst={"query": qg}, scale=scale)
    dq, dk, dv = torch.autograd.grad(out, (qg, kg, vg), dy.cuda())
    ops.check_async_errors()
    assert dk.shape == k.shape and dv.shape == v.shape
    qf = q.float().numpy()
    kf, vf = (t.float().repeat_interleave(group, dim=1).numpy() for t in (k, v))
    ref, _ = oracle.varlen_attn_fwd(cu.numpy(), qf, kf, vf, scale, causal=causal)
    np.testing.assert_allclose(out.detach().float().cpu().numpy(), ref, rtol=2e-2, atol=2e-2)
    rq, rk, rv = oracle.varlen_attn_bwd(cu.numpy(), qf, kf, vf, ref, dy.float().numpy(), scale, causal=causal)
    rk, rv = (r.reshape(T, H_kv, group, D).sum(2) for r in (rk, rv))
    for got, want in ((dq, rq), (dk, rk), (dv, rv)):
        np.testing.assert_allclose(got.float().cpu().numpy(), want, rtol=2e-2, atol=2e-2 * np.abs(want).max())
    # against Torch's grouped-query SDPA on the first sequence, as the reference's own test does
    if causal:
        n = lengths[0]
        expected = torch.nn.functional.scaled_dot_product_attention(
            qg[:n].detach().permute(1, 0, 2), kg[:n].detach().permute(1, 0, 2), vg[:n].detach().permute(1, 0, 2),
            is_causal=True, enable_gqa=True).permute(1, 0, 2)
        torch.testing.assert_close(out[:n].detach().float(), expected.float(), rtol=2e-2, atol=2e-2)
