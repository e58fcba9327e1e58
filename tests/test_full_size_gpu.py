"""Parity at the benchmark configurations' full sizes through size-independent
properties (the CPU oracle would take minutes there): adjoint identities that
tie forward, dx and dw together, column-sum checksums computed independently in
float64, the CPU oracle on sampled rows, and softmax rows that must sum to one."""
import numpy as np
import pytest
import torch

import tiga as tg
from tiga import ops
from baseline import synthetic as syn

pytestmark = pytest.mark.gpu


class WeightedSum(tg.MessagePassing):
    reducer = tg.sum()

    def edge(self, src, dst, edge):
        return edge.weight * src.x


class GAT(tg.MessagePassing):
    reducer = tg.online_softmax()

    def edge(self, src, dst, edge, a_src, a_dst):
        s = (src.x * a_src).sum(dim=-1) + (dst.x * a_dst).sum(dim=-1)
        return self.reducer(tg.math.maximum(s, 0.2 * s), src.x)


class Attention(tg.MessagePassing):
    reducer = tg.online_softmax()

    def edge(self, src, dst, edge, scale):
        return self.reducer((src.key * dst.query).sum(dim=-1) * scale, src.value)


def test_gcn_layer_configuration_full_size(oracle):
    # config 2: R-MAT 2^20 nodes, 32 * 2^20 generated edges, symmetrised, de-duplicated; F = 128
    device = torch.device("cuda")
    row_ptr, col = syn.rmat_csr(20, 32, seed=20261125, symmetrize=True, device=device)
    n, E, F = row_ptr.numel() - 1, col.numel(), 128
    w = syn.gcn_norm_weights(row_ptr, col)
    x = syn.normal((n, F), seed=1, device=device)
    dy = syn.normal((n, F), seed=2, device=device)
    graph = tg.Graph.from_csr(row_ptr, col, num_src=n)
    xg, wg = x.clone().requires_grad_(), w.clone().requires_grad_()
    out = WeightedSum()(graph=graph, src={"x": xg}, dst={}, edge={"weight": wg})
    dx, dw = torch.autograd.grad(out, (xg, wg), dy)
    out = out.detach()
    # the graph is symmetric with symmetric weights: the transposed relation must equal the relation
    plan = graph.native_plan(transpose=True)
    assert torch.equal(plan.array(1), row_ptr) and torch.equal(plan.array(2).long(), col)
    # adjoint identities in float64: <A x, dy> = <x, A^T dy> = sum_e w_e dw_e
    lhs = (out.double() * dy.double()).sum().item()
    mid = (x.double() * dx.double()).sum().item()
    rhs = (w.double() * dw.double()).sum().item()
    scale = (out.double().abs() * dy.double().abs()).sum().item()
    assert abs(lhs - mid) < 1e-6 * scale and abs(lhs - rhs) < 1e-6 * scale
    # column-sum checksum: sum_i out[i, :] = (sum_{e: col = j} w_e)^T x, computed independently in float64
    col_weight = torch.zeros(n, dtype=torch.float64, device=device).index_add_(0, col, w.double())
    want = col_weight @ x.double()
    got = out.double().sum(0)
    magnitude = col_weight.abs() @ x.double().abs()
    assert torch.all((got - want).abs() <= 1e-6 * magnitude + 1e-6)
    # linearity in x
    x2 = syn.normal((n, F), seed=3, device=device)
    a, _ = ops.csr_reduce_forward(plan, "sum", x2, w, 0.0)
    b, _ = ops.csr_reduce_forward(plan, "sum", x + x2, w, 0.0)
    assert torch.allclose(b, out + a, rtol=1e-4, atol=1e-4)
    # the CPU oracle on sampled destination rows (hubs, empty rows and ordinary rows)
    deg = row_ptr.diff()
    picks = torch.cat((torch.topk(deg, 4).indices, torch.nonzero(deg == 0)[:4, 0],
                       torch.randint(0, n, (300,), device=device, generator=torch.Generator(device).manual_seed(5))))
    picks = torch.unique(picks).cpu()
    rp, ci, xs, ws = row_ptr.cpu(), col.cpu(), x.cpu(), w.cpu()
    sub_deg = deg.cpu()[picks]
    sub_ptr = torch.cat((torch.zeros(1, dtype=torch.int64), sub_deg.cumsum(0)))
    edges = torch.cat([torch.arange(rp[r], rp[r + 1]) for r in picks.tolist()])
    ref = oracle.wsum_fwd(sub_ptr.numpy(), ci[edges].numpy(), xs.numpy(), ws[edges].numpy())
    mag = oracle.wsum_fwd(sub_ptr.numpy(), ci[edges].numpy(), xs.abs().numpy(), ws[edges].numpy())
    err = np.abs(out.cpu()[picks].numpy() - ref)
    assert np.all(err <= 1e-5 * np.abs(ref) + 1e-6 + 8 * np.finfo(np.float32).eps * mag)
    ref_dw = oracle.wsum_bwd_dw(sub_ptr.numpy(), ci[edges].numpy(), dy.cpu()[picks].numpy(), xs.numpy())
    np.testing.assert_allclose(dw.cpu()[edges].numpy(), ref_dw, rtol=1e-4, atol=1e-4)


def test_gcn_layer_configuration_max_reducer_full_size(oracle):
    # config 2, maximum reducer: values and winning edges bit for bit, at 2^20 nodes and 128 floats per row
    device = torch.device("cuda")
    row_ptr, col = syn.rmat_csr(20, 32, seed=20261125, symmetrize=True, device=device)
    n, E, F = row_ptr.numel() - 1, col.numel(), 128
    w = syn.gcn_norm_weights(row_ptr, col)
    x = syn.normal((n, F), seed=1, device=device)
    graph = tg.Graph.from_csr(row_ptr, col, num_src=n)

    class WeightedMax(tg.MessagePassing):
        reducer = tg.max()

        def edge(self, src, dst, edge):
            return self.reducer(edge.weight * src.x)

    kernel = WeightedMax()
    xg, wg = x.clone().requires_grad_(), w.clone().requires_grad_()
    out = kernel(graph=graph, src={"x": xg}, dst={}, edge={"weight": wg})
    plan = graph.native_plan(transpose=True)
    values, winners = ops.csr_reduce_forward(plan, "max", x, w, float("-inf"))
    assert torch.equal(values, out.detach())
    deg = row_ptr.diff()
    assert torch.all(out.detach()[deg == 0] == float("-inf"))         # an empty row keeps the start value
    # (1) the product's second, independent statement of the semantics -- reference()'s scatter amax --
    # on blocks of destination rows (the eager evaluator materialises [edges, F]), bit for bit
    for first in (0, 1 << 18, (1 << 20) - (1 << 16)):
        last = first + (1 << 16)
        lo, hi = int(row_ptr[first]), int(row_ptr[last])
        block = tg.Graph.from_csr(row_ptr[first:last + 1] - lo, col[lo:hi], num_src=n)
        eager = kernel.reference(graph=block, src={"x": x}, dst={}, edge={"weight": w[lo:hi, None]})
        assert torch.equal(eager, out.detach()[first:last])
    # (2) the CPU oracle on sampled rows, hubs included: values and winners
    picks = torch.unique(torch.cat((torch.topk(deg, 3).indices, torch.nonzero(deg == 0)[:3, 0], torch.randint(
        0, n, (300,), device=device, generator=torch.Generator(device).manual_seed(9))))).cpu()
    rp, ci = row_ptr.cpu(), col.cpu()
    sub_ptr = torch.cat((torch.zeros(1, dtype=torch.int64), deg.cpu()[picks].cumsum(0)))
    edges = torch.cat([torch.arange(rp[r], rp[r + 1]) for r in picks.tolist()])
    ref_values, ref_winners = oracle.max_fwd(sub_ptr.numpy(), ci[edges].numpy(), x.cpu().numpy(),
                                             w.cpu()[edges].numpy())
    np.testing.assert_array_equal(values.cpu()[picks].numpy(), ref_values)
    # winners are positions in the full edge list; the oracle's are positions in the sampled list
    got_winners = winners.cpu()[picks].numpy()
    want = np.where(ref_winners >= 0, edges.numpy()[np.clip(ref_winners, 0, None)], -1)
    np.testing.assert_array_equal(got_winners, want)
    # (3) backward: every (row, element) cotangent reaches exactly one edge and one source element
    dy = syn.normal((n, F), seed=2, device=device)
    dx, dw = torch.autograd.grad(out, (xg, wg), dy)
    routed = torch.where(winners >= 0, dy, torch.zeros_like(dy))
    lhs = (routed.double() * out.detach().double().nan_to_num(neginf=0.0)).sum().item()
    mid = (dx.double() * x.double()).sum().item()
    rhs = (dw.double() * w.double()).sum().item()
    scale = (routed.double().abs() * out.detach().double().nan_to_num(neginf=0.0).abs()).sum().item()
    assert abs(lhs - mid) < 1e-6 * scale and abs(lhs - rhs) < 1e-6 * scale


def test_gat_configuration_full_size():
    # config 3: directed R-MAT 2^21 nodes, 64M generated edges, bf16 [N, 8, 32]
    device = torch.device("cuda")
    row_ptr, col = syn.rmat_csr(21, 32, seed=20261125, symmetrize=False, device=device)
    n, H, D = row_ptr.numel() - 1, 8, 32
    graph = tg.Graph.from_csr(row_ptr, col, num_src=n)
    a_src = syn.normal((H, D), seed=2, device=device, dtype=torch.bfloat16, std=0.1)
    a_dst = syn.normal((H, D), seed=3, device=device, dtype=torch.bfloat16, std=0.1)
    deg = row_ptr.diff()
    # softmax weights of a row sum to one: constant value rows must come back unchanged, empty rows are zero
    x = syn.normal((n, H, D), seed=1, device=device, dtype=torch.bfloat16)
    x[:, :, 1:] = x[:, :, :1]                      # logits still vary per node and head
    const = torch.full((n, H, D), 0.75, device=device, dtype=torch.bfloat16)
    # value == src.x, so use x whose rows are constant across d: out[i, h, :] is a convex mix of x[j, h, 0]
    out = GAT()(graph=graph, ndata={"x": x}, a_src=a_src, a_dst=a_dst).float()
    assert torch.all(out[deg == 0] == 0)
    nz = deg > 0
    assert torch.allclose(out[nz][:, :, 1:], out[nz][:, :, :1].expand(-1, -1, D - 1))   # same mix for every d
    lo = torch.full((n, H), float("inf"), device=device).scatter_reduce_(
        0, torch.repeat_interleave(torch.arange(n, device=device), deg)[:, None].expand(-1, H),
        x[col][:, :, 0].float(), reduce="amin")
    hi = torch.full((n, H), float("-inf"), device=device).scatter_reduce_(
        0, torch.repeat_interleave(torch.arange(n, device=device), deg)[:, None].expand(-1, H),
        x[col][:, :, 0].float(), reduce="amax")
    tol = 2e-2 * x.float().abs().max()
    assert torch.all(out[nz][:, :, 0] >= lo[nz] - tol) and torch.all(out[nz][:, :, 0] <= hi[nz] + tol)
    del const
    # sampled destination rows (two hubs + random rows) against the CPU oracle on the compacted sub-problem:
    # forward rows and the destination-side gradient depend on the row's own edges only
    x = syn.normal((n, H, D), seed=7, device=device, dtype=torch.bfloat16)
    dy = syn.normal((n, H, D), seed=8, device=device, dtype=torch.bfloat16)
    xs, xd = x.clone().requires_grad_(), x.clone().requires_grad_()
    out = GAT()(graph=graph, src={"x": xs}, dst={"x": xd}, a_src=a_src, a_dst=a_dst)
    dxs, dxd = torch.autograd.grad(out, (xs, xd), dy)
    picks = torch.unique(torch.cat((torch.topk(deg, 2).indices, torch.randint(
        0, n, (200,), device=device, generator=torch.Generator(device).manual_seed(5))))).cpu()
    rp, ci = row_ptr.cpu(), col.cpu()
    edges = torch.cat([torch.arange(rp[r], rp[r + 1]) for r in picks.tolist()])
    sources, local = torch.unique(ci[edges], return_inverse=True)
    sub_ptr = torch.cat((torch.zeros(1, dtype=torch.int64), deg.cpu()[picks].cumsum(0)))

    def bits(t):
        return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)

    from oracle import oracle
    ref_out, _, _, _ = oracle.gat_fwd(sub_ptr.numpy(), local.numpy(), bits(x.cpu()[sources]), bits(x.cpu()[picks]),
                                      bits(a_src), bits(a_dst))
    np.testing.assert_allclose(out.detach().float().cpu()[picks].numpy(), oracle.bf16_to_f32(ref_out),
                               rtol=2e-2, atol=2e-2)
    _, ref_dxd, _, _ = oracle.gat_bwd(sub_ptr.numpy(), local.numpy(), bits(x.cpu()[sources]), bits(x.cpu()[picks]),
                                      bits(a_src), bits(a_dst), bits(dy.cpu()[picks]))
    np.testing.assert_allclose(dxd.float().cpu()[picks].numpy(), ref_dxd, rtol=2e-2,
                               atol=2e-2 * np.abs(ref_dxd).max() + 1e-6)
    assert torch.isfinite(dxs.float()).all()


def test_varlen_attention_configuration_full_size():
    # config 4: 32 sequences, lengths ~ U[512, 8192], 16 heads, head width 128, bf16, causal
    device = torch.device("cuda")
    gen = torch.Generator().manual_seed(20260821)
    lengths = torch.randint(512, 8193, (32,), generator=gen)
    cu = torch.cat((torch.zeros(1, dtype=torch.int64), lengths.cumsum(0)))
    T, H, D = int(cu[-1]), 16, 128
    graph = tg.Graph.cu_seqlens(cu.to(device), causal=True)
    q = syn.normal((T, H, D), seed=1, device=device, dtype=torch.bfloat16)
    k = syn.normal((T, H, D), seed=2, device=device, dtype=torch.bfloat16)
    ones = torch.ones((T, H, D), device=device, dtype=torch.bfloat16)
    scale = D ** -0.5
    # rows of the softmax sum to one: V = 1 must give exactly-representable ones back
    out = Attention()(graph=graph, src={"key": k, "value": ones}, dst={"query": q}, scale=scale)
    assert torch.allclose(out.float(), torch.ones_like(out, dtype=torch.float32), atol=8e-3)
    # the first token of every sequence sees only itself: out = its own value
    v = syn.normal((T, H, D), seed=3, device=device, dtype=torch.bfloat16)
    qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
    out = Attention()(graph=graph, src={"key": kg, "value": vg}, dst={"query": qg}, scale=scale)
    starts = cu[:-1].to(device)
    assert torch.equal(out[starts], v[starts])
    # the longest sequence against float32 math on the GPU (torch ops as an independent check)
    s = int(torch.argmax(lengths))
    b, e = int(cu[s]), int(cu[s + 1])
    qs, ks, vs = (t[b:e, 3].float() for t in (q, k, v))
    logits = (qs @ ks.t()) * scale
    logits = logits.masked_fill(torch.triu(torch.ones_like(logits, dtype=torch.bool), 1), float("-inf"))
    ref = torch.softmax(logits, -1) @ vs
    assert torch.allclose(out[b:e, 3].float(), ref, rtol=2e-2, atol=2e-2)
    # backward: sum(out * dy) with V-gradient identity dV = P^T dy; check total mass: sum_j dV[j] = sum_i dy[i]
    dy = syn.normal((T, H, D), seed=4, device=device, dtype=torch.bfloat16)
    dq, dk, dv = torch.autograd.grad(out, (qg, kg, vg), dy)
    ops.check_async_errors()
    for sb, se in ((int(cu[i]), int(cu[i + 1])) for i in (0, s, 31)):
        got = dv[sb:se].float().sum(0)
        want = dy[sb:se].float().sum(0)
        assert torch.allclose(got, want, rtol=2e-2, atol=2e-2 * want.abs().max().item() + 0.5)
    # softmax cotangents sum to zero per query: dq = scale * dS K with rows of dS summing to ~0 => compare
    # against autograd of the float32 formula on the longest sequence, one head
    qs, ks, vs = (t[b:e, 3].float().requires_grad_() for t in (q, k, v))
    logits = (qs @ ks.t()) * scale
    logits = logits.masked_fill(torch.triu(torch.ones_like(logits, dtype=torch.bool), 1), float("-inf"))
    ref = torch.softmax(logits, -1) @ vs
    rq, rk, rv = torch.autograd.grad(ref, (qs, ks, vs), dy[b:e, 3].float())
    for got, want in ((dq, rq), (dk, rk), (dv, rv)):
        assert torch.allclose(got[b:e, 3].float(), want, rtol=3e-2, atol=3e-2 * want.abs().max().item())


def test_runtime_compiled_edge_program_against_the_dedicated_kernels_full_size():
    """Two independent native paths at config 2's size: the flux `edge.weight * (src.u - dst.u)` through
    the kernels generated for that expression, and the same sum written with the dedicated kernels,
    `wsum(weight, u) - dst.u * wsum(weight, 1)`; forward and all three cotangents.  The graph has
    10^5-edge rows (the generated long-row kernels) and rows without edges.
    Tolerance: float32 sums over up to 10^5 terms added in different orders: 2e-4 of the row's
    sum of magnitudes (measured spread is a few 1e-6)."""
    device = torch.device("cuda")
    row_ptr, col = syn.rmat_csr(20, 32, seed=20261125, symmetrize=True, device=device)
    n, F = row_ptr.numel() - 1, 16
    E = col.numel()
    u = syn.normal((n, F), seed=3, device=device)
    v = syn.normal((n, F), seed=4, device=device)
    w = torch.rand(E, 1, device=device, generator=torch.Generator(device=device).manual_seed(5))
    dy = syn.normal((n, F), seed=6, device=device)
    graph = tg.Graph.from_csr(row_ptr, col, num_src=n)

    class Flux(tg.MessagePassing):
        reducer = tg.sum()

        def edge(self, src, dst, edge):
            return edge.weight * (src.u - dst.u)

    ug, vg, wg = (t.clone().requires_grad_() for t in (u, v, w))
    kernel = Flux()
    out = kernel(graph=graph, src={"u": ug}, dst={"u": vg}, edge={"weight": wg})
    assert kernel.last_variant.lowering == "b200-generic-csr-scalar-reducer"
    grads = torch.autograd.grad(out, (ug, vg, wg), dy)

    ud, vd, wd = (t.clone().requires_grad_() for t in (u, v, w))
    gathered = WeightedSum()(graph=graph, src={"x": ud}, dst={}, edge={"weight": wd.reshape(-1)})
    row_weight = WeightedSum()(graph=graph, src={"x": torch.ones(n, 1, device=device)}, dst={},
                               edge={"weight": wd.reshape(-1)})
    want = gathered - vd * row_weight
    want_grads = torch.autograd.grad(want, (ud, vd, wd), dy)

    magnitude = WeightedSum()(graph=graph, src={"x": u.abs()}, dst={}, edge={"weight": w.reshape(-1)}) \
        + v.abs() * row_weight.detach()
    assert torch.all((out.detach() - want.detach()).abs() <= 2e-4 * magnitude + 1e-5)
    for got, ref in zip(grads, want_grads):
        scale = float(ref.abs().max())
        assert float((got - ref).abs().max()) <= 2e-4 * scale
