"""GraphProgram (captured applications, horizontal fusion, cross-apply dataflow) and the
control loops (repeat with CUDA-graph replay, while_loop) on the GPU."""
from dataclasses import replace

import pytest
import torch

import tiga as tg
from baseline import synthetic as syn
from tiga import _native

pytestmark = pytest.mark.gpu


class Weighted(tg.MessagePassing):
    reducer = tg.sum()

    def edge(self, src, dst, edge):
        return src.x * edge.weight


def _case(features=(16, 8)):
    row_ptr, col = syn.rmat_csr(10, 8, seed=3)
    n, E = row_ptr.numel() - 1, col.numel()
    graph = tg.Graph.from_csr(row_ptr.cuda(), col.cuda(), num_src=n)
    gen = torch.Generator().manual_seed(1)
    xs = [torch.randn(n, f, generator=gen).cuda() for f in features]
    w0, w1 = torch.rand(E, generator=gen).cuda(), torch.rand(E, generator=gen).cuda()
    graph.native_plan(transpose=False)      # the plan's own set-up launches are not what the tests count
    return graph, xs, w0, w1


def test_horizontal_fusion_runs_one_gather_for_applications_that_share_graph_and_weights():
    graph, (xa, xb), w0, w1 = _case()

    @tg.program
    def captured():
        return (Weighted()(graph=graph, src={"x": xa}, dst={}, edge={"weight": w0}),
                Weighted()(graph=graph, src={"x": xb}, dst={}, edge={"weight": w0}),
                Weighted()(graph=graph, src={"x": xa}, dst={}, edge={"weight": w1}))

    first, second, third = captured()
    assert first.program is second.program is third.program
    assert first.shape == (graph.num_dst, 16) and second.shape == (graph.num_dst, 8)
    before = _native.launch_count()
    results = first.program.run()
    launched = _native.launch_count() - before
    assert first.program.launches == ((0, 1), (2,))            # two applications fused, the third alone
    assert "fused gather" in first.program.explain()
    plain = [Weighted()(graph=graph, src={"x": x}, dst={}, edge={"weight": w}) for x, w in
             ((xa, w0), (xb, w0), (xa, w1))]
    for got, want in zip(results, plain):
        torch.testing.assert_close(got, want, rtol=1e-6, atol=1e-6)
    before = _native.launch_count()
    for x, w in ((xa, w0), (xb, w0), (xa, w1)):
        Weighted()(graph=graph, src={"x": x}, dst={}, edge={"weight": w})
    assert launched < _native.launch_count() - before              # fewer kernel launches than unfused


def test_cross_apply_dataflow_arithmetic_and_stale_values():
    graph, (xa, _), w0, w1 = _case()
    prog = tg.GraphProgram()
    first = prog.apply(Weighted(), graph=graph, src={"x": xa}, dst={}, edge={"weight": w0})
    second = prog.apply(Weighted(), graph=graph, src={"x": first}, dst={}, edge={"weight": w1})
    prog.outputs(second)
    out = prog.run()
    step1 = Weighted()(graph=graph, src={"x": xa}, dst={}, edge={"weight": w0})
    step2 = Weighted()(graph=graph, src={"x": step1}, dst={}, edge={"weight": w1})
    assert torch.equal(out, step2) and prog.launches == ((0,), (1,))
    assert torch.equal(first + 1.0, step1 + 1.0) and torch.equal(2.0 * second, 2.0 * step2)
    stale = replace(first, version=first.version + 1)
    with pytest.raises(ValueError, match="stale ProgramValue"):
        prog.apply(Weighted(), graph=graph, src={"x": stale}, dst={}, edge={"weight": w1})
    # gradients flow through a program like through the plain calls
    xg = xa.clone().requires_grad_()
    prog = tg.GraphProgram()
    value = prog.apply(Weighted(), graph=graph, src={"x": xg}, dst={}, edge={"weight": w0})
    (grad,) = torch.autograd.grad(value.materialize().sum(), (xg,))
    xr = xa.clone().requires_grad_()
    (want,) = torch.autograd.grad(Weighted()(graph=graph, src={"x": xr}, dst={}, edge={"weight": w0}).sum(), (xr,))
    assert torch.equal(grad, want)


def test_repeat_replays_a_cuda_graph_and_matches_the_host_loop():
    graph, (xa, _), w0, _ = _case()
    degree = graph.resolve_csr()[0].diff().clamp(min=1).float()[:, None]
    layer = Weighted()

    def diffuse(state):
        mixed = layer(graph=graph, src={"x": state}, dst={}, edge={"weight": w0}) / degree
        return state + 0.25 * (mixed - state)

    want = xa
    for _ in range(20):
        want = diffuse(want)
    got = tg.repeat(xa, diffuse, iterations=20, cuda_graph=True)
    torch.testing.assert_close(got, want, rtol=1e-6, atol=1e-6)
    assert torch.equal(tg.repeat(xa, diffuse, iterations=20, cuda_graph=False), want)
    assert torch.equal(tg.repeat(xa, diffuse, iterations=0), xa)

    class Diffusion(tg.control.Repeat):
        def body(self, state):
            return diffuse(state)

    torch.testing.assert_close(Diffusion()(xa, iterations=20), want, rtol=1e-6, atol=1e-6)
    # two carried states, and the argument checks of the reference's repeat
    a, b = tg.repeat((xa, xa * 2), lambda p, q: (q, p), iterations=5)
    assert torch.equal(a, xa * 2) and torch.equal(b, xa)
    with pytest.raises(ValueError, match="preserve its state shape"):
        tg.repeat(xa, lambda s: s[:, :4], iterations=2)
    with pytest.raises(TypeError):
        tg.repeat(xa, diffuse, iterations=2.5)
    with pytest.raises(ValueError):
        tg.repeat(xa, diffuse, iterations=-1)
    # a state that needs a gradient runs the unrolled loop and differentiates
    xg = xa.clone().requires_grad_()
    out = tg.repeat(xg, diffuse, iterations=4)
    (grad,) = torch.autograd.grad(out.sum(), (xg,))
    assert grad.shape == xa.shape and torch.isfinite(grad).all()


def test_while_loop_stops_on_its_condition():
    graph, (xa, _), w0, _ = _case()
    layer = Weighted()

    def grow(state):
        return state + layer(graph=graph, src={"x": state}, dst={}, edge={"weight": w0}).abs()

    limit = float(xa.abs().max()) * 50
    out = tg.control.while_loop(xa, lambda s: s.abs().max() < limit, grow, max_iterations=100)
    assert float(out.abs().max()) >= limit
    assert torch.equal(tg.control.while_loop(xa, lambda s: s.abs().max() < limit, grow, max_iterations=0), xa)


def test_repeat_replays_a_runtime_compiled_edge_program():
    """A loop body whose edge expression has no dedicated kernel: the generated kernels are launched
    through the driver's module interface, which a CUDA-graph capture records like any other launch."""
    class Flux(tg.MessagePassing):
        reducer = tg.sum()

        def edge(self, src, dst, edge, rate):
            return edge.weight * (src.u - dst.u) * rate

    row_ptr, col = syn.rmat_csr(9, 6, seed=3, symmetrize=True)
    n = row_ptr.numel() - 1
    graph = tg.Graph.from_csr(row_ptr.cuda(), col.cuda(), num_src=n)
    gen = torch.Generator().manual_seed(2)
    u0 = torch.randn(n, 4, generator=gen).cuda()
    weight = (0.01 * torch.rand(col.numel(), 1, generator=gen)).cuda()
    kernel = Flux()

    def diffuse(state):
        return state + kernel(graph=graph, src={"u": state}, dst={"u": state}, edge={"weight": weight}, rate=0.5)

    want = u0
    for _ in range(12):
        want = diffuse(want)
    got = tg.repeat(u0, diffuse, iterations=12, cuda_graph=True)
    assert kernel.last_variant.lowering == "b200-generic-csr-scalar-reducer"
    assert torch.equal(got, want)
