"""User algebras on the GPU: reducers none of the dedicated kernels folds (tuple states, several
messages, non-commutative combine) through the interpreting kernels, forward and reverse mode.

Pinned by the values the reference's own tests assert (tests/python/test_message_passing_autograd.py:
353-390 and 516-532 of walkerchi/TIGA-lang) and, on larger graphs, by the definition evaluated row by
row with Torch operations and differentiated by Torch autograd (``kernel.reference``).
Tolerance: float32, rel 1e-4 of the largest magnitude (cotangent sums run in another order)."""
import pytest
import torch

import tiga as tg
from baseline import synthetic as syn

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=("generated", "interpreted"))
def kernels(request, monkeypatch):
    """Every test runs twice: on the kernels compiled at run time for the program, and on the
    interpreting kernels that take over when the runtime compiler is missing."""
    monkeypatch.setenv("TGB_EDGE_JIT", "1" if request.param == "generated" else "0")
    return request.param


class StableWeightedMean(tg.Reducer):
    name = "deliberately_not_online_softmax"
    associative = True
    commutative = True

    def identity(self):
        return -1.0e30, 0.0, 0.0

    def lift(self, score, value):
        return score, 1.0, value

    def combine(self, left, right):
        maximum = left[0].maximum(right[0])
        left_scale = (left[0] - maximum).exp()
        right_scale = (right[0] - maximum).exp()
        return (maximum, left_scale * left[1] + right_scale * right[1],
                left_scale * left[2] + right_scale * right[2])

    def finalize(self, state):
        return state[2] / state[1]


class AffineComposition(tg.Reducer):
    """Associative, not commutative: the later edge's map after the earlier one's."""

    associative = True
    commutative = False

    def identity(self):
        return 1.0, 0.0

    def lift(self, scale, bias):
        return scale, bias

    def combine(self, left, right):
        return right[0] * left[0], right[0] * left[1] + right[1]

    def finalize(self, state):
        return state[1]


class StableAttention(tg.MessagePassing):
    reducer = StableWeightedMean()

    def edge(self, src, dst, edge):
        return self.reducer(src.score, src.value)


class BuiltinAttention(tg.MessagePassing):
    reducer = tg.online_softmax()

    def edge(self, src, dst, edge):
        return self.reducer(edge.score, src.value)


class Composition(tg.MessagePassing):
    reducer = AffineComposition(deterministic=True)

    def edge(self, src, dst, edge):
        return self.reducer(src.scale, src.bias)


class WeightedComposition(tg.MessagePassing):
    reducer = AffineComposition(deterministic=True)

    def edge(self, src, dst, edge, gain):
        return self.reducer(1.0 + edge.w * (src.scale - 1.0), gain * src.bias - dst.y)


def small_graph(device="cuda"):
    return tg.Graph.from_csr(torch.tensor([0, 2, 2, 5], device=device), torch.tensor([0, 1, 0, 1, 2], device=device),
                             num_src=3)


def test_noncommutative_composition_known_answers():
    scale = torch.tensor([2.0, 3.0, 5.0], device="cuda", requires_grad=True)
    bias = torch.tensor([1.0, 4.0, 2.0], device="cuda", requires_grad=True)
    kernel = Composition()
    out = kernel(graph=small_graph(), src={"scale": scale, "bias": bias}, dst={})
    assert kernel.last_variant.lowering == "b200-csr-algebra-tile"
    assert out.tolist() == [7.0, 0.0, 37.0]
    dscale, dbias = torch.autograd.grad(out.sum(), (scale, bias))
    assert dscale.tolist() == [0.0, 6.0, 7.0]
    assert dbias.tolist() == [18.0, 6.0, 1.0]


def test_user_stable_weighted_mean_known_answers_and_builtin_softmax():
    score = torch.tensor([1000.0, 999.0, 998.0], device="cuda", requires_grad=True)
    value = torch.tensor([1.0, -2.0, 3.0], device="cuda", requires_grad=True)
    graph = small_graph()
    out = StableAttention()(graph=graph, src={"score": score, "value": value}, dst={})
    got = out.tolist()
    assert abs(got[0] - 0.1931757) < 1e-5 and got[1] != got[1] and abs(got[2] - 0.4458758) < 1e-5
    # rows with edges: the same numbers and cotangents as the built-in online softmax fed the same scores
    _, col = graph.resolve_csr()
    edge_score = score.detach()[col].clone().requires_grad_()
    value_b = value.detach().clone().requires_grad_()
    builtin = BuiltinAttention()(graph=graph, src={"value": value_b}, dst={}, edge={"score": edge_score})
    rows = torch.tensor([0, 2], device="cuda")
    torch.testing.assert_close(out[rows], builtin.reshape(-1)[rows], rtol=1e-5, atol=1e-6)
    dy = torch.tensor([0.7, 0.0, -1.3], device="cuda")
    dscore, dvalue = torch.autograd.grad(out, (score, value), dy)
    dscore_e, dvalue_b = torch.autograd.grad(builtin.reshape(-1), (edge_score, value_b), dy)
    torch.testing.assert_close(dvalue, dvalue_b, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(dscore, torch.zeros(3, device="cuda").index_add_(0, col, dscore_e), rtol=1e-4, atol=1e-6)


def test_builtin_online_softmax_with_source_scores_known_answers():
    """``self.reducer(src.score, src.value)``: a score per source and a payload vector, the values the
    reference's test asserts (tests/python/test_message_passing_autograd.py:318-351)."""
    class SourceScoreAttention(tg.MessagePassing):
        reducer = tg.online_softmax()

        def edge(self, src, dst, edge):
            return self.reducer(src.score, src.value)

    graph = tg.Graph.from_csr(torch.tensor([0, 2, 3, 5]).cuda(), torch.tensor([0, 2, 1, 0, 1]).cuda(), num_src=3)
    score = torch.tensor([1000.0, 999.0, 998.0], device="cuda", requires_grad=True)
    value = torch.tensor([[1.0, 0.0], [0.0, 2.0], [3.0, 1.0]], device="cuda", requires_grad=True)
    kernel = SourceScoreAttention()
    out = kernel(graph=graph, src={"score": score, "value": value}, dst={})
    assert kernel.last_variant.lowering == "b200-csr-algebra-tile"
    want = torch.tensor([[1.2384058, 0.1192029], [0.0, 2.0], [0.7310586, 0.5378829]])
    torch.testing.assert_close(out.detach().cpu(), want, rtol=1e-5, atol=1e-5)
    dscore, dvalue = torch.autograd.grad(out.sum(), (score, value))
    torch.testing.assert_close(dscore.cpu(), torch.tensor([-0.5115927, 0.1966119, 0.3149807]), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(dvalue.cpu(), torch.tensor([[1.6118556] * 2, [1.2689414] * 2, [0.1192029] * 2]),
                               rtol=1e-5, atol=1e-5)
    # a row without edges is exactly zero
    graph = small_graph()
    out = SourceScoreAttention()(graph=graph, src={"score": score, "value": value}, dst={})
    assert out[1].tolist() == [0.0, 0.0]
    want = SourceScoreAttention().reference(graph=tg.Graph.from_csr(torch.tensor([0, 2, 2, 5]), torch.tensor([0, 1, 0, 1, 2]),
                                                                     num_src=3),
                                            src={"score": score.detach().cpu(), "value": value.detach().cpu()}, dst={})
    torch.testing.assert_close(out.detach().cpu(), want, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("features", ((), (5,)))
def test_against_the_definition_on_a_random_graph(features):
    row_ptr, col = syn.rmat_csr(7, 5, seed=3, symmetrize=False)
    n, edges = row_ptr.numel() - 1, col.numel()
    gen = torch.Generator().manual_seed(7 + len(features))
    scale = 1.0 + 0.2 * torch.randn((n,) + features, generator=gen)
    bias = torch.randn((n,) + features, generator=gen)
    y = torch.randn((n,) + features, generator=gen)
    w = torch.rand((edges,) + (1,) * len(features), generator=gen)
    gain = torch.randn(features, generator=gen)
    dy = torch.randn((n,) + features, generator=gen)

    def leaves(device):
        return [t.clone().to(device).requires_grad_() for t in (scale, bias, y, w, gain)]

    cs, cb, cy, cw, cg = leaves("cpu")
    want = WeightedComposition().reference(graph=tg.Graph.from_csr(row_ptr, col, num_src=n),
                                           src={"scale": cs, "bias": cb}, dst={"y": cy}, edge={"w": cw}, gain=cg)
    want_grads = torch.autograd.grad(want, (cs, cb, cy, cw, cg), dy)
    gs, gb, gy, gw, gg = leaves("cuda")
    got = WeightedComposition()(graph=tg.Graph.from_csr(row_ptr.cuda(), col.cuda(), num_src=n),
                                src={"scale": gs, "bias": gb}, dst={"y": gy}, edge={"w": gw}, gain=gg)
    torch.testing.assert_close(got.detach().cpu(), want.detach(), rtol=1e-4, atol=1e-4 * float(want.detach().abs().max()))
    for a, b in zip(torch.autograd.grad(got, (gs, gb, gy, gw, gg), dy.cuda()), want_grads):
        torch.testing.assert_close(a.cpu(), b, rtol=1e-3, atol=2e-4 * float(b.abs().max()))


def test_long_rows_join_their_slices_in_order():
    """A destination with 1 500 in-edges (above the split threshold): one CTA folds it in slices that
    `combine` joins in order -- for a non-commutative algebra any other order gives other numbers."""
    n = 400
    gen = torch.Generator().manual_seed(2)
    hub = torch.randint(0, n, (1500,), generator=gen)
    fan = torch.randint(0, n, (n - 1, 2), generator=gen)
    degree = torch.full((n,), 2)
    degree[0] = 1500
    row_ptr = torch.cat((torch.zeros(1, dtype=torch.int64), degree.cumsum(0)))
    col = torch.cat((hub, fan.reshape(-1)))
    scale = 1.0 + 0.01 * torch.randn(n, 3, generator=gen)
    bias = torch.randn(n, 3, generator=gen)
    dy = torch.randn(n, 3, generator=gen)
    cs, cb = scale.clone().requires_grad_(), bias.clone().requires_grad_()
    want = Composition().reference(graph=tg.Graph.from_csr(row_ptr, col, num_src=n), src={"scale": cs, "bias": cb},
                                   dst={})
    want_grads = torch.autograd.grad(want, (cs, cb), dy)
    gs, gb = scale.cuda().requires_grad_(), bias.cuda().requires_grad_()
    graph = tg.Graph.from_csr(row_ptr.cuda(), col.cuda(), num_src=n)
    assert graph.native_plan(transpose=False).info["long_rows"] >= 1
    got = Composition()(graph=graph, src={"scale": gs, "bias": gb}, dst={})
    torch.testing.assert_close(got.detach().cpu(), want.detach(), rtol=1e-4, atol=1e-4 * float(want.detach().abs().max()))
    for a, b in zip(torch.autograd.grad(got, (gs, gb), dy.cuda()), want_grads):
        torch.testing.assert_close(a.cpu(), b, rtol=1e-3, atol=2e-4 * float(b.abs().max()))


def test_a_reducer_that_is_not_associative_is_refused():
    class Midpoint(tg.Reducer):
        def identity(self):
            return 0.0

        def combine(self, left, right):
            return (left + right) * 0.5

    class Kernel(tg.MessagePassing):
        reducer = Midpoint()

        def edge(self, src, dst, edge):
            return self.reducer(src.x)

    with pytest.raises(NotImplementedError, match="associative"):
        Kernel()(graph=small_graph(), src={"x": torch.ones(3, device="cuda")}, dst={})


@pytest.mark.parametrize("kernel_class", (WeightedComposition, StableAttention))
def test_generated_algebra_kernels_equal_the_interpreting_kernels(kernel_class, monkeypatch):
    """The fold and its reverse sweep as runtime-compiled straight-line CUDA against the interpreter:
    same graph (a 1 500-edge row, rows without edges), unsplit rows bit for bit, the rest to rounding."""
    n = 400
    gen = torch.Generator().manual_seed(17)
    hub = torch.randint(0, n, (1500,), generator=gen)
    fan = torch.randint(0, n, (n - 1, 2), generator=gen)
    degree = torch.full((n,), 2)
    degree[0] = 1500
    degree[9] = 0
    row_ptr = torch.cat((torch.zeros(1, dtype=torch.int64), degree.cumsum(0)))
    col = torch.cat((hub, fan[:8].reshape(-1), fan[9:].reshape(-1)))
    assert col.numel() == int(row_ptr[-1])
    edges = col.numel()
    graph = tg.Graph.from_csr(row_ptr.cuda(), col.cuda(), num_src=n)
    if kernel_class is WeightedComposition:
        fields = {"scale": 1.0 + 0.01 * torch.randn(n, 3, generator=gen), "bias": torch.randn(n, 3, generator=gen),
                  "y": torch.randn(n, 3, generator=gen), "w": torch.rand(edges, 1, generator=gen),
                  "gain": torch.randn(3, generator=gen)}
    else:
        fields = {"score": torch.randn(n, 1, generator=gen), "value": torch.randn(n, 3, generator=gen)}
    dy = torch.randn(n, 3, generator=gen).cuda()
    results = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("TGB_EDGE_JIT", mode)
        leaves = {name: t.clone().cuda().requires_grad_() for name, t in fields.items()}
        if kernel_class is WeightedComposition:
            out = kernel_class()(graph=graph, src={"scale": leaves["scale"], "bias": leaves["bias"]},
                                 dst={"y": leaves["y"]}, edge={"w": leaves["w"]}, gain=leaves["gain"])
        else:
            out = kernel_class()(graph=graph, src=leaves, dst={})
        cotangent = torch.where(torch.isfinite(out.detach()), dy, torch.zeros_like(dy))
        results[mode] = (out.detach(), torch.autograd.grad(out, list(leaves.values()), cotangent))
    # rows below the split threshold are folded edge by edge by both: bit for bit; the long row is cut
    # into more slices by the generated kernel (wider CTA), so its joins associate differently
    generated, interpreted = (torch.nan_to_num(results[mode][0], nan=7.0) for mode in ("1", "0"))
    assert torch.equal(generated[1:], interpreted[1:])
    torch.testing.assert_close(generated[0], interpreted[0], rtol=1e-4, atol=1e-5 * float(interpreted[0].abs().max()))
    for a, b in zip(results["1"][1], results["0"][1]):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5 * float(b.abs().max()), equal_nan=True)
