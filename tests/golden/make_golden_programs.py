"""Generate tests/golden/program_cases.npz by running the UNMODIFIED reference on the CPU.

    make -C oracle
    python tests/golden/make_golden_programs.py [--reference /path/to/TIGA-lang]

Edge expressions outside the weighted-sum / attention patterns (the reference's generic CSR path):
the reference's eager evaluator ``kernel.reference(...)`` plus ``torch.autograd.grad`` give outputs and
cotangents for every operand role (src, dst, edge, tensor parameter), sum, mean and product reducers
(rows with no, one and several zero messages), scalar and vector features, rows without edges and a
hub row.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", default=os.environ.get("TIGA_REFERENCE"))
    args = parser.parse_args()
    if not args.reference:
        sibling = os.path.join(os.path.dirname(ROOT), "reference")
        if not os.path.isdir(sibling):
            raise SystemExit("pass --reference /path/to/TIGA-lang (or set TIGA_REFERENCE)")
        args.reference = sibling
    runtime = os.path.join(ROOT, "oracle", "_ref", "libtiga_runtime.so")
    if not os.path.exists(runtime):
        raise SystemExit("build oracle/_ref first: make -C oracle")
    os.environ["TIGA_RUNTIME_LIBRARY"] = runtime
    sys.dont_write_bytecode = True
    sys.path.insert(0, os.path.join(args.reference, "python"))
    import tiga as tg

    assert os.path.realpath(tg.__file__).startswith(os.path.realpath(args.reference))
    torch.manual_seed(0)
    torch.set_num_threads(1)

    class DiffusionFlux(tg.MessagePassing):
        reducer = tg.sum()

        def edge(self, src, dst, edge):
            return edge.weight * (src.u - dst.u)

    class MeanFlux(DiffusionFlux):
        reducer = tg.mean()

    class Gated(tg.MessagePassing):
        reducer = tg.sum()

        def edge(self, src, dst, edge, gain, slope):
            s = (src.x * gain + dst.y) / (edge.w + 2.0)
            return tg.math.maximum(s, slope * s) - (-edge.w).exp() * src.x

    gen = torch.Generator().manual_seed(99)
    degree = torch.tensor([3, 0, 1, 70, 2, 0, 5, 9, 1, 4])          # empty rows, a row longer than one tile
    row_ptr = torch.cat((torch.zeros(1, dtype=torch.int64), degree.cumsum(0)))
    n_dst, n_src, edges = degree.numel(), 14, int(row_ptr[-1])
    col = torch.randint(0, n_src, (edges,), generator=gen)
    graph = tg.Graph.from_csr(row_ptr, col, num_src=n_src)
    saved = {"row_ptr": row_ptr.numpy(), "col": col.numpy(), "num_src": np.int64(n_src)}

    def record(tag, kernel, fields, params, wrt):
        tensors = {name: value for group in (*fields.values(), params) for name, value in group.items()}
        out = kernel.reference(graph=graph, src=fields["src"], dst=fields["dst"], edge=fields["edge"], **params)
        dy = torch.randn(out.shape, generator=gen)
        grads = torch.autograd.grad(out, [tensors[name] for name in wrt], dy)
        saved[tag + "_out"] = out.detach().numpy()
        saved[tag + "_dy"] = dy.numpy()
        for name, value in tensors.items():
            if isinstance(value, torch.Tensor):
                saved[f"{tag}_in_{name}"] = value.detach().numpy()
        for name, grad in zip(wrt, grads):
            saved[f"{tag}_d_{name}"] = grad.numpy()

    # scalar fields (the reference's own generic kernels take exactly these)
    u = torch.randn(n_src, generator=gen).requires_grad_()
    weight = torch.rand(edges, generator=gen).requires_grad_()
    # a square relation is needed for src.u - dst.u with one field: bind separate tensors per role
    u_dst = torch.randn(n_dst, generator=gen).requires_grad_()
    for tag, kernel in (("flux_sum", DiffusionFlux()), ("flux_mean", MeanFlux())):
        out = kernel.reference(graph=graph, src={"u": u}, dst={"u": u_dst}, edge={"weight": weight})
        dy = torch.randn(out.shape, generator=gen)
        du, dud, dw = torch.autograd.grad(out, (u, u_dst, weight), dy)
        saved[tag + "_out"], saved[tag + "_dy"] = out.detach().numpy(), dy.numpy()
        saved[tag + "_in_src_u"], saved[tag + "_in_dst_u"] = u.detach().numpy(), u_dst.detach().numpy()
        saved[tag + "_in_weight"] = weight.detach().numpy()
        saved[tag + "_d_src_u"], saved[tag + "_d_dst_u"], saved[tag + "_d_weight"] = du.numpy(), dud.numpy(), dw.numpy()
    # vector features, per-edge scalar with a trailing 1, full-width and scalar tensor parameters
    x = torch.randn(n_src, 6, generator=gen).requires_grad_()
    y = torch.randn(n_dst, 6, generator=gen).requires_grad_()
    w = torch.rand(edges, 1, generator=gen).requires_grad_()
    gain = torch.randn(6, generator=gen).requires_grad_()
    record("gated", Gated(), {"src": {"x": x}, "dst": {"y": y}, "edge": {"w": w}},
           {"gain": gain, "slope": 0.1}, ("x", "y", "w", "gain"))

    # the product monoid (tg.prod): plain source field with rows holding no, one and several zeros,
    # a per-edge field, and an expression; cotangents are Torch's zero-safe index_reduce("prod") rule
    class SourceProduct(tg.MessagePassing):
        reducer = tg.prod()

        def edge(self, src, dst, edge):
            return self.reducer(src.x)

    class EdgeProduct(tg.MessagePassing):
        reducer = tg.prod()

        def edge(self, src, dst, edge):
            return self.reducer(edge.x)

    class ShiftedProduct(tg.MessagePassing):
        reducer = tg.prod()

        def edge(self, src, dst, edge, bias):
            return 1.0 + edge.w * (src.x - dst.y) * bias

    px = (1.0 + 0.2 * torch.randn(n_src, 3, generator=gen))
    px[2, 0] = 0.0
    px[5, :] = 0.0
    px[9, 1] = 0.0
    px = px.requires_grad_()
    record("prod_src", SourceProduct(), {"src": {"x": px}, "dst": {}, "edge": {}}, {}, ("x",))
    pe = (1.0 + 0.2 * torch.randn(edges, generator=gen))
    pe[[0, 1, 4, 80, 90]] = 0.0                      # row 0: two zeros; row 3 (the hub): one zero; row 6: one
    pe = pe.requires_grad_()
    record("prod_edge", EdgeProduct(), {"src": {}, "dst": {}, "edge": {"x": pe}}, {}, ("x",))
    sx = (0.3 * torch.randn(n_src, 4, generator=gen)).requires_grad_()
    sy = (0.3 * torch.randn(n_dst, 4, generator=gen)).requires_grad_()
    sw = torch.rand(edges, 1, generator=gen).requires_grad_()
    bias = torch.randn(4, generator=gen).requires_grad_()
    record("prod_shifted", ShiftedProduct(), {"src": {"x": sx}, "dst": {"y": sy}, "edge": {"w": sw}},
           {"bias": bias}, ("x", "y", "w", "bias"))

    out_path = os.path.join(HERE, "program_cases.npz")
    np.savez_compressed(out_path, **saved)
    print(f"wrote {out_path}: {len(saved)} arrays, {os.path.getsize(out_path) / 1024:.1f} KiB")


if __name__ == "__main__":
    main()
