"""Generate tests/golden/*.npz by running the UNMODIFIED reference.

Run in a container that has the reference checkout (read-only is fine):

    make -C oracle                      # builds oracle/_ref/libtiga_runtime.so
    python tests/golden/make_golden.py  [--reference /path/to/TIGA-lang]

The script puts the reference's ``python/`` on sys.path, points
``TIGA_RUNTIME_LIBRARY`` at the runtime compiled from the reference's own two
C++ sources, and evaluates small seeded cases through the reference's public
API: ``kernel.reference(...)`` (its eager semantic evaluator) plus
``torch.autograd.grad``, ``tg.Graph.from_coo/cu_seqlens``, and
``tiga.distributed.derive_halo_map``.  Inputs and outputs are saved together
so the fixtures can be replayed anywhere without the reference.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def _graphs(gen):
    """Small CSR graphs covering the reference tests' edge cases."""
    out = {}
    # fixed degree 16 (config-1 shape, scaled down)
    n = 96
    out["fixed16"] = (torch.arange(0, n * 16 + 1, 16), torch.randint(0, n, (n * 16,), generator=gen), n)
    # ragged with empty rows and a degree-65 row (tests/python/test_torch_default.py:124-144)
    deg = torch.tensor([2, 1, 0, 65, 0, 3, 7, 33, 1, 0])
    rp = torch.cat((torch.zeros(1, dtype=torch.int64), deg.cumsum(0)))
    out["ragged"] = (rp, torch.randint(0, 12, (int(rp[-1]),), generator=gen), 12)
    # a hub row (degree 700) among short rows: exercises the split-row path
    deg = torch.tensor([1, 700, 2, 0, 5, 300, 1, 1])
    rp = torch.cat((torch.zeros(1, dtype=torch.int64), deg.cumsum(0)))
    out["hub"] = (rp, torch.randint(0, 40, (int(rp[-1]),), generator=gen), 40)
    # empty graph (tests/python/test_reference.py:708-723)
    out["empty"] = (torch.zeros(4, dtype=torch.int64), torch.zeros(0, dtype=torch.int64), 3)
    return out


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", default=os.environ.get("TIGA_REFERENCE"),
                        help="root of the unmodified reference checkout (or set TIGA_REFERENCE)")
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
    from tiga.distributed import derive_halo_map
    from tiga.distributed.model import destination_owner, owned_range

    assert os.path.realpath(tg.__file__).startswith(os.path.realpath(args.reference))
    torch.manual_seed(0)
    torch.set_num_threads(1)

    class WeightedSum(tg.MessagePassing):
        reducer = tg.sum()

        def edge(self, src, dst, edge):
            return edge.weight * src.x

    class PlainSum(tg.MessagePassing):
        reducer = tg.sum(identity=0.5)

        def edge(self, src, dst, edge):
            return src.x

    class WeightedMean(tg.MessagePassing):
        reducer = tg.mean()

        def edge(self, src, dst, edge):
            return edge.weight * src.x

    class PlainMean(tg.MessagePassing):
        reducer = tg.mean()

        def edge(self, src, dst, edge):
            return src.x

    class Softmax(tg.MessagePassing):
        reducer = tg.online_softmax()

        def edge(self, src, dst, edge):
            return self.reducer(edge.score, src.value)

    class GAT(tg.MessagePassing):
        reducer = tg.online_softmax()

        def edge(self, src, dst, edge, a_src, a_dst):
            s = (src.x * a_src).sum(dim=-1) + (dst.x * a_dst).sum(dim=-1)
            return self.reducer(tg.math.maximum(s, 0.2 * s), src.x)

    class Attention(tg.MessagePassing):
        reducer = tg.online_softmax()

        def edge(self, src, dst, edge, scale):
            score = (src.key * dst.query).sum(dim=-1) * scale
            return self.reducer(score, src.value)

    gen = torch.Generator().manual_seed(1234)
    saved = {}

    # ---------------------------------------------------------- sum / mean
    for name, (row_ptr, col, num_src) in _graphs(gen).items():
        g = tg.Graph.from_csr(row_ptr, col, num_src=num_src)
        n = row_ptr.numel() - 1
        for F in (1, 3, 64):
            shape = (num_src,) if F == 1 else (num_src, F)
            x = torch.randn(shape, generator=gen).requires_grad_()
            w = torch.rand(col.numel(), generator=gen)
            w = (w if F == 1 else w[:, None]).requires_grad_()
            dy = torch.randn((n,) + shape[1:], generator=gen)
            for tag, kernel, weighted in (("wsum", WeightedSum(), True), ("psum", PlainSum(), False),
                                          ("wmean", WeightedMean(), True), ("pmean", PlainMean(), False)):
                edge = {"weight": w} if weighted else {}
                out = kernel.reference(graph=g, src={"x": x}, dst={}, edge=edge)
                key = f"{tag}_{name}_f{F}"
                saved[key + "_row_ptr"] = row_ptr.numpy()
                saved[key + "_col"] = col.numpy()
                saved[key + "_x"] = x.detach().numpy()
                saved[key + "_dy"] = dy.numpy()
                saved[key + "_out"] = out.detach().numpy()
                if weighted:
                    saved[key + "_w"] = w.detach().numpy()
                if col.numel():
                    loss = torch.nan_to_num(out * dy, nan=0.0).sum() if "mean" in tag else (out * dy).sum()
                    grads = torch.autograd.grad(loss, (x, w) if weighted else (x,))
                    saved[key + "_dx"] = grads[0].numpy()
                    if weighted:
                        saved[key + "_dw"] = grads[1].numpy()

    # ------------------------------------------------------ online softmax
    # tests/python/test_reference.py:416-444 style: +-1000 scores, 2 heads x 3 payload, empty row
    row_ptr = torch.tensor([0, 3, 3, 4, 9])
    col = torch.tensor([0, 1, 2, 1, 0, 1, 2, 3, 3])
    g = tg.Graph.from_csr(row_ptr, col, num_src=4)
    score = torch.randn(9, 2, generator=gen)
    score[0, 0], score[1, 0], score[4, 1], score[5, 1] = 1000.0, -1000.0, 1000.0, 999.0
    score.requires_grad_()
    value = torch.randn(4, 2, 3, generator=gen).requires_grad_()
    out = Softmax().reference(graph=g, src={"value": value}, dst={}, edge={"score": score})
    dy = torch.randn(out.shape, generator=gen)
    ds, dv = torch.autograd.grad((out * dy).sum(), (score, value))
    saved.update(softmax_row_ptr=row_ptr.numpy(), softmax_col=col.numpy(), softmax_score=score.detach().numpy(),
                 softmax_value=value.detach().numpy(), softmax_out=out.detach().numpy(), softmax_dy=dy.numpy(),
                 softmax_dscore=ds.numpy(), softmax_dvalue=dv.numpy())

    # ------------------------------------------------------------- GAT bf16
    for name, (row_ptr, col, num_src) in _graphs(gen).items():
        if name == "empty":
            continue
        n = row_ptr.numel() - 1
        nn = max(n, num_src)  # homogeneous relation: one node set plays both roles
        g = tg.Graph.from_csr(row_ptr if n == nn else torch.cat((row_ptr, row_ptr[-1:].expand(nn - n))), col, num_src=nn)
        x = torch.randn(nn, 8, 32, generator=gen).to(torch.bfloat16).requires_grad_()
        a_src = (0.1 * torch.randn(8, 32, generator=gen)).to(torch.bfloat16).requires_grad_()
        a_dst = (0.1 * torch.randn(8, 32, generator=gen)).to(torch.bfloat16).requires_grad_()
        out = GAT().reference(graph=g, src={"x": x}, dst={"x": x}, a_src=a_src, a_dst=a_dst)
        dy = torch.randn(out.shape, generator=gen).to(torch.bfloat16)
        dx, das, dad = torch.autograd.grad((out.float() * dy.float()).sum(), (x, a_src, a_dst))
        key = f"gat_{name}"
        saved[key + "_row_ptr"] = (row_ptr if n == nn else torch.cat((row_ptr, row_ptr[-1:].expand(nn - n)))).numpy()
        saved[key + "_col"] = col.numpy()
        for nm, t in (("x", x), ("a_src", a_src), ("a_dst", a_dst), ("out", out), ("dy", dy), ("dx", dx),
                      ("da_src", das), ("da_dst", dad)):
            saved[f"{key}_{nm}"] = t.detach().view(torch.int16).numpy().view(np.uint16)

    # ------------------------------------- varlen causal attention (dense)
    lengths = [5, 1, 9, 16]
    cu = torch.tensor([0] + list(np.cumsum(lengths)))
    g = tg.Graph.cu_seqlens(cu, causal=True)
    T = int(cu[-1])
    q = torch.randn(T, 2, 16, generator=gen).requires_grad_()
    k = torch.randn(T, 2, 16, generator=gen).requires_grad_()
    v = torch.randn(T, 2, 16, generator=gen).requires_grad_()
    scale = 16 ** -0.5
    out = Attention().reference(graph=g, src={"key": k, "value": v}, dst={"query": q}, scale=scale)
    dy = torch.randn(out.shape, generator=gen)
    dq, dk, dv = torch.autograd.grad((out * dy).sum(), (q, k, v))
    from tiga.interop.torch.graph import from_native
    rp, ci = from_native(g).resolve_csr()
    saved.update(attn_cu=cu.numpy(), attn_row_ptr=rp.numpy(), attn_col=ci.numpy(), attn_q=q.detach().numpy(),
                 attn_k=k.detach().numpy(), attn_v=v.detach().numpy(), attn_out=out.detach().numpy(),
                 attn_dy=dy.numpy(), attn_dq=dq.numpy(), attn_dk=dk.numpy(), attn_dv=dv.numpy(),
                 attn_scale=np.float32(scale))

    # ----------------------------------------------- CSR construction (int)
    src = torch.randint(0, 23, (200,), generator=gen)
    dst = torch.randint(0, 17, (200,), generator=gen)
    from tiga.interop.torch.graph import Graph as TorchGraph
    tgc = TorchGraph.from_coo(src, dst, num_src=23, num_dst=17)
    rp, ci = tgc.resolve_csr()
    dest = tgc.destination_index(rp)
    order = torch.argsort(ci, stable=True)  # relation_vjp.py:75
    saved.update(coo_src=src.numpy(), coo_dst=dst.numpy(), coo_row_ptr=rp.numpy(), coo_col=ci.numpy(),
                 coo_destination=dest.numpy(), coo_t_order=order.numpy(), coo_t_col=dest[order].numpy(),
                 coo_t_ptr=torch.cat((torch.zeros(1, dtype=torch.int64),
                                      torch.bincount(ci, minlength=23).cumsum(0))).numpy(),
                 coo_degree_bounds=np.array(tgc.degree_bounds(), dtype=np.int64))

    # --------------------------------------------------- partition + halos
    table = []
    for entities in (0, 1, 7, 16, 17, 1000):
        for world in (1, 2, 3, 4, 8):
            for rank in range(world):
                b, e = owned_range(entities, world, rank)
                table.append((entities, world, rank, b, e))
    saved["owned_range_table"] = np.array(table, dtype=np.int64)
    owners = [(e, 17, w, destination_owner(e, 17, w)) for w in (1, 2, 3, 4, 8) for e in range(17)]
    saved["destination_owner_table"] = np.array(owners, dtype=np.int64)
    n = 37
    deg = torch.randint(0, 9, (n,), generator=gen)
    rp = torch.cat((torch.zeros(1, dtype=torch.int64), deg.cumsum(0)))
    ci = torch.randint(0, n, (int(rp[-1]),), generator=gen)
    saved["halo_row_ptr"], saved["halo_col"] = rp.numpy(), ci.numpy()
    for world in (2, 3, 4):
        maps = [derive_halo_map(rp.tolist(), ci.tolist(), num_entities=n, world_size=world, rank=r)
                for r in range(world)]
        for r, m in enumerate(maps):
            requests = [[i for i in maps[p].ghost_ids if m.owned_begin <= i < m.owned_end] for p in range(world)]
            full = derive_halo_map(rp.tolist(), ci.tolist(), num_entities=n, world_size=world, rank=r,
                                   peer_requests=requests)
            saved[f"halo_w{world}_r{r}_ghosts"] = np.array(full.ghost_ids, dtype=np.int64)
            saved[f"halo_w{world}_r{r}_range"] = np.array([full.owned_begin, full.owned_end], dtype=np.int64)
            for peer, ids in full.receive_from:
                saved[f"halo_w{world}_r{r}_recv{peer}"] = np.array(ids, dtype=np.int64)
            for peer, ids in full.send_to:
                saved[f"halo_w{world}_r{r}_send{peer}"] = np.array(ids, dtype=np.int64)
            saved[f"halo_w{world}_r{r}_bytes"] = np.int64(full.bytes_for(4, 64))

    path = os.path.join(HERE, "reference_cases.npz")
    np.savez_compressed(path, **{k: v for k, v in saved.items() if v is not None})
    print(f"wrote {path}: {len(saved)} arrays, {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    main()
