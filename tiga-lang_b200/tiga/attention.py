"""Online-softmax programs on the native kernels: GAT edge attention over CSR
rows and (dense / packed causal) relation attention.

The autograd Functions save only inputs, the output and the per-row softmax
state (m, l), like the reference's ``_EdgeNNAttentionFunction``
(python/tiga/interop/torch/message_passing.py:193-277), and recompute per-edge
quantities in the backward.
"""
from __future__ import annotations

import ctypes

import torch

from . import _native


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _gat_scratch(plan, H, D, backward, device):
    size = ctypes.c_uint64()
    _native.check(_native.lib().tgb_gat_scratch_bytes(plan.handle, H, D, int(backward), ctypes.byref(size)),
                  "tgb_gat_scratch_bytes")
    buffer = torch.empty(max(int(size.value), 256), dtype=torch.uint8, device=device)
    return buffer, int(size.value)


def _node_scores(x, a, H, D):
    scores = torch.empty((x.shape[0], H), dtype=torch.float32, device=x.device)
    _native.check(_native.lib().tgb_gat_node_scores(x.data_ptr(), a.data_ptr(), x.shape[0], H, D,
                                                    scores.data_ptr(), _stream(x.device)), "tgb_gat_node_scores")
    return scores


class GATFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_src, x_dst, a_src, a_dst, graph, slope):
        for name, t in (("src feature", x_src), ("dst feature", x_dst), ("a_src", a_src), ("a_dst", a_dst)):
            if t.dtype != torch.bfloat16:
                raise NotImplementedError(f"edge attention kernels take bfloat16 inputs; {name} is {t.dtype}")
        if x_src.ndim != 3 or x_dst.shape[1:] != x_src.shape[1:] or a_src.shape != x_src.shape[1:] \
                or a_dst.shape != x_src.shape[1:]:
            raise NotImplementedError("edge attention expects x [N, H, D] and a_src, a_dst [H, D]")
        H, D = x_src.shape[1], x_src.shape[2]
        xs, xd = x_src.contiguous(), x_dst.contiguous()
        a_s, a_d = a_src.contiguous(), a_dst.contiguous()
        needs_grad = any(t.requires_grad for t in (x_src, x_dst, a_src, a_dst))
        plan = graph.native_plan(transpose=needs_grad)
        lib = _native.lib()
        with torch.cuda.device(xs.device):
            s_src = _node_scores(xs, a_s, H, D)
            s_dst = s_src if (xd is xs or xd.data_ptr() == xs.data_ptr()) and a_d.data_ptr() == a_s.data_ptr() \
                else _node_scores(xd, a_d, H, D)
            out = torch.empty((graph.num_dst, H, D), dtype=torch.bfloat16, device=xs.device)
            m = torch.empty((graph.num_dst, H), dtype=torch.float32, device=xs.device)
            l = torch.empty_like(m)
            scratch, size = _gat_scratch(plan, H, D, False, xs.device)
            _native.check(lib.tgb_gat_fwd(plan.handle, xs.data_ptr(), s_src.data_ptr(), s_dst.data_ptr(),
                                          out.data_ptr(), m.data_ptr(), l.data_ptr(), H, D, float(slope),
                                          scratch.data_ptr(), size, _stream(xs.device)), "tgb_gat_fwd")
        ctx.graph, ctx.slope = graph, float(slope)
        ctx.save_for_backward(x_src, x_dst, a_src, a_dst, s_src, s_dst, out, m, l)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        x_src, x_dst, a_src, a_dst, s_src, s_dst, out, m, l = ctx.saved_tensors
        graph = ctx.graph
        H, D = x_src.shape[1], x_src.shape[2]
        plan = graph.native_plan(transpose=True)
        xs, xd = x_src.contiguous(), x_dst.contiguous()
        a_s, a_d = a_src.contiguous(), a_dst.contiguous()
        dout = grad_output.contiguous().to(torch.bfloat16)
        device = xs.device
        dx_src = torch.empty_like(xs)
        dx_dst = torch.empty_like(xd)
        da_src = torch.empty((H, D), dtype=torch.float32, device=device)
        da_dst = torch.empty_like(da_src)
        with torch.cuda.device(device):
            scratch, size = _gat_scratch(plan, H, D, True, device)
            _native.check(_native.lib().tgb_gat_bwd(
                plan.handle, xs.data_ptr(), xd.data_ptr(), a_s.data_ptr(), a_d.data_ptr(), s_src.data_ptr(),
                s_dst.data_ptr(), out.data_ptr(), dout.data_ptr(), m.data_ptr(), l.data_ptr(), H, D, ctx.slope,
                dx_src.data_ptr(), dx_dst.data_ptr(), da_src.data_ptr(), da_dst.data_ptr(), scratch.data_ptr(),
                size, _stream(device)), "tgb_gat_bwd")
        needs = ctx.needs_input_grad
        return (dx_src if needs[0] else None, dx_dst if needs[1] else None,
                da_src.to(a_src.dtype) if needs[2] else None, da_dst.to(a_dst.dtype) if needs[3] else None,
                None, None)


def gat_attention(graph, x_src, x_dst, a_src, a_dst, slope: float):
    if not x_src.is_cuda:
        raise RuntimeError("edge attention runs on CUDA tensors only (no CPU fallback)")
    if x_src.dtype == torch.float32:
        return _gat_attention_float32(graph, x_src, x_dst, a_src, a_dst, slope)
    return GATFunction.apply(x_src, x_dst, a_src, a_dst, graph, slope)


def _gat_attention_float32(graph, x_src, x_dst, a_src, a_dst, slope: float):
    """float32 edge attention (the precision of the reference's nn-attention kernel,
    python/tiga/compiler/edge_nn_attention.py:127-338).  The fused bf16 kernels do not apply; the
    program is lowered onto the stable-weighted softmax kernels instead: the per-node halves of the
    logit and the per-edge score [E, H] are assembled with Torch element-wise / gather ops (a
    per-edge scalar per head, never an [E, H, D] temporary), and the gather-heavy part -- softmax
    over each destination row and the weighted sum of source rows, forward and backward -- runs in
    tgb_softmax_field_fwd / _bwd.  Autograd carries the score's cotangent back to x and a; the
    per-source accumulation there is Torch's index_add (atomic adds)."""
    for name, t in (("dst feature", x_dst), ("a_src", a_src), ("a_dst", a_dst)):
        if t.dtype != torch.float32:
            raise NotImplementedError(f"edge attention inputs must share one dtype; {name} is {t.dtype}")
    if x_src.ndim != 3 or x_dst.shape[1:] != x_src.shape[1:] or a_src.shape != x_src.shape[1:] \
            or a_dst.shape != x_src.shape[1:]:
        raise NotImplementedError("edge attention expects x [N, H, D] and a_src, a_dst [H, D]")
    row_ptr, col_idx = graph.resolve_csr()
    destination = graph.destination_index(row_ptr).long()
    s_src = (x_src * a_src).sum(dim=-1)                     # [num_src, H]
    s_dst = (x_dst * a_dst).sum(dim=-1)                     # [num_dst, H]
    pre = s_src.index_select(0, col_idx.long()) + s_dst.index_select(0, destination)
    score = torch.maximum(pre, pre * slope)
    return FieldSoftmaxFunction.apply(score, x_src, graph)


class FieldSoftmaxFunction(torch.autograd.Function):
    """``online_softmax(edge.score, src.value)``: scores per edge, values per source.

    score [E, *lanes] (trailing singleton dims are dropped, as the reference's evaluator does,
    python/tiga/interop/torch/reducer_oracle.py:69-72), value [num_src, *lanes, *payload];
    float32 state; the result has the value's dtype and is exactly 0 for a row without edges."""

    @staticmethod
    def forward(ctx, score, value, graph):
        squeezed = score
        while squeezed.ndim > 1 and squeezed.shape[-1] == 1:
            squeezed = squeezed.squeeze(-1)
        lanes = tuple(squeezed.shape[1:])
        if tuple(value.shape[1:1 + len(lanes)]) != lanes:
            raise ValueError(f"value {tuple(value.shape)} does not carry the score's lanes {lanes}")
        if value.dtype not in (torch.float32, torch.bfloat16):
            raise NotImplementedError(f"online-softmax values must be float32 or bfloat16, got {value.dtype}")
        if not score.dtype.is_floating_point:
            raise NotImplementedError("online-softmax scores must be floating point")
        H = 1
        for extent in lanes:
            H *= int(extent)
        E, num_src = squeezed.shape[0], value.shape[0]
        D = max(int(value.numel() // max(num_src * H, 1)), 1) if num_src else 1
        s32 = squeezed.reshape(E, H).to(torch.float32).contiguous()
        v = value.contiguous()
        needs_grad = score.requires_grad or value.requires_grad
        plan = graph.native_plan(transpose=needs_grad)
        if plan.num_edges != E or plan.num_src != num_src:
            raise ValueError("score must have one row per edge and value one row per source")
        device = v.device
        out = torch.empty((plan.num_dst, H * D), dtype=torch.float32, device=device)
        m = torch.empty((plan.num_dst, H), dtype=torch.float32, device=device)
        l = torch.empty_like(m)
        dtype_id = _native.DTYPE_BF16 if v.dtype == torch.bfloat16 else _native.DTYPE_F32
        with torch.cuda.device(device):
            _native.check(_native.lib().tgb_softmax_field_fwd(
                plan.handle, s32.data_ptr(), v.data_ptr(), dtype_id, out.data_ptr(), m.data_ptr(), l.data_ptr(),
                H, D, _stream(device)), "tgb_softmax_field_fwd")
        ctx.graph, ctx.H, ctx.D, ctx.dtype_id = graph, H, D, dtype_id
        ctx.score_meta, ctx.value_meta = (score.shape, score.dtype), (value.shape, value.dtype)
        ctx.save_for_backward(s32, v, out, m, l)
        return out.reshape((plan.num_dst,) + tuple(value.shape[1:])).to(value.dtype)

    @staticmethod
    def backward(ctx, grad_output):
        s32, v, out, m, l = ctx.saved_tensors
        plan = ctx.graph.native_plan(transpose=True)
        H, D = ctx.H, ctx.D
        device = v.device
        dout = grad_output.reshape(plan.num_dst, H * D).to(torch.float32).contiguous()
        d_score = torch.empty_like(s32)
        d_value = torch.empty((plan.num_src, H * D), dtype=torch.float32, device=device)
        weights = torch.empty_like(s32)
        with torch.cuda.device(device):
            _native.check(_native.lib().tgb_softmax_field_bwd(
                plan.handle, s32.data_ptr(), v.data_ptr(), ctx.dtype_id, out.data_ptr(), dout.data_ptr(),
                m.data_ptr(), l.data_ptr(), H, D, d_score.data_ptr(), d_value.data_ptr(), weights.data_ptr(),
                _stream(device)), "tgb_softmax_field_bwd")
        (score_shape, score_dtype), (value_shape, value_dtype) = ctx.score_meta, ctx.value_meta
        needs = ctx.needs_input_grad
        return (d_score.reshape(score_shape).to(score_dtype) if needs[0] else None,
                d_value.reshape(value_shape).to(value_dtype) if needs[1] else None, None)


def field_softmax(graph, score, value):
    if not value.is_cuda:
        raise RuntimeError("the online-softmax reducer runs on CUDA tensors only (no CPU fallback)")
    return FieldSoftmaxFunction.apply(score, value, graph)


def _attention_tiles(graph, device, heads, kv_heads):
    """int32 [n, 4] = (first token of the tile, sequence begin, sequence end, head) for every
    (128-token tile, head).  Order: longest sequence first, then head, then the heaviest tile of
    that (sequence, head) first -- CTAs that are resident together then read the same K/V (or
    Q/dO) stream, which keeps it in L2, while the long tiles still start early.  Returns the
    table for the query-major kernels (query heads), the causal flag and the table for the
    key-major kernel (key/value heads)."""
    cached = graph.__dict__.get("_attention_tiles")
    if cached is not None and cached[0].device == device and cached[3] == (heads, kv_heads):
        return cached
    bounds = graph.sequence_boundaries().tolist()
    causal = graph._dense_boundary == "lower_inclusive"
    sequences = sorted(zip(bounds[:-1], bounds[1:]), key=lambda be: be[0] - be[1])

    def table(key_major, count):
        rows = []
        for begin, end in sequences:
            starts = list(range(begin, end, 128))
            # query-major + causal: later tiles see more keys; key-major + causal: earlier tiles see more queries
            if causal and not key_major:
                starts.reverse()
            for head in range(count):
                rows.extend((t0, begin, end, head) for t0 in starts)
        return torch.tensor(rows, dtype=torch.int32).reshape(-1, 4).to(device)

    graph.__dict__["_attention_tiles"] = (table(False, heads), causal, table(True, kv_heads), (heads, kv_heads))
    return graph.__dict__["_attention_tiles"]


class VarlenAttentionFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, query, key, value, graph, scale):
        from . import ops

        for name, t in (("query", query), ("key", key), ("value", value)):
            if t.dtype != torch.bfloat16:
                raise NotImplementedError(f"dense attention kernels take bfloat16 inputs; {name} is {t.dtype}")
            if t.ndim != 3:
                raise NotImplementedError("dense attention expects fields of shape [tokens, heads, D]")
        tokens, H, D = query.shape
        H_kv = key.shape[1]
        if key.shape != value.shape or key.shape[0] != tokens or key.shape[2] != D or H % max(H_kv, 1):
            raise NotImplementedError(
                "dense attention expects key and value of one shape [tokens, H_kv, D] with the query's tokens "
                f"and D, and H a multiple of H_kv (grouped queries); got query {tuple(query.shape)}, "
                f"key {tuple(key.shape)}, value {tuple(value.shape)}")
        if tokens != graph.num_dst:
            raise ValueError(f"fields must have {graph.num_dst} rows, got {tokens}")
        q, k, v = query.contiguous(), key.contiguous(), value.contiguous()
        tiles, causal, _, _ = _attention_tiles(graph, q.device, H, H_kv)
        out = torch.empty_like(q)
        lse = torch.empty((tokens, H), dtype=torch.float32, device=q.device)
        with torch.cuda.device(q.device):
            _native.check(_native.lib().tgb_varlen_attn_fwd(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), tiles.data_ptr(),
                tiles.shape[0], tokens, H, H_kv, D, float(scale), int(causal), ops.error_flag(q.device).data_ptr(),
                _stream(q.device)), "tgb_varlen_attn_fwd")
            ops.launched(q.device)
        ctx.graph, ctx.scale = graph, float(scale)
        ctx.save_for_backward(q, k, v, out, lse)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        from . import ops

        q, k, v, out, lse = ctx.saved_tensors
        tokens, H, D = q.shape
        H_kv = k.shape[1]
        d_out = grad_output.contiguous().to(torch.bfloat16)
        query_tiles, causal, key_tiles, _ = _attention_tiles(ctx.graph, q.device, H, H_kv)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        delta = torch.empty((tokens, H), dtype=torch.float32, device=q.device)
        with torch.cuda.device(q.device):
            _native.check(_native.lib().tgb_varlen_attn_bwd(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), d_out.data_ptr(), lse.data_ptr(),
                dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), delta.data_ptr(), query_tiles.data_ptr(),
                key_tiles.data_ptr(), query_tiles.shape[0], key_tiles.shape[0], tokens, H, H_kv, D, ctx.scale,
                int(causal), ops.error_flag(q.device).data_ptr(), _stream(q.device)), "tgb_varlen_attn_bwd")
            ops.launched(q.device)
        return dq, dk, dv, None, None


def varlen_attention(graph, query, key, value, scale):
    """softmax(q k^T * scale [+ causal]) v inside every sequence of a packed batch; with fewer
    key/value heads than query heads, consecutive query heads share one (grouped queries)."""
    if not query.is_cuda:
        raise RuntimeError("dense attention runs on CUDA tensors only (no CPU fallback)")
    return VarlenAttentionFunction.apply(query, key, value, graph, scale)
