"""``tg.MessagePassing``: relation traversal + edge UDF + reducer.

Public surface of python/tiga/message_passing/core.py:543-775 of the
reference (keyword-only call, ``ndata=`` sugar, ``prepare``, ``reference``,
``explain()/cache_info``), with the Torch adapter's dispatcher
(python/tiga/interop/torch/message_passing.py:1523-1651,2817-2894,3564-3584,
3800-3882) replaced by a small recogniser that routes CUDA inputs to the
hand-written sm_100a kernels:

* ``edge.w * src.x`` / ``src.x`` with ``tg.sum()``, ``tg.mean()`` or a
  maximum algebra          -> tgb_csr_reduce_fwd / _bwd_dx / _bwd_dw
* GAT edge attention with ``tg.online_softmax()``  -> tgb_gat_fwd / _bwd
* dense / packed causal attention                  -> tgb_varlen_attn_fwd / _bwd

There is no CPU execution path and no library fallback: inputs that fit no
native kernel raise ``NotImplementedError``.  ``kernel.reference(...)`` is the
reference's eager semantic evaluator (plain Torch ops, any device) and is kept
as a public debugging API only; nothing in ``__call__`` routes through it.
"""
from __future__ import annotations

from collections.abc import Mapping
from types import SimpleNamespace
from typing import Any

import torch

from . import capture as cap
from .graph import Graph
from .kernel import CompiledVariant, Kernel
from .reducer import (MaxReducer, MeanReducer, OnlineSoftmaxItem, OnlineSoftmaxReducer, ProductReducer, Reducer,
                      ReducerCall, SumReducer)

PROVIDER = "b200-native"


def _resolve_node_fields(graph, src, dst, ndata):
    if ndata is not None:
        if src is not None or dst is not None:
            raise TypeError("ndata= cannot be combined with src=/dst=")
        if graph.schema.num_src != graph.schema.num_dst:
            raise ValueError("ndata= requires a homogeneous relation (num_src == num_dst); "
                             "declare src= and dst= separately for bipartite graphs")
        src = dst = dict(ndata)
    if src is None or dst is None:
        raise TypeError("message passing requires ndata= or both src= and dst= mappings")
    return src, dst


def _validate_fields(role, fields, entities, device) -> None:
    if not isinstance(fields, Mapping):
        raise TypeError(f"{role} fields must be a mapping")
    for name, value in fields.items():
        if not isinstance(value, torch.Tensor):
            raise TypeError(f"{role}.{name} must be a torch.Tensor")
        if value.ndim == 0 or value.shape[0] != entities:
            raise ValueError(f"{role}.{name} leading dimension must be {entities}, got {tuple(value.shape)}")
        if value.device != device:
            raise ValueError(f"{role}.{name} must be on {device}")


def _reducer_kind(reducer) -> str | None:
    if isinstance(reducer, SumReducer):
        return "sum"
    if isinstance(reducer, MeanReducer):
        return "mean"
    if isinstance(reducer, MaxReducer):
        return "max"
    if isinstance(reducer, (OnlineSoftmaxReducer, ProductReducer)):
        return None
    algebra = cap.reducer_algebra(reducer)
    return algebra


class _Prepared:
    """Zero-argument callable returned by ``prepare`` (tensor contents stay live)."""

    def __init__(self, kernel, graph, src, dst, edge, params):
        self._call = lambda: kernel(graph=graph, src=src, dst=dst, edge=edge, **params)
        self.graph = graph
        self._kernel = kernel
        self._call()  # specialise now, like the reference's prepare
        self.variant = kernel.last_variant

    def __call__(self):
        return self._call()


class MessagePassing(Kernel):
    reducer: Reducer = SumReducer()

    def __init__(self) -> None:
        super().__init__()
        self._torch_fast_path = None

    def edge(self, src, dst, edge, **params):
        raise NotImplementedError

    def node(self, dst, aggregate, **params):
        return aggregate

    # ------------------------------------------------------------------ call
    def __call__(self, *, graph: Graph, src=None, dst=None, edge=None, ndata=None, **params: Any):
        if not getattr(graph, "_tiga_graph", False):
            raise TypeError("graph must be a tiga.Graph")
        src, dst = _resolve_node_fields(graph, src, dst, ndata)
        edge = {} if edge is None else edge
        if graph.is_distributed:
            from .distributed.runtime import current_distributed_runtime, execute_sharded_message_passing

            if current_distributed_runtime() is None:
                raise RuntimeError("a Graph.halo() snapshot needs an active DistributedRuntime")
            return execute_sharded_message_passing(self, graph=graph, src=src, dst=dst, edge=edge, params=params)
        _validate_fields("src", src, graph.schema.num_src, graph.device)
        _validate_fields("dst", dst, graph.schema.num_dst, graph.device)
        if graph.device.type != "cuda":
            raise NotImplementedError(
                "this build executes MessagePassing on CUDA tensors only; there is no CPU path "
                "(kernel.reference(...) evaluates the eager semantic definition on any device)")
        aggregate = self._execute_native(graph, src, dst, edge, params)
        if type(self).node is MessagePassing.node:
            return aggregate
        return cap.call_region(self.node, (SimpleNamespace(**dst), aggregate), params)

    def _record(self, graph, lowering, passes, remarks, extra_key=()):
        key = (type(self).__qualname__, self.reducer.specialization_key(), graph.specialization_key(),
               lowering, *extra_key)
        if self._lookup_variant(key) is None:
            self._cache_misses += 1
            self._record_variant(CompiledVariant(
                key=key, backend=str(graph.device), provider=PROVIDER, lowering=lowering,
                domain_plan=f"gf.apply @{type(self).__name__} reducer={self.reducer.name}",
                passes=passes, remarks=remarks))
        else:
            self._cache_hits += 1

    def _execute_native(self, graph, src, dst, edge, params):
        from . import ops

        staged = cap.capture_edge(self.edge, params)
        if staged is None:
            raise NotImplementedError(
                f"edge() of {type(self).__name__} leaves the staging vocabulary "
                "(field, +, -, *, /, sum(-1), maximum, exp); no native kernel and no fallback exists")
        if isinstance(self.reducer, OnlineSoftmaxReducer):
            return self._execute_online_softmax(graph, src, dst, edge, params, staged)
        kind = _reducer_kind(self.reducer)
        pattern = cap.recognize_weighted_sum(staged)
        if kind is None or pattern is None:
            raise NotImplementedError(
                f"no native kernel for reducer {type(self.reducer).__name__} with this edge expression")
        if graph.schema.realization not in {"materialized_csr"} and graph._row_ptr is None:
            graph.resolve_csr()
        row_ptr, col_idx = graph.resolve_csr()
        _validate_fields("edge", edge, col_idx.numel(), graph.device)
        if pattern.src_field not in src:
            raise KeyError(f"edge() reads src.{pattern.src_field}, which was not bound")
        x = src[pattern.src_field]
        w = None
        if pattern.edge_field is not None:
            if pattern.edge_field not in edge:
                raise KeyError(f"edge() reads edge.{pattern.edge_field}, which was not bound")
            w = edge[pattern.edge_field]
            if w.numel() != col_idx.numel():
                raise NotImplementedError("edge weights must be one scalar per edge ([E] or [E, 1])")
        identity = float(self.reducer.identity()) if kind in ("sum", "max") else 0.0
        out = ops.csr_reduce(graph, kind, x, w, identity)
        info = graph.native_plan(transpose=False).info
        self._record(
            graph, f"b200-csr-{'weighted-sum' if kind == 'sum' else kind}-degree-bucket",
            ("capture-edge-udf", "recognize-weighted-sum", "plan-degree-buckets", "plan-split-rows",
             "cache-transposed-relation"),
            (f"rows by degree bucket, {info['long_rows']} split rows in {info['segments']} segments of "
             f"{info['segment_edges']} edges",
             "backward: dx gathers over the cached stable transposed relation (no atomics), "
             "dw is a per-edge dot product"),
            extra_key=(tuple(x.shape[1:]), w is not None))
        return out

    def _execute_online_softmax(self, graph, src, dst, edge, params, staged):
        gat = cap.recognize_gat(staged)
        if gat is not None:
            from . import attention

            out = attention.gat_attention(graph, src[gat.src_field], dst[gat.dst_field],
                                          params[gat.src_param], params[gat.dst_param], gat.slope)
            self._record(graph, "b200-csr-edge-attention-online-softmax",
                         ("capture-edge-udf", "recognize-gat-logit", "plan-degree-buckets"),
                         ("row-centric online softmax, float32 state, (m, l) saved for backward",))
            return out
        dense = cap.recognize_dense_attention(self._with_scalar_params(params))
        if dense is not None and graph.sequence_boundaries() is not None:
            from . import attention

            out = attention.varlen_attention(graph, dst[dense.query_field], src[dense.key_field],
                                             src[dense.value_field], dense.scale)
            self._record(graph, "b200-dense-streaming-reduction-tcgen05",
                         ("capture-edge-udf", "recognize-dense-attention", "schedule-varlen-tiles"),
                         ("implicit block-lower-triangular relation; no edge is materialised",))
            return out
        raise NotImplementedError("no native kernel for this online_softmax edge expression")

    def _with_scalar_params(self, params):
        # float params (e.g. scale) must appear as constants in the staged tree
        return cap.capture_edge(self.edge, params)

    # ------------------------------------------------------------- prepare
    def prepare(self, *, graph: Graph, src=None, dst=None, edge=None, ndata=None, **params: Any):
        src, dst = _resolve_node_fields(graph, src, dst, ndata)
        return _Prepared(self, graph, src, dst, {} if edge is None else edge, params)

    # ----------------------------------------------------------- reference
    def reference(self, *, graph: Graph, src, dst, edge=None, **params: Any):
        """Eager semantic evaluator (materialises per-edge tensors with Torch
        ops), the reference's ``kernel.reference``
        (python/tiga/interop/torch/message_passing.py:2817-2894).  A debugging
        aid: it is never used by ``__call__``."""
        if isinstance(self.reducer, OnlineSoftmaxReducer) and self.reducer.block_prune_threshold is not None:
            raise NotImplementedError("the block-pruned approximation has no eager reference")
        if graph.is_distributed:
            raise NotImplementedError("reference() cannot evaluate one shard of a Graph.halo() snapshot")
        edge = {} if edge is None else edge
        _validate_fields("src", src, graph.schema.num_src, graph.device)
        _validate_fields("dst", dst, graph.schema.num_dst, graph.device)
        row_ptr, col_idx = graph.resolve_csr()
        _validate_fields("edge", edge, col_idx.numel(), graph.device)
        destination = graph.destination_index(row_ptr)
        src_at_edge = SimpleNamespace(**{name: value[col_idx] for name, value in src.items()})
        dst_at_edge = SimpleNamespace(**{name: value[destination] for name, value in dst.items()})
        message = cap.call_region(self.edge, (src_at_edge, dst_at_edge, SimpleNamespace(**edge)), params)
        if isinstance(message, ReducerCall):
            if len(message.messages) != 1:
                raise NotImplementedError("the eager evaluator takes single-message reducer bindings")
            message = message.messages[0]
        aggregate = _eager_reduce(self.reducer, message, destination, graph.schema.num_dst)
        if type(self).node is MessagePassing.node:
            return aggregate
        return cap.call_region(self.node, (SimpleNamespace(**dst), aggregate), params)


def _eager_reduce(reducer, message, destination, num_dst):
    """Torch restatement of the reducer semantics
    (python/tiga/interop/torch/reducer_oracle.py:44-208)."""
    destination = destination.to(torch.int64)
    if isinstance(reducer, OnlineSoftmaxReducer):
        if not isinstance(message, OnlineSoftmaxItem):
            raise TypeError("online_softmax edge() must return self.reducer(score, value)")
        score, value = message.score, message.value
        while score.ndim > 1 and score.shape[-1] == 1:
            score = score.squeeze(-1)
        acc = torch.float32 if score.dtype in (torch.float16, torch.bfloat16) else score.dtype
        s, v = score.to(acc), value.to(acc)
        lanes = tuple(s.shape[1:])
        payload = v.ndim - s.ndim
        maximum = torch.full((num_dst, *lanes), -torch.inf, device=s.device, dtype=acc)
        index = destination.reshape(-1, *((1,) * len(lanes))).expand_as(s)
        maximum.scatter_reduce_(0, index, s, reduce="amax", include_self=True)
        scale = torch.exp(s - maximum[destination])
        denominator = torch.zeros_like(maximum).index_add_(0, destination, scale)
        numerator = torch.zeros((num_dst, *v.shape[1:]), device=v.device, dtype=acc)
        numerator.index_add_(0, destination, v * scale.reshape(*scale.shape, *((1,) * payload)))
        denominator = denominator.reshape(*denominator.shape, *((1,) * payload))
        result = torch.where(denominator > 0, numerator / denominator.clamp_min(torch.finfo(acc).tiny),
                             torch.zeros_like(numerator))
        return result.to(value.dtype)
    if not isinstance(message, torch.Tensor):
        raise TypeError(f"{reducer.name} reducer message must be a Tensor")
    shape = (num_dst, *message.shape[1:])
    kind = _reducer_kind(reducer)
    if kind == "sum":
        return torch.full(shape, reducer.identity(), dtype=message.dtype,
                          device=message.device).index_add_(0, destination, message)
    if kind == "mean":
        total = torch.zeros(shape, dtype=message.dtype, device=message.device).index_add_(0, destination, message)
        count = torch.zeros(num_dst, dtype=message.dtype, device=message.device).index_add_(
            0, destination, torch.ones_like(destination, dtype=message.dtype))
        return total / count.reshape(num_dst, *((1,) * (message.ndim - 1)))
    if kind == "max":
        start = torch.full(shape, float(reducer.identity()), dtype=message.dtype, device=message.device)
        index = destination.reshape(-1, *((1,) * (message.ndim - 1))).expand_as(message)
        return start.scatter_reduce(0, index, message, reduce="amax", include_self=True)
    if isinstance(reducer, ProductReducer):
        start = torch.full(shape, reducer.identity(), dtype=message.dtype, device=message.device)
        return start.index_reduce(0, destination, message, "prod")
    raise NotImplementedError(f"no eager evaluator for reducer {type(reducer).__name__}")


__all__ = ["MessagePassing"]
