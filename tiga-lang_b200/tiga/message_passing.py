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


def _active_program():
    from .program import active_program

    return active_program()


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


def _implicit_edge_names(graph) -> tuple[str, ...]:
    """Names of the edge fields a relation provides by itself (geometric relations only)."""
    return ("displacement", "distance") if getattr(graph, "_geometry", None) is not None else ()


def _refuse_shadowing(implicit, edge) -> None:
    overlap = set(implicit) & set(edge)
    if overlap:
        raise ValueError(f"edge fields shadow graph-provided fields: {', '.join(sorted(overlap))}")


def _reducer_kind(reducer) -> str | None:
    """'sum' / 'mean' / 'max' / 'prod' / 'additive' for reducers the CSR kernels can fold, else None.
    'prod' is folded by the edge-program kernels only."""
    if isinstance(reducer, SumReducer):
        return "sum"
    if isinstance(reducer, MeanReducer):
        return "mean"
    if isinstance(reducer, MaxReducer):
        return "max"
    if isinstance(reducer, ProductReducer):
        return "prod"
    if isinstance(reducer, OnlineSoftmaxReducer):
        return None
    return cap.reducer_algebra(reducer)


class _StableSoftmaxAlgebra(Reducer):
    """``tg.online_softmax()`` as a plain tuple algebra -- state (running maximum, denominator,
    numerator), the regions of the reference's ``capture_online_softmax``
    (python/tiga/compiler/reducer_capture.py:133-189) -- for score / value expressions no dedicated
    kernel takes.  A row without edges finalizes to 0 / tiny = 0, the reference's empty-row value."""

    name = "online_softmax"
    associative = commutative = True

    def identity(self):
        return -1.0e30, 0.0, 0.0

    def lift(self, score, value):
        return score, 1.0, value

    def combine(self, left, right):
        from . import math as tg_math

        top = tg_math.maximum(left[0], right[0])
        keep_left, keep_right = tg_math.exp(left[0] - top), tg_math.exp(right[0] - top)
        return top, keep_left * left[1] + keep_right * right[1], keep_left * left[2] + keep_right * right[2]

    def finalize(self, state):
        from . import math as tg_math

        return state[2] / tg_math.maximum(state[1], 1.0e-30)


_MISS = object()


def _tensor_spec(t: torch.Tensor):
    return (t.dtype, tuple(t.shape), tuple(t.stride()), t.device, t.requires_grad)


class _GuardedLaunch:
    """A specialised call kept for the warm path.

    The first call of a (kernel, reducer, graph, field layout, parameter) combination stages
    ``edge()``, recognises the program, builds launch plans and records a variant.  What it
    learned is stored here as `runner` plus the guards under which the runner stays valid:
    the same Graph object (graphs are immutable snapshots, so identity proves topology and plan),
    the same reducer object, and for every tensor the runner reads the same dtype, shape, strides,
    device and requires_grad; non-tensor parameters (they are folded into the staged program as
    constants) must compare equal.  A warm call therefore does no staging, no recognition and no
    key building: it checks the guards and launches.  The reference keeps the same kind of record
    (``_GuardedExecutable`` and the installed fast path,
    python/tiga/interop/torch/message_passing.py:974-1007, 3680-3797)."""

    __slots__ = ("graph", "reducer", "bindings", "specs", "constants", "scalars", "runner", "variant", "signature")

    def __init__(self, graph, reducer, bindings, tensors, constants, runner, variant):
        self.graph = graph
        # dynamic relations (Graph.radius / Graph.knn) are rebuilt per call, usually as new Graph
        # objects: their launches are guarded by the search signature instead of object identity and
        # the runner is re-pointed at the graph of the call (the reference's ranked executable reuse,
        # python/tiga/interop/torch/message_passing.py `_RankedExecutable`)
        self.signature = graph.dynamic_signature() if hasattr(runner, "cell") else None
        self.reducer = reducer
        self.bindings = tuple(bindings)            # (role, name) per tensor the runner takes
        self.specs = tuple(_tensor_spec(t) for t in tensors)
        # float params the compiled program reads at every call (the runner takes their current values)
        self.scalars = tuple(getattr(runner, "scalars", ()))
        # the other non-tensor params: absorbed into the staged program, so they must compare equal
        self.constants = {name: value for name, value in constants.items() if name not in self.scalars}
        self.runner = runner
        self.variant = variant

    def try_run(self, kernel, graph, src, dst, edge, params):
        if kernel.reducer is not self.reducer:
            return _MISS
        if graph is not self.graph:
            if self.signature is None or graph.dynamic_signature() != self.signature:
                return _MISS
        spaces = {"src": src, "dst": dst, "edge": edge, "param": params}
        tensors = []
        try:
            for (role, name), spec in zip(self.bindings, self.specs):
                t = spaces[role][name]
                if (t.dtype, tuple(t.shape), tuple(t.stride()), t.device, t.requires_grad) != spec:
                    return _MISS
                tensors.append(t)
            for name, value in self.constants.items():
                if params[name] != value:
                    return _MISS
            for name in self.scalars:
                if type(params[name]) not in (float, int):
                    return _MISS
        except (KeyError, TypeError, AttributeError):
            return _MISS
        # only the parameters edge() takes are part of the staged program; node() may take others
        if kernel._edge_parameter_count(params) != len(self.constants) + len(self.scalars) + sum(
                1 for role, _ in self.bindings if role == "param"):
            return _MISS
        if graph is not self.graph:
            self.runner.cell.graph = self.graph = graph
        if self.scalars:
            return self.runner(*tensors, scalars={name: params[name] for name in self.scalars})
        return self.runner(*tensors)


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
        self._launches: list[_GuardedLaunch] = []   # most recently used first

    @property
    def _torch_fast_path(self):
        """``(graph, src, dst, edge, params) -> (hit, result)`` once a call has specialised the
        kernel, else None: the hook name of the reference (python/tiga/message_passing/core.py:550-556)."""
        if not self._launches:
            return None

        def fast_path(graph, src, dst, edge, params):
            result = self._warm(graph, src, dst, edge, params)
            return (False, None) if result is _MISS else (True, result)

        return fast_path

    def edge(self, src, dst, edge, **params):
        raise NotImplementedError

    def _edge_parameter_count(self, params) -> int:
        """How many of the call's keyword parameters ``edge()`` receives (the signature is read once)."""
        spec = self.__dict__.get("_edge_parameter_spec")
        if spec is None:
            import inspect

            declared = inspect.signature(self.edge).parameters
            spec = (any(p.kind is inspect.Parameter.VAR_KEYWORD for p in declared.values()), frozenset(declared))
            self.__dict__["_edge_parameter_spec"] = spec
        return len(params) if spec[0] else sum(1 for name in params if name in spec[1])

    def node(self, dst, aggregate, **params):
        return aggregate

    # ------------------------------------------------------------------ call
    def __call__(self, *, graph: Graph, src=None, dst=None, edge=None, ndata=None, **params: Any):
        if not getattr(graph, "_tiga_graph", False):
            raise TypeError("graph must be a tiga.Graph")
        src, dst = _resolve_node_fields(graph, src, dst, ndata)
        edge = {} if edge is None else edge
        recording = _active_program()
        if recording is not None:          # inside @tg.program: the call becomes a lazy application
            return recording.apply(self, graph=graph, src=src, dst=dst, edge=edge, **params)
        if graph.schema.realization == "paged_csr" and graph._row_ptr is None:
            return self._execute_paged(graph, src, dst, edge, params)
        aggregate = self._warm(graph, src, dst, edge, params) if self._launches else _MISS
        if aggregate is _MISS:
            aggregate = self._cold(graph, src, dst, edge, params)
        if type(self).node is MessagePassing.node:
            return aggregate
        from .ops import as_aggregate      # `aggregate @ W` inside node() reaches the tensor-core linear

        return cap.call_region(self.node, (SimpleNamespace(**dst), as_aggregate(aggregate)), params)

    def _execute_paged(self, graph, src, dst, edge, params):
        """A graph whose topology lives in a .gfg directory: blocks of `graph.page_rows` destination
        rows are read from the memory-mapped files, moved to the device and reduced one after the
        other by the same kernels as a resident graph (execute_paged_message_passing,
        python/tiga/message_passing/paged.py:434-583 of the reference, which runs its host evaluator
        per page).  Source fields are whole tensors on the device, destination and edge fields are
        sliced per page; every page's plan is dropped before the next is built, so device memory
        holds one page of topology at a time.  Autograd works through the pages."""
        store = graph._paged_store
        _validate_fields("src", src, graph.schema.num_src, graph.device)
        _validate_fields("dst", dst, graph.schema.num_dst, graph.device)
        _validate_fields("edge", edge, store.num_edges, graph.device)
        if graph.device.type != "cuda":
            raise NotImplementedError("this build executes MessagePassing on CUDA tensors only; open the graph "
                                      "with tg.load(path, device='cuda')")
        pieces = []
        rows_per_page = max(int(graph.page_rows), 1)
        for begin in range(0, graph.schema.num_dst, rows_per_page):
            end = min(graph.schema.num_dst, begin + rows_per_page)
            row_ptr, col_idx, first = store.page_tensors(begin, end, graph.device)
            page = Graph.from_csr(row_ptr, col_idx, num_src=graph.schema.num_src)
            page_dst = {name: value[begin:end] for name, value in dst.items()}
            page_edge = {name: value[first:first + col_idx.numel()] for name, value in edge.items()}
            _, tensors, _, runner = self._specialise(page, src, page_dst, page_edge, params)
            aggregate = runner(*tensors)
            if type(self).node is not MessagePassing.node:
                aggregate = cap.call_region(self.node, (SimpleNamespace(**page_dst), aggregate), params)
            pieces.append(aggregate)
        if not pieces:
            raise NotImplementedError("a persistent graph without destination rows has nothing to execute")
        return torch.cat(pieces, dim=0)

    def _warm(self, graph, src, dst, edge, params):
        launches = self._launches
        for position, launch in enumerate(launches):
            result = launch.try_run(self, graph, src, dst, edge, params)
            if result is not _MISS:
                if position:
                    launches.insert(0, launches.pop(position))
                self._cache.hits += 1
                self._cache.last = launch.variant
                return result
        return _MISS

    def _cold(self, graph, src, dst, edge, params):
        if graph.is_distributed:
            from .distributed.runtime import current_distributed_runtime, specialise_sharded_message_passing

            if current_distributed_runtime() is None:
                raise RuntimeError("a Graph.halo() snapshot needs an active DistributedRuntime")
            bindings, tensors, constants, runner = specialise_sharded_message_passing(
                self, graph=graph, src=src, dst=dst, edge=edge, params=params)
        else:
            _validate_fields("src", src, graph.schema.num_src, graph.device)
            _validate_fields("dst", dst, graph.schema.num_dst, graph.device)
            if graph.device.type != "cuda":
                raise NotImplementedError(
                    "this build executes MessagePassing on CUDA tensors only; there is no CPU path "
                    "(kernel.reference(...) evaluates the eager semantic definition on any device)")
            bindings, tensors, constants, runner = self._specialise(graph, src, dst, edge, params)
        result = runner(*tensors)
        launch = _GuardedLaunch(graph, self.reducer, bindings, tensors, constants, runner, self.last_variant)
        self._launches.insert(0, launch)
        del self._launches[8:]
        return result

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

    # ------------------------------------------------------ specialisation
    def _specialise(self, graph, src, dst, edge, params):
        """Stage ``edge()``, recognise the program and return
        (bindings, tensors, constants, runner): `runner(*tensors)` launches the native kernels."""
        consumed: set = set()           # float params whose value Python itself used while edge() was staged
        staged = cap.capture_edge(self.edge, params, consumed)
        self._baked_scalars = frozenset(consumed)
        if staged is None:
            raise NotImplementedError(
                f"edge() of {type(self).__name__} leaves the staging vocabulary "
                "(field, +, -, *, /, sum(-1), maximum, exp); no native kernel and no fallback exists")
        constants = {name: value for name, value in cap.selected_params(self.edge, params).items()
                     if not isinstance(value, torch.Tensor)}
        if isinstance(self.reducer, OnlineSoftmaxReducer):
            return self._specialise_online_softmax(graph, src, dst, edge, params, staged, constants)
        kind = _reducer_kind(self.reducer)
        if isinstance(staged, ReducerCall) or kind is None:
            generic = self._specialise_algebra(graph, src, dst, edge, params, staged, constants)
            if generic is None:
                raise NotImplementedError(
                    f"no native kernel for reducer {type(self.reducer).__name__} with this edge expression: "
                    "a user algebra needs associative = True, a state of at most four numbers, one finalized "
                    "value and element-wise edge expressions")
            return generic
        pattern = cap.recognize_weighted_sum(staged)
        if kind in ("sum", "mean", "max", "prod") and isinstance(staged, cap.Expr):
            vector_weight = (pattern is not None and pattern.edge_field is not None and pattern.edge_field in edge
                             and pattern.src_field in src
                             and edge[pattern.edge_field].numel() != edge[pattern.edge_field].shape[0])
            if pattern is None or vector_weight or kind == "prod":
                generic = self._specialise_edge_program(graph, src, dst, edge, params, staged, constants, kind)
                if generic is not None:
                    return generic
        if kind is None or kind == "prod" or pattern is None:
            raise NotImplementedError(
                f"no native kernel for reducer {type(self.reducer).__name__} with this edge expression")
        from . import ops

        implicit = _implicit_edge_names(graph)
        _refuse_shadowing(implicit, edge)
        if pattern.src_field not in src:
            raise KeyError(f"edge() reads src.{pattern.src_field}, which was not bound")
        cell = SimpleNamespace(graph=graph)     # the graph the runner works on; re-pointed on warm rebinds
        implicit_weight = pattern.edge_field is not None and pattern.edge_field in implicit
        if implicit_weight and pattern.edge_field != "distance":
            raise NotImplementedError("only the scalar edge.distance can weight a source field; "
                                      "edge.displacement is a vector per edge")
        identity = float(self.reducer.identity()) if kind in ("sum", "max") else 0.0
        x_probe = src[pattern.src_field]
        if (kind == "sum" and identity == 0.0 and graph._geometry is not None and graph._geometry.fusable()
                and (pattern.edge_field is None or implicit_weight) and x_probe.dtype == torch.float32
                and x_probe.is_cuda and x_probe.numel() <= 128 * max(int(x_probe.shape[0]), 1)):
            # the relation is never written: the walk over the cell directory folds the messages
            from . import geometry

            weight = geometry.PAIR_WEIGHT_DISTANCE if implicit_weight else geometry.PAIR_WEIGHT_ONE

            def fused_runner(x):
                relation = cell.graph._geometry
                return geometry.RadiusWeightedSumFunction.apply(
                    relation.positions, x, relation.directory(), relation.scalar_cutoff(),
                    relation.exclude_self, weight)

            fused_runner.cell = cell
            self._record(
                graph, "b200-generated-radius-distance-sum" if implicit_weight else "b200-generated-radius-sum",
                ("capture-edge-udf", "recognize-weighted-sum", "elide-implicit-edge-geometry",
                 "build-hash-cell-directory"),
                ("radius relation consumed from the cell directory: no edge, distance or displacement "
                 "is materialised; backward folds dy over the same (symmetric) relation and has a "
                 "position-cotangent kernel",),
                extra_key=(tuple(x_probe.shape[1:]), implicit_weight))
            return [("src", pattern.src_field)], [x_probe], constants, fused_runner
        row_ptr, col_idx = graph.resolve_csr()
        _validate_fields("edge", edge, col_idx.numel(), graph.device)
        bindings, tensors = [("src", pattern.src_field)], [x_probe]
        if pattern.edge_field is not None and not implicit_weight:
            if pattern.edge_field not in edge:
                raise KeyError(f"edge() reads edge.{pattern.edge_field}, which was not bound")
            if edge[pattern.edge_field].numel() != col_idx.numel():
                raise NotImplementedError("edge weights must be one scalar per edge ([E] or [E, 1])")
            bindings.append(("edge", pattern.edge_field))
            tensors.append(edge[pattern.edge_field])
        weighted = pattern.edge_field is not None
        implicit_name = pattern.edge_field if implicit_weight else None

        def graph_weight(w):
            """The weight array of this call: the bound edge field, or the relation's own field."""
            if implicit_name is None:
                return w
            current = cell.graph
            return current.implicit_edge_fields(*current.resolve_csr())[implicit_name]

        info = graph.native_plan(transpose=False).info
        planner_remark = (f"rows by degree bucket, {info['long_rows']} split rows in {info['segments']} "
                          f"segments of {info['segment_edges']} edges")
        if kind == "additive":
            algebra = cap.capture_reducer(self.reducer)
            additive = _additive_runner(cell, self.reducer, algebra, weighted)

            def additive_runner(x, w=None):
                return additive(x, graph_weight(w))

            additive_runner.cell = cell
            self._record(
                graph, "b200-csr-additive-tuple-state",
                ("capture-edge-udf", "capture-reducer", "prove-additive-state", "plan-degree-buckets"),
                (planner_remark, f"{algebra.arity} state components, one fused CSR sum per non-constant "
                                 "component; finalize runs on the finished states"),
                extra_key=(tuple(tensors[0].shape[1:]), weighted, algebra.components))
            return bindings, tensors, constants, additive_runner

        def runner(x, w=None):
            return ops.csr_reduce(cell.graph, kind, x, graph_weight(w), identity)

        runner.cell = cell
        self._record(
            graph, f"b200-csr-{'weighted-sum' if kind == 'sum' else kind}-degree-bucket",
            ("capture-edge-udf", "recognize-weighted-sum", "plan-degree-buckets", "plan-split-rows",
             "cache-transposed-relation"),
            (planner_remark,
             "backward: dx gathers over the cached stable transposed relation (no atomics), "
             "dw is a per-edge dot product"),
            extra_key=(tuple(tensors[0].shape[1:]), weighted))
        return bindings, tensors, constants, runner

    def _specialise_edge_program(self, graph, src, dst, edge, params, staged, constants, kind):
        """Any element-wise edge expression: compiled to a register program for the interpreting
        kernels (forward, destination-major and source-major reverse mode)."""
        from . import edge_program as ep

        program = ep.compile_expression(staged)
        if program is None:
            return None
        program = program.literalised(self._baked_scalars)
        implicit = _implicit_edge_names(graph)
        _refuse_shadowing(implicit, edge)
        row_ptr, col_idx = graph.resolve_csr()
        _validate_fields("edge", edge, col_idx.numel(), graph.device)
        spaces = {"src": src, "dst": dst, "edge": edge, "param": params}
        bindings, tensors, slots = [], [], []        # slots: index into the bound tensors, or an implicit name
        for operand in program.operands:
            if operand.role == "edge" and operand.name in implicit:
                slots.append(operand.name)
                continue
            if operand.name not in spaces[operand.role]:
                raise KeyError(f"edge() reads {operand.role}.{operand.name}, which was not bound")
            slots.append(len(tensors))
            bindings.append((operand.role, operand.name))
            tensors.append(spaces[operand.role][operand.name])
        cell = SimpleNamespace(graph=graph)
        reducer_id = {"sum": ep.REDUCE_SUM, "mean": ep.REDUCE_MEAN, "max": ep.REDUCE_MAX, "prod": ep.REDUCE_PROD}[kind]
        identity = float(self.reducer.identity()) if kind in ("sum", "max", "prod") else 0.0

        def runner(*bound, scalars=None):
            current = cell.graph
            provided = None
            operands = []
            for slot in slots:
                if isinstance(slot, str):
                    if provided is None:
                        provided = current.implicit_edge_fields(*current.resolve_csr())
                    operands.append(provided[slot])
                else:
                    operands.append(bound[slot])
            bound_program = program if scalars is None else program.rebound(scalars)
            return ep.EdgeProgramFunction.apply(current, bound_program, reducer_id, identity, *operands)

        runner.cell = cell
        runner.scalars = program.scalar_names()
        probe_shapes = tuple(tuple(t.shape[1:]) if role != "param" else tuple(t.shape)
                             for (role, _), t in zip(bindings, tensors))
        self._record(
            graph, "b200-generic-csr-scalar-reducer",
            ("capture-edge-udf", "compile-edge-register-program", "reverse-mode-edge-program"),
            (f"{len(program.ops)} instructions over {len(program.operands)} operands, evaluated per edge and "
             "feature element; rows folded in edge order; cotangents by a destination-major and a "
             "source-major pass without atomics",),
            extra_key=(program.key(), probe_shapes, kind))
        return bindings, tensors, constants, runner

    def _specialise_algebra(self, graph, src, dst, edge, params, staged, constants, reducer=None,
                            scalars_broadcast=False):
        """A reducer none of the dedicated kernels folds: its staged ``lift / combine / finalize`` run
        as register programs inside the interpreting kernels, forward and reverse mode.
        ``scalars_broadcast``: fields with one number per entity are taken as ``[n, 1, ...]`` against
        fields with more dimensions (a score per edge against a payload vector)."""
        from . import algebra as alg
        from . import edge_program as ep

        reducer = self.reducer if reducer is None else reducer
        messages = staged.messages if isinstance(staged, ReducerCall) else (staged,)
        if not all(isinstance(m, cap.Expr) for m in messages):
            return None
        rules = alg.capture_algebra(reducer, len(messages))
        compiled = ep.compile_expressions(messages)
        if rules is None or compiled is None:
            return None
        program, message_slots = compiled
        program = program.literalised(self._baked_scalars)
        implicit = _implicit_edge_names(graph)
        _refuse_shadowing(implicit, edge)
        row_ptr, col_idx = graph.resolve_csr()
        _validate_fields("edge", edge, col_idx.numel(), graph.device)
        spaces = {"src": src, "dst": dst, "edge": edge, "param": params}
        bindings, tensors, slots = [], [], []
        for operand in program.operands:
            if operand.role == "edge" and operand.name in implicit:
                slots.append(operand.name)
                continue
            if operand.name not in spaces[operand.role]:
                raise KeyError(f"edge() reads {operand.role}.{operand.name}, which was not bound")
            slots.append(len(tensors))
            bindings.append((operand.role, operand.name))
            tensors.append(spaces[operand.role][operand.name])
        cell = SimpleNamespace(graph=graph)

        def runner(*bound, scalars=None):
            current = cell.graph
            provided = None
            operands = []
            for slot in slots:
                if isinstance(slot, str):
                    if provided is None:
                        provided = current.implicit_edge_fields(*current.resolve_csr())
                    operands.append(provided[slot])
                else:
                    operands.append(bound[slot])
            bound_program = program if scalars is None else program.rebound(scalars)
            if scalars_broadcast:
                rank = max(t.ndim - 1 for o, t in zip(program.operands, operands) if o.role != "param")
                operands = [t.reshape(t.shape[0], *((1,) * rank)) if o.role != "param" and t.ndim == 1 and rank else t
                            for o, t in zip(program.operands, operands)]
            return alg.EdgeAlgebraFunction.apply(current, bound_program, message_slots, rules, *operands)

        runner.cell = cell
        runner.scalars = program.scalar_names()
        probe_shapes = tuple(tuple(t.shape[1:]) if role != "param" else tuple(t.shape)
                             for (role, _), t in zip(bindings, tensors))
        self._record(
            graph, "b200-csr-algebra-tile",
            ("capture-edge-udf", "capture-reducer-regions", "compile-edge-register-program",
             "reverse-mode-fold", "reverse-mode-edge-program"),
            (f"{len(messages)} message(s), state of {rules.arity}: step / combine / finalize of "
             f"{len(rules.step.ops)} / {len(rules.combine.ops)} / {len(rules.finalize.ops)} instructions; rows "
             "folded from the identity in edge order (combine(earlier, later)); the fold is differentiated "
             "by a forward sweep that keeps the state before each edge and a backward sweep through step",),
            extra_key=(program.key(), message_slots, rules.key(), probe_shapes))
        return bindings, tensors, constants, runner

    def _specialise_online_softmax(self, graph, src, dst, edge, params, staged, constants):
        from . import attention

        gat = cap.recognize_gat(staged)
        if gat is not None:
            slope = gat.slope
            bindings = [("src", gat.src_field), ("dst", gat.dst_field), ("param", gat.src_param),
                        ("param", gat.dst_param)]
            tensors = [src[gat.src_field], dst[gat.dst_field], params[gat.src_param], params[gat.dst_param]]

            def runner(x_src, x_dst, a_src, a_dst):
                return attention.gat_attention(graph, x_src, x_dst, a_src, a_dst, slope)

            self._record(graph, "b200-csr-edge-attention-online-softmax",
                         ("capture-edge-udf", "recognize-gat-logit", "plan-degree-buckets"),
                         ("row-centric online softmax, float32 state, (m, l) saved for backward",))
            return bindings, tensors, constants, runner
        field = cap.recognize_field_softmax(staged)
        if field is not None and graph.sequence_boundaries() is None:
            row_ptr, col_idx = graph.resolve_csr()
            _validate_fields("edge", edge, col_idx.numel(), graph.device)
            bindings = [("edge", field.score_field), ("src", field.value_field)]
            tensors = [edge[field.score_field], src[field.value_field]]

            def runner(score, value):
                return attention.field_softmax(graph, score, value)

            self._record(graph, "b200-csr-stable-weighted-online-softmax",
                         ("capture-edge-udf", "recognize-field-score-softmax", "plan-degree-buckets",
                          "cache-transposed-relation"),
                         ("per-edge scores, per-source values; float32 (m, l) state saved for backward; "
                          "d_value gathers over the transposed relation (no atomics)",))
            return bindings, tensors, constants, runner
        dense = cap.recognize_dense_attention(staged)
        if dense is not None and graph.sequence_boundaries() is not None:
            scale = dense.scale
            bindings = [("dst", dense.query_field), ("src", dense.key_field), ("src", dense.value_field)]
            tensors = [dst[dense.query_field], src[dense.key_field], src[dense.value_field]]

            def runner(query, key, value):
                return attention.varlen_attention(graph, query, key, value, scale)

            self._record(graph, "b200-dense-streaming-reduction-tcgen05",
                         ("capture-edge-udf", "recognize-dense-attention", "schedule-varlen-tiles"),
                         ("implicit block-lower-triangular relation; no edge is materialised",))
            return bindings, tensors, constants, runner
        # any other score / value expressions with one score per edge: the reducer written as a plain
        # tuple algebra and folded by the interpreting kernels
        if graph.sequence_boundaries() is None and isinstance(staged, OnlineSoftmaxItem):
            messages = (cap.as_expr(staged.score), cap.as_expr(staged.value))
            generic = self._specialise_algebra(graph, src, dst, edge, params,
                                               ReducerCall(reducer=self.reducer, messages=messages), constants,
                                               reducer=_StableSoftmaxAlgebra(), scalars_broadcast=True)
            if generic is not None:
                return generic
        raise NotImplementedError("no native kernel for this online_softmax edge expression")

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
        implicit = graph.implicit_edge_fields(row_ptr, col_idx)
        _refuse_shadowing(implicit, edge)
        edge = {**implicit, **edge}
        src_at_edge = SimpleNamespace(**{name: value[col_idx] for name, value in src.items()})
        dst_at_edge = SimpleNamespace(**{name: value[destination] for name, value in dst.items()})
        message = cap.call_region(self.edge, (src_at_edge, dst_at_edge, SimpleNamespace(**edge)), params)
        if isinstance(message, ReducerCall) and len(message.messages) == 1:
            message = message.messages[0]
        if isinstance(message, ReducerCall) or (
                not isinstance(self.reducer, OnlineSoftmaxReducer) and _reducer_kind(self.reducer) is None):
            # a user algebra: the definition itself, row by row (small graphs only)
            from .algebra import fold_eagerly

            messages = message.messages if isinstance(message, ReducerCall) else (message,)
            edges = col_idx.numel()
            messages = tuple(m if isinstance(m, torch.Tensor) else torch.full((edges,), float(m), device=graph.device)
                             for m in messages)
            aggregate = fold_eagerly(self.reducer, messages, row_ptr, graph.schema.num_dst)
        else:
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
    if kind == "prod":
        import warnings

        start = torch.full(shape, reducer.identity(), dtype=message.dtype, device=message.device)
        with warnings.catch_warnings():         # Torch still tags the differentiable segment product "beta"
            warnings.simplefilter("ignore", UserWarning)
            return start.index_reduce(0, destination, message, "prod")
    if kind == "additive":
        algebra = cap.capture_reducer(reducer)
        states = []
        for coefficient, power in algebra.components:
            term = torch.ones_like(message) if power == 0 else message ** power
            states.append(torch.zeros(shape, dtype=message.dtype, device=message.device)
                          .index_add_(0, destination, term * coefficient))
        return reducer.finalize(states[0] if algebra.scalar else tuple(states))
    raise NotImplementedError(f"no eager evaluator for reducer {type(reducer).__name__}")


def _additive_runner(cell, reducer, algebra, weighted: bool):
    """Additive tuple-state reducer: state component k is sum_e c_k * m_e**p_k with m_e = w_e * x[src_e]
    (or x[src_e]).  Because (w x)**p = w**p * x**p, every component with p >= 1 is one fused CSR sum
    over element-wise powers of the node and edge arrays (never an [E, F] temporary); p = 0 counts
    the row's edges.  ``finalize`` then runs on the finished [num_dst, ...] states with Torch ops,
    and autograd differentiates through both."""
    from . import ops

    def runner(x, w=None):
        graph = cell.graph
        row_ptr = graph.resolve_csr()[0]
        shape = (graph.num_dst,) + (1,) * (x.ndim - 1)
        states = []
        for coefficient, power in algebra.components:
            if power == 0:
                degree = (row_ptr[1:] - row_ptr[:-1]).to(x.dtype).reshape(shape)
                state = degree.expand((graph.num_dst,) + tuple(x.shape[1:]))
            else:
                xs = x if power == 1 else x ** power
                ws = w if (w is None or power == 1) else w ** power
                state = ops.csr_reduce(graph, "sum", xs, ws, 0.0)
            states.append(state if coefficient == 1.0 else state * coefficient)
        return reducer.finalize(states[0] if algebra.scalar else tuple(states))

    return runner


__all__ = ["MessagePassing"]
