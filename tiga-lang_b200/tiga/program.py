"""``tg.GraphProgram`` / ``@tg.program``: several MessagePassing applications captured as one program.

The reference captures coarse relation operations into a typed acyclic program, fuses
applications over the same relation snapshot horizontally into one multi-result kernel (its
"product tile", lib/Target/Triton/Translate.cpp:1239-1411) and runs the rest as a task DAG
(python/tiga/program/core.py:172-655 of walkerchi/TIGA-lang).  The same surface is kept here --
``GraphProgram.apply(kernel, graph=, src=, dst=, edge=, **params) -> ProgramValue``,
``outputs(...)``, ``run()``, ``explain()``, the ``@tg.program`` capture boundary, lazy
``ProgramValue`` arithmetic, a ``ProgramValue`` as the source field of a later application -- over
Torch tensors and the native kernels:

* applications are recorded, nothing runs until a value is observed (``materialize()``, arithmetic
  with a tensor, ``run()``);
* horizontal fusion: weighted-sum applications over the SAME graph with the SAME edge-weight tensor
  (or none) whose inputs are available at the same depth of the DAG are executed as ONE gather over
  the concatenated feature columns -- the neighbour ids and weights are read once for all of them,
  and the result is split.  Applications that differ in weights, reducer or program run as separate
  launches in dependency order;
* results are ordinary differentiable Torch tensors.
"""
from __future__ import annotations

import contextvars
import functools
from dataclasses import dataclass, field
from typing import Any, Mapping

import torch

from . import capture as cap
from .reducer import SumReducer

_ACTIVE = contextvars.ContextVar("tiga_graph_program", default=None)


def active_program():
    return _ACTIVE.get()


@dataclass(eq=False)
class ProgramValue:
    """Result of one captured application; observing it runs the program."""

    program: "GraphProgram"
    producer: int
    shape: tuple[int, ...]
    dtype: torch.dtype
    version: int = 0

    def materialize(self) -> torch.Tensor:
        return self.program._result(self.producer)

    def _binary(self, other, op):
        left = self.materialize()
        right = other.materialize() if isinstance(other, ProgramValue) else other
        return op(left, right)

    def __add__(self, other):
        return self._binary(other, torch.add)

    def __radd__(self, other):
        return self._binary(other, lambda a, b: torch.add(b, a))

    def __sub__(self, other):
        return self._binary(other, torch.sub)

    def __rsub__(self, other):
        return self._binary(other, lambda a, b: torch.sub(b, a))

    def __mul__(self, other):
        return self._binary(other, torch.mul)

    def __rmul__(self, other):
        return self._binary(other, lambda a, b: torch.mul(b, a))

    def __truediv__(self, other):
        return self._binary(other, torch.div)

    def __rtruediv__(self, other):
        return self._binary(other, lambda a, b: torch.div(b, a))

    def __neg__(self):
        return -self.materialize()

    def __pos__(self):
        return self.materialize()


@dataclass
class _Apply:
    kernel: Any
    graph: Any
    src: dict
    dst: dict
    edge: dict
    params: dict
    depends: tuple[int, ...] = ()
    fusable: tuple | None = None      # (graph id, weight tensor id or None, src field, edge field)
    result: torch.Tensor | None = field(default=None, repr=False)


class GraphProgram:
    def __init__(self) -> None:
        self._applies: list[_Apply] = []
        self._values: list[ProgramValue] = []
        self._outputs: tuple[int, ...] = ()
        self._launch_groups: list[tuple[int, ...]] = []

    # ----------------------------------------------------------------- capture
    def apply(self, kernel, *, graph, src: Mapping[str, Any], dst: Mapping[str, Any],
              edge: Mapping[str, Any] | None = None, **params: Any) -> ProgramValue:
        edge = {} if edge is None else dict(edge)
        src, dst = dict(src), dict(dst)
        depends = []
        for group in (src, dst, edge):
            for name, value in group.items():
                if isinstance(value, ProgramValue):
                    if value.program is not self:
                        raise ValueError("a ProgramValue can only feed applications of its own program")
                    if value.version != self._values[value.producer].version:
                        raise ValueError("stale ProgramValue: it does not match the program's current value")
                    depends.append(value.producer)
        fusable, shape, dtype = None, None, None
        staged = cap.capture_edge(kernel.edge, params)
        pattern = cap.recognize_weighted_sum(staged) if staged is not None else None
        from .message_passing import MessagePassing

        plain_node = type(kernel).node is MessagePassing.node
        if pattern is not None and isinstance(kernel.reducer, SumReducer) and kernel.reducer.identity() == 0 \
                and plain_node and not graph.is_distributed:
            weight = edge.get(pattern.edge_field) if pattern.edge_field else None
            if not isinstance(weight, ProgramValue):
                fusable = (id(graph), None if weight is None else id(weight), pattern.src_field, pattern.edge_field)
        # result shape: rows of the destination side, trailing dims of the gathered source field
        probe = src.get(pattern.src_field) if pattern is not None else None
        if probe is not None:
            shape = (graph.num_dst,) + tuple(probe.shape[1:])
            dtype = probe.dtype
        value = ProgramValue(self, len(self._values), shape or (graph.num_dst,), dtype or torch.float32)
        self._applies.append(_Apply(kernel, graph, src, dst, edge, dict(params), tuple(depends), fusable))
        self._values.append(value)
        self._outputs = (value.producer,)
        return value

    def outputs(self, *values) -> "GraphProgram":
        producers = []
        for value in values:
            if isinstance(value, ProgramValue):
                if value.program is not self:
                    raise ValueError("outputs must belong to this program")
                producers.append(value.producer)
        if not producers:
            raise ValueError("a program needs at least one output")
        self._outputs = tuple(producers)
        return self

    # --------------------------------------------------------------- execution
    def _resolve(self, group: dict) -> dict:
        return {name: (value.materialize() if isinstance(value, ProgramValue) else value)
                for name, value in group.items()}

    def _depth(self, index: int, memo: dict) -> int:
        if index not in memo:
            memo[index] = 1 + max((self._depth(d, memo) for d in self._applies[index].depends), default=-1)
        return memo[index]

    def run(self):
        """Execute every application that has no result yet; returns the output tensors."""
        pending = [i for i, a in enumerate(self._applies) if a.result is None]
        depth: dict[int, int] = {}
        levels: dict[int, list[int]] = {}
        for i in pending:
            levels.setdefault(self._depth(i, depth), []).append(i)
        token = _ACTIVE.set(None)          # kernel calls made while executing launch, they do not record
        try:
            for level in sorted(levels):
                groups: dict[Any, list[int]] = {}
                for i in levels[level]:
                    key = self._applies[i].fusable
                    groups.setdefault(("solo", i) if key is None else key, []).append(i)
                for members in groups.values():
                    self._launch(members)
        finally:
            _ACTIVE.reset(token)
        results = tuple(self._applies[i].result for i in self._outputs)
        return results[0] if len(results) == 1 else results

    def _launch(self, members: list[int]) -> None:
        first = self._applies[members[0]]
        if len(members) == 1 or first.fusable is None:
            for i in members:
                a = self._applies[i]
                a.result = a.kernel(graph=a.graph, src=self._resolve(a.src), dst=self._resolve(a.dst),
                                    edge=self._resolve(a.edge), **a.params)
                self._launch_groups.append((i,))
            return
        # horizontal fusion: one gather over the concatenated feature columns
        _, _, src_field, edge_field = first.fusable
        inputs = [self._resolve(self._applies[i].src)[src_field] for i in members]
        rows = inputs[0].shape[0]
        same_layout = all(t.shape[0] == rows and t.dtype == inputs[0].dtype and t.device == inputs[0].device
                          for t in inputs)
        if not same_layout:
            for i in members:
                self._launch([i])
            return
        flat = [t.reshape(rows, -1) for t in inputs]
        widths = [t.shape[1] for t in flat]
        stacked = torch.cat(flat, dim=1)
        edge = self._resolve(first.edge)
        fused = first.kernel(graph=first.graph, src={src_field: stacked}, dst={},
                             edge={edge_field: edge[edge_field]} if edge_field else {}, **first.params)
        offset = 0
        for i, width, original in zip(members, widths, inputs):
            piece = fused[:, offset:offset + width]
            self._applies[i].result = piece.reshape((fused.shape[0],) + tuple(original.shape[1:]))
            offset += width
        self._launch_groups.append(tuple(members))

    def _result(self, producer: int) -> torch.Tensor:
        if self._applies[producer].result is None:
            self.run()
        return self._applies[producer].result

    # ---------------------------------------------------------------- reporting
    def explain(self) -> str:
        lines = [f"program: {len(self._applies)} applications, {len(self._launch_groups)} launches executed"]
        for group in self._launch_groups:
            kind = "fused gather over concatenated features" if len(group) > 1 else "single launch"
            names = ", ".join(f"%{i}:{type(self._applies[i].kernel).__name__}" for i in group)
            lines.append(f"  [{kind}] {names}")
        return "\n".join(lines)

    @property
    def launches(self) -> tuple[tuple[int, ...], ...]:
        return tuple(self._launch_groups)


def capture_boundary(function):
    """Run `function` with a fresh GraphProgram active: MessagePassing calls made inside register as
    applications and return ProgramValues; the values the function returns become the program's
    outputs.  Nested boundaries reuse the active program."""

    @functools.wraps(function)
    def captured(*args, **kwargs):
        if active_program() is not None:
            return function(*args, **kwargs)
        graph_program = GraphProgram()
        token = _ACTIVE.set(graph_program)
        try:
            result = function(*args, **kwargs)
        finally:
            _ACTIVE.reset(token)
        values = result if isinstance(result, tuple) else (result,)
        produced = [v for v in values if isinstance(v, ProgramValue)]
        if produced:
            graph_program.outputs(*produced)
        return result

    return captured


def program(function):
    """``@tg.program``: the capture boundary as a decorator."""
    return capture_boundary(function)


__all__ = ["GraphProgram", "ProgramValue", "active_program", "capture_boundary", "program"]
