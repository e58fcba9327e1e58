"""``tg.control``: loops over tensor-carried state (``repeat``, ``while_loop``, ``Repeat``, ``While``).

The reference captures such loops as compiler control flow over its lazy tensors
(python/tiga/control/__init__.py:56-294 of walkerchi/TIGA-lang: PageRank, diffusion, solver
iterations).  Over Torch tensors the loop runs on the host -- but a fixed-count loop whose body is a
handful of short kernels is bound by launch overhead, so ``repeat`` records ONE iteration of the body
into a CUDA graph and replays it: the state lives in static buffers, every replay reads the state,
runs the body's kernels (the native message-passing kernels included) and writes the new state back.
Replay is used when the states are CUDA tensors, nothing requires a gradient and there are at least
``GRAPH_MIN_ITERATIONS`` iterations; otherwise the body is simply called ``iterations`` times
(autograd then sees an ordinary unrolled loop).  Same argument checks and error texts as the
reference's ``repeat``.
"""
from __future__ import annotations

from collections.abc import Callable, Sequence

import torch

GRAPH_MIN_ITERATIONS = 4


def _as_states(initial, what: str):
    single = isinstance(initial, torch.Tensor)
    states = (initial,) if single else tuple(initial)
    if not states or any(not isinstance(item, torch.Tensor) for item in states):
        raise TypeError(f"{what} initial state must be a Tensor or non-empty Tensor sequence")
    return single, states


def _call_body(body, states, what: str):
    returned = body(*states)
    outputs = (returned,) if isinstance(returned, torch.Tensor) else tuple(returned)
    if len(outputs) != len(states) or any(not isinstance(item, torch.Tensor) for item in outputs):
        raise TypeError(f"{what} body must return one Tensor per loop-carried state")
    for index, (output, item) in enumerate(zip(outputs, states)):
        if output.shape != item.shape or output.dtype != item.dtype or output.device != item.device:
            raise ValueError(f"{what} body result {index} must preserve its state shape, dtype, and device")
    return outputs


def repeat(initial, body: Callable, *, iterations: int, cuda_graph: bool | None = None):
    """Apply ``body`` ``iterations`` times to the carried state(s).

    ``cuda_graph``: None = decide (see the module text), False = never, True = require replay."""
    single, states = _as_states(initial, "repeat")
    if not callable(body):
        raise TypeError("repeat body must be callable")
    if not isinstance(iterations, int) or isinstance(iterations, bool):
        raise TypeError("repeat iterations must be an integer")
    if iterations < 0:
        raise ValueError("repeat iterations must be non-negative")
    differentiable = torch.is_grad_enabled() and any(item.requires_grad for item in states)
    eligible = (all(item.is_cuda for item in states) and not differentiable
                and iterations >= GRAPH_MIN_ITERATIONS and not torch.cuda.is_current_stream_capturing())
    if cuda_graph is True and not eligible:
        raise ValueError("cuda_graph=True needs CUDA states, no gradient and enough iterations")
    if iterations == 0:
        return states[0] if single else states
    if cuda_graph is False or not eligible:
        for _ in range(iterations):
            states = _call_body(body, states, "repeat")
        return states[0] if single else states
    results = _replay(body, states, iterations)
    return results[0] if single else results


def _write_back(static, produced) -> None:
    """static[i] <- produced[i].  A body may hand back its own inputs (a swap, a view): such values
    are staged first, so that no buffer is overwritten before it has been read."""
    storages = {item.untyped_storage().data_ptr() for item in static}
    staged = [value.clone() if value.untyped_storage().data_ptr() in storages else value for value in produced]
    for target, value in zip(static, staged):
        target.copy_(value)


def _replay(body, states, iterations: int):
    """One iteration captured into a CUDA graph, then replayed.  The first iteration runs eagerly
    (it builds launch plans and caches, which may synchronise and must not be captured)."""
    with torch.no_grad():
        current = _call_body(body, states, "repeat")                  # iteration 1, eager
        if iterations == 1:
            return current
        static = tuple(item.clone() for item in current)
        side = torch.cuda.Stream(device=static[0].device)
        side.wait_stream(torch.cuda.current_stream(static[0].device))
        with torch.cuda.stream(side):                                  # iteration 2, eager on the capture stream
            _write_back(static, _call_body(body, static, "repeat"))
        torch.cuda.current_stream(static[0].device).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            _write_back(static, _call_body(body, static, "repeat"))
        for _ in range(iterations - 2):
            graph.replay()
        return tuple(item.clone() for item in static)


def while_loop(initial, condition: Callable, body: Callable, *, max_iterations: int):
    """Repeat ``body`` while ``condition(*states)`` (a boolean scalar tensor) holds, at most
    ``max_iterations`` times.  The condition is read on the host every iteration."""
    single, states = _as_states(initial, "while_loop")
    if not callable(condition) or not callable(body):
        raise TypeError("while_loop condition and body must be callable")
    if not isinstance(max_iterations, int) or isinstance(max_iterations, bool) or max_iterations < 0:
        raise ValueError("max_iterations must be a non-negative integer")
    for _ in range(max_iterations):
        keep = condition(*states)
        if isinstance(keep, torch.Tensor):
            if keep.numel() != 1:
                raise TypeError("while_loop condition must return a scalar")
            keep = bool(keep.item())
        if not keep:
            break
        states = _call_body(body, states, "while_loop")
    return states[0] if single else states


class Repeat:
    """Class form of ``repeat``: subclass, override ``body``, call with ``iterations=``."""

    def body(self, *states):
        raise NotImplementedError

    def __call__(self, initial, *, iterations: int, cuda_graph: bool | None = None):
        return repeat(initial, self.body, iterations=iterations, cuda_graph=cuda_graph)


class While:
    """Class form of ``while_loop``: override ``condition`` and ``body``."""

    def condition(self, *states):
        raise NotImplementedError

    def body(self, *states):
        raise NotImplementedError

    def __call__(self, initial, *, max_iterations: int):
        return while_loop(initial, self.condition, self.body, max_iterations=max_iterations)


__all__ = ["Repeat", "While", "repeat", "while_loop"]
