"""Reducers: how the messages of one destination row are folded.

A reducer is a small algebra -- ``identity()``, ``lift(message)``,
``combine(left, right)``, ``finalize(state)`` -- plus three declarations
(``associative``, ``commutative``, ``deterministic``) that the planner trusts.
The fold it describes is ``finalize(combine(...combine(identity, lift(m1))...))``.

The vocabulary is the reference's (python/tiga/reducer/core.py:24-229 of
walkerchi/TIGA-lang): ``tg.sum(identity=)``, ``tg.mean()`` (tuple state
``(sum, count)``; an empty row is 0/0 = NaN), ``tg.prod()``,
``tg.online_softmax(accumulation_dtype=, deterministic=,
block_prune_threshold=)``, user subclasses of ``Reducer``, and the two staged
bindings an ``edge()`` may return: ``self.reducer(message, ...)`` ->
``ReducerCall`` and, for the softmax reducer, ``self.reducer(score, value)`` ->
``OnlineSoftmaxItem``.

``tg.max()`` is an addition.  The reference documents that it has no built-in
maximum (docs/reducers.md:270-277) but accepts a user reducer whose
``combine`` is ``tg.math.maximum``; ``MaxReducer`` is such a reducer with the
start value as a constructor argument.

How a reducer reaches a CUDA kernel is decided in ``tiga.capture`` by staging
these methods on symbols, never by looking at the class.
"""
from __future__ import annotations

import dataclasses
from typing import Any

from .kernel import Kernel


@dataclasses.dataclass(frozen=True)
class ReducerCall:
    """``self.reducer(m0, m1, ...)`` inside ``edge()``: the messages bound to a reducer."""

    reducer: "Reducer"
    messages: tuple[Any, ...]


@dataclasses.dataclass(frozen=True)
class OnlineSoftmaxItem:
    """``self.reducer(score, value)`` of the online-softmax reducer."""

    score: Any
    value: Any


def _public_configuration(obj) -> tuple[tuple[str, str], ...]:
    """Constructor-set attributes that distinguish two instances of one reducer class."""
    pairs = []
    for name in sorted(vars(obj)):
        if name.startswith("_") or name == "deterministic":
            continue
        pairs.append((name, repr(getattr(obj, name))))
    return tuple(pairs)


class Reducer(Kernel):
    """Base class of user reducers.  Override ``identity`` and ``combine``; ``lift`` and
    ``finalize`` default to the identity map."""

    name = "custom"
    associative = False
    commutative = False
    deterministic = False

    def __init__(self, *, deterministic: bool = False) -> None:
        super().__init__()
        self.deterministic = bool(deterministic)

    def identity(self):
        raise NotImplementedError(f"{type(self).__name__} must define identity()")

    def lift(self, *messages):
        if len(messages) == 1:
            return messages[0]
        return tuple(messages)

    def combine(self, left, right):
        raise NotImplementedError(f"{type(self).__name__} must define combine(left, right)")

    def finalize(self, state):
        return state

    def __call__(self, *messages: Any) -> ReducerCall:
        if len(messages) == 0:
            raise TypeError("a reducer binding requires at least one message")
        return ReducerCall(reducer=self, messages=tuple(messages))

    def specialization_key(self) -> tuple[object, ...]:
        cls = type(self)
        return (cls.__module__, cls.__qualname__, self.name, self.associative, self.commutative,
                self.deterministic, _public_configuration(self))


class SumReducer(Reducer):
    name = "sum"
    associative = commutative = True

    def __init__(self, *, identity: float | int = 0, deterministic: bool = False) -> None:
        super().__init__(deterministic=deterministic)
        self.identity_value = identity

    def identity(self):
        return self.identity_value

    def combine(self, left, right):
        return left + right

    def specialization_key(self) -> tuple[object, ...]:
        return (self.name, self.identity_value, self.deterministic)


class MeanReducer(Reducer):
    """State ``(sum of messages, number of messages)``; the result is their quotient, so a
    row without edges yields 0/0 = NaN."""

    name = "mean"
    associative = commutative = True

    def identity(self):
        return (0.0, 0.0)

    def lift(self, message):
        return (message, 1.0)

    def combine(self, left, right):
        total = left[0] + right[0]
        count = left[1] + right[1]
        return (total, count)

    def finalize(self, state):
        total, count = state
        return total / count


class ProductReducer(Reducer):
    name = "prod"
    associative = commutative = True

    def identity(self):
        return 1.0

    def combine(self, left, right):
        return left * right


class MaxReducer(Reducer):
    """Element-wise maximum in which a NaN message poisons the element (``arith.maximumf``
    semantics); an empty row yields the start value."""

    name = "max"
    associative = commutative = True

    def __init__(self, *, identity: float = float("-inf"), deterministic: bool = False) -> None:
        super().__init__(deterministic=deterministic)
        self.identity_value = float(identity)

    def identity(self):
        return self.identity_value

    def combine(self, left, right):
        from . import math as tg_math

        return tg_math.maximum(left, right)


class OnlineSoftmaxReducer(Reducer):
    """Softmax-weighted sum of values, folded in one pass with a running maximum.

    ``accumulation_dtype``     state dtype (float32 for half-precision inputs when None)
    ``block_prune_threshold``  in (0, 1]: the approximate block-pruned variant of the reference;
                               accepted and keyed on, no native kernel implements it
    """

    name = "online_softmax"
    associative = commutative = True

    def __init__(self, *, accumulation_dtype: object | None = None, deterministic: bool = False,
                 block_prune_threshold: float | None = None) -> None:
        super().__init__(deterministic=deterministic)
        if block_prune_threshold is not None:
            block_prune_threshold = float(block_prune_threshold)
            if not 0.0 < block_prune_threshold <= 1.0:
                raise ValueError("block_prune_threshold must be in (0, 1]")
        self.accumulation_dtype = accumulation_dtype
        self.block_prune_threshold = block_prune_threshold

    def __call__(self, score: Any, value: Any) -> OnlineSoftmaxItem:
        return OnlineSoftmaxItem(score=score, value=value)

    def specialization_key(self) -> tuple[object, ...]:
        return (self.name, str(self.accumulation_dtype), self.deterministic, self.block_prune_threshold)


# ---- the lower-case factories programs call (tg.sum(), tg.mean(), ...) -------------------------
def sum(*, identity: float | int = 0, deterministic: bool = False) -> SumReducer:  # noqa: A001
    return SumReducer(identity=identity, deterministic=deterministic)


def mean(*, deterministic: bool = False) -> MeanReducer:
    return MeanReducer(deterministic=deterministic)


def prod(*, deterministic: bool = False) -> ProductReducer:
    return ProductReducer(deterministic=deterministic)


def max(*, identity: float = float("-inf"), deterministic: bool = False) -> MaxReducer:  # noqa: A001
    return MaxReducer(identity=identity, deterministic=deterministic)


def online_softmax(*, accumulation_dtype: object | None = None, deterministic: bool = False,
                   block_prune_threshold: float | None = None) -> OnlineSoftmaxReducer:
    return OnlineSoftmaxReducer(accumulation_dtype=accumulation_dtype, deterministic=deterministic,
                                block_prune_threshold=block_prune_threshold)


__all__ = ["MaxReducer", "MeanReducer", "OnlineSoftmaxItem", "OnlineSoftmaxReducer", "ProductReducer",
           "Reducer", "ReducerCall", "SumReducer", "max", "mean", "online_softmax", "prod", "sum"]
