"""Reducer kernels: sum, mean, prod, online_softmax and user algebras.

Same public surface as python/tiga/reducer/core.py:24-229 of the reference
(``Reducer`` with identity/lift/combine/finalize and the
associative/commutative/deterministic declarations, ``tg.sum(identity=)``,
``tg.mean()``, ``tg.online_softmax(accumulation_dtype=, deterministic=,
block_prune_threshold=)``, staged bindings ``ReducerCall`` /
``OnlineSoftmaxItem``).  ``tg.max()`` is an addition of this package: the
reference has no built-in maximum (docs/reducers.md:270-277) but runs a user
``Reducer`` whose ``combine`` is ``tg.math.maximum``; ``MaxReducer`` is exactly
such a reducer.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .kernel import Kernel


@dataclass(frozen=True)
class ReducerCall:
    reducer: "Reducer"
    messages: tuple[Any, ...]


@dataclass(frozen=True)
class OnlineSoftmaxItem:
    score: Any
    value: Any


class Reducer(Kernel):
    name = "custom"
    associative = False
    commutative = False
    deterministic = False

    def __init__(self, *, deterministic: bool = False) -> None:
        super().__init__()
        self.deterministic = bool(deterministic)

    def identity(self):
        raise NotImplementedError

    def lift(self, *messages):
        return messages[0] if len(messages) == 1 else tuple(messages)

    def combine(self, left, right):
        raise NotImplementedError

    def finalize(self, state):
        return state

    def __call__(self, *messages: Any) -> ReducerCall:
        if not messages:
            raise TypeError("a reducer binding requires at least one message")
        return ReducerCall(self, tuple(messages))

    def specialization_key(self) -> tuple[object, ...]:
        configuration = tuple(sorted(
            (name, repr(value)) for name, value in vars(self).items()
            if not name.startswith("_") and name != "deterministic"))
        return (type(self).__module__, type(self).__qualname__, self.name, self.associative,
                self.commutative, self.deterministic, configuration)


class SumReducer(Reducer):
    name = "sum"
    associative = True
    commutative = True

    def __init__(self, *, identity: float | int = 0, deterministic: bool = False) -> None:
        super().__init__(deterministic=deterministic)
        self.identity_value = identity

    def identity(self):
        return self.identity_value

    def combine(self, left, right):
        return left + right

    def specialization_key(self) -> tuple[object, ...]:
        return self.name, self.identity_value, self.deterministic


class MeanReducer(Reducer):
    """Neighbour mean as tuple state (sum, count); an empty row is 0/0 = NaN."""

    name = "mean"
    associative = True
    commutative = True

    def identity(self):
        return 0.0, 0.0

    def lift(self, message):
        return message, 1.0

    def combine(self, left, right):
        return left[0] + right[0], left[1] + right[1]

    def finalize(self, state):
        return state[0] / state[1]


class ProductReducer(Reducer):
    name = "prod"
    associative = True
    commutative = True

    def identity(self):
        return 1.0

    def combine(self, left, right):
        return left * right


class MaxReducer(Reducer):
    """Element-wise NaN-propagating maximum with a configurable start value."""

    name = "max"
    associative = True
    commutative = True

    def __init__(self, *, identity: float = float("-inf"), deterministic: bool = False) -> None:
        super().__init__(deterministic=deterministic)
        self.identity_value = float(identity)

    def identity(self):
        return self.identity_value

    def combine(self, left, right):
        from . import math as tg_math

        return tg_math.maximum(left, right)


class OnlineSoftmaxReducer(Reducer):
    name = "online_softmax"
    associative = True
    commutative = True

    def __init__(self, *, accumulation_dtype: object | None = None, deterministic: bool = False,
                 block_prune_threshold: float | None = None) -> None:
        super().__init__(deterministic=deterministic)
        if block_prune_threshold is not None and not (0.0 < float(block_prune_threshold) <= 1.0):
            raise ValueError("block_prune_threshold must be in (0, 1]")
        self.accumulation_dtype = accumulation_dtype
        self.block_prune_threshold = None if block_prune_threshold is None else float(block_prune_threshold)

    def __call__(self, score: Any, value: Any) -> OnlineSoftmaxItem:
        return OnlineSoftmaxItem(score=score, value=value)

    def specialization_key(self) -> tuple[object, ...]:
        return self.name, str(self.accumulation_dtype), self.deterministic, self.block_prune_threshold


def sum(*, identity: float | int = 0, deterministic: bool = False) -> SumReducer:
    return SumReducer(identity=identity, deterministic=deterministic)


def mean(*, deterministic: bool = False) -> MeanReducer:
    return MeanReducer(deterministic=deterministic)


def prod(*, deterministic: bool = False) -> ProductReducer:
    return ProductReducer(deterministic=deterministic)


def max(*, identity: float = float("-inf"), deterministic: bool = False) -> MaxReducer:
    return MaxReducer(identity=identity, deterministic=deterministic)


def online_softmax(*, accumulation_dtype: object | None = None, deterministic: bool = False,
                   block_prune_threshold: float | None = None) -> OnlineSoftmaxReducer:
    return OnlineSoftmaxReducer(accumulation_dtype=accumulation_dtype, deterministic=deterministic,
                                block_prune_threshold=block_prune_threshold)


__all__ = ["MaxReducer", "MeanReducer", "OnlineSoftmaxItem", "OnlineSoftmaxReducer", "ProductReducer",
           "Reducer", "ReducerCall", "SumReducer", "max", "mean", "online_softmax", "prod", "sum"]
