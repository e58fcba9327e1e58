"""Restricted staging language for ``edge()`` and the pattern recognisers.

The user's ``edge(self, src, dst, edge, **params)`` is run once on symbolic
field namespaces; the result is an expression tree of ``Expr(op, args)`` with
the vocabulary of the reference's capture layer
(python/tiga/compiler/capture.py:16-145 of walkerchi/TIGA-lang: ``field``,
``constant``, ``add/sub/mul/div/neg``, ``sum``, ``maximum``, ``exp``).  Tensor
parameters are staged as ``param`` leaves so that ``a * src.x`` and
``src.x * a`` capture identically.

The recognisers classify the tree into the programs the native CUDA library
implements:

* weighted sum  ``edge.w * src.x`` / plain ``src.x``  (recognize_weighted_sum,
  python/tiga/compiler/capture.py:123-145)
* GAT edge attention ``online_softmax(maximum(s, c*s), src.x)`` with
  ``s = (src.x*a).sum(-1) + (dst.x*b).sum(-1)``
* dense-relation attention ``online_softmax((src.k*dst.q).sum(-1)*scale, src.v)``
  (capture_structured_message_passing,
  python/tiga/compiler/domain_capture.py:384-463)
"""
from __future__ import annotations

import inspect
from dataclasses import dataclass
from typing import Any, Mapping


@dataclass(frozen=True, eq=False)
class Expr:
    op: str
    args: tuple[Any, ...]

    def _binary(self, op: str, other):
        return Expr(op, (self, as_expr(other)))

    def __add__(self, other):
        return self._binary("add", other)

    def __radd__(self, other):
        return as_expr(other)._binary("add", self)

    def __sub__(self, other):
        return self._binary("sub", other)

    def __rsub__(self, other):
        return as_expr(other)._binary("sub", self)

    def __mul__(self, other):
        return self._binary("mul", other)

    def __rmul__(self, other):
        return as_expr(other)._binary("mul", self)

    def __truediv__(self, other):
        return self._binary("div", other)

    def __rtruediv__(self, other):
        return as_expr(other)._binary("div", self)

    def __neg__(self):
        return Expr("neg", (self,))

    def sum(self, dim=None, keepdim=False):
        return Expr("sum", (self, dim, keepdim))

    def maximum(self, other):
        return Expr("maximum", (self, as_expr(other)))

    def exp(self):
        return Expr("exp", (self,))


def as_expr(value) -> Expr:
    return value if isinstance(value, Expr) else Expr("constant", (value,))


def same(left: Any, right: Any) -> bool:
    """Structural equality of two staged expressions."""
    if isinstance(left, Expr) and isinstance(right, Expr):
        return (left.op == right.op and len(left.args) == len(right.args)
                and all(same(a, b) for a, b in zip(left.args, right.args)))
    if isinstance(left, Expr) or isinstance(right, Expr):
        return False
    return left is right or (type(left) is type(right) and not hasattr(left, "shape") and left == right)


class FieldNamespace:
    def __init__(self, role: str) -> None:
        self._role = role

    def __getattr__(self, name: str) -> Expr:
        if name.startswith("__"):
            raise AttributeError(name)
        return Expr("field", (self._role, name))


def selected_params(method, params: Mapping[str, Any]):
    signature = inspect.signature(method)
    accepts_rest = any(item.kind is inspect.Parameter.VAR_KEYWORD for item in signature.parameters.values())
    return params if accepts_rest else {
        name: value for name, value in params.items() if name in signature.parameters}


def call_region(method, positional, params):
    """Call a user region with only the params it declares (or all with **rest)."""
    return method(*positional, **selected_params(method, params))


def _stage_params(params: Mapping[str, Any]):
    staged = {}
    for name, value in params.items():
        is_tensor = type(value).__module__.split(".")[0] == "torch" and hasattr(value, "shape")
        staged[name] = Expr("param", (name,)) if is_tensor else value
    return staged


def capture_edge(method, params: Mapping[str, Any]):
    """Run ``edge`` on symbolic fields; returns an Expr, an OnlineSoftmaxItem or
    a ReducerCall of Exprs, or None when the body leaves the vocabulary."""
    from .reducer import OnlineSoftmaxItem, ReducerCall

    try:
        result = method(FieldNamespace("src"), FieldNamespace("dst"), FieldNamespace("edge"),
                        **_stage_params(selected_params(method, params)))
    except Exception:
        return None
    if isinstance(result, (Expr, OnlineSoftmaxItem)):
        return result
    if isinstance(result, ReducerCall) and len(result.messages) == 1 and isinstance(result.messages[0], Expr):
        return result.messages[0]
    return None


@dataclass(frozen=True)
class WeightedSumPattern:
    src_field: str
    edge_field: str | None  # None: the message is the plain source field


def _field(expr, role=None):
    if isinstance(expr, Expr) and expr.op == "field" and (role is None or expr.args[0] == role):
        return expr.args
    return None


def recognize_weighted_sum(expr) -> WeightedSumPattern | None:
    if not isinstance(expr, Expr):
        return None
    plain = _field(expr, "src")
    if plain:
        return WeightedSumPattern(src_field=plain[1], edge_field=None)
    if expr.op != "mul":
        return None
    roles = {}
    for item in expr.args:
        leaf = _field(item)
        if leaf is None or leaf[0] in roles:
            return None
        roles[leaf[0]] = leaf[1]
    if set(roles) == {"src", "edge"}:
        return WeightedSumPattern(src_field=roles["src"], edge_field=roles["edge"])
    return None


@dataclass(frozen=True)
class GATPattern:
    src_field: str       # gathered feature, also the value
    dst_field: str
    src_param: str       # attention vector applied to the source feature
    dst_param: str
    slope: float


def _is_last_dim_sum(expr):
    if isinstance(expr, Expr) and expr.op == "sum" and expr.args[1] in (-1,) and not expr.args[2]:
        return expr.args[0]
    return None


def _field_times_param(expr, role):
    if not (isinstance(expr, Expr) and expr.op == "mul"):
        return None
    left, right = expr.args
    for a, b in ((left, right), (right, left)):
        leaf = _field(a, role)
        if leaf and isinstance(b, Expr) and b.op == "param":
            return leaf[1], b.args[0]
    return None


def _constant(expr):
    if isinstance(expr, Expr) and expr.op == "constant" and isinstance(expr.args[0], (int, float)):
        return float(expr.args[0])
    return None


def recognize_gat(item) -> GATPattern | None:
    from .reducer import OnlineSoftmaxItem

    if not isinstance(item, OnlineSoftmaxItem):
        return None
    score, value = item.score, item.value
    value_leaf = _field(value, "src")
    if value_leaf is None or not (isinstance(score, Expr) and score.op == "maximum"):
        return None
    left, right = score.args
    pre, slope = None, None
    for a, b in ((left, right), (right, left)):
        if isinstance(b, Expr) and b.op == "mul":
            for c, s in (b.args, b.args[::-1]):
                if _constant(c) is not None and same(s, a):
                    pre, slope = a, _constant(c)
    if pre is None or not (isinstance(pre, Expr) and pre.op == "add") or not 0.0 <= slope <= 1.0:
        return None
    parts = {}
    for term in pre.args:
        inner = _is_last_dim_sum(term)
        if inner is None:
            return None
        for role in ("src", "dst"):
            hit = _field_times_param(inner, role)
            if hit:
                if role in parts:
                    return None
                parts[role] = hit
    if set(parts) != {"src", "dst"} or parts["src"][0] != value_leaf[1]:
        return None
    return GATPattern(src_field=parts["src"][0], dst_field=parts["dst"][0], src_param=parts["src"][1],
                      dst_param=parts["dst"][1], slope=slope)


@dataclass(frozen=True)
class DenseAttentionPattern:
    key_field: str
    query_field: str
    value_field: str
    scale: Any  # float or the name of a float param (already resolved to float)


def recognize_dense_attention(item) -> DenseAttentionPattern | None:
    from .reducer import OnlineSoftmaxItem

    if not isinstance(item, OnlineSoftmaxItem):
        return None
    value_leaf = _field(item.value, "src")
    score = item.score
    if value_leaf is None or not isinstance(score, Expr):
        return None
    scale = 1.0
    if score.op == "mul":
        left, right = score.args
        if _constant(right) is not None:
            score, scale = left, _constant(right)
        elif _constant(left) is not None:
            score, scale = right, _constant(left)
        else:
            return None
    inner = _is_last_dim_sum(score)
    if inner is None or not (isinstance(inner, Expr) and inner.op == "mul"):
        return None
    roles = {}
    for term in inner.args:
        leaf = _field(term)
        if leaf is None or leaf[0] in roles:
            return None
        roles[leaf[0]] = leaf[1]
    if set(roles) != {"src", "dst"}:
        return None
    return DenseAttentionPattern(key_field=roles["src"], query_field=roles["dst"], value_field=value_leaf[1],
                                 scale=scale)


def reducer_algebra(reducer) -> str | None:
    """Classify a user ``Reducer`` by capturing ``combine`` on two symbols:
    'sum' (left+right) or 'max' (tg.math.maximum); None otherwise.  This is the
    structural proof the reference does on captured reducer regions
    (python/tiga/message_passing/core.py:84-132)."""
    left, right = Expr("reducer_arg", (0,)), Expr("reducer_arg", (1,))
    try:
        combined = reducer.combine(left, right)
    except Exception:
        return None
    if not isinstance(combined, Expr) or len(combined.args) != 2:
        return None
    operands = {id(combined.args[0]), id(combined.args[1])}
    if operands != {id(left), id(right)}:
        return None
    try:
        lifted = reducer.lift(left)
        final = reducer.finalize(left)
    except Exception:
        return None
    if lifted is not left or final is not left:
        return None
    return {"add": "sum", "maximum": "max"}.get(combined.op)
