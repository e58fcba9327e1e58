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
from typing import Any, Callable, Mapping


class Expr:
    """A node of a staged expression: an operation name and its operands.

    Nodes compare and hash by identity (two structurally equal trees are different objects;
    ``same`` compares structure).  The arithmetic operators and the three methods a staged body
    may call (``sum``, ``maximum``, ``exp``) build new nodes; plain Python numbers met on the way
    become ``constant`` leaves."""

    __slots__ = ("op", "args")

    def __init__(self, op: str, args: tuple[Any, ...]):
        self.op = op
        self.args = tuple(args)

    def __repr__(self) -> str:
        return f"Expr({self.op!r}, {self.args!r})"

    def __neg__(self):
        return Expr("neg", (self,))

    def sum(self, dim=None, keepdim=False):
        return Expr("sum", (self, dim, keepdim))

    def maximum(self, other):
        return Expr("maximum", (self, as_expr(other)))

    def exp(self):
        return Expr("exp", (self,))


def as_expr(value) -> Expr:
    """Operand of a staged operation: an Expr as it is, anything else as a constant leaf."""
    if isinstance(value, Expr):
        return value
    return Expr("constant", (value,))


def _install_arithmetic() -> None:
    # `a <op> b` and the reflected `b <op> a` (b a plain number) for the four binary operations
    for op, dunder in (("add", "add"), ("sub", "sub"), ("mul", "mul"), ("div", "truediv")):
        def forward(self, other, _op=op):
            return Expr(_op, (self, as_expr(other)))

        def reflected(self, other, _op=op):
            return Expr(_op, (as_expr(other), self))

        setattr(Expr, f"__{dunder}__", forward)
        setattr(Expr, f"__r{dunder}__", reflected)


_install_arithmetic()


def same(left: Any, right: Any) -> bool:
    """Structural equality of two staged expressions (leaves: identical objects, or equal
    non-tensor values of one type)."""
    left_is_expr, right_is_expr = isinstance(left, Expr), isinstance(right, Expr)
    if left_is_expr != right_is_expr:
        return False
    if left_is_expr:
        if left.op != right.op or len(left.args) != len(right.args):
            return False
        return all(same(a, b) for a, b in zip(left.args, right.args))
    if left is right:
        return True
    return type(left) is type(right) and not hasattr(left, "shape") and left == right


class FieldNamespace:
    """``src`` / ``dst`` / ``edge`` as ``edge()`` sees them while it is staged: every attribute
    is a ``field`` leaf naming (role, attribute)."""

    def __init__(self, role: str) -> None:
        object.__setattr__(self, "_role", role)

    def __getattr__(self, name: str) -> Expr:
        if name[:2] == "__":          # copy / pickle / inspect probes are not fields
            raise AttributeError(name)
        return Expr("field", (self._role, name))


def selected_params(method, params: Mapping[str, Any]):
    """The subset of ``params`` a user region takes: all of them if it declares ``**rest``,
    otherwise those it names."""
    declared = inspect.signature(method).parameters
    if any(p.kind is inspect.Parameter.VAR_KEYWORD for p in declared.values()):
        return params
    return {name: params[name] for name in params if name in declared}


def call_region(method, positional, params):
    """Call a user region with only the params it declares (or all with **rest)."""
    return method(*positional, **selected_params(method, params))


class NamedScalar(float):
    """A float keyword parameter as ``edge()`` sees it while it is staged.  It behaves like the
    number; when it meets a staged expression it becomes a ``constant`` leaf that remembers which
    parameter it came from, so a compiled program can take the parameter's value at every call
    instead of baking it in.  Anything Python itself does with the number (arithmetic with other
    numbers, comparisons, truth tests, conversions, hashing) is recorded in ``observed``: the value
    has then shaped the staged program in a way nothing can re-bind."""

    __slots__ = ("name", "observed")

    def __new__(cls, value, name, observed):
        self = super().__new__(cls, value)
        self.name, self.observed = name, observed
        return self


def _install_observation() -> None:
    def watch(dunder):
        plain = getattr(float, dunder)

        def method(self, *args):
            if not any(isinstance(a, Expr) for a in args):
                self.observed.add(self.name)
            return plain(self, *args)

        return method

    for dunder in ("__add__", "__radd__", "__sub__", "__rsub__", "__mul__", "__rmul__", "__truediv__",
                   "__rtruediv__", "__floordiv__", "__rfloordiv__", "__mod__", "__rmod__", "__pow__", "__rpow__",
                   "__neg__", "__pos__", "__abs__", "__lt__", "__le__", "__gt__", "__ge__", "__eq__", "__ne__",
                   "__bool__", "__int__", "__float__", "__round__", "__trunc__", "__floor__", "__ceil__",
                   "__hash__", "__index__" if hasattr(float, "__index__") else "__hash__"):
        setattr(NamedScalar, dunder, watch(dunder))


_install_observation()


def _stage_params(params: Mapping[str, Any], observed: set | None = None):
    staged = {}
    for name, value in params.items():
        is_tensor = type(value).__module__.split(".")[0] == "torch" and hasattr(value, "shape")
        if is_tensor:
            staged[name] = Expr("param", (name,))
        elif observed is not None and type(value) is float:
            staged[name] = NamedScalar(value, name, observed)
        else:
            staged[name] = value
    return staged


def capture_edge(method, params: Mapping[str, Any], observed: set | None = None):
    """Run ``edge`` on symbolic fields; returns an Expr (one message), an OnlineSoftmaxItem, a
    ReducerCall of several Exprs (``self.reducer(m0, m1, ...)``), or None when the body leaves the
    vocabulary.  With ``observed`` (a set), float parameters are staged as ``NamedScalar`` and the
    names whose values Python itself consumed are added to the set."""
    from .reducer import OnlineSoftmaxItem, ReducerCall

    try:
        result = method(FieldNamespace("src"), FieldNamespace("dst"), FieldNamespace("edge"),
                        **_stage_params(selected_params(method, params), observed))
    except Exception:
        return None
    if isinstance(result, (Expr, OnlineSoftmaxItem)):
        return result
    if isinstance(result, ReducerCall) and len(result.messages) == 1 and isinstance(result.messages[0], Expr):
        return result.messages[0]
    if isinstance(result, ReducerCall) and all(
            isinstance(m, Expr) or (isinstance(m, (int, float)) and not isinstance(m, bool)) for m in result.messages):
        return ReducerCall(reducer=result.reducer, messages=tuple(as_expr(m) for m in result.messages))
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


@dataclass(frozen=True)
class FieldSoftmaxPattern:
    """``self.reducer(edge.<score>, src.<value>)``: scores stored per edge, values per source."""

    score_field: str
    value_field: str


def recognize_field_softmax(item) -> FieldSoftmaxPattern | None:
    from .reducer import OnlineSoftmaxItem

    if not isinstance(item, OnlineSoftmaxItem):
        return None
    score, value = _field(item.score, "edge"), _field(item.value, "src")
    if score is None or value is None:
        return None
    return FieldSoftmaxPattern(score_field=score[1], value_field=value[1])


# --------------------------------------------------------------------------- reducers
@dataclass(frozen=True)
class ReducerAlgebra:
    """What staging a reducer's methods proved about it.

    kind        "sum"       combine is ``left + right`` on a scalar state, lift and finalize are
                            the identity map
                "max"       combine is ``tg.math.maximum(left, right)``, lift / finalize identity
                "prod"      combine is ``left * right`` (the product monoid), lift / finalize identity
                "additive"  tuple (or scalar) state whose components add independently and whose
                            lift is, per component, ``coefficient * message ** power`` (power 0 is a
                            count); ``finalize`` is arbitrary and runs on the finished states
    components  (coefficient, power) per state component (additive only)
    arity       number of state components
    scalar      the state is a bare value, not a tuple
    """

    kind: str
    components: tuple[tuple[float, int], ...] = ()
    arity: int = 1
    scalar: bool = True


def _monomial(expr, message) -> tuple[float, int] | None:
    """(c, p) with expr == c * message**p, or None.  Numbers are degree-0 monomials."""
    if isinstance(expr, (int, float)) and not isinstance(expr, bool):
        return float(expr), 0
    if not isinstance(expr, Expr):
        return None
    if expr is message:
        return 1.0, 1
    if expr.op == "constant":
        return _monomial(expr.args[0], message)
    if expr.op == "neg":
        inner = _monomial(expr.args[0], message)
        return None if inner is None else (-inner[0], inner[1])
    if expr.op in ("mul", "div"):
        a, b = (_monomial(arg, message) for arg in expr.args)
        if a is None or b is None:
            return None
        if expr.op == "mul":
            return a[0] * b[0], a[1] + b[1]
        if b[1] != 0 or b[0] == 0.0:      # only division by a non-zero number keeps a monomial
            return None
        return a[0] / b[0], a[1]
    return None


def _as_components(value) -> tuple[tuple[Any, ...], bool]:
    if isinstance(value, (tuple, list)):
        return tuple(value), False
    return (value,), True


def capture_reducer(reducer) -> ReducerAlgebra | None:
    """Stage ``identity / lift / combine / finalize`` of a user reducer on symbols and classify
    the algebra they form; None when nothing native matches.  The reference proves the same
    properties on captured reducer regions before it picks a reduction tile
    (python/tiga/compiler/reducer_capture.py:53-189, python/tiga/message_passing/core.py:84-132)."""
    try:
        start, scalar = _as_components(reducer.identity())
    except Exception:
        return None
    arity = len(start)
    message = Expr("reducer_message", ())
    left = tuple(Expr("reducer_state", (0, k)) for k in range(arity))
    right = tuple(Expr("reducer_state", (1, k)) for k in range(arity))
    try:
        lifted, lifted_scalar = _as_components(reducer.lift(message))
        combined, combined_scalar = _as_components(
            reducer.combine(left[0], right[0]) if scalar else reducer.combine(left, right))
    except Exception:
        return None
    if len(lifted) != arity or len(combined) != arity or lifted_scalar != scalar or combined_scalar != scalar:
        return None

    def pairs_own_operands(expr, k, op):
        if not (isinstance(expr, Expr) and expr.op == op and len(expr.args) == 2):
            return False
        return {id(expr.args[0]), id(expr.args[1])} == {id(left[k]), id(right[k])}

    if scalar and lifted[0] is message:
        try:
            untouched = reducer.finalize(left[0]) is left[0]
        except Exception:
            untouched = False
        if untouched and pairs_own_operands(combined[0], 0, "add"):
            return ReducerAlgebra(kind="sum")
        if untouched and pairs_own_operands(combined[0], 0, "maximum"):
            return ReducerAlgebra(kind="max")
        if untouched and pairs_own_operands(combined[0], 0, "mul"):
            return ReducerAlgebra(kind="prod")
    if not all(pairs_own_operands(combined[k], k, "add") for k in range(arity)):
        return None
    if any(not isinstance(v, (int, float)) or isinstance(v, bool) or float(v) != 0.0 for v in start):
        return None        # an additive state has to start from zero
    components = tuple(_monomial(lifted[k], message) for k in range(arity))
    if any(c is None or c[1] < 0 or c[1] > 8 for c in components):
        return None
    return ReducerAlgebra(kind="additive", components=components, arity=arity, scalar=scalar)


def reducer_algebra(reducer) -> str | None:
    """'sum' / 'max' / 'prod' / 'additive' for a user reducer, or None."""
    algebra = capture_reducer(reducer)
    return None if algebra is None else algebra.kind
