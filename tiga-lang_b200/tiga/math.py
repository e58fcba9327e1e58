"""tg.math: the two intrinsics the staging language knows beyond arithmetic.

Follows python/tiga/math/__init__.py:13-21 of the reference: ``maximum`` and
``exp`` work on staged expressions (capture) and on torch tensors (eager
evaluation in ``kernel.reference``).
"""
from __future__ import annotations


def maximum(left, right):
    from .capture import Expr, as_expr

    if isinstance(left, Expr) or isinstance(right, Expr):
        return Expr("maximum", (as_expr(left), as_expr(right)))
    import torch

    if isinstance(left, torch.Tensor) or isinstance(right, torch.Tensor):
        if not isinstance(left, torch.Tensor):
            left = torch.as_tensor(left, dtype=right.dtype, device=right.device)
        if not isinstance(right, torch.Tensor):
            right = torch.as_tensor(right, dtype=left.dtype, device=left.device)
        return torch.maximum(left, right)
    return left if left >= right else right


def exp(value):
    from .capture import Expr

    if isinstance(value, Expr):
        return Expr("exp", (value,))
    import torch

    if isinstance(value, torch.Tensor):
        return torch.exp(value)
    import math as _math

    return _math.exp(value)


__all__ = ["exp", "maximum"]
