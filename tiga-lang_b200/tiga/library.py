"""A specialised MessagePassing call as a ``torch.library`` dispatcher op.

``register_message_passing(kernel, graph=, src=, dst=, edge=, **params)`` fixes
one call shape -- kernel class, reducer, graph, field names, dtypes and shapes,
static (non-tensor) parameters -- and publishes it as a functional op

    tiga::message_passing_<digest>(Tensor row_ptr, Tensor col_idx,
                                   Tensor input_0, ..., Tensor input_k) -> Tensor

with a fake (meta) kernel and an autograd formula, so the call can sit inside
``torch.compile`` / ``torch.export`` graphs.  Name, argument convention and the
attributes of the returned handle (``qualified_name``, ``operation``,
``topology``, ``bindings``, ``static_params``, ``opcheck``) are those of the
reference's facade (python/tiga/interop/torch/library.py:63-205 of
walkerchi/TIGA-lang).

What differs is underneath.  Forward and backward both run the native CUDA
kernels.  The backward is a second dispatcher op (``..._backward``) that calls
the kernel again under autograd and differentiates it -- a dispatcher op cannot
carry the saved state of the inner ``autograd.Function``, so the forward is
recomputed -- whereas the reference replays its eager evaluator there.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass
from typing import Any, Mapping, Sequence

import torch

NAMESPACE = "tiga"
ROLES = ("src", "dst", "edge")

# Fragments must stay alive for as long as their ops are callable.
_fragments: list[Any] = []
_ops_by_name: dict[str, "RegisteredMessagePassingOp"] = {}


@dataclass(frozen=True)
class RegisteredMessagePassingOp:
    qualified_name: str
    operation: Any
    topology: tuple[Any, Any]
    bindings: tuple[tuple[str, str], ...]
    static_params: Mapping[str, Any]

    def _names(self, role: str) -> list[str]:
        return sorted(field for r, field in self.bindings if r == role)

    def __call__(self, *, src, dst, edge=None):
        given = dict(zip(ROLES, (src, dst, edge if edge is not None else {})))
        for role in ROLES:
            wanted = self._names(role)
            if sorted(given[role]) != wanted:
                raise ValueError(f"{role} fields must be {wanted}, got {sorted(given[role])}")
        flat = [given[role][field] for role, field in self.bindings]
        return self.operation(*self.topology, *flat)

    def opcheck(self, *values: Any) -> dict[str, str]:
        return torch.library.opcheck(self.operation, (*self.topology, *values))


class _Specialisation:
    """Everything fixed at registration time, plus the two op bodies."""

    def __init__(self, kernel, graph, groups: Mapping[str, Mapping[str, torch.Tensor]], params):
        self.kernel = kernel
        self.graph = graph
        self.params = dict(params)
        self.row_ptr, self.col_idx = graph.resolve_csr()
        self.bindings = tuple((role, field) for role in ROLES for field in sorted(groups[role]))
        self.samples = tuple(groups[role][field] for role, field in self.bindings)
        self.differentiable = tuple(i for i, t in enumerate(self.samples) if t.is_floating_point())

    # ---- plumbing between the flat dispatcher signature and the keyword call
    def fields(self, flat: Sequence[torch.Tensor]):
        groups = {role: {} for role in ROLES}
        for (role, field), tensor in zip(self.bindings, flat):
            groups[role][field] = tensor
        return groups

    def graph_for(self, row_ptr, col_idx):
        """The registered graph (with its cached launch plan) when the op is called on its own
        topology tensors, otherwise a fresh graph over the tensors that were passed."""
        if row_ptr.data_ptr() == self.row_ptr.data_ptr() and col_idx.data_ptr() == self.col_idx.data_ptr():
            return self.graph
        from .graph import Graph

        return Graph.from_csr(row_ptr, col_idx, num_src=self.graph.schema.num_src, validate="basic")

    def run(self, row_ptr, col_idx, flat):
        groups = self.fields(flat)
        return self.kernel(graph=self.graph_for(row_ptr, col_idx), src=groups["src"], dst=groups["dst"],
                           edge=groups["edge"], **self.params)

    # ---- op bodies
    def forward(self, row_ptr, col_idx, *flat):
        return self.run(row_ptr, col_idx, flat)

    def backward(self, grad_output, row_ptr, col_idx, *flat):
        leaves = [t.detach() for t in flat]
        targets = [leaves[i].requires_grad_(True) for i in self.differentiable]
        with torch.enable_grad():
            result = self.run(row_ptr, col_idx, leaves)
            grads = torch.autograd.grad(result, targets, grad_output.contiguous(), allow_unused=True)
        return [torch.zeros_like(t) if g is None else g for g, t in zip(grads, targets)]

    # ---- identity of the specialisation
    def digest(self, output: torch.Tensor) -> str:
        parts = (
            type(self.kernel).__module__, type(self.kernel).__qualname__,
            self.kernel.reducer.specialization_key(), self.graph.planning_key(), self.bindings,
            tuple((tuple(t.shape), str(t.dtype)) for t in self.samples),
            tuple(sorted((name, repr(value)) for name, value in self.params.items())),
            tuple(output.shape), str(output.dtype),
        )
        return hashlib.sha256(repr(parts).encode()).hexdigest()[:20]


def _check_name(name: str) -> None:
    if not (name[:1].isalpha() and name.replace("_", "").isalnum()):
        raise ValueError("Torch op name must begin with a letter and be alphanumeric/_")


def register_message_passing(kernel, *, graph, src: Mapping[str, Any], dst: Mapping[str, Any],
                             edge: Mapping[str, Any] | None = None, name: str | None = None,
                             **params: Any) -> RegisteredMessagePassingOp:
    schema = graph.schema
    if schema.realization != "materialized_csr" or schema.lifecycle != "static":
        raise NotImplementedError("torch.library registration requires a static CSR graph")
    groups = {"src": src, "dst": dst, "edge": edge if edge is not None else {}}
    spec = _Specialisation(kernel, graph, groups, params)
    if len(spec.samples) == 0 or not all(isinstance(t, torch.Tensor) for t in spec.samples):
        raise TypeError("registered MessagePassing fields must be torch.Tensor values")
    if any(isinstance(value, torch.Tensor) for value in params.values()):
        raise TypeError("Tensor parameters must be expressed as src/dst/edge fields")

    # One real call pins down the result's shape and dtype for the fake kernel and the digest.
    with torch.no_grad():
        probe = spec.forward(spec.row_ptr, spec.col_idx, *spec.samples)
    if not isinstance(probe, torch.Tensor):
        raise NotImplementedError("the torch.library facade requires one Tensor result")
    out_shape, out_dtype = tuple(probe.shape), probe.dtype

    op_name = name if name else f"message_passing_{spec.digest(probe)}"
    _check_name(op_name)
    qualified = f"{NAMESPACE}::{op_name}"
    known = _ops_by_name.get(qualified)
    if known is not None:
        return known

    fragment = torch.library.Library(NAMESPACE, "FRAGMENT")
    tensor_args = ", ".join(["Tensor row_ptr", "Tensor col_idx"]
                            + [f"Tensor input_{i}" for i in range(len(spec.bindings))])
    grad_name = f"{op_name}_backward"
    fragment.define(f"{op_name}({tensor_args}) -> Tensor")
    fragment.define(f"{grad_name}(Tensor grad_output, {tensor_args}) -> Tensor[]")
    fragment.impl(op_name, spec.forward, "CompositeExplicitAutograd")
    fragment.impl(grad_name, spec.backward, "CompositeExplicitAutograd")

    def fake_forward(row_ptr, col_idx, *flat):
        return flat[0].new_empty(out_shape, dtype=out_dtype)

    def fake_backward(grad_output, row_ptr, col_idx, *flat):
        return [torch.empty_like(flat[i]) for i in spec.differentiable]

    torch.library.register_fake(qualified, fake_forward, lib=fragment)
    torch.library.register_fake(f"{NAMESPACE}::{grad_name}", fake_backward, lib=fragment)
    grad_op = getattr(getattr(torch.ops, NAMESPACE), grad_name).default
    offset = 2  # row_ptr, col_idx precede the fields

    def save_inputs(ctx, inputs, output):
        ctx.save_for_backward(*inputs)

    def autograd_formula(ctx, grad_output):
        inputs = ctx.saved_tensors
        wanted = [i for i in spec.differentiable if ctx.needs_input_grad[offset + i]]
        result: list[Any] = [None] * len(inputs)
        if wanted:
            computed = dict(zip(spec.differentiable, grad_op(grad_output, *inputs)))
            for i in wanted:
                result[offset + i] = computed[i]
        return tuple(result)

    torch.library.register_autograd(qualified, autograd_formula, setup_context=save_inputs, lib=fragment)
    handle = RegisteredMessagePassingOp(
        qualified_name=qualified, operation=getattr(getattr(torch.ops, NAMESPACE), op_name).default,
        topology=(spec.row_ptr, spec.col_idx), bindings=spec.bindings, static_params=dict(params))
    _fragments.append(fragment)
    _ops_by_name[qualified] = handle
    return handle


__all__ = ["RegisteredMessagePassingOp", "register_message_passing"]
