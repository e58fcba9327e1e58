"""``torch.library`` operator facade over the native kernels.

``register_message_passing(kernel, graph=, src=, dst=, edge=, **params)`` turns
one specialised MessagePassing call into a functional dispatcher op
``tiga::message_passing_<digest>(Tensor row_ptr, Tensor col_idx, Tensor
input_0, ...) -> Tensor`` with a registered fake (meta) implementation and an
autograd formula, the same boundary the reference offers
(python/tiga/interop/torch/library.py:63-205 of walkerchi/TIGA-lang: same
function name, same argument convention, same ``RegisteredMessagePassingOp``
attributes).  The difference is underneath: both the implementation and the
backward run the native CUDA kernels (the reference's backward replays its
eager evaluator).  The backward re-enters the kernel under autograd, i.e. it
recomputes the forward, because a dispatcher op cannot carry the inner
Function's saved state.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass
from typing import Any, Mapping

import torch

_LIBRARIES: list[Any] = []
_REGISTERED: dict[str, "RegisteredMessagePassingOp"] = {}


def _ordered_fields(src, dst, edge):
    return tuple((role, name) for role, group in (("src", src), ("dst", dst), ("edge", edge))
                 for name in sorted(group))


@dataclass(frozen=True)
class RegisteredMessagePassingOp:
    qualified_name: str
    operation: Any
    topology: tuple[Any, Any]
    bindings: tuple[tuple[str, str], ...]
    static_params: Mapping[str, Any]

    def __call__(self, *, src, dst, edge=None):
        groups = {"src": src, "dst": dst, "edge": {} if edge is None else edge}
        for role, group in groups.items():
            expected = sorted(name for r, name in self.bindings if r == role)
            if sorted(group) != expected:
                raise ValueError(f"{role} fields must be {expected}, got {sorted(group)}")
        return self.operation(*self.topology, *(groups[role][name] for role, name in self.bindings))

    def opcheck(self, *values: Any) -> dict[str, str]:
        return torch.library.opcheck(self.operation, (*self.topology, *values))


def register_message_passing(kernel, *, graph, src: Mapping[str, Any], dst: Mapping[str, Any],
                             edge: Mapping[str, Any] | None = None, name: str | None = None,
                             **params: Any) -> RegisteredMessagePassingOp:
    from .graph import Graph

    edge = {} if edge is None else edge
    if graph.schema.realization != "materialized_csr" or graph.schema.lifecycle != "static":
        raise NotImplementedError("torch.library registration requires a static CSR graph")
    row_ptr, col_idx = graph.resolve_csr()
    bindings = _ordered_fields(src, dst, edge)
    groups = {"src": src, "dst": dst, "edge": edge}
    values = tuple(groups[role][field] for role, field in bindings)
    if not values or any(not isinstance(value, torch.Tensor) for value in values):
        raise TypeError("registered MessagePassing fields must be torch.Tensor values")
    if any(isinstance(value, torch.Tensor) for value in params.values()):
        raise TypeError("Tensor parameters must be expressed as src/dst/edge fields")
    with torch.no_grad():   # one native call fixes the result shape and dtype
        sample = kernel(graph=graph, src=src, dst=dst, edge=edge, **params)
    if not isinstance(sample, torch.Tensor):
        raise NotImplementedError("the torch.library facade requires one Tensor result")
    output_shape, output_dtype = tuple(sample.shape), sample.dtype
    signature = repr((type(kernel).__module__, type(kernel).__qualname__, kernel.reducer.specialization_key(),
                      graph.planning_key(), bindings,
                      tuple((tuple(v.shape), str(v.dtype)) for v in values),
                      tuple(sorted((k, repr(v)) for k, v in params.items())), output_shape, str(output_dtype)))
    op_name = name or f"message_passing_{hashlib.sha256(signature.encode()).hexdigest()[:20]}"
    if not op_name.replace("_", "").isalnum() or not op_name[0].isalpha():
        raise ValueError("Torch op name must begin with a letter and be alphanumeric/_")
    qualified = f"tiga::{op_name}"
    if qualified in _REGISTERED:
        return _REGISTERED[qualified]

    library = torch.library.Library("tiga", "FRAGMENT")
    arguments = ", ".join(["Tensor row_ptr", "Tensor col_idx",
                           *(f"Tensor input_{i}" for i in range(len(bindings)))])
    library.define(f"{op_name}({arguments}) -> Tensor")

    def unpack(flat):
        fields = {"src": {}, "dst": {}, "edge": {}}
        for (role, field), value in zip(bindings, flat):
            fields[role][field] = value
        return fields

    def runtime_graph(flat):
        # the registered graph (and its cached launch plan) is reused when the op is called with its own topology
        if flat[0].data_ptr() == row_ptr.data_ptr() and flat[1].data_ptr() == col_idx.data_ptr():
            return graph
        return Graph.from_csr(flat[0], flat[1], num_src=graph.schema.num_src, validate="basic")

    def implementation(*flat):
        fields = unpack(flat[2:])
        return kernel(graph=runtime_graph(flat), src=fields["src"], dst=fields["dst"], edge=fields["edge"],
                      **params)

    library.impl(op_name, implementation, "CompositeExplicitAutograd")
    torch.library.register_fake(qualified, lambda *flat: flat[2].new_empty(output_shape, dtype=output_dtype),
                                lib=library)

    # The backward is a dispatcher op of its own (opaque to tracing, with a fake implementation), so
    # compiled / exported graphs can differentiate through the forward op.
    float_positions = tuple(i for i, v in enumerate(values) if v.is_floating_point())
    backward_name = f"{op_name}_backward"
    library.define(f"{backward_name}(Tensor grad_output, {arguments}) -> Tensor[]")

    def backward_implementation(grad_output, *flat):
        replay = [value.detach() for value in flat]
        wanted = []
        for position in float_positions:
            replay[2 + position].requires_grad_(True)
            wanted.append(replay[2 + position])
        fields = unpack(replay[2:])
        with torch.enable_grad():
            output = kernel(graph=runtime_graph(replay), src=fields["src"], dst=fields["dst"],
                            edge=fields["edge"], **params)
            computed = torch.autograd.grad(output, wanted, grad_output.contiguous(), allow_unused=True)
        return [g if g is not None else torch.zeros_like(w) for g, w in zip(computed, wanted)]

    library.impl(backward_name, backward_implementation, "CompositeExplicitAutograd")
    torch.library.register_fake(
        f"tiga::{backward_name}",
        lambda grad_output, *flat: [torch.empty_like(flat[2 + position]) for position in float_positions],
        lib=library)
    backward_operation = getattr(getattr(torch.ops.tiga, backward_name), "default")

    def setup_context(ctx, inputs, output):
        ctx.save_for_backward(*inputs)

    def backward(ctx, grad_output):
        saved = ctx.saved_tensors
        if not any(ctx.needs_input_grad[2 + position] for position in float_positions):
            return (None,) * len(saved)
        computed = backward_operation(grad_output, *saved)
        gradients = [None] * len(saved)
        for position, gradient in zip(float_positions, computed):
            if ctx.needs_input_grad[2 + position]:
                gradients[2 + position] = gradient
        return tuple(gradients)

    torch.library.register_autograd(qualified, backward, setup_context=setup_context, lib=library)
    operation = getattr(getattr(torch.ops.tiga, op_name), "default")
    registered = RegisteredMessagePassingOp(qualified_name=qualified, operation=operation,
                                            topology=(row_ptr, col_idx), bindings=bindings,
                                            static_params=dict(params))
    _LIBRARIES.append(library)
    _REGISTERED[qualified] = registered
    return registered


__all__ = ["RegisteredMessagePassingOp", "register_message_passing"]
