"""Generic edge programs: any staged ``edge()`` expression over scalar-per-element arithmetic, run
by one interpreting CUDA kernel and differentiated by its two reverse-mode companions.

The reference lowers an arbitrary scalar edge expression (``add / sub / mul / div / neg / maximum /
exp`` over ``src`` / ``dst`` / ``edge`` fields, tensor parameters and constants) to its generic CSR
kernels (``gf_csr_additive_tile`` K6 and ``gf_csr_scalar_reduce`` K11,
lib/Target/Triton/Translate.cpp:2630-2783, 3452-3634 of walkerchi/TIGA-lang, reached through
``_execute_generic_csr``, python/tiga/interop/torch/message_passing.py:2579-2815) and keeps the
gradients on Torch autograd.  Here the expression tree is compiled to a small register program
(instruction i: ``value[i] = op(value[a], value[b])``) that the kernels of ``csrc/tgb_edge_program.cu``
evaluate per edge and feature element:

* forward: one thread group per destination row folds the messages in edge order (sum / mean / max);
* backward, destination-major: re-evaluates every edge, runs the reverse sweep and accumulates the
  cotangents of ``dst`` fields (per row), ``edge`` fields (per edge) and tensor parameters (per row,
  then a strip sum) -- no atomics;
* backward, source-major over the plan's transposed relation: the cotangents of ``src`` fields.

Widths: an operand is a full feature row (``F`` elements per entity), a scalar per entity, or a
trailing-dimension broadcast (element ``f % m``); anything else is refused.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _native
from .capture import Expr

MAX_INSTRUCTIONS = 48
MAX_OPERANDS = 8
MAX_CONSTANTS = 16

OP_LOAD, OP_CONST, OP_ADD, OP_SUB, OP_MUL, OP_DIV, OP_MAX, OP_EXP, OP_NEG = range(9)
_BINARY = {"add": OP_ADD, "sub": OP_SUB, "mul": OP_MUL, "div": OP_DIV, "maximum": OP_MAX}
_UNARY = {"exp": OP_EXP, "neg": OP_NEG}
ROLE_SRC, ROLE_DST, ROLE_EDGE, ROLE_PARAM = range(4)
_ROLES = {"src": ROLE_SRC, "dst": ROLE_DST, "edge": ROLE_EDGE}
REDUCE_SUM, REDUCE_MEAN, REDUCE_MAX, REDUCE_PROD = range(4)


class ProgramStruct(ctypes.Structure):
    """``tgb_edge_program`` of include/tiga_b200.h."""

    _fields_ = [("num_instructions", ctypes.c_int32), ("num_operands", ctypes.c_int32),
                ("width", ctypes.c_int32), ("reserved", ctypes.c_int32),
                ("op", ctypes.c_uint8 * MAX_INSTRUCTIONS), ("a", ctypes.c_uint8 * MAX_INSTRUCTIONS),
                ("b", ctypes.c_uint8 * MAX_INSTRUCTIONS),
                ("constants", ctypes.c_float * MAX_CONSTANTS),
                ("operand_role", ctypes.c_int32 * MAX_OPERANDS), ("operand_modulus", ctypes.c_int32 * MAX_OPERANDS)]


@dataclass(frozen=True)
class Operand:
    role: str          # "src" | "dst" | "edge" | "param"
    name: str


@dataclass
class EdgeProgram:
    """Compiled expression: instructions in evaluation order, the distinct operands they load."""

    ops: tuple[int, ...]
    lhs: tuple[int, ...]
    rhs: tuple[int, ...]
    constants: tuple[float, ...]
    operands: tuple[Operand, ...]
    # per constant: the float keyword parameter it is read from at every call, or None for a literal
    constant_names: tuple[str | None, ...] = ()

    def key(self):
        """Identity of the program: a constant read from a parameter counts by name, not by value."""
        names = self.constant_names or (None,) * len(self.constants)
        constants = tuple(("scalar", name) if name is not None else value
                          for name, value in zip(names, self.constants))
        return (self.ops, self.lhs, self.rhs, constants, self.operands)

    def scalar_names(self) -> tuple[str, ...]:
        return tuple(name for name in self.constant_names if name is not None)

    def literalised(self, names) -> "EdgeProgram":
        """The program with the constants of ``names`` frozen at their staged values."""
        if not any(name in names for name in self.constant_names if name is not None):
            return self
        kept = tuple(None if name in names else name for name in self.constant_names)
        return EdgeProgram(self.ops, self.lhs, self.rhs, self.constants, self.operands, kept)

    def rebound(self, params) -> "EdgeProgram":
        """The program with its parameter-fed constants taken from ``params`` (the current call)."""
        if not any(name is not None for name in self.constant_names):
            return self
        constants = tuple(float(params[name]) if name is not None else value
                          for name, value in zip(self.constant_names, self.constants))
        return EdgeProgram(self.ops, self.lhs, self.rhs, constants, self.operands, self.constant_names)


def compile_expression(expr) -> EdgeProgram | None:
    """Register program of a staged expression, or None when it leaves the element-wise vocabulary
    (a ``sum`` over features, a non-numeric constant) or exceeds the kernel's table sizes.
    Structurally equal sub-expressions (``s`` used twice in ``maximum(s, 0.2 * s)``) are evaluated once.
    The message is the value of the last instruction."""
    compiled = compile_expressions((expr,))
    return None if compiled is None else compiled[0]


def compile_expressions(roots) -> tuple[EdgeProgram, tuple[int, ...]] | None:
    """One register program for several staged expressions (the messages ``self.reducer(m0, m1, ...)``
    binds) and, per expression, the instruction that holds its value."""
    from .capture import NamedScalar

    ops, lhs, rhs, constants, operands = [], [], [], [], []
    constant_keys: list = []          # ("scalar", name) for a parameter-fed constant, else the literal's value
    memo: dict[int, int] = {}

    def emit(op, a=0, b=0):
        ops.append(op), lhs.append(a), rhs.append(b)
        return len(ops) - 1

    def visit(node) -> int | None:
        if not isinstance(node, Expr):
            return None
        if id(node) in memo:
            return memo[id(node)]
        if node.op == "field" or node.op == "param":
            operand = Operand(*node.args) if node.op == "field" else Operand("param", node.args[0])
            if operand not in operands:
                operands.append(operand)
            for index in range(len(ops)):            # one load per operand
                if ops[index] == OP_LOAD and lhs[index] == operands.index(operand):
                    memo[id(node)] = index
                    return index
            result = emit(OP_LOAD, operands.index(operand))
        elif node.op == "constant":
            value = node.args[0]
            if isinstance(value, bool) or not isinstance(value, (int, float)):
                return None
            key = ("scalar", value.name) if isinstance(value, NamedScalar) else float(value)
            if key not in constant_keys:
                constant_keys.append(key)
                constants.append(float.__float__(value) if isinstance(value, NamedScalar) else float(value))
            result = emit(OP_CONST, constant_keys.index(key))
        elif node.op in _BINARY:
            a, b = visit(node.args[0]), visit(node.args[1])
            if a is None or b is None:
                return None
            result = emit(_BINARY[node.op], a, b)
        elif node.op in _UNARY:
            a = visit(node.args[0])
            if a is None:
                return None
            result = emit(_UNARY[node.op], a)
        else:
            return None
        memo[id(node)] = result
        return result

    slots = []
    for root in roots:
        slot = visit(root)
        if slot is None:
            return None
        slots.append(slot)
    if len(ops) > MAX_INSTRUCTIONS or len(operands) > MAX_OPERANDS or len(constants) > MAX_CONSTANTS:
        return None
    if not operands:
        return None
    names = tuple(key[1] if isinstance(key, tuple) else None for key in constant_keys)
    return EdgeProgram(tuple(ops), tuple(lhs), tuple(rhs), tuple(constants), tuple(operands), names), tuple(slots)


def _entity_shape(operand: Operand, tensor: torch.Tensor) -> tuple[int, ...]:
    return tuple(tensor.shape) if operand.role == "param" else tuple(tensor.shape[1:])


def bind(program: EdgeProgram, tensors):
    """(feature shape, per-operand modulus) of a call: every field must have the same rank per entity
    and broadcast element-wise; tensor parameters broadcast from the right.  modulus 0 = full row,
    1 = one value per entity, m = element ``f % m``."""
    field_shapes = [_entity_shape(o, t) for o, t in zip(program.operands, tensors) if o.role != "param"]
    if not field_shapes:
        raise NotImplementedError("an edge program needs at least one src / dst / edge field")
    ranks = {len(shape) for shape in field_shapes}
    if len(ranks) != 1:
        raise NotImplementedError(
            "the fields of a generic edge program must have the same number of dimensions per entity "
            f"(got {sorted(field_shapes)}); give per-edge scalars a trailing dimension of 1")
    try:
        feature_shape = tuple(torch.broadcast_shapes(
            *field_shapes, *[_entity_shape(o, t) for o, t in zip(program.operands, tensors) if o.role == "param"]))
    except RuntimeError as error:
        raise NotImplementedError(f"operand shapes do not broadcast: {error}") from None
    if len(feature_shape) != len(field_shapes[0]):
        raise NotImplementedError("a tensor parameter may not add dimensions to the message")
    rank = len(feature_shape)
    moduli = []
    for operand, tensor in zip(program.operands, tensors):
        shape = _entity_shape(operand, tensor)
        padded = (1,) * (rank - len(shape)) + shape
        if padded == feature_shape:
            moduli.append(0)
            continue
        leading_ones = 0
        while leading_ones < rank and padded[leading_ones] == 1:
            leading_ones += 1
        if leading_ones == rank:
            moduli.append(1)
            continue
        if padded[leading_ones:] == feature_shape[leading_ones:]:
            count = 1
            for extent in padded[leading_ones:]:
                count *= extent
            moduli.append(count)
            continue
        raise NotImplementedError(
            f"{operand.role}.{operand.name} of per-entity shape {shape} does not broadcast along trailing "
            f"dimensions of the message shape {feature_shape}")
    return feature_shape, tuple(moduli)


def make_struct(program: EdgeProgram, width: int, moduli) -> ProgramStruct:
    struct = ProgramStruct()
    struct.num_instructions = len(program.ops)
    struct.num_operands = len(program.operands)
    struct.width = int(width)
    for i, (op, a, b) in enumerate(zip(program.ops, program.lhs, program.rhs)):
        struct.op[i], struct.a[i], struct.b[i] = op, a, b
    for i, value in enumerate(program.constants):
        struct.constants[i] = value
    for i, (operand, modulus) in enumerate(zip(program.operands, moduli)):
        struct.operand_role[i] = ROLE_PARAM if operand.role == "param" else _ROLES[operand.role]
        struct.operand_modulus[i] = int(modulus)
    return struct


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _pointers(tensors):
    array = (ctypes.c_void_p * MAX_OPERANDS)()
    for i, tensor in enumerate(tensors):
        array[i] = tensor.data_ptr()
    return array


class EdgeProgramFunction(torch.autograd.Function):
    """out[i, f] = reduce over the edges e of row i of program(src[col[e]], dst[i], edge[e], params)[f]."""

    @staticmethod
    def forward(ctx, graph, program: EdgeProgram, reducer: int, identity: float, *tensors):
        lib = _native.lib()
        feature_shape, moduli = bind(program, tensors)
        width = 1
        for extent in feature_shape:
            width *= extent
        rows = [t.detach().contiguous() for t in tensors]
        for operand, tensor in zip(program.operands, rows):
            if tensor.dtype != torch.float32:
                raise NotImplementedError(
                    f"generic edge programs compute in float32; {operand.role}.{operand.name} is {tensor.dtype}")
        struct = make_struct(program, width, moduli)
        plan = graph.native_plan(transpose=False)
        device = rows[0].device
        out = torch.empty((graph.num_dst, width), dtype=torch.float32, device=device)
        # what the reverse mode of max / prod needs of the row (winning entry; zero count and the
        # product of the non-zero messages), written by the forward kernel when gradients are wanted
        wants_grad = any(ctx.needs_input_grad[4:])
        saved_index = saved_value = None
        if wants_grad and reducer in (REDUCE_MAX, REDUCE_PROD):
            saved_index = torch.empty((graph.num_dst, width), dtype=torch.int32, device=device)
        if wants_grad and reducer == REDUCE_PROD:
            saved_value = torch.empty((graph.num_dst, width), dtype=torch.float32, device=device)
        # kernels generated and compiled for this program when the runtime compiler is there,
        # the interpreting kernels otherwise (same arithmetic, same order of every sum)
        from . import edge_jit

        module = edge_jit.module_for(program, width, moduli, reducer) if edge_jit.enabled() else None
        with torch.cuda.device(device):
            if module is not None:
                _native.check(lib.tgb_edge_program_jit_fwd(
                    plan.handle, module.handle, ctypes.byref(struct), _pointers(rows), int(reducer), float(identity),
                    out.data_ptr(), None if saved_value is None else saved_value.data_ptr(),
                    None if saved_index is None else saved_index.data_ptr(), _stream(device)),
                    "tgb_edge_program_jit_fwd")
            else:
                _native.check(lib.tgb_edge_program_fwd(plan.handle, ctypes.byref(struct), _pointers(rows), int(reducer),
                                                       float(identity), out.data_ptr(),
                                                       None if saved_value is None else saved_value.data_ptr(),
                                                       None if saved_index is None else saved_index.data_ptr(),
                                                       _stream(device)),
                              "tgb_edge_program_fwd")
        ctx.module = module
        ctx.graph, ctx.program, ctx.reducer, ctx.struct = graph, program, reducer, struct
        ctx.moduli, ctx.width = moduli, width
        ctx.count = len(rows)
        ctx.save_for_backward(*rows, *[t for t in (saved_value, saved_index) if t is not None])
        ctx.shapes = [tuple(t.shape) for t in tensors]
        return out.reshape((graph.num_dst,) + feature_shape)

    @staticmethod
    def backward(ctx, dy):
        lib = _native.lib()
        rows, kept = ctx.saved_tensors[:ctx.count], ctx.saved_tensors[ctx.count:]
        saved_value = kept[0].data_ptr() if ctx.reducer == REDUCE_PROD else None
        saved_index = kept[-1].data_ptr() if ctx.reducer in (REDUCE_MAX, REDUCE_PROD) else None
        program, graph, struct = ctx.program, ctx.graph, ctx.struct
        needs = ctx.needs_input_grad[4:]
        device = dy.device
        dy = dy.detach().contiguous().reshape(graph.num_dst, ctx.width)
        grads: list[torch.Tensor | None] = [None] * len(rows)
        wanted = (ctypes.c_void_p * MAX_OPERANDS)()
        param_partials = {}
        any_dst_major = any_src_major = False
        for i, (operand, tensor, need) in enumerate(zip(program.operands, rows, needs)):
            if not need:
                continue
            if operand.role == "param":        # one partial per destination row, summed afterwards
                count = max(int(tensor.numel()), 1)
                param_partials[i] = torch.zeros((graph.num_dst, count), dtype=torch.float32, device=device)
                wanted[i] = param_partials[i].data_ptr()
                any_dst_major = True
            else:
                grads[i] = torch.zeros_like(tensor)
                wanted[i] = grads[i].data_ptr()
                if operand.role == "src":
                    any_src_major = True
                else:
                    any_dst_major = True
        with torch.cuda.device(device):
            module = ctx.module
            if any_dst_major:
                plan = graph.native_plan(transpose=False)
                if module is not None:
                    _native.check(lib.tgb_edge_program_jit_bwd(
                        plan.handle, module.handle, ctypes.byref(struct), _pointers(rows), ctx.reducer, dy.data_ptr(),
                        wanted, saved_value, saved_index, 0, _stream(device)), "tgb_edge_program_jit_bwd")
                else:
                    _native.check(lib.tgb_edge_program_bwd_rows(plan.handle, ctypes.byref(struct), _pointers(rows),
                                                                ctx.reducer, dy.data_ptr(), wanted, saved_value,
                                                                saved_index, _stream(device)),
                                  "tgb_edge_program_bwd_rows")
            if any_src_major:
                plan = graph.native_plan(transpose=True)
                if module is not None:
                    _native.check(lib.tgb_edge_program_jit_bwd(
                        plan.handle, module.handle, ctypes.byref(struct), _pointers(rows), ctx.reducer, dy.data_ptr(),
                        wanted, saved_value, saved_index, 1, _stream(device)), "tgb_edge_program_jit_bwd")
                else:
                    _native.check(lib.tgb_edge_program_bwd_sources(plan.handle, ctypes.byref(struct), _pointers(rows),
                                                                   ctx.reducer, dy.data_ptr(), wanted, saved_value,
                                                                   saved_index, _stream(device)),
                                  "tgb_edge_program_bwd_sources")
            for i, partial in param_partials.items():
                total = torch.empty(partial.shape[1], dtype=torch.float32, device=device)
                _native.check(lib.tgb_column_sum(partial.data_ptr(), partial.shape[0], partial.shape[1],
                                                 total.data_ptr(), _stream(device)), "tgb_column_sum")
                grads[i] = total
        return (None, None, None, None, *[None if g is None else g.reshape(shape)
                                           for g, shape in zip(grads, ctx.shapes)])


__all__ = ["EdgeProgram", "EdgeProgramFunction", "Operand", "compile_expression", "compile_expressions", "bind",
           "make_struct",
           "REDUCE_SUM", "REDUCE_MEAN", "REDUCE_MAX", "REDUCE_PROD"]
