"""User algebras: any associative reducer with a (tuple) state, folded by the interpreting kernels.

The reference stages ``identity / lift / combine / finalize`` of a ``Reducer`` subclass into typed
regions (python/tiga/compiler/reducer_capture.py:53-130 of walkerchi/TIGA-lang) and, when no
dedicated tile matches (zero-additive states, stable weighted means), runs them with its generic
CSR tile ``gf_csr_algebra_tile`` (lib/Target/Triton/Translate.cpp:3065-3092; reached through
``_execute_generic_csr``, python/tiga/interop/torch/message_passing.py:2579-2815), left fold in edge
order.  Here the same four methods are staged on symbols and compiled to three register programs
over arguments:

* ``step(state, messages) = combine(state, lift(messages))``  -- one edge of the fold;
* ``combine(left, right)``                                    -- joins the slices of a long row;
* ``finalize(state)``                                         -- one output.

``csrc/tgb_edge_program.cu`` folds every destination row from the identity, edges in order
(commutativity is not needed: ``combine(earlier, later)``), and differentiates the fold itself: a
forward sweep keeps the state before each edge, a backward sweep through ``step`` hands every edge
the cotangents of its messages, and the edge program's two reverse-mode passes turn those into
the cotangents of the fields -- no atomics, no Torch replay.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _native
from . import edge_program as ep
from .capture import Expr, as_expr

MAX_INSTRUCTIONS = 40
MAX_STATE = 4
MAX_MESSAGES = 4
MAX_CONSTANTS = 8


class RegionStruct(ctypes.Structure):
    """``tgb_region`` of include/tiga_b200.h."""

    _fields_ = [("num_instructions", ctypes.c_int32),
                ("op", ctypes.c_uint8 * MAX_INSTRUCTIONS), ("a", ctypes.c_uint8 * MAX_INSTRUCTIONS),
                ("b", ctypes.c_uint8 * MAX_INSTRUCTIONS), ("out", ctypes.c_uint8 * MAX_STATE),
                ("constants", ctypes.c_float * MAX_CONSTANTS)]


class AlgebraStruct(ctypes.Structure):
    """``tgb_edge_algebra`` of include/tiga_b200.h."""

    _fields_ = [("arity", ctypes.c_int32), ("num_messages", ctypes.c_int32),
                ("identity", ctypes.c_float * MAX_STATE), ("message_slot", ctypes.c_uint8 * MAX_MESSAGES),
                ("step", RegionStruct), ("combine", RegionStruct), ("finalize", RegionStruct)]


@dataclass(frozen=True)
class Region:
    """A register program over numbered arguments; ``outs[k]`` is the instruction holding output k."""

    ops: tuple[int, ...]
    lhs: tuple[int, ...]
    rhs: tuple[int, ...]
    constants: tuple[float, ...]
    outs: tuple[int, ...]

    def fill(self, struct: RegionStruct) -> None:
        struct.num_instructions = len(self.ops)
        for i, (op, a, b) in enumerate(zip(self.ops, self.lhs, self.rhs)):
            struct.op[i], struct.a[i], struct.b[i] = op, a, b
        for i, value in enumerate(self.constants):
            struct.constants[i] = value
        for i, out in enumerate(self.outs):
            struct.out[i] = out


@dataclass(frozen=True)
class Algebra:
    identity: tuple[float, ...]
    num_messages: int
    scalar_state: bool
    step: Region
    combine: Region
    finalize: Region

    @property
    def arity(self) -> int:
        return len(self.identity)

    def key(self):
        return (self.identity, self.num_messages, self.step, self.combine, self.finalize)


def _compile_region(outputs, argument_of) -> Region | None:
    """``outputs``: staged expressions (or numbers) over argument symbols; ``argument_of(node)`` gives
    the argument number of a symbol leaf, or None."""
    ops, lhs, rhs, constants = [], [], [], []
    memo: dict[int, int] = {}

    def emit(op, a=0, b=0):
        ops.append(op), lhs.append(a), rhs.append(b)
        return len(ops) - 1

    def visit(node):
        if not isinstance(node, Expr):
            node = as_expr(node)
        if id(node) in memo:
            return memo[id(node)]
        argument = argument_of(node)
        if argument is not None:
            result = emit(ep.OP_LOAD, argument)
        elif node.op == "constant":
            value = node.args[0]
            if isinstance(value, bool) or not isinstance(value, (int, float)):
                return None
            value = float(value)
            if value not in constants:
                constants.append(value)
            result = emit(ep.OP_CONST, constants.index(value))
        elif node.op in ep._BINARY:
            a, b = visit(node.args[0]), visit(node.args[1])
            if a is None or b is None:
                return None
            result = emit(ep._BINARY[node.op], a, b)
        elif node.op in ep._UNARY:
            a = visit(node.args[0])
            if a is None:
                return None
            result = emit(ep._UNARY[node.op], a)
        else:
            return None
        memo[id(node)] = result
        return result

    outs = []
    for output in outputs:
        slot = visit(output)
        if slot is None:
            return None
        outs.append(slot)
    if len(ops) > MAX_INSTRUCTIONS or len(constants) > MAX_CONSTANTS:
        return None
    return Region(tuple(ops), tuple(lhs), tuple(rhs), tuple(constants), tuple(outs))


def _components(value) -> tuple[tuple, bool]:
    if isinstance(value, (tuple, list)):
        return tuple(value), False
    return (value,), True


def capture_algebra(reducer, num_messages: int) -> Algebra | None:
    """Stage the reducer's four methods on symbols and compile the three regions; None when a
    method leaves the element-wise vocabulary, the state is not a flat tuple of at most four
    numbers, ``finalize`` gives more than one value, or the reducer does not declare itself
    associative (the kernels join slices of long rows with ``combine``)."""
    if not getattr(reducer, "associative", False) or not 1 <= num_messages <= MAX_MESSAGES:
        return None
    try:
        start, scalar = _components(reducer.identity())
    except Exception:
        return None
    arity = len(start)
    if not 1 <= arity <= MAX_STATE:
        return None
    if any(isinstance(v, bool) or not isinstance(v, (int, float)) for v in start):
        return None
    messages = tuple(Expr("reducer_message", (j,)) for j in range(num_messages))
    left = tuple(Expr("reducer_state", (0, k)) for k in range(arity))
    right = tuple(Expr("reducer_state", (1, k)) for k in range(arity))

    def pack(side):
        return side[0] if scalar else side

    try:
        lifted, lifted_scalar = _components(reducer.lift(*messages))
        if len(lifted) != arity or lifted_scalar != scalar:
            return None
        lifted = tuple(as_expr(v) for v in lifted)          # ``lift`` may put plain numbers into the state
        stepped, stepped_scalar = _components(reducer.combine(pack(left), pack(lifted)))
        combined, combined_scalar = _components(reducer.combine(pack(left), pack(right)))
        final, _ = _components(reducer.finalize(pack(left)))
    except Exception:
        return None
    if len(stepped) != arity or len(combined) != arity or stepped_scalar != scalar or combined_scalar != scalar:
        return None
    if len(final) != 1:
        return None

    def step_argument(node):
        if node.op == "reducer_state" and node.args[0] == 0:
            return node.args[1]
        if node.op == "reducer_message":
            return arity + node.args[0]
        return None

    def combine_argument(node):
        if node.op == "reducer_state":
            return node.args[0] * arity + node.args[1]
        return None

    step = _compile_region(stepped, step_argument)
    combine = _compile_region(combined, combine_argument)
    finalize = _compile_region(final, lambda node: node.args[1] if node.op == "reducer_state" and node.args[0] == 0
                               else None)
    if step is None or combine is None or finalize is None:
        return None
    return Algebra(tuple(float(v) for v in start), num_messages, scalar, step, combine, finalize)


def make_struct(algebra: Algebra, slots) -> AlgebraStruct:
    struct = AlgebraStruct()
    struct.arity, struct.num_messages = algebra.arity, algebra.num_messages
    for k, value in enumerate(algebra.identity):
        struct.identity[k] = value
    for j, slot in enumerate(slots):
        struct.message_slot[j] = slot
    algebra.step.fill(struct.step)
    algebra.combine.fill(struct.combine)
    algebra.finalize.fill(struct.finalize)
    return struct


class EdgeAlgebraFunction(torch.autograd.Function):
    """out[i, f] = finalize(fold over the edges e of row i, in order, of step(state, messages(e))[f])."""

    @staticmethod
    def forward(ctx, graph, program: ep.EdgeProgram, slots, algebra: Algebra, *tensors):
        lib = _native.lib()
        feature_shape, moduli = ep.bind(program, tensors)
        width = 1
        for extent in feature_shape:
            width *= extent
        rows = [t.detach().contiguous() for t in tensors]
        for operand, tensor in zip(program.operands, rows):
            if tensor.dtype != torch.float32:
                raise NotImplementedError(
                    f"generic edge programs compute in float32; {operand.role}.{operand.name} is {tensor.dtype}")
        struct = ep.make_struct(program, width, moduli)
        rules = make_struct(algebra, slots)
        plan = graph.native_plan(transpose=False)
        device = rows[0].device
        out = torch.empty((graph.num_dst, width), dtype=torch.float32, device=device)
        # kernels generated for this program and this algebra when the runtime compiler is there
        from . import edge_jit

        module = edge_jit.module_for(program, width, moduli, 0, algebra, slots) if edge_jit.enabled() else None
        with torch.cuda.device(device):
            if module is not None:
                _native.check(lib.tgb_edge_algebra_jit_fwd(plan.handle, module.handle, ctypes.byref(struct),
                                                           ep._pointers(rows), out.data_ptr(), ep._stream(device)),
                              "tgb_edge_algebra_jit_fwd")
            else:
                _native.check(lib.tgb_edge_algebra_fwd(plan.handle, ctypes.byref(struct), ctypes.byref(rules),
                                                       ep._pointers(rows), out.data_ptr(), ep._stream(device)),
                              "tgb_edge_algebra_fwd")
        ctx.module = module
        ctx.graph, ctx.program, ctx.algebra, ctx.struct, ctx.rules = graph, program, algebra, struct, rules
        ctx.width, ctx.edges = width, int(plan.num_edges)
        ctx.save_for_backward(*rows)
        ctx.shapes = [tuple(t.shape) for t in tensors]
        return out.reshape((graph.num_dst,) + feature_shape)

    @staticmethod
    def backward(ctx, dy):
        lib = _native.lib()
        rows = ctx.saved_tensors
        program, graph, algebra, struct, rules = ctx.program, ctx.graph, ctx.algebra, ctx.struct, ctx.rules
        needs = ctx.needs_input_grad[4:]
        device = dy.device
        width = ctx.width
        dy = dy.detach().contiguous().reshape(graph.num_dst, width)
        edges = ctx.edges
        grads: list[torch.Tensor | None] = [None] * len(rows)
        wanted = (ctypes.c_void_p * ep.MAX_OPERANDS)()
        param_partials = {}
        any_dst_major = any_src_major = False
        for i, (operand, tensor, need) in enumerate(zip(program.operands, rows, needs)):
            if not need:
                continue
            if operand.role == "param":
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
        # the state before every edge (kept between the two sweeps over a row) and the cotangent of
        # every message of every edge
        prefix = torch.empty((max(edges, 1), algebra.arity, width), dtype=torch.float32, device=device)
        message_grads = torch.zeros((algebra.num_messages, max(edges, 1), width), dtype=torch.float32, device=device)
        module = ctx.module
        with torch.cuda.device(device):
            plan = graph.native_plan(transpose=False)
            if module is not None:
                _native.check(lib.tgb_edge_algebra_jit_bwd_messages(
                    plan.handle, module.handle, ctypes.byref(struct), ep._pointers(rows), dy.data_ptr(),
                    prefix.data_ptr(), message_grads.data_ptr(), ep._stream(device)), "tgb_edge_algebra_jit_bwd_messages")
            else:
                _native.check(lib.tgb_edge_algebra_bwd_messages(plan.handle, ctypes.byref(struct), ctypes.byref(rules),
                                                                ep._pointers(rows), dy.data_ptr(), prefix.data_ptr(),
                                                                message_grads.data_ptr(), ep._stream(device)),
                              "tgb_edge_algebra_bwd_messages")
            del prefix
            for source_major, wanted_pass in ((0, any_dst_major), (1, any_src_major)):
                if not wanted_pass:
                    continue
                if source_major:
                    plan = graph.native_plan(transpose=True)
                if module is not None:
                    _native.check(lib.tgb_edge_algebra_jit_bwd(
                        plan.handle, module.handle, ctypes.byref(struct), ep._pointers(rows), message_grads.data_ptr(),
                        wanted, source_major, ep._stream(device)), "tgb_edge_algebra_jit_bwd")
                elif source_major:
                    _native.check(lib.tgb_edge_algebra_bwd_sources(
                        plan.handle, ctypes.byref(struct), ctypes.byref(rules), ep._pointers(rows),
                        message_grads.data_ptr(), wanted, ep._stream(device)), "tgb_edge_algebra_bwd_sources")
                else:
                    _native.check(lib.tgb_edge_algebra_bwd_rows(
                        plan.handle, ctypes.byref(struct), ctypes.byref(rules), ep._pointers(rows),
                        message_grads.data_ptr(), wanted, ep._stream(device)), "tgb_edge_algebra_bwd_rows")
            for i, partial in param_partials.items():
                total = torch.empty(partial.shape[1], dtype=torch.float32, device=device)
                _native.check(lib.tgb_column_sum(partial.data_ptr(), partial.shape[0], partial.shape[1],
                                                 total.data_ptr(), ep._stream(device)), "tgb_column_sum")
                grads[i] = total
        return (None, None, None, None, *[None if g is None else g.reshape(shape)
                                           for g, shape in zip(grads, ctx.shapes)])


def fold_eagerly(reducer, messages, row_ptr, num_dst: int):
    """The definition, row by row with Torch operations (a debugging evaluator for small graphs):
    ``finalize(combine(...combine(identity, lift(m_first))..., lift(m_last)))`` per destination."""
    bounds = row_ptr.tolist()
    template = messages[0]
    feature_shape = tuple(template.shape[1:])

    def constant(value):
        if isinstance(value, torch.Tensor):
            return value
        return torch.full(feature_shape, float(value), dtype=template.dtype, device=template.device)

    def normalise(state):
        if isinstance(state, (tuple, list)):
            return tuple(constant(v) for v in state)
        return constant(state)

    rows = []
    for row in range(num_dst):
        state = normalise(reducer.identity())
        for e in range(bounds[row], bounds[row + 1]):
            state = normalise(reducer.combine(state, normalise(reducer.lift(*[m[e] for m in messages]))))
        rows.append(constant(reducer.finalize(state)))
    if not rows:
        return template.new_zeros((0,) + feature_shape)
    return torch.stack(rows)


__all__ = ["Algebra", "EdgeAlgebraFunction", "Region", "capture_algebra", "fold_eagerly", "make_struct"]
