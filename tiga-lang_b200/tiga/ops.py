"""Thin tensor-level wrappers of the C-ABI kernels plus their autograd glue.

Each wrapper passes raw device addresses and Torch's current CUDA stream to
the library (the provider discipline of python/tiga/interop/torch/provider.py:
8-14,170-198 of the reference: run on the caller's current stream, return a
fresh output tensor with its own storage).
"""
from __future__ import annotations

import torch

from . import _native
from .plan import CSRPlan

_REDUCER_IDS = {"sum": _native.REDUCER_SUM, "mean": _native.REDUCER_MEAN, "max": _native.REDUCER_MAX}


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(tensor) -> int:
    return 0 if tensor is None else tensor.data_ptr()


def _as_rows(tensor: torch.Tensor, rows: int) -> torch.Tensor:
    """[rows, F] contiguous float32 view of a field with arbitrary trailing dims."""
    if tensor.dtype != torch.float32:
        raise NotImplementedError(
            f"the CSR reduce kernels take float32 fields, got {tensor.dtype}")
    if tensor.ndim == 2 and tensor.is_contiguous():
        return tensor
    return tensor.contiguous().reshape(rows, -1)


class _OnDevice:
    """`with _OnDevice(device):` makes `device` current for a launch; costs nothing when it already is
    (the usual case: one process per GPU)."""

    __slots__ = ("guard",)

    def __init__(self, device):
        self.guard = None if torch.cuda.current_device() == device.index else torch.cuda.device(device)

    def __enter__(self):
        if self.guard is not None:
            self.guard.__enter__()

    def __exit__(self, *exc):
        if self.guard is not None:
            self.guard.__exit__(*exc)
        return False


def csr_reduce_forward(plan: CSRPlan, reducer: str, x: torch.Tensor, w: torch.Tensor | None,
                       identity: float = 0.0, accumulate_into: torch.Tensor | None = None):
    """out[i] = reduce over row i of w[e]*x[col[e]]; returns (out2d, argmax or None).
    With ``accumulate_into`` (sum only) the row sums are added to that tensor in place."""
    lib = _native.lib()
    rid = _REDUCER_IDS[reducer]
    F = x.shape[1]
    out = accumulate_into if accumulate_into is not None else torch.empty(
        (plan.num_dst, F), dtype=torch.float32, device=x.device)
    flags = _native.REDUCE_ACCUMULATE if accumulate_into is not None else 0
    forget_transposed_weights(plan)
    aux = torch.empty((plan.num_dst, F), dtype=torch.int32, device=x.device) if reducer == "max" else None
    keep, scratch, scratch_bytes = plan.scratch(0, rid, F)
    with _OnDevice(x.device):
        _native.check(lib.tgb_csr_reduce_fwd(plan.handle, rid, _ptr(x), _ptr(w), _ptr(out), _ptr(aux), F,
                                             _native.DTYPE_F32, float(identity), flags, scratch, scratch_bytes,
                                             _stream(x.device)), "tgb_csr_reduce_fwd")
    return out, aux


def forget_transposed_weights(plan: CSRPlan) -> None:
    """Every forward over a plan drops the transposed weights kept from the last backward."""
    plan.__dict__.pop("_transposed_weights", None)


def transposed_weights(plan: CSRPlan, w: torch.Tensor) -> torch.Tensor:
    """The weights in the order of the plan's transposed relation.  They are kept on the plan from
    one backward call to the next while the same weight tensor (same memory, same version counter)
    comes back, and dropped by the next forward over the plan: the layers of a network that share
    one edge-weight array permute it once per backward pass, not once per layer, and nothing
    survives into the next step.  The cache holds a reference to the weight tensor so that its
    memory cannot be handed to another tensor meanwhile."""
    cached = plan.__dict__.get("_transposed_weights")
    if cached is not None:
        held, version, w_t = cached
        if held.data_ptr() == w.data_ptr() and held.numel() == w.numel() and w._version == version \
                and held._version == version:
            return w_t
    w_t = torch.empty(plan.num_edges, dtype=torch.float32, device=w.device)
    with _OnDevice(w.device):
        _native.check(_native.lib().tgb_csr_transposed_weights(plan.handle, w.data_ptr(), w_t.data_ptr(),
                                                               _stream(w.device)), "tgb_csr_transposed_weights")
    plan.__dict__["_transposed_weights"] = (w, w._version, w_t)
    return w_t


def csr_reduce_backward_dx(plan: CSRPlan, reducer: str, dy: torch.Tensor, w: torch.Tensor | None, aux=None):
    lib = _native.lib()
    rid = _REDUCER_IDS[reducer]
    F = dy.shape[1]
    dx = torch.empty((plan.num_src, F), dtype=torch.float32, device=dy.device)
    ready = w is not None and reducer != "max" and plan.num_edges > 0
    if ready:
        aux = transposed_weights(plan, w)
    keep, scratch, scratch_bytes = plan.scratch(2 if ready else 1, rid, F)
    with _OnDevice(dy.device):
        _native.check(lib.tgb_csr_reduce_bwd_dx(plan.handle, rid, _ptr(dy), _ptr(w), _ptr(aux), _ptr(dx), F,
                                                _native.DTYPE_F32, scratch, scratch_bytes,
                                                _stream(dy.device)), "tgb_csr_reduce_bwd_dx")
    return dx


def csr_reduce_backward_dw(plan: CSRPlan, reducer: str, dy: torch.Tensor, x: torch.Tensor, aux=None, out=None):
    """dw per edge; with a plan that has an edge map the results are written to out[edge_map[e]]."""
    lib = _native.lib()
    rid = _REDUCER_IDS[reducer]
    F = dy.shape[1]
    if plan.edge_map is not None and out is None:
        raise ValueError("a plan with an edge map writes dw into the caller's full-length array: pass out=")
    dw = out if out is not None else torch.empty((plan.num_edges,), dtype=torch.float32, device=dy.device)
    keep, scratch, scratch_bytes = plan.scratch(0, rid, F)
    with _OnDevice(dy.device):
        _native.check(lib.tgb_csr_reduce_bwd_dw(plan.handle, rid, _ptr(dy), _ptr(x), _ptr(aux), _ptr(dw), F,
                                                _native.DTYPE_F32, scratch, scratch_bytes,
                                                _stream(dy.device)), "tgb_csr_reduce_bwd_dw")
    return dw


class CSRReduceFunction(torch.autograd.Function):
    """Fused CSR gather+reduce with a native backward.

    Replaces ``_CSRWeightedSumFunction`` of the reference
    (python/tiga/interop/torch/message_passing.py:378-409), whose backward
    replays Torch gather / mul / index_add: here dx is one gather kernel over
    the cached transposed relation and dw one per-edge dot kernel.  Only the
    inputs are saved (plus the winning-edge table for the max reducer)."""

    @staticmethod
    def forward(ctx, x, w, graph, reducer: str, identity: float):
        rows_x = _as_rows(x, graph.num_src)
        w_flat = None
        if w is not None:
            if w.dtype != torch.float32:
                raise NotImplementedError(f"edge weights must be float32, got {w.dtype}")
            w_flat = w.contiguous().reshape(-1)
        needs_grad = x.requires_grad or (w is not None and w.requires_grad)
        plan = graph.native_plan(transpose=bool(needs_grad and x.requires_grad))
        out, aux = csr_reduce_forward(plan, reducer, rows_x, w_flat, identity)
        ctx.graph = graph
        ctx.reducer = reducer
        ctx.x_shape = x.shape
        ctx.w_shape = None if w is None else w.shape
        ctx.save_for_backward(x, w, aux)
        return out.reshape((graph.num_dst,) + tuple(x.shape[1:]))

    @staticmethod
    def backward(ctx, grad_output):
        x, w, aux = ctx.saved_tensors
        graph = ctx.graph
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dy = _as_rows(grad_output, graph.num_dst)
        w_flat = None if w is None else w.contiguous().reshape(-1)
        dx = dw = None
        if need_x:
            plan = graph.native_plan(transpose=True)
            dx = csr_reduce_backward_dx(plan, ctx.reducer, dy, w_flat, aux).reshape(ctx.x_shape)
        if need_w and w is not None:
            plan = graph.native_plan(transpose=False)
            dw = csr_reduce_backward_dw(plan, ctx.reducer, dy, _as_rows(x, graph.num_src), aux)
            dw = dw.reshape(ctx.w_shape)
        return dx, dw, None, None, None


def csr_reduce(graph, reducer: str, x: torch.Tensor, w: torch.Tensor | None, identity: float = 0.0):
    """Differentiable ``reduce_{e in row i} w[e] * x[col[e]]`` on the GPU."""
    if not x.is_cuda:
        raise RuntimeError("csr_reduce runs on CUDA tensors only (no CPU fallback)")
    if not (torch.is_grad_enabled() and (x.requires_grad or (w is not None and w.requires_grad))):
        # nothing to differentiate: launch the forward kernel without building an autograd node
        if w is not None:
            if w.dtype != torch.float32:
                raise NotImplementedError(f"edge weights must be float32, got {w.dtype}")
            w = w if w.ndim == 1 and w.is_contiguous() else w.contiguous().reshape(-1)
        out, _ = csr_reduce_forward(graph.native_plan(transpose=False), reducer, _as_rows(x, graph.num_src), w,
                                    float(identity))
        return out if x.ndim == 2 else out.reshape((graph.num_dst,) + tuple(x.shape[1:]))
    return CSRReduceFunction.apply(x, w, graph, reducer, float(identity))


# --------------------------------------------------------------------------- dense linear
class _ErrorWord:
    """One int32 per device that the tensor-core kernels set when a bounded wait gives up, with a
    pinned host mirror.  After every launch that may set it, the word is mirrored on the
    launching stream (asynchronously, by a one-thread kernel); the next tensor-core call on the device looks at the mirror of
    the copies that have completed by then and raises, so a give-up surfaces without the caller
    asking and without a synchronisation on the good path."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.word = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.mirror = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.copied = None

    def after_launch(self):
        # a one-thread kernel stores the word into the pinned mirror: a copy-engine transfer would
        # queue behind any bulk device-to-host copy another stream has in flight and stall this stream
        stream = torch.cuda.current_stream(self.device)
        with torch.cuda.device(self.device):
            _native.check(_native.lib().tgb_mirror_word(self.word.data_ptr(), self.mirror.data_ptr(),
                                                        stream.cuda_stream), "tgb_mirror_word")
        self.copied = torch.cuda.Event()
        self.copied.record(stream)

    def raise_if_set(self, wait: bool):
        if wait:
            code = int(self.word.item())
        elif self.copied is not None and self.copied.query():
            code = int(self.mirror[0])
        else:
            return
        if code:
            self.word.zero_()
            self.mirror.zero_()
            raise RuntimeError(f"a tensor-core kernel gave up on a bounded wait (code {code}); "
                               "the results of that call are invalid")


_error_words = {}


def _error_word(device) -> _ErrorWord:
    key = torch.device(device).index
    if key is None:
        key = torch.cuda.current_device()
    if key not in _error_words:
        _error_words[key] = _ErrorWord(torch.device("cuda", key))
    return _error_words[key]


def error_flag(device) -> torch.Tensor:
    """The device's error word, for a launch that is about to start: raises first if an earlier
    kernel on this device is known to have given up on a wait."""
    state = _error_word(device)
    state.raise_if_set(wait=False)
    return state.word


def launched(device) -> None:
    """To be called after a launch that was given `error_flag(device)`."""
    _error_word(device).after_launch()


def check_async_errors(device=None) -> None:
    """Synchronises and raises if a tensor-core kernel reported a timed-out wait."""
    for key, state in list(_error_words.items()):
        if device is not None and torch.device(device).index not in (None, key):
            continue
        state.raise_if_set(wait=True)


def linear_supported(a: torch.Tensor, weight: torch.Tensor) -> bool:
    """Shapes every pass (forward, d(a), d(W)) runs on the tensor cores: K and N in {64, 128}.
    K = 32 or 96 works forward-only (the d(a) pass would need an output width of 32 / 96)."""
    if not (a.is_cuda and a.dtype == torch.float32 and weight.dtype == torch.float32 and a.ndim == 2
            and weight.ndim == 2 and weight.shape[1] in (64, 128)):
        return False
    if weight.shape[0] in (64, 128):
        return True
    return weight.shape[0] in (32, 96) and not (a.requires_grad and torch.is_grad_enabled())


def _linear_raw(a: torch.Tensor, b_t: torch.Tensor) -> torch.Tensor:
    """a [M, K] @ b_t[N, K]^T on the tensor cores (3xTF32)."""
    a, b_t = a.contiguous(), b_t.contiguous()
    M, K = a.shape
    N = b_t.shape[0]
    out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    with torch.cuda.device(a.device):
        _native.check(_native.lib().tgb_linear_f32(a.data_ptr(), b_t.data_ptr(), out.data_ptr(), M, K, N,
                                                   error_flag(a.device).data_ptr(), _stream(a.device)),
                      "tgb_linear_f32")
        launched(a.device)
    return out


def _linear_dw_raw(a: torch.Tensor, d_out: torch.Tensor) -> torch.Tensor:
    """a[M, K]^T @ d_out[M, N] on the tensor cores (3xTF32, deterministic split over the rows)."""
    import ctypes

    a, d_out = a.contiguous(), d_out.contiguous()
    M, K = a.shape
    N = d_out.shape[1]
    lib = _native.lib()
    count = ctypes.c_int32()
    with torch.cuda.device(a.device):
        _native.check(lib.tgb_linear_dw_partials(M, ctypes.byref(count)), "tgb_linear_dw_partials")
        partial = torch.empty((count.value, 128, N), dtype=torch.float32, device=a.device)   # 128-row accumulators
        dw = torch.empty((K, N), dtype=torch.float32, device=a.device)
        _native.check(lib.tgb_linear_dw_f32(a.data_ptr(), d_out.data_ptr(), dw.data_ptr(), partial.data_ptr(),
                                            partial.numel() * 4, M, K, N, error_flag(a.device).data_ptr(),
                                            _stream(a.device)), "tgb_linear_dw_f32")
        launched(a.device)
    return dw


class DenseLinearFunction(torch.autograd.Function):
    """out = a @ W with W [K, N]; forward, d(a) = dout @ W^T and d(W) = a^T @ dout all run on tcgen05."""

    @staticmethod
    def forward(ctx, a, weight):
        ctx.save_for_backward(a, weight)
        return _linear_raw(a, weight.t())

    @staticmethod
    def backward(ctx, grad_output):
        a, weight = ctx.saved_tensors
        grad_output = grad_output.contiguous()
        da = dw = None
        if ctx.needs_input_grad[0]:
            # d(a) = dout @ W^T is the same kernel with the roles of K and N swapped: it needs an output
            # width (K) of 64 or 128; narrower inputs are refused by dense_linear up front
            da = _linear_raw(grad_output, weight)
        if ctx.needs_input_grad[1]:
            dw = _linear_dw_raw(a, grad_output)
        return da, dw


def dense_linear(a: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``a @ weight`` for float32 [M, K] x [K, N] with K, N <= 128 on the tensor cores."""
    if not linear_supported(a, weight):
        raise NotImplementedError("dense_linear takes float32 CUDA matrices with K, N in {64, 128} "
                                  "(K in {32, 96} too when the input needs no gradient)")
    return DenseLinearFunction.apply(a, weight)


def linear(a: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``a @ weight``: the tensor-core kernels when the shapes are theirs (float32 CUDA, K and N in
    {64, 128}), Torch's matmul otherwise."""
    if isinstance(a, torch.Tensor) and isinstance(weight, torch.Tensor) and linear_supported(a, weight):
        return DenseLinearFunction.apply(a, weight)
    return torch.matmul(a, weight)


_MATMULS = (torch.matmul, torch.mm, torch.Tensor.matmul, torch.Tensor.mm, torch.Tensor.__matmul__)


class AggregateTensor(torch.Tensor):
    """What ``node(dst, aggregate)`` receives: an ordinary tensor whose ``aggregate @ W`` (the GCN
    layer's linear, written by the user the way the reference's examples write it) runs on the
    tcgen05 linear kernels when the shapes are theirs.  Every other operation behaves as on a plain
    tensor and returns plain tensors."""

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        with torch._C.DisableTorchFunctionSubclass():
            if func in _MATMULS and len(args) == 2 and not kwargs and isinstance(args[0], AggregateTensor) \
                    and isinstance(args[1], torch.Tensor):
                left = args[0].as_subclass(torch.Tensor)
                right = args[1].as_subclass(torch.Tensor)
                if linear_supported(left, right):
                    return DenseLinearFunction.apply(left, right)
            result = func(*args, **kwargs)
        if isinstance(result, AggregateTensor):
            return result.as_subclass(torch.Tensor)
        return result


def as_aggregate(tensor: torch.Tensor) -> torch.Tensor:
    return tensor.as_subclass(AggregateTensor) if tensor.is_cuda and tensor.dtype == torch.float32 else tensor


# --------------------------------------------------------------------------- halo row movers
def rows_gather(rows: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """packed[i] = rows[ids[i]] for float32 rows and int64 ids."""
    packed = torch.empty((ids.numel(), rows.shape[1]), dtype=rows.dtype, device=rows.device)
    with torch.cuda.device(rows.device):
        _native.check(_native.lib().tgb_rows_gather(rows.data_ptr(), ids.data_ptr(), packed.data_ptr(), ids.numel(),
                                                    rows.shape[1], _stream(rows.device)), "tgb_rows_gather")
    return packed


def rows_scatter_add(rows: torch.Tensor, ids: torch.Tensor, packed: torch.Tensor) -> None:
    """rows[ids[i]] += packed[i] in place; the ids must be unique."""
    with torch.cuda.device(rows.device):
        _native.check(_native.lib().tgb_rows_scatter_add(rows.data_ptr(), ids.data_ptr(), packed.data_ptr(),
                                                         ids.numel(), rows.shape[1], _stream(rows.device)),
                      "tgb_rows_scatter_add")
