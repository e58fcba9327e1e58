"""Benchmark of the fused CSR message-passing path (forward + backward).

    python bench.py --gpus 1 --steps K --warmup W           # this build, on B200
    python bench.py --impl reference --steps K --warmup W   # the CPU arm

Workload at one GPU: the "GCN layer" configuration -- an R-MAT graph
(a, b, c, d = 0.57, 0.19, 0.19, 0.05) with 2^20 nodes and 32 * 2^20 generated
edges, symmetrised and de-duplicated, CSR by destination; edge weight
1/sqrt(deg_i * deg_j); float32 features [N, 128]; sum reducer followed by a
dense 128x128 float32 linear.  One step = forward plus the backward of
out.sum() with respect to the features, the edge weights and the linear
weights; the cotangent of out.sum() is a resident matrix of ones handed to
autograd, in this arm and in the CPU arm alike.  Metric: directed edges per
second for forward + backward.

The JSON line carries, besides the base fields:
  roofline     achieved algorithmic GB/s of the dominant gather kernel, timed
               with CUDA events inside the timed region, against the measured
               HBM copy bandwidth of MEASURED_PEAKS.json
  e2e          the same step through the public API with host (pinned) inputs
               copied to the device and gradients copied back every step
  cpu_baseline the CPU oracle port (test infrastructure, OpenMP over rows)
               timed on a bounded sample of the same workload
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "tiga-lang_b200"))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "GEdges/s fwd+bwd for fused CSR message passing"
UNIT = "GEdges/s"
FALLBACK_HBM_GBS = 6650.0


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="native", choices=("native", "reference"))
    p.add_argument("--scale", type=int, default=20, help="log2 of the node count")
    p.add_argument("--edge-factor", type=int, default=32)
    p.add_argument("--features", type=int, default=128)
    p.add_argument("--seed", type=int, default=20261125)
    p.add_argument("--labels", default="random", choices=("natural", "random"),
                   help="multi-GPU workload: relabel the vertices at random as Graph500-style generators "
                        "prescribe (default), or keep the generator's ids with the hubs at low ids; the "
                        "single-GPU workload always keeps the generator's ids")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--cpu-sample-seconds", type=float, default=15.0)
    p.add_argument("--workload", default="gcn", choices=("gcn", "gat", "attention"),
                   help="gcn = the headline GCN-layer configuration; gat / attention measure the edge-attention "
                        "and dense-attention configurations (one GPU)")
    p.add_argument("--kernel-table", action="store_true",
                   help="after the timed run, print a per-kernel device-time table of two more steps to stderr")
    return p.parse_args()


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as handle:
            return float(json.load(handle)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def workload_name(args):
    return (f"gcn-layer rmat scale={args.scale} edge_factor={args.edge_factor} symmetrized dedup "
            f"F={args.features} fp32 sum+linear fwd+bwd")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while timing."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.lines = []
        self.process = None

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.process = None

    def _pump(self):
        for line in self.process.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.process.terminate()
        clocks, reasons, max_clock = [], set(), None
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                max_clock = float(parts[2])
            except ValueError:
                continue
            for name, value in zip(names, parts[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": max_clock,
                "samples": len(clocks), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- GPU arm
def build_inputs(args, device):
    from baseline import synthetic as syn

    row_ptr, col = syn.rmat_csr(args.scale, args.edge_factor, seed=args.seed, symmetrize=True, device=device)
    n = row_ptr.numel() - 1
    weight = syn.gcn_norm_weights(row_ptr, col)
    x = syn.normal((n, args.features), seed=args.seed + 1, device=device)
    lin = syn.normal((args.features, args.features), seed=args.seed + 2, device=device, std=args.features ** -0.5)
    return row_ptr, col, weight, x, lin


def algorithmic_bytes(E, N, F):
    """No-reuse algorithmic traffic per launch: 8-byte indices as given by the
    API, 4-byte weights, one F*4-byte row per edge, pointer + one row per node."""
    row = 4 * F
    return {
        "fwd": E * (8 + 4 + row) + N * (8 + row),
        "dx": E * (8 + 8 + 4 + row) + N * (8 + row),
        "dw": E * (8 + row + 4) + N * (8 + row),
    }


def bf16_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as handle:
            return float(json.load(handle)["bf16_tflops"]), "measured"
    except Exception:
        return 1590.0, "fallback"


def time_steps(step, steps, warmup):
    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()
    begin.record()
    for _ in range(steps):
        step()
    end.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    return begin.elapsed_time(end) / steps


def run_gat(args, device):
    """Edge-attention configuration: directed R-MAT (2^21 nodes, 64M generated edges, de-duplicated),
    bf16 features [N, 8, 32], GAT logit, online-softmax reducer, forward + backward."""
    import tiga as tg
    from tiga import _native, ops
    from baseline import synthetic as syn

    scale = args.scale + 1 if args.scale == 20 else args.scale
    row_ptr, col = syn.rmat_csr(scale, args.edge_factor, seed=args.seed, symmetrize=False, device=device)
    N, E, H, D = row_ptr.numel() - 1, col.numel(), 8, 32
    x = syn.normal((N, H, D), seed=args.seed + 1, device=device, dtype=torch.bfloat16).requires_grad_()
    a_src = syn.normal((H, D), seed=args.seed + 2, device=device, dtype=torch.bfloat16, std=0.1).requires_grad_()
    a_dst = syn.normal((H, D), seed=args.seed + 3, device=device, dtype=torch.bfloat16, std=0.1).requires_grad_()
    graph = tg.Graph.from_csr(row_ptr, col, num_src=N)

    class GAT(tg.MessagePassing):
        reducer = tg.online_softmax()

        def edge(self, src, dst, edge, a_src, a_dst):
            s = (src.x * a_src).sum(dim=-1) + (dst.x * a_dst).sum(dim=-1)
            return self.reducer(tg.math.maximum(s, 0.2 * s), src.x)

    layer = GAT()
    dy = syn.normal((N, H, D), seed=args.seed + 4, device=device, dtype=torch.bfloat16)
    fwd_ms = time_steps(lambda: layer(graph=graph, ndata={"x": x.detach()}, a_src=a_src.detach(),
                                      a_dst=a_dst.detach()), args.steps, args.warmup)

    def step():
        out = layer(graph=graph, ndata={"x": x}, a_src=a_src, a_dst=a_dst)
        return torch.autograd.grad(out, (x, a_src, a_dst), dy)

    before = _native.launch_count()
    ms = time_steps(step, args.steps, args.warmup)
    launches = (_native.launch_count() - before) // (args.steps + max(args.warmup, 3))
    peak, kind = hbm_peak()
    alg = 1696 * E + 3152 * N
    alg_fwd = 520 * E + 1032 * N
    print(json.dumps({
        "metric": METRIC, "value": round(E / (ms * 1e-3) / 1e9, 4), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"gat edge attention rmat scale={scale} directed dedup bf16 [N,8,32] fwd+bwd",
                   "num_nodes": N, "num_edges": E, "forward_ms": round(fwd_ms, 4), "l2": "inputs exceed L2"},
        "roofline": {"bound": "hbm", "kernel": "k_gat_fwd + k_gat_bwd_dst + k_gat_bwd_src (whole step)",
                     "achieved": round(alg / (ms * 1e-3) / 1e9, 1), "peak": peak, "peak_kind": f"of {kind}",
                     "unit": "GB/s", "frac": round(alg / (ms * 1e-3) / 1e9 / peak, 4), "traffic": None,
                     "forward_frac": round(alg_fwd / (fwd_ms * 1e-3) / 1e9 / peak, 4)},
        "gpu_launches": int(launches)}), flush=True)


def run_attention(args, device):
    """Dense-relation configuration: 32 sequences with lengths uniform in [512, 8192], 16 heads,
    head width 128, bf16, causal inside each sequence, forward + backward."""
    import tiga as tg
    from tiga import _native, ops
    from baseline import synthetic as syn

    gen = torch.Generator().manual_seed(20260821)
    lengths = torch.randint(512, 8193, (32,), generator=gen)
    cu = torch.cat((torch.zeros(1, dtype=torch.int64), lengths.cumsum(0)))
    T, H, D = int(cu[-1]), 16, 128
    q, k, v = (syn.normal((T, H, D), seed=args.seed + i, device=device, dtype=torch.bfloat16).requires_grad_()
               for i in range(3))
    dy = syn.normal((T, H, D), seed=args.seed + 9, device=device, dtype=torch.bfloat16)
    graph = tg.Graph.cu_seqlens(cu.to(device), causal=True)

    class Attention(tg.MessagePassing):
        reducer = tg.online_softmax()

        def edge(self, src, dst, edge, scale):
            return self.reducer((src.key * dst.query).sum(dim=-1) * scale, src.value)

    layer = Attention()
    scale = D ** -0.5
    fwd_ms = time_steps(lambda: layer(graph=graph, src={"key": k.detach(), "value": v.detach()},
                                      dst={"query": q.detach()}, scale=scale), args.steps, args.warmup)

    def step():
        out = layer(graph=graph, src={"key": k, "value": v}, dst={"query": q}, scale=scale)
        return torch.autograd.grad(out, (q, k, v), dy)

    ms = time_steps(step, args.steps, args.warmup)
    ops.check_async_errors()
    if args.kernel_table:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step()
            torch.cuda.synchronize()
        print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=12, max_name_column_width=70), flush=True)
    pairs = float((lengths.double() * (lengths.double() + 1) / 2).sum())
    fwd_flops = 4.0 * H * D * pairs
    total_flops = 3.5 * fwd_flops
    peak, kind = bf16_peak()
    print(json.dumps({
        "metric": "TFLOP/s fwd+bwd for varlen causal dense-relation attention", "value": round(total_flops / (ms * 1e-3) / 1e12, 2),
        "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "varlen causal attention 32 sequences L~U[512,8192] H=16 D=128 bf16 fwd+bwd",
                   "tokens": T, "forward_ms": round(fwd_ms, 4),
                   "forward_tflops": round(fwd_flops / (fwd_ms * 1e-3) / 1e12, 2)},
        "roofline": {"bound": "tensor", "kernel": "k_attn_fwd + k_attn_bwd_dkv + k_attn_bwd_dq",
                     "achieved": round(total_flops / (ms * 1e-3) / 1e12, 2), "peak": peak, "peak_kind": f"of {kind}",
                     "unit": "TFLOP/s", "frac": round(total_flops / (ms * 1e-3) / 1e12 / peak, 4), "traffic": None,
                     "forward_frac": round(fwd_flops / (fwd_ms * 1e-3) / 1e12 / peak, 4)}}), flush=True)


def clock_record_rejects(clocks):
    """Why a timed region has to be measured again, or None: a slowdown reason
    that invalidates the number, or a clock record without a single sample (the
    sampler could not run beside the steps, so the host was not keeping up)."""
    bad = [r for r in clocks.get("reasons", []) if r in ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown")]
    if bad:
        return ",".join(bad)
    if not clocks.get("samples"):
        return "no clock sample during the timed region"
    return None


def measured_dram_traffic(args, kernel):
    """DRAM bytes (read + write) of one launch of `kernel` ("fwd", "dx" or
    "dw"), taken from a one-pass ncu capture of dram__bytes_read.sum and
    dram__bytes_write.sum on this exact workload (the table is in
    profiles/csr_reduce_gcn_layer_ncu.md).  The
    figure is a recorded measurement, not something this run can observe, so it
    is reported only for the workload it was captured on."""
    if getattr(args, "workload", "gcn") == "gcn" and args.scale == 20 and args.features == 128 \
            and args.edge_factor == 32:
        return {"fwd": 7.69e9, "dx": 12.36e9, "dw": 7.02e9}[kernel]
    return None


def run_native(args):
    import torch.distributed as dist

    import tiga as tg
    from tiga import _native, ops

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        try:
            return run_native_multi(args, rank, world, device)
        finally:
            dist.destroy_process_group()

    _native.lib()
    torch.backends.cuda.matmul.allow_tf32 = False
    if args.workload == "gat":
        return run_gat(args, device)
    if args.workload == "attention":
        return run_attention(args, device)
    row_ptr, col, weight, x, lin = build_inputs(args, device)
    N, E, F = row_ptr.numel() - 1, col.numel(), args.features
    graph = tg.Graph.from_csr(row_ptr, col, num_src=N)

    class GCNLayer(tg.MessagePassing):
        reducer = tg.sum()

        def edge(self, src, dst, edge):
            return edge.weight * src.x

    layer = GCNLayer()
    x.requires_grad_()
    weight.requires_grad_()
    lin.requires_grad_()

    # per-kernel CUDA-event timing inside the step (events on the launching stream)
    timings = {"fwd": [], "dx": [], "dw": []}
    recording = {"on": False}

    instrument(ops, timings, recording)

    ones = torch.ones((N, lin.shape[1]), dtype=torch.float32, device=device)   # d(out.sum()) / d(out)

    def step(xs, ws, ls):
        agg = layer(graph=graph, src={"x": xs}, dst={}, edge={"weight": ws})
        out = ops.dense_linear(agg, ls)
        return torch.autograd.grad(out, (xs, ws, ls), ones)

    plan_start = time.perf_counter()
    graph.native_plan(transpose=True)
    torch.cuda.synchronize()
    plan_ms = (time.perf_counter() - plan_start) * 1e3

    for _ in range(max(args.warmup, 3)):
        step(x, weight, lin)
    torch.cuda.synchronize()
    def timed_region():
        for v in timings.values():
            v.clear()
        sampler = ClockSampler(local)
        sampler.start()
        # nvidia-smi needs a moment to come up: keep the GPU under the same load, untimed, until its
        # first sample is in (at most 1.5 s), so that the record covers clocks under load
        waited = time.perf_counter()
        while sampler.process is not None and not sampler.lines and time.perf_counter() - waited < 1.5:
            step(x, weight, lin)
            torch.cuda.synchronize()
        launches_before = _native.launch_count()
        recording["on"] = True
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()   # lets a profiler started with --profile-from-start off see only the timed steps
        begin.record()
        for _ in range(args.steps):
            step(x, weight, lin)
        end.record()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        recording["on"] = False
        return (begin.elapsed_time(end) / args.steps, _native.launch_count() - launches_before, sampler.stop())

    ms_per_step, launches, clocks = timed_region()
    rejected = clock_record_rejects(clocks)
    if rejected:        # thermal / hardware slowdown, or no clock sample at all: measure once more
        ms_per_step, launches, clocks = timed_region()
        clocks["remeasured_after"] = rejected
    ops.check_async_errors()
    value = E / (ms_per_step * 1e-3) / 1e9

    bytes_per = algorithmic_bytes(E, N, F)
    kernel_ms = {k: sum(a.elapsed_time(b) for a, b in v) / max(len(v), 1) for k, v in timings.items()}
    dominant = max(kernel_ms, key=kernel_ms.get)
    peak, peak_kind = hbm_peak()
    achieved = bytes_per[dominant] / (kernel_ms[dominant] * 1e-3) / 1e9
    total_alg = sum(bytes_per.values())
    total_kernel_ms = sum(kernel_ms.values())
    roofline = {
        "bound": "hbm", "kernel": {"fwd": "k_gather_vec (forward)", "dx": "k_gather_vec (transposed, dx)",
                                   "dw": "k_edge_dot_vec (dw)"}[dominant],
        "achieved": round(achieved, 1), "peak": peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s",
        "frac": round(achieved / peak, 4), "traffic": measured_dram_traffic(args, dominant),
        "algorithmic_bytes_per_launch": bytes_per[dominant],
        "kernel_ms": {k: round(v, 4) for k, v in kernel_ms.items()},
        "kernel_gbs": {k: round(bytes_per[k] / (kernel_ms[k] * 1e-3) / 1e9, 1) for k in kernel_ms},
        "fwd_bwd_frac": round(total_alg / (total_kernel_ms * 1e-3) / 1e9 / peak, 4),
    }

    result = {
        "metric": METRIC, "value": round(value, 4), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args), "num_nodes": N, "num_edges": E, "features": F,
                   "index_dtype": "int64", "max_degree": int(graph.native_plan(transpose=True).info["max_degree"]),
                   "l2": "inputs exceed L2 (features and indices are each > 126 MB)", "plan_ms": round(plan_ms, 2)},
        "roofline": roofline, "gpu_launches": int(launches), "clocks": clocks,
    }

    if args.kernel_table:
        kernel_table(lambda: step(x, weight, lin), 0)
    if not args.no_e2e:
        result["e2e"] = run_e2e(args, step, x, weight, lin, E)
    if not args.no_cpu_baseline:
        result["cpu_baseline"] = cpu_baseline(args, row_ptr.cpu(), col.cpu(), weight.detach().cpu(),
                                              x.detach().cpu(), lin.detach().cpu(), steps=1, warmup=0)
    print(json.dumps(result), flush=True)


def kernel_table(run, rank, steps=2):
    """Device time per kernel over a few steps (torch profiler), for analysis only."""
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        for _ in range(steps):
            run()
        torch.cuda.synchronize()
    table = prof.key_averages().table(sort_by="cuda_time_total", row_limit=28, max_name_column_width=70)
    print(f"---- rank {rank}: device time over {steps} steps\n{table}", file=sys.stderr, flush=True)


def instrument(ops, timings, recording):
    """Wraps the three kernel entry points with CUDA events on the launching stream."""
    def timed(name, function):
        def wrapper(*a, **k):
            if not recording["on"]:
                return function(*a, **k)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            result = function(*a, **k)
            stop.record()
            timings[name].append((start, stop))
            return result
        return wrapper

    ops.csr_reduce_forward = timed("fwd", ops.csr_reduce_forward)
    ops.csr_reduce_backward_dx = timed("dx", ops.csr_reduce_backward_dx)
    ops.csr_reduce_backward_dw = timed("dw", ops.csr_reduce_backward_dw)


def run_native_multi(args, rank, world, device):
    """N > 1: the same GCN layer on a graph that grows with N (weak scaling:
    2^scale * N nodes), partitioned into N contiguous destination ranges with
    balanced cost (edges + 32 per row); features of ghost rows are exchanged with NCCL
    send/recv every step (forward) and their cotangents sent back (backward);
    the linear weights are replicated and their gradient all-reduced."""
    import math

    import torch.distributed as dist

    import tiga as tg
    from tiga import _native, ops
    from baseline import synthetic as syn
    from tiga.distributed.runtime import DistributedRuntime, NCCLTransport, shard_plan_for

    _native.lib()
    torch.backends.cuda.matmul.allow_tf32 = False
    scale = args.scale + int(round(math.log2(world)))
    F = args.features
    row_ptr, col = syn.rmat_csr(scale, args.edge_factor, seed=args.seed, symmetrize=True, device=device,
                                relabel=args.labels == "random")
    N, E = row_ptr.numel() - 1, col.numel()
    graph = tg.Graph.from_csr(row_ptr, col, num_src=N).halo(
        tg.DeviceMesh("cuda", world), partition=tg.ByDestination(balance="cost"))
    runtime = DistributedRuntime(NCCLTransport(device=device), trace=True)

    class GCNLayer(tg.MessagePassing):
        reducer = tg.sum()

        def edge(self, src, dst, edge):
            return edge.weight * src.x

    layer = GCNLayer()
    with runtime:
        shard = shard_plan_for(graph, runtime)
    b, e = shard.begin, shard.end
    lo, hi = int(row_ptr[b].item()), int(row_ptr[e].item())
    weight = syn.gcn_norm_weights(row_ptr, col)[lo:hi].clone().requires_grad_()
    x = syn.normal((N, F), seed=args.seed + 1, device=device)[b:e].clone().requires_grad_()
    lin = syn.normal((F, F), seed=args.seed + 2, device=device, std=F ** -0.5).requires_grad_()
    del row_ptr, col
    graph._row_ptr = graph._col_idx = None      # the shard plan holds the local relations
    torch.cuda.empty_cache()
    for g in (shard.graph_own, shard.graph_ghost):
        g.native_plan(transpose=True)

    timings = {"fwd": [], "dx": [], "dw": []}
    recording = {"on": False}
    instrument(ops, timings, recording)

    ones = torch.ones((e - b, lin.shape[1]), dtype=torch.float32, device=device)   # d(out.sum()) / d(out)

    def step(xs, ws, ls):
        with runtime:
            agg = layer(graph=graph, src={"x": xs}, dst={}, edge={"weight": ws})
        out = ops.dense_linear(agg, ls)
        dx, dw, dl = torch.autograd.grad(out, (xs, ws, ls), ones)
        dist.all_reduce(dl)
        return dx, dw, dl

    for _ in range(max(args.warmup, 3)):
        step(x, weight, lin)
    torch.cuda.synchronize()
    runtime.reset_trace()
    dist.barrier()
    sampler = ClockSampler(device.index)
    sampler.start()
    launches_before = _native.launch_count()
    recording["on"] = True
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    begin.record()
    for _ in range(args.steps):
        step(x, weight, lin)
    end.record()
    torch.cuda.synchronize()
    dist.barrier()
    recording["on"] = False
    launches = _native.launch_count() - launches_before
    clocks = sampler.stop()
    phases = runtime.phase_times()
    runtime.trace = False
    phase_names = sorted(phases)
    mine = torch.tensor([phases[k] / args.steps for k in phase_names] + [begin.elapsed_time(end) / args.steps],
                        device=device, dtype=torch.float64)
    all_phases = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(all_phases, mine)
    elapsed = torch.tensor([begin.elapsed_time(end)], device=device, dtype=torch.float64)
    dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    ms_per_step = float(elapsed.item()) / args.steps
    value = E / (ms_per_step * 1e-3) / 1e9

    if args.kernel_table:
        kernel_table(lambda: step(x, weight, lin), rank)
    stats = torch.tensor([hi - lo, e - b, int(shard.ghosts.numel()), int(shard.edges_ghost.numel())],
                         device=device, dtype=torch.int64)
    gathered = [torch.empty_like(stats) for _ in range(world)]
    dist.all_gather(gathered, stats)
    e2e = None if args.no_e2e else run_e2e(args, step, x, weight, lin, E, reduce_max=True)

    if rank == 0:
        kernel_ms = {k: sum(a.elapsed_time(b_) for a, b_ in v) / max(args.steps, 1) for k, v in timings.items()}
        peak, peak_kind = hbm_peak()
        local_edges = hi - lo
        bytes_per = algorithmic_bytes(local_edges, e - b, F)
        dominant = max(kernel_ms, key=kernel_ms.get)
        achieved = bytes_per[dominant] / (kernel_ms[dominant] * 1e-3) / 1e9
        per_rank = torch.stack(gathered).tolist()
        result = {
            "metric": METRIC, "value": round(value, 4), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"halo gcn-layer rmat scale={scale} (2^{args.scale} nodes per GPU) "
                                   f"edge_factor={args.edge_factor} symmetrized dedup F={F} fp32 sum+linear fwd+bwd",
                       "num_nodes": N, "num_edges": E, "features": F, "vertex_labels": args.labels,
                       "partition": "contiguous ranges balancing edges + 32 per row",
                       "per_rank_edges_rows_ghosts_ghostedges": per_rank,
                       "halo_bytes_per_step_rank0": int(shard.ghosts.numel()) * F * 4 * 2,
                       "phase_ms_per_rank": {name: [round(float(r[i]), 3) for r in all_phases]
                                             for i, name in enumerate(phase_names + ["step (own clock)"])},
                       "l2": "inputs exceed L2"},
            "roofline": {"bound": "hbm", "kernel": f"rank 0 {dominant} (owned + ghost parts)",
                         "achieved": round(achieved, 1), "peak": peak, "peak_kind": f"of {peak_kind}",
                         "unit": "GB/s", "frac": round(achieved / peak, 4), "traffic": None,
                         "kernel_ms": {k: round(v, 4) for k, v in kernel_ms.items()}},
            "gpu_launches": int(launches), "clocks": clocks,
        }
        if e2e is not None:
            result["e2e"] = e2e
        print(json.dumps(result), flush=True)


def run_e2e(args, step, x, weight, lin, E, reduce_max=False):
    """The step through the public API with HOST inputs and HOST results: every step copies its
    inputs (features, edge weights, linear weights) from pinned host memory to the device and
    copies the three gradients back to pinned host memory.  Copies run on their own streams so
    that step i+1's upload and step i-1's download overlap step i's kernels (a three-stage
    pipeline over double-buffered device and host buffers); the timed region covers every copy."""
    device = x.device
    host_in = [t.detach().cpu().pin_memory() for t in (x, weight, lin)]
    host_out = [[torch.empty_like(t).pin_memory() for t in host_in] for _ in range(2)]
    dev_in = [[torch.empty_like(t, device=device) for t in host_in] for _ in range(2)]
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = sum(t.numel() * t.element_size() for t in host_out[0])
    compute = torch.cuda.current_stream(device)
    upload, download = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def run(steps):
        uploaded = [None, None]
        computed = [None, None]
        downloaded = [None, None]

        def start_upload(i):
            slot = i & 1
            with torch.cuda.stream(upload):
                if computed[slot] is not None:           # step i-2 has read this input slot
                    upload.wait_event(computed[slot])
                for d, h in zip(dev_in[slot], host_in):
                    d.copy_(h, non_blocking=True)
                uploaded[slot] = upload.record_event()

        start_upload(0)
        for i in range(steps):
            slot = i & 1
            if i + 1 < steps:
                start_upload(i + 1)
            compute.wait_event(uploaded[slot])
            leaves = [d.detach().requires_grad_() for d in dev_in[slot]]
            grads = step(*leaves)
            computed[slot] = compute.record_event()
            with torch.cuda.stream(download):
                download.wait_event(computed[slot])
                if downloaded[slot] is not None:
                    downloaded[slot].synchronize()        # host buffer of step i-2 is free again
                for h, g in zip(host_out[slot], grads):
                    g.record_stream(download)
                    h.copy_(g, non_blocking=True)
                downloaded[slot] = download.record_event()
        torch.cuda.synchronize(device)

    run(2)
    steps = max(4, min(args.steps, 10))
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    begin.record()
    run(steps)
    end.record()
    torch.cuda.synchronize(device)
    ms = begin.elapsed_time(end) / steps
    if reduce_max:
        import torch.distributed as dist

        slowest = torch.tensor([ms], device=x.device, dtype=torch.float64)
        dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
        ms = float(slowest.item())
    return {"value": round(E / (ms * 1e-3) / 1e9, 4), "unit": UNIT, "ms_per_step": round(ms, 3),
            "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "steps": steps,
            "pipeline": "upload / compute / download on three streams, double buffered"}


# --------------------------------------------------------------------------- CPU arm
def cpu_step_factory(row_ptr, col, weight, x, lin, rows):
    """One forward+backward of the GCN layer on the first `rows` destination
    rows, evaluated by the CPU oracle port (aggregation, dx, dw) and torch.mm
    (the linear, which is ordinary Torch user code in the reference)."""
    import numpy as np

    from oracle import oracle

    rp = row_ptr[: rows + 1].numpy().copy()
    edges = int(rp[-1])
    ci = col[:edges].numpy().copy()
    w = weight[:edges].numpy().copy()
    xn = x.numpy()
    n_src = x.shape[0]
    t_ptr, t_col, order = oracle.csr_transpose(rp, ci, n_src)
    ones = torch.ones(rows, lin.shape[1])

    def step():
        agg = oracle.wsum_fwd(rp, ci, xn, w)
        agg_t = torch.from_numpy(agg)
        out = agg_t @ lin
        d_agg = ones @ lin.t()
        d_lin = agg_t.t() @ ones
        d_agg_n = d_agg.numpy()
        dx = oracle.wsum_bwd_dx_pre(rp, t_ptr, t_col, order, n_src, d_agg_n, w)
        dw = oracle.wsum_bwd_dw(rp, ci, d_agg_n, xn)
        return out, dx, dw, d_lin

    return step, edges


def cpu_baseline(args, row_ptr, col, weight, x, lin, steps, warmup):
    from oracle import oracle

    oracle.build()
    cores = oracle.num_threads()
    torch.set_num_threads(max(cores, 1))
    N = row_ptr.numel() - 1
    # size the sample from a small probe so the whole leg stays bounded
    probe_rows = max(N // 64, 1)
    probe, probe_edges = cpu_step_factory(row_ptr, col, weight, x, lin, probe_rows)
    t0 = time.perf_counter()
    probe()
    probe_s = time.perf_counter() - t0
    budget = args.cpu_sample_seconds / max(steps + warmup, 1)
    E = col.numel()
    target_edges = min(E, int(probe_edges * budget / max(probe_s, 1e-6)))
    rows = int(torch.searchsorted(row_ptr, torch.tensor(target_edges), right=True).item()) - 1
    rows = max(min(rows, N), probe_rows)
    step, edges = cpu_step_factory(row_ptr, col, weight, x, lin, rows)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    seconds = (time.perf_counter() - t0) / steps
    return {"value": round(edges / seconds / 1e9, 5), "unit": UNIT, "cores": cores, "kind": "port",
            "seconds_per_step": round(seconds, 3),
            "sample": f"first {rows} of {N} destination rows ({edges} of {E} edges), full feature matrix"}


def run_reference(args):
    """CPU arm: the oracle port on the host cores, same workload and metric."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from baseline import synthetic as syn

    row_ptr, col = syn.rmat_csr(args.scale, args.edge_factor, seed=args.seed, symmetrize=True, device="cpu")
    n = row_ptr.numel() - 1
    weight = syn.gcn_norm_weights(row_ptr, col)
    x = syn.normal((n, args.features), seed=args.seed + 1)
    lin = syn.normal((args.features, args.features), seed=args.seed + 2, std=args.features ** -0.5)
    args.cpu_sample_seconds = 60.0
    base = cpu_baseline(args, row_ptr, col, weight, x, lin, steps=args.steps, warmup=args.warmup)
    value = base["value"]
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(base["seconds_per_step"] * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args), "num_nodes": n, "num_edges": col.numel(),
                   "features": args.features},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
