"""Benchmark of the fused CSR message-passing path (forward + backward).

    python bench.py --gpus N --steps K --warmup W            # this build, on B200s
    python bench.py --impl reference --steps K --warmup W    # the CPU arm

Headline workload, the same at every N (strong scaling): the distributed-halo GCN
configuration -- an R-MAT graph (a, b, c, d = 0.57, 0.19, 0.19, 0.05), 2^scale
nodes and 16 * 2^scale generated edges, symmetrised and de-duplicated, vertex ids
relabelled at random, CSR by destination; edge weight 1/sqrt(deg_i * deg_j);
float32 features [N, 64]; two layers of (sum reducer, dense 64x64 float32
linear); one step = forward plus the backward of out.sum() with respect to the
features, the edge weights and both linear weights.  With N > 1 the graph is cut
into N contiguous destination ranges (the reference's owned_range rule), every
rank generates only its own rows, ghost features are exchanged with NCCL every
layer and their cotangents sent back.  Default scale 25 (the largest that fits
one GPU, so that N = 1 runs the same graph); --scale 26 is the full-size
configuration for N >= 2.  Metric: directed edges traversed per second for
forward + backward, every edge counted once per layer.

Before timing, one step is checked against the CPU oracle on sampled rows
("check" in the JSON line; a miss exits non-zero).  The JSON line carries,
besides the base fields:
  roofline     the dominant kernel's algorithmic GB/s (CUDA events on the
               launching stream inside the timed region) against the measured
               HBM copy bandwidth, the compulsory-traffic figure, and measured
               DRAM traffic when a capture of the current kernel source exists
  e2e          the same step with HOST inputs copied in and gradients copied out
  cpu_baseline the CPU oracle port on a bounded sample of the same workload
  extra        (N = 1) the other configurations: config-1 weighted sum with its
               warm-call host overhead, the GCN layer (sum and max), GAT edge
               attention, varlen causal attention next to flash-attn, and an
               L2-hostile uniform-random gather
"""
from __future__ import annotations

import argparse
import hashlib
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
FALLBACK_BF16_TFLOPS = 1590.0


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="native", choices=("native", "reference"))
    p.add_argument("--scale", type=int, default=25, help="log2 of the node count of the headline graph")
    p.add_argument("--gat-scale", type=int, default=21, help="log2 of the node count of the gat workload's graph")
    p.add_argument("--edge-factor", type=int, default=16)
    p.add_argument("--features", type=int, default=64)
    p.add_argument("--layers", type=int, default=2)
    p.add_argument("--seed", type=int, default=20261125)
    p.add_argument("--labels", default="random", choices=("natural", "random"),
                   help="vertex ids relabelled at random (what Graph500-style generators prescribe; contiguous "
                        "ranges then hold the same mix of degrees) or the generator's ids with hubs at low ids")
    p.add_argument("--waves", type=int, default=None, help="forward halo exchange waves (multi-GPU)")
    p.add_argument("--halo", default="nccl", choices=("nccl", "push"),
                   help="multi-GPU halo transport: grouped NCCL send/recv, or stores into the peers' "
                        "ghost buffers through CUDA IPC windows")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-check", action="store_true")
    p.add_argument("--no-extra", action="store_true")
    p.add_argument("--cpu-sample-seconds", type=float, default=12.0)
    p.add_argument("--workload", default="halo-gcn",
                   choices=("halo-gcn", "gcn-layer", "gcn-layer-max", "weighted-sum", "gat", "attention", "l2-hostile",
                            "generic-program", "user-algebra", "dynamic-radius", "dynamic-knn"),
                   help="halo-gcn = the headline; the others print one of the `extra` sub-results alone (one GPU)")
    p.add_argument("--kernel-table", action="store_true",
                   help="after the timed run, print a per-kernel device-time table of two more steps to stderr")
    return p.parse_args()


def measured_peak(key, fallback):
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as handle:
            return float(json.load(handle)[key]), "measured"
    except Exception:
        return fallback, "fallback"


def hbm_peak():
    return measured_peak("hbm_gbs", FALLBACK_HBM_GBS)


def bf16_peak():
    return measured_peak("bf16_tflops", FALLBACK_BF16_TFLOPS)


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
        return self

    def _pump(self):
        for line in self.process.stdout:
            self.lines.append(line.strip())

    def wait_for_first_sample(self, keep_busy, limit=1.5):
        """nvidia-smi needs a moment to come up: keep the GPU under the same load, untimed, until
        its first sample is in, so that the record covers clocks under load."""
        waited = time.perf_counter()
        while self.process is not None and not self.lines and time.perf_counter() - waited < limit:
            keep_busy()
            torch.cuda.synchronize()

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


def clock_record_rejects(clocks):
    """Why a timed region has to be measured again, or None: a slowdown reason that invalidates
    the number, or a clock record without a single sample."""
    bad = [r for r in clocks.get("reasons", []) if r in ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown")]
    if bad:
        return ",".join(bad)
    if not clocks.get("samples"):
        return "no clock sample during the timed region"
    return None


def timed(step, steps, warmup, device_index=0):
    """(ms per step, clock record): W >= 3 warm-up steps, then `steps` steps between CUDA events on
    the current stream with a synchronize on both sides; measured again once if the clock record
    shows a slowdown."""
    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()

    def region():
        sampler = ClockSampler(device_index).start()
        sampler.wait_for_first_sample(step)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()       # a profiler started with --profile-from-start off sees the timed steps only
        begin.record()
        for _ in range(steps):
            step()
        end.record()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        return begin.elapsed_time(end) / steps, sampler.stop()

    ms, clocks = region()
    rejected = clock_record_rejects(clocks)
    if rejected:
        ms, clocks = region()
        clocks["remeasured_after"] = rejected
    return ms, clocks


# --------------------------------------------------------------------------- roofline figures
def algorithmic_bytes(E, N, F, index_bytes=8):
    """No-reuse algorithmic traffic per launch: indices as given by the API, 4-byte weights, one
    F*4-byte row per edge, a pointer and one row per node."""
    row = 4 * F
    i = index_bytes
    return {"fwd": E * (i + 4 + row) + N * (i + row),
            "dx": E * (2 * i + 4 + row) + N * (i + row),
            "dw": E * (i + row + 4) + N * (i + row)}


def ideal_cache_bytes(E, N, F, index_bytes=8):
    """Compulsory traffic: every array moved exactly once (a perfect cache for the gathered rows)."""
    row = 4 * F
    i = index_bytes
    return {"fwd": E * (i + 4) + N * (i + 2 * row),
            "dx": E * (2 * i + 4) + N * (i + 2 * row),
            "dw": E * (i + 4) + N * (i + 2 * row)}


def kernel_source_id():
    """Identifies the gather kernels' source: recorded DRAM captures apply to one version of it."""
    digest = hashlib.sha1()
    for name in ("tgb_csr_reduce.cu", "tgb_common.cuh"):
        with open(os.path.join(ROOT, "tiga-lang_b200", "csrc", name), "rb") as handle:
            digest.update(handle.read())
    return digest.hexdigest()[:12]


def recorded_dram_traffic(workload_key):
    """DRAM bytes per launch from a committed one-pass ncu capture (dram__bytes_read.sum +
    dram__bytes_write.sum) of this workload, or None.  A capture is used only while the kernel
    source it was taken from is the one that runs now."""
    try:
        with open(os.path.join(ROOT, "baseline", "dram_traffic.json")) as handle:
            table = json.load(handle)
    except Exception:
        return None
    entry = table.get(workload_key)
    if not entry or entry.get("kernel_source") != kernel_source_id():
        return None
    return entry


def instrument(ops, timings, recording):
    """Wraps the three kernel entry points with CUDA events on the launching stream."""
    def wrap(name, function):
        def wrapper(*a, **k):
            if not recording["on"]:
                return function(*a, **k)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            result = function(*a, **k)
            stop.record()
            timings[name].append((start, stop))
            return result
        wrapper.__wrapped__ = function
        return wrapper

    for name, attribute in (("fwd", "csr_reduce_forward"), ("dx", "csr_reduce_backward_dx"),
                            ("dw", "csr_reduce_backward_dw")):
        current = getattr(ops, attribute)
        setattr(ops, attribute, wrap(name, getattr(current, "__wrapped__", current)))


def gather_roofline(kernel_ms, bytes_per, ideal_per, workload_key, launches_per_step):
    """Roofline object for the dominant CSR kernel of a step.  `kernel_ms` is device time per step
    per kernel kind, `bytes_per` / `ideal_per` the algorithmic and compulsory bytes per step."""
    peak, peak_kind = hbm_peak()
    dominant = max(kernel_ms, key=kernel_ms.get)
    achieved = bytes_per[dominant] / (kernel_ms[dominant] * 1e-3) / 1e9
    names = {"fwd": "k_gather_vec (forward)", "dx": "k_gather_vec (transposed relation, dx)",
             "dw": "k_edge_dot_vec (dw)"}
    capture = recorded_dram_traffic(workload_key)
    traffic = capture["bytes_per_launch"].get(dominant) if capture else None
    per_launch = max(launches_per_step.get(dominant, 1), 1)
    roofline = {
        "bound": "hbm", "kernel": names[dominant], "achieved": round(achieved, 1), "peak": peak,
        "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": round(achieved / peak, 4),
        "traffic": traffic,
        "launches_per_step": per_launch,
        "algorithmic_bytes_per_launch": int(bytes_per[dominant] // per_launch),
        "ideal_cache_bytes_per_launch": int(ideal_per[dominant] // per_launch),
        "ideal_cache_frac": round(ideal_per[dominant] / (kernel_ms[dominant] * 1e-3) / 1e9 / peak, 4),
        "kernel_ms_per_step": {k: round(v, 4) for k, v in kernel_ms.items()},
        "kernel_algorithmic_gbs": {k: round(bytes_per[k] / (kernel_ms[k] * 1e-3) / 1e9, 1) for k in kernel_ms
                                   if kernel_ms[k] > 0},
        "step_algorithmic_frac": round(sum(bytes_per.values()) / (sum(kernel_ms.values()) * 1e-3) / 1e9 / peak, 4),
        "note": "algorithmic bytes count every gathered row once per edge (no reuse); rows that hit in the "
                "126 MB L2 make frac exceed 1, ideal_cache_frac is the same time against compulsory bytes",
    }
    if capture:
        launch_ms = kernel_ms[dominant] / per_launch
        roofline["dram_frac"] = round(traffic / (launch_ms * 1e-3) / 1e9 / peak, 4) if traffic else None
        roofline["traffic_capture"] = {k: capture[k] for k in ("commit", "kernel_source", "how") if k in capture}
    else:
        roofline["dram_frac"] = None
    return roofline


# --------------------------------------------------------------------------- headline: halo GCN
def headline_name(args):
    return (f"halo gcn {args.layers} layers rmat scale={args.scale} edge_factor={args.edge_factor} symmetrized "
            f"dedup labels={args.labels} F={args.features} fp32 sum+linear fwd+bwd")


def build_gcn_layer_class():
    import tiga as tg

    class GCNLayer(tg.MessagePassing):
        reducer = tg.sum()

        def edge(self, src, dst, edge):
            return edge.weight * src.x

    return GCNLayer


class _NullContext:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def run_halo_gcn(args):
    import torch.distributed as dist

    import tiga as tg
    from baseline import synthetic as syn
    from baseline import verify
    from tiga import _native, ops
    from tiga.distributed.model import owned_range
    from tiga.distributed.runtime import DistributedRuntime, NCCLTransport, shard_plan_for

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    _native.lib()
    torch.backends.cuda.matmul.allow_tf32 = False
    F, layers, N = args.features, args.layers, 1 << args.scale
    first, last = owned_range(N, world, rank)

    # ---- this rank's rows only: the whole graph is never held anywhere
    setup = time.perf_counter()
    row_ptr, col = syn.rmat_csr_rows(args.scale, args.edge_factor, first, last, seed=args.seed, symmetrize=True,
                                     relabel=args.labels == "random", device=device)
    local_degree = row_ptr[1:] - row_ptr[:-1]
    if world > 1:
        sizes = [owned_range(N, world, r) for r in range(world)]
        widest = max(e - b for b, e in sizes)
        padded = torch.zeros(widest, dtype=torch.int64, device=device)
        padded[:local_degree.numel()] = local_degree
        pieces = [torch.empty_like(padded) for _ in range(world)]
        dist.all_gather(pieces, padded)
        degree = torch.cat([piece[:e - b] for piece, (b, e) in zip(pieces, sizes)])
        del pieces, padded
    else:
        degree = local_degree
    E_local = int(col.numel())
    totals = torch.tensor([E_local], dtype=torch.int64, device=device)
    if world > 1:
        dist.all_reduce(totals)
    E = int(totals.item())
    weight = syn.gcn_norm_weights_rows(row_ptr, col, degree, first).requires_grad_()
    max_degree = int(degree.max().item())
    del degree, local_degree
    x = syn.normal_rows(first, last, F, seed=args.seed + 1, device=device).requires_grad_()
    linears = [syn.normal((F, F), seed=args.seed + 2 + k, device=device, std=F ** -0.5).requires_grad_()
               for k in range(layers)]
    runtime = None
    if world > 1:
        graph = tg.Graph.from_csr_shard(row_ptr, col, num_nodes=N, first_row=first).halo(tg.DeviceMesh("cuda", world))
        runtime = DistributedRuntime(NCCLTransport(device=device), trace=True, waves=args.waves,
                                     push=args.halo == "push")
        with runtime:
            shard = shard_plan_for(graph, runtime)
        for relation in (shard.graph_own, shard.graph_ghost):
            relation.native_plan(transpose=True)
        for _, relation in shard.waves:
            relation.native_plan(transpose=False)
    else:
        graph = tg.Graph.from_csr(row_ptr, col, num_src=N)
        graph.native_plan(transpose=True)
        shard = None
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    setup_s = time.perf_counter() - setup
    rows = last - first
    layer = build_gcn_layer_class()()
    ones = torch.ones((rows, F), dtype=torch.float32, device=device)     # d(out.sum()) / d(out)

    def forward(xs, ws, ls, keep=None):
        h = xs
        for k, matrix in enumerate(ls):
            agg = layer(graph=graph, src={"x": h}, dst={}, edge={"weight": ws})
            h = ops.dense_linear(agg, matrix)
            if keep is not None:
                keep[f"agg{k + 1}"], keep[f"h{k + 1}"] = agg, h
        return h

    def step(xs=x, ws=weight, ls=linears):
        if runtime is not None:
            with runtime:
                out = forward(xs, ws, ls)
                grads = torch.autograd.grad(out, (xs, ws, *ls), ones)
            flat = torch.cat([g.reshape(-1) for g in grads[2:]])
            dist.all_reduce(flat)                # replicated linear weights: one all-reduce of their gradients
            return grads[0], grads[1], flat
        out = forward(xs, ws, ls)
        grads = torch.autograd.grad(out, (xs, ws, *ls), ones)
        return grads[0], grads[1], torch.cat([g.reshape(-1) for g in grads[2:]])

    # ---- verification step: sampled rows against the CPU oracle, on every rank
    check = None
    if not args.no_check and layers == 2:
        from oracle import oracle

        oracle.build()
        keep = {}
        with (runtime if runtime is not None else _NullContext()):
            out = forward(x, weight, linears, keep)
            wanted = (x, weight, linears[0], linears[1], keep["agg1"], keep["h1"], keep["agg2"])
            dx, dw, dW1, dW2, d_agg1, d_h1, d_agg2 = torch.autograd.grad(out, wanted, ones)
        if world > 1:
            dist.all_reduce(dW1)
            dist.all_reduce(dW2)
        tensors = {"agg1": keep["agg1"], "h1": keep["h1"], "agg2": keep["agg2"], "out": out, "d_agg1": d_agg1,
                   "d_h1": d_h1, "d_agg2": d_agg2, "dx": dx, "dw": dw, "dW1": dW1, "dW2": dW2}
        mine = verify.check_two_layer_gcn(
            oracle, row_ptr=row_ptr, col_idx=col, first_row=first, num_nodes=N, weight=weight,
            feature_of=lambda ids: syn.normal_rows(0, 0, F, seed=args.seed + 1, ids=ids), tensors=tensors,
            linears=linears, world=world)
        del tensors, keep, out, dx, dw, d_agg1, d_h1, d_agg2, wanted, dW1, dW2
        ops.check_async_errors()
        gathered = [mine]
        if world > 1:
            gathered = [None] * world
            dist.all_gather_object(gathered, mine)
        worst = max(gathered, key=lambda c: c["max_excess"])
        check = {"rows": sum(c["rows"] for c in gathered), "edges": sum(c["edges"] for c in gathered),
                 "max_excess": worst["max_excess"], "worst": worst["worst"],
                 "ok": all(c["ok"] for c in gathered), "ranks": len(gathered),
                 "checked": "agg1 agg2 h1 out dx d_h1 d_agg1 dw dW1 dW2 on sampled owned rows of every rank vs the "
                            "CPU oracle (rel 1e-5 / abs 1e-6 + 8 ulp of sum |terms|); remote rows fetched by all-reduce",
                 "excess_rank0": gathered[0]["excess"]}
        torch.cuda.empty_cache()

    # ---- timed region
    timings = {"fwd": [], "dx": [], "dw": []}
    recording = {"on": False}
    instrument(ops, timings, recording)
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    sync = dist.barrier if world > 1 else None

    def region():
        for v in timings.values():
            v.clear()
        if runtime is not None:
            runtime.reset_trace()
        sampler = ClockSampler(local).start()
        if world == 1:
            sampler.wait_for_first_sample(step)
        if sync:
            sync()
        before = _native.launch_count()
        recording["on"] = True
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        begin.record()
        for _ in range(args.steps):
            step()
        end.record()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        if sync:
            sync()
        recording["on"] = False
        return begin.elapsed_time(end) / args.steps, _native.launch_count() - before, sampler.stop()

    ms_mine, launches, clocks = region()
    rejected = clock_record_rejects(clocks)
    again = bool(rejected)
    if world > 1:       # every rank must agree on a second measurement
        flag = torch.tensor([1 if rejected else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        again = bool(flag.item())
    if again:
        ms_mine, launches, clocks = region()
        clocks["remeasured_after"] = rejected or "a peer's clock record"
    ops.check_async_errors()
    slowest = torch.tensor([ms_mine], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
    ms_per_step = float(slowest.item())
    traversed = layers * E
    value = traversed / (ms_per_step * 1e-3) / 1e9

    kernel_ms = {k: sum(a.elapsed_time(b) for a, b in v) / args.steps for k, v in timings.items()}
    launches_per_step = {k: len(v) // args.steps for k, v in timings.items()}
    table_rows = rows + (int(shard.ghosts.numel()) if shard is not None else 0)
    bytes_per = {k: v * layers for k, v in algorithmic_bytes(E_local, rows, F).items()}
    ideal_per = {k: v * layers for k, v in ideal_cache_bytes(E_local, table_rows, F).items()}
    workload = headline_name(args)
    roofline = gather_roofline(kernel_ms, bytes_per, ideal_per, f"{workload} n_gpus={world}", launches_per_step)
    if world > 1:
        roofline["kernel"] = f"rank 0: {roofline['kernel']} (owned-source + ghost-source passes)"

    config = {"workload": workload, "num_nodes": N, "num_edges": E, "layers": layers, "features": F,
              "edges_traversed_per_step": traversed, "index_dtype": "int64", "max_degree": max_degree,
              "partition": "contiguous destination ranges, balanced node counts (the reference's owned_range rule)",
              "l2": "inputs exceed L2 (feature table and index arrays are each far above 126 MB)",
              "setup_s": round(setup_s, 2)}
    if shard is not None:
        stats = torch.tensor([E_local, rows, int(shard.ghosts.numel()), int(shard.edges_ghost.numel())],
                             device=device, dtype=torch.int64)
        gathered = [torch.empty_like(stats) for _ in range(world)]
        dist.all_gather(gathered, stats)
        phases = runtime.phase_times()
        runtime.trace = False
        names = sorted(phases)
        mine = torch.tensor([phases[k] / args.steps for k in names] + [ms_mine], device=device, dtype=torch.float64)
        everyone = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(everyone, mine)
        config.update({
            "waves": len(shard.waves),
            "halo_transport": ("stores into the peers' ghost buffers through CUDA IPC windows + one-element "
                               "all-reduce signals" if args.halo == "push" else "grouped NCCL send/recv"),
            "per_rank_edges_rows_ghosts_ghostedges": torch.stack(gathered).tolist(),
            "halo_bytes_per_layer_rank0": int(shard.ghosts.numel()) * F * 4,
            "phase_ms_per_rank": {name: [round(float(r[i]), 3) for r in everyone]
                                  for i, name in enumerate(names + ["step (own clock)"])}})

    if args.kernel_table:
        kernel_table(step, rank)
    e2e = None if args.no_e2e else run_e2e(args, step, x, weight, linears, traversed, world)
    result = {
        "metric": METRIC, "value": round(value, 4), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
        "roofline": roofline, "gpu_launches": int(launches), "clocks": clocks,
    }
    if check is not None:
        result["check"] = check
    if e2e is not None:
        result["e2e"] = e2e
    failed = check is not None and not check["ok"]
    if rank == 0 and world == 1 and not failed and not args.no_cpu_baseline:
        result["cpu_baseline"] = cpu_baseline_halo(args, row_ptr, col, weight, x, linears, steps=1, warmup=0,
                                                   seconds=args.cpu_sample_seconds)
    # free the headline workload before the other configurations run
    del x, weight, linears, ones, row_ptr, col, graph, layer, step, forward, shard
    torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not failed and not args.no_extra:
        from baseline import bench_extra

        result["extra"] = bench_extra.run_all(args, device, sys.modules[__name__])
    if rank == 0:
        print(json.dumps(result), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if failed:
        raise SystemExit(f"verification failed: {check['worst']} exceeds its bound by {check['max_excess']:.3e}")


def kernel_table(run, rank, steps=2):
    """Device time per kernel over a few steps (torch profiler), for analysis only."""
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        for _ in range(steps):
            run()
        torch.cuda.synchronize()
    table = prof.key_averages().table(sort_by="cuda_time_total", row_limit=28, max_name_column_width=70)
    print(f"---- rank {rank}: device time over {steps} steps\n{table}", file=sys.stderr, flush=True)


def run_e2e(args, step, x, weight, linears, traversed, world):
    """The step through the public API with HOST inputs and HOST results: every step copies its
    inputs (features, edge weights, linear weights) from pinned host memory to the device and
    copies the gradients back to pinned host memory.  Upload, compute and download run on their
    own streams, so step i+1's upload and step i-1's download overlap step i's kernels; the timed
    region covers every copy.  Device input buffers are double buffered while they fit."""
    device = x.device
    host_in = [t.detach().cpu().pin_memory() for t in (x, weight, *linears)]
    # a second set of device input buffers lets step i + 1 upload while step i computes; it is used
    # whenever it fits beside the step's own working set with 16 GB to spare
    torch.cuda.empty_cache()
    input_bytes = sum(t.numel() * t.element_size() for t in host_in)
    free_bytes, _ = torch.cuda.mem_get_info(device)
    slots = 2 if free_bytes - 3 * input_bytes > 16e9 else 1       # two input sets and the staging set
    packed = sum(m.numel() for m in linears)
    host_out = [[torch.empty_like(host_in[0]).pin_memory(), torch.empty_like(host_in[1]).pin_memory(),
                 torch.empty(packed, dtype=torch.float32).pin_memory()] for _ in range(slots)]
    dev_in = [[torch.empty_like(t, device=device) for t in host_in] for _ in range(slots)]
    # the gradients leave through one persistent staging set: the step's own tensors are released as soon
    # as they are copied into it (a device-to-device copy on the compute stream), so the caching allocator
    # never holds blocks back for the download stream and never has to synchronise to find memory
    dev_out = [torch.empty_like(t, device=device) for t in host_out[0]]
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = sum(t.numel() * t.element_size() for t in host_out[0])
    compute = torch.cuda.current_stream(device)
    upload, download = torch.cuda.Stream(device), torch.cuda.Stream(device)

    timeline = []     # per step: events at the start / end of its upload, compute and download

    def stamp(stream):
        event = torch.cuda.Event(enable_timing=True)
        event.record(stream)
        return event

    def run(steps):
        uploaded, computed, downloaded = [None] * slots, [None] * slots, [None] * slots
        staged = {"free": None}
        del timeline[:]
        timeline.extend({} for _ in range(steps))

        def start_upload(i):
            slot = i % slots
            with torch.cuda.stream(upload):
                if computed[slot] is not None:           # the step that read this input slot is done
                    upload.wait_event(computed[slot])
                timeline[i]["upload"] = [stamp(upload)]
                for d, h in zip(dev_in[slot], host_in):
                    d.copy_(h, non_blocking=True)
                uploaded[slot] = upload.record_event()
                timeline[i]["upload"].append(stamp(upload))

        start_upload(0)
        for i in range(steps):
            slot = i % slots
            if slots > 1 and i + 1 < steps:
                start_upload(i + 1)
            compute.wait_event(uploaded[slot])
            timeline[i]["compute"] = [stamp(compute)]
            leaves = [d.detach().requires_grad_() for d in dev_in[slot]]
            grads = step(leaves[0], leaves[1], leaves[2:])
            if staged["free"] is not None:
                compute.wait_event(staged["free"])        # the previous step's download has read the staging set
            for staging, g in zip(dev_out, grads):
                staging.copy_(g.reshape(staging.shape))
            computed[slot] = compute.record_event()
            timeline[i]["compute"].append(stamp(compute))
            if slots == 1 and i + 1 < steps:
                start_upload(i + 1)
            with torch.cuda.stream(download):
                download.wait_event(computed[slot])
                if downloaded[slot] is not None:
                    downloaded[slot].synchronize()        # the host buffer is free again
                timeline[i]["download"] = [stamp(download)]
                for h, staging in zip(host_out[slot], dev_out):
                    h.copy_(staging, non_blocking=True)
                downloaded[slot] = download.record_event()
                staged["free"] = downloaded[slot]
                timeline[i]["download"].append(stamp(download))
            del grads, leaves
        torch.cuda.synchronize(device)

    run(2)
    # the same number of steps as the device-resident measurement (bounded: a step moves 25 GB over the
    # host link); the pipeline starts empty and is drained inside the timed region
    steps = max(3, min(args.steps, 40))
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    begin.record()
    run(steps)
    end.record()
    torch.cuda.synchronize(device)
    ms = begin.elapsed_time(end) / steps
    # when each phase of each timed step ran on the device, in ms from the start of the timed region
    phases = [{name: [round(begin.elapsed_time(a), 1), round(begin.elapsed_time(b), 1)]
               for name, (a, b) in entry.items()} for entry in timeline]
    if world > 1:
        import torch.distributed as dist

        slowest = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
        ms = float(slowest.item())
    return {"value": round(traversed / (ms * 1e-3) / 1e9, 4), "unit": UNIT, "ms_per_step": round(ms, 3),
            "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "steps": steps,
            "pipeline": f"upload / compute / download on three streams, {slots} input slot(s); bytes are per rank",
            "timeline_ms": phases}


# --------------------------------------------------------------------------- CPU arm
def cpu_gcn_step_factory(rp, ci, w, table, linears, layers):
    """One forward+backward of the GCN layers on a block of destination rows, evaluated by the
    CPU oracle port (aggregation, dx, dw) and torch.mm (the linear, which is ordinary Torch user
    code in the reference).  Every layer gathers from the same feature table (a sample of rows
    cannot produce the hidden features of all its neighbours; the work per layer is the same)."""
    from oracle import oracle

    rows = rp.shape[0] - 1
    n_src = table.shape[0]
    t_ptr, t_col, order = oracle.csr_transpose(rp, ci, n_src)
    mats = [m.detach().cpu() for m in linears]
    ones = torch.ones(rows, mats[0].shape[1])

    def step():
        results = []
        for k in range(layers):
            agg = oracle.wsum_fwd(rp, ci, table, w)
            agg_t = torch.from_numpy(agg)
            out = agg_t @ mats[k]
            d_agg = ones @ mats[k].t()
            d_lin = agg_t.t() @ ones
            d_agg_n = d_agg.numpy()
            dx = oracle.wsum_bwd_dx_pre(rp, t_ptr, t_col, order, n_src, d_agg_n, w)
            dw = oracle.wsum_bwd_dw(rp, ci, d_agg_n, table)
            results.append((out, dx, dw, d_lin))
        return results

    return step


def cpu_sample(row_ptr, col, weight, feature_rows, rows):
    """The first `rows` destination rows with their edges, sources renumbered onto the compact
    table of the feature rows they read (numpy arrays on the host).  `feature_rows(ids)` returns
    the feature rows of global ids as a tensor."""
    edges = int(row_ptr[rows].item())
    rp = row_ptr[:rows + 1].cpu().numpy().copy()
    sources, compact = torch.unique(col[:edges], return_inverse=True)
    table = feature_rows(sources).cpu().numpy()
    return rp, compact.cpu().numpy(), weight.detach()[:edges].cpu().numpy().copy(), table, edges


def cpu_baseline_rows(row_ptr, col, weight, feature_rows, linears, steps, warmup, seconds):
    """Oracle port on the first rows of a graph, sized from a probe so that the whole leg takes
    about `seconds`.  Uses every host core."""
    from oracle import oracle

    oracle.build()
    cores = os.cpu_count() or 1
    oracle.set_num_threads(cores)        # a launcher may have exported OMP_NUM_THREADS=1
    torch.set_num_threads(cores)
    cores = oracle.num_threads()
    N = row_ptr.numel() - 1
    layers = len(linears)

    def make(rows):
        rp, ci, w, table, edges = cpu_sample(row_ptr, col, weight, feature_rows, rows)
        return cpu_gcn_step_factory(rp, ci, w, table, linears, layers), edges, table.shape[0]

    probe_rows = max(min(N // 64, 1 << 14), 1)
    probe, probe_edges, _ = make(probe_rows)
    t0 = time.perf_counter()
    probe()
    probe_s = time.perf_counter() - t0
    budget = seconds / max(steps + warmup, 1)
    target = min(int(col.numel()), int(probe_edges * budget / max(probe_s, 1e-6)))
    rows = int(torch.searchsorted(row_ptr, torch.tensor(target, device=row_ptr.device), right=True).item()) - 1
    rows = max(min(rows, N), probe_rows)
    step, edges, table_rows = make(rows)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    per_step = (time.perf_counter() - t0) / steps
    return {"value": round(layers * edges / per_step / 1e9, 5), "unit": UNIT, "cores": cores, "kind": "port",
            "seconds_per_step": round(per_step, 3),
            "sample": f"first {rows} of {N} held destination rows ({edges} of {col.numel()} held edges) x {layers} "
                      f"layer(s), gathering from the {table_rows} feature rows those edges read"}


def cpu_baseline_halo(args, row_ptr, col, weight, x, linears, steps, warmup, seconds):
    return cpu_baseline_rows(row_ptr, col, weight, lambda ids: x.detach().index_select(0, ids), linears,
                             steps, warmup, seconds)


def run_reference(args):
    """CPU arm: the oracle port (the reference's MLIR/LLVM CPU path cannot be built here and its
    Python evaluator cannot travel to the GPU box) on all host cores, same workload and metric.
    The sample's inputs are generated on the GPU when one is present (generation is not timed) and
    copied to the host; under a multi-rank launch rank 0 alone works."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from baseline import synthetic as syn

    device = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    if device.type != "cuda":
        args.scale = min(args.scale, 20)          # generating 2^25 * 16 edges on host cores takes many minutes
    N, F = 1 << args.scale, args.features
    held = max(N // 64, 1)                         # a block of rows larger than any sample the time budget allows
    row_ptr, col = syn.rmat_csr_rows(args.scale, args.edge_factor, 0, held, seed=args.seed, symmetrize=True,
                                     relabel=args.labels == "random", device=device)
    # source degrees outside the held block are unknown here; the graph-wide mean stands in for them
    # (a weight's value does not change the work that is timed)
    degree = torch.full((N,), float(col.numel()) / held, device=device)
    degree[:held] = (row_ptr[1:] - row_ptr[:-1]).clamp(min=1).float()
    weight = syn.gcn_norm_weights_rows(row_ptr, col, degree, 0)
    linears = [syn.normal((F, F), seed=args.seed + 2 + k, std=F ** -0.5) for k in range(args.layers)]
    steps = max(args.steps, 1)
    base = cpu_baseline_rows(
        row_ptr, col, weight, lambda ids: syn.normal_rows(0, 0, F, seed=args.seed + 1, device=device, ids=ids),
        linears, steps=steps, warmup=args.warmup, seconds=min(150.0, max(45.0, 8.0 * (steps + args.warmup))))
    value = base["value"]
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": round(base["seconds_per_step"] * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": headline_name(args), "num_nodes": N, "layers": args.layers, "features": F},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    args = parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    if args.workload == "halo-gcn":
        return run_halo_gcn(args)
    from baseline import bench_extra

    torch.cuda.set_device(0)
    print(json.dumps(bench_extra.run_one(args.workload, args, torch.device("cuda", 0), sys.modules[__name__])),
          flush=True)


if __name__ == "__main__":
    main()
