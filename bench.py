"""Benchmark of the UVU TensorProductConv hot path: forward + backward edges/s and HBM roofline fraction.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2|cfg3|cfg4|cfg5|cfg1|lmax1|sh6]
                    [--impl reference]

One "step" is one forward plus one backward (gx, gy, gw) of the convolution over the whole synthetic graph (for
``cfg3``: one force-training step, energy -> forces -> loss -> dL/dweight, through the public modules; for ``sh6``:
spherical harmonics of 4 M vectors, forward and backward).  With N > 1 (launched by torchrun, one rank per GPU) the
graph has N times as many atoms, destination ranges are assigned to ranks (weak scaling), the source rows a rank
needs from other ranks are exchanged with one all-to-all before the forward and their gradients go back with one
all-to-all after the backward, both inside the step.  Rank 0 prints one JSON line.

The default run (N = 1, workload cfg2) also measures the other workloads briefly and reports them under ``others``.
``--impl reference`` times the CPU restatement of the reference's path on all host cores (the reference has no CPU
implementation of the convolution); if a GPU and the reference's own compiled kernels (``oracle/_ref``) are present
it adds their throughput on the same graph as ``reference_gpu``.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from bench_workloads import CUTOFF, DENSITY, WORKLOADS, build_graph_edges, build_paths  # noqa: E402

# DRAM traffic per edge (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture, divided by the edges of the
# captured launch), keyed by workload and by the kernel variant that was captured; the summaries under profiles/ give
# the commands.  The captures are single-pass runs of the two byte counters on this workload at its full size (50,000
# atoms); a run on another atom count scales them by its edges, which is what the traffic grows with.  A run whose plan
# picks another variant reports null.
NCU_TRAFFIC_BYTES_PER_EDGE = {
    ("cfg2", "forward", "staged"): 9.48e3,
    ("cfg2", "backward", "row"): 18.31e3,
}
SH6_ITEMS = 4_000_000
# algorithmic FLOPs per edge of the forward pass (sum over paths of channels * (2 * terms + d2))
FORWARD_FLOPS_PER_EDGE = {"cfg1": 288, "cfg2": 64128, "cfg3": 64128, "cfg4": 51520, "cfg5": 12864}


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="native", choices=["native", "reference"])
    p.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS) + ["sh6"])
    p.add_argument("--atoms-per-gpu", type=int, default=None)
    p.add_argument("--e2e-steps", type=int, default=3)
    p.add_argument("--skip-e2e", action="store_true")
    p.add_argument("--skip-cpu", action="store_true")
    p.add_argument("--skip-others", action="store_true")
    p.add_argument("--cpu-seconds", type=float, default=15.0)
    p.add_argument("--generic", action="store_true", help="force the table-driven kernels")
    p.add_argument("--overlap", action="store_true",
                   help="N > 1: hide the halo exchanges behind the interior piece of the shard (sharded."
                        "overlapped_step) instead of exchange, forward, backward, return one after the other; "
                        "measured slower at N = 2 and N = 8 on cfg2 (three launches per pass cost more than the "
                        "exchanges), so it is not the default")
    p.add_argument("--e2e-chunks", type=int, default=32, help="pieces of the host-streamed step")
    return p.parse_args()


def algorithmic_bytes(n_dst, n_src, edges, X, Y, O, W, S):
    """Bytes that must cross HBM once per pass: forward and backward (gx, gy, gw)."""
    fwd = edges * (W + Y) * S + 4 * edges + 4 * (n_dst + 1) + n_src * X * S + n_dst * O * S
    bwd = 2 * edges * (W + Y) * S + n_src * X * S + n_dst * O * S + n_src * X * S + 12 * edges
    return fwd, bwd


def static_config(name, atoms, world):
    """What both arms print as ``config``: the workload as asked for, nothing measured."""
    if name == "sh6":
        return {"workload": "sh6", "items": SH6_ITEMS, "lmax": 6, "normalize": True, "normalization": "component",
                "parallelism": f"replicas x{world}"}
    in1, in2, out, instructions, dtype, default_atoms, kind, lmax = build_paths(name)
    step = "energy -> forces -> loss -> dL/dweight" if name == "cfg3" else "forward + backward (gx, gy, gw)"
    return {"workload": name, "irreps_in1": in1, "irreps_in2": in2, "irreps_out": out, "paths": len(instructions),
            "atoms_per_gpu": atoms or default_atoms, "graph": kind, "density": DENSITY, "cutoff": CUTOFF,
            "atom_order": "cell (spatial) order", "step": step, "parallelism": f"dst-range x{world}",
            "cache": "inputs larger than L2 (the per-edge weights alone are GBs)"}


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as handle:
            peaks = json.load(handle)
        return float(peaks["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, "fallback"


# ------------------------------------------------------------------------------------------------- clocks


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, device):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.proc = None
        try:
            uuid = str(torch.cuda.get_device_properties(device).uuid)
            target = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", target, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                self.samples.append(float(parts[0]))
                self.max_mhz = float(parts[1])
            except ValueError:
                continue
            for name, value in zip(self.NAMES, parts[2:6]):
                if value == "Active":
                    self.reasons.add(name)

    def reset(self):
        """Drop the samples taken so far (warm-up); the timed region starts now."""
        self.samples, self.reasons = [], set()

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------- CPU arm


def host_threads() -> int:
    """All host cores this process may use, whatever OMP_NUM_THREADS says (torchrun sets it to 1)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_sample_rate(name, seconds, atoms=None):
    """Edges/s of the CPU restatement (oracle) for forward + backward on a contiguous destination range of the
    workload's own graph, sized to take about ``seconds``."""
    import bench_workloads as workloads
    from oracle import spherical_harmonics as oracle_sh
    from oracle import uvu_conv as oracle_conv

    torch.set_num_threads(host_threads())
    in1, in2, out, instructions, dtype, default_atoms, kind, lmax = build_paths(name)
    atoms = atoms or default_atoms
    meta = oracle_conv.build_specs(in1, in2, out, instructions)
    generator = torch.Generator().manual_seed(0)
    degrees = (1,) if name == "cfg1" else tuple(range(lmax + 1))
    if kind == "radius":
        pos, box, cells = workloads.periodic_positions(atoms, DENSITY, 0, "cpu", CUTOFF)

        def edges_of(count):
            return workloads.radius_graph_periodic(pos, box, CUTOFF, cells, 0, count)
    else:
        full = build_graph_edges(name, atoms, 1, 0, "cpu")

        def edges_of(count):
            keep = full[1] < count
            return full[0][keep], full[1][keep], full[2][keep]

    x = torch.randn(atoms, meta["in1_dim"], generator=generator, dtype=dtype)

    def run(sample_nodes):
        src, dst, vec = edges_of(sample_nodes)
        edges = src.numel()
        y = oracle_sh.spherical_harmonics(degrees, vec.to(dtype), True, "component")
        w = torch.randn(edges, meta["weight_numel"], generator=generator, dtype=dtype)
        g = torch.randn(sample_nodes, meta["out_dim"], generator=generator, dtype=dtype)
        t0 = time.perf_counter()
        oracle_conv.conv_forward_backward_chunked(meta, x, y, w, g, src, dst, sample_nodes, chunk_edges=8192)
        return edges, time.perf_counter() - t0

    run(8)  # warm-up (thread pools, allocator)
    edges, elapsed = run(32)
    rate = edges / elapsed
    per_node = max(1.0, edges / 32)
    sample_nodes = int(max(32, min(atoms, rate * seconds / per_node)))
    edges, elapsed = run(sample_nodes)
    return dict(value=edges / elapsed, unit="edges/s", cores=torch.get_num_threads(), kind="port", seconds=elapsed,
                sample=f"destination nodes 0..{sample_nodes - 1} of the {name} graph ({atoms} atoms, {kind}) with "
                       f"all their {edges} incoming edges, forward+backward in {dtype}, {elapsed:.1f} s")


def reference_gpu_rate(name, atoms):
    """Forward + backward of the reference's own compiled kernels on this box's GPU, if both are there."""
    from oracle import ref_kernels

    in1, in2, out, instructions, dtype, default_atoms, kind, lmax = build_paths(name)
    key = f"{name}.{str(dtype).removeprefix('torch.')}"
    if not torch.cuda.is_available():
        return {"unavailable": "no GPU visible to the reference arm"}
    if not ref_kernels.available(key):
        return {"unavailable": f"oracle/_ref holds no build of the reference's kernels for {key}"}
    import lunaequivariance_b200 as luna

    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    atoms = atoms or default_atoms
    reference = ref_kernels.ReferenceKernels(key)
    src, dst, vec = build_graph_edges(name, atoms, 1, 0, device)
    graph = luna.make_graph(src, dst, atoms)
    y = luna.spherical_harmonics(list(range(lmax + 1)), vec.to(dtype), True, "component").contiguous()
    generator = torch.Generator(device=device).manual_seed(100)
    entry = reference.entry
    x = torch.randn(atoms, entry["in1_dim"], device=device, dtype=dtype, generator=generator)
    w = torch.randn(graph.num_edges, entry["weight_numel"], device=device, dtype=dtype, generator=generator)
    g = torch.randn(atoms, entry["out_dim"], device=device, dtype=dtype, generator=generator)
    for _ in range(2):
        reference.forward(x, y, w, graph)
        reference.backward(x, y, w, g, graph)
    events = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    torch.cuda.synchronize()
    reps = 5
    fwd_ms = bwd_ms = 0.0
    for _ in range(reps):
        events[0].record()
        reference.forward(x, y, w, graph)
        events[1].record()
        reference.backward(x, y, w, g, graph)
        events[2].record()
        torch.cuda.synchronize()
        fwd_ms += events[0].elapsed_time(events[1]) / reps
        bwd_ms += events[1].elapsed_time(events[2]) / reps
    return {"value": graph.num_edges / ((fwd_ms + bwd_ms) * 1e-3), "unit": "edges/s", "forward_ms": fwd_ms,
            "backward_ms": bwd_ms, "edges": graph.num_edges,
            "what": "the reference's generated CUDA kernels, built for sm_100 by oracle/build_ref.py, same graph"}


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    name = "cfg2" if args.workload == "sh6" else args.workload
    in1, in2, out, instructions, dtype, atoms, kind, lmax = build_paths(name)
    rates = []
    for step in range(args.warmup + args.steps):
        result = cpu_sample_rate(name, max(2.0, args.cpu_seconds / 3), args.atoms_per_gpu)
        if step >= args.warmup:
            rates.append(result)
    value = statistics.mean(r["value"] for r in rates)
    sample = rates[-1]
    try:
        gpu = reference_gpu_rate(name, args.atoms_per_gpu)
    except Exception as error:  # the CPU number stands on its own
        gpu = {"unavailable": f"{type(error).__name__}: {error}"[:300]}
    line = {
        "impl": "reference", "metric": "uvu_conv_fwd_bwd_edges_per_s", "value": value, "unit": "edges/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * statistics.mean(r["seconds"] for r in rates),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f64" if dtype == torch.float64 else "f32", "data": "synthetic",
        "config": static_config(name, args.atoms_per_gpu, args.gpus),
        "note": "CPU restatement of the reference path on all host cores: the reference has no CPU implementation "
                "of the convolution",
        "cpu_baseline": dict(sample, value=value),
        "e2e": {"value": value, "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "reference_gpu": gpu,
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------- measurements


def time_steps(step, steps, warmup, marks, world, sampler=None):
    """Runs ``warmup`` untimed and ``steps`` timed calls of ``step(events)``; ``events`` is a list of ``marks`` CUDA
    events the step records in order.  Returns the ms per step over the whole timed region (max over ranks) and the
    mean of each interval between consecutive marks."""
    import torch.distributed as dist

    for _ in range(warmup):
        step(None)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    if sampler is not None:
        sampler.reset()
    events = [[torch.cuda.Event(enable_timing=True) for _ in range(marks)] for _ in range(steps)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for k in range(steps):
        step(events[k])
    stop.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    elapsed = torch.tensor([start.elapsed_time(stop)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    intervals = [statistics.mean(e[i].elapsed_time(e[i + 1]) for e in events) for i in range(marks - 1)]
    if os.environ.get("LUNA_BENCH_DEBUG"):
        print("DEBUG per-step intervals", [[round(e[i].elapsed_time(e[i + 1]), 2) for i in range(marks - 1)]
                                           for e in events], file=sys.stderr)
    return elapsed.item() / steps, intervals


class ConvWorkload:
    """One workload's tensors on this rank, the step that is timed, and its accounting."""

    def __init__(self, name, atoms, world, rank, device, generic=False, overlap=False):
        import lunaequivariance_b200 as luna
        from lunaequivariance_b200 import sharded

        self.name, self.world, self.rank, self.device = name, world, rank, device
        self.overlap = overlap
        in1, in2, out, instructions, dtype, default_atoms, kind, lmax = build_paths(name)
        self.atoms = atoms or default_atoms
        self.dtype, self.kind, self.lmax = dtype, kind, lmax
        self.module = luna.TensorProductConv(in1, in2, out, instructions, internal_weights=False,
                                             shared_weights=False, dtype=dtype)
        self.op = self.module.op
        if generic:
            self.op.force_generic(True)
        src, dst, vec = build_graph_edges(name, self.atoms, world, rank, device)

        def timed(fn):  # set-up steps that are not part of the timed step, reported on their own
            torch.cuda.synchronize()
            start = time.perf_counter()
            value = fn()
            torch.cuda.synchronize()
            return value, (time.perf_counter() - start) * 1e3

        sharded.make_graph_shard(src, dst, [self.atoms] * world, rank, group=None)  # first use: one-time set-up
        self.shard, self.graph_build_ms = timed(
            lambda: sharded.make_graph_shard(src, dst, [self.atoms] * world, rank, group=None))
        self.graph = self.shard.graph
        self.edges = self.graph.num_edges
        self.degrees = [1] if name == "cfg1" else list(range(lmax + 1))
        self.vec = vec.to(dtype)
        luna.spherical_harmonics(self.degrees, self.vec[:1024], True, "component")  # first-use set-up
        self.sh, self.edge_attr_ms = timed(
            lambda: luna.spherical_harmonics(self.degrees, self.vec, True, "component").contiguous())
        generator = torch.Generator(device=device).manual_seed(100 + rank)
        op = self.op
        self.x = torch.randn(self.atoms, op.in1_dim, device=device, dtype=dtype, generator=generator)
        self.w = torch.randn(self.edges, op.weight_numel, device=device, dtype=dtype, generator=generator)
        self.g = torch.randn(self.atoms, op.out_dim, device=device, dtype=dtype, generator=generator)
        torch.cuda.synchronize()

    def step(self, events):
        """exchange | forward | backward | return of the halo gradients; records 5 events."""
        from lunaequivariance_b200 import conv as conv_mod
        from lunaequivariance_b200 import sharded

        if self.world > 1 and self.overlap:
            # the exchanges run on a side stream behind the interior piece of the shard; the intervals are then
            # "enqueue", "forward pieces incl. any wait for the halo", "backward pieces", "wait + add of the returns"
            return sharded.overlapped_step(self.op, self.x, self.sh, self.w, self.g, self.shard, events=events)
        mark = (lambda i: events[i].record()) if events is not None else (lambda i: None)
        mark(0)
        x_full = sharded.exchange_halo(self.x, self.shard) if self.world > 1 else self.x
        mark(1)
        out = conv_mod.run_forward(self.op, x_full, self.sh, self.w, self.graph)
        mark(2)
        gx_full, gy, gw = conv_mod.run_backward(self.op, x_full, self.sh, self.w, self.g, self.graph)
        mark(3)
        gx = sharded.return_halo(gx_full, self.shard) if self.world > 1 else gx_full
        mark(4)
        return out, gx, gy, gw

    def force_step(self, events):
        """The force-training step through the public modules; records 2 events."""
        import lunaequivariance_b200 as luna

        if events is not None:
            events[0].record()
        w = self.w.detach().requires_grad_(True)
        vec = self.vec.detach().requires_grad_(True)
        harmonics = luna.spherical_harmonics(self.degrees, vec, True, "component")
        out = self.module(self.x, harmonics, w, graph=self.graph)
        energy = out.square().sum()
        (force,) = torch.autograd.grad(energy, vec, create_graph=True)
        loss = force.square().sum()
        (grad_w,) = torch.autograd.grad(loss, w)
        if events is not None:
            events[1].record()
        return grad_w

    def measure(self, steps, warmup, sampler=None):
        import torch.distributed as dist

        op = self.op
        S = 8 if self.dtype == torch.float64 else 4
        X, Y, O, W = op.in1_dim, op.in2_dim, op.out_dim, op.weight_numel
        peak, peak_kind = load_peaks()
        edges_total = torch.tensor([float(self.edges)], device=self.device, dtype=torch.float64)
        if self.world > 1:
            dist.all_reduce(edges_total, op=dist.ReduceOp.SUM)
        result = {"edges_rank0": self.edges, "edges_total": int(edges_total.item()),
                  "source_rows_rank0": self.graph.source_rows, "halo_rows_rank0": self.shard.halo_rows,
                  "kernels": "staged" if op.uses_staged_kernels else "table-driven",
                  "backward_variant": op.backward_variant,
                  # outside the timed step (built once per topology / per geometry), wall clock with a synchronise
                  "graph_build_ms": self.graph_build_ms, "edge_attr_harmonics_ms": self.edge_attr_ms}
        if self.name == "cfg3":
            ms, _ = time_steps(self.force_step, steps, warmup, 2, self.world, sampler)
            # minimum traffic of the step: three reads of the weights (forward, backward for gy, tangent forward)
            # and two weight-sized writes (the two terms of dL/dweight)
            step_bytes = 5 * self.edges * W * S
            gbs = step_bytes / (ms * 1e-3) / 1e9
            result.update(ms_per_step=ms, value=edges_total.item() / (ms * 1e-3),
                          roofline={"bound": "hbm", "kernel": "force step", "achieved": gbs, "peak": peak,
                                    "unit": "GB/s", "frac": gbs / peak, "peak_kind": peak_kind, "traffic": None,
                                    "algorithmic_bytes": step_bytes})
            return result
        ms, (gather_ms, fwd_ms, bwd_ms, return_ms) = time_steps(self.step, steps, warmup, 5, self.world, sampler)
        # a rank reads and writes the rows of its compact source buffer (owned + halo), not all gathered rows
        fwd_bytes, bwd_bytes = algorithmic_bytes(self.atoms, self.graph.source_rows, self.edges, X, Y, O, W, S)
        dominant = "backward" if bwd_ms >= fwd_ms else "forward"
        dom_bytes, dom_ms = (bwd_bytes, bwd_ms) if dominant == "backward" else (fwd_bytes, fwd_ms)
        achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
        step_gbs = (fwd_bytes + bwd_bytes) / ((fwd_ms + bwd_ms) * 1e-3) / 1e9
        variant = "staged" if dominant == "forward" else op.backward_variant
        per_edge = NCU_TRAFFIC_BYTES_PER_EDGE.get((self.name, dominant, variant)) if op.uses_staged_kernels else None
        result.update(
            ms_per_step=ms, value=edges_total.item() / (ms * 1e-3), collective_ms=gather_ms + return_ms,
            roofline={
                "bound": "hbm", "kernel": dominant, "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_kind": peak_kind,
                "traffic": None if per_edge is None else per_edge * self.edges,
                "traffic_note": "bytes per launch: ncu dram read + write of this kernel on this workload at 50,000 "
                                "atoms (profiles/), scaled by the edge count",
                "algorithmic_bytes": dom_bytes,
                "forward": {"ms": fwd_ms, "GB/s": fwd_bytes / (fwd_ms * 1e-3) / 1e9, "bytes": fwd_bytes},
                "backward": {"ms": bwd_ms, "GB/s": bwd_bytes / (bwd_ms * 1e-3) / 1e9, "bytes": bwd_bytes},
                "step_GB/s": step_gbs, "step_frac_of_peak": step_gbs / peak, "step_frac_of_8TBs": step_gbs / 8000.0,
            })
        return result


def measure_sh6(steps, warmup, device):
    """Spherical harmonics of 4 M unit vectors, degrees 0..6, FP32: forward, and forward + backward."""
    import bench_workloads as workloads
    import lunaequivariance_b200  # noqa: F401

    sh_mod = sys.modules["lunaequivariance_b200.spherical_harmonics"]
    dtype = torch.float32
    vec = workloads.random_unit_vectors(SH6_ITEMS, 3, device, dtype)
    config = sh_mod.SphericalHarmonicsConfig(tuple(range(7)), True, "component", dtype)
    g = torch.randn(SH6_ITEMS, 49, device=device, dtype=dtype)

    def fwd(events):
        if events is not None:
            events[0].record()
        sh_mod.run_forward(config, vec)
        if events is not None:
            events[1].record()

    def both(events):
        if events is not None:
            events[0].record()
        sh_mod.run_forward(config, vec)
        sh_mod.run_backward(config, vec, g)
        if events is not None:
            events[1].record()

    peak, peak_kind = load_peaks()
    fwd_ms, _ = time_steps(fwd, steps, warmup, 2, 1)
    both_ms, _ = time_steps(both, steps, warmup, 2, 1)
    fwd_bytes = SH6_ITEMS * (3 + 49) * 4
    both_bytes = fwd_bytes + SH6_ITEMS * (3 + 49 + 3) * 4
    fwd_gbs, both_gbs = fwd_bytes / (fwd_ms * 1e-3) / 1e9, both_bytes / (both_ms * 1e-3) / 1e9
    return {"items": SH6_ITEMS, "ms": both_ms, "forward_ms": fwd_ms, "forward_backward_ms": both_ms,
            "items_per_s_forward": SH6_ITEMS / (fwd_ms * 1e-3), "forward_GB/s": fwd_gbs, "forward_frac": fwd_gbs / peak,
            "GB/s": both_gbs, "frac": both_gbs / peak, "peak_kind": peak_kind,
            "algorithmic_bytes": {"forward": fwd_bytes, "forward_backward": both_bytes}}


def measure_cfg1_graph(device, steps=200):
    """The reference's CPU-runnable configuration (1,000 atoms, 16,000 edges, FP64): a step is launch-bound, so it is
    timed both as eager calls and as one captured CUDA graph replayed."""
    work = ConvWorkload("cfg1", None, 1, 0, device)

    def step():
        work.step(None)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            step()
    torch.cuda.current_stream().wait_stream(side)
    captured = torch.cuda.CUDAGraph()
    with torch.cuda.graph(captured):
        step()

    def timed(fn):
        for _ in range(10):
            fn()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / steps

    eager_ms, graph_ms = timed(step), timed(captured.replay)
    return {"edges": work.edges, "dtype": "f64", "eager_ms": eager_ms, "cuda_graph_ms": graph_ms,
            "edges_per_s_eager": work.edges / (eager_ms * 1e-3), "edges_per_s_cuda_graph": work.edges / (graph_ms * 1e-3),
            "step": "forward + backward (gx, gy, gw), " + str(steps) + " back-to-back steps"}


def fma_peaks(device):
    """Register-resident FMA chains: the packed-FP32 and the FP64 arithmetic peaks of this GPU, measured."""
    import ctypes

    from lunaequivariance_b200 import _native

    lib = _native.library()
    result = {}
    for kind, name in ((0, "f32x2"), (1, "f64")):
        flops = ctypes.c_double(0.0)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sink = torch.zeros(1 << 16, device=device, dtype=torch.float64)
        stream = _native.current_stream(device)
        _native.check(lib.luna_probe_fma(kind, 1 << 10, sink.data_ptr(), ctypes.byref(flops), stream))  # warm-up
        torch.cuda.synchronize()
        start.record()
        _native.check(lib.luna_probe_fma(kind, 1 << 14, sink.data_ptr(), ctypes.byref(flops), stream))
        stop.record()
        torch.cuda.synchronize()
        result[name + "_tflops"] = flops.value / (start.elapsed_time(stop) * 1e-3) / 1e12
    return result


def secondary_roofline(name, measurement, peaks):
    """Arithmetic bound next to the HBM bound: algorithmic FLOPs over the measured FMA peak of the workload's dtype."""
    per_edge = FORWARD_FLOPS_PER_EDGE.get(name)
    if per_edge is None or peaks is None:
        return None
    dtype_peak = peaks["f64_tflops"] if WORKLOADS[name][3] == torch.float64 else peaks["f32x2_tflops"]
    edges = measurement["edges_rank0"]
    if name == "cfg3":
        # forward, backward for gy, tangent forward (each one contraction) and two weight-gradient contractions
        flops, seconds, what = 5 * per_edge * edges, measurement["ms_per_step"] * 1e-3, "five contractions of the step"
    else:
        roof = measurement["roofline"]
        flops, seconds = 4 * per_edge * edges, (roof["forward"]["ms"] + roof["backward"]["ms"]) * 1e-3
        what = "forward plus the backward's three outputs"
    return {"bound": "fma", "achieved": flops / seconds / 1e12, "peak": dtype_peak, "unit": "TFLOP/s",
            "frac": flops / seconds / 1e12 / dtype_peak, "flops_per_edge_forward": per_edge,
            "note": f"algorithmic FLOPs ({what}) over the measured register-resident FMA peak"}


def sharded_parity(world, rank, device):
    """A small partitioned problem on all ranks against the same problem unpartitioned on every rank's own GPU."""
    import torch.distributed as dist

    import bench_workloads as workloads
    import lunaequivariance_b200 as luna
    from lunaequivariance_b200 import sharded

    in1, in2, out, instructions, dtype, _, _, lmax = build_paths("cfg5")
    module = luna.TensorProductConv(in1, in2, out, instructions, internal_weights=False, shared_weights=False,
                                    dtype=dtype)
    op = module.op
    atoms = 600 * world
    pos, box, cells = workloads.periodic_positions(atoms, DENSITY, 0, device, CUTOFF)
    src, dst, vec = workloads.radius_graph_periodic(pos, box, CUTOFF, cells)
    generator = torch.Generator(device=device).manual_seed(17)  # same seed on every rank: same global problem
    rand = lambda *shape: torch.randn(*shape, device=device, dtype=dtype, generator=generator)
    edges = src.numel()
    y = luna.spherical_harmonics(list(range(lmax + 1)), vec.to(dtype), True, "component")
    x, w, g = rand(atoms, op.in1_dim), rand(edges, op.weight_numel), rand(atoms, op.out_dim)
    # uneven destination ranges, balanced by edge count
    rowptr = torch.zeros(atoms + 1, dtype=torch.int64, device=device)
    rowptr[1:] = torch.bincount(dst, minlength=atoms).cumsum(0)
    ranges = sharded.balanced_node_ranges(rowptr, world)
    counts = [b - a for a, b in ranges]
    begin, end = ranges[rank]
    mine = (dst >= begin) & (dst < end)
    shard = sharded.make_graph_shard(src[mine], dst[mine], counts, rank, group=None)
    xl = x[begin:end].clone().requires_grad_(True)
    yl, wl = y[mine].clone().requires_grad_(True), w[mine].clone().requires_grad_(True)
    out_local = sharded.sharded_conv(module, xl, yl, wl, shard)
    gx, gy, gw = torch.autograd.grad(out_local, (xl, yl, wl), g[begin:end])
    graph = module.create_graph(src, dst, atoms)
    xf, yf, wf = (t.clone().requires_grad_(True) for t in (x, y, w))
    full = module(xf, yf, wf, graph=graph)
    fx, fy, fw = torch.autograd.grad(full, (xf, yf, wf), g)
    # the same step with both exchanges hidden behind the interior piece (what the timed loop runs)
    o_out, o_gx, o_gy, o_gw = sharded.overlapped_step(op, x[begin:end].contiguous(), y[mine].contiguous(),
                                                      w[mine].contiguous(), g[begin:end].contiguous(), shard)
    worst = torch.zeros(1, device=device, dtype=torch.float64)
    for mine_t, ref_t in ((out_local, full[begin:end]), (gx, fx[begin:end]), (gy, fy[mine]), (gw, fw[mine]),
                          (o_out, full[begin:end]), (o_gx, fx[begin:end]), (o_gy, fy[mine]), (o_gw, fw[mine])):
        scale = ref_t.abs().max().clamp_min(1e-30)
        worst = torch.maximum(worst, ((mine_t - ref_t).abs().max() / scale).double().reshape(1))
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    return {"max_rel_err": worst.item(), "ok": bool(worst.item() <= 1e-5), "atoms": atoms, "edges": edges,
            "interior_rank0": list(shard.interior),
            "what": "cfg5 irreps, uneven destination ranges: out, gx (after the halo return), gy, gw of every rank, "
                    "from the autograd path and from the overlapped step, against the unpartitioned run of the same "
                    "problem"}


# ------------------------------------------------------------------------------------------------- native arm


def measure_others(world, rank, device, main_name, peaks, overlap=False):
    """Brief measurements of the workloads that are not the headline, so that one run records them all."""
    others = {}
    if world == 1:
        for other in ("cfg3", "cfg4", "cfg5"):
            if other == main_name:
                continue
            try:
                work = ConvWorkload(other, None, 1, 0, device)
                m = work.measure(3, 3)
                work.op.check_status(device)
                roof = m["roofline"]
                entry = {"ms": m["ms_per_step"], "edges": m["edges_rank0"], "edges_per_s": m["value"],
                         "GB/s": roof["achieved"], "frac": roof["frac"], "kernel": roof["kernel"],
                         "backward_variant": m["backward_variant"],
                         "dtype": "f64" if work.dtype == torch.float64 else "f32",
                         "secondary": secondary_roofline(other, m, peaks), "config": static_config(other, None, 1)}
                if "forward" in roof:
                    entry.update(forward_ms=roof["forward"]["ms"], backward_ms=roof["backward"]["ms"],
                                 step_frac=roof["step_frac_of_peak"])
                others[other] = entry
                del work
            except Exception as error:  # an entry that cannot run must not take the headline down
                others[other] = {"error": f"{type(error).__name__}: {error}"[:300]}
            torch.cuda.empty_cache()
        try:
            others["sh6"] = measure_sh6(5, 3, device)
        except Exception as error:
            others["sh6"] = {"error": f"{type(error).__name__}: {error}"[:300]}
        try:
            others["cfg1"] = measure_cfg1_graph(device)
        except Exception as error:
            others["cfg1"] = {"error": f"{type(error).__name__}: {error}"[:300]}
    elif main_name != "cfg5":
        try:  # the partitioned configuration itself: 250,000 atoms per GPU
            work = ConvWorkload("cfg5", None, world, rank, device, overlap=overlap)
            m = work.measure(3, 3)
            others["cfg5"] = {"ms": m["ms_per_step"], "edges_total": m["edges_total"], "edges_per_s": m["value"],
                              "collective_ms": m["collective_ms"], "forward_ms": m["roofline"]["forward"]["ms"],
                              "backward_ms": m["roofline"]["backward"]["ms"],
                              "halo_rows_rank0": m["halo_rows_rank0"], "config": static_config("cfg5", None, world)}
            del work
        except Exception as error:
            others["cfg5"] = {"error": f"{type(error).__name__}: {error}"[:300]}
        torch.cuda.empty_cache()
    return others


def main():
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    # the clock sampler starts before the warm-up: the first nvidia-smi query can stall the device for milliseconds
    sampler = ClockSampler(device) if rank == 0 else None
    parity = sharded_parity(world, rank, device) if world > 1 else None

    if args.workload == "sh6":
        sh = measure_sh6(args.steps, args.warmup, device)
        clocks = sampler.stop() if sampler else None
        if rank == 0:
            print(json.dumps({
                "metric": "spherical_harmonics_items_per_s", "value": sh["items_per_s_forward"] * world,
                "unit": "items/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": sh["forward_ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic", "config": static_config("sh6", None, world),
                "roofline": {"bound": "hbm", "achieved": sh["forward_GB/s"], "peak": load_peaks()[0], "unit": "GB/s",
                             "frac": sh["forward_frac"], "traffic": None}, "details": sh, "clocks": clocks,
                "gpu_launches": args.steps}))
        if world > 1:
            dist.destroy_process_group()
        return

    work = ConvWorkload(args.workload, args.atoms_per_gpu, world, rank, device, args.generic,
                        overlap=args.overlap)
    result = work.measure(args.steps, args.warmup, sampler)
    clocks = sampler.stop() if sampler else None
    op_status = None
    try:
        work.op.check_status(device)
    except RuntimeError as error:  # a bounded device wait gave up: the numbers are invalid
        op_status = str(error)
    e2e = None if args.skip_e2e else measure_e2e(args, work, world, device)
    staged, dtype, name = work.op.uses_staged_kernels, work.dtype, work.name
    lo, hi = work.shard.interior
    pieces = sum(1 for b, e in ((0, lo), (lo, hi), (hi, work.shard.local_nodes)) if e > b)
    del work
    torch.cuda.empty_cache()

    peaks = others = None
    if not args.skip_others:
        if world == 1:
            peaks = fma_peaks(device)
        others = measure_others(world, rank, device, name, peaks, overlap=args.overlap)
    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu:
        cpu = cpu_sample_rate(name, args.cpu_seconds, args.atoms_per_gpu)

    if rank == 0:
        # kernels of this library per step: forward + backward (+ the harmonics and second-order launches of cfg3)
        # (a partitioned step with overlap runs forward and backward as up to three pieces each)
        launches_per_step = 9 if name == "cfg3" else (2 if staged else 4)
        if world > 1 and args.overlap and name != "cfg3":
            launches_per_step *= pieces
        line = {
            "metric": "uvu_conv_fwd_bwd_edges_per_s", "value": result["value"], "unit": "edges/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": result["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f64" if dtype == torch.float64 else "f32", "data": "synthetic",
            "config": static_config(name, args.atoms_per_gpu, world),
            "graph": {k: result[k] for k in ("edges_rank0", "edges_total", "source_rows_rank0", "halo_rows_rank0",
                                             "kernels", "backward_variant", "graph_build_ms",
                                             "edge_attr_harmonics_ms")},
            "roofline": dict(result["roofline"], secondary=secondary_roofline(name, result, peaks)),
            "fma_peaks": peaks, "collective_ms": result.get("collective_ms"), "parity": parity,
            "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks, "others": others,
            "gpu_launches": args.steps * launches_per_step, "device_status": op_status,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def measure_e2e(args, work, world, device):
    """Same step with the inputs in pinned host memory: H2D of x, edge_attr, weight and the cotangent, D2H of out, gx,
    gy, gw, every step, through the library's host-streaming executor (``HostStreamedConv``): the per-edge tensors
    cross PCIe chunk by chunk, uploads, kernels and downloads overlapping.  On a partitioned graph the node features
    take the usual halo exchange on the device."""
    import torch.distributed as dist

    from lunaequivariance_b200 import sharded
    from lunaequivariance_b200.streaming import HostStreamedConv

    module, shard = work.module, work.shard

    def pinned(t):
        try:
            host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        except RuntimeError:
            host = torch.empty(t.shape, dtype=t.dtype)
        host.copy_(t)
        return host

    host_in = [pinned(t) for t in (work.x, work.sh, work.w, work.g)]
    E = work.edges
    streamed = HostStreamedConv(module.op, shard.graph, chunks=args.e2e_chunks)
    host_gx = pinned(work.x)
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    work.w = work.g = None  # the step owns its device copies
    torch.cuda.empty_cache()
    d2h = 0

    def one():
        nonlocal d2h
        x_host, y_host, w_host, g_host = host_in
        if world > 1:
            x_full = sharded.exchange_halo(x_host.to(device, non_blocking=True), shard)
            out, gx_full, gy, gw = streamed.step(x_full, y_host, w_host, g_host)
            host_gx.copy_(sharded.return_halo(gx_full, shard), non_blocking=True)
            torch.cuda.current_stream().synchronize()
            gx = host_gx
        else:
            out, gx, gy, gw = streamed.step(x_host, y_host, w_host, g_host)
        d2h = sum(t.numel() * t.element_size() for t in (out, gx, gy, gw))

    one()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        one()
    torch.cuda.synchronize()
    elapsed = torch.tensor([time.perf_counter() - t0], device=device, dtype=torch.float64)
    edges = torch.tensor([float(E)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        dist.all_reduce(edges, op=dist.ReduceOp.SUM)
    return {"value": edges.item() * args.e2e_steps / elapsed.item(), "unit": "edges/s",
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": args.e2e_steps,
            "pinned": bool(host_in[2].is_pinned()), "api": "HostStreamedConv.step",
            "chunks": len(streamed.pieces)}


if __name__ == "__main__":
    main()
