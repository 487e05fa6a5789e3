"""Benchmark of the UVU TensorProductConv hot path: forward + backward edges/s and HBM roofline fraction.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2|cfg5|cfg4|cfg1] [--impl reference]

One "step" is one forward plus one backward (gx, gy, gw) of the convolution over the whole synthetic graph.
With N > 1 (launched by torchrun, one rank per GPU) the graph has N times as many atoms, destination ranges are
assigned to ranks (weak scaling), source features are all-gathered and gx is reduce-scattered inside the step.
Rank 0 prints one JSON line.  ``--impl reference`` times the CPU restatement of the reference's path (the
reference itself has no CPU implementation of the convolution and cannot run its generated CUDA here) on host
cores instead.
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

WORKLOADS = {
    # name: (irreps_in1, sh lmax, irreps_out, dtype, atoms per GPU, graph kind)
    "cfg2": ("128x0e+128x1o+128x2e", 3, "128x0e+128x1o+128x2e+128x3o", torch.float32, 50_000, "radius"),
    "cfg5": ("64x0e+64x1o+64x2e", 2, "64x0e+64x1o+64x2e", torch.float32, 250_000, "radius"),
    "cfg4": ("64x0e+64x1o+64x2e+64x3o", 3, "64x0e+64x1o+64x2e+64x3o", torch.float32, 100_000, "degree40"),
    "cfg1": ("32x1o", 1, "32x0e", torch.float64, 1_000, "degree16"),
    "lmax1": ("128x0e+128x1o", 1, "128x0e+128x1o", torch.float32, 100_000, "radius"),
}
DENSITY, CUTOFF = 0.1, 5.0
# DRAM traffic per edge (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture, divided by the edges of
# the captured launch) for the staged kernels; the captures ran a smaller graph of the same workload (12,000 atoms,
# larger than L2) and traffic grows with the edge count, so bench scales it to its own launch.
NCU_TRAFFIC_BYTES_PER_EDGE = {"cfg2": {"forward": 11.51e3, "backward": 22.32e3}}


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="native", choices=["native", "reference"])
    p.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    p.add_argument("--atoms-per-gpu", type=int, default=None)
    p.add_argument("--e2e-steps", type=int, default=2)
    p.add_argument("--skip-e2e", action="store_true")
    p.add_argument("--skip-cpu", action="store_true")
    p.add_argument("--cpu-seconds", type=float, default=15.0)
    p.add_argument("--generic", action="store_true", help="force the table-driven kernels")
    return p.parse_args()


# ------------------------------------------------------------------------------------------------- workload


def irreps_of(name):
    in1, lmax, out, dtype, atoms, kind = WORKLOADS[name]
    in2 = "+".join(f"1x{l}{'e' if l % 2 == 0 else 'o'}" for l in range(lmax + 1))
    if name == "cfg1":
        in2 = "1x1o"
    return in1, in2, out, dtype, atoms, kind, lmax


def build_paths(name):
    import bench_workloads as workloads

    in1, in2, out, dtype, atoms, kind, lmax = irreps_of(name)
    instructions = [(0, 0, 0, "uvu", True)] if name == "cfg1" else workloads.all_uvu_instructions(in1, in2, out)
    return in1, in2, out, instructions, dtype, atoms, kind, lmax


def build_graph_edges(name, atoms_per_gpu, world, rank, device):
    """This rank's destination-sorted edge slice (global ids) and unit edge vectors."""
    import bench_workloads as workloads

    kind = WORKLOADS[name][5]
    total = atoms_per_gpu * world
    begin, end = rank * atoms_per_gpu, (rank + 1) * atoms_per_gpu
    if kind == "radius":
        pos, box, cells = workloads.periodic_positions(total, DENSITY, 0, device, CUTOFF)
        src, dst, vec = workloads.radius_graph_periodic(pos, box, CUTOFF, cells, begin, end)
        return src, dst, vec
    degree = 40 if kind == "degree40" else 16
    src, dst = workloads.fixed_degree_graph(total, degree, 0, device)
    mine = (dst >= begin) & (dst < end)
    src, dst = src[mine], dst[mine]
    vec = workloads.random_unit_vectors(src.numel(), 1 + rank, device)
    return src, dst, vec


def algorithmic_bytes(n_dst, n_src, edges, X, Y, O, W, S):
    """Bytes that must cross HBM once per pass: forward and backward (gx, gy, gw)."""
    fwd = edges * (W + Y) * S + 4 * edges + 4 * (n_dst + 1) + n_src * X * S + n_dst * O * S
    bwd = 2 * edges * (W + Y) * S + n_src * X * S + n_dst * O * S + n_src * X * S + 12 * edges
    return fwd, bwd


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


def cpu_sample_rate(name, seconds, threads=None):
    """Edges/s of the CPU restatement (oracle) for forward + backward on a bounded sample of the workload."""
    from oracle import uvu_conv as oracle_conv
    from oracle import spherical_harmonics as oracle_sh

    in1, in2, out, instructions, dtype, atoms, kind, lmax = build_paths(name)
    if threads:
        torch.set_num_threads(threads)
    meta = oracle_conv.build_specs(in1, in2, out, instructions)
    generator = torch.Generator().manual_seed(0)
    degree = {"radius": 52, "degree40": 40, "degree16": 16}[kind]
    nodes_total = min(atoms, 20_000)

    def run(sample_nodes):
        edges = sample_nodes * degree
        dst = torch.arange(sample_nodes).repeat_interleave(degree)
        src = torch.randint(nodes_total, (edges,), generator=generator)
        x = torch.randn(nodes_total, meta["in1_dim"], generator=generator, dtype=dtype)
        vec = torch.nn.functional.normalize(torch.randn(edges, 3, generator=generator, dtype=dtype), dim=-1)
        degrees = (1,) if name == "cfg1" else tuple(range(lmax + 1))
        y = oracle_sh.spherical_harmonics(degrees, vec, True, "component")
        w = torch.randn(edges, meta["weight_numel"], generator=generator, dtype=dtype)
        g = torch.randn(sample_nodes, meta["out_dim"], generator=generator, dtype=dtype)
        t0 = time.perf_counter()
        oracle_conv.conv_forward_backward_chunked(meta, x, y, w, g, src, dst, sample_nodes, chunk_edges=8192)
        return edges, time.perf_counter() - t0

    run(8)  # warm-up (thread pools, allocator)
    edges, elapsed = run(32)
    rate = edges / elapsed
    sample_nodes = int(max(32, min(atoms, rate * seconds / degree)))
    edges, elapsed = run(sample_nodes)
    return dict(value=edges / elapsed, unit="edges/s", cores=torch.get_num_threads(), kind="port", seconds=elapsed,
                sample=f"{sample_nodes} destination nodes x {degree} incoming edges ({edges} edges) of {name}, "
                       f"forward+backward in {dtype}, {elapsed:.1f} s")


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    in1, in2, out, instructions, dtype, atoms, kind, lmax = build_paths(args.workload)
    rates = []
    for step in range(args.warmup + args.steps):
        result = cpu_sample_rate(args.workload, max(2.0, args.cpu_seconds / 3))
        if step >= args.warmup:
            rates.append(result)
    value = statistics.mean(r["value"] for r in rates)
    sample = rates[-1]
    line = {
        "impl": "reference", "metric": "uvu_conv_fwd_bwd_edges_per_s", "value": value, "unit": "edges/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * statistics.mean(r["seconds"] for r in rates),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f64" if dtype == torch.float64 else "f32", "data": "synthetic",
        "config": {"workload": args.workload, "irreps_in1": in1, "irreps_in2": in2, "irreps_out": out,
                   "note": "CPU restatement of the reference path (the reference has no CPU implementation of "
                           "the convolution and its generated CUDA needs a JIT build on a GPU)"},
        "cpu_baseline": dict(sample, value=value),
        "e2e": {"value": value, "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------- native arm


def main():
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    import torch.distributed as dist

    import lunaequivariance_b200 as luna
    from lunaequivariance_b200 import conv as conv_mod
    from lunaequivariance_b200 import sharded

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    in1, in2, out, instructions, dtype, atoms, kind, lmax = build_paths(args.workload)
    atoms = args.atoms_per_gpu or atoms
    module = luna.TensorProductConv(in1, in2, out, instructions, internal_weights=False, shared_weights=False,
                                    dtype=dtype)
    op = module.op
    if args.generic:
        op.force_generic(True)
    X, Y, O, W = op.in1_dim, op.in2_dim, op.out_dim, op.weight_numel
    S = 8 if dtype == torch.float64 else 4

    src, dst, vec = build_graph_edges(args.workload, atoms, world, rank, device)
    counts = [atoms] * world
    shard = sharded.make_graph_shard(src, dst, counts, rank, group=None)
    graph = shard.graph
    E = graph.num_edges
    degrees = [1] if args.workload == "cfg1" else list(range(lmax + 1))
    sh = luna.spherical_harmonics(degrees, vec.to(dtype), True, "component").contiguous()
    del vec, src, dst
    generator = torch.Generator(device=device).manual_seed(100 + rank)
    x_local = torch.randn(atoms, X, device=device, dtype=dtype, generator=generator)
    w = torch.randn(E, W, device=device, dtype=dtype, generator=generator)
    g = torch.randn(atoms, O, device=device, dtype=dtype, generator=generator)
    torch.cuda.synchronize()

    def step(record=None):
        x_full = sharded.gather_sources(x_local, shard) if world > 1 else x_local
        if record is not None:
            record[0].record()
        result = conv_mod.run_forward(op, x_full, sh, w, graph)
        if record is not None:
            record[1].record()
        gx_full, gy, gw = conv_mod.run_backward(op, x_full, sh, w, g, graph)
        if record is not None:
            record[2].record()
        if world > 1:
            gx_full = sharded._reduce_scatter_rows(gx_full, world, None)[:atoms]
        return result, gx_full, gy, gw

    # the clock sampler starts before the warm-up: the first nvidia-smi query can stall the device for milliseconds
    sampler = ClockSampler(device) if rank == 0 else None
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    if sampler is not None:
        sampler.reset()
    events = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for k in range(args.steps):
        outputs = step(events[k])
    stop.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop() if sampler else None
    elapsed_ms = torch.tensor([start.elapsed_time(stop)], device=device, dtype=torch.float64)
    edges_total = torch.tensor([float(E)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(elapsed_ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(edges_total, op=dist.ReduceOp.SUM)
    ms_per_step = elapsed_ms.item() / args.steps
    value = edges_total.item() / (ms_per_step * 1e-3)
    op_status = None
    try:
        luna._native.check(luna._native.library().luna_uvu_check_status(op._plan.handle, None))
    except RuntimeError as error:  # a bounded device wait gave up: the numbers are invalid
        op_status = str(error)

    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in events)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in events)
    fwd_bytes, bwd_bytes = algorithmic_bytes(atoms, graph.source_rows, E, X, Y, O, W, S)
    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as handle:
            peaks = json.load(handle)
    except OSError:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_kind = "measured" if "hbm_gbs" in peaks else "fallback"
    staged = op.uses_staged_kernels and not args.generic
    dominant = "backward" if bwd_ms >= fwd_ms else "forward"
    dom_bytes, dom_ms = (bwd_bytes, bwd_ms) if dominant == "backward" else (fwd_bytes, fwd_ms)
    achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
    step_gbs = (fwd_bytes + bwd_bytes) / ((fwd_ms + bwd_ms) * 1e-3) / 1e9
    per_edge = NCU_TRAFFIC_BYTES_PER_EDGE.get(args.workload, {}).get(dominant) if staged else None
    roofline = {
        "bound": "hbm", "kernel": dominant, "achieved": achieved, "peak": peak, "unit": "GB/s",
        "frac": achieved / peak, "peak_kind": peak_kind,
        "traffic": None if per_edge is None else per_edge * E,
        "traffic_note": "bytes per launch, scaled by edges from an ncu capture of a 12,000-atom case",
        "algorithmic_bytes": dom_bytes,
        "forward": {"ms": fwd_ms, "GB/s": fwd_bytes / (fwd_ms * 1e-3) / 1e9, "bytes": fwd_bytes},
        "backward": {"ms": bwd_ms, "GB/s": bwd_bytes / (bwd_ms * 1e-3) / 1e9, "bytes": bwd_bytes},
        "step_GB/s": step_gbs, "step_frac_of_peak": step_gbs / peak, "step_frac_of_8TBs": step_gbs / 8000.0,
    }

    # ---- end to end through the public module with host buffers
    e2e = None
    if not args.skip_e2e:
        e2e = measure_e2e(args, module, shard, x_local, sh, w, g, world, atoms, device)
    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu:
        cpu = cpu_sample_rate(args.workload, args.cpu_seconds)

    if rank == 0:
        line = {
            "metric": "uvu_conv_fwd_bwd_edges_per_s", "value": value, "unit": "edges/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f64" if dtype == torch.float64 else "f32",
            "data": "synthetic",
            "config": {
                "workload": args.workload, "irreps_in1": in1, "irreps_in2": in2, "irreps_out": out,
                "paths": len(instructions), "weight_numel": W, "atoms_per_gpu": atoms, "edges_rank0": E,
                "edges_total": int(edges_total.item()), "graph": kind, "density": DENSITY, "cutoff": CUTOFF,
                "atom_order": "cell (spatial) order", "parallelism": f"dst-range x{world}",
                "cache": "inputs larger than L2 (per-edge weights alone are %.1f GB)" % (E * W * S / 1e9),
                "kernels": "staged" if staged else "table-driven",
            },
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks,
            "gpu_launches": args.steps * ((1 + (1 if staged else 3))),
            "device_status": op_status,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def measure_e2e(args, module, shard, x_local, sh, w, g, world, atoms, device):
    """Same step through TensorProductConv + autograd with pinned host buffers: H2D of x, edge_attr, weight and
    the cotangent, D2H of out, gx, gy, gw, every step."""
    import torch.distributed as dist

    from lunaequivariance_b200 import sharded

    def pinned(t):
        try:
            host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        except RuntimeError:
            host = torch.empty(t.shape, dtype=t.dtype)
        host.copy_(t)
        return host

    host_in = [pinned(t) for t in (x_local, sh, w, g)]
    E = w.shape[0]
    out_shapes = [(atoms, module.op.out_dim), tuple(x_local.shape), tuple(sh.shape), tuple(w.shape)]
    try:
        host_out = [torch.empty(s, dtype=w.dtype, pin_memory=True) for s in out_shapes]
    except RuntimeError:
        host_out = [torch.empty(s, dtype=w.dtype) for s in out_shapes]
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = sum(t.numel() * t.element_size() for t in host_out)
    del w, g  # the step owns its device copies
    torch.cuda.empty_cache()

    def one():
        xd, yd, wd, gd = (t.to(device, non_blocking=True) for t in host_in)
        xd.requires_grad_(True)
        yd.requires_grad_(True)
        wd.requires_grad_(True)
        result = sharded.sharded_conv(module, xd, yd, wd, shard) if world > 1 else module(xd, yd, wd, graph=shard.graph)
        grads = torch.autograd.grad(result, (xd, yd, wd), gd)
        for host, dev in zip(host_out, (result.detach(), *grads)):
            host.copy_(dev, non_blocking=True)
        torch.cuda.current_stream().synchronize()

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
            "pinned": bool(host_in[2].is_pinned())}


if __name__ == "__main__":
    main()
