"""Parity at the benchmark's full sizes: the CUDA path runs the whole graph, the CPU oracle checks a seeded sample.

The oracle cannot evaluate millions of edges, but every output row depends on few of them: an output row on the
in-edges of its node, a row of gx on the out-edges of its node, a row of gy or gw on its own edge.  So the oracle is
run on exactly those edges (renumbered into a small problem) for 64 sampled destination rows, 64 sampled source rows
and 4,096 sampled edges, and compared with the matching rows of the full-size result.  The force-training step
decomposes by destination node in the same way (the energy is a sum over nodes of a function of the node's in-edges).
Tolerances: 1e-5 (FP32) and 1e-12 (FP64) of the tensor's largest magnitude.
"""

import pytest
import torch

import bench_workloads as workloads
import lunaequivariance_b200 as luna
from lunaequivariance_b200 import conv as conv_mod
from oracle import spherical_harmonics as oracle_sh
from oracle import uvu_conv as oracle_conv
from tests.helpers import EdgeSample, assert_rows_close, in_edges_of, out_edges_of

pytestmark = pytest.mark.gpu
DEVICE = "cuda"


def build_problem(name, atoms=None):
    torch.cuda.empty_cache()  # these cases hold tens of GB: start from an unfragmented pool
    in1, in2, out, instructions, dtype, default_atoms, kind, lmax = workloads.build_paths(name)
    atoms = atoms or default_atoms
    module = luna.TensorProductConv(in1, in2, out, instructions, internal_weights=False, shared_weights=False,
                                    dtype=dtype)
    meta = oracle_conv.build_specs(in1, in2, out, instructions)
    src, dst, vec = workloads.build_graph_edges(name, atoms, 1, 0, DEVICE)
    graph = module.create_graph(src, dst, atoms)
    return module, meta, graph, vec, dtype, atoms, lmax


def first_order_case(name, atoms=None):
    module, meta, graph, vec, dtype, atoms, lmax = build_problem(name, atoms)
    op = module.op
    assert op.uses_staged_kernels
    edges = graph.num_edges
    generator = torch.Generator(device=DEVICE).manual_seed(11)
    rand = lambda *shape: torch.randn(*shape, device=DEVICE, dtype=dtype, generator=generator)
    y = luna.spherical_harmonics(list(range(lmax + 1)), vec.to(dtype), True, "component").contiguous()
    x, w, g = rand(atoms, op.in1_dim), rand(edges, op.weight_numel), rand(atoms, op.out_dim)
    out = conv_mod.run_forward(op, x, y, w, graph)
    gx, gy, gw = conv_mod.run_backward(op, x, y, w, g, graph)
    op.check_status()
    scales = {k: v.abs().max().item() for k, v in dict(out=out, gx=gx, gy=gy, gw=gw).items()}

    pick = torch.Generator(device=DEVICE).manual_seed(5)
    # 64 destination rows of out, each from exactly its in-edges
    rows = torch.randperm(atoms, device=DEVICE, generator=pick)[:64].sort()[0]
    sample = EdgeSample(graph.src, graph.dst, in_edges_of(graph.dst_rowptr, rows))
    ref = oracle_conv.conv_forward(meta, sample.take_sources(x), sample.take_edges(y), sample.take_edges(w),
                                   sample.cpu_src, sample.cpu_dst, sample.dst_nodes.numel())
    assert_rows_close(out[sample.dst_nodes], ref, scales["out"], dtype, f"{name} out rows")
    # 64 source rows of gx, each from exactly its out-edges
    rows = torch.randperm(atoms, device=DEVICE, generator=pick)[:64].sort()[0]
    sample = EdgeSample(graph.src, graph.dst, out_edges_of(graph.src_rowptr, graph.edge_ids_by_src, rows))
    ref = oracle_conv.conv_derivatives(meta, sample.take_sources(x), sample.take_edges(y), sample.take_edges(w),
                                       sample.cpu_src, sample.cpu_dst, sample.dst_nodes.numel(),
                                       sample.take_destinations(g))
    assert_rows_close(gx[sample.src_nodes], ref["gx"], scales["gx"], dtype, f"{name} gx rows")
    # 4,096 edges of gy and gw
    ids = torch.randperm(edges, device=DEVICE, generator=pick)[:4096].sort()[0]
    sample = EdgeSample(graph.src, graph.dst, ids)
    ref = oracle_conv.conv_derivatives(meta, sample.take_sources(x), sample.take_edges(y), sample.take_edges(w),
                                       sample.cpu_src, sample.cpu_dst, sample.dst_nodes.numel(),
                                       sample.take_destinations(g))
    assert_rows_close(gy[ids], ref["gy"], scales["gy"], dtype, f"{name} gy rows")
    assert_rows_close(gw[ids], ref["gw"], scales["gw"], dtype, f"{name} gw rows")


def test_config2_full_size_forward_backward():
    """50,000 atoms, 0.1 / A^3, 5 A cutoff (about 2.6 M edges), FP32: several waves, e * W beyond 2^31 elements."""
    first_order_case("cfg2")


def test_config4_full_size_forward_backward():
    """100,000 nodes x 40 random incoming edges (4 M edges), FP32, 64 channels, degrees to 3."""
    first_order_case("cfg4")


def test_config5_share_forward_backward():
    """One GPU's share of the partitioned run: 250,000 atoms (about 13 M edges), FP32, degrees to 2."""
    first_order_case("cfg5")


def test_config3_force_training_step():
    """20,000 atoms, FP64, harmonics inside the differentiated graph: energy = sum(out^2), forces = -dE/dvec,
    loss = sum(forces^2), then dL/dweight; forces and dL/dweight rows of sampled nodes against the oracle."""
    module, meta, graph, vec, dtype, atoms, lmax = build_problem("cfg3")
    op = module.op
    edges = graph.num_edges
    generator = torch.Generator(device=DEVICE).manual_seed(13)
    x = torch.randn(atoms, op.in1_dim, device=DEVICE, dtype=dtype, generator=generator)
    w = torch.randn(edges, op.weight_numel, device=DEVICE, dtype=dtype, generator=generator).requires_grad_(True)
    vec = vec.to(dtype).requires_grad_(True)
    harmonics = luna.SphericalHarmonics(list(range(lmax + 1)), True, "component", dtype=dtype)
    out = module(x, harmonics(vec), w, graph=graph)
    energy = out.square().sum()
    (force,) = torch.autograd.grad(energy, vec, create_graph=True)
    force = -force
    loss = force.square().sum()
    (grad_w,) = torch.autograd.grad(loss, w)
    op.check_status()
    scales = dict(out=out.abs().max().item(), force=force.abs().max().item(), grad_w=grad_w.abs().max().item())

    pick = torch.Generator(device=DEVICE).manual_seed(7)
    rows = torch.randperm(atoms, device=DEVICE, generator=pick)[:24].sort()[0]
    sample = EdgeSample(graph.src, graph.dst, in_edges_of(graph.dst_rowptr, rows))
    xs = sample.take_sources(x)
    ws = sample.take_edges(w).requires_grad_(True)
    vs = sample.take_edges(vec).requires_grad_(True)
    ys = oracle_sh.spherical_harmonics(tuple(range(lmax + 1)), vs, True, "component")
    ref_out = oracle_conv.conv_forward(meta, xs, ys, ws, sample.cpu_src, sample.cpu_dst, sample.dst_nodes.numel())
    (ref_force,) = torch.autograd.grad(ref_out.square().sum(), vs, create_graph=True)
    ref_force = -ref_force
    (ref_grad_w,) = torch.autograd.grad(ref_force.square().sum(), ws)
    assert_rows_close(out[sample.dst_nodes], ref_out.detach(), scales["out"], dtype, "cfg3 out rows")
    assert_rows_close(force[sample.edge_ids], ref_force.detach(), scales["force"], dtype, "cfg3 forces")
    assert_rows_close(grad_w[sample.edge_ids], ref_grad_w, scales["grad_w"], dtype, "cfg3 dL/dweight rows")
