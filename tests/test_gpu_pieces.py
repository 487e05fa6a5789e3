"""A graph's work done in pieces: destination ranges, the host-streaming executor and the overlapped shard step.

All three rest on the same two facts, checked here against one call on the whole graph: the edges of a destination
range are a contiguous slice of the edge list whose per-edge tensors are row ranges of the whole graph's, and the
source-row gradients of the pieces add up (``luna_uvu_conv_bwd_add_gx``).
"""

import pytest
import torch

import bench_workloads as workloads
import lunaequivariance_b200 as luna
from lunaequivariance_b200 import conv as conv_mod
from lunaequivariance_b200 import sharded
from lunaequivariance_b200.streaming import HostStreamedConv
from tests.helpers import assert_close, config

pytestmark = pytest.mark.gpu
DEVICE = "cuda"


def problem(name, dtype, atoms=240, seed=5):
    in1, in2, out, instructions, _ = config(name)
    module = luna.TensorProductConv(in1, in2, out, instructions, internal_weights=False, shared_weights=False,
                                    dtype=dtype)
    pos, box, cells = workloads.periodic_positions(atoms, workloads.DENSITY, 0, DEVICE, workloads.CUTOFF)
    src, dst, _ = workloads.radius_graph_periodic(pos, box, workloads.CUTOFF, cells)
    graph = luna.make_graph(src, dst, atoms)
    op = module.op
    generator = torch.Generator(device=DEVICE).manual_seed(seed)
    rand = lambda *shape: torch.randn(*shape, generator=generator, dtype=dtype, device=DEVICE)
    tensors = dict(x=rand(atoms, op.in1_dim), y=rand(graph.num_edges, op.in2_dim),
                   w=rand(graph.num_edges, op.weight_numel), g=rand(atoms, op.out_dim))
    return module, op, graph, tensors, (src, dst)


def whole(op, graph, t):
    out = conv_mod.run_forward(op, t["x"], t["y"], t["w"], graph)
    gx, gy, gw = conv_mod.run_backward(op, t["x"], t["y"], t["w"], t["g"], graph)
    return dict(out=out, gx=gx, gy=gy, gw=gw)


@pytest.mark.parametrize("name,dtype", [("cfg2", torch.float32), ("cfg5", torch.float32), ("cfg2", torch.float64),
                                        ("fixture", torch.float32)])
def test_destination_ranges_add_up(name, dtype):
    module, op, graph, t, _ = problem(name, dtype)
    ref = whole(op, graph, t)
    nodes = graph.num_nodes
    out = torch.full_like(ref["out"], float("nan"))
    gy, gw = torch.full_like(ref["gy"], float("nan")), torch.full_like(ref["gw"], float("nan"))
    gx = torch.zeros_like(ref["gx"])
    covered = 0
    for begin, end in ((0, 17), (17, 17), (17, 150), (150, nodes)):  # uneven, one empty
        piece, e0, e1 = graph.destination_range(begin, end)
        assert piece.num_nodes == end - begin and piece.num_edges == e1 - e0 and piece.source_rows == nodes
        covered += e1 - e0
        conv_mod.run_forward(op, t["x"], t["y"][e0:e1], t["w"][e0:e1], piece, out=out[begin:end])
        conv_mod.run_backward(op, t["x"], t["y"][e0:e1], t["w"][e0:e1], t["g"][begin:end], piece,
                              out=(gx, gy[e0:e1], gw[e0:e1]), add_gx=True)
    op.check_status()
    assert covered == graph.num_edges
    assert torch.equal(out, ref["out"]) and torch.equal(gy, ref["gy"]) and torch.equal(gw, ref["gw"])
    assert_close(gx, ref["gx"].cpu(), dtype, f"{name} gx summed over pieces")
    assert graph.destination_range(17, 150)[0] is graph.destination_range(17, 150)[0]  # cached


def test_add_gx_needs_a_tensor_and_out_shapes_are_checked():
    module, op, graph, t, _ = problem("cfg5", torch.float32, atoms=60)
    with pytest.raises(ValueError, match="add_gx"):
        conv_mod.run_backward(op, t["x"], t["y"], t["w"], t["g"], graph, add_gx=True)
    with pytest.raises(ValueError, match="out must be"):
        conv_mod.run_forward(op, t["x"], t["y"], t["w"], graph, out=torch.empty(3, 3, device=DEVICE))
    with pytest.raises(ValueError, match="outside"):
        graph.destination_range(5, graph.num_nodes + 1)


@pytest.mark.parametrize("name,dtype,chunks", [("cfg2", torch.float32, 5), ("cfg5", torch.float32, 1),
                                                ("cfg2", torch.float64, 3)])
def test_host_streamed_step_matches_one_call(name, dtype, chunks):
    module, op, graph, t, _ = problem(name, dtype, atoms=300)
    ref = whole(op, graph, t)
    host = {k: v.cpu().pin_memory() for k, v in t.items()}
    streamed = HostStreamedConv(op, graph, chunks=chunks)
    assert 1 <= len(streamed.pieces) <= chunks
    for _ in range(2):  # buffers and host outputs are reused from step to step
        out, gx, gy, gw = streamed.step(host["x"], host["y"], host["w"], host["g"])
    op.check_status()
    assert out.device.type == "cpu" and gw.shape == ref["gw"].shape
    assert torch.equal(out, ref["out"].cpu()) and torch.equal(gy, ref["gy"].cpu())
    assert torch.equal(gw, ref["gw"].cpu())
    assert_close(gx, ref["gx"].cpu(), dtype, f"{name} streamed gx")
    # node features already on the device: gx stays there
    out2, gx_device, _, _ = streamed.step(t["x"], host["y"], host["w"], t["g"])
    assert gx_device.is_cuda and torch.equal(gx_device.cpu(), gx) and torch.equal(out2, ref["out"].cpu())
    with pytest.raises(ValueError, match="host tensor"):
        streamed.step(host["x"], t["y"], host["w"], host["g"])


@pytest.mark.parametrize("rank", [0, 1, 2])
def test_overlapped_step_on_one_rank_of_a_partition(rank):
    """The piece schedule of the overlapped step (interior, then the two ends; ends first in the backward), with the
    halo rows supplied by hand in place of the exchange, against plain calls on the shard's graph."""
    dtype = torch.float32
    module, op, _, t, (src, dst) = problem("cfg2", dtype, atoms=300)
    counts = (110, 50, 140)
    begin = sum(counts[:rank])
    mine = (dst >= begin) & (dst < begin + counts[rank])
    shard = sharded.make_graph_shard(src[mine], dst[mine], counts, rank, exchange=False)
    lo, hi = shard.interior
    assert 0 <= lo <= hi <= counts[rank]
    remote = shard.graph.src.long() >= counts[rank]
    touched = torch.unique(shard.graph.dst[remote].long())
    assert not ((touched >= lo) & (touched < hi)).any()  # interior destinations read owned rows only
    x_local, halo = t["x"][begin:begin + counts[rank]], t["x"][shard.halo_ids]
    y, w, g = t["y"][mine], t["w"][mine], t["g"][begin:begin + counts[rank]]
    x_full = torch.cat([x_local, halo])
    ref_out = conv_mod.run_forward(op, x_full, y, w, shard.graph)
    ref_gx, ref_gy, ref_gw = conv_mod.run_backward(op, x_full, y, w, g, shard.graph)
    events = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
    out, gx_full, gy, gw = sharded.overlapped_step(op, x_local, y, w, g, shard, halo_rows=halo, events=events)
    torch.cuda.synchronize()
    op.check_status()
    assert events[0].elapsed_time(events[4]) > 0
    assert torch.equal(out, ref_out) and torch.equal(gy, ref_gy) and torch.equal(gw, ref_gw)
    assert_close(gx_full, ref_gx.cpu(), dtype, f"rank {rank} gx of the compact buffer")


def test_host_streamed_step_on_tiny_and_empty_graphs():
    in1, in2, out, instructions, _ = config("fixture")
    dtype = torch.float32
    module = luna.TensorProductConv(in1, in2, out, instructions, internal_weights=False, shared_weights=False,
                                    dtype=dtype)
    op = module.op
    nodes = 7
    dst = torch.tensor([0, 0, 1, 1, 1, 4, 4, 4, 4, 6], device=DEVICE)  # destinations 2, 3, 5 have no edge
    src = torch.tensor([1, 6, 0, 2, 3, 4, 5, 0, 1, 2], device=DEVICE)
    graph = luna.make_graph(src, dst, nodes)
    generator = torch.Generator(device=DEVICE).manual_seed(2)
    rand = lambda *shape: torch.randn(*shape, generator=generator, dtype=dtype, device=DEVICE)
    t = dict(x=rand(nodes, op.in1_dim), y=rand(10, op.in2_dim), w=rand(10, op.weight_numel), g=rand(nodes, op.out_dim))
    ref = whole(op, graph, t)
    streamed = HostStreamedConv(op, graph, chunks=16)  # more chunks than nodes
    assert 1 <= len(streamed.pieces) <= nodes
    host = {k: v.cpu() for k, v in t.items()}  # pageable memory works too
    out_rows, gx, gy, gw = streamed.step(host["x"], host["y"], host["w"], host["g"])
    assert torch.equal(out_rows, ref["out"].cpu()) and torch.equal(gy, ref["gy"].cpu())
    assert torch.equal(gw, ref["gw"].cpu())
    assert_close(gx, ref["gx"].cpu(), dtype, "tiny graph gx")
    assert not out_rows[[2, 3, 5]].any()

    empty = luna.make_graph(src[:0], dst[:0], 4)
    streamed = HostStreamedConv(op, empty, chunks=3)
    out_rows, gx, gy, gw = streamed.step(host["x"][:4], host["y"][:0], host["w"][:0], host["g"][:4])
    assert out_rows.shape == (4, op.out_dim) and not out_rows.any() and not gx.any()
    assert gy.shape == (0, op.in2_dim) and gw.shape == (0, op.weight_numel)
