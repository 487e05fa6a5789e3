"""One rank of a destination-range partition on a single GPU.

A shard's graph has more source rows than destination rows: the owned rows followed by the halo rows (remote sources,
renumbered).  That shape - and the kernels' handling of it - never occurs in an unpartitioned graph, so it is checked
here without any other rank: the shard is built with ``exchange=False``, the feature buffer is assembled by hand
from the global features (``x[own range]`` then ``x[halo_ids]``), and every output is compared with the CPU oracle on
the shard's own edge list: out, gx over all rows of the buffer, gy, gw and the second derivatives.
"""

import pytest
import torch

import bench_workloads as workloads
import lunaequivariance_b200 as luna
from lunaequivariance_b200 import conv as conv_mod
from lunaequivariance_b200 import sharded
from oracle import uvu_conv as oracle_conv
from tests.helpers import assert_close, config

pytestmark = pytest.mark.gpu
DEVICE = "cuda"


@pytest.mark.parametrize("name,dtype,rank", [("cfg5", torch.float32, 1), ("cfg2", torch.float64, 2),
                                              ("cfg2", torch.float32, 0)])
def test_one_rank_of_an_uneven_partition(name, dtype, rank):
    in1, in2, out, instructions, options = config(name)
    module = luna.TensorProductConv(in1, in2, out, instructions, internal_weights=False, shared_weights=False,
                                    dtype=dtype)
    meta = oracle_conv.build_specs(in1, in2, out, instructions)
    op = module.op
    atoms = 300
    pos, box, cells = workloads.periodic_positions(atoms, workloads.DENSITY, 0, DEVICE, workloads.CUTOFF)
    src, dst, _ = workloads.radius_graph_periodic(pos, box, workloads.CUTOFF, cells)
    counts = (110, 50, 140)  # uneven on purpose
    begin = sum(counts[:rank])
    mine = (dst >= begin) & (dst < begin + counts[rank])
    shard = sharded.make_graph_shard(src[mine], dst[mine], counts, rank, exchange=False)
    graph = shard.graph
    assert graph.source_rows == counts[rank] + shard.halo_rows and shard.halo_rows > 0
    edges = graph.num_edges
    generator = torch.Generator().manual_seed(21)
    rand = lambda *shape: torch.randn(*shape, generator=generator, dtype=torch.float64).to(dtype)
    x_global = rand(atoms, op.in1_dim)
    x_full = torch.cat([x_global[begin:begin + counts[rank]], x_global[shard.halo_ids.cpu()]])
    p = dict(x=x_full, y=rand(edges, op.in2_dim), w=rand(edges, op.weight_numel), g=rand(counts[rank], op.out_dim),
             rx=rand(graph.source_rows, op.in1_dim), ry=rand(edges, op.in2_dim), rw=rand(edges, op.weight_numel))
    ref = oracle_conv.conv_derivatives(meta, *(p[k].double() for k in ("x", "y", "w")), graph.src.cpu(),
                                       graph.dst.cpu(), counts[rank], p["g"].double(),
                                       *(p[k].double() for k in ("rx", "ry", "rw")))
    d = {k: v.to(DEVICE) for k, v in p.items()}
    out_rows = conv_mod.run_forward(op, d["x"], d["y"], d["w"], graph)
    gx, gy, gw = conv_mod.run_backward(op, d["x"], d["y"], d["w"], d["g"], graph)
    hx, hy, hw, hg = conv_mod.run_double_backward(op, d["x"], d["y"], d["w"], d["g"], d["rx"], d["ry"], d["rw"], graph)
    op.check_status()
    assert op.uses_staged_kernels
    assert gx.shape[0] == graph.source_rows
    for key, value in dict(out=out_rows, gx=gx, gy=gy, gw=gw, hx=hx, hy=hy, hw=hw, hg=hg).items():
        assert_close(value, ref[key], dtype, f"{name} rank {rank} {key}")
