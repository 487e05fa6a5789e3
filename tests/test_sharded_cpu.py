"""Destination-range sharding on CPU ranks (gloo): halo exchange of source rows, return of their gradients, uneven
shards.

The convolution itself needs a GPU, so the CPU oracle stands in for it here; what is under test is the partition,
the renumbering into [owned rows | halo rows], the two all-to-all exchanges and their autograd wiring.
"""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import bench_workloads as workloads
from lunaequivariance_b200 import sharded
from oracle import uvu_conv as oracle_conv


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _problem():
    generator = torch.Generator().manual_seed(4)
    nodes, edges = 23, 160
    meta = oracle_conv.build_specs("4x0e+4x1o", "1x0e+1x1o", "4x0e+4x1o",
                                   workloads.all_uvu_instructions("4x0e+4x1o", "1x0e+1x1o", "4x0e+4x1o"))
    src = torch.randint(nodes, (edges,), generator=generator)
    dst = torch.sort(torch.randint(nodes, (edges,), generator=generator))[0]
    rand = lambda *s: torch.randn(*s, generator=generator, dtype=torch.float64)
    return meta, nodes, src, dst, rand(nodes, meta["in1_dim"]), rand(edges, meta["in2_dim"]), \
        rand(edges, meta["weight_numel"]), rand(nodes, meta["out_dim"]), rand(nodes, meta["in1_dim"])


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        meta, nodes, src, dst, x, y, w, g, rx = _problem()
        counts = COUNTS[world]  # uneven on purpose
        begin = sum(counts[:rank])
        mine = (dst >= begin) & (dst < begin + counts[rank])
        shard = sharded.make_graph_shard(src[mine], dst[mine], counts, rank)
        remote = src[mine][(src[mine] < begin) | (src[mine] >= begin + counts[rank])]
        assert shard.halo_ids.tolist() == sorted(set(remote.tolist()))
        assert shard.graph.num_nodes == counts[rank]
        assert shard.graph.source_rows == counts[rank] + shard.halo_rows
        assert sum(shard.recv_counts) == shard.halo_rows and shard.send_rows.numel() == sum(shard.send_counts)
        assert shard.recv_counts[rank] == 0 and shard.send_counts[rank] == 0
        x_local = x[begin:begin + counts[rank]].clone().requires_grad_(True)
        w_local = w[mine].clone().requires_grad_(True)

        def conv(x_full, edge_attr, weight, graph):
            return oracle_conv.conv_forward(meta, x_full, edge_attr, weight, graph.src, graph.dst, graph.num_nodes)

        out = sharded.sharded_conv(conv, x_local, y[mine], w_local, shard)
        g_local = g[begin:begin + counts[rank]]
        gx, gw = torch.autograd.grad(out, (x_local, w_local), g_local, create_graph=True)
        (hw,) = torch.autograd.grad(gx, w_local, rx[begin:begin + counts[rank]])
        results[rank] = (out.detach(), gx.detach(), gw.detach(), hw.detach(), mine)
    finally:
        dist.destroy_process_group()


COUNTS = {2: (9, 14), 3: (9, 3, 11)}


@pytest.mark.parametrize("world", [2, 3])
def test_sharding_matches_single_rank(world):
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    meta, nodes, src, dst, x, y, w, g, rx = _problem()
    ref = oracle_conv.conv_derivatives(meta, x, y, w, src, dst, nodes, g, rx, None, None)
    out = torch.cat([results[r][0] for r in range(world)])
    gx = torch.cat([results[r][1] for r in range(world)])
    torch.testing.assert_close(out, ref["out"], atol=1e-12, rtol=1e-12)
    torch.testing.assert_close(gx, ref["gx"], atol=1e-12, rtol=1e-12)
    for r in range(world):
        mine = results[r][4]
        torch.testing.assert_close(results[r][2], ref["gw"][mine], atol=1e-12, rtol=1e-12)
        torch.testing.assert_close(results[r][3], ref["hw"][mine], atol=1e-12, rtol=1e-12)


def test_single_shard_without_exchange_and_ranges():
    # one rank of a partition built without its peers: the halo ids say which rows to append by hand
    src, dst = torch.tensor([0, 7, 4, 9, 3, 9]), torch.tensor([3, 3, 4, 4, 5, 5])
    shard = sharded.make_graph_shard(src, dst, (3, 3, 4), 1, exchange=False)
    assert shard.halo_ids.tolist() == [0, 7, 9] and shard.recv_counts == (1, 0, 2) and shard.send_counts == (0, 0, 0)
    assert shard.graph.src.tolist() == [3, 4, 1, 5, 0, 5] and shard.graph.dst.tolist() == [0, 0, 1, 1, 2, 2]
    assert shard.graph.source_rows == 6
    rowptr = torch.tensor([0, 10, 10, 30, 35, 60, 100])
    ranges = sharded.balanced_node_ranges(rowptr, 2)
    assert ranges[0][0] == 0 and ranges[-1][1] == 6 and ranges[0][1] == ranges[1][0]
    with pytest.raises(ValueError, match="range"):
        sharded.make_graph_shard(torch.tensor([0]), torch.tensor([4]), (3, 3), 0)


def test_radius_graph_matches_brute_force():
    pos, box, cells = workloads.periodic_positions(400, 0.1, 0, "cpu", 5.0)
    assert cells >= 3
    src, dst, vec = workloads.radius_graph_periodic(pos, box, 5.0, cells, chunk=97)
    delta = pos[None] - pos[:, None]
    delta = delta - box * torch.round(delta / box)
    mask = delta.square().sum(-1) < 25.0
    mask.fill_diagonal_(False)
    assert int(mask.sum()) == src.numel()
    assert bool((dst[1:] >= dst[:-1]).all())
    assert bool(mask[dst, src].all())
    torch.testing.assert_close(vec, delta[dst, src])
    part = workloads.radius_graph_periodic(pos, box, 5.0, cells, 100, 250)
    assert part[0].numel() == int(mask[100:250].sum())
    s2, d2 = workloads.fixed_degree_graph(50, 7, 0, "cpu")
    assert bool((torch.bincount(d2) == 7).all()) and not bool((s2 == d2).any())
