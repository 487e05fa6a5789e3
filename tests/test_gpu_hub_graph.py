"""Graphs with hub nodes: rows longer than ``ROW_SPLIT_EDGES`` run as several virtual rows.

The reference cuts source rows into segments of 32 edges and orders nodes by degree tier for the same reason
(``src/lunatp/uvu_conv/graph.py:38-99``, ``kernels/forward.py:239-254``).  Checked here: a node with thousands of
incoming and outgoing edges, and - with the limit lowered - an ordinary graph in which most rows are split, against the
CPU oracle to second order.
"""

import pytest
import torch

import lunaequivariance_b200 as luna
from lunaequivariance_b200 import conv as conv_mod
from lunaequivariance_b200 import graph as graph_mod
from oracle import uvu_conv as oracle_conv
from tests.helpers import assert_close, config, random_graph

pytestmark = pytest.mark.gpu
DEVICE = "cuda"


def hub_edges(nodes, hub, hub_degree, others, generator):
    """Random edges plus ``hub_degree`` edges into and out of one node; sorted by destination."""
    into = torch.stack([torch.randint(0, nodes, (hub_degree,), generator=generator), torch.full((hub_degree,), hub)])
    out_of = torch.stack([torch.full((hub_degree,), hub), torch.randint(0, nodes, (hub_degree,), generator=generator)])
    rest = torch.randint(0, nodes, (2, others), generator=generator)
    src, dst = torch.cat([into, out_of, rest], 1)
    order = torch.argsort(dst, stable=True)
    return src[order], dst[order]


def check(name, dtype, src, dst, nodes, expect_rows_above):
    in1, in2, out, instructions, _ = config(name)
    module = luna.TensorProductConv(in1, in2, out, instructions, internal_weights=False, shared_weights=False,
                                    dtype=dtype)
    op, meta = module.op, oracle_conv.build_specs(in1, in2, out, instructions)
    graph = luna.make_graph(src.to(DEVICE), dst.to(DEVICE), nodes)
    split = graph.split_rows()
    assert split is not None and split.graph.num_nodes > expect_rows_above
    assert split.graph.source_rows > expect_rows_above and split.graph.split_rows() is None
    assert int(split.graph.dst_rowptr.diff().max()) <= graph_mod.ROW_SPLIT_EDGES
    assert int(split.graph.src_rowptr.diff().max()) <= graph_mod.ROW_SPLIT_EDGES
    edges = src.numel()
    generator = torch.Generator().manual_seed(9)
    rand = lambda *shape: torch.randn(*shape, generator=generator, dtype=torch.float64).to(dtype)
    p = dict(x=rand(nodes, op.in1_dim), y=rand(edges, op.in2_dim), w=rand(edges, op.weight_numel),
             g=rand(nodes, op.out_dim), rx=rand(nodes, op.in1_dim), ry=rand(edges, op.in2_dim),
             rw=rand(edges, op.weight_numel))
    ref = oracle_conv.conv_derivatives(meta, *(p[k].double() for k in ("x", "y", "w")), src, dst, nodes,
                                       p["g"].double(), *(p[k].double() for k in ("rx", "ry", "rw")))
    d = {k: v.to(DEVICE) for k, v in p.items()}
    got = dict(out=conv_mod.run_forward(op, d["x"], d["y"], d["w"], graph))
    got["gx"], got["gy"], got["gw"] = conv_mod.run_backward(op, d["x"], d["y"], d["w"], d["g"], graph)
    got["hx"], got["hy"], got["hw"], got["hg"] = conv_mod.run_double_backward(
        op, d["x"], d["y"], d["w"], d["g"], d["rx"], d["ry"], d["rw"], graph)
    op.check_status()
    for key, value in got.items():
        assert value.shape == ref[key].shape
        assert_close(value, ref[key], dtype, f"{name} hub graph {key}")
    # through the module and autograd as well
    x, y, w = (d[k].clone().requires_grad_(True) for k in ("x", "y", "w"))
    result = module(x, y, w, graph=graph)
    gx, gy, gw = torch.autograd.grad(result, (x, y, w), d["g"])
    assert_close(result, ref["out"], dtype, "module out")
    assert_close(gx, ref["gx"], dtype, "module gx")
    assert_close(gw, ref["gw"], dtype, "module gw")
    # twice the same bits: the pieces of a row are added in a fixed order
    again = conv_mod.run_forward(op, d["x"], d["y"], d["w"], graph)
    assert torch.equal(again, got["out"])


@pytest.mark.parametrize("name,dtype", [("fixture", torch.float32), ("fixture", torch.float64), ("cfg5", torch.float32)])
def test_hub_node(name, dtype):
    nodes, hub = 150, 7
    src, dst = hub_edges(nodes, hub, 2600, 1500, torch.Generator().manual_seed(3))
    check(name, dtype, src, dst, nodes, expect_rows_above=nodes + 1)


def test_most_rows_split(monkeypatch):
    monkeypatch.setattr(graph_mod, "ROW_SPLIT_EDGES", 5)
    nodes = 41
    src, dst = random_graph(nodes, 700, torch.Generator().manual_seed(4))
    check("small", torch.float64, src, dst, nodes, expect_rows_above=2 * nodes)


def test_regular_graph_is_left_alone():
    src, dst = random_graph(60, 400, torch.Generator().manual_seed(1))
    graph = luna.make_graph(src.to(DEVICE), dst.to(DEVICE), 60)
    assert graph.split_rows() is None
