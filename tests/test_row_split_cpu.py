"""Virtual rows for nodes with very many edges: the bookkeeping, on host graphs."""

import torch

import lunaequivariance_b200 as luna
from lunaequivariance_b200 import graph as graph_mod
from tests.helpers import random_graph


def test_virtual_rows_cover_the_same_edges(monkeypatch):
    monkeypatch.setattr(graph_mod, "ROW_SPLIT_EDGES", 7)
    nodes = 23
    src, dst = random_graph(nodes, 500, torch.Generator().manual_seed(2))
    graph = luna.make_graph(src, dst, nodes)
    split = graph.split_rows()
    assert split is not None and split is graph.split_rows()
    virtual = split.graph
    assert virtual.num_edges == graph.num_edges and virtual.split_rows() is None
    # every edge keeps its place in the edge list and maps back to its real end points
    assert torch.equal(split.destinations.rows[virtual.dst.long()], graph.dst.long())
    assert torch.equal(split.sources.rows[virtual.src.long()], graph.src.long())
    assert int(virtual.dst_rowptr.diff().max()) <= 7 and int(virtual.src_rowptr.diff().max()) <= 7
    # pieces: ceil(degree / limit), at least one per node, consecutive
    for side, rowptr in ((split.destinations, graph.dst_rowptr), (split.sources, graph.src_rowptr)):
        degree = rowptr.long().diff()
        pieces = torch.clamp((degree + 6) // 7, min=1)
        assert side.virtual_rows == int(pieces.sum())
        assert torch.equal(torch.bincount(side.rows, minlength=nodes), pieces)
        assert torch.equal(side.rows, torch.sort(side.rows)[0])
        # reduce sums the pieces of a node; gather repeats a node's row for each of its pieces
        values = torch.randn(side.virtual_rows, 3, dtype=torch.float64)
        expected = torch.zeros(nodes, 3, dtype=torch.float64).index_add_(0, side.rows, values)
        assert torch.allclose(side.reduce(values), expected, atol=1e-12)
        node_values = torch.randn(nodes, 2)
        assert torch.equal(side.gather(node_values), node_values[side.rows])
        assert side.gather(None) is None and side.reduce(None) is None


def test_no_split_below_the_limit():
    src, dst = random_graph(30, 200, torch.Generator().manual_seed(5))
    assert luna.make_graph(src, dst, 30).split_rows() is None
    assert luna.make_graph(src[:0], dst[:0], 4).split_rows() is None
