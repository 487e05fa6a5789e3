"""CPU oracle for the graph tables of the convolution. TEST INFRASTRUCTURE ONLY.

Test infrastructure: only the tests, the repository's smoke check and the benchmark's CPU-baseline legs may import this module.

Restates, in numpy, the CPU branch of the reference's ``make_graph`` (``src/lunatp/graph.py:49-141``) and
``make_source_segments`` (``src/lunatp/uvu_conv/graph.py:38-99``): validation messages, destination CSR, source
CSR, the edge permutation that groups edges by source, degree-descending node orders, the three quartile tiers and
the bounded source segments (at most 32 edges each, one empty segment per isolated node).

Where the reference's result is not unique (ties in ``argsort`` of degrees, order inside one source row of
``edge_ids_by_src`` - the reference's CPU branch uses a non-stable ``torch.argsort``) this oracle uses stable sorts
and the tests compare order-insensitive invariants for those tables, exactly like the reference's own tests
(``tests/lunatp/test_make_graph.py:33-55``).

Parity pin: ``tests/golden/graph_tables.npz`` holds the tables produced by the reference's ``make_graph`` on CPU.
"""

from __future__ import annotations

import numpy as np

SOURCE_SEGMENT_EDGES = 32


def validate(src, dst, num_nodes=None):
    src = np.asarray(src).reshape(-1)
    dst = np.asarray(dst).reshape(-1)
    if src.shape != dst.shape:
        raise ValueError("src and dst must have equal shape [edges] or [edges, 1].")
    required = 0
    if src.size:
        if min(src.min(), dst.min()) < 0:
            raise ValueError("graph indices must be nonnegative.")
        if np.any(dst[1:] < dst[:-1]):
            raise ValueError(
                "dst must be sorted in ascending order; src and edge data must follow the same order.")
        required = int(max(src.max(), dst.max())) + 1
    if num_nodes is None:
        num_nodes = required
    if num_nodes < required:
        raise ValueError(
            f"num_nodes={num_nodes} must be nonnegative and at least {required} for the supplied indices.")
    return src, dst, int(num_nodes)


def rowptr(index, num_nodes):
    counts = np.bincount(index, minlength=num_nodes) if index.size else np.zeros(num_nodes, dtype=np.int64)
    return np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)


def source_segments(src_rowptr, limit=SOURCE_SEGMENT_EDGES):
    degree = np.diff(src_rowptr)
    count = np.maximum((degree + limit - 1) // limit, 1)
    seg_rowptr = np.concatenate([[0], np.cumsum(count)]).astype(np.int64)
    nodes = np.repeat(np.arange(degree.size), count)
    local = np.arange(seg_rowptr[-1]) - np.repeat(seg_rowptr[:-1], count)
    begin = src_rowptr[nodes] + limit * local
    end = begin + np.minimum(limit, src_rowptr[nodes + 1] - begin)
    length = end - begin
    by_degree = np.argsort(-degree[nodes], kind="stable")
    order = by_degree[np.argsort(-length[by_degree], kind="stable")]
    return dict(nodes=nodes, begin=begin, end=end, rowptr=seg_rowptr, order=order)


def make_graph(src, dst, num_nodes=None):
    src, dst, num_nodes = validate(src, dst, num_nodes)
    edges = src.size
    dst_rowptr = rowptr(dst, num_nodes)
    src_rowptr = rowptr(src, num_nodes)
    in_degree, out_degree = np.diff(dst_rowptr), np.diff(src_rowptr)
    node_order = np.argsort(-in_degree, kind="stable")
    source_node_order = np.argsort(-out_degree, kind="stable")
    if num_nodes and edges:
        cumulative = np.cumsum(in_degree[node_order])
        thresholds = np.arange(1, 4) * edges // 4
        tiers = np.searchsorted(cumulative, thresholds, side="left") + 1
    else:
        tiers = np.full(3, num_nodes)
    return dict(
        src=src.astype(np.int32), dst=dst.astype(np.int32), num_nodes=num_nodes,
        dst_rowptr=dst_rowptr, src_rowptr=src_rowptr,
        edge_ids_by_src=np.argsort(src, kind="stable"), edge_ids_by_dst=np.arange(edges),
        node_order=node_order, source_node_order=source_node_order, node_tiers=tiers,
        source_segments=source_segments(src_rowptr),
    )
