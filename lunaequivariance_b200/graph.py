"""Graph validation and the CSR / permutation tables shared by every order of the convolution.

Public behaviour follows the reference's ``make_graph`` and ``LunaTPGraph`` (``src/lunatp/graph.py:17-141``) and
``make_source_segments`` (``src/lunatp/uvu_conv/graph.py:38-99``): same field names, same validation messages,
inputs are copied into owned int32 tensors, ``dst`` must be ascending.  On CUDA tensors the tables are built by
the library's ``luna_graph_build`` (radix sorts and scans on the caller's stream); CPU tensors use torch ops so
that graphs can be prepared and inspected without a GPU.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from operator import index

import torch

from . import _native

SOURCE_SEGMENT_EDGES = 32
# A warp walks a node's edges one after the other, so a node with very many edges would hold one warp for the whole
# launch.  Rows longer than this are cut into virtual rows of at most this many edges (LunaTPGraph.split_rows).
ROW_SPLIT_EDGES = 1024


@dataclass(frozen=True)
class SourceSegmentTables:
    """Source-CSR rows cut into pieces of at most 32 edges; every node keeps at least one (possibly empty) piece."""

    nodes: torch.Tensor
    begin: torch.Tensor
    end: torch.Tensor
    rowptr: torch.Tensor
    order: torch.Tensor


class RowSplit:
    """One side (destinations or sources) of a graph whose long rows were cut into virtual rows.

    ``rows[v]`` is the real node of virtual row ``v`` (pieces of a node are consecutive virtual rows); ``gather``
    expands node rows to virtual rows, ``reduce`` sums virtual rows back to node rows, adding the pieces of a node in
    ascending order so that results are reproducible.
    """

    def __init__(self, rowptr: torch.Tensor, limit: int):
        degree = rowptr.to(torch.int64).diff()
        pieces = torch.clamp((degree + limit - 1) // limit, min=1)
        self.first = torch.cumsum(pieces, 0) - pieces             # first virtual row of each node
        self.virtual_rows = int(pieces.sum())
        self.rows = torch.repeat_interleave(torch.arange(degree.numel(), device=rowptr.device), pieces)
        self.limit = limit
        # nodes that have a (j + 1)-th piece, for j = 1, 2, ...: the targets of the j-th round of additions
        self.rounds = []
        for j in range(1, int(pieces.max()) if degree.numel() else 1):
            nodes = torch.nonzero(pieces > j).squeeze(1)
            self.rounds.append((nodes, self.first[nodes] + j))

    def gather(self, tensor: torch.Tensor | None) -> torch.Tensor | None:
        return None if tensor is None else tensor.index_select(0, self.rows)

    def reduce(self, virtual: torch.Tensor | None) -> torch.Tensor | None:
        if virtual is None:
            return None
        out = virtual.index_select(0, self.first)
        for nodes, rows in self.rounds:  # distinct targets within a round: plain indexed add, fixed order
            out[nodes] += virtual[rows]
        return out


class SplitGraph:
    """A graph with the same edges in the same order whose long rows are virtual rows (see ``ROW_SPLIT_EDGES``)."""

    def __init__(self, graph: "LunaTPGraph", limit: int):
        self.destinations = RowSplit(graph.dst_rowptr, limit)
        self.sources = RowSplit(graph.src_rowptr, limit)
        edges = graph.num_edges
        position = torch.arange(edges, device=graph.src.device, dtype=torch.int64)
        dst = graph.dst.to(torch.int64)
        dst_virtual = self.destinations.first[dst] + (position - graph.dst_rowptr.to(torch.int64)[dst]) // limit
        by_src = graph.edge_ids_by_src.to(torch.int64)
        src_sorted = graph.src.to(torch.int64)[by_src]
        rank = position - graph.src_rowptr.to(torch.int64)[src_sorted]  # of an edge among its source's edges
        src_virtual = torch.empty_like(position)
        src_virtual[by_src] = self.sources.first[src_sorted] + rank // limit
        self.graph = make_graph(src_virtual, dst_virtual, self.destinations.virtual_rows,
                                num_src_nodes=self.sources.virtual_rows, split=False)


@dataclass(frozen=True)
class LunaTPGraph:
    """Prepared topology; immutable and reusable across layers and dtypes."""

    src: torch.Tensor
    dst: torch.Tensor
    num_nodes: int
    dst_rowptr: torch.Tensor
    src_rowptr: torch.Tensor
    edge_ids_by_src: torch.Tensor
    edge_ids_by_dst: torch.Tensor
    node_order: torch.Tensor | None = None
    source_node_order: torch.Tensor | None = None
    node_tiers: torch.Tensor | None = None
    source_segments: SourceSegmentTables | None = None
    # Rows of x / gx.  Equals num_nodes except on a destination-range shard of a partitioned graph, where the
    # sources keep their global numbering (no counterpart in the reference, which is single-GPU).
    num_src_nodes: int | None = None
    can_split: bool = True  # False for the virtual-row graphs themselves
    _tables: dict = field(default_factory=dict, init=False, repr=False, compare=False)

    @property
    def num_edges(self) -> int:
        return int(self.src.numel())

    @property
    def source_rows(self) -> int:
        return self.num_nodes if self.num_src_nodes is None else int(self.num_src_nodes)

    def native(self) -> "_native.Graph":
        """The C-ABI view of this graph (cached; the tensors it points to are owned by the graph)."""
        view = self._tables.get("native")
        if view is None:
            view = _native.Graph(
                self.num_nodes, self.source_rows, self.num_edges, self.src.data_ptr(), self.dst.data_ptr(),
                self.dst_rowptr.data_ptr(), self.src_rowptr.data_ptr(), self.edge_ids_by_src.data_ptr(),
            )
            self._tables["native"] = view
        return view

    def destination_range(self, begin: int, end: int) -> "tuple[LunaTPGraph, int, int]":
        """The graph of the edges whose destination lies in ``[begin, end)``, and that slice ``[e0, e1)`` of the edge
        list: destinations renumbered from zero, sources as they are.

        Because edges are sorted by destination the slice is contiguous, so per-edge tensors of the piece are row
        ranges of the whole graph's (``y[e0:e1]``, ``w[e0:e1]``) and its output rows are ``out[begin:end]``.  Pieces
        that tile ``[0, num_nodes)`` together do the work of the whole graph; only the source-row gradients of the
        pieces have to be added up.  No counterpart in the reference.  Cached per range.
        """
        if not 0 <= begin <= end <= self.num_nodes:
            raise ValueError(f"destination range [{begin}, {end}) outside [0, {self.num_nodes}]")
        key = ("range", int(begin), int(end))
        cached = self._tables.get(key)
        if cached is None:
            e0, e1 = (int(v) for v in self.dst_rowptr[[begin, end]].tolist())
            piece = make_graph(self.src[e0:e1], self.dst[e0:e1] - begin, end - begin, num_src_nodes=self.source_rows)
            cached = self._tables[key] = (piece, e0, e1)
        return cached

    def split_rows(self) -> "SplitGraph | None":
        """The virtual-row form of this graph if a node has more than ``ROW_SPLIT_EDGES`` edges on either side, else
        ``None``.  Decided once per graph (one read of the largest degree) and cached."""
        if "split" not in self._tables:
            split = None
            if self.can_split and self.num_edges:
                longest = int(torch.maximum(self.dst_rowptr.diff().max(), self.src_rowptr.diff().max()))
                if longest > ROW_SPLIT_EDGES:
                    split = SplitGraph(self, ROW_SPLIT_EDGES)
            self._tables["split"] = split
        return self._tables["split"]

    def table_list(self) -> list:
        """The 13 tensors the reference passes to its custom ops (``src/lunatp/uvu_conv/interface.py:186-192``)."""
        seg = self.source_segments
        return [self.src, self.dst, self.dst_rowptr, self.src_rowptr, self.edge_ids_by_src,
                self.source_node_order, self.node_order,
                seg.nodes, seg.begin, seg.end, seg.rowptr, seg.order, self.node_tiers]


def make_source_segments(src_rowptr: torch.Tensor) -> SourceSegmentTables:
    rowptr = src_rowptr.to(torch.int64)
    degree = rowptr[1:] - rowptr[:-1]
    count = ((degree + (SOURCE_SEGMENT_EDGES - 1)) // SOURCE_SEGMENT_EDGES).clamp_min(1)
    seg_rowptr = torch.zeros(degree.numel() + 1, dtype=torch.int64, device=rowptr.device)
    torch.cumsum(count, 0, out=seg_rowptr[1:])
    total = int(seg_rowptr[-1].item()) if degree.numel() else 0
    nodes = torch.repeat_interleave(torch.arange(degree.numel(), device=rowptr.device), count, output_size=total)
    local = torch.arange(total, device=rowptr.device) - seg_rowptr[:-1][nodes]
    begin = rowptr[nodes] + SOURCE_SEGMENT_EDGES * local
    end = torch.minimum(begin + SOURCE_SEGMENT_EDGES, rowptr[nodes + 1])
    by_degree = torch.argsort(degree[nodes], descending=True, stable=True)
    order = by_degree[torch.argsort((end - begin)[by_degree], descending=True, stable=True)]
    narrow = src_rowptr.dtype
    return SourceSegmentTables(nodes.to(torch.int32), begin.to(narrow), end.to(narrow), seg_rowptr.to(narrow),
                               order.to(narrow))


def _node_tiers(dst_rowptr, node_order, num_nodes, num_edges, device):
    if num_nodes and num_edges:
        cumulative = dst_rowptr.diff().to(torch.int64)[node_order.long()].cumsum(0)
        thresholds = torch.arange(1, 4, device=device, dtype=torch.int64) * num_edges // 4
        return (torch.searchsorted(cumulative, thresholds) + 1).to(torch.int32)
    return torch.full((3,), num_nodes, device=device, dtype=torch.int32)


def _bounds_host(src, dst):
    low = min(int(src.min()), int(dst.min()))
    unsorted = bool((dst[1:] < dst[:-1]).any()) if src.numel() > 1 else False
    return low, int(src.max()), int(dst.max()), unsorted


def _bounds_cuda(src, dst):
    lib = _native.library()
    edges = src.numel()
    scratch_bytes = lib.luna_graph_scratch_bytes(0, edges)
    scratch = torch.empty(max(scratch_bytes, 1), dtype=torch.uint8, device=src.device)
    low, high_src, high_dst, unsorted = ctypes.c_int64(0), ctypes.c_int64(-1), ctypes.c_int64(-1), ctypes.c_int(0)
    bits = 64 if src.dtype == torch.int64 else 32
    _native.check(lib.luna_graph_bounds(src.data_ptr(), dst.data_ptr(), bits, edges, ctypes.byref(low),
                                        ctypes.byref(high_src), ctypes.byref(high_dst), ctypes.byref(unsorted),
                                        scratch.data_ptr(), scratch_bytes, _native.current_stream(src.device)))
    return low.value, high_src.value, high_dst.value, bool(unsorted.value)


def make_graph(src: torch.Tensor, dst: torch.Tensor, num_nodes: int | None = None, *,
               num_src_nodes: int | None = None, split: bool = True) -> LunaTPGraph:
    """Build the topology tables from a destination-sorted edge list.

    ``src`` and ``dst`` are ``[edges]`` or ``[edges, 1]`` int32/int64 tensors on one device, ``dst`` ascending and
    all edge data in the same order.  Build once per topology and reuse across layers.  ``num_src_nodes`` (keyword
    only, default ``num_nodes``) gives the row count of ``x`` when sources are numbered in a larger range than the
    destinations, as on one shard of a partitioned graph.  ``split=False`` marks a graph whose rows must stay as
    they are (``split_rows`` then returns ``None``).
    """
    if src.ndim == 2 and src.shape[1] == 1:
        src = src.squeeze(-1)
    if dst.ndim == 2 and dst.shape[1] == 1:
        dst = dst.squeeze(-1)
    if src.ndim != 1 or dst.ndim != 1 or src.shape != dst.shape:
        raise ValueError("src and dst must have equal shape [edges] or [edges, 1].")
    if src.dtype not in (torch.int32, torch.int64) or dst.dtype not in (torch.int32, torch.int64):
        raise TypeError("graph indices must be int32 or int64.")
    if src.device != dst.device:
        raise ValueError("src and dst must be on the same device.")
    if num_nodes is not None and not isinstance(num_nodes, int):
        num_nodes = index(num_nodes)
    if src.dtype != dst.dtype:
        src, dst = src.to(torch.int64), dst.to(torch.int64)
    src, dst = src.contiguous(), dst.contiguous()

    num_edges = src.numel()
    device = src.device
    required = 0
    if num_edges:
        with torch.cuda.device(device) if device.type == "cuda" else _NullContext():
            low, high_src, high_dst, unsorted = (_bounds_cuda if device.type == "cuda" else _bounds_host)(src, dst)
        if low < 0:
            raise ValueError("graph indices must be nonnegative.")
        if unsorted:
            raise ValueError("dst must be sorted in ascending order; src and edge data must follow the same order.")
        required = (high_dst if num_src_nodes is not None else max(high_src, high_dst)) + 1
        if num_src_nodes is not None and num_src_nodes < high_src + 1:
            raise ValueError(
                f"num_src_nodes={num_src_nodes} must be at least {high_src + 1} for the supplied indices.")
    if num_nodes is None:
        num_nodes = required
    if num_nodes < required:
        raise ValueError(
            f"num_nodes={num_nodes} must be nonnegative and at least {required} for the supplied indices.")
    source_rows = num_nodes if num_src_nodes is None else int(num_src_nodes)
    if max(num_nodes, source_rows) >= (1 << 31):
        raise OverflowError("graph node count exceeds signed int32 capacity.")
    if max(num_edges, num_nodes + num_edges // SOURCE_SEGMENT_EDGES) >= (1 << 31) - 1024:
        raise OverflowError("graph edge count exceeds the int32 table capacity of this build.")

    if device.type == "cuda":
        tables = _build_cuda(src, dst, num_nodes, source_rows)
    else:
        tables = _build_host(src, dst, num_nodes, source_rows)
    src_out, dst_out, dst_rowptr, src_rowptr, edge_ids_by_src, node_order, source_node_order = tables
    graph = LunaTPGraph(
        src=src_out, dst=dst_out, num_nodes=num_nodes, dst_rowptr=dst_rowptr, src_rowptr=src_rowptr,
        edge_ids_by_src=edge_ids_by_src,
        edge_ids_by_dst=torch.arange(num_edges, device=device, dtype=torch.int32),
        node_order=node_order, source_node_order=source_node_order,
        node_tiers=_node_tiers(dst_rowptr, node_order, num_nodes, num_edges, device),
        source_segments=make_source_segments(src_rowptr),
        num_src_nodes=None if num_src_nodes is None else source_rows,
        can_split=split,
    )
    return graph


class _NullContext:
    def __enter__(self):
        return None

    def __exit__(self, *args):
        return False


def _build_host(src, dst, num_nodes, source_rows):
    device = src.device

    def rowptr(index_tensor, rows):
        out = torch.zeros(rows + 1, dtype=torch.int32, device=device)
        if index_tensor.numel():
            counts = torch.bincount(index_tensor.long(), minlength=rows)
            out[1:] = torch.cumsum(counts, 0).to(torch.int32)
        return out

    src_rowptr, dst_rowptr = rowptr(src, source_rows), rowptr(dst, num_nodes)
    node_order = torch.argsort(dst_rowptr.diff().long(), descending=True, stable=True).to(torch.int32)
    source_node_order = torch.argsort(src_rowptr.diff().long(), descending=True, stable=True).to(torch.int32)
    edge_ids_by_src = torch.argsort(src.long(), stable=True).to(torch.int32)
    return (src.to(torch.int32, copy=True), dst.to(torch.int32, copy=True), dst_rowptr, src_rowptr, edge_ids_by_src,
            node_order, source_node_order)


def _build_cuda(src, dst, num_nodes, source_rows):
    lib = _native.library()
    device = src.device
    edges = src.numel()
    i32 = dict(dtype=torch.int32, device=device)
    out = [torch.empty(edges, **i32), torch.empty(edges, **i32), torch.empty(num_nodes + 1, **i32),
           torch.empty(source_rows + 1, **i32), torch.empty(edges, **i32), torch.empty(num_nodes, **i32),
           torch.empty(source_rows, **i32)]
    with torch.cuda.device(device):
        scratch_bytes = lib.luna_graph_scratch_bytes(max(num_nodes, source_rows), edges)
        scratch = torch.empty(max(scratch_bytes, 1), dtype=torch.uint8, device=device)
        view = _native.GraphOut(*(t.data_ptr() for t in out))
        bits = 64 if src.dtype == torch.int64 else 32
        _native.check(lib.luna_graph_build(src.data_ptr(), dst.data_ptr(), bits, num_nodes, source_rows, edges,
                                           ctypes.byref(view), scratch.data_ptr(), scratch_bytes,
                                           _native.current_stream(device)))
    return tuple(out)


__all__ = ["LunaTPGraph", "SourceSegmentTables", "SplitGraph", "RowSplit", "make_graph", "make_source_segments"]
