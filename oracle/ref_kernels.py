"""Calls the reference's own compiled CUDA kernels (built by ``oracle/build_ref.py``) on a machine with a GPU.

Test infrastructure: only the tests and the bench's reference leg import this; the product never does.

The libraries under ``oracle/_ref`` are the torch extensions the reference generates for its UVU convolution
(forward: ``src/lunatp/uvu_conv/kernels/forward.py:1291-1343``; backward: ``kernels/backward.py:572-681``).  The
launch protocol below restates what those two ``run`` functions do around the extension call: allocate the outputs
and the partial slabs the kernels reduce into, choose between whole source rows and the 32-edge source segments, and
pass the graph tables in the extension's argument order.  Graph tables come from this repository's ``make_graph``,
whose output is pinned to the reference's own tables by the golden fixtures.
"""

from __future__ import annotations

import importlib.util
import json
import os

import torch

REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


def available(key: str | None = None) -> bool:
    path = os.path.join(REF_DIR, "manifest.json")
    if not os.path.exists(path):
        return False
    if key is None:
        return True
    with open(path) as handle:
        entry = json.load(handle).get(key)
    return bool(entry) and all(os.path.exists(os.path.join(REF_DIR, entry[k]["file"])) for k in ("forward", "backward"))


def _load(module_name: str, filename: str):
    spec = importlib.util.spec_from_file_location(module_name, os.path.join(REF_DIR, filename))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module  # holds the 32-bit (``i32``) and the 64-bit (``i64``) index variants of the same kernels


class _WideTables:
    """The graph tables the 64-bit variant reads as int64 (``src/lunatp/graph.py:147-170``): row pointers, the
    edge permutation and the segment begin / end / rowptr / order; node lists stay int32."""

    def __init__(self, graph):
        wide = lambda t: t.to(torch.int64)
        self.num_nodes, self.num_edges = graph.num_nodes, graph.num_edges
        self.src, self.dst = graph.src, graph.dst
        self.node_order, self.source_node_order, self.node_tiers = (
            graph.node_order, graph.source_node_order, graph.node_tiers)
        self.dst_rowptr, self.src_rowptr = wide(graph.dst_rowptr), wide(graph.src_rowptr)
        self.edge_ids_by_src = wide(graph.edge_ids_by_src)
        seg = graph.source_segments
        self.source_segments = type(seg)(nodes=seg.nodes, begin=wide(seg.begin), end=wide(seg.end),
                                         rowptr=wide(seg.rowptr), order=wide(seg.order))


class ReferenceKernels:
    """The reference's forward and first-order backward for one configuration and dtype (``"cfg2.float32"``)."""

    def __init__(self, key: str, force_wide: bool = False):
        self.force_wide = force_wide  # always use the 64-bit index variant (to check it on small graphs)
        with open(os.path.join(REF_DIR, "manifest.json")) as handle:
            self.entry = json.load(handle)[key]
        self.dtype = getattr(torch, self.entry["dtype"])
        self._fwd = _load(self.entry["forward"]["module"], self.entry["forward"]["file"])
        self._bwd = _load(self.entry["backward"]["module"], self.entry["backward"]["file"])
        self._streams = None
        self._stream_state = {}
        self._wide = {}

    def _variant(self, graph):
        """(forward module, backward module, graph tables) of the index width the reference would pick: its 32-bit
        kernels are only valid up to the node and edge counts recorded at build time."""
        if (not self.force_wide and graph.num_nodes <= self.entry["index_node_limit"]
                and graph.num_edges <= self.entry["index_edge_limit"]):
            return self._fwd.i32, self._bwd.i32, graph
        tables = self._wide.get(id(graph))
        if tables is None:
            tables = self._wide[id(graph)] = _WideTables(graph)
        return self._fwd.i64, self._bwd.i64, tables

    def forward(self, x, y, w, graph):
        fwd, _, graph = self._variant(graph)
        info = self.entry["forward"]
        out = torch.empty((graph.num_nodes, self.entry["out_dim"]), device=x.device, dtype=self.dtype)
        if info["output_needs_zero"]:  # several paths add into one output block with atomics
            out.zero_()
        if graph.num_nodes:
            tiers = graph.node_tiers if info["degree_tiers"] else None
            fwd.run_uvu_conv_fwd_ordered(x, y, w, None, None, graph.src, graph.dst_rowptr, graph.node_order, tiers, out,
                                         graph.num_nodes)
        return out

    def backward(self, x, y, w, g, graph):
        _, bwd, graph = self._variant(graph)
        info = self.entry["backward"]
        edges = graph.num_edges
        if info["vectorized"]:
            w = w.clone() if w.data_ptr() % 16 else w
            g = g.clone() if g.data_ptr() % 16 else g
        gx, gy, gw = torch.empty_like(x), torch.empty_like(y), torch.empty_like(w)
        if info["segmented"]:
            seg = graph.source_segments
            nodes, begin, end, order, rowptr = seg.nodes, seg.begin, seg.end, seg.order, seg.rowptr
            make = torch.zeros if info["zero_x"] else torch.empty
            gx_partial = make((nodes.numel(), self.entry["in1_dim"]), device=x.device, dtype=self.dtype)
        else:
            nodes = order = graph.source_node_order
            begin = end = rowptr = graph.src_rowptr
            gx_partial = gx
            if info["zero_x"]:
                gx.zero_()
        make = torch.zeros if info["zero_y"] else torch.empty
        gy_partial = make((info["partials"], edges, self.entry["in2_dim"]), device=x.device, dtype=self.dtype)
        state = ()
        if info["stream_count"]:
            if self._streams is None:
                self._streams = [torch.cuda.Stream(x.device, priority=info["stream_priority"])
                                 for _ in range(info["stream_count"])]
            if bwd not in self._stream_state:
                self._stream_state[bwd] = bwd._Streams(x.device.index, [s.cuda_stream for s in self._streams])
            state = (self._stream_state[bwd],)
        bwd.run_uvu_conv_bwd(*state, x, y, w, g, graph.dst, graph.edge_ids_by_src, nodes, begin, end, order, rowptr,
                             gx_partial, gy_partial, gx, gy, gw, graph.num_nodes, edges, nodes.numel(), None, None, None,
                             None)
        return gx, gy, gw
