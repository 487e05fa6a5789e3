"""Destination-range partition of the convolution across the ranks of a ``torch.distributed`` process group.

The reference is single-GPU; this module is the multi-GPU design for its convolution.  Each rank owns a contiguous
range of destination nodes, hence one contiguous slice of the destination-sorted edge list with its edge attributes
and per-edge weights - the bulk of the bytes never moves.  Only node features cross ranks, and only the rows that are
needed:

* when the shard is built, a rank lists the distinct remote sources its edges read (its *halo*), tells every owner
  which of the owner's rows it wants, and renumbers its sources into a compact buffer ``[owned rows | halo rows]``;
* forward: owners send the requested ``x`` rows (one NCCL all-to-all) straight into the halo part of that buffer;
* backward: the kernels produce gradient rows for the compact buffer; the halo part goes back to the owners with
  the reverse all-to-all and is added to the owned rows one peer at a time, in rank order (rows of one peer are
  distinct, so the sum has a fixed order: results are reproducible for a given partition).

Both exchanges are autograd functions whose backward is the other one, so first and second derivatives work.  The
kernels only ever dereference local memory.  For a spatially ordered graph (atoms numbered cell by cell, contiguous
ranges = slabs) the halo is the atoms within one cutoff of the slab faces, a small fraction of all rows.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from .graph import LunaTPGraph, make_graph


@dataclass(frozen=True)
class GraphShard:
    """One rank's part of a partitioned graph."""

    graph: LunaTPGraph        # local destinations; sources renumbered into [owned rows | halo rows]
    node_begin: int           # first global node owned by this rank
    node_counts: tuple        # nodes owned by each rank
    halo_ids: torch.Tensor    # global ids of the remote sources this rank reads, ascending (so grouped by owner)
    recv_counts: tuple        # halo rows that come from each rank
    send_counts: tuple        # owned rows each rank wants from this one
    send_rows: torch.Tensor   # local indices of those rows, grouped by requesting rank
    group: object = None
    interior: tuple = (0, 0)  # longest run [begin, end) of local destinations all of whose sources are owned

    @property
    def local_nodes(self) -> int:
        return self.graph.num_nodes

    @property
    def halo_rows(self) -> int:
        return int(self.halo_ids.numel())

    @property
    def world_size(self) -> int:
        return len(self.node_counts)


def _bounds(node_counts, device) -> torch.Tensor:
    return torch.tensor([0] + list(node_counts), device=device, dtype=torch.int64).cumsum(0)


def make_graph_shard(src_global: torch.Tensor, dst_global: torch.Tensor, node_counts, rank: int, group=None, *,
                     exchange: bool | None = None) -> GraphShard:
    """Build this rank's shard from its slice of the edge list (global node ids, ``dst`` ascending and inside the
    rank's node range).

    With more than one rank this is a collective call: every rank of ``group`` (the default group if ``None``) must
    make it, because the ranks tell each other which rows they will request.  ``exchange=False`` skips that step and
    leaves the send lists empty: the shard can then be used on its own with a hand-assembled feature buffer
    (``x[own range]`` followed by ``x[halo_ids]``), which is how one rank of a partition is checked on a single GPU.
    """
    node_counts = tuple(int(c) for c in node_counts)
    world = len(node_counts)
    begin, local = sum(node_counts[:rank]), node_counts[rank]
    device = src_global.device
    if dst_global.numel():
        low, high = int(dst_global.min()), int(dst_global.max())
        if low < begin or high >= begin + local:
            raise ValueError(f"destination ids must lie in this rank's range [{begin}, {begin + local})")
    src64 = src_global.to(torch.int64)
    owned = (src64 >= begin) & (src64 < begin + local)
    halo_ids = torch.unique(src64[~owned])  # sorted ascending
    compact = torch.where(owned, src64 - begin, local + torch.searchsorted(halo_ids, src64))
    dst_local = dst_global.to(torch.int64) - begin
    graph = make_graph(compact, dst_local, local, num_src_nodes=local + halo_ids.numel())
    interior = _longest_interior_run(torch.unique(dst_local[~owned]), local)

    bounds = _bounds(node_counts, device)
    owner = torch.searchsorted(bounds, halo_ids, right=True) - 1
    recv_counts = torch.bincount(owner, minlength=world)[:world]
    if exchange is None:
        exchange = world > 1
    if exchange and world > 1:
        send_counts = torch.empty_like(recv_counts)
        dist.all_to_all_single(send_counts, recv_counts, group=group)
        recv_list, send_list = recv_counts.tolist(), send_counts.tolist()
        wanted = (halo_ids - bounds[owner]).contiguous()  # row numbers inside each owner's range
        send_rows = torch.empty(sum(send_list), dtype=torch.int64, device=device)
        dist.all_to_all_single(send_rows, wanted, output_split_sizes=send_list, input_split_sizes=recv_list,
                               group=group)
    else:
        recv_list, send_list = recv_counts.tolist(), [0] * world
        send_rows = torch.empty(0, dtype=torch.int64, device=device)
    return GraphShard(graph=graph, node_begin=begin, node_counts=node_counts, halo_ids=halo_ids,
                      recv_counts=tuple(recv_list), send_counts=tuple(send_list), send_rows=send_rows, group=group,
                      interior=interior)


def _longest_interior_run(boundary_nodes: torch.Tensor, local: int) -> tuple:
    """``boundary_nodes``: ascending local ids of the destinations that read a remote source.  Returns the longest
    run of consecutive destinations between them."""
    if local == 0:
        return (0, 0)
    if boundary_nodes.numel() == 0:
        return (0, local)
    fence = torch.cat([boundary_nodes.new_tensor([-1]), boundary_nodes, boundary_nodes.new_tensor([local])])
    gaps = fence[1:] - fence[:-1] - 1
    where = int(torch.argmax(gaps))
    start = int(fence[where]) + 1
    return (start, start + int(gaps[where]))


def exchange_halo(x_local: torch.Tensor, shard: GraphShard) -> torch.Tensor:
    """``[owned rows | halo rows]``: the owned rows copied, the halo rows received from their owners."""
    local = shard.local_nodes
    out = x_local.new_empty((local + shard.halo_rows, *x_local.shape[1:]))
    out[:local] = x_local
    outgoing = x_local.index_select(0, shard.send_rows)
    dist.all_to_all_single(out[local:], outgoing, output_split_sizes=list(shard.recv_counts),
                           input_split_sizes=list(shard.send_counts), group=shard.group)
    return out


def return_halo(full: torch.Tensor, shard: GraphShard) -> torch.Tensor:
    """Inverse of ``exchange_halo`` for gradients: halo rows travel back to their owners and are added to the owned
    rows, one requesting rank after the other."""
    local = shard.local_nodes
    incoming = full.new_empty((sum(shard.send_counts), *full.shape[1:]))
    dist.all_to_all_single(incoming, full[local:].contiguous(), output_split_sizes=list(shard.send_counts),
                           input_split_sizes=list(shard.recv_counts), group=shard.group)
    return _add_returned_rows(full[:local].clone(), incoming, shard)


def _add_returned_rows(own: torch.Tensor, incoming: torch.Tensor, shard: GraphShard) -> torch.Tensor:
    """Adds the gradient rows that came back from the other ranks to the owned rows, one requesting rank after the
    other: the rows one rank asked for are distinct, so each of these adds has a fixed result."""
    offset = 0
    for count in shard.send_counts:
        if count:
            own.index_add_(0, shard.send_rows[offset:offset + count], incoming[offset:offset + count])
            offset += count
    return own


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, shard):
        ctx.shard = shard
        return exchange_halo(x_local, shard)

    @staticmethod
    def backward(ctx, grad_full):
        if grad_full is None:
            return None, None
        return _Scatter.apply(grad_full, ctx.shard), None


class _Scatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, full, shard):
        ctx.shard = shard
        return return_halo(full, shard)

    @staticmethod
    def backward(ctx, grad_local):
        if grad_local is None:
            return None, None
        return _Gather.apply(grad_local, ctx.shard), None


def gather_sources(x_local: torch.Tensor, shard: GraphShard) -> torch.Tensor:
    """The feature rows this rank's edges read, ``[owned rows | halo rows]``; differentiable."""
    if shard.world_size == 1:
        return x_local
    return _Gather.apply(x_local, shard)


def scatter_source_gradients(full: torch.Tensor, shard: GraphShard) -> torch.Tensor:
    """Gradient rows of the compact buffer summed onto their owners; differentiable."""
    if shard.world_size == 1:
        return full
    return _Scatter.apply(full, shard)


def sharded_conv(conv, x_local: torch.Tensor, edge_attr: torch.Tensor, weight: torch.Tensor,
                 shard: GraphShard) -> torch.Tensor:
    """``conv`` (a ``TensorProductConv`` or any callable with its signature) on this rank's destination range.

    ``x_local`` holds the features of the nodes this rank owns; ``edge_attr`` and ``weight`` are the rank's edge
    slice.  Returns the output rows of the owned nodes.
    """
    return conv(gather_sources(x_local, shard), edge_attr, weight, graph=shard.graph)


_side_streams: dict = {}


def _side_stream(device) -> "torch.cuda.Stream":
    key = torch.device(device)
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(key)
    return _side_streams[key]


def overlapped_step(op, x_local: torch.Tensor, edge_attr: torch.Tensor, weight: torch.Tensor,
                    grad_out: torch.Tensor, shard: GraphShard, *, halo_rows: torch.Tensor | None = None,
                    events=None):
    """Forward and first derivatives on this rank's shard with both halo exchanges hidden behind kernels.

    The destinations of a shard whose sources are all owned form (for a spatially ordered partition) one long
    interior run; the rest sit at the two ends of the range.  The three runs are three pieces of the
    destination-sorted edge list (``LunaTPGraph.destination_range``), so:

    * forward: the ``x`` halo travels on a side stream while the interior piece runs; the two end pieces follow;
    * backward: the end pieces run first - they alone produce gradient rows for the halo - then those rows travel
      back while the interior piece runs, and are added to the owned rows at the end (one peer after the other, as
      in ``return_halo``).

    Returns ``(out, gx_local, gy, gw)`` for the owned rows and the rank's edges; the values are those of
    ``exchange_halo`` + one forward + one backward + ``return_halo``.  ``op`` is the prepared operator
    (``TensorProductConv(...).op``).  ``halo_rows`` replaces the forward exchange with rows the caller already has
    and skips the return exchange (``gx`` then has the compact buffer's rows): this is how one rank of a partition
    is checked on a single GPU.  ``events``: optional five CUDA events recorded at start, after the forward
    exchange was enqueued, after the forward pieces, after the backward pieces, at the end.
    """
    from .conv import run_backward, run_forward

    graph, local, halo = shard.graph, shard.local_nodes, shard.halo_rows
    lo, hi = shard.interior
    exchange = halo_rows is None and shard.world_size > 1
    main = torch.cuda.current_stream(x_local.device)
    side = _side_stream(x_local.device)
    mark = (lambda i: events[i].record(main)) if events is not None else (lambda i: None)
    pieces = [(b, e, *graph.destination_range(b, e)) for b, e in ((0, lo), (hi, local), (lo, hi)) if e > b]
    ends, inner = [p for p in pieces if (p[0], p[1]) != (lo, hi)], [p for p in pieces if (p[0], p[1]) == (lo, hi)]

    mark(0)
    full = x_local.new_empty((local + halo, *x_local.shape[1:]))
    full[:local] = x_local
    arrived = torch.cuda.Event()
    if exchange:
        ready = torch.cuda.Event()
        ready.record(main)
        with torch.cuda.stream(side):
            side.wait_event(ready)
            outgoing = x_local.index_select(0, shard.send_rows)
            dist.all_to_all_single(full[local:], outgoing, output_split_sizes=list(shard.recv_counts),
                                   input_split_sizes=list(shard.send_counts), group=shard.group)
            arrived.record(side)
            outgoing.record_stream(side)
    elif halo:
        full[local:] = halo_rows
    mark(1)
    out = x_local.new_empty((local, op.out_dim))
    for begin, end, piece, e0, e1 in inner:  # reads owned rows only
        run_forward(op, full, edge_attr[e0:e1], weight[e0:e1], piece, out=out[begin:end])
    if exchange:
        main.wait_event(arrived)
    for begin, end, piece, e0, e1 in ends:
        run_forward(op, full, edge_attr[e0:e1], weight[e0:e1], piece, out=out[begin:end])
    mark(2)

    gx_full = torch.zeros_like(full)
    gy, gw = torch.empty_like(edge_attr), torch.empty_like(weight)

    def backward_piece(begin, end, piece, e0, e1):
        run_backward(op, full, edge_attr[e0:e1], weight[e0:e1], grad_out[begin:end], piece,
                     out=(gx_full, gy[e0:e1], gw[e0:e1]), add_gx=True)

    for item in ends:
        backward_piece(*item)
    incoming, returned = None, torch.cuda.Event()
    if exchange:
        produced = torch.cuda.Event()
        produced.record(main)
        with torch.cuda.stream(side):
            side.wait_event(produced)
            incoming = gx_full.new_empty((sum(shard.send_counts), *gx_full.shape[1:]))
            dist.all_to_all_single(incoming, gx_full[local:], output_split_sizes=list(shard.send_counts),
                                   input_split_sizes=list(shard.recv_counts), group=shard.group)
            returned.record(side)
    for item in inner:  # adds to owned rows only
        backward_piece(*item)
    mark(3)
    if not exchange:
        mark(4)
        return out, (gx_full if halo_rows is not None else gx_full[:local]), gy, gw
    main.wait_event(returned)
    incoming.record_stream(main)
    own = _add_returned_rows(gx_full[:local], incoming, shard)
    mark(4)
    return out, own, gy, gw


def balanced_node_ranges(dst_rowptr: torch.Tensor, parts: int) -> list[tuple[int, int]]:
    """Contiguous destination ranges with near-equal edge counts (row-pointer search, not node counts)."""
    rowptr = dst_rowptr.to("cpu", torch.int64)
    total, nodes = int(rowptr[-1]), rowptr.numel() - 1
    cuts = [0]
    for part in range(1, parts):
        cuts.append(int(torch.searchsorted(rowptr, torch.tensor(total * part // parts)).clamp(max=nodes)))
    cuts.append(nodes)
    return [(cuts[i], max(cuts[i], cuts[i + 1])) for i in range(parts)]


__all__ = ["GraphShard", "make_graph_shard", "gather_sources", "scatter_source_gradients", "exchange_halo",
           "return_halo", "sharded_conv", "overlapped_step", "balanced_node_ranges"]
