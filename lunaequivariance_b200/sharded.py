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
    graph = make_graph(compact, dst_global.to(torch.int64) - begin, local, num_src_nodes=local + halo_ids.numel())

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
                      recv_counts=tuple(recv_list), send_counts=tuple(send_list), send_rows=send_rows, group=group)


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
    own = full[:local].clone()
    offset = 0
    for count in shard.send_counts:
        if count:  # the rows one rank asked for are distinct, so each of these adds has a fixed result
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
           "return_halo", "sharded_conv", "balanced_node_ranges"]
