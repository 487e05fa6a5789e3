"""Destination-range partition of the convolution across the ranks of a ``torch.distributed`` process group.

The reference is single-GPU; this module is the multi-GPU design for its convolution.  Each rank owns a contiguous
range of destination nodes, hence one contiguous slice of the destination-sorted edge list with its edge attributes
and per-edge weights - the bulk of the bytes never moves.  Only node features cross ranks:

* forward:  ``x`` rows of all ranks are all-gathered (NCCL over NVLink) into a local buffer the kernels read;
* backward: every rank produces gradient rows for all sources it touched; a reduce-scatter sums them and hands
  each rank the rows of the nodes it owns.

Both collectives are autograd functions whose backward is the other one, so first and second derivatives work.
Rows are padded to the largest shard so that the tensor collectives apply to uneven partitions; source indices are
renumbered into the padded layout once, when the shard is built.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from .graph import LunaTPGraph, make_graph


@dataclass(frozen=True)
class GraphShard:
    """One rank's part of a partitioned graph."""

    graph: LunaTPGraph        # local destinations, sources renumbered into the padded global layout
    node_begin: int           # first global node owned by this rank
    node_counts: tuple        # nodes owned by each rank
    padded_rows: int          # rows per rank in the gathered buffer (max of node_counts)
    group: object = None

    @property
    def local_nodes(self) -> int:
        return self.graph.num_nodes

    @property
    def world_size(self) -> int:
        return len(self.node_counts)


def padded_source_index(src_global: torch.Tensor, node_counts, padded_rows: int) -> torch.Tensor:
    """Map global node ids to rows of the gathered buffer ``[world * padded_rows, dim]``."""
    bounds = torch.tensor([0] + list(node_counts), device=src_global.device, dtype=torch.int64).cumsum(0)
    owner = torch.searchsorted(bounds, src_global.to(torch.int64), right=True) - 1
    return owner * padded_rows + (src_global.to(torch.int64) - bounds[owner])


def make_graph_shard(src_global: torch.Tensor, dst_global: torch.Tensor, node_counts, rank: int,
                     group=None) -> GraphShard:
    """Build this rank's shard from its slice of the edge list (global node ids, ``dst`` ascending and inside the
    rank's node range)."""
    node_counts = tuple(int(c) for c in node_counts)
    begin = sum(node_counts[:rank])
    local = node_counts[rank]
    padded = max(node_counts) if node_counts else 0
    if dst_global.numel():
        low, high = int(dst_global.min()), int(dst_global.max())
        if low < begin or high >= begin + local:
            raise ValueError(f"destination ids must lie in this rank's range [{begin}, {begin + local})")
    src = padded_source_index(src_global, node_counts, padded)
    dst = dst_global.to(torch.int64) - begin
    graph = make_graph(src, dst, local, num_src_nodes=padded * len(node_counts))
    return GraphShard(graph=graph, node_begin=begin, node_counts=node_counts, padded_rows=padded, group=group)


def balanced_node_ranges(dst_rowptr: torch.Tensor, parts: int) -> list[tuple[int, int]]:
    """Contiguous destination ranges with near-equal edge counts (row-pointer search, not node counts)."""
    rowptr = dst_rowptr.to("cpu", torch.int64)
    total, nodes = int(rowptr[-1]), rowptr.numel() - 1
    cuts = [0]
    for part in range(1, parts):
        cuts.append(int(torch.searchsorted(rowptr, torch.tensor(total * part // parts)).clamp(max=nodes)))
    cuts.append(nodes)
    return [(cuts[i], max(cuts[i], cuts[i + 1])) for i in range(parts)]


def _all_gather_rows(x_padded: torch.Tensor, world: int, group) -> torch.Tensor:
    out = x_padded.new_empty((world * x_padded.shape[0], *x_padded.shape[1:]))
    dist.all_gather_into_tensor(out, x_padded.contiguous(), group=group)
    return out


def _reduce_scatter_rows(full: torch.Tensor, world: int, group) -> torch.Tensor:
    rows = full.shape[0] // world
    if dist.get_backend(group) == "gloo":  # gloo has no reduce-scatter: all-reduce and keep the own slice
        total = full.contiguous().clone()
        dist.all_reduce(total, group=group)
        rank = dist.get_rank(group)
        return total[rank * rows:(rank + 1) * rows].contiguous()
    out = full.new_empty((rows, *full.shape[1:]))
    dist.reduce_scatter_tensor(out, full.contiguous(), group=group)
    return out


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, padded_rows, world, group):
        ctx.local_rows, ctx.padded_rows, ctx.world, ctx.group = x_local.shape[0], padded_rows, world, group
        if x_local.shape[0] != padded_rows:
            pad = x_local.new_zeros((padded_rows - x_local.shape[0], *x_local.shape[1:]))
            x_local = torch.cat([x_local, pad], 0)
        return _all_gather_rows(x_local, world, group)

    @staticmethod
    def backward(ctx, grad_full):
        if grad_full is None:
            return None, None, None, None
        return _Scatter.apply(grad_full, ctx.local_rows, ctx.padded_rows, ctx.world, ctx.group), None, None, None


class _Scatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, full, local_rows, padded_rows, world, group):
        ctx.padded_rows, ctx.world, ctx.group = padded_rows, world, group
        return _reduce_scatter_rows(full, world, group)[:local_rows]

    @staticmethod
    def backward(ctx, grad_local):
        if grad_local is None:
            return None, None, None, None, None
        return _Gather.apply(grad_local, ctx.padded_rows, ctx.world, ctx.group), None, None, None, None


def gather_sources(x_local: torch.Tensor, shard: GraphShard) -> torch.Tensor:
    """All ranks' node features in the padded layout ``[world * padded_rows, dim]``; differentiable."""
    if shard.world_size == 1:
        return x_local
    return _Gather.apply(x_local, shard.padded_rows, shard.world_size, shard.group)


def sharded_conv(conv, x_local: torch.Tensor, edge_attr: torch.Tensor, weight: torch.Tensor,
                 shard: GraphShard) -> torch.Tensor:
    """``conv`` (a ``TensorProductConv`` or any callable with its signature) on this rank's destination range.

    ``x_local`` holds the features of the nodes this rank owns; ``edge_attr`` and ``weight`` are the rank's edge
    slice.  Returns the output rows of the owned nodes.
    """
    return conv(gather_sources(x_local, shard), edge_attr, weight, graph=shard.graph)


__all__ = ["GraphShard", "make_graph_shard", "gather_sources", "sharded_conv", "padded_source_index",
           "balanced_node_ranges"]
