"""Forward and first derivatives of the convolution for per-edge tensors that live in host memory.

The per-edge tensors dominate the bytes of this operator (for 128 channels and degrees up to 3 a weight row is 8.7 KB
per edge against a few KB per *node* for the features), and a caller that keeps them in host memory - because they do
not fit beside the model, or because another process produces them - pays for two PCIe crossings per step: weights
and edge attributes in, their gradients out.  Run as "copy everything in, compute, copy everything out" the two
directions never overlap and the link is idle during the kernels.

``HostStreamedConv`` cuts the graph's destination nodes into chunks.  A chunk is a contiguous slice of the
destination-sorted edge list (``LunaTPGraph.destination_range``), so its per-edge tensors are contiguous slices of the
host tensors.  Three streams run a pipeline over the chunks: the upload of chunk ``c + 1``, the two kernels of chunk
``c`` and the download of the gradients of chunk ``c - 1`` proceed at the same time, and PCIe carries traffic in both
directions for the whole step.  Node features and their gradients stay on the device for the whole step; the
source-row gradient is accumulated across chunks by the kernels (``luna_uvu_conv_bwd_add_gx``).

The reference has no counterpart (its operators take device tensors only); results are those of one call on the
whole graph, bit for bit in ``out``, ``gy`` and ``gw`` and up to the order of the per-chunk additions in ``gx``.
"""

from __future__ import annotations

import torch

from .conv import LunaTPUVUConv, run_backward, run_forward
from .graph import LunaTPGraph


def _pinned_like(shape, dtype) -> torch.Tensor:
    try:
        return torch.empty(shape, dtype=dtype, pin_memory=True)
    except RuntimeError:  # no pinned memory left: pageable memory works, without overlap
        return torch.empty(shape, dtype=dtype)


class HostStreamedConv:
    """``step(x, edge_attr, weight, grad_out)`` with host tensors in and host tensors out.

    ``op`` is a prepared operator (``TensorProductConv(...).op`` or ``prepare_tensor_product(..., convolution=True)``),
    ``graph`` a device graph.  ``chunks`` bounds the device memory used for per-edge data: four buffers of about
    ``edges / chunks`` rows each for weights and for weight gradients.
    """

    def __init__(self, op: LunaTPUVUConv, graph: LunaTPGraph, *, chunks: int = 16, device=None):
        if graph.src.device.type != "cuda":
            raise RuntimeError("CUDA is required: the graph must be a device graph")
        self.op, self.graph = op, graph
        self.device = torch.device(device) if device is not None else graph.src.device
        nodes = graph.num_nodes
        chunks = max(1, min(int(chunks), max(nodes, 1)))
        # chunk boundaries: equal edge counts, rounded to whole destination nodes
        rowptr = graph.dst_rowptr.to(torch.int64)
        targets = torch.arange(1, chunks, device=rowptr.device, dtype=torch.int64) * graph.num_edges // chunks
        cuts = torch.searchsorted(rowptr, targets).clamp_(0, nodes).tolist()
        bounds = sorted(set([0, *cuts, nodes]))
        self.pieces = [(b, e, *graph.destination_range(b, e)) for b, e in zip(bounds[:-1], bounds[1:])]
        self.max_edges = max((e1 - e0 for _, _, _, e0, e1 in self.pieces), default=0)
        self.upload, self.download = torch.cuda.Stream(self.device), torch.cuda.Stream(self.device)
        self._buffers = None
        self._host_out = None

    def _device_buffers(self, dtype):
        if self._buffers is None or self._buffers[0][0].dtype != dtype:
            op, rows = self.op, max(self.max_edges, 1)
            make = lambda cols: [torch.empty((rows, cols), dtype=dtype, device=self.device) for _ in range(2)]
            self._buffers = (make(op.in2_dim), make(op.weight_numel), make(op.in2_dim), make(op.weight_numel))
        return self._buffers

    def host_outputs(self, dtype):
        """Pinned host tensors the results are written to (reused from step to step)."""
        if self._host_out is None or self._host_out[0].dtype != dtype:
            op, graph = self.op, self.graph
            self._host_out = (_pinned_like((graph.num_nodes, op.out_dim), dtype),
                              _pinned_like((graph.source_rows, op.in1_dim), dtype),
                              _pinned_like((graph.num_edges, op.in2_dim), dtype),
                              _pinned_like((graph.num_edges, op.weight_numel), dtype))
        return self._host_out

    def step(self, x, edge_attr, weight, grad_out):
        """Returns ``(out, gx, gy, gw)``; the tensors are valid when the call returns.

        ``edge_attr [edges, in2]`` and ``weight [edges, weight_numel]`` are host tensors (pinned memory is what makes
        the copies asynchronous); ``gy``, ``gw`` and ``out`` come back as host tensors.  The node features
        ``x [source rows, in1]`` and ``grad_out [nodes, out]`` may be host or device tensors; ``gx`` comes back where
        ``x`` was (a shard of a partitioned graph passes its compact device buffer and sends the halo part of ``gx``
        on to its owners).
        """
        for name, tensor in (("edge_attr", edge_attr), ("weight", weight)):
            if tensor.device.type != "cpu" or not tensor.is_contiguous():
                raise ValueError(f"{name} must be a contiguous host tensor")
        for name, tensor in (("x", x), ("grad_out", grad_out)):
            if not tensor.is_contiguous():
                raise ValueError(f"{name} must be contiguous")
        op, graph, dtype = self.op, self.graph, x.dtype
        if tuple(weight.shape) != (graph.num_edges, op.weight_numel):
            raise ValueError(f"weight must have shape ({graph.num_edges}, {op.weight_numel})")
        if tuple(edge_attr.shape) != (graph.num_edges, op.in2_dim):
            raise ValueError(f"edge_attr must have shape ({graph.num_edges}, {op.in2_dim})")
        out_h, gx_h, gy_h, gw_h = self.host_outputs(dtype)
        y_in, w_in, gy_out, gw_out = self._device_buffers(dtype)
        compute = torch.cuda.current_stream(self.device)
        upload, download = self.upload, self.download
        with torch.cuda.device(self.device):
            start = torch.cuda.Event()
            start.record(compute)
            upload.wait_event(start)
            download.wait_event(start)
            with torch.cuda.stream(upload):
                x_d = x if x.is_cuda else x.to(self.device, non_blocking=True)
                g_d = grad_out if grad_out.is_cuda else grad_out.to(self.device, non_blocking=True)
                nodes_in = torch.cuda.Event()
                nodes_in.record(upload)
            out_d = torch.empty((graph.num_nodes, op.out_dim), dtype=dtype, device=self.device)
            gx_d = torch.zeros((graph.source_rows, op.in1_dim), dtype=dtype, device=self.device)
            compute.wait_event(nodes_in)
            uploaded = [None, None]   # per buffer: event "chunk is on the device"
            computed = [None, None]   # per buffer: event "kernels are done with the input and output buffers"
            drained = [None, None]    # per buffer: event "gradients have left the output buffers"
            for index, (begin, end, piece, e0, e1) in enumerate(self.pieces):
                slot, rows = index % 2, e1 - e0
                with torch.cuda.stream(upload):
                    if computed[slot] is not None:
                        upload.wait_event(computed[slot])  # the kernels two chunks back have read this buffer
                    y_in[slot][:rows].copy_(edge_attr[e0:e1], non_blocking=True)
                    w_in[slot][:rows].copy_(weight[e0:e1], non_blocking=True)
                    uploaded[slot] = torch.cuda.Event()
                    uploaded[slot].record(upload)
                compute.wait_event(uploaded[slot])
                if drained[slot] is not None:
                    compute.wait_event(drained[slot])  # the gradients two chunks back have left this buffer
                y_c, w_c = y_in[slot][:rows], w_in[slot][:rows]
                run_forward(op, x_d, y_c, w_c, piece, out=out_d[begin:end])
                run_backward(op, x_d, y_c, w_c, g_d[begin:end], piece,
                             out=(gx_d, gy_out[slot][:rows], gw_out[slot][:rows]), add_gx=True)
                computed[slot] = torch.cuda.Event()
                computed[slot].record(compute)
                with torch.cuda.stream(download):
                    download.wait_event(computed[slot])
                    gy_h[e0:e1].copy_(gy_out[slot][:rows], non_blocking=True)
                    gw_h[e0:e1].copy_(gw_out[slot][:rows], non_blocking=True)
                    out_h[begin:end].copy_(out_d[begin:end], non_blocking=True)
                    drained[slot] = torch.cuda.Event()
                    drained[slot].record(download)
            if not x.is_cuda:
                with torch.cuda.stream(download):
                    download.wait_event(computed[(len(self.pieces) - 1) % 2] or start)
                    gx_h.copy_(gx_d, non_blocking=True)
            for tensor in (x_d, g_d):  # allocated on the upload stream (if uploaded), read by the kernels
                tensor.record_stream(compute)
            for tensor in (out_d, gx_d):  # allocated on the compute stream, read by the download stream
                tensor.record_stream(download)
            download.synchronize()
            compute.synchronize()
        return out_h, (gx_d if x.is_cuda else gx_h), gy_h, gw_h


__all__ = ["HostStreamedConv"]
