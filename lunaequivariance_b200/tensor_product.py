"""UVU tensor product of independent items (no graph): ``z[n] = TP(x[n], y[n]; w[n])``.

Counterpart of the reference's ``LunaTPUVU`` / ``tensor_product`` (``src/lunatp/interface.py:210-235,291-312``,
``src/lunatp/uvu/interface.py:26-297``).  The reference generates a separate kernel family for this; here it is the
graph convolution on the *identity graph*, in which item ``n`` is the one source of destination ``n``: the gather reads
row ``n``, the scatter-sum has one term, and every derivative order of the convolution carries over unchanged.  The
kernels read consecutive rows, so the gather costs nothing extra.

Weights are one row per item, or a single shared vector ``[weight_numel]`` when the paths were prepared with
``shared_weights=True`` (expanded to one row per item before the launch, since the kernels stream per-item rows).
"""

from __future__ import annotations

from copy import copy

import torch

from .conv import LunaTPUVUConv, lunatp_uvu_conv_func
from .graph import make_graph
from .paths import TensorProductPaths, build_uvu_conv_metadata


class LunaTPUVU:
    """Prepared UVU tensor product for one path list and dtype."""

    mode = "uvu"
    index_mode = "uvu"

    def __init__(self, tp, *, dtype=None, index_bits: int = 32):
        tp = TensorProductPaths.from_tensor_product(tp)
        self.tp = tp
        self.compute_dtype = tp.dtype if dtype is None else dtype
        if self.compute_dtype not in (torch.float32, torch.float64):
            raise ValueError("UVU supports float32 and float64 inputs")
        self.shared_weights = bool(tp.shared_weights)
        self.weight_mode = "shared" if self.shared_weights else "external"
        per_item = copy(tp)  # the kernels always see one weight row per item
        per_item.shared_weights = False
        per_item.internal_weights = False
        self.meta = build_uvu_conv_metadata(per_item, self.compute_dtype)
        self.index_bits = index_bits
        self.conv = LunaTPUVUConv(self.meta, dtype=self.compute_dtype, index_bits=index_bits)
        self.in1_dim, self.in2_dim = self.conv.in1_dim, self.conv.in2_dim
        self.out_dim, self.weight_numel = self.conv.out_dim, self.conv.weight_numel
        self._graphs: dict = {}

    def identity_graph(self, items: int, device):
        """The graph whose only edge into item ``n`` comes from item ``n``; kept for the sizes seen recently."""
        key = (items, str(device))
        graph = self._graphs.get(key)
        if graph is None:
            if len(self._graphs) >= 8:
                self._graphs.pop(next(iter(self._graphs)))
            own = torch.arange(items, device=device, dtype=torch.int32)
            graph = self._graphs[key] = make_graph(own, own, items)
        return graph

    @staticmethod
    def run(op, x, y, weight):
        return lunatp_uvu_func(op, x, y, weight)


def lunatp_uvu_func(op: LunaTPUVU, x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``x[..., in1_dim]``, ``y[..., in2_dim]`` with equal leading shapes; returns ``[..., out_dim]``."""
    if weight is None:
        raise TypeError("UVU tensor products require weights (shared or one row per item)")
    if x.shape[-1] != op.in1_dim or y.shape[-1] != op.in2_dim:
        raise ValueError(f"expected last dimensions {op.in1_dim} and {op.in2_dim}, got {x.shape[-1]} and {y.shape[-1]}")
    if x.shape[:-1] != y.shape[:-1]:
        raise ValueError("x and y must have equal leading shapes")
    batch = x.shape[:-1]
    items = int(torch.Size(batch).numel())
    x2, y2 = x.reshape(items, op.in1_dim), y.reshape(items, op.in2_dim)
    if weight.ndim == 1:
        if not op.shared_weights:
            raise ValueError("a single weight vector needs paths prepared with shared_weights=True")
        if weight.shape[0] != op.weight_numel:
            raise ValueError(f"shared weights must have shape ({op.weight_numel},), got {tuple(weight.shape)}")
        w2 = weight.unsqueeze(0).expand(items, op.weight_numel)
    else:
        if weight.shape[-1] != op.weight_numel or weight.shape[:-1] != batch:
            raise ValueError(f"weights must have shape {tuple(batch) + (op.weight_numel,)}, got {tuple(weight.shape)}")
        w2 = weight.reshape(items, op.weight_numel)
    if items == 0:
        return x.new_zeros(batch + (op.out_dim,)) + 0.0 * (x2.sum() + y2.sum() + w2.sum())
    out = lunatp_uvu_conv_func(op.conv, x2, y2, w2, graph=op.identity_graph(items, x.device))
    return out.reshape(batch + (op.out_dim,))


__all__ = ["LunaTPUVU", "lunatp_uvu_func"]
