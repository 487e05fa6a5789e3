"""``torch.nn.Module`` shells: ``TensorProductConv`` and ``SphericalHarmonics``.

Constructor arguments, attributes and dtype migration follow the reference's
``src/modules/tensorproduct.py:119-206`` and ``src/modules/spherical_harmonics.py:13-129``.
"""

from __future__ import annotations

from collections.abc import Mapping

import torch

from .conv import create_uvu_conv_operator
from .functional import tensor_product_conv
from .graph import make_graph
from .paths import TensorProductConfig
from .spherical_harmonics import UNSET, SphericalHarmonicsConfig, parse_irreps, spherical_harmonics


class TensorProductConv(torch.nn.Module):
    """Fused UVU tensor product and destination-sorted graph aggregation.

    Pass irreps and ``uvu`` instructions, an existing tensor-product-like module/configuration, or prebuilt
    metadata with ``mode="uvu"``.  Weights are explicit per-edge inputs.  Prepare the topology once with
    ``create_graph`` and pass it on every call.
    """

    def __init__(self, irreps_in1, irreps_in2=None, irreps_out=None, instructions=None, in1_var=None, in2_var=None,
                 out_var=None, irrep_normalization=None, path_normalization=None, internal_weights=None,
                 shared_weights=None, *, dtype=None, mode=None):
        super().__init__()
        metadata = isinstance(irreps_in1, Mapping)
        if metadata or isinstance(irreps_in1, torch.nn.Module):
            if any(v is not None for v in (irreps_in2, irreps_out, instructions, in1_var, in2_var, out_var,
                                           irrep_normalization, path_normalization, internal_weights,
                                           shared_weights)):
                raise TypeError("Pass either an existing tensor product/metadata or irreps and path options")
            tp = irreps_in1
        else:
            if irreps_in2 is None or irreps_out is None or instructions is None:
                raise TypeError("irreps_in2, irreps_out and instructions are required")
            tp = TensorProductConfig(
                irreps_in1, irreps_in2, irreps_out, instructions, in1_var=in1_var, in2_var=in2_var,
                out_var=out_var, irrep_normalization=irrep_normalization, path_normalization=path_normalization,
                internal_weights=internal_weights, shared_weights=shared_weights)
            if dtype is not None and tp.weight.dtype != dtype:
                tp.to(dtype=dtype)
        if metadata:
            if mode not in ("uuu", "uvu"):
                raise ValueError('Prebuilt metadata requires mode="uuu" or mode="uvu"')
            dtype = torch.float32 if dtype is None else dtype
        else:
            modes = {instruction.connection_mode for instruction in tp.instructions}
            if len(modes) != 1 or not modes <= {"uuu", "uvu", "uvw"}:
                raise ValueError("TensorProductConv requires one connection mode: uuu, uvu or uvw")
            inferred = modes.pop()
            if mode is not None and mode != inferred:
                raise ValueError("mode must match the tensor-product instructions")
            mode = inferred
            dtype = tp.weight.dtype if dtype is None else dtype
        if mode != "uvu":
            raise NotImplementedError(f"this build provides the uvu convolution only, got mode {mode!r}")
        self.mode = "uvu_conv"
        self.op = create_uvu_conv_operator(tp, dtype=dtype)
        if metadata:
            self.weight_numel = tp["weight_numel"]
            self.internal_weights = self.shared_weights = False
        else:
            self.tp = tp
            self.irreps_in1, self.irreps_in2, self.irreps_out = tp.irreps_in1, tp.irreps_in2, tp.irreps_out
            self.instructions = tp.instructions
            self.weight_numel = tp.weight_numel
            self.internal_weights, self.shared_weights = tp.internal_weights, tp.shared_weights
            self.train(getattr(tp, "training", True))

    @property
    def weight(self):
        tp = getattr(self, "tp", None)
        return tp.weight if tp is not None else None

    def _apply(self, fn, recurse=True):
        dtype = fn(torch.empty(0, dtype=self.op.compute_dtype)).dtype
        if dtype not in (torch.float32, torch.float64):
            raise ValueError("Tensor products support float32 and float64 inputs")
        result = super()._apply(fn, recurse=recurse)
        if dtype != self.op.compute_dtype:
            source = self.tp if hasattr(self, "tp") else self.op.meta
            self.op = create_uvu_conv_operator(source, dtype=dtype)
        return result

    @staticmethod
    def create_graph(src, dst, num_nodes=None, **kwargs):
        """Prepare the shared topology once per batch."""
        return make_graph(src, dst, num_nodes, **kwargs)

    def forward(self, x, edge_attr, weight=None, *, graph, **kwargs):
        if weight is None and self.internal_weights:
            weight = self.weight
        return tensor_product_conv(x, edge_attr, weight, graph=graph, config=self.op, **kwargs)


class SphericalHarmonics(torch.nn.Module):
    """Real spherical harmonics of a 3-vector, e3nn conventions, degrees through 12."""

    def __init__(self, irreps_out, normalize=UNSET, normalization="integral", irreps_in=None, *, dtype=None):
        super().__init__()
        if hasattr(irreps_out, "_ls_list"):
            other = irreps_out
            self.training = other.training
            irreps_out, normalize, normalization, irreps_in = (
                tuple(other._ls_list), other.normalize, other.normalization, other.irreps_in)
        if normalize is UNSET:
            raise TypeError("SphericalHarmonics requires normalize=True or False")
        if normalization not in ("component", "norm", "integral"):
            raise ValueError("normalization must be component, norm or integral")
        if dtype is None:
            dtype = torch.get_default_dtype()
        if dtype not in (torch.float16, torch.bfloat16, torch.float32, torch.float64):
            raise ValueError("SphericalHarmonics requires a floating dtype")
        self.irreps_in, self.irreps_out, degrees = parse_irreps(irreps_out, irreps_in)
        self._ls_list = list(degrees)
        self._lmax = max(degrees)
        self.normalize, self.normalization = bool(normalize), normalization
        self.compute_dtype = dtype
        self._dtype_anchor = torch.empty(0, dtype=dtype)
        self.last_execution_backend = "uninitialized"

    def _apply(self, fn, recurse=True):
        anchor = fn(self._dtype_anchor)
        if anchor.dtype not in (torch.float16, torch.bfloat16, torch.float32, torch.float64):
            raise ValueError("SphericalHarmonics requires a floating dtype")
        result = super()._apply(fn, recurse=recurse)
        self._dtype_anchor = anchor
        self.compute_dtype = anchor.dtype
        return result

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        config = SphericalHarmonicsConfig(tuple(self._ls_list), self.normalize, self.normalization, x.dtype,
                                          irreps_in=str(self.irreps_in))
        result = spherical_harmonics(self._ls_list, x, self.normalize, self.normalization, config=config)
        self.last_execution_backend = "cuda_fused"
        return result


LunaEqSphericalHarmonics = SphericalHarmonics

__all__ = ["TensorProductConv", "SphericalHarmonics", "LunaEqSphericalHarmonics"]
