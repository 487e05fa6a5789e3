"""``torch.nn.Module`` shells: ``TensorProductConv`` and ``SphericalHarmonics``.

Constructor arguments, attributes and dtype migration follow the reference's
``src/modules/tensorproduct.py:119-206`` and ``src/modules/spherical_harmonics.py:13-129``.
"""

from __future__ import annotations

from collections.abc import Mapping

import torch

from .conv import create_uvu_conv_operator
from .functional import require_uvu, resolve_source, tensor_product, tensor_product_conv
from .graph import make_graph
from .paths import TensorProductConfig
from .tensor_product import LunaTPUVU
from .spherical_harmonics import UNSET, SphericalHarmonicsConfig, spherical_harmonics


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
        options = dict(in1_var=in1_var, in2_var=in2_var, out_var=out_var, irrep_normalization=irrep_normalization,
                       path_normalization=path_normalization, internal_weights=internal_weights,
                       shared_weights=shared_weights)
        prebuilt = isinstance(irreps_in1, (Mapping, torch.nn.Module))
        if prebuilt and not all(v is None for v in (irreps_in2, irreps_out, instructions, *options.values())):
            raise TypeError("Pass either an existing tensor product/metadata or irreps and path options")

        def build():
            if None in (irreps_in2, irreps_out, instructions):
                raise TypeError("irreps_in2, irreps_out and instructions are required")
            product = TensorProductConfig(irreps_in1, irreps_in2, irreps_out, instructions, **options)
            if dtype is not None and product.weight.dtype != dtype:
                product.to(dtype=dtype)
            return product

        resolved = resolve_source(
            irreps_in1, build=build, mode=mode,
            metadata_message='Prebuilt metadata requires mode="uuu" or mode="uvu"',
            mode_message="TensorProductConv requires one connection mode: uuu, uvu or uvw")
        require_uvu(resolved.mode, "mode")
        source = resolved.source
        if dtype is None:
            dtype = torch.float32 if resolved.from_metadata else source.weight.dtype
        self.mode = "uvu_conv"
        self.op = create_uvu_conv_operator(source, dtype=dtype)
        if resolved.from_metadata:
            self.weight_numel = source["weight_numel"]
            self.internal_weights = self.shared_weights = False
            return
        self.tp = source
        for name in ("irreps_in1", "irreps_in2", "irreps_out", "instructions", "weight_numel", "internal_weights",
                     "shared_weights"):
            setattr(self, name, getattr(source, name))
        self.train(getattr(source, "training", True))

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


class TensorProduct(torch.nn.Module):
    """UVU tensor product of independent items with e3nn path and normalisation arguments.

    Pass irreps and ``uvu`` instructions, or an existing tensor-product-like module/configuration
    (``src/modules/tensorproduct.py:19-117``).  Weights are one row per item, or a shared vector when the paths
    have ``shared_weights=True`` (with ``internal_weights=True`` the module owns it).
    """

    def __init__(self, irreps_in1, irreps_in2=None, irreps_out=None, instructions=None, in1_var=None, in2_var=None,
                 out_var=None, irrep_normalization=None, path_normalization=None, internal_weights=None,
                 shared_weights=None, *, dtype=None):
        super().__init__()
        options = dict(in1_var=in1_var, in2_var=in2_var, out_var=out_var, irrep_normalization=irrep_normalization,
                       path_normalization=path_normalization, internal_weights=internal_weights,
                       shared_weights=shared_weights)
        if isinstance(irreps_in1, torch.nn.Module) and not all(
                v is None for v in (irreps_in2, irreps_out, instructions, *options.values())):
            raise TypeError("Pass either an existing tensor product or irreps and path options")

        def build():
            if None in (irreps_in2, irreps_out, instructions):
                raise TypeError("irreps_in2, irreps_out and instructions are required")
            product = TensorProductConfig(irreps_in1, irreps_in2, irreps_out, instructions, **options)
            if dtype is not None and product.weight.dtype != dtype:
                product.to(dtype=dtype)
            return product

        resolved = resolve_source(
            irreps_in1, build=build, mode=None, metadata_message="TensorProduct takes irreps or a tensor product",
            mode_message="TensorProduct requires one connection mode: uuu, uvu or uvw")
        require_uvu(resolved.mode, "mode")
        source = resolved.source
        self.mode = resolved.mode
        self.op = LunaTPUVU(source, dtype=dtype)
        self.tp = source
        for name in ("irreps_in1", "irreps_in2", "irreps_out", "instructions", "weight_numel", "internal_weights",
                     "shared_weights"):
            setattr(self, name, getattr(source, name))
        self.train(getattr(source, "training", True))

    @property
    def weight(self):
        return getattr(self.tp, "weight", None)

    def _apply(self, fn, recurse=True):
        dtype = fn(torch.empty(0, dtype=self.op.compute_dtype)).dtype
        if dtype not in (torch.float32, torch.float64):
            raise ValueError("Tensor products support float32 and float64 inputs")
        result = super()._apply(fn, recurse=recurse)
        if dtype != self.op.compute_dtype:
            self.op = LunaTPUVU(self.tp, dtype=dtype, index_bits=self.op.index_bits)
        return result

    def forward(self, x, y, weight=None):
        if weight is None and self.internal_weights:
            weight = self.weight
        return tensor_product(x, y, weight, config=self.op)


_SH_DTYPES = (torch.float16, torch.bfloat16, torch.float32, torch.float64)


def _checked_sh_dtype(dtype):
    if dtype not in _SH_DTYPES:
        raise ValueError("SphericalHarmonics requires a floating dtype")
    return dtype


class SphericalHarmonics(torch.nn.Module):
    """Real spherical harmonics of a 3-vector, e3nn conventions, degrees through 12.

    The module is a thin holder of one ``SphericalHarmonicsConfig``; ``irreps_in``, ``irreps_out``, ``normalize``
    and ``normalization`` read through to it.  ``.to()/.double()/.float()`` move a zero-element anchor tensor, which is
    how the module learns its new dtype.
    """

    def __init__(self, irreps_out, normalize=UNSET, normalization="integral", irreps_in=None, *, dtype=None):
        super().__init__()
        if hasattr(irreps_out, "_ls_list"):  # another harmonics module (this library's, the reference's, e3nn's)
            template, irreps_out = irreps_out, tuple(irreps_out._ls_list)
            normalize, normalization, irreps_in = template.normalize, template.normalization, template.irreps_in
            self.training = template.training
        if normalize is UNSET:
            raise TypeError("SphericalHarmonics requires normalize=True or False")
        if normalization not in ("component", "norm", "integral"):
            raise ValueError("normalization must be component, norm or integral")
        self._dtype_anchor = torch.empty(0, dtype=_checked_sh_dtype(torch.get_default_dtype() if dtype is None else dtype))
        self._config = SphericalHarmonicsConfig(irreps_out, normalize, normalization, self._dtype_anchor.dtype,
                                                irreps_in=irreps_in)
        # the kernels evaluate in the dtype of the input, whatever the module's own dtype: one config for each
        self._by_dtype = {
            t: SphericalHarmonicsConfig(self._config._ls_list, self._config.normalize, normalization, t,
                                        irreps_in=str(self._config.irreps_in))
            for t in (torch.float32, torch.float64)}
        self.last_execution_backend = "uninitialized"

    irreps_in = property(lambda self: self._config.irreps_in)
    irreps_out = property(lambda self: self._config.irreps_out)
    normalize = property(lambda self: self._config.normalize)
    normalization = property(lambda self: self._config.normalization)
    compute_dtype = property(lambda self: self._dtype_anchor.dtype)
    _ls_list = property(lambda self: list(self._config._ls_list))
    _lmax = property(lambda self: self._config._lmax)

    def _apply(self, fn, recurse=True):
        moved = fn(self._dtype_anchor)
        _checked_sh_dtype(moved.dtype)
        result = super()._apply(fn, recurse=recurse)
        self._dtype_anchor = moved
        return result

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        config = self._by_dtype.get(x.dtype, self._config)
        result = spherical_harmonics(config._ls_list, x, config.normalize, config.normalization, config=config)
        self.last_execution_backend = "cuda_fused"
        return result


LunaEqSphericalHarmonics = SphericalHarmonics

__all__ = ["TensorProductConv", "TensorProduct", "SphericalHarmonics", "LunaEqSphericalHarmonics"]
