"""Functional entry points: ``prepare_tensor_product``, ``tensor_product_conv`` and ``tensor_product``.

Same names, arguments and error messages as the reference (``src/lunatp/interface.py:147-262``), restricted to
``uvu`` instructions: the graph convolution with explicit per-edge weights (``convolution=True``) and the tensor
product of independent items (``convolution=False``).

``TensorProductConv`` and ``prepare_tensor_product`` accept the same three kinds of first argument (irreps strings,
a tensor-product-like object, prebuilt path metadata).  Both go through ``resolve_source`` below, which sorts the
argument out once; the two callers differ only in the words of their error messages, which are part of the public
behaviour and are passed in.
"""

from __future__ import annotations

from collections.abc import Mapping
from copy import copy
from dataclasses import dataclass
from functools import lru_cache

import torch

from .conv import LunaTPUVUConv, create_uvu_conv_operator
from .irreps import as_irreps
from .paths import TensorProductPaths
from .tensor_product import LunaTPUVU

PATH_OPTIONS = ("in1_var", "in2_var", "out_var", "irrep_normalization", "path_normalization")
_MODES = frozenset(("uuu", "uvu", "uvw"))


@dataclass
class ResolvedSource:
    """What an operator is built from: ``source`` is path metadata (a mapping) or a tensor-product-like object."""

    source: object
    from_metadata: bool
    mode: str


def connection_mode_of(instructions, message: str) -> str:
    """The single connection mode of an instruction list; ``message`` is raised if there is not exactly one."""
    found = {instruction.connection_mode for instruction in instructions}
    if len(found) == 1 and found <= _MODES:
        return next(iter(found))
    raise ValueError(message)


def resolve_source(first, *, build, mode, metadata_message: str, mode_message: str) -> ResolvedSource:
    """Classify the first constructor argument.

    ``first`` is prebuilt metadata, an object that already carries instructions, or anything else, in which case
    ``build()`` is called to make the tensor-product object from the remaining arguments.
    """
    if isinstance(first, Mapping):
        if mode not in ("uuu", "uvu"):
            raise ValueError(metadata_message)
        return ResolvedSource(first, True, mode)
    product = first if hasattr(first, "instructions") else build()
    inferred = connection_mode_of(product.instructions, mode_message)
    if mode not in (None, inferred):
        raise ValueError("mode must match the tensor-product instructions")
    return ResolvedSource(product, False, inferred)


def require_uvu(mode: str, what: str) -> None:
    if mode != "uvu":
        raise NotImplementedError(f"this build provides the uvu convolution only, got {what} {mode!r}")


def prepare_tensor_product(irreps_in1, irreps_in2=None, irreps_out=None, instructions=None, *, in1_var=None,
                           in2_var=None, out_var=None, irrep_normalization=None, path_normalization=None,
                           shared_weights=False, dtype=torch.float32, convolution=False, mode=None):
    """Prepare parameter-free paths and the native plan for repeated calls."""
    options = dict(in1_var=in1_var, in2_var=in2_var, out_var=out_var, irrep_normalization=irrep_normalization,
                   path_normalization=path_normalization)

    def build():
        if None in (irreps_in2, irreps_out, instructions):
            raise TypeError("All three irreps and instructions are required")
        return TensorProductPaths(irreps_in1, irreps_in2, irreps_out, instructions, internal_weights=False,
                                  shared_weights=shared_weights, **options)

    if isinstance(irreps_in1, Mapping) and not convolution:
        mode = None  # metadata is only meaningful for convolutions: fall into the metadata error below
    resolved = resolve_source(
        copy(irreps_in1) if isinstance(irreps_in1, TensorProductPaths) else irreps_in1, build=build, mode=mode,
        metadata_message='Metadata requires convolution=True and mode="uuu" or "uvu"',
        mode_message="Tensor products require one connection mode: uuu, uvu or uvw")
    require_uvu(resolved.mode, "mode")
    if not resolved.from_metadata:
        resolved.source.dtype = dtype
        if not convolution:
            return LunaTPUVU(resolved.source, dtype=dtype)
    return create_uvu_conv_operator(resolved.source, dtype=dtype)


@lru_cache(maxsize=128)
def _prepared_from_strings(irreps_in1, irreps_in2, irreps_out, instructions, in1_var, in2_var, out_var,
                           irrep_normalization, path_normalization, shared_weights, dtype):
    return prepare_tensor_product(
        irreps_in1, irreps_in2, irreps_out, instructions, in1_var=in1_var, in2_var=in2_var, out_var=out_var,
        irrep_normalization=irrep_normalization, path_normalization=path_normalization,
        shared_weights=shared_weights, dtype=dtype, convolution=True)


def _hashable(value):
    return None if value is None else tuple(value)


def tensor_product_conv(x, edge_attr, weight=None, *, graph, irreps_in1=None, irreps_in2=None, irreps_out=None,
                        instructions=None, in1_var=None, in2_var=None, out_var=None, irrep_normalization=None,
                        path_normalization=None, shared_weights=False, config=None, **kwargs):
    """Contract edge messages and sum by destination, with explicit weights and an explicit graph."""
    if config is None:
        if None in (irreps_in1, irreps_in2, irreps_out, instructions):
            raise TypeError("Supply irreps and instructions, or a prepared config")
        config = _prepared_from_strings(
            *(str(as_irreps(r)) for r in (irreps_in1, irreps_in2, irreps_out)),
            tuple(tuple(i) for i in instructions), _hashable(in1_var), _hashable(in2_var), _hashable(out_var),
            irrep_normalization, path_normalization, shared_weights, x.dtype)
    if not isinstance(config, LunaTPUVUConv):
        raise TypeError("config must come from prepare_tensor_product(..., convolution=True)")
    return config.run(config, x, edge_attr, weight, graph=graph, **kwargs)


def tensor_product(x, y, weight=None, *, irreps_in1=None, irreps_in2=None, irreps_out=None, instructions=None,
                   in1_var=None, in2_var=None, out_var=None, irrep_normalization=None, path_normalization=None,
                   shared_weights=False, config=None):
    """Independent tensor products, one per item; shared weights are ``[weight_numel]``, external weights one row
    per item."""
    if config is None:
        if None in (irreps_in1, irreps_in2, irreps_out, instructions):
            raise TypeError("Supply irreps and instructions, or a prepared config")
        config = _prepared_item_product(
            *(str(as_irreps(r)) for r in (irreps_in1, irreps_in2, irreps_out)),
            tuple(tuple(i) for i in instructions), _hashable(in1_var), _hashable(in2_var), _hashable(out_var),
            irrep_normalization, path_normalization, shared_weights, x.dtype)
    if not isinstance(config, LunaTPUVU):
        raise TypeError("config must come from prepare_tensor_product(..., convolution=False)")
    return config.run(config, x, y, weight)


@lru_cache(maxsize=128)
def _prepared_item_product(irreps_in1, irreps_in2, irreps_out, instructions, in1_var, in2_var, out_var,
                           irrep_normalization, path_normalization, shared_weights, dtype):
    return prepare_tensor_product(
        irreps_in1, irreps_in2, irreps_out, instructions, in1_var=in1_var, in2_var=in2_var, out_var=out_var,
        irrep_normalization=irrep_normalization, path_normalization=path_normalization,
        shared_weights=shared_weights, dtype=dtype, convolution=False)


__all__ = ["prepare_tensor_product", "tensor_product_conv", "tensor_product"]
