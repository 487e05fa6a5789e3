"""Functional entry points: ``prepare_tensor_product`` and ``tensor_product_conv``.

Same names, arguments and errors as the reference (``src/lunatp/interface.py:147-262``), restricted to what the
UVU convolution path needs: ``convolution=True`` with ``uvu`` instructions and explicit per-edge weights.
"""

from __future__ import annotations

from collections.abc import Mapping
from copy import copy
from functools import lru_cache

import torch

from .conv import LunaTPUVUConv, create_uvu_conv_operator
from .irreps import as_irreps
from .paths import TensorProductPaths


def _single_mode(instructions) -> str:
    modes = {instruction.connection_mode for instruction in instructions}
    if len(modes) != 1 or not modes <= {"uuu", "uvu", "uvw"}:
        raise ValueError("Tensor products require one connection mode: uuu, uvu or uvw")
    return modes.pop()


def prepare_tensor_product(irreps_in1, irreps_in2=None, irreps_out=None, instructions=None, *, in1_var=None,
                           in2_var=None, out_var=None, irrep_normalization=None, path_normalization=None,
                           shared_weights=False, dtype=torch.float32, convolution=False, mode=None):
    """Prepare parameter-free paths and the native plan for repeated calls."""
    if isinstance(irreps_in1, Mapping):
        if not convolution or mode not in ("uuu", "uvu"):
            raise ValueError('Metadata requires convolution=True and mode="uuu" or "uvu"')
        if mode != "uvu":
            raise NotImplementedError("this build provides the uvu convolution only")
        return create_uvu_conv_operator(irreps_in1, dtype=dtype)
    if isinstance(irreps_in1, TensorProductPaths):
        paths = copy(irreps_in1)
    else:
        if irreps_in2 is None or irreps_out is None or instructions is None:
            raise TypeError("All three irreps and instructions are required")
        paths = TensorProductPaths(
            irreps_in1, irreps_in2, irreps_out, instructions, in1_var=in1_var, in2_var=in2_var, out_var=out_var,
            irrep_normalization=irrep_normalization, path_normalization=path_normalization,
            internal_weights=False, shared_weights=shared_weights)
    paths.dtype = dtype
    inferred = _single_mode(paths.instructions)
    if mode is not None and mode != inferred:
        raise ValueError("mode must match the tensor-product instructions")
    if not convolution or inferred != "uvu":
        raise NotImplementedError("this build provides the uvu convolution only (convolution=True, uvu instructions)")
    return create_uvu_conv_operator(paths, dtype=dtype)


@lru_cache(maxsize=128)
def _cached(irreps_in1, irreps_in2, irreps_out, instructions, in1_var, in2_var, out_var, irrep_normalization,
            path_normalization, shared_weights, dtype):
    return prepare_tensor_product(
        irreps_in1, irreps_in2, irreps_out, instructions, in1_var=in1_var, in2_var=in2_var, out_var=out_var,
        irrep_normalization=irrep_normalization, path_normalization=path_normalization,
        shared_weights=shared_weights, dtype=dtype, convolution=True)


def tensor_product_conv(x, edge_attr, weight=None, *, graph, irreps_in1=None, irreps_in2=None, irreps_out=None,
                        instructions=None, in1_var=None, in2_var=None, out_var=None, irrep_normalization=None,
                        path_normalization=None, shared_weights=False, config=None, **kwargs):
    """Contract edge messages and sum by destination, with explicit weights and an explicit graph."""
    if config is None:
        if irreps_in1 is None or irreps_in2 is None or irreps_out is None or instructions is None:
            raise TypeError("Supply irreps and instructions, or a prepared config")
        config = _cached(
            str(as_irreps(irreps_in1)), str(as_irreps(irreps_in2)), str(as_irreps(irreps_out)),
            tuple(tuple(i) for i in instructions),
            None if in1_var is None else tuple(in1_var), None if in2_var is None else tuple(in2_var),
            None if out_var is None else tuple(out_var), irrep_normalization, path_normalization, shared_weights,
            x.dtype)
    if not isinstance(config, LunaTPUVUConv):
        raise TypeError("config must come from prepare_tensor_product(..., convolution=True)")
    return config.run(config, x, edge_attr, weight, graph=graph, **kwargs)


__all__ = ["prepare_tensor_product", "tensor_product_conv"]
