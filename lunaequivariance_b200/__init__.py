"""B200-native UVU TensorProductConv hot path (sm_100a CUDA behind a C-ABI) with the reference's Python surface.

Public names follow HPC-AI-Team/LunaEquivariance (``src/__init__.py:3-45``) for the path this library covers:
``TensorProductConv``, ``TensorProduct`` / ``tensor_product`` (uvu), ``TensorProductConfig``, ``make_graph`` / ``LunaTPGraph``, ``prepare_tensor_product``,
``tensor_product_conv``, ``SphericalHarmonics`` / ``spherical_harmonics``, ``Irrep`` / ``Irreps`` and the ``o3``
namespace.  ``HostStreamedConv`` (per-edge tensors streamed from host memory) and the ``sharded`` module (graphs
partitioned over GPUs) have no counterpart there.
"""

from . import o3
from .conv import LunaTPUVUConv, create_uvu_conv_operator
from .functional import prepare_tensor_product, tensor_product, tensor_product_conv
from .graph import LunaTPGraph, make_graph
from .irreps import Irrep, Irreps
from .modules import LunaEqSphericalHarmonics, SphericalHarmonics, TensorProduct, TensorProductConv
from .streaming import HostStreamedConv
from .tensor_product import LunaTPUVU
from .paths import Instruction, TensorProductConfig, TensorProductPaths, build_uvu_conv_metadata
from .spherical_harmonics import spherical_harmonics

__all__ = [
    "TensorProductConv", "TensorProduct", "tensor_product", "LunaTPUVU", "TensorProductConfig", "TensorProductPaths", "Instruction", "build_uvu_conv_metadata",
    "LunaTPGraph", "make_graph", "prepare_tensor_product", "tensor_product_conv", "LunaTPUVUConv",
    "create_uvu_conv_operator", "SphericalHarmonics", "LunaEqSphericalHarmonics", "spherical_harmonics",
    "Irrep", "Irreps", "o3", "HostStreamedConv",
]
