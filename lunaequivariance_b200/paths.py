"""Tensor-product path lists with e3nn-compatible normalisation, and the UVU convolution metadata built from them.

Behaviour restated from the reference:

* ``TensorProductPaths`` / ``TensorProductConfig`` / ``Instruction`` — ``src/lunatp/utils/layout.py:239-438``:
  the stored ``path_weight`` of an instruction is ``sqrt(alpha)`` with
  ``alpha = irrep_norm_factor / fan_in * out_var * user_path_weight``; weights are counted as
  ``prod(path_shape)`` per weighted instruction.
* ``build_uvu_conv_metadata`` — ``src/lunatp/uvu_conv/kernels/utils.py:23-119``: one spec per
  (instruction, edge channel ``v``); the weight of channel ``u`` sits at ``weight_offset + u * mul_in2`` with
  ``weight_offset`` already including ``v`` (e3nn's ``[u, v]`` row-major layout).

The metadata is a plain ``dict`` with the reference's key names so that metadata produced by either library can be
handed to ``TensorProductConv(meta, mode="uvu")``.
"""

from __future__ import annotations

from math import prod, sqrt
from typing import Any, NamedTuple, Sequence

import torch

from .coupling import cg_terms
from .irreps import Irreps, as_irreps


class Instruction(NamedTuple):
    i_in1: int
    i_in2: int
    i_out: int
    connection_mode: str
    has_weight: bool
    path_weight: float
    path_shape: tuple


_MODES = ("uvw", "uvu", "uuu")


def _path_shape(mode: str, mul1: int, mul2: int, mul_out: int) -> tuple:
    if mode == "uvw":
        return (mul1, mul2, mul_out)
    if mode == "uvu":
        return (mul1, mul2)
    return (mul1,)


def _fan_in(mode: str, mul1: int, mul2: int) -> int:
    """Number of (u, v) input pairs feeding one output channel."""
    if mode == "uvw":
        return mul1 * mul2
    if mode == "uvu":
        return mul2
    return 1


def _variances(values, count: int, label: str, irreps_label: str) -> list[float]:
    if values is None:
        return [1.0] * count
    values = [float(v) for v in values]
    assert len(values) == count, f"Len of {label} must be equal to len({irreps_label})"
    return values


class TensorProductPaths:
    """Normalised instruction list; holds no parameters and no module state."""

    dtype: torch.dtype

    def __init__(
        self,
        irreps_in1,
        irreps_in2,
        irreps_out,
        instructions: Sequence[tuple],
        *,
        in1_var=None,
        in2_var=None,
        out_var=None,
        irrep_normalization: str | None = None,
        path_normalization: str | None = None,
        internal_weights: bool | None = None,
        shared_weights: bool | None = None,
    ) -> None:
        irrep_normalization = "component" if irrep_normalization is None else irrep_normalization
        path_normalization = "element" if path_normalization is None else path_normalization
        assert irrep_normalization in ("component", "norm", "none")
        assert path_normalization in ("element", "path", "none")
        in1, in2, out = as_irreps(irreps_in1), as_irreps(irreps_in2), as_irreps(irreps_out)
        self.irreps_in1, self.irreps_in2, self.irreps_out = in1, in2, out

        raw = []
        for item in instructions:
            item = tuple(item)
            if len(item) == 5:
                item = item + (1.0,)
            i1, i2, io, mode, has_weight, user_weight = item[:6]
            assert mode in _MODES
            raw.append((int(i1), int(i2), int(io), mode, bool(has_weight), user_weight))

        var1 = _variances(in1_var, len(in1), "ir1_var", "irreps_in1")
        var2 = _variances(in2_var, len(in2), "ir2_var", "irreps_in2")
        var_out = _variances(out_var, len(out), "out_var", "irreps_out")

        def contribution(entry) -> float:
            i1, i2, _, mode, _, _ = entry
            return var1[i1] * var2[i2] * _fan_in(mode, in1[i1].mul, in2[i2].mul)

        normalised = []
        for entry in raw:
            i1, i2, io, mode, has_weight, user_weight = entry
            b1, b2, bo = in1[i1], in2[i2], out[io]
            assert b1.ir.p * b2.ir.p == bo.ir.p
            assert abs(b1.ir.l - b2.ir.l) <= bo.ir.l <= b1.ir.l + b2.ir.l
            if mode == "uuu":
                assert b1.mul == b2.mul == bo.mul, "UUU requires equal input and output multiplicities"
            alpha: float = {
                "component": bo.ir.dim,
                "norm": b1.ir.dim * b2.ir.dim,
                "none": 1,
            }[irrep_normalization]
            siblings = [other for other in raw if other[2] == io]
            if path_normalization == "element":
                total = sum(contribution(other) for other in siblings)
            elif path_normalization == "path":
                total = contribution(entry) * len(siblings)
            else:
                total = 1
            if total > 0.0:
                alpha /= total
            alpha *= var_out[io]
            alpha *= user_weight
            normalised.append(
                Instruction(i1, i2, io, mode, has_weight, sqrt(alpha), _path_shape(mode, b1.mul, b2.mul, bo.mul))
            )
        self.instructions = normalised

        if shared_weights is False and internal_weights is None:
            internal_weights = False
        if shared_weights is None:
            shared_weights = True
        if internal_weights is None:
            internal_weights = shared_weights and any(ins.has_weight for ins in normalised)
        assert shared_weights or not internal_weights
        self.internal_weights = internal_weights
        self.shared_weights = shared_weights
        self.weight_numel = sum(prod(ins.path_shape) for ins in normalised if ins.has_weight)

    @classmethod
    def from_tensor_product(cls, tp: Any) -> "TensorProductPaths":
        """Copy static path attributes from any tensor-product-like object (ours, the reference's or e3nn's)."""
        if isinstance(tp, cls):
            return tp
        paths = cls.__new__(cls)
        paths.irreps_in1 = as_irreps(tp.irreps_in1)
        paths.irreps_in2 = as_irreps(tp.irreps_in2)
        paths.irreps_out = as_irreps(tp.irreps_out)
        paths.instructions = [
            Instruction(int(i.i_in1), int(i.i_in2), int(i.i_out), str(i.connection_mode), bool(i.has_weight),
                        float(i.path_weight), tuple(int(s) for s in i.path_shape))
            for i in tp.instructions
        ]
        paths.internal_weights = bool(tp.internal_weights)
        paths.shared_weights = bool(tp.shared_weights)
        paths.weight_numel = int(tp.weight_numel)
        weight = getattr(tp, "weight", None)
        paths.dtype = weight.dtype if isinstance(weight, torch.Tensor) else getattr(tp, "dtype", torch.float32)
        return paths


class TensorProductConfig(torch.nn.Module):
    """Paths plus (for shared internal weights only) a registered weight parameter."""

    def __init__(self, irreps_in1, irreps_in2, irreps_out, instructions, *, in1_var=None, in2_var=None,
                 out_var=None, irrep_normalization=None, path_normalization=None, internal_weights=None,
                 shared_weights=None) -> None:
        super().__init__()
        paths = TensorProductPaths(
            irreps_in1, irreps_in2, irreps_out, instructions, in1_var=in1_var, in2_var=in2_var, out_var=out_var,
            irrep_normalization=irrep_normalization, path_normalization=path_normalization,
            internal_weights=internal_weights, shared_weights=shared_weights,
        )
        self.__dict__.update(vars(paths))
        if self.internal_weights and self.weight_numel > 0:
            self.weight = torch.nn.Parameter(torch.randn(self.weight_numel))
        else:
            self.register_buffer("weight", torch.Tensor())


def _narrowed_terms(l1: int, l2: int, l3: int, path_weight: float, dtype: torch.dtype):
    """Sparse coupling terms ``(i, j, k, value)`` of one instruction in the coefficient dtype."""
    terms = cg_terms(l1, l2, l3, path_weight)
    if dtype != torch.float32:
        return terms
    # The reference rounds the coupling tensor to float32 before it multiplies by the path weight
    # (src/lunatp/utils/cg.py:31-41 on a float32 tensor); doing the same keeps the coefficients bit-identical.
    import numpy as np

    from .coupling import wigner_3j

    rounded = wigner_3j(l1, l2, l3).astype(np.float32)
    return [(i, j, k, float(rounded[i, j, k]) * path_weight) for i, j, k, _ in terms]


def build_uvu_conv_metadata(tp, coefficient_dtype: torch.dtype = torch.float64) -> dict:
    """Lower UVU instructions to flat per-path specs (offsets, dims, sparse coupling terms).

    The returned dict has the reference's format (``src/lunatp/uvu_conv/kernels/utils.py:23-119``) so that either
    library's metadata can be handed to the other's operator: one spec per (instruction, channel ``v`` of the second
    input); element ``u`` of that spec's weights sits at ``weight_offset + u * weight_stride``.
    """
    if coefficient_dtype not in (torch.float32, torch.float64):
        raise ValueError(f"UVU convolution coefficients require float32 or float64; got {coefficient_dtype}.")
    for flag in ("internal_weights", "shared_weights"):
        if getattr(tp, flag):
            raise ValueError(f"Generated SO3 kernels require {flag}=False.")
    blocks = [as_irreps(r) for r in (tp.irreps_in1, tp.irreps_in2, tp.irreps_out)]
    starts = [[piece.start for piece in irreps.slices()] for irreps in blocks]

    specs: list[dict] = []
    widest = 0
    weights_used = 0
    for position, ins in enumerate(tp.instructions):
        if ins.connection_mode != "uvu":
            raise ValueError(f"Only connection_mode='uvu' is supported, got {ins.connection_mode!r}.")
        if not ins.has_weight:
            raise ValueError("Generated SO3 kernels require weighted uvu instructions.")
        slots = (ins.i_in1, ins.i_in2, ins.i_out)
        (mul1, ir1), (mul2, ir2), (mul3, ir3) = (irreps[slot] for irreps, slot in zip(blocks, slots))
        if mul1 != mul3:
            raise ValueError(
                f"UVU requires equal input/output multiplicities; got {mul1} and {mul3} "
                f"for path ({ins.i_in1}, {ins.i_in2}, {ins.i_out})."
            )
        if tuple(ins.path_shape) != (mul1, mul2):
            raise ValueError(f"UVU expects path_shape=({mul1}, {mul2}); got {tuple(ins.path_shape)}.")
        x_start, y_start, out_start = (table[slot] for table, slot in zip(starts, slots))
        shared = dict(x_offset=x_start, out_offset=out_start, channels=mul1, d1=ir1.dim, d2=ir2.dim, d3=ir3.dim,
                      l1=ir1.l, l2=ir2.l, l3=ir3.l,
                      terms=_narrowed_terms(ir1.l, ir2.l, ir3.l, float(ins.path_weight), coefficient_dtype))
        # several channels of the second input share the instruction's weight block, interleaved [u, v]
        extra = dict(weight_stride=mul2, l0_path=position) if mul2 != 1 else {}
        specs += [dict(shared, y_offset=y_start + v * ir2.dim, weight_offset=weights_used + v, **extra)
                  for v in range(mul2)]
        weights_used += mul1 * mul2
        widest = max(widest, mul1)

    if not specs:
        raise ValueError("No uvu instructions found.")
    if weights_used != tp.weight_numel:
        raise ValueError(f"Lowered weight_numel={weights_used}, but configuration reports {tp.weight_numel}.")
    if min(spec["channels"] for spec in specs) <= 0:
        raise ValueError("SO3 uvu kernels require positive channels per irrep.")
    in1, in2, out = blocks
    return dict(in1_dim=in1.dim, in2_dim=in2.dim, out_dim=out.dim, weight_numel=int(tp.weight_numel),
                max_channels=widest, generated_specs=specs)


__all__ = ["Instruction", "TensorProductPaths", "TensorProductConfig", "build_uvu_conv_metadata", "Irreps"]
