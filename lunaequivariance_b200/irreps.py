"""O(3) irrep bookkeeping: ``Irrep`` (degree l, parity p) and ``Irreps`` (ordered multiset).

Follows the public behaviour of the reference's ``src/o3/irreps.py:17-241`` (itself e3nn-shaped):
string syntax ``"32x0e + 32x1o"``, iteration as ``(mul, ir)`` pairs, ``dim``, ``slices()``,
``Irreps.spherical_harmonics(lmax)``, and ``ir1 * ir2`` enumerating the coupled irreps.
Only what the UVU convolution path and the spherical harmonics need is provided.
"""

from __future__ import annotations

import re
from typing import Iterable, Iterator, NamedTuple

import torch

_IRREP_RE = re.compile(r"^\s*(\d+)\s*([eoy])\s*$")


class Irrep(NamedTuple):
    """One irreducible representation of O(3): degree ``l`` and parity ``p`` (+1 even, -1 odd)."""

    l: int
    p: int

    @classmethod
    def parse(cls, value) -> "Irrep":
        if isinstance(value, Irrep):
            return value
        if isinstance(value, MulIrrep):
            return value.ir
        if isinstance(value, str):
            match = _IRREP_RE.match(value)
            if match is None:
                raise ValueError(f'unable to convert string "{value}" into an Irrep')
            degree = int(match.group(1))
            parity = {"e": 1, "o": -1, "y": (-1) ** degree}[match.group(2)]
            return cls(degree, parity)
        if isinstance(value, tuple) and len(value) == 2:
            degree, parity = value
            if not isinstance(degree, int) or degree < 0:
                raise ValueError(f"l must be positive integer, got {degree}")
            if parity not in (-1, 1):
                raise ValueError(f"parity must be on of (-1, 1), got {parity}")
            return cls(int(degree), int(parity))
        # Duck-typed irreps from another library (attributes l and p).
        if hasattr(value, "l") and hasattr(value, "p"):
            return cls(int(value.l), int(value.p))
        raise ValueError(f"unable to interpret {value!r} as an Irrep")

    @property
    def dim(self) -> int:
        return 2 * self.l + 1

    def is_scalar(self) -> bool:
        return self.l == 0 and self.p == 1

    def __mul__(self, other) -> Iterator["Irrep"]:  # type: ignore[override]
        other = Irrep.parse(other)
        parity = self.p * other.p
        for degree in range(abs(self.l - other.l), self.l + other.l + 1):
            yield Irrep(degree, parity)

    def __rmul__(self, mul):  # type: ignore[override]
        if not isinstance(mul, int):
            raise TypeError("an Irrep can only be multiplied by an integer multiplicity")
        return Irreps([(mul, self)])

    def __add__(self, other):  # type: ignore[override]
        return Irreps(self) + Irreps(other)

    def __repr__(self) -> str:
        return f"{self.l}{'e' if self.p == 1 else 'o'}"

    __str__ = __repr__


class MulIrrep(NamedTuple):
    """An irrep repeated ``mul`` times (``mul`` channels of dimension ``2l+1`` each)."""

    mul: int
    ir: Irrep

    @property
    def dim(self) -> int:
        return self.mul * self.ir.dim

    def __repr__(self) -> str:
        return f"{self.mul}x{self.ir}"

    __str__ = __repr__


def _parse_entry(entry) -> MulIrrep:
    if isinstance(entry, MulIrrep):
        return entry
    if isinstance(entry, (str, Irrep)):
        return MulIrrep(1, Irrep.parse(entry))
    try:
        mul, ir = entry
    except (TypeError, ValueError):
        raise ValueError(f'Unable to interpret "{entry}" as an irrep.') from None
    if not isinstance(mul, int) or mul < 0:
        raise ValueError(f'Unable to interpret "{entry}" as an irrep.')
    return MulIrrep(mul, Irrep.parse(ir))


class Irreps(tuple):
    """Ordered list of ``mul x irrep`` blocks; a feature row is their concatenation.

    Within a block the layout is channel-major, component-minor ("mul_ir"): element ``(u, m)`` of a block
    that starts at ``offset`` lives at ``offset + u * (2l+1) + m``.
    """

    def __new__(cls, irreps=None):
        if isinstance(irreps, Irreps):
            return super().__new__(cls, tuple(irreps))
        blocks: list[MulIrrep] = []
        if irreps is None:
            pass
        elif isinstance(irreps, Irrep):
            blocks.append(MulIrrep(1, irreps))
        elif isinstance(irreps, str):
            text = irreps.strip()
            if text:
                try:
                    for part in text.split("+"):
                        if "x" in part:
                            mul_text, ir_text = part.split("x")
                            blocks.append(MulIrrep(int(mul_text), Irrep.parse(ir_text)))
                        else:
                            blocks.append(MulIrrep(1, Irrep.parse(part)))
                except ValueError:
                    raise ValueError(f'Unable to convert string "{irreps}" into an Irreps') from None
                if any(block.mul < 0 for block in blocks):
                    raise ValueError(f'Unable to convert string "{irreps}" into an Irreps')
        else:
            blocks.extend(_parse_entry(entry) for entry in irreps)
        return super().__new__(cls, blocks)

    @staticmethod
    def spherical_harmonics(lmax: int, p: int = -1) -> "Irreps":
        return Irreps([(1, (degree, p**degree)) for degree in range(lmax + 1)])

    def slices(self) -> list[slice]:
        bounds, start = [], 0
        for block in self:
            bounds.append(slice(start, start + block.dim))
            start += block.dim
        return bounds

    def randn(self, *size: int, normalization: str = "component", requires_grad: bool = False,
              dtype=None, device=None) -> torch.Tensor:
        axis = size.index(-1)
        lead, trail = size[:axis], size[axis + 1:]
        if normalization == "component":
            return torch.randn(*lead, self.dim, *trail, requires_grad=requires_grad, dtype=dtype, device=device)
        if normalization != "norm":
            raise ValueError("Normalization needs to be 'norm' or 'component'")
        out = torch.zeros(*lead, self.dim, *trail, dtype=dtype, device=device)
        for piece, block in zip(self.slices(), self):
            sample = torch.randn(*lead, block.mul, block.ir.dim, *trail, dtype=dtype, device=device)
            sample = sample / sample.norm(2, dim=axis + 1, keepdim=True)
            out.narrow(axis, piece.start, block.dim).copy_(sample.reshape(*lead, -1, *trail))
        return out.requires_grad_(requires_grad)

    def __getitem__(self, item):
        value = super().__getitem__(item)
        return Irreps(value) if isinstance(item, slice) else value

    def __contains__(self, ir) -> bool:
        ir = Irrep.parse(ir)
        return any(block.ir == ir for block in self)

    def count(self, ir) -> int:  # type: ignore[override]
        ir = Irrep.parse(ir)
        return sum(block.mul for block in self if block.ir == ir)

    def __add__(self, other) -> "Irreps":
        return Irreps(tuple(self) + tuple(Irreps(other)))

    def __mul__(self, other) -> "Irreps":
        if isinstance(other, Irreps):
            raise NotImplementedError("Use a tensor product for Irreps x Irreps")
        return Irreps(tuple(self) * other)

    __rmul__ = __mul__

    def simplify(self) -> "Irreps":
        merged: list[tuple[int, Irrep]] = []
        for mul, ir in self:
            if merged and merged[-1][1] == ir:
                merged[-1] = (merged[-1][0] + mul, ir)
            elif mul > 0:
                merged.append((mul, ir))
        return Irreps(merged)

    def remove_zero_multiplicities(self) -> "Irreps":
        return Irreps([(mul, ir) for mul, ir in self if mul > 0])

    @property
    def dim(self) -> int:
        return sum(block.dim for block in self)

    @property
    def num_irreps(self) -> int:
        return sum(block.mul for block in self)

    @property
    def ls(self) -> list[int]:
        return [block.ir.l for block in self for _ in range(block.mul)]

    @property
    def lmax(self) -> int:
        if len(self) == 0:
            raise ValueError("Cannot get lmax of empty Irreps")
        return max(self.ls)

    def __repr__(self) -> str:
        return "+".join(str(block) for block in self)

    __str__ = __repr__


def as_irreps(value) -> Irreps:
    """Accept our Irreps, a string, an iterable of (mul, ir), or another library's Irreps object."""
    if isinstance(value, Irreps):
        return value
    if isinstance(value, (str, Irrep)) or value is None:
        return Irreps(value)
    if isinstance(value, Iterable):
        return Irreps([(int(mul), Irrep.parse(ir)) for mul, ir in value])
    raise ValueError(f"Unable to interpret {value!r} as Irreps")


__all__ = ["Irrep", "MulIrrep", "Irreps", "as_irreps"]
