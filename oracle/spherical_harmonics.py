"""CPU oracle for real spherical harmonics in the e3nn convention. TEST INFRASTRUCTURE ONLY.

Test infrastructure: only the tests, the repository's smoke check and the benchmark's CPU-baseline legs may import this module.

Restates the reference's own CPU evaluation ``polynomial_forward``
(``src/o3/spherical_harmonics/replay.py:112-120``) of the Cartesian recurrence listed in
``src/o3/spherical_harmonics/kernels/forward.py:21-219``; scaling rules from ``forward.py:309-322``;
``normalize=True`` divides by ``max(|v|, 1e-12)`` (``torch.nn.functional.normalize``).
Instead of the listed expressions this file generates the recurrence coefficients in closed form:

    Y_{l,0}    = sqrt((2l+1)/(2l)) (Y_{l-1,0} z + Y_{l-1,2l-2} x)
    Y_{l,2l}   = sqrt((2l+1)/(2l)) (Y_{l-1,2l-2} z - Y_{l-1,0} x)
    Y_{l,1}    = sqrt(2l+1) y Y_{l-1,0},     Y_{l,2l-1} = sqrt(2l+1) y Y_{l-1,2l-2}
    Y_{l,m}    = sqrt((2l+1)(2l-1)/(l^2-mu^2)) y Y_{l-1,m-1}
                 - sqrt((2l+1)/(2l-3) ((l-1)^2-mu^2)/(l^2-mu^2)) r^2 Y_{l-2,m-2},   mu = m - l, 2 <= m <= 2l-2

with "component" normalisation (sum_m Y_lm^2 = 2l+1 on the unit sphere).  Derivatives come from autograd.

Parity pin: ``tests/golden/sh_vectors.npz`` holds values, first and second derivatives produced by the reference's
``polynomial_forward`` in float64 for every degree 0..12 and all three normalisations.
"""

from __future__ import annotations

import math

import torch


def recurrence_coefficients(l: int, m: int) -> tuple[float, float]:
    """(a, b) of the interior rule ``Y_{l,m} = a*y*Y_{l-1,m-1} - b*r2*Y_{l-2,m-2}``."""
    mu = m - l
    a = math.sqrt((2 * l + 1) * (2 * l - 1) / (l * l - mu * mu))
    b = math.sqrt((2 * l + 1) / (2 * l - 3) * ((l - 1) ** 2 - mu * mu) / (l * l - mu * mu))
    return a, b


def polynomial(lmax: int, x, y, z) -> list[list[torch.Tensor]]:
    """Component-normalised harmonics for degrees 0..lmax as nested lists ``Y[l][m]``."""
    levels = [[torch.ones_like(x)]]
    if lmax >= 1:
        s3 = math.sqrt(3.0)
        levels.append([s3 * x, s3 * y, s3 * z])
    r2 = x * x + y * y + z * z
    for l in range(2, lmax + 1):
        prev, prev2 = levels[l - 1], levels[l - 2]
        edge = math.sqrt((2 * l + 1) / (2 * l))
        row = [None] * (2 * l + 1)
        row[0] = edge * (prev[0] * z + prev[2 * l - 2] * x)
        row[2 * l] = edge * (prev[2 * l - 2] * z - prev[0] * x)
        row[1] = math.sqrt(2 * l + 1) * y * prev[0]
        row[2 * l - 1] = math.sqrt(2 * l + 1) * y * prev[2 * l - 2]
        for m in range(2, 2 * l - 1):
            a, b = recurrence_coefficients(l, m)
            row[m] = a * y * prev[m - 1] - b * r2 * prev2[m - 2]
        levels.append(row)
    return levels


def spherical_harmonics(degrees, vectors: torch.Tensor, normalize: bool, normalization: str = "integral"):
    """``[..., 3] -> [..., sum(2l+1)]`` for the listed degrees."""
    degrees = [degrees] if isinstance(degrees, int) else list(degrees)
    if normalize:
        vectors = torch.nn.functional.normalize(vectors, dim=-1)
    levels = polynomial(max(degrees), vectors[..., 0], vectors[..., 1], vectors[..., 2])
    columns = []
    for l in degrees:
        if normalization == "integral":
            scale = 1.0 / math.sqrt(4 * math.pi)
        elif normalization == "norm":
            scale = 1.0 / math.sqrt(2 * l + 1)
        elif normalization == "component":
            scale = 1.0
        else:
            raise ValueError("normalization must be component, norm or integral")
        columns.extend(value * scale for value in levels[l])
    return torch.stack(columns, dim=-1)


def derivatives(degrees, vectors, normalize, normalization, g, rx=None):
    """Value, first derivative ``dx = J^T g`` and, when ``rx`` is given, the second-order pair
    ``sx = d<rx,dx>/dx`` and ``sg = d<rx,dx>/dg`` (the reference's double-backward outputs,
    ``src/o3/spherical_harmonics/interface.py:118-126``)."""
    v = vectors.detach().clone().requires_grad_(True)
    g = g.detach().clone().requires_grad_(True)
    out = spherical_harmonics(degrees, v, normalize, normalization)
    (dx,) = torch.autograd.grad(out, v, g, create_graph=rx is not None, allow_unused=True)
    if dx is None:
        dx = torch.zeros_like(v)
    result = dict(out=out.detach(), dx=dx.detach())
    if rx is not None and dx.requires_grad:
        sx, sg = torch.autograd.grad(dx, (v, g), rx, allow_unused=True)
        result["sx"] = torch.zeros_like(v) if sx is None else sx
        result["sg"] = torch.zeros_like(g) if sg is None else sg
    elif rx is not None:
        result["sx"], result["sg"] = torch.zeros_like(v), torch.zeros_like(g)
    return result
