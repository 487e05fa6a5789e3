"""Synthetic graphs for the benchmark and the full-size parity tests: periodic radius graphs and fixed-degree graphs.

Not part of the library: these generators stand in for the neighbour list of an MD code.  They produce
destination-sorted edge lists on the device of the input.  Atoms are numbered in cell order (a z-fastest sweep
over the cells of a uniform grid), so consecutive destination nodes share most of their sources - the numbering an
MD neighbour list gives - and contiguous destination ranges are spatial slabs.
"""

from __future__ import annotations

import math

import torch


def all_uvu_instructions(irreps_in1, irreps_in2, irreps_out):
    """Every parity-allowed (i_in1, i_in2, i_out, 'uvu', True) triple, in (i, j, k) order."""
    from lunaequivariance_b200.irreps import as_irreps

    in1, in2, out = as_irreps(irreps_in1), as_irreps(irreps_in2), as_irreps(irreps_out)
    return [(i, j, k, "uvu", True)
            for i, (_, a) in enumerate(in1) for j, (_, b) in enumerate(in2) for k, (_, c) in enumerate(out)
            if c in a * b]


def periodic_positions(num_atoms: int, density: float, seed: int, device, cutoff: float):
    """Uniform positions in a periodic cube of the given number density, renumbered in cell order.

    Returns ``(positions[float64, N, 3], box_length, cells_per_side)``.
    """
    box = (num_atoms / density) ** (1.0 / 3.0)
    generator = torch.Generator().manual_seed(seed)
    pos = (torch.rand(num_atoms, 3, generator=generator, dtype=torch.float64) * box).to(device)
    cells = max(1, int(math.floor(box / cutoff)))
    size = box / cells
    index3 = torch.clamp((pos / size).floor().long(), max=cells - 1)
    cell = (index3[:, 0] * cells + index3[:, 1]) * cells + index3[:, 2]
    order = torch.argsort(cell, stable=True)
    return pos[order].contiguous(), box, cells


def radius_graph_periodic(pos: torch.Tensor, box: float, cutoff: float, cells: int, dst_begin: int = 0,
                          dst_end: int | None = None, chunk: int = 8192):
    """Edges ``src -> dst`` with minimum-image distance below ``cutoff`` for ``dst`` in ``[dst_begin, dst_end)``.

    ``pos`` must be numbered in cell order (see ``periodic_positions``).  Returns ``(src, dst, vec)`` sorted by
    ``dst`` with global atom indices (int64) and ``vec = pos[src] - pos[dst]`` under the minimum-image convention.
    """
    n = pos.shape[0]
    dst_end = n if dst_end is None else dst_end
    device = pos.device
    if cells < 3:  # too few cells for a 27-cell stencil without duplicates: brute force
        src_parts, dst_parts, vec_parts = [], [], []
        for a in range(dst_begin, dst_end, 1024):
            b = min(dst_end, a + 1024)
            delta = pos[None, :, :] - pos[a:b, None, :]
            delta = delta - box * torch.round(delta / box)
            mask = (delta.square().sum(-1) < cutoff * cutoff)
            mask[torch.arange(b - a, device=device), torch.arange(a, b, device=device)] = False
            d, s = mask.nonzero(as_tuple=True)
            src_parts.append(s)
            dst_parts.append(d + a)
            vec_parts.append(delta[d, s])
        return torch.cat(src_parts), torch.cat(dst_parts), torch.cat(vec_parts)

    size = box / cells
    index3 = torch.clamp((pos / size).floor().long(), max=cells - 1)
    cell = (index3[:, 0] * cells + index3[:, 1]) * cells + index3[:, 2]
    counts = torch.bincount(cell, minlength=cells ** 3)
    starts = torch.cumsum(counts, 0) - counts
    width = int(counts.max().item())
    offsets = torch.tensor([(a, b, c) for a in (-1, 0, 1) for b in (-1, 0, 1) for c in (-1, 0, 1)], device=device)
    slot = torch.arange(width, device=device)
    src_parts, dst_parts, vec_parts = [], [], []
    for a in range(dst_begin, dst_end, chunk):
        b = min(dst_end, a + chunk)
        neighbour3 = (index3[a:b, None, :] + offsets[None, :, :]) % cells           # [c, 27, 3]
        neighbour = (neighbour3[..., 0] * cells + neighbour3[..., 1]) * cells + neighbour3[..., 2]
        first, count = starts[neighbour], counts[neighbour]                          # [c, 27]
        candidate = first[..., None] + slot                                          # [c, 27, width]
        valid = slot < count[..., None]
        candidate = torch.where(valid, candidate, torch.zeros_like(candidate))
        delta = pos[candidate] - pos[a:b, None, None, :]
        delta = delta - box * torch.round(delta / box)
        hit = valid & (delta.square().sum(-1) < cutoff * cutoff)
        hit &= candidate != torch.arange(a, b, device=device)[:, None, None]
        d, o, k = hit.nonzero(as_tuple=True)                                          # row-major: sorted by d
        src_parts.append(candidate[d, o, k])
        dst_parts.append(d + a)
        vec_parts.append(delta[d, o, k])
    return torch.cat(src_parts), torch.cat(dst_parts), torch.cat(vec_parts)


def fixed_degree_graph(num_nodes: int, degree: int, seed: int, device):
    """Exactly ``degree`` incoming edges per node, sources uniform over the other nodes; sorted by destination."""
    generator = torch.Generator().manual_seed(seed)
    dst = torch.arange(num_nodes).repeat_interleave(degree)
    src = torch.randint(num_nodes - 1, (dst.numel(),), generator=generator)
    src = src + (src >= dst).long()
    return src.to(device), dst.to(device)


def random_unit_vectors(count: int, seed: int, device, dtype=torch.float64):
    generator = torch.Generator().manual_seed(seed)
    v = torch.randn(count, 3, generator=generator, dtype=torch.float64)
    return torch.nn.functional.normalize(v, dim=-1).to(device=device, dtype=dtype)


__all__ = ["all_uvu_instructions", "periodic_positions", "radius_graph_periodic", "fixed_degree_graph",
           "random_unit_vectors"]
