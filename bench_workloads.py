"""Synthetic graphs for the benchmark and the full-size parity tests: periodic radius graphs and fixed-degree graphs.

Not part of the library: these generators stand in for the neighbour list of an MD code.  They produce
destination-sorted edge lists on the device of the input.  Atoms are numbered in cell order (a z-fastest sweep
over the cells of a uniform grid), so consecutive destination nodes share most of their sources - the numbering an
MD neighbour list gives - and contiguous destination ranges are spatial slabs.
"""

from __future__ import annotations

import math

import torch


WORKLOADS = {
    # name: (irreps_in1, sh lmax, irreps_out, dtype, atoms per GPU, graph kind)
    "cfg2": ("128x0e+128x1o+128x2e", 3, "128x0e+128x1o+128x2e+128x3o", torch.float32, 50_000, "radius"),
    # cfg3 is cfg2's convolution in FP64 inside a force-training step (energy -> forces -> loss -> dL/dweight)
    "cfg3": ("128x0e+128x1o+128x2e", 3, "128x0e+128x1o+128x2e+128x3o", torch.float64, 20_000, "radius"),
    "cfg5": ("64x0e+64x1o+64x2e", 2, "64x0e+64x1o+64x2e", torch.float32, 250_000, "radius"),
    "cfg4": ("64x0e+64x1o+64x2e+64x3o", 3, "64x0e+64x1o+64x2e+64x3o", torch.float32, 100_000, "degree40"),
    "cfg1": ("32x1o", 1, "32x0e", torch.float64, 1_000, "degree16"),
    "lmax1": ("128x0e+128x1o", 1, "128x0e+128x1o", torch.float32, 100_000, "radius"),
}
DENSITY, CUTOFF = 0.1, 5.0


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

def irreps_of(name):
    in1, lmax, out, dtype, atoms, kind = WORKLOADS[name]
    in2 = "+".join(f"1x{l}{'e' if l % 2 == 0 else 'o'}" for l in range(lmax + 1))
    if name == "cfg1":
        in2 = "1x1o"
    return in1, in2, out, dtype, atoms, kind, lmax


def build_paths(name):
    in1, in2, out, dtype, atoms, kind, lmax = irreps_of(name)
    instructions = [(0, 0, 0, "uvu", True)] if name == "cfg1" else all_uvu_instructions(in1, in2, out)
    return in1, in2, out, instructions, dtype, atoms, kind, lmax


def build_graph_edges(name, atoms_per_gpu, world, rank, device):
    """This rank's destination-sorted edge slice (global ids) and unit edge vectors."""
    kind = WORKLOADS[name][5]
    total = atoms_per_gpu * world
    begin, end = rank * atoms_per_gpu, (rank + 1) * atoms_per_gpu
    if kind == "radius":
        pos, box, cells = periodic_positions(total, DENSITY, 0, device, CUTOFF)
        src, dst, vec = radius_graph_periodic(pos, box, CUTOFF, cells, begin, end)
        return src, dst, vec
    degree = 40 if kind == "degree40" else 16
    src, dst = fixed_degree_graph(total, degree, 0, device)
    mine = (dst >= begin) & (dst < end)
    src, dst = src[mine], dst[mine]
    vec = random_unit_vectors(src.numel(), 1 + rank, device)
    return src, dst, vec


__all__ = ["WORKLOADS", "DENSITY", "CUTOFF", "irreps_of", "build_paths", "build_graph_edges",
           "all_uvu_instructions", "periodic_positions", "radius_graph_periodic", "fixed_degree_graph",
           "random_unit_vectors"]
