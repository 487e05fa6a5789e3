"""Helpers shared by the parity tests: configurations, seeded problems and the reference's tolerance rule."""

import torch

from lunaequivariance_b200 import Irreps

# (irreps_in1, irreps_in2, irreps_out, instructions or None for "all parity-allowed uvu paths", options)
CONFIGS = {
    "cfg1": ("32x1o", "1x1o", "32x0e", [(0, 0, 0, "uvu", True)], {}),
    "cfg2": ("128x0e+128x1o+128x2e", "1x0e+1x1o+1x2e+1x3o", "128x0e+128x1o+128x2e+128x3o", None, {}),
    "cfg4": ("64x0e+64x1o+64x2e+64x3o", "1x0e+1x1o+1x2e+1x3o", "64x0e+64x1o+64x2e+64x3o", None, {}),
    "cfg5": ("64x0e+64x1o+64x2e", "1x0e+1x1o+1x2e", "64x0e+64x1o+64x2e", None, {}),
    "fixture": ("32x0e+32x1o", "1x0e+1x1o", "32x0e+32x1o", None, {}),
    "small": ("4x0e+4x1o+4x2e", "1x0e+1x1o+1x2e", "4x0e+4x1o+4x2e", None, {}),
    "mul2": ("5x0e+5x1o", "2x0e+3x1o", "5x0e+5x1o", None, {}),
    "odd": ("33x0e+33x1o", "1x0e+1x1o", "33x0e+33x1o", None, {}),
    "one": ("1x0e+1x1o", "1x0e+1x1o", "1x0e+1x1o", None, {}),
    "mixed": ("3x0e+3x1o+3x1e", "1x0e+1x1o", "3x0e+3x1o+3x1e+3x1o", None, {}),
    "highl": ("3x5o", "2x5o", "3x0e+3x2e+3x4e", None, {}),
    "partial": ("32x0e+32x1o", "1x0e+1x1o", "32x0e+32x1o+32x2e", [(0, 0, 0, "uvu", True), (1, 1, 0, "uvu", True),
                                                                   (1, 1, 2, "uvu", True)], {}),
    "wide": ("256x0e+256x1o", "1x0e+1x1o", "256x0e+256x1o", None, {}),
    "norm_path": ("4x0e+4x1o", "1x0e+1x1o", "4x0e+4x1o", None,
                  {"irrep_normalization": "norm", "path_normalization": "path"}),
}


def all_paths(in1, in2, out):
    in1, in2, out = Irreps(in1), Irreps(in2), Irreps(out)
    return [(i, j, k, "uvu", True)
            for i, (_, a) in enumerate(in1) for j, (_, b) in enumerate(in2) for k, (_, c) in enumerate(out)
            if c in a * b]


def config(name):
    in1, in2, out, instructions, options = CONFIGS[name]
    if instructions is None:
        instructions = all_paths(in1, in2, out)
    return in1, in2, out, instructions, options


def random_graph(nodes, edges, generator, exact_degree=None):
    """Destination-sorted random edge list on CPU (int64)."""
    if exact_degree is not None:
        dst = torch.arange(nodes).repeat_interleave(exact_degree)
        src = torch.randint(nodes - 1, (dst.numel(),), generator=generator)
        src = src + (src >= dst).long()  # uniform over the other nodes
        return src, dst
    src = torch.randint(nodes, (edges,), generator=generator)
    dst = torch.sort(torch.randint(nodes, (edges,), generator=generator))[0]
    return src, dst


def random_problem(meta_dims, nodes, src, dtype, generator):
    in1_dim, in2_dim, out_dim, weight_numel = meta_dims
    edges = src.numel()
    rand = lambda *shape: torch.randn(*shape, generator=generator, dtype=torch.float64).to(dtype)
    return dict(x=rand(nodes, in1_dim), y=rand(edges, in2_dim), w=rand(edges, weight_numel),
                g=rand(nodes, out_dim), rx=rand(nodes, in1_dim), ry=rand(edges, in2_dim),
                rw=rand(edges, weight_numel))


def tolerance(dtype):
    """north-star bound: 1e-5 relative in FP32, 1e-12 in FP64.  "Relative" is checked in both of the reference's
    senses: the largest deviation over the largest reference magnitude (tests/testing_utils.py:14-41:
    max|a - r| <= atol + rtol * max|r|) and the relative L2 error |a - r|_2 / |r|_2 (src/utils/testing.py:290-313)."""
    return 1e-5 if dtype == torch.float32 else 1e-12


def assert_close(actual, expected, dtype, what=""):
    expected = expected.to(torch.float64)
    actual = actual.detach().to("cpu", torch.float64)
    assert actual.shape == expected.shape, (what, actual.shape, expected.shape)
    scale = max(expected.abs().max().item(), 1e-30) if expected.numel() else 1.0
    error = (actual - expected).abs().max().item() if expected.numel() else 0.0
    assert error <= tolerance(dtype) * scale + 1e-300, f"{what}: max error {error:.3e} vs scale {scale:.3e}"
    norm = expected.norm().item() if expected.numel() else 0.0
    if norm > 0.0:
        relative_l2 = (actual - expected).norm().item() / norm
        assert relative_l2 <= tolerance(dtype), f"{what}: relative L2 error {relative_l2:.3e}"
    return error / scale


class EdgeSample:
    """A subset of a large graph's edges as a small self-contained problem for the CPU oracle.

    The sampled edges keep their order; the source rows and destination rows they touch are renumbered compactly.
    ``take_*`` pull the matching rows of full-size device tensors to the CPU in float64.
    """

    def __init__(self, src, dst, edge_ids):
        self.edge_ids = edge_ids
        s, d = src[edge_ids].long(), dst[edge_ids].long()
        self.src_nodes, self.src = torch.unique(s, return_inverse=True)
        self.dst_nodes, self.dst = torch.unique(d, return_inverse=True)

    @staticmethod
    def _cpu(t):
        return t.detach().to("cpu", torch.float64)

    def take_edges(self, t):
        return self._cpu(t[self.edge_ids])

    def take_sources(self, t):
        return self._cpu(t[self.src_nodes])

    def take_destinations(self, t):
        return self._cpu(t[self.dst_nodes])

    @property
    def cpu_src(self):
        return self.src.cpu()

    @property
    def cpu_dst(self):
        return self.dst.cpu()


def in_edges_of(dst_rowptr, nodes):
    """Edge ids (ascending) of all edges into the given destination nodes."""
    begin, end = dst_rowptr[nodes].long(), dst_rowptr[nodes + 1].long()
    return torch.cat([torch.arange(int(b), int(e), device=dst_rowptr.device) for b, e in zip(begin, end)])


def out_edges_of(src_rowptr, edge_ids_by_src, nodes):
    """Edge ids of all edges out of the given source nodes."""
    begin, end = src_rowptr[nodes].long(), src_rowptr[nodes + 1].long()
    return torch.cat([edge_ids_by_src[int(b):int(e)].long() for b, e in zip(begin, end)])


def assert_rows_close(actual_rows, expected_rows, scale, dtype, what):
    """``max|a - r| <= tol * scale`` where ``scale`` is the largest magnitude of the whole tensor."""
    error = (actual_rows.detach().to("cpu", torch.float64) - expected_rows).abs().max().item()
    assert error <= tolerance(dtype) * scale, f"{what}: max error {error:.3e} vs scale {scale:.3e}"
    return error / scale
