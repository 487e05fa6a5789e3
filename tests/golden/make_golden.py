"""Generate the golden fixtures in this directory from the reference's own Python code.

Run once in a container that has the reference checkout (it is not needed to run the tests):

    python tests/golden/make_golden.py /path/to/LunaEquivariance

The reference package cannot be imported normally without e3nn, so a stub parent package is registered and
only these CPU-runnable pieces are imported:

* ``lunatp.utils.layout.TensorProductPaths``  (path normalisation, weight_numel)
* ``lunatp.utils.cg.wigner_3j``               (real-basis coupling tensors)
* ``lunatp.uvu_conv.kernels.utils.build_uvu_conv_metadata`` (offsets and sparse terms of every path)
* ``lunatp.uvu_conv.graph.make_source_segments`` and the CPU branch of ``lunatp.graph.make_graph``
* ``o3.spherical_harmonics.replay.polynomial_forward`` (the reference's CPU spherical harmonics)

Outputs (all small):
  reference_wigner.npz     coupling tensors for all valid (l1,l2,l3) with l<=4, plus (5,5,l3)
  reference_tables.json    instructions, weight_numel and full path metadata of the benchmark/test configurations
  graph_tables.npz         graph tables of three small graphs
  sh_vectors.npz           harmonics, first and second derivatives (float64) at 24 seeded points
  conv_vectors.npz         convolution forward/first/second derivatives computed from the reference's metadata by
                           dense float64 einsum + index_add (the formulation of the reference's tests with e3nn)
"""

from __future__ import annotations

import json
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def import_reference(root):
    package = types.ModuleType("LunaEquivariance")
    package.__path__ = [os.path.join(root, "src")]
    sys.modules["LunaEquivariance"] = package


def all_paths(in1, in2, out, Irreps):
    in1, in2, out = Irreps(in1), Irreps(in2), Irreps(out)
    return [
        (i, j, k, "uvu", True)
        for i, (_, a) in enumerate(in1)
        for j, (_, b) in enumerate(in2)
        for k, (_, c) in enumerate(out)
        if c in a * b
    ]


CONFIGS = {
    "cfg1": ("32x1o", "1x1o", "32x0e", [(0, 0, 0, "uvu", True)], {}),
    "cfg2": ("128x0e+128x1o+128x2e", "1x0e+1x1o+1x2e+1x3o", "128x0e+128x1o+128x2e+128x3o", None, {}),
    "cfg4": ("64x0e+64x1o+64x2e+64x3o", "1x0e+1x1o+1x2e+1x3o", "64x0e+64x1o+64x2e+64x3o", None, {}),
    "cfg5": ("64x0e+64x1o+64x2e", "1x0e+1x1o+1x2e", "64x0e+64x1o+64x2e", None, {}),
    "fixture": ("32x0e+32x1o", "1x0e+1x1o", "32x0e+32x1o", None, {}),
    "small": ("4x0e+4x1o+4x2e", "1x0e+1x1o+1x2e", "4x0e+4x1o+4x2e", None, {}),
    "mul2": ("5x0e+5x1o", "2x0e+3x1o", "5x0e+5x1o", None, {}),
    "odd": ("33x0e+33x1o", "1x0e+1x1o", "33x0e+33x1o", None, {}),
    "mixed": ("3x0e+3x1o+3x1e", "1x0e+1x1o", "3x0e+3x1o+3x1e+3x1o", None, {}),
    "highl": ("3x5o", "2x5o", "3x0e+3x2e+3x4e", None, {}),
    "norm_path": ("4x0e+4x1o", "1x0e+1x1o", "4x0e+4x1o", None,
                  {"irrep_normalization": "norm", "path_normalization": "path"}),
    "none_var": ("4x0e+4x1o", "1x0e+1x1o", "4x0e+4x1o", None,
                 {"irrep_normalization": "none", "path_normalization": "none",
                  "in1_var": [1.0, 2.0], "in2_var": [0.5, 1.0], "out_var": [3.0, 1.0]}),
    "weighted": ("4x0e+4x1o", "1x0e+1x1o", "4x0e", [(0, 0, 0, "uvu", True, 2.0), (1, 1, 0, "uvu", True, 0.5)], {}),
}


def dense_conv(meta, x, y, w, src, dst, num_nodes):
    out = x.new_zeros((num_nodes, meta["out_dim"]))
    xs = x[src]
    for spec in meta["generated_specs"]:
        ch, d1, d2, d3 = spec["channels"], spec["d1"], spec["d2"], spec["d3"]
        cg = x.new_zeros((d1, d2, d3))
        for i, j, k, c in spec["terms"]:
            cg[i, j, k] = c
        stride = spec.get("weight_stride", 1)
        xb = xs[:, spec["x_offset"]: spec["x_offset"] + ch * d1].reshape(-1, ch, d1)
        yb = y[:, spec["y_offset"]: spec["y_offset"] + d2]
        wb = w[:, spec["weight_offset"]: spec["weight_offset"] + (ch - 1) * stride + 1: stride]
        msg = torch.einsum("ijk,eui,ej,eu->euk", cg, xb, yb, wb).reshape(-1, ch * d3)
        block = x.new_zeros((num_nodes, ch * d3)).index_add(0, dst, msg)
        out = out + torch.nn.functional.pad(block, (spec["out_offset"], meta["out_dim"] - spec["out_offset"] - ch * d3))
    return out


def main(root):
    import_reference(root)
    from LunaEquivariance.lunatp.graph import make_graph
    from LunaEquivariance.lunatp.utils.cg import wigner_3j
    from LunaEquivariance.lunatp.utils.layout import TensorProductPaths
    from LunaEquivariance.lunatp.uvu_conv.kernels.utils import build_uvu_conv_metadata
    from LunaEquivariance.o3.irreps import Irreps
    from LunaEquivariance.o3.spherical_harmonics.replay import polynomial_forward

    # ---- coupling tensors
    wigner = {}
    for l1 in range(5):
        for l2 in range(5):
            for l3 in range(abs(l1 - l2), min(l1 + l2, 4) + 1):
                wigner[f"{l1}_{l2}_{l3}"] = wigner_3j(l1, l2, l3, dtype=torch.float64).numpy()
    for l3 in range(0, 11):
        wigner[f"5_5_{l3}"] = wigner_3j(5, 5, l3, dtype=torch.float64).numpy()
    np.savez_compressed(os.path.join(HERE, "reference_wigner.npz"), **wigner)

    # ---- path tables
    tables = {}
    metas = {}
    for name, (in1, in2, out, instructions, kwargs) in CONFIGS.items():
        if instructions is None:
            instructions = all_paths(in1, in2, out, Irreps)
        tp = TensorProductPaths(in1, in2, out, instructions, internal_weights=False, shared_weights=False, **kwargs)
        meta = build_uvu_conv_metadata(tp, torch.float64)
        metas[name] = meta
        tables[name] = dict(
            irreps_in1=in1, irreps_in2=in2, irreps_out=out, kwargs=kwargs,
            instructions_in=[list(i) for i in instructions],
            instructions=[[i.i_in1, i.i_in2, i.i_out, i.connection_mode, i.has_weight, i.path_weight,
                           list(i.path_shape)] for i in tp.instructions],
            weight_numel=tp.weight_numel,
            meta=dict(
                in1_dim=meta["in1_dim"], in2_dim=meta["in2_dim"], out_dim=meta["out_dim"],
                weight_numel=meta["weight_numel"], max_channels=meta["max_channels"],
                generated_specs=[
                    {key: ([list(t) for t in value] if key == "terms" else value) for key, value in spec.items()}
                    for spec in meta["generated_specs"]
                ],
            ),
        )
    with open(os.path.join(HERE, "reference_tables.json"), "w") as handle:
        json.dump(tables, handle, separators=(",", ":"))

    # ---- graphs
    generator = torch.Generator().manual_seed(11)
    graphs = {}
    cases = {
        "tiny": (torch.tensor([2, 0, 1, 0]), torch.tensor([0, 1, 1, 2]), 4),
        "random": (torch.randint(23, (150,), generator=generator),
                   torch.sort(torch.randint(23, (150,), generator=generator))[0], 25),
        "hub": (torch.cat([torch.zeros(70, dtype=torch.long), torch.randint(9, (30,), generator=generator)]),
                torch.sort(torch.randint(9, (100,), generator=generator))[0], 9),
    }
    for name, (src, dst, n) in cases.items():
        graph = make_graph(src, dst, n)
        seg = graph.source_segments
        for key, value in dict(
            src_in=src, dst_in=dst, num_nodes=torch.tensor(n), src=graph.src, dst=graph.dst,
            dst_rowptr=graph.dst_rowptr, src_rowptr=graph.src_rowptr, edge_ids_by_src=graph.edge_ids_by_src,
            edge_ids_by_dst=graph.edge_ids_by_dst, node_order=graph.node_order,
            source_node_order=graph.source_node_order, node_tiers=graph.node_tiers,
            seg_nodes=seg.nodes, seg_begin=seg.begin, seg_end=seg.end, seg_rowptr=seg.rowptr, seg_order=seg.order,
        ).items():
            graphs[f"{name}.{key}"] = value.numpy()
    np.savez_compressed(os.path.join(HERE, "graph_tables.npz"), **graphs)

    # ---- spherical harmonics
    generator = torch.Generator().manual_seed(5)
    points = torch.randn(24, 3, generator=generator, dtype=torch.float64)
    points[0] = torch.tensor([0.0, 1.0, 0.0])
    points[1] = torch.tensor([0.3, -0.2, 2.5])
    sh = {"points": points.numpy()}
    degrees = tuple(range(13))
    g = torch.randn(24, 169, generator=generator, dtype=torch.float64)
    rx = torch.randn(24, 3, generator=generator, dtype=torch.float64)
    sh["g"], sh["rx"] = g.numpy(), rx.numpy()
    for normalize in (False, True):
        for normalization in ("component", "norm", "integral"):
            v = points.clone().requires_grad_(True)
            gg = g.clone().requires_grad_(True)
            out = polynomial_forward(v, normalize=normalize, degrees=degrees, normalization=normalization)
            (dx,) = torch.autograd.grad(out, v, gg, create_graph=True)
            sx, sg = torch.autograd.grad(dx, (v, gg), rx)
            tag = f"{int(normalize)}.{normalization}"
            sh[f"out.{tag}"] = out.detach().numpy()
            sh[f"dx.{tag}"] = dx.detach().numpy()
            sh[f"sx.{tag}"] = sx.numpy()
            sh[f"sg.{tag}"] = sg.numpy()
    # a non-contiguous degree selection, as the reference's tests use ([3, 1, 3, 0])
    v = points.clone()
    sh["out.sel"] = polynomial_forward(v, normalize=True, degrees=(3, 1, 3, 0), normalization="norm").numpy()
    np.savez_compressed(os.path.join(HERE, "sh_vectors.npz"), **sh)

    # ---- convolution vectors from the reference's metadata
    conv = {}
    for name, nodes, edges in (("cfg1", 9, 40), ("small", 7, 19), ("mul2", 6, 17), ("mixed", 5, 13),
                               ("highl", 4, 9), ("fixture", 7, 19)):
        meta = metas[name]
        generator = torch.Generator().manual_seed(731)
        dt = torch.float64
        x = torch.randn(nodes, meta["in1_dim"], generator=generator, dtype=dt, requires_grad=True)
        y = torch.randn(edges, meta["in2_dim"], generator=generator, dtype=dt, requires_grad=True)
        w = torch.randn(edges, meta["weight_numel"], generator=generator, dtype=dt, requires_grad=True)
        src = torch.randint(nodes, (edges,), generator=generator)
        dst = torch.sort(torch.randint(nodes, (edges,), generator=generator))[0]
        g = torch.randn(nodes, meta["out_dim"], generator=generator, dtype=dt, requires_grad=True)
        rx, ry, rw = (torch.randn(t.shape, generator=generator, dtype=dt) for t in (x, y, w))
        out = dense_conv(meta, x, y, w, src, dst, nodes)
        gx, gy, gw = torch.autograd.grad(out, (x, y, w), g, create_graph=True)
        hx, hy, hw, hg = torch.autograd.grad((gx, gy, gw), (x, y, w, g), (rx, ry, rw))
        for key, value in dict(x=x, y=y, w=w, src=src, dst=dst, g=g, rx=rx, ry=ry, rw=rw, out=out, gx=gx, gy=gy,
                               gw=gw, hx=hx, hy=hy, hw=hw, hg=hg, num_nodes=torch.tensor(nodes)).items():
            conv[f"{name}.{key}"] = value.detach().numpy()
    np.savez_compressed(os.path.join(HERE, "conv_vectors.npz"), **conv)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/LunaEquivariance")
    main(sys.argv[1])
