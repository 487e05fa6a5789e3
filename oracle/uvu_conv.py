"""CPU oracle for the UVU tensor-product convolution. TEST INFRASTRUCTURE ONLY.

Test infrastructure: only the tests, the repository's smoke check and the benchmark's CPU-baseline legs may import this module; the
product package never does.

The reference (HPC-AI-Team/LunaEquivariance v0.3.0) has no CPU implementation of the convolution: its operator
raises "CUDA is required" (``src/utils/extension.py:46-47``).  This file restates the *specification* the
reference's CUDA generators consume, in dense float64 torch code, and differentiates it with autograd the same way
the reference's tests differentiate e3nn (``tests/lunatp/test_uvu_conv.py:52-99``):

* irreps strings and block offsets ............ ``src/o3/irreps.py:106-156``
* path normalisation ......................... ``src/lunatp/utils/layout.py:323-382``
* SU(2) Clebsch-Gordan, real basis, norm ..... ``src/lunatp/utils/cg.py:102-180``
* per-path offsets and weight layout ......... ``src/lunatp/uvu_conv/kernels/utils.py:43-98``
* semantics of the op ........................ ``docs/operators/tensor_product_conv.md:237-251``:
  ``out[t] = sum_{e: dst[e]=t} sum_p  w[e, wo_p + u*mul2 + v] * C^p_ijk * x[src[e], xo_p + u*d1 + i] * y[e, yo_p + j]``

Parity pin: the path tables produced here are compared with tables dumped from the reference's own
``TensorProductPaths`` / ``build_uvu_conv_metadata`` / ``wigner_3j`` (``tests/golden/reference_tables.json`` and
``reference_wigner.npz``, written by ``tests/golden/make_golden.py``), the convolution values with vectors computed
from the reference's metadata (``tests/golden/conv_vectors.npz``) and with the closed form of
``examples/basic_uvu_conv.py:35-38``.  The reference's CUDA kernels cannot run without a GPU, so no stored vectors
of theirs exist; instead ``oracle/build_ref.py`` compiles the kernels the reference generates and
``tests/test_gpu_reference_kernels.py`` runs them beside the library on the same GPU and inputs (small graphs to
second order, and two configurations at full size element by element): that is the pin of the convolution values.
"""

from __future__ import annotations

import math
from math import factorial

import numpy as np
import torch

# ----------------------------------------------------------------------------- irreps


def parse_irreps(text) -> list[tuple[int, int, int]]:
    """``"32x0e+32x1o"`` -> ``[(mul, l, parity), ...]``; also accepts an iterable of (mul, (l, p))."""
    if not isinstance(text, str):
        return [(int(mul), int(ir[0]), int(ir[1])) for mul, ir in text]
    blocks = []
    for part in text.replace(" ", "").split("+"):
        if not part:
            continue
        mul, name = part.split("x") if "x" in part else ("1", part)
        degree = int(name[:-1])
        parity = {"e": 1, "o": -1, "y": (-1) ** degree}[name[-1]]
        blocks.append((int(mul), degree, parity))
    return blocks


def block_offsets(blocks) -> list[int]:
    offsets, cursor = [], 0
    for mul, degree, _ in blocks:
        offsets.append(cursor)
        cursor += mul * (2 * degree + 1)
    return offsets


def irreps_dim(blocks) -> int:
    return sum(mul * (2 * degree + 1) for mul, degree, _ in blocks)


# ----------------------------------------------------------------------------- Clebsch-Gordan


def _su2_cg(j1, j2, j3):
    """<j1 m1 j2 m2|j3 m3>, Condon-Shortley phases, by the Racah series in float64."""
    table = np.zeros((2 * j1 + 1, 2 * j2 + 1, 2 * j3 + 1))
    if not abs(j1 - j2) <= j3 <= j1 + j2:
        return table
    delta = math.sqrt(
        factorial(j1 + j2 - j3) * factorial(j1 - j2 + j3) * factorial(-j1 + j2 + j3) / factorial(j1 + j2 + j3 + 1)
    )
    for m1 in range(-j1, j1 + 1):
        for m2 in range(-j2, j2 + 1):
            m3 = m1 + m2
            if abs(m3) > j3:
                continue
            norm = math.sqrt(
                (2 * j3 + 1)
                * factorial(j3 + m3) * factorial(j3 - m3)
                * factorial(j1 + m1) * factorial(j1 - m1)
                * factorial(j2 + m2) * factorial(j2 - m2)
            )
            total = 0.0
            for k in range(0, j1 + j2 - j3 + 1):
                args = (k, j1 + j2 - j3 - k, j1 - m1 - k, j2 + m2 - k, j3 - j2 + m1 + k, j3 - j1 - m2 + k)
                if min(args) < 0:
                    continue
                total += (-1) ** k / np.prod([float(factorial(a)) for a in args])
            table[j1 + m1, j2 + m2, j3 + m3] = delta * norm * total
    return table


def _real_basis(l):
    """Rows: complex m=-l..l; columns: real components (e3nn order), global phase (-i)^l."""
    q = np.zeros((2 * l + 1, 2 * l + 1), dtype=complex)
    s = 1 / math.sqrt(2)
    q[l, l] = 1
    for m in range(1, l + 1):
        q[l + m, l + m], q[l + m, l - m] = (-1) ** m * s, 1j * (-1) ** m * s
        q[l - m, l + m], q[l - m, l - m] = s, -1j * s
    return (-1j) ** l * q


_CG_CACHE: dict = {}


def real_cg(l1, l2, l3):
    """Real-basis coupling tensor with unit Frobenius norm (``src/lunatp/utils/cg.py:131-141``)."""
    key = (l1, l2, l3)
    if key not in _CG_CACHE:
        c = np.einsum("ai,bj,ck,abc->ijk", _real_basis(l1), _real_basis(l2), _real_basis(l3).conj(),
                      _su2_cg(l1, l2, l3).astype(complex))
        assert np.abs(c.imag).max() < 1e-5
        c = c.real
        _CG_CACHE[key] = c / np.linalg.norm(c)
    return _CG_CACHE[key]


# ----------------------------------------------------------------------------- paths


def normalised_paths(in1, in2, out, instructions, *, in1_var=None, in2_var=None, out_var=None,
                     irrep_normalization="component", path_normalization="element"):
    """Return ``[(i1, i2, io, sqrt(alpha)), ...]`` for uvu instructions (``layout.py:323-382``)."""
    in1_var = in1_var or [1.0] * len(in1)
    in2_var = in2_var or [1.0] * len(in2)
    out_var = out_var or [1.0] * len(out)
    ins = [tuple(i) + ((1.0,) if len(i) == 5 else ()) for i in instructions]
    for entry in ins:
        assert entry[3] == "uvu" and entry[4], "the oracle covers weighted uvu paths only"
    result = []
    for i1, i2, io, _, _, user in ins:
        d_out = 2 * out[io][1] + 1
        alpha = {"component": d_out, "norm": (2 * in1[i1][1] + 1) * (2 * in2[i2][1] + 1), "none": 1}[irrep_normalization]
        if path_normalization == "element":
            fan = sum(in1_var[a] * in2_var[b] * in2[b][0] for a, b, c, *_ in ins if c == io)
        elif path_normalization == "path":
            fan = in1_var[i1] * in2_var[i2] * in2[i2][0] * len([1 for *_, c, _, _, _ in ins if c == io])
        else:
            fan = 1
        if fan > 0:
            alpha /= fan
        alpha *= out_var[io]
        alpha *= user
        result.append((i1, i2, io, math.sqrt(alpha)))
    return result


def build_specs(irreps_in1, irreps_in2, irreps_out, instructions, **norm_kwargs):
    """Dense per-(instruction, edge channel) specs: offsets, dims and ``C * path_weight``."""
    in1, in2, out = parse_irreps(irreps_in1), parse_irreps(irreps_in2), parse_irreps(irreps_out)
    off1, off2, off_out = block_offsets(in1), block_offsets(in2), block_offsets(out)
    specs, weight_cursor = [], 0
    for i1, i2, io, path_weight in normalised_paths(in1, in2, out, instructions, **norm_kwargs):
        (mul1, l1, p1), (mul2, l2, p2), (mul_out, l3, p3) = in1[i1], in2[i2], out[io]
        assert p1 * p2 == p3 and abs(l1 - l2) <= l3 <= l1 + l2 and mul1 == mul_out
        for v in range(mul2):
            specs.append(dict(
                x_offset=off1[i1], y_offset=off2[i2] + v * (2 * l2 + 1), out_offset=off_out[io],
                weight_offset=weight_cursor + v, weight_stride=mul2, channels=mul1,
                d1=2 * l1 + 1, d2=2 * l2 + 1, d3=2 * l3 + 1, l1=l1, l2=l2, l3=l3,
                path_weight=path_weight, cg=real_cg(l1, l2, l3) * path_weight,
            ))
        weight_cursor += mul1 * mul2
    meta = dict(in1_dim=irreps_dim(in1), in2_dim=irreps_dim(in2), out_dim=irreps_dim(out),
                weight_numel=weight_cursor, specs=specs)
    return meta


def specs_from_reference_meta(meta):
    """Turn a reference-format metadata mapping (sparse ``terms``) into the dense specs used here."""
    specs = []
    for spec in meta["generated_specs"]:
        cg = np.zeros((spec["d1"], spec["d2"], spec["d3"]))
        for i, j, k, c in spec["terms"]:
            cg[i, j, k] = c
        specs.append(dict(
            x_offset=spec["x_offset"], y_offset=spec["y_offset"], out_offset=spec["out_offset"],
            weight_offset=spec["weight_offset"], weight_stride=spec.get("weight_stride", 1),
            channels=spec["channels"], d1=spec["d1"], d2=spec["d2"], d3=spec["d3"], cg=cg,
        ))
    return dict(in1_dim=meta["in1_dim"], in2_dim=meta["in2_dim"], out_dim=meta["out_dim"],
                weight_numel=meta["weight_numel"], specs=specs)


# ----------------------------------------------------------------------------- the convolution


def conv_forward(meta, x, y, w, src, dst, num_nodes):
    """Differentiable dense evaluation: gather, couple, weight, scatter-sum by destination."""
    src = src.long()
    dst = dst.long()
    out = x.new_zeros((num_nodes, meta["out_dim"]))
    if src.numel() == 0:
        return out + 0.0 * (x.sum() + y.sum() + w.sum())
    xs = x[src]
    pieces = []
    for spec in meta["specs"]:
        ch, d1, d2, d3 = spec["channels"], spec["d1"], spec["d2"], spec["d3"]
        cg = torch.as_tensor(spec["cg"], dtype=x.dtype)
        xb = xs[:, spec["x_offset"]: spec["x_offset"] + ch * d1].reshape(-1, ch, d1)
        yb = y[:, spec["y_offset"]: spec["y_offset"] + d2]
        stride = spec["weight_stride"]
        wb = w[:, spec["weight_offset"]: spec["weight_offset"] + (ch - 1) * stride + 1: stride]
        msg = torch.einsum("ijk,eui,ej,eu->euk", cg, xb, yb, wb).reshape(-1, ch * d3)
        pieces.append((spec["out_offset"], ch * d3, msg))
    result = x.new_zeros((num_nodes, meta["out_dim"]))
    for offset, width, msg in pieces:
        block = x.new_zeros((num_nodes, width)).index_add(0, dst, msg)
        result = result + torch.nn.functional.pad(block, (offset, meta["out_dim"] - offset - width))
    return result


def conv_derivatives(meta, x, y, w, src, dst, num_nodes, g, rx=None, ry=None, rw=None):
    """Forward, first derivatives (cotangent g) and second derivatives (cotangents rx, ry, rw of gx, gy, gw).

    Returns a dict with out, gx, gy, gw and - when any r* is given - hx, hy, hw, hg, following the reference's
    double-backward contract (``src/lunatp/utils/contractions.py:41-49``).
    """
    x = x.detach().clone().requires_grad_(True)
    y = y.detach().clone().requires_grad_(True)
    w = w.detach().clone().requires_grad_(True)
    g = g.detach().clone().requires_grad_(True)
    out = conv_forward(meta, x, y, w, src, dst, num_nodes)
    second = any(r is not None for r in (rx, ry, rw))
    gx, gy, gw = torch.autograd.grad(out, (x, y, w), g, create_graph=second)
    result = dict(out=out.detach(), gx=gx.detach(), gy=gy.detach(), gw=gw.detach())
    if second:
        outs, seeds = [], []
        for value, seed in ((gx, rx), (gy, ry), (gw, rw)):
            if seed is not None:
                outs.append(value)
                seeds.append(seed)
        hx, hy, hw, hg = torch.autograd.grad(outs, (x, y, w, g), seeds, allow_unused=True)
        for name, value, like in (("hx", hx, x), ("hy", hy, y), ("hw", hw, w), ("hg", hg, g)):
            result[name] = torch.zeros_like(like) if value is None else value.detach()
    return result


def conv_forward_chunked(meta, x, y, w, src, dst, num_nodes, chunk_edges=65536):
    """Memory-bounded forward for timing on large graphs (no autograd); any float dtype."""
    out = x.new_zeros((num_nodes, meta["out_dim"]))
    edges = src.numel()
    with torch.no_grad():
        for begin in range(0, edges, chunk_edges):
            end = min(edges, begin + chunk_edges)
            s, d = src[begin:end].long(), dst[begin:end].long()
            xs = x[s]
            for spec in meta["specs"]:
                ch, d1, d2, d3 = spec["channels"], spec["d1"], spec["d2"], spec["d3"]
                cg = torch.as_tensor(spec["cg"], dtype=x.dtype)
                xb = xs[:, spec["x_offset"]: spec["x_offset"] + ch * d1].reshape(-1, ch, d1)
                yb = y[begin:end, spec["y_offset"]: spec["y_offset"] + d2]
                stride = spec["weight_stride"]
                wb = w[begin:end, spec["weight_offset"]: spec["weight_offset"] + (ch - 1) * stride + 1: stride]
                m = torch.einsum("ijk,ej->eik", cg, yb)
                msg = (torch.einsum("eik,eui->euk", m, xb) * wb[:, :, None]).reshape(-1, ch * d3)
                out[:, spec["out_offset"]: spec["out_offset"] + ch * d3].index_add_(0, d, msg)
    return out


def conv_forward_backward_chunked(meta, x, y, w, g, src, dst, num_nodes, chunk_edges=32768):
    """Forward + first derivatives on a large graph, chunked over edges, via autograd per chunk."""
    out = x.new_zeros((num_nodes, meta["out_dim"]))
    gx = torch.zeros_like(x)
    gy = torch.empty_like(y)
    gw = torch.empty_like(w)
    edges = src.numel()
    for begin in range(0, edges, chunk_edges):
        end = min(edges, begin + chunk_edges)
        xc = x.detach().requires_grad_(True)
        yc = y[begin:end].detach().requires_grad_(True)
        wc = w[begin:end].detach().requires_grad_(True)
        part = conv_forward(meta, xc, yc, wc, src[begin:end], dst[begin:end], num_nodes)
        a, b, c = torch.autograd.grad(part, (xc, yc, wc), g)
        out += part.detach()
        gx += a
        gy[begin:end] = b
        gw[begin:end] = c
    return out, gx, gy, gw
