"""Parity of the CUDA convolution (through the C-ABI) with the CPU oracle: forward, first and second derivatives."""

import pytest
import torch

import lunaequivariance_b200 as luna
from oracle import uvu_conv as oracle_conv
from tests.helpers import assert_close, config, random_graph, random_problem

pytestmark = pytest.mark.gpu
DEVICE = "cuda"


def build(name, dtype):
    in1, in2, out, instructions, options = config(name)
    conv = luna.TensorProductConv(in1, in2, out, instructions, internal_weights=False, shared_weights=False,
                                  dtype=dtype, **options)
    meta = oracle_conv.build_specs(in1, in2, out, instructions, **options)
    return conv, meta


def run_case(name, dtype, nodes, edges, *, exact_degree=None, generic=False, seed=0, second=True):
    conv, meta = build(name, dtype)
    if generic:
        conv.op.force_generic(True)
    generator = torch.Generator().manual_seed(seed)
    src, dst = random_graph(nodes, edges, generator, exact_degree)
    dims = (meta["in1_dim"], meta["in2_dim"], meta["out_dim"], meta["weight_numel"])
    p = random_problem(dims, nodes, src, dtype, generator)
    ref = oracle_conv.conv_derivatives(
        meta, *(p[k].double() for k in ("x", "y", "w")), src, dst, nodes, p["g"].double(),
        *((p[k].double() for k in ("rx", "ry", "rw")) if second else (None, None, None)))
    graph = conv.create_graph(src.to(DEVICE), dst.to(DEVICE), nodes)
    x, y, w, g = (p[k].to(DEVICE).requires_grad_(True) for k in ("x", "y", "w", "g"))
    out = conv(x, y, w, graph=graph)
    assert_close(out, ref["out"], dtype, f"{name} out")
    gx, gy, gw = torch.autograd.grad(out, (x, y, w), g, create_graph=second)
    for key, value in (("gx", gx), ("gy", gy), ("gw", gw)):
        assert_close(value, ref[key], dtype, f"{name} {key}")
    if second:
        seeds = tuple(p[k].to(DEVICE) for k in ("rx", "ry", "rw"))
        hx, hy, hw, hg = torch.autograd.grad((gx, gy, gw), (x, y, w, g), seeds)
        for key, value in (("hx", hx), ("hy", hy), ("hw", hw), ("hg", hg)):
            assert_close(value, ref[key], dtype, f"{name} {key}")
    return conv


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
@pytest.mark.parametrize("name", ["cfg1", "fixture", "small", "mul2", "odd", "one", "mixed", "highl", "partial",
                                  "norm_path"])
def test_generic_kernels_match_oracle(name, dtype):
    run_case(name, dtype, nodes=13, edges=57, generic=True)


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
@pytest.mark.parametrize("name", ["cfg1", "fixture", "cfg5", "cfg2", "cfg4", "partial", "wide"])
def test_staged_kernels_match_oracle(name, dtype):
    conv = run_case(name, dtype, nodes=41, edges=333)
    assert conv.op.uses_staged_kernels


def test_config1_full_size_fp64():
    """Benchmark configuration 1: 1000 atoms x 16 incoming edges, FP64, forward + first + second derivatives."""
    run_case("cfg1", torch.float64, nodes=1000, edges=None, exact_degree=16)


@pytest.mark.parametrize("name", ["cfg1", "small", "mul2", "mixed", "highl", "fixture"])
def test_golden_vectors_from_reference_metadata(name, golden_npz):
    data = golden_npz("conv_vectors.npz")
    get = lambda key: torch.from_numpy(data[f"{name}.{key}"])
    conv, _ = build(name, torch.float64)
    nodes = int(data[f"{name}.num_nodes"])
    graph = conv.create_graph(get("src").to(DEVICE), get("dst").to(DEVICE), nodes)
    x, y, w, g = (get(k).to(DEVICE).requires_grad_(True) for k in ("x", "y", "w", "g"))
    out = conv(x, y, w, graph=graph)
    gx, gy, gw = torch.autograd.grad(out, (x, y, w), g, create_graph=True)
    hx, hy, hw, hg = torch.autograd.grad((gx, gy, gw), (x, y, w, g), tuple(get(k).to(DEVICE) for k in ("rx", "ry", "rw")))
    for key, value in dict(out=out, gx=gx, gy=gy, gw=gw, hx=hx, hy=hy, hw=hw, hg=hg).items():
        assert_close(value, get(key), torch.float64, f"{name} {key}")


def test_closed_form_dot_product_example():
    """Cx1o (x) 1x1o -> Cx0e equals dot(x, y) * w / sqrt(3) (reference examples/basic_uvu_conv.py:35-38)."""
    torch.manual_seed(7)
    dtype, nodes, edges, channels = torch.float64, 3, 4, 32
    tp = luna.TensorProductConfig(f"{channels}x1o", "1x1o", f"{channels}x0e", [(0, 0, 0, "uvu", True)],
                                  internal_weights=False, shared_weights=False).to(device=DEVICE, dtype=dtype)
    op = luna.TensorProductConv(tp, dtype=dtype)
    src = torch.tensor([0, 2, 1, 0], device=DEVICE)
    dst = torch.tensor([2, 0, 2, 1], device=DEVICE)
    x = torch.randn(nodes, tp.irreps_in1.dim, device=DEVICE, dtype=dtype, requires_grad=True)
    edge_attr = torch.randn(edges, 3, device=DEVICE, dtype=dtype)
    weight = torch.randn(edges, tp.weight_numel, device=DEVICE, dtype=dtype, requires_grad=True)
    order = dst.argsort(stable=True)
    graph = op.create_graph(src[order], dst[order], nodes)
    out = op(x, edge_attr[order], weight[order], graph=graph)
    messages = (x[src].reshape(edges, channels, 3) * edge_attr[:, None, :]).sum(-1) * weight / 3 ** 0.5
    reference = x.new_zeros(nodes, channels).index_add(0, dst, messages)
    torch.testing.assert_close(out, reference, atol=1e-12, rtol=1e-11)
    out.square().mean().backward()
    assert x.grad is not None and weight.grad is not None


@pytest.mark.parametrize("generic", [True, False])
def test_empty_graph_and_isolated_nodes(generic):
    conv, meta = build("fixture", torch.float64)
    if generic:
        conv.op.force_generic(True)
    empty = torch.zeros(0, dtype=torch.long, device=DEVICE)
    graph = conv.create_graph(empty, empty, 5)
    x = torch.randn(5, meta["in1_dim"], device=DEVICE, dtype=torch.float64, requires_grad=True)
    y = torch.zeros(0, meta["in2_dim"], device=DEVICE, dtype=torch.float64, requires_grad=True)
    w = torch.zeros(0, meta["weight_numel"], device=DEVICE, dtype=torch.float64, requires_grad=True)
    out = conv(x, y, w, graph=graph)
    assert out.shape == (5, meta["out_dim"]) and not out.any()
    (gx,) = torch.autograd.grad(out.sum(), x)
    assert not gx.any()
    # nodes 0, 3 and 6 have no incoming edge and 5 has no outgoing edge
    src = torch.tensor([1, 2, 2, 4], device=DEVICE)
    dst = torch.tensor([1, 2, 4, 5], device=DEVICE)
    graph = conv.create_graph(src, dst, 7)
    x = torch.randn(7, meta["in1_dim"], device=DEVICE, dtype=torch.float64, requires_grad=True)
    y = torch.randn(4, meta["in2_dim"], device=DEVICE, dtype=torch.float64)
    w = torch.randn(4, meta["weight_numel"], device=DEVICE, dtype=torch.float64)
    out = conv(x, y, w, graph=graph)
    assert not out[[0, 3, 6]].any() and out[[1, 2, 4, 5]].abs().sum() > 0
    ref = oracle_conv.conv_forward(meta, x.detach().cpu(), y.cpu(), w.cpu(), src.cpu(), dst.cpu(), 7)
    assert_close(out, ref, torch.float64, "isolated nodes")
    (gx,) = torch.autograd.grad(out.square().sum(), x)
    assert not gx[[0, 3, 5, 6]].any()


def test_bitwise_determinism_and_staged_equals_generic():
    conv, meta = build("cfg5", torch.float32)
    generator = torch.Generator().manual_seed(3)
    nodes = 200
    src, dst = random_graph(nodes, 3000, generator)
    dims = (meta["in1_dim"], meta["in2_dim"], meta["out_dim"], meta["weight_numel"])
    p = random_problem(dims, nodes, src, torch.float32, generator)
    graph = conv.create_graph(src.to(DEVICE), dst.to(DEVICE), nodes)
    args = [p[k].to(DEVICE) for k in ("x", "y", "w")]

    def step():
        x, y, w = (a.clone().requires_grad_(True) for a in args)
        out = conv(x, y, w, graph=graph)
        return (out,) + torch.autograd.grad(out, (x, y, w), p["g"].to(DEVICE))

    first, second = step(), step()
    for a, b in zip(first, second):
        assert torch.equal(a, b)
    conv.op.force_generic(True)
    for a, b in zip(first, step()):
        torch.testing.assert_close(a, b, rtol=2e-5, atol=2e-5 * a.abs().max().item())


def test_non_contiguous_and_offset_inputs():
    conv, meta = build("fixture", torch.float32)
    generator = torch.Generator().manual_seed(5)
    nodes, edges = 7, 19
    src, dst = random_graph(nodes, edges, generator)
    graph = conv.create_graph(src.to(DEVICE), dst.to(DEVICE), nodes)
    x = torch.randn(meta["in1_dim"], nodes, generator=generator).to(DEVICE).t()
    y = torch.randn(meta["in2_dim"], edges, generator=generator).to(DEVICE).t()
    w = torch.randn(edges + 1, meta["weight_numel"] + 1, generator=generator).to(DEVICE)[1:, 1:]
    assert not x.is_contiguous() and not w.is_contiguous()
    out = conv(x, y, w, graph=graph)
    ref = oracle_conv.conv_forward(meta, x.cpu().double(), y.cpu().double(), w.cpu().double(), src, dst, nodes)
    assert_close(out, ref, torch.float32, "strided inputs")


def test_dtype_migration_rebuilds_operator():
    conv, _ = build("fixture", torch.float32)
    assert conv.op.compute_dtype == torch.float32
    conv = conv.double()
    assert conv.op.compute_dtype == torch.float64
    run_case("fixture", torch.float64, 9, 30, second=False)


def test_missing_cotangents_are_not_materialised():
    """Force-training pattern: only the edge attributes are differentiated twice."""
    conv, meta = build("fixture", torch.float64)
    generator = torch.Generator().manual_seed(9)
    nodes, edges = 11, 47
    src, dst = random_graph(nodes, edges, generator)
    dims = (meta["in1_dim"], meta["in2_dim"], meta["out_dim"], meta["weight_numel"])
    p = random_problem(dims, nodes, src, torch.float64, generator)
    graph = conv.create_graph(src.to(DEVICE), dst.to(DEVICE), nodes)
    x = p["x"].to(DEVICE)
    y = p["y"].to(DEVICE).requires_grad_(True)
    w = p["w"].to(DEVICE).requires_grad_(True)
    energy = conv(x, y, w, graph=graph).square().sum()
    (force,) = torch.autograd.grad(energy, y, create_graph=True)
    (gw,) = torch.autograd.grad(force.square().sum(), w)
    xo, yo, wo = p["x"].clone(), p["y"].clone().requires_grad_(True), p["w"].clone().requires_grad_(True)
    e_ref = oracle_conv.conv_forward(meta, xo, yo, wo, src, dst, nodes).square().sum()
    (f_ref,) = torch.autograd.grad(e_ref, yo, create_graph=True)
    (gw_ref,) = torch.autograd.grad(f_ref.square().sum(), wo)
    assert_close(force, f_ref.detach(), torch.float64, "force")
    assert_close(gw, gw_ref, torch.float64, "dL/dw through forces")


def test_input_validation_errors():
    conv, meta = build("fixture", torch.float32)
    graph = conv.create_graph(torch.tensor([0, 1], device=DEVICE), torch.tensor([0, 1], device=DEVICE), 2)
    x = torch.randn(2, meta["in1_dim"], device=DEVICE)
    y = torch.randn(2, meta["in2_dim"], device=DEVICE)
    w = torch.randn(2, meta["weight_numel"], device=DEVICE)
    with pytest.raises(TypeError):
        conv(x.double(), y, w, graph=graph)
    with pytest.raises(ValueError):
        conv(x[:, :-1], y, w, graph=graph)
    with pytest.raises(ValueError):
        conv(x, y, w, graph=graph, env=torch.ones(3, device=DEVICE))
    with pytest.raises(TypeError):
        conv(x, y, w, graph=graph, env=torch.ones(2, device=DEVICE, dtype=torch.float64))
    with pytest.raises(RuntimeError, match="CUDA is required"):
        conv(x.cpu(), y.cpu(), w.cpu(), graph=graph)


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
@pytest.mark.parametrize("name", ["cfg2", "cfg5", "cfg4"])
@pytest.mark.parametrize("knob", ["LUNA_B200_NO_CANON=1", "LUNA_B200_NO_SPARSE=1", "LUNA_B200_BWD_KERNEL=row",
                                  "LUNA_B200_BWD_KERNEL=units", "LUNA_B200_NO_PLAIN=1"])
def test_staged_kernel_variants_match_oracle(name, dtype, knob, monkeypatch):
    """The canonical configurations through the kernels they do not all take by default: loops over run-time path
    tables (NO_CANON), the unrolled kernel with dense coupling matrices (NO_SPARSE), and the two data-movement
    variants of the backward kernel with compiled-in coupling patterns (row stages / unit ring)."""
    monkeypatch.setenv(*knob.split("="))
    conv = run_case(name, dtype, nodes=37, edges=301, seed=3)
    assert conv.op.uses_staged_kernels and conv.op.canonical_l2 >= 0


def test_backward_skips_source_rows_without_edges():
    """A block of source rows with no out-edges (as on a destination-range shard) must come back as zeros."""
    dtype = torch.float32
    conv, meta = build("cfg5", dtype)
    generator = torch.Generator().manual_seed(11)
    nodes, edges = 96, 700
    src = torch.randint(32, (edges,), generator=generator)  # only the first third of the rows are sources
    dst = torch.sort(torch.randint(nodes, (edges,), generator=generator))[0]
    dims = (meta["in1_dim"], meta["in2_dim"], meta["out_dim"], meta["weight_numel"])
    p = random_problem(dims, nodes, src, dtype, generator)
    ref = oracle_conv.conv_derivatives(meta, *(p[k].double() for k in ("x", "y", "w")), src, dst, nodes,
                                       p["g"].double(), None, None, None)
    graph = conv.create_graph(src.to(DEVICE), dst.to(DEVICE), nodes)
    x, y, w, g = (p[k].to(DEVICE).requires_grad_(True) for k in ("x", "y", "w", "g"))
    out = conv(x, y, w, graph=graph)
    gx, gy, gw = torch.autograd.grad(out, (x, y, w), g)
    assert_close(gx, ref["gx"], dtype, "gx with empty rows")
    assert float(gx[32:].abs().max()) == 0.0
    assert_close(gy, ref["gy"], dtype, "gy")
    assert_close(gw, ref["gw"], dtype, "gw")
