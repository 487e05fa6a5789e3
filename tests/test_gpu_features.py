"""Envelope, per-edge scalar features and third-order derivatives on the GPU against the float64 oracle.

The reference exercises these together (``tests/lunatp/test_uvu_conv.py:297-329,649-930``): ``env`` scales every
edge's message before aggregation, ``return_l0_feat`` also returns the raw per-edge contributions of the paths into
degree 0 (without ``env``), and the whole operator is differentiable three times.
"""

import pytest
import torch

import lunaequivariance_b200 as luna
from oracle import uvu_conv as oracle_conv
from tests.helpers import assert_close, config, random_graph

pytestmark = pytest.mark.gpu
DEVICE = "cuda"


def dense_reference(meta, x, y, w, env, src, dst, nodes):
    """out (with envelope) and the per-edge scalar features (without), from per-edge messages of every path."""
    xs = x[src]
    out = x.new_zeros((nodes, meta["out_dim"]))
    scalar_blocks, block_of = [], {}
    order = sorted(range(len(meta["specs"])), key=lambda i: meta["specs"][i]["out_offset"])
    messages = {}
    for index, spec in enumerate(meta["specs"]):
        ch, d1, d2, d3 = spec["channels"], spec["d1"], spec["d2"], spec["d3"]
        xb = xs[:, spec["x_offset"]: spec["x_offset"] + ch * d1].reshape(-1, ch, d1)
        yb = y[:, spec["y_offset"]: spec["y_offset"] + d2]
        wb = w[:, spec["weight_offset"]: spec["weight_offset"] + (ch - 1) * spec["weight_stride"] + 1:
               spec["weight_stride"]]
        msg = torch.einsum("ijk,eui,ej,eu->euk", torch.as_tensor(spec["cg"], dtype=x.dtype), xb, yb, wb)
        messages[index] = msg
        scaled = msg if env is None else msg * env.reshape(-1, 1, 1)
        piece = x.new_zeros((nodes, ch * d3)).index_add(0, dst, scaled.reshape(-1, ch * d3))
        out = out + torch.nn.functional.pad(piece, (spec["out_offset"], meta["out_dim"] - spec["out_offset"] - ch * d3))
    # one block per instruction into degree 0, in the order of the output offsets; the specs one instruction was
    # split into (consecutive, weights interleaved) share its block
    instruction, count = {}, 0
    for index, spec in enumerate(meta["specs"]):
        previous = meta["specs"][index - 1] if index else None
        continues = (previous is not None and spec["weight_stride"] > 1
                     and all(spec[k] == previous[k] for k in ("x_offset", "out_offset", "l1", "l2", "weight_stride"))
                     and spec["weight_offset"] == previous["weight_offset"] + 1)
        count += 0 if continues else 1
        instruction[index] = count
    for index in order:
        if meta["specs"][index]["l3"] != 0:
            continue
        if instruction[index] in block_of:
            scalar_blocks[block_of[instruction[index]]] = scalar_blocks[block_of[instruction[index]]] + messages[index][:, :, 0]
        else:
            block_of[instruction[index]] = len(scalar_blocks)
            scalar_blocks.append(messages[index][:, :, 0])
    l0 = torch.cat(scalar_blocks, dim=1) if scalar_blocks else x.new_zeros((src.numel(), 0))
    return out, l0


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
@pytest.mark.parametrize("name", ["fixture", "cfg5", "mul2", "highl"])
def test_envelope_and_scalar_features_with_gradients(name, dtype):
    in1, in2, out_irreps, instructions, options = config(name)
    module = luna.TensorProductConv(in1, in2, out_irreps, instructions, internal_weights=False, shared_weights=False,
                                    dtype=dtype, **options)
    meta = oracle_conv.build_specs(in1, in2, out_irreps, instructions, **options)
    generator = torch.Generator().manual_seed(12)
    nodes, edges = 29, 211
    src, dst = random_graph(nodes, edges, generator)
    rand = lambda *shape: torch.randn(*shape, generator=generator, dtype=torch.float64).to(dtype)
    host = dict(x=rand(nodes, meta["in1_dim"]), y=rand(edges, meta["in2_dim"]), w=rand(edges, meta["weight_numel"]),
                env=rand(edges, 1))
    graph = module.create_graph(src.to(DEVICE), dst.to(DEVICE), nodes)
    dev = {k: v.to(DEVICE).requires_grad_(True) for k, v in host.items()}
    out, l0 = module(dev["x"], dev["y"], dev["w"], graph=graph, env=dev["env"], return_l0_feat=True)
    ref = {k: v.double().requires_grad_(True) for k, v in host.items()}
    ref_out, ref_l0 = dense_reference(meta, ref["x"], ref["y"], ref["w"], ref["env"], src, dst, nodes)
    assert l0.shape == (edges, module.op.l0_dim) == tuple(ref_l0.shape)
    assert_close(out, ref_out.detach(), dtype, f"{name} out with env")
    assert_close(l0, ref_l0.detach(), dtype, f"{name} l0 features")
    seeds = (rand(*out.shape), rand(*l0.shape))
    names = ("x", "y", "w", "env")
    got = torch.autograd.grad((out, l0), [dev[k] for k in names], [s.to(DEVICE) for s in seeds], create_graph=True)
    want = torch.autograd.grad((ref_out, ref_l0), [ref[k] for k in names], [s.double() for s in seeds],
                               create_graph=True)
    for key, a, b in zip(names, got, want):
        assert_close(a, b.detach(), dtype, f"{name} d/d{key}")
    # one second-order check through both outputs: the force-style contraction of the envelope gradient
    second = torch.autograd.grad(got[3].square().sum(), dev["w"])[0]
    second_ref = torch.autograd.grad(want[3].square().sum(), ref["w"])[0]
    assert_close(second, second_ref, dtype, f"{name} d/dw of |d/denv|^2")
    # 1-d envelopes are accepted too
    flat = module(dev["x"], dev["y"], dev["w"], graph=graph, env=dev["env"].detach().reshape(-1))
    assert_close(flat, ref_out.detach(), dtype, f"{name} out with 1-d env")
    with pytest.raises(ValueError):
        module(dev["x"], dev["y"], dev["w"], graph=graph, env=dev["env"][:-1])


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
@pytest.mark.parametrize("name", ["fixture", "cfg2"])
def test_third_order_derivatives(name, dtype):
    in1, in2, out_irreps, instructions, options = config(name)
    module = luna.TensorProductConv(in1, in2, out_irreps, instructions, internal_weights=False, shared_weights=False,
                                    dtype=dtype, **options)
    meta = oracle_conv.build_specs(in1, in2, out_irreps, instructions, **options)
    generator = torch.Generator().manual_seed(4)
    nodes, edges = 17, 90
    src, dst = random_graph(nodes, edges, generator)
    rand = lambda *shape: torch.randn(*shape, generator=generator, dtype=torch.float64).to(dtype)
    shapes = dict(x=(nodes, meta["in1_dim"]), y=(edges, meta["in2_dim"]), w=(edges, meta["weight_numel"]),
                  g=(nodes, meta["out_dim"]))
    host = {k: rand(*shape) for k, shape in shapes.items()}
    for k in ("x", "y", "w"):
        host["r" + k] = rand(*shapes[k])
    for k in ("x", "y", "w", "g"):
        host["b" + k] = rand(*shapes[k])
    graph = module.create_graph(src.to(DEVICE), dst.to(DEVICE), nodes)

    def chain(conv, t):
        out = conv(t["x"], t["y"], t["w"])
        first = torch.autograd.grad(out, (t["x"], t["y"], t["w"]), t["g"], create_graph=True)
        second = torch.autograd.grad(first, (t["x"], t["y"], t["w"], t["g"]), (t["rx"], t["ry"], t["rw"]),
                                     create_graph=True)
        third = torch.autograd.grad(second, (t["x"], t["y"], t["w"], t["g"], t["rx"], t["ry"], t["rw"]),
                                    (t["bx"], t["by"], t["bw"], t["bg"]), allow_unused=True)
        return out, first, second, third

    need = ("x", "y", "w", "g", "rx", "ry", "rw")
    dev = {k: v.to(DEVICE).requires_grad_(k in need) for k, v in host.items()}
    ref = {k: v.double().requires_grad_(k in need) for k, v in host.items()}
    got = chain(lambda x, y, w: module(x, y, w, graph=graph), dev)
    want = chain(lambda x, y, w: oracle_conv.conv_forward(meta, x, y, w, src, dst, nodes), ref)
    labels = ("dx", "dy", "dw", "dg", "drx", "dry", "drw")
    for label, a, b in zip(labels, got[3], want[3]):
        assert (a is None) == (b is None), label
        if a is not None:
            assert_close(a, b, dtype, f"{name} third order {label}")
    module.op.check_status()


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
@pytest.mark.parametrize("shared", [False, True])
def test_tensor_product_without_graph(shared, dtype):
    """The per-item UVU tensor product (``TensorProduct`` / ``tensor_product``): values, first and second derivatives
    against the oracle on the identity graph; batch dimensions and shared weights."""
    in1, in2, out_irreps, instructions, options = config("cfg5")
    module = luna.TensorProduct(in1, in2, out_irreps, instructions, internal_weights=False, shared_weights=shared,
                                dtype=dtype)
    meta = oracle_conv.build_specs(in1, in2, out_irreps, instructions)
    generator = torch.Generator().manual_seed(31)
    batch = (3, 5)
    items = 15
    rand = lambda *shape: torch.randn(*shape, generator=generator, dtype=torch.float64).to(dtype)
    host = dict(x=rand(*batch, meta["in1_dim"]), y=rand(*batch, meta["in2_dim"]),
                w=rand(meta["weight_numel"]) if shared else rand(*batch, meta["weight_numel"]))
    dev = {k: v.to(DEVICE).requires_grad_(True) for k, v in host.items()}
    ref = {k: v.double().requires_grad_(True) for k, v in host.items()}
    own = torch.arange(items)

    def dense(t):
        w = t["w"].unsqueeze(0).expand(items, -1) if shared else t["w"].reshape(items, -1)
        return oracle_conv.conv_forward(meta, t["x"].reshape(items, -1), t["y"].reshape(items, -1), w, own, own,
                                        items).reshape(*batch, meta["out_dim"])

    out, ref_out = module(dev["x"], dev["y"], dev["w"]), dense(ref)
    assert out.shape == (*batch, meta["out_dim"])
    assert_close(out, ref_out.detach(), dtype, "tensor product")
    g = rand(*out.shape)
    names = ("x", "y", "w")
    got = torch.autograd.grad(out, [dev[k] for k in names], g.to(DEVICE), create_graph=True)
    want = torch.autograd.grad(ref_out, [ref[k] for k in names], g.double(), create_graph=True)
    for key, a, b in zip(names, got, want):
        assert_close(a, b.detach(), dtype, f"tensor product d/d{key}")
    second = torch.autograd.grad(got[1].square().sum(), dev["w"])[0]
    second_ref = torch.autograd.grad(want[1].square().sum(), ref["w"])[0]
    assert_close(second, second_ref, dtype, "tensor product second order")
    functional = luna.tensor_product(dev["x"], dev["y"], dev["w"], irreps_in1=in1, irreps_in2=in2,
                                     irreps_out=out_irreps, instructions=instructions, shared_weights=shared)
    assert_close(functional, ref_out.detach(), dtype, "functional tensor product")
