"""Host-side logic of the differentiable operator, checked on CPU with the oracle standing in for the kernels.

What is under test is everything above the C-ABI: the autograd chain to third order (the fused first- and
second-order functions and the partial-derivative function that closes the chain), the pruning of gradients nobody
consumes, and the composition of ``env`` and ``return_l0_feat`` from plain convolutions.  The three launch wrappers are
replaced by the float64 oracle evaluated on the operator's own metadata, so any operator (including the per-edge
scalar-feature operator) is covered by the same substitute.
"""

import pytest
import torch

import lunaequivariance_b200 as luna
from lunaequivariance_b200 import conv as conv_mod
from oracle import uvu_conv as oracle_conv
from tests.helpers import config, random_graph


@pytest.fixture()
def oracle_kernels(monkeypatch):
    calls = []

    def meta_of(op):
        return oracle_conv.specs_from_reference_meta(op.meta)

    def forward(op, x, y, w, graph):
        calls.append(("forward",))
        return oracle_conv.conv_forward(meta_of(op), x, y, w, graph.src, graph.dst, graph.num_nodes).detach()

    def backward(op, x, y, w, g, graph, needs=(True, True, True)):
        calls.append(("backward", tuple(bool(n) for n in needs)))
        with torch.enable_grad():  # launch wrappers are called from autograd.Function.forward, where grad mode is off
            ref = oracle_conv.conv_derivatives(meta_of(op), x, y, w, graph.src, graph.dst, graph.num_nodes, g)
        return tuple(ref[k] if need else None for k, need in zip(("gx", "gy", "gw"), needs))

    def double_backward(op, x, y, w, g, rx, ry, rw, graph, needs=(True, True, True, True)):
        calls.append(("double", tuple(bool(n) for n in needs)))
        with torch.enable_grad():
            ref = oracle_conv.conv_derivatives(meta_of(op), x, y, w, graph.src, graph.dst, graph.num_nodes, g, rx, ry, rw)
        return tuple(ref[k] if need else None for k, need in zip(("hx", "hy", "hw", "hg"), needs))

    monkeypatch.setattr(conv_mod, "run_forward", forward)
    monkeypatch.setattr(conv_mod, "run_backward", backward)
    monkeypatch.setattr(conv_mod, "run_double_backward", double_backward)
    return calls


def _problem(name, nodes=9, edges=31, seed=5):
    in1, in2, out, instructions, options = config(name)
    module = luna.TensorProductConv(in1, in2, out, instructions, internal_weights=False, shared_weights=False,
                                    dtype=torch.float64, **options)
    meta = oracle_conv.build_specs(in1, in2, out, instructions, **options)
    generator = torch.Generator().manual_seed(seed)
    src, dst = random_graph(nodes, edges, generator)
    graph = module.create_graph(src, dst, nodes)
    rand = lambda *shape: torch.randn(*shape, generator=generator, dtype=torch.float64)
    tensors = dict(x=rand(nodes, meta["in1_dim"]), y=rand(edges, meta["in2_dim"]), w=rand(edges, meta["weight_numel"]))
    return module, meta, graph, src, dst, tensors, rand


def _third_order(function, x, y, w, seeds):
    out = function(x, y, w)
    first = torch.autograd.grad(out, (x, y, w), seeds["g"], create_graph=True)
    second = torch.autograd.grad(first, (x, y, w, seeds["g"]), (seeds["rx"], seeds["ry"], seeds["rw"]),
                                 create_graph=True)
    third = torch.autograd.grad(second, (x, y, w, seeds["g"], seeds["rx"], seeds["ry"], seeds["rw"]),
                                (seeds["bx"], seeds["by"], seeds["bw"], seeds["bg"]), allow_unused=True)
    return out, first, second, third


@pytest.mark.parametrize("name", ["small", "mul2"])
def test_third_order_chain_matches_dense_autograd(name, oracle_kernels):
    module, meta, graph, src, dst, t, rand = _problem(name)
    nodes = graph.num_nodes
    seeds = dict(g=rand(nodes, meta["out_dim"]), rx=rand(*t["x"].shape), ry=rand(*t["y"].shape), rw=rand(*t["w"].shape),
                 bx=rand(*t["x"].shape), by=rand(*t["y"].shape), bw=rand(*t["w"].shape),
                 bg=rand(nodes, meta["out_dim"]))
    for key in ("g", "rx", "ry", "rw"):
        seeds[key].requires_grad_(True)
    leaves = lambda: tuple(t[k].clone().requires_grad_(True) for k in ("x", "y", "w"))
    got = _third_order(lambda x, y, w: module(x, y, w, graph=graph), *leaves(), seeds)
    want = _third_order(lambda x, y, w: oracle_conv.conv_forward(meta, x, y, w, src, dst, nodes), *leaves(), seeds)
    for order, (a, b) in enumerate(zip(got[1:], want[1:]), start=1):
        for position, (u, v) in enumerate(zip(a, b)):
            assert (u is None) == (v is None), (order, position)
            if u is not None:
                torch.testing.assert_close(u, v, atol=1e-10, rtol=1e-10, msg=f"order {order} output {position}")
    torch.testing.assert_close(got[0], want[0], atol=1e-12, rtol=1e-12)


def test_force_step_skips_unused_gradients(oracle_kernels):
    """Energy differentiated with respect to the edge attributes only, then the loss with respect to the weights:
    the weight-sized first-order gradient and the x gradients are never asked of the kernels."""
    module, meta, graph, src, dst, t, rand = _problem("small")
    x = t["x"]
    vec = t["y"].clone().requires_grad_(True)
    w = t["w"].clone().requires_grad_(True)
    out = module(x, vec * 1.5, w, graph=graph)
    (force,) = torch.autograd.grad(out.square().sum(), vec, create_graph=True)
    (grad_w,) = torch.autograd.grad(force.square().sum(), w)
    assert ("backward", (False, True, False)) in oracle_kernels
    assert ("double", (False, False, True, True)) in oracle_kernels
    assert ("backward", (False, False, True)) in oracle_kernels
    assert all(call[0] != "backward" or call[1] != (True, True, True) for call in oracle_kernels)
    ws = t["w"].clone().requires_grad_(True)
    vs = t["y"].clone().requires_grad_(True)
    ref = oracle_conv.conv_forward(meta, x, vs * 1.5, ws, src, dst, graph.num_nodes)
    (ref_force,) = torch.autograd.grad(ref.square().sum(), vs, create_graph=True)
    (ref_grad_w,) = torch.autograd.grad(ref_force.square().sum(), ws)
    torch.testing.assert_close(grad_w, ref_grad_w, atol=1e-10, rtol=1e-10)


@pytest.mark.parametrize("name", ["fixture", "mul2", "highl"])
def test_envelope_and_scalar_features(name, oracle_kernels):
    module, meta, graph, src, dst, t, rand = _problem(name)
    edges = graph.num_edges
    env = rand(edges).requires_grad_(True)
    x, y, w = (t[k].clone().requires_grad_(True) for k in ("x", "y", "w"))
    out, l0 = module(x, y, w, graph=graph, env=env, return_l0_feat=True)

    # dense restatement: per-edge messages of every path, envelope after the scalar features are taken
    xs = x[src]
    ref_out = x.new_zeros((graph.num_nodes, meta["out_dim"]))
    messages = {}
    for index, spec in enumerate(meta["specs"]):
        ch, d1, d2, d3 = spec["channels"], spec["d1"], spec["d2"], spec["d3"]
        xb = xs[:, spec["x_offset"]: spec["x_offset"] + ch * d1].reshape(-1, ch, d1)
        yb = y[:, spec["y_offset"]: spec["y_offset"] + d2]
        wb = w[:, spec["weight_offset"]: spec["weight_offset"] + (ch - 1) * spec["weight_stride"] + 1:
               spec["weight_stride"]]
        msg = torch.einsum("ijk,eui,ej,eu->euk", torch.as_tensor(spec["cg"]), xb, yb, wb)
        messages[index] = msg
        piece = (msg * env[:, None, None]).reshape(edges, ch * d3)
        ref_out = ref_out + torch.nn.functional.pad(
            x.new_zeros((graph.num_nodes, ch * d3)).index_add(0, dst, piece),
            (spec["out_offset"], meta["out_dim"] - spec["out_offset"] - ch * d3))
    # scalar features: one block per instruction into degree 0, blocks in the order of the output offsets; the specs
    # one instruction was split into (one per channel of the second input, consecutive in the list) share its block
    run_of, runs = {}, 0
    for index, spec in enumerate(meta["specs"]):
        signature = tuple(spec[k] for k in ("x_offset", "out_offset", "l1", "l2", "weight_stride"))
        previous = meta["specs"][index - 1] if index else None
        same = (previous is not None and spec["weight_stride"] > 1
                and signature == tuple(previous[k] for k in ("x_offset", "out_offset", "l1", "l2", "weight_stride"))
                and spec["weight_offset"] == previous["weight_offset"] + 1)
        if not same:
            runs += 1
        run_of[index] = runs
    columns, block_of = [], {}
    for index in sorted(range(len(meta["specs"])), key=lambda i: meta["specs"][i]["out_offset"]):
        spec = meta["specs"][index]
        if spec["l3"] != 0:
            continue
        if run_of[index] not in block_of:
            block_of[run_of[index]] = len(columns)
            columns.append(messages[index][:, :, 0])
        else:
            columns[block_of[run_of[index]]] = columns[block_of[run_of[index]]] + messages[index][:, :, 0]
    ref_l0 = torch.cat(columns, dim=1) if columns else x.new_zeros((edges, 0))
    assert l0.shape == (edges, module.op.l0_dim) == tuple(ref_l0.shape)
    torch.testing.assert_close(out, ref_out, atol=1e-12, rtol=1e-12)
    torch.testing.assert_close(l0, ref_l0, atol=1e-12, rtol=1e-12)

    seeds = (rand(*out.shape), rand(*l0.shape))
    got = torch.autograd.grad((out, l0), (x, y, w, env), seeds, allow_unused=True)
    want = torch.autograd.grad((ref_out, ref_l0), (x, y, w, env), seeds, allow_unused=True)
    for a, b in zip(got, want):
        torch.testing.assert_close(a, b, atol=1e-10, rtol=1e-10)
