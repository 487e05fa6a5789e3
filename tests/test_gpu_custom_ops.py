"""The ``torch.library`` custom-op path on a GPU: direct op calls, ``torch.compile`` and ``make_fx``.

The reference checks its operators under ``torch.compile(fullgraph=True, dynamic=True)`` against eager execution
(``tests/testing_utils.py:54-79``) and traces higher-order gradients with ``make_fx``
(``tests/lunatp/test_uvu_conv.py:1221-1269``).  Same here: the compiled and the traced programs must contain the
``lunatp`` / ``lunaeq`` ops and reproduce the eager chain's output, first and second derivatives.
"""

import pytest
import torch

import lunaequivariance_b200 as luna
from oracle import uvu_conv as oracle_conv
from tests.helpers import assert_close, config, random_graph, random_problem

pytestmark = pytest.mark.gpu
DEVICE = "cuda"


def _problem(name, dtype, nodes=23, edges=160, seed=2):
    in1, in2, out, instructions, options = config(name)
    module = luna.TensorProductConv(in1, in2, out, instructions, internal_weights=False, shared_weights=False,
                                    dtype=dtype, **options)
    meta = oracle_conv.build_specs(in1, in2, out, instructions, **options)
    generator = torch.Generator().manual_seed(seed)
    src, dst = random_graph(nodes, edges, generator)
    p = random_problem((meta["in1_dim"], meta["in2_dim"], meta["out_dim"], meta["weight_numel"]), nodes, src, dtype,
                       generator)
    graph = module.create_graph(src.to(DEVICE), dst.to(DEVICE), nodes)
    ref = oracle_conv.conv_derivatives(meta, *(p[k].double() for k in ("x", "y", "w")), src, dst, nodes,
                                       p["g"].double(), *(p[k].double() for k in ("rx", "ry", "rw")))
    return module, graph, {k: v.to(DEVICE) for k, v in p.items()}, ref


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
@pytest.mark.parametrize("name", ["fixture", "cfg5", "mul2"])
def test_custom_ops_differentiate_twice(name, dtype):
    """``torch.ops.lunatp.uvu_conv_forward`` with the graph's table list, differentiated twice through the
    registered autograd chain, against the oracle."""
    module, graph, p, ref = _problem(name, dtype)
    x, y, w, g = (p[k].clone().requires_grad_(True) for k in ("x", "y", "w", "g"))
    out, l0 = torch.ops.lunatp.uvu_conv_forward(x, y, w, None, graph.table_list(), graph.num_nodes, False,
                                                module.op.torch_config)
    assert l0 is None
    assert_close(out, ref["out"], dtype, f"{name} op out")
    gx, gy, gw = torch.autograd.grad(out, (x, y, w), g, create_graph=True)
    for key, value in (("gx", gx), ("gy", gy), ("gw", gw)):
        assert_close(value, ref[key], dtype, f"{name} op {key}")
    hx, hy, hw, hg = torch.autograd.grad((gx, gy, gw), (x, y, w, g), (p["rx"], p["ry"], p["rw"]))
    for key, value in (("hx", hx), ("hy", hy), ("hw", hw), ("hg", hg)):
        assert_close(value, ref[key], dtype, f"{name} op {key}")


def test_opcheck_forward_op():
    module, graph, p, _ = _problem("one", torch.float64, nodes=5, edges=9)
    args = (p["x"].requires_grad_(True), p["y"].requires_grad_(True), p["w"].requires_grad_(True), None,
            graph.table_list(), graph.num_nodes, False, module.op.torch_config)
    torch.library.opcheck(torch.ops.lunatp.uvu_conv_forward.default, args,
                          test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_compiled_modules_match_eager(dtype):
    """Both modules under ``torch.compile(fullgraph=True, dynamic=True)``: outputs and first gradients."""
    module, graph, p, ref = _problem("fixture", dtype)
    harmonics = luna.SphericalHarmonics("1x0e+1x1o", True, "component", dtype=dtype)
    torch._dynamo.reset()
    compiled_conv = torch.compile(module, fullgraph=True, dynamic=True, options={"triton.cudagraphs": False})
    compiled_sh = torch.compile(harmonics, fullgraph=True, dynamic=True, options={"triton.cudagraphs": False})
    vec = torch.randn(graph.num_edges, 3, device=DEVICE, dtype=dtype)

    def run(conv, sh):
        x, w = p["x"].clone().requires_grad_(True), p["w"].clone().requires_grad_(True)
        v = vec.clone().requires_grad_(True)
        out = conv(x, sh(v), w, graph=graph)
        return (out, *torch.autograd.grad(out, (x, v, w), p["g"]))

    eager = run(module, harmonics)
    compiled = run(compiled_conv, compiled_sh)
    for what, a, b in zip(("out", "gx", "gvec", "gw"), compiled, eager):
        assert_close(a, b.detach().cpu(), dtype, f"compiled {what}")


def test_make_fx_trace_holds_the_ops():
    from torch.fx.experimental.proxy_tensor import make_fx

    dtype = torch.float64
    module, graph, p, ref = _problem("fixture", dtype)

    def first_and_second(x, y, w, g, ry):
        out = module(x, y, w, graph=graph)
        gx, gy, gw = torch.autograd.grad(out, (x, y, w), g, create_graph=True)
        (hw,) = torch.autograd.grad(gy, w, ry)
        return out, gx, gy, gw, hw

    args = tuple(p[k].clone().requires_grad_(k in ("x", "y", "w", "g")) for k in ("x", "y", "w", "g", "ry"))
    traced = make_fx(first_and_second)(*args)
    targets = {str(node.target) for node in traced.graph.nodes if node.op == "call_function"}
    assert any("lunatp.uvu_conv_forward" in t for t in targets), targets
    assert any("lunatp.uvu_conv_backward" in t for t in targets), targets
    assert any("lunatp.uvu_conv_double_backward" in t for t in targets), targets
    out, gx, gy, gw, hw = traced(*args)
    eager = first_and_second(*args)
    for what, a, b in zip(("out", "gx", "gy", "gw", "hw"), (out, gx, gy, gw, hw), eager):
        assert_close(a, b.detach().cpu(), dtype, f"traced {what}")
    assert_close(out, ref["out"], dtype, "traced out vs oracle")
    assert_close(gy, ref["gy"], dtype, "traced gy vs oracle")


def test_spherical_harmonics_fragment_op():
    """``lunaeq::spherical_harmonics(Tensor x, int[] degrees, bool normalize, str normalization)``."""
    x = torch.randn(50, 3, device=DEVICE, dtype=torch.float64, requires_grad=True)
    direct = luna.spherical_harmonics([0, 1, 2, 3], x, True, "component")
    through_op = torch.ops.lunaeq.spherical_harmonics(x, [0, 1, 2, 3], True, "component")
    torch.testing.assert_close(through_op, direct)
    (a,) = torch.autograd.grad(through_op.square().sum(), x, create_graph=True)
    (b,) = torch.autograd.grad(direct.square().sum(), x, create_graph=True)
    torch.testing.assert_close(a, b)
