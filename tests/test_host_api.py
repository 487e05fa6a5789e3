"""CPU-only checks: the C-ABI library loads and exports every declared symbol, host-side validation, graph tables
on CPU tensors (the reference's known-answer tests, tests/lunatp/test_make_graph.py:9-55), module surface."""

import os
import re

import pytest
import torch

import lunaequivariance_b200 as luna
from lunaequivariance_b200 import _native

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "luna_b200.h")).read()
    declared = set(re.findall(r"LUNA_API [\w\s\*]+?\b(luna_\w+)\(", header))
    assert declared and declared == set(_native.EXPORTED_SYMBOLS)
    lib = _native.library()
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.luna_compiled_sm() == 100


def test_plan_creation_and_errors_without_gpu():
    op = luna.prepare_tensor_product("32x0e+32x1o", "1x0e+1x1o", "32x0e+32x1o",
                                     [(0, 0, 0, "uvu", True), (1, 1, 0, "uvu", True), (0, 1, 1, "uvu", True),
                                      (1, 0, 1, "uvu", True)], convolution=True)
    assert op.weight_numel == 128 and op.out_dim == 128 and op.uses_staged_kernels
    odd = luna.prepare_tensor_product("33x0e", "1x0e", "33x0e", [(0, 0, 0, "uvu", True)], convolution=True)
    assert not odd.uses_staged_kernels
    bad = dict(op.meta)
    bad["generated_specs"] = [dict(op.meta["generated_specs"][0], x_offset=10_000)]
    with pytest.raises(ValueError, match="outside its tensor dimension"):
        luna.TensorProductConv(bad, mode="uvu")
    with pytest.raises(ValueError, match="float32 or torch.float64"):
        luna.create_uvu_conv_operator(op.meta, dtype=torch.float16)
    with pytest.raises(ValueError, match='mode="uuu" or mode="uvu"'):
        luna.TensorProductConv(op.meta)
    with pytest.raises(TypeError):
        luna.TensorProductConv("32x0e")
    with pytest.raises(ValueError, match="one connection mode"):
        luna.TensorProductConv("2x0e", "2x0e", "2x0e", [(0, 0, 0, "uvu", True), (0, 0, 0, "uuu", True)],
                               internal_weights=False, shared_weights=False)
    with pytest.raises(ValueError, match="internal_weights=False"):
        luna.TensorProductConv("2x0e", "1x0e", "2x0e", [(0, 0, 0, "uvu", True)])


def test_module_surface():
    conv = luna.TensorProductConv("4x0e+4x1o", "1x0e+1x1o", "4x0e+4x1o",
                                  [(0, 0, 0, "uvu", True), (1, 1, 0, "uvu", True)],
                                  internal_weights=False, shared_weights=False)
    assert conv.mode == "uvu_conv" and conv.weight_numel == 8
    assert str(conv.irreps_in1) == "4x0e+4x1o" and len(conv.instructions) == 2
    assert conv.internal_weights is False and conv.shared_weights is False
    assert conv.op.compute_dtype == torch.float32
    assert conv.double().op.compute_dtype == torch.float64
    meta_conv = luna.TensorProductConv(conv.op.meta, mode="uvu", dtype=torch.float64)
    assert meta_conv.weight_numel == 8
    import pickle

    restored = pickle.loads(pickle.dumps(conv.op))
    assert restored.weight_numel == 8 and restored.compute_dtype == torch.float64


def test_destination_sorted_endpoints_are_preserved():
    src, dst = torch.tensor([2, 0, 1]), torch.tensor([0, 1, 2])
    graph = luna.make_graph(src, dst, 4)
    assert torch.equal(graph.dst, dst.to(graph.dst.dtype)) and torch.equal(graph.src, src.to(graph.src.dtype))
    assert graph.dst_rowptr.tolist() == [0, 1, 2, 3, 3]


def test_invalid_graph_includes_values():
    with pytest.raises(ValueError, match="num_nodes=2.*at least 4"):
        luna.make_graph(torch.tensor([3]), torch.tensor([0]), 2)
    with pytest.raises(ValueError, match="nonnegative"):
        luna.make_graph(torch.tensor([-1]), torch.tensor([0]), 2)
    with pytest.raises(TypeError):
        luna.make_graph(torch.tensor([0.0]), torch.tensor([0.0]), 2)
    with pytest.raises(ValueError, match="equal shape"):
        luna.make_graph(torch.tensor([0, 1]), torch.tensor([0]), 2)


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_generated_graph_tables_and_input_ownership(dtype):
    src = torch.tensor([2, 0, 1, 0], dtype=dtype)
    dst = torch.tensor([0, 1, 1, 2], dtype=dtype)
    graph = luna.make_graph(src, dst, 4)
    assert graph.src_rowptr.tolist() == [0, 2, 3, 4, 4]
    assert graph.dst_rowptr.tolist() == [0, 1, 3, 4, 4]
    assert graph.edge_ids_by_src.sort().values.tolist() == [0, 1, 2, 3]
    assert graph.src[graph.edge_ids_by_src.long()].tolist() == [0, 0, 1, 2]
    assert graph.edge_ids_by_dst.tolist() == [0, 1, 2, 3]
    for rowptr, order in ((graph.dst_rowptr, graph.node_order), (graph.src_rowptr, graph.source_node_order)):
        assert order.sort().values.tolist() == [0, 1, 2, 3]
        assert rowptr.diff()[order.long()].tolist() == [2, 1, 1, 0]
    assert graph.src.data_ptr() != src.data_ptr() and graph.dst.data_ptr() != dst.data_ptr()
    src.zero_()
    dst.zero_()
    assert graph.src.tolist() == [2, 0, 1, 0] and graph.dst.tolist() == [0, 1, 1, 2]
    assert len(graph.table_list()) == 13


def test_spherical_harmonics_argument_handling():
    from lunaequivariance_b200.spherical_harmonics import parse_irreps

    irreps_in, out, degrees = parse_irreps("1x0e+1x1o+1x2e")
    assert str(irreps_in) == "1x1o" and degrees == (0, 1, 2) and out.dim == 9
    assert parse_irreps([3, 1, 3, 0])[2] == (3, 1, 3, 0)
    assert str(parse_irreps("1x1e")[0]) == "1x1e"
    with pytest.raises(ValueError, match="parity"):
        parse_irreps("1x1e", "1o")
    with pytest.raises(NotImplementedError):
        parse_irreps(13)
    with pytest.raises(TypeError):
        luna.SphericalHarmonics("1x0e")
    with pytest.raises(ValueError):
        luna.SphericalHarmonics("1x0e", normalize=True, normalization="bogus")


def test_custom_op_fake_shapes():
    """The shape functions registered for torch.compile run on meta tensors without any kernel."""
    op = luna.prepare_tensor_product("4x0e+4x1o", "1x0e+1x1o", "4x0e+4x1o",
                                     [(0, 0, 0, "uvu", True), (1, 1, 0, "uvu", True)], convolution=True)
    x = torch.empty(5, 16, device="meta")
    y = torch.empty(9, 4, device="meta")
    w = torch.empty(9, 8, device="meta")
    tables = [torch.empty(9, dtype=torch.int32, device="meta")] * 13
    out, l0 = torch.ops.lunatp.uvu_conv_forward(x, y, w, None, tables, 5, False, op.torch_config)
    assert out.shape == (5, 16) and l0 is None
    grads = torch.ops.lunatp.uvu_conv_backward(x, y, w, None, out, None, tables, 5, [True, False, True, False],
                                               op.torch_config)
    assert grads[0].shape == x.shape and grads[1] is None and grads[2].shape == w.shape
    v = torch.empty(7, 3, device="meta")
    from lunaequivariance_b200.spherical_harmonics import SphericalHarmonicsConfig

    desc = SphericalHarmonicsConfig((0, 1, 2), True, "component", torch.float32).descriptor()
    assert torch.ops.lunaeq.spherical_harmonics_forward(v, desc).shape == (7, 9)


def test_canonical_path_lists_are_detected_without_gpu():
    """Full lists of allowed couplings select the kernels unrolled at compile time; anything else does not."""
    from tests.helpers import config

    expected = {"cfg2": 3, "cfg4": 3, "cfg5": 2, "fixture": 1, "wide": 1, "cfg1": -1, "partial": -1}
    for name, l2 in expected.items():
        in1, in2, out, instructions, options = config(name)
        op = luna.prepare_tensor_product(in1, in2, out, instructions, convolution=True, **options)
        assert op.uses_staged_kernels, name
        assert op.canonical_l2 == l2, (name, op.canonical_l2)
        assert op.uses_compiled_patterns == (l2 >= 0), name
    # the same couplings in another order are not canonical (weight blocks follow the instruction order)
    in1, in2, out, instructions, options = config("fixture")
    shuffled = luna.prepare_tensor_product(in1, in2, out, instructions[::-1], convolution=True)
    assert shuffled.uses_staged_kernels and shuffled.canonical_l2 == -1
