"""The CPU oracles against golden vectors produced by the reference's own code, and against closed forms."""

import numpy as np
import pytest
import torch

from oracle import graph as oracle_graph
from oracle import spherical_harmonics as oracle_sh
from oracle import uvu_conv as oracle_conv


def _t(a):
    return torch.from_numpy(np.asarray(a))


@pytest.mark.parametrize("name", ["cfg1", "small", "mul2", "mixed", "highl", "fixture"])
def test_conv_oracle_matches_reference_metadata_vectors(name, reference_tables, golden_npz):
    data = golden_npz("conv_vectors.npz")
    entry = reference_tables[name]
    meta = oracle_conv.build_specs(entry["irreps_in1"], entry["irreps_in2"], entry["irreps_out"],
                                   [tuple(i) for i in entry["instructions_in"]], **entry["kwargs"])
    get = lambda key: _t(data[f"{name}.{key}"])
    result = oracle_conv.conv_derivatives(meta, get("x"), get("y"), get("w"), get("src"), get("dst"),
                                          int(data[f"{name}.num_nodes"]), get("g"), get("rx"), get("ry"), get("rw"))
    for key in ("out", "gx", "gy", "gw", "hx", "hy", "hw", "hg"):
        ref = get(key)
        err = (result[key] - ref).abs().max().item()
        assert err <= 1e-12 * max(1.0, ref.abs().max().item()), (name, key, err)


def test_conv_oracle_closed_form_dot_product():
    """Cx1o (x) 1x1o -> Cx0e is a dot product scaled by w / sqrt(3) (reference examples/basic_uvu_conv.py:35-38)."""
    torch.manual_seed(7)
    channels, nodes, edges = 32, 3, 4
    meta = oracle_conv.build_specs(f"{channels}x1o", "1x1o", f"{channels}x0e", [(0, 0, 0, "uvu", True)])
    src, dst = torch.tensor([1, 0, 0, 2]), torch.tensor([0, 1, 2, 2])
    x = torch.randn(nodes, 3 * channels, dtype=torch.float64)
    y = torch.randn(edges, 3, dtype=torch.float64)
    w = torch.randn(edges, channels, dtype=torch.float64)
    out = oracle_conv.conv_forward(meta, x, y, w, src, dst, nodes)
    messages = (x[src].reshape(edges, channels, 3) * y[:, None, :]).sum(-1) * w / 3 ** 0.5
    expected = torch.zeros(nodes, channels, dtype=torch.float64).index_add(0, dst, messages)
    torch.testing.assert_close(out, expected, atol=1e-12, rtol=1e-11)


def test_conv_oracle_chunked_variants_agree():
    torch.manual_seed(0)
    meta = oracle_conv.build_specs("4x0e+4x1o", "1x0e+1x1o", "4x0e+4x1o",
                                   [(0, 0, 0, "uvu", True), (0, 1, 1, "uvu", True), (1, 0, 1, "uvu", True),
                                    (1, 1, 0, "uvu", True)])
    n, e = 11, 50
    x = torch.randn(n, 16, dtype=torch.float64)
    y = torch.randn(e, 4, dtype=torch.float64)
    w = torch.randn(e, meta["weight_numel"], dtype=torch.float64)
    g = torch.randn(n, 16, dtype=torch.float64)
    src = torch.randint(n, (e,))
    dst = torch.sort(torch.randint(n, (e,)))[0]
    full = oracle_conv.conv_derivatives(meta, x, y, w, src, dst, n, g)
    torch.testing.assert_close(oracle_conv.conv_forward_chunked(meta, x, y, w, src, dst, n, chunk_edges=7), full["out"])
    out, gx, gy, gw = oracle_conv.conv_forward_backward_chunked(meta, x, y, w, g, src, dst, n, chunk_edges=7)
    for a, b in ((out, full["out"]), (gx, full["gx"]), (gy, full["gy"]), (gw, full["gw"])):
        torch.testing.assert_close(a, b, atol=1e-12, rtol=1e-12)


@pytest.mark.parametrize("normalize", [False, True])
@pytest.mark.parametrize("normalization", ["component", "norm", "integral"])
def test_sh_oracle_matches_reference_polynomial(normalize, normalization, golden_npz):
    data = golden_npz("sh_vectors.npz")
    tag = f"{int(normalize)}.{normalization}"
    result = oracle_sh.derivatives(tuple(range(13)), _t(data["points"]), normalize, normalization,
                                   _t(data["g"]), _t(data["rx"]))
    for key in ("out", "dx", "sx", "sg"):
        ref = _t(data[f"{key}.{tag}"])
        err = (result[key] - ref).abs().max().item()
        assert err <= 1e-11 * max(1.0, ref.abs().max().item()), (key, tag, err)


def test_sh_oracle_degree_selection(golden_npz):
    data = golden_npz("sh_vectors.npz")
    out = oracle_sh.spherical_harmonics((3, 1, 3, 0), _t(data["points"]), True, "norm")
    torch.testing.assert_close(out, _t(data["out.sel"]), atol=1e-13, rtol=1e-12)


def test_sh_oracle_component_norm_on_sphere():
    v = torch.nn.functional.normalize(torch.randn(50, 3, dtype=torch.float64), dim=-1)
    out = oracle_sh.spherical_harmonics(tuple(range(7)), v, False, "component")
    start = 0
    for l in range(7):
        block = out[:, start:start + 2 * l + 1]
        torch.testing.assert_close(block.square().sum(-1), torch.full((50,), 2.0 * l + 1, dtype=torch.float64))
        start += 2 * l + 1


@pytest.mark.parametrize("name", ["tiny", "random", "hub"])
def test_graph_oracle_matches_reference(name, golden_npz):
    data = golden_npz("graph_tables.npz")
    get = lambda key: data[f"{name}.{key}"]
    g = oracle_graph.make_graph(get("src_in"), get("dst_in"), int(get("num_nodes")))
    for key in ("src", "dst", "dst_rowptr", "src_rowptr", "edge_ids_by_dst", "node_tiers"):
        np.testing.assert_array_equal(g[key], get(key), err_msg=key)
    # order-insensitive invariants for tables whose tie-breaking is unspecified in the reference
    src = get("src")
    np.testing.assert_array_equal(np.sort(g["edge_ids_by_src"]), np.arange(src.size))
    np.testing.assert_array_equal(src[g["edge_ids_by_src"]], src[get("edge_ids_by_src")])
    for order_key, rowptr_key in (("node_order", "dst_rowptr"), ("source_node_order", "src_rowptr")):
        degree = np.diff(get(rowptr_key))
        np.testing.assert_array_equal(degree[g[order_key]], degree[get(order_key)])
    seg = g["source_segments"]
    for key in ("nodes", "begin", "end", "rowptr"):
        np.testing.assert_array_equal(seg[key], get(f"seg_{key}"), err_msg=key)
    length = get("seg_end") - get("seg_begin")
    np.testing.assert_array_equal(length[seg["order"]], length[get("seg_order")])


def test_graph_oracle_errors():
    with pytest.raises(ValueError, match="num_nodes=2.*at least 4"):
        oracle_graph.make_graph([3], [0], 2)
    with pytest.raises(ValueError, match="nonnegative"):
        oracle_graph.make_graph([-1], [0], 2)
    with pytest.raises(ValueError, match="sorted"):
        oracle_graph.make_graph([0, 0], [1, 0], 2)
