"""Parity of the CUDA spherical harmonics and graph builder with golden vectors and the CPU oracles."""

import numpy as np
import pytest
import torch

import lunaequivariance_b200 as luna
from oracle import graph as oracle_graph
from oracle import spherical_harmonics as oracle_sh
from tests.helpers import assert_close

pytestmark = pytest.mark.gpu
DEVICE = "cuda"


@pytest.mark.parametrize("normalize", [False, True])
@pytest.mark.parametrize("normalization", ["component", "norm", "integral"])
def test_sh_matches_reference_vectors_fp64(normalize, normalization, golden_npz):
    data = golden_npz("sh_vectors.npz")
    tag = f"{int(normalize)}.{normalization}"
    v = torch.from_numpy(data["points"]).to(DEVICE).requires_grad_(True)
    g = torch.from_numpy(data["g"]).to(DEVICE).requires_grad_(True)
    rx = torch.from_numpy(data["rx"]).to(DEVICE)
    out = luna.spherical_harmonics(tuple(range(13)), v, normalize, normalization)
    (dx,) = torch.autograd.grad(out, v, g, create_graph=True)
    sx, sg = torch.autograd.grad(dx, (v, g), rx)
    for key, value in dict(out=out, dx=dx, sx=sx, sg=sg).items():
        ref = torch.from_numpy(data[f"{key}.{tag}"])
        # values of degree 12 reach 1e6 for unnormalised inputs; the bound is relative to the largest magnitude
        assert_close(value, ref, torch.float64, f"sh {key} {tag}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("normalize,normalization", [(True, "component"), (False, "integral"), (True, "norm")])
@pytest.mark.parametrize("lmax", [1, 2, 3, 4, 5, 6, 7])
def test_sh_degrees_zero_to_lmax_match_oracle(lmax, normalize, normalization, dtype):
    """Degree lists 0..lmax: up to lmax 6 these take the kernels unrolled per lmax, 7 the run-time recurrence."""
    generator = torch.Generator().manual_seed(lmax)
    v = torch.randn(1000, 3, generator=generator, dtype=torch.float64)
    v = torch.nn.functional.normalize(v, dim=-1) * (1.0 if normalize else 0.7)
    C = (lmax + 1) ** 2
    g = torch.randn(1000, C, generator=generator, dtype=torch.float64)
    rx = torch.randn(1000, 3, generator=generator, dtype=torch.float64)
    ref = oracle_sh.derivatives(tuple(range(lmax + 1)), v, normalize, normalization, g, rx)
    module = luna.o3.SphericalHarmonics(luna.Irreps.spherical_harmonics(lmax), normalize=normalize,
                                        normalization=normalization)
    vd = v.to(DEVICE, dtype).requires_grad_(True)
    gd = g.to(DEVICE, dtype).requires_grad_(True)
    out = module(vd)
    (dx,) = torch.autograd.grad(out, vd, gd, create_graph=True)
    sx, sg = torch.autograd.grad(dx, (vd, gd), rx.to(DEVICE, dtype))
    for key, value in dict(out=out, dx=dx, sx=sx, sg=sg).items():
        assert_close(value, ref[key], dtype, f"sh lmax {lmax} {key}")


def test_sh_degree_selection_and_shapes(golden_npz):
    data = golden_npz("sh_vectors.npz")
    v = torch.from_numpy(data["points"]).to(DEVICE)
    out = luna.spherical_harmonics([3, 1, 3, 0], v, True, "norm")
    assert_close(out, torch.from_numpy(data["out.sel"]), torch.float64, "degree selection")
    batched = luna.spherical_harmonics(2, v.reshape(4, 6, 3), False, "integral")
    assert batched.shape == (4, 6, 5)
    with pytest.raises(NotImplementedError):
        luna.spherical_harmonics(13, v, True)
    with pytest.raises(RuntimeError):
        luna.spherical_harmonics(2, v.cpu(), True)


@pytest.mark.parametrize("name", ["tiny", "random", "hub"])
@pytest.mark.parametrize("index_dtype", [torch.int32, torch.int64])
def test_graph_tables_match_reference(name, index_dtype, golden_npz):
    data = golden_npz("graph_tables.npz")
    get = lambda key: data[f"{name}.{key}"]
    src = torch.from_numpy(get("src_in")).to(DEVICE, index_dtype)
    dst = torch.from_numpy(get("dst_in")).to(DEVICE, index_dtype)
    graph = luna.make_graph(src, dst, int(get("num_nodes")))
    for key in ("src", "dst", "dst_rowptr", "src_rowptr", "edge_ids_by_dst", "node_tiers"):
        np.testing.assert_array_equal(getattr(graph, key).cpu().numpy(), get(key), err_msg=key)
    host_src = get("src")
    by_src = graph.edge_ids_by_src.cpu().numpy()
    np.testing.assert_array_equal(np.sort(by_src), np.arange(host_src.size))
    np.testing.assert_array_equal(host_src[by_src], host_src[get("edge_ids_by_src")])
    stable = oracle_graph.make_graph(get("src_in"), get("dst_in"), int(get("num_nodes")))
    np.testing.assert_array_equal(by_src, stable["edge_ids_by_src"])
    np.testing.assert_array_equal(graph.node_order.cpu().numpy(), stable["node_order"])
    np.testing.assert_array_equal(graph.source_node_order.cpu().numpy(), stable["source_node_order"])
    seg = graph.source_segments
    for key in ("nodes", "begin", "end", "rowptr"):
        np.testing.assert_array_equal(getattr(seg, key).cpu().numpy(), get(f"seg_{key}"), err_msg=key)
    assert graph.src.data_ptr() != src.data_ptr()


def test_graph_errors_on_device():
    t = lambda v: torch.tensor(v, device=DEVICE)
    with pytest.raises(ValueError, match="num_nodes=2.*at least 4"):
        luna.make_graph(t([3]), t([0]), 2)
    with pytest.raises(ValueError, match="nonnegative"):
        luna.make_graph(t([-1]), t([0]), 2)
    with pytest.raises(ValueError, match="sorted"):
        luna.make_graph(t([0, 0]), t([1, 0]), 2)
    graph = luna.make_graph(t([2, 0, 1]), t([0, 1, 2]))
    assert graph.num_nodes == 3 and graph.dst_rowptr.tolist() == [0, 1, 2, 3]
