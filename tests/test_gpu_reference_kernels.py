"""GPU-to-GPU parity with the reference's own kernels.

``oracle/build_ref.py`` lets the reference generate and compile its CUDA extensions (forward and first-order
backward) for sm_100; the libraries travel with the repository under ``oracle/_ref``.  Here this library and the
reference's kernels run on identical seeded inputs on the same GPU.  Second-order outputs are checked against the
reference's first-order kernels applied to tangent operands, which is what they are by multilinearity of the form
``F(x, y, w, g)`` (``src/lunatp/utils/contractions.py:41-49``): ``hg = F_g(rx,y,w) + F_g(x,ry,w) + F_g(x,y,rw)`` etc.

Tolerance: 1e-5 (FP32) / 1e-12 (FP64) of each tensor's largest magnitude.  The reference's FP32 kernels are built with
``--use_fast_math`` and its forward adds colliding paths with atomics, so FP32 agreement is to rounding, not bitwise.
"""

import pytest
import torch

import bench_workloads as workloads
import lunaequivariance_b200 as luna
from lunaequivariance_b200 import conv as conv_mod
from oracle import ref_kernels
from tests.helpers import assert_close, config, random_graph, random_problem

pytestmark = pytest.mark.gpu
DEVICE = "cuda"

CASES = [("fixture", torch.float32), ("fixture", torch.float64), ("cfg1", torch.float64), ("cfg2", torch.float32),
         ("cfg2", torch.float64), ("cfg5", torch.float32)]


def _key(name, dtype):
    return f"{name}.{str(dtype).removeprefix('torch.')}"


def _setup(name, dtype, nodes, edges, exact_degree=None, seed=3, force_wide=False):
    if not ref_kernels.available(_key(name, dtype)):
        pytest.skip("oracle/_ref holds no build of the reference's kernels for this configuration")
    in1, in2, out, instructions, options = config(name)
    module = luna.TensorProductConv(in1, in2, out, instructions, internal_weights=False, shared_weights=False,
                                    dtype=dtype, **options)
    reference = ref_kernels.ReferenceKernels(_key(name, dtype), force_wide=force_wide)
    op = module.op
    assert (op.in1_dim, op.in2_dim, op.out_dim, op.weight_numel) == tuple(
        reference.entry[k] for k in ("in1_dim", "in2_dim", "out_dim", "weight_numel"))
    generator = torch.Generator().manual_seed(seed)
    src, dst = random_graph(nodes, edges, generator, exact_degree)
    p = random_problem((op.in1_dim, op.in2_dim, op.out_dim, op.weight_numel), nodes, src, dtype, generator)
    graph = module.create_graph(src.to(DEVICE), dst.to(DEVICE), nodes)
    return module, reference, graph, {k: v.to(DEVICE) for k, v in p.items()}


def _compare(name, dtype, module, reference, graph, p):
    op = module.op
    x, y, w, g, rx, ry, rw = (p[k] for k in ("x", "y", "w", "g", "rx", "ry", "rw"))
    out = conv_mod.run_forward(op, x, y, w, graph)
    assert_close(out, reference.forward(x, y, w, graph).cpu(), dtype, f"{name} out vs reference kernel")
    gx, gy, gw = conv_mod.run_backward(op, x, y, w, g, graph)
    rgx, rgy, rgw = reference.backward(x, y, w, g, graph)
    for what, mine, theirs in (("gx", gx, rgx), ("gy", gy, rgy), ("gw", gw, rgw)):
        assert_close(mine, theirs.cpu(), dtype, f"{name} {what} vs reference kernel")
    hx, hy, hw, hg = conv_mod.run_double_backward(op, x, y, w, g, rx, ry, rw, graph)
    ref_hg = reference.forward(rx, y, w, graph) + reference.forward(x, ry, w, graph) + reference.forward(x, y, rw, graph)
    a = reference.backward(rx, y, w, g, graph)   # F_y(rx, w, g), F_w(rx, y, g)
    b = reference.backward(x, ry, w, g, graph)   # F_x(ry, w, g), F_w(x, ry, g)
    c = reference.backward(x, y, rw, g, graph)   # F_x(y, rw, g), F_y(x, rw, g)
    for what, mine, theirs in (("hg", hg, ref_hg), ("hx", hx, b[0] + c[0]), ("hy", hy, a[1] + c[1]),
                               ("hw", hw, a[2] + b[2])):
        assert_close(mine, theirs.cpu(), dtype, f"{name} {what} vs reference kernels on tangents")
    op.check_status()


@pytest.mark.parametrize("name,dtype", CASES)
def test_small_random_graph_matches_reference_kernels(name, dtype):
    module, reference, graph, p = _setup(name, dtype, nodes=41, edges=333)
    _compare(name, dtype, module, reference, graph, p)


@pytest.mark.parametrize("name,dtype", [("fixture", torch.float32), ("cfg2", torch.float32), ("cfg2", torch.float64)])
def test_wide_index_variant_of_reference_kernels(name, dtype):
    """The reference switches to 64-bit offsets on large graphs (cfg2 beyond 932,067 edges); the same variant, forced
    on a small graph, must agree as well."""
    module, reference, graph, p = _setup(name, dtype, nodes=41, edges=333, force_wide=True)
    _compare(name, dtype, module, reference, graph, p)


def test_config1_full_size_matches_reference_kernels():
    module, reference, graph, p = _setup("cfg1", torch.float64, nodes=1000, edges=None, exact_degree=16)
    _compare("cfg1", torch.float64, module, reference, graph, p)


@pytest.mark.parametrize("name,dtype,atoms", [("cfg2", torch.float32, 2000), ("cfg2", torch.float64, 1000),
                                               ("cfg5", torch.float32, 4000)])
def test_radius_graph_matches_reference_kernels(name, dtype, atoms):
    """A small periodic radius graph of the benchmark's kind (about 52 neighbours per atom)."""
    if not ref_kernels.available(_key(name, dtype)):
        pytest.skip("oracle/_ref holds no build of the reference's kernels for this configuration")
    in1, in2, out, instructions, options = config(name)
    module = luna.TensorProductConv(in1, in2, out, instructions, internal_weights=False, shared_weights=False,
                                    dtype=dtype)
    reference = ref_kernels.ReferenceKernels(_key(name, dtype))
    pos, box, cells = workloads.periodic_positions(atoms, workloads.DENSITY, 0, DEVICE, workloads.CUTOFF)
    src, dst, vec = workloads.radius_graph_periodic(pos, box, workloads.CUTOFF, cells)
    graph = module.create_graph(src, dst, atoms)
    op = module.op
    lmax = {"cfg2": 3, "cfg5": 2}[name]
    y = luna.spherical_harmonics(list(range(lmax + 1)), vec.to(dtype), True, "component").contiguous()
    generator = torch.Generator(device=DEVICE).manual_seed(9)
    rand = lambda *shape: torch.randn(*shape, device=DEVICE, dtype=dtype, generator=generator)
    edges = graph.num_edges
    p = dict(x=rand(atoms, op.in1_dim), y=y, w=rand(edges, op.weight_numel), g=rand(atoms, op.out_dim),
             rx=rand(atoms, op.in1_dim), ry=rand(edges, op.in2_dim), rw=rand(edges, op.weight_numel))
    _compare(name, dtype, module, reference, graph, p)


@pytest.mark.parametrize("dtype,atoms,tol", [(torch.float32, 50_000, 1e-5), (torch.float64, 20_000, 1e-12)])
def test_config2_at_full_size_matches_reference_kernels_everywhere(dtype, atoms, tol):
    """BASELINE configurations 2 (FP32, 50,000 atoms, 2.6 M edges) and 3's convolution (FP64, 20,000 atoms, 1.0 M
    edges) at their sizes: every element of out, gx, gy and gw against the reference's own kernels on the same GPU
    (its 64-bit index variant at these sizes)."""
    name = "cfg2"
    if not ref_kernels.available(_key(name, dtype)):
        pytest.skip("oracle/_ref holds no build of the reference's kernels for this configuration")
    in1, in2, out, instructions, _ = config(name)
    module = luna.TensorProductConv(in1, in2, out, instructions, internal_weights=False, shared_weights=False,
                                    dtype=dtype)
    reference = ref_kernels.ReferenceKernels(_key(name, dtype))
    pos, box, cells = workloads.periodic_positions(atoms, workloads.DENSITY, 0, DEVICE, workloads.CUTOFF)
    src, dst, vec = workloads.radius_graph_periodic(pos, box, workloads.CUTOFF, cells)
    graph = module.create_graph(src, dst, atoms)
    op = module.op
    y = luna.spherical_harmonics([0, 1, 2, 3], vec.to(dtype), True, "component").contiguous()
    generator = torch.Generator(device=DEVICE).manual_seed(31)
    rand = lambda *shape: torch.randn(*shape, device=DEVICE, dtype=dtype, generator=generator)
    x, w, g = rand(atoms, op.in1_dim), rand(graph.num_edges, op.weight_numel), rand(atoms, op.out_dim)

    def worst(mine, theirs):  # on the device: the tensors are GBs
        scale = theirs.abs().max().clamp_min(1e-30)
        return float((mine - theirs).abs().max() / scale)

    errors = {"out": worst(conv_mod.run_forward(op, x, y, w, graph), reference.forward(x, y, w, graph))}
    mine, theirs = conv_mod.run_backward(op, x, y, w, g, graph), reference.backward(x, y, w, g, graph)
    for what, a, b in zip(("gx", "gy", "gw"), mine, theirs):
        errors[what] = worst(a, b)
    del mine, theirs
    torch.cuda.empty_cache()
    op.check_status()
    assert graph.num_edges > 1_000_000
    assert all(e <= tol for e in errors.values()), errors
