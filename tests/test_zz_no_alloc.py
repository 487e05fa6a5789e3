"""The allocation-free backward entry point (``luna_uvu_conv_bwd_noalloc``) against the regular one.

Some embedders of the library cannot give the backward pass a scratch buffer because they cannot allocate device
memory at the point where they call it (a plugin inside another program's step, a loop that must avoid
``cudaMalloc``'s device-wide synchronisation, a process with a closed memory pool).  For them the library carries
an 8 MiB array of its own.  These tests call that entry point through the C-ABI on a configuration whose backward
pass really uses scratch (128 channels in FP64 are split over two warps), twice in a row because the array is
shared between calls and keeps the previous call's contents, and compare with ``luna_uvu_conv_bwd``.  This file
is collected last so that a run that stops at the first failure has already run everything else.
"""

import ctypes

import pytest
import torch

import lunaequivariance_b200 as luna
from lunaequivariance_b200 import _native
from lunaequivariance_b200 import conv as conv_mod
from tests.helpers import assert_close, config, random_graph, random_problem

pytestmark = pytest.mark.gpu
DEVICE = "cuda"


def make_conv(name, dtype):
    in1, in2, out, instructions, options = config(name)
    return luna.TensorProductConv(in1, in2, out, instructions, internal_weights=False, shared_weights=False,
                                  dtype=dtype, **options)


def problem(conv, nodes, edges, dtype, seed):
    generator = torch.Generator().manual_seed(seed)
    src, dst = random_graph(nodes, edges, generator)
    op = conv.op
    p = random_problem((op.in1_dim, op.in2_dim, op.out_dim, op.weight_numel), nodes, src, dtype, generator)
    graph = conv.create_graph(src.to(DEVICE), dst.to(DEVICE), nodes)
    return graph, tuple(p[k].to(DEVICE).contiguous() for k in ("x", "y", "w", "g"))


def call_noalloc(op, graph, x, y, w, g):
    gx, gy, gw = torch.empty_like(x), torch.empty_like(y), torch.empty_like(w)
    with torch.cuda.device(x.device):
        status = _native.library().luna_uvu_conv_bwd_noalloc(
            op._plan.handle, ctypes.byref(graph.native()), x.data_ptr(), y.data_ptr(), w.data_ptr(), g.data_ptr(),
            gx.data_ptr(), gy.data_ptr(), gw.data_ptr(), _native.current_stream(x.device))
    return status, (gx, gy, gw)


def test_noalloc_backward_matches_regular_entry_point_twice():
    dtype = torch.float64
    conv = make_conv("cfg2", dtype)
    op = conv.op
    assert op.uses_staged_kernels
    lib = _native.library()
    limit = lib.luna_uvu_conv_noalloc_max_scratch_bytes()
    assert limit == 8 << 20
    with torch.cuda.device(DEVICE):
        _native.check(lib.luna_uvu_conv_noalloc_prepare(op._plan.handle))  # set-up: the one step that may allocate
    # two different graphs back to back: the second call finds the first call's partial rows in the array
    for seed, (nodes, edges) in enumerate(((41, 333), (57, 1201))):
        graph, (x, y, w, g) = problem(conv, nodes, edges, dtype, seed)
        need = lib.luna_uvu_conv_scratch_bytes(op._plan.handle, nodes, edges)
        assert 0 < need <= limit, "the case must exercise the scratch path"
        want = conv_mod.run_backward(op, x, y, w, g, graph)  # regular entry point, torch-allocated scratch
        gx, gy, gw = torch.empty_like(x), torch.empty_like(y), torch.empty_like(w)  # outputs exist before the call
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        with torch.cuda.device(x.device):
            status = lib.luna_uvu_conv_bwd_noalloc(
                op._plan.handle, ctypes.byref(graph.native()), x.data_ptr(), y.data_ptr(), w.data_ptr(),
                g.data_ptr(), gx.data_ptr(), gy.data_ptr(), gw.data_ptr(), _native.current_stream(x.device))
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
        _native.check(status)
        got = (gx, gy, gw)
        for name, a, b in zip(("gx", "gy", "gw"), got, want):
            assert_close(a, b.detach().cpu(), dtype, f"noalloc {name} (call {seed + 1})")
    _native.check(lib.luna_uvu_check_status(op._plan.handle, None))


def test_noalloc_refuses_instead_of_allocating():
    dtype = torch.float32
    conv = make_conv("wide", dtype)  # 256 channels in FP32: two chunks, 32 bytes of scratch per edge
    op = conv.op
    lib = _native.library()
    nodes, edges = 4096, 270_000  # needs 8.64 MB > 8 MiB
    # correctly sized operands, so that even a missed refusal would stay inside its buffers
    generator = torch.Generator().manual_seed(7)
    src, dst = random_graph(nodes, edges, generator)
    graph = conv.create_graph(src.to(DEVICE), dst.to(DEVICE), nodes)
    x, y, w, g = (torch.randn(rows, cols, device=DEVICE, dtype=dtype) for rows, cols in (
        (nodes, op.in1_dim), (edges, op.in2_dim), (edges, op.weight_numel), (nodes, op.out_dim)))
    assert lib.luna_uvu_conv_scratch_bytes(op._plan.handle, nodes, edges) > lib.luna_uvu_conv_noalloc_max_scratch_bytes()
    status, _ = call_noalloc(op, graph, x, y, w, g)
    assert status == _native.LUNA_ERR_SCRATCH
    assert "8388608" in _native.last_error()
    # without the edge-attribute gradient no scratch is used, so the same large graph is accepted
    with torch.cuda.device(DEVICE):
        _native.check(lib.luna_uvu_conv_noalloc_prepare(op._plan.handle))
    want_x, _, want_w = conv_mod.run_backward(op, x, y, w, g, graph, needs=(True, False, True))
    gx, gw = torch.empty_like(x), torch.empty_like(w)
    with torch.cuda.device(x.device):
        _native.check(lib.luna_uvu_conv_bwd_noalloc(
            op._plan.handle, ctypes.byref(graph.native()), x.data_ptr(), y.data_ptr(), w.data_ptr(), g.data_ptr(),
            gx.data_ptr(), None, gw.data_ptr(), _native.current_stream(x.device)))
    torch.cuda.synchronize()
    assert_close(gx, want_x.cpu(), dtype, "noalloc gx without gy")
    assert_close(gw, want_w.cpu(), dtype, "noalloc gw without gy")

    fresh = make_conv("wide", dtype)  # its tables have never been uploaded to this device
    small_graph, (x, y, w, g) = problem(fresh, 33, 200, dtype, 8)
    status, _ = call_noalloc(fresh.op, small_graph, x, y, w, g)
    assert status == _native.LUNA_ERR_INVALID_ARGUMENT
    assert "luna_uvu_conv_noalloc_prepare" in _native.last_error()
    with torch.cuda.device(DEVICE):
        _native.check(lib.luna_uvu_conv_noalloc_prepare(fresh.op._plan.handle))
    want = conv_mod.run_backward(fresh.op, x, y, w, g, small_graph)
    status, got = call_noalloc(fresh.op, small_graph, x, y, w, g)
    _native.check(status)
    torch.cuda.synchronize()
    for name, a, b in zip(("gx", "gy", "gw"), got, want):
        assert_close(a, b.detach().cpu(), dtype, f"noalloc wide {name}")
