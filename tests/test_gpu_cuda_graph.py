"""The convolution's launches inside a CUDA graph.

A step on a small graph is bound by launch and Python overhead, not by the kernels; capturing forward and backward
once and replaying them removes that.  Nothing in the launch path synchronises or allocates outside torch's allocator
once a plan has been used on the device (its tables are uploaded on first use), and the kernels' tile counters put
themselves back to zero, so a captured launch can be replayed as it is.  Checked: replays with new input values give
the eager results, bit for bit.
"""

import pytest
import torch

import lunaequivariance_b200 as luna
from lunaequivariance_b200 import conv as conv_mod
from tests.helpers import config, random_graph

pytestmark = pytest.mark.gpu
DEVICE = "cuda"


@pytest.mark.parametrize("name,dtype", [("fixture", torch.float32), ("cfg5", torch.float32), ("small", torch.float64)])
def test_capture_and_replay(name, dtype):
    in1, in2, out, instructions, _ = config(name)
    module = luna.TensorProductConv(in1, in2, out, instructions, internal_weights=False, shared_weights=False,
                                    dtype=dtype)
    op = module.op
    nodes = 200
    src, dst = random_graph(nodes, 3000, torch.Generator().manual_seed(8))
    graph = luna.make_graph(src.to(DEVICE), dst.to(DEVICE), nodes)
    generator = torch.Generator(device=DEVICE).manual_seed(12)
    rand = lambda *shape: torch.randn(*shape, generator=generator, dtype=dtype, device=DEVICE)
    static = dict(x=rand(nodes, op.in1_dim), y=rand(graph.num_edges, op.in2_dim),
                  w=rand(graph.num_edges, op.weight_numel), g=rand(nodes, op.out_dim))

    def step():
        out_rows = conv_mod.run_forward(op, static["x"], static["y"], static["w"], graph)
        return (out_rows, *conv_mod.run_backward(op, static["x"], static["y"], static["w"], static["g"], graph))

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # warm-up on a side stream, as torch asks for before a capture
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    captured = torch.cuda.CUDAGraph()
    with torch.cuda.graph(captured):
        results = step()
    for trial in range(3):
        for tensor in static.values():
            tensor.copy_(rand(*tensor.shape))
        captured.replay()
        replayed = [t.clone() for t in results]
        eager = step()
        for a, b in zip(replayed, eager):
            assert torch.equal(a, b), f"{name} trial {trial}"
    op.check_status()
