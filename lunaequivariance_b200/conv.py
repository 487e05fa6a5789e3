"""UVU graph convolution: operator object, launch wrappers, autograd chain and ``torch.library`` custom ops.

Mirrors the reference's layers for this path:

* ``LunaTPUVUConv`` / ``create_uvu_conv_operator`` - ``src/lunatp/interface.py:123-144,379-393``;
* ``lunatp_uvu_conv_func`` and the ``UVUConvForward/Backward/DoubleBackward`` autograd functions -
  ``src/lunatp/uvu_conv/interface.py:143-434``;
* custom ops ``lunatp::uvu_conv_{forward,backward,double_backward}`` with the reference's schemas, fake
  (shape) implementations and ``register_autograd`` chain - ``src/lunatp/uvu_conv/interface.py:18-140``.

All arithmetic happens in the C-ABI library; missing cotangents are passed as null pointers and never
materialised.

Beyond the fused first- and second-order kernels, three features of the reference are composed from the same
kernels rather than given kernels of their own:

* ``env`` (per-edge envelope, ``src/lunatp/uvu_conv/kernels/forward.py:141-148``): the message of an edge is linear in
  the edge attributes, so scaling the message by ``env[e]`` is scaling ``edge_attr[e]`` (16 numbers instead of a
  weight row); the product is a torch op and autograd supplies the envelope's gradients at every order;
* ``return_l0_feat`` (per-edge scalar outputs, layout of ``src/lunatp/utils/layout.py:171-189``): the same operator
  restricted to the paths into degree 0, run on the graph in which every edge is its own destination;
* third and higher derivatives (``kernels/triple_backward.py``): every derivative of the four-linear form
  ``F(x, y, w, g)`` is again a partial derivative of ``F`` with other operands, so one autograd function
  (``_Partial``) that maps each free slot onto the forward or the backward kernel is closed under differentiation.
"""

from __future__ import annotations

import ctypes
import json
from collections.abc import Mapping
from functools import lru_cache

import numpy as np
import torch

from . import _native
from .graph import LunaTPGraph, make_graph
from .paths import TensorProductPaths, build_uvu_conv_metadata

_DTYPE_NAMES = {torch.float32: "float32", torch.float64: "float64"}


def is_compiling() -> bool:
    """True while Dynamo or make_fx records a graph (``src/utils/__init__.py:8-12``)."""
    from torch.fx.experimental.proxy_tensor import get_proxy_mode
    from torch.utils._python_dispatch import is_in_torch_dispatch_mode

    return torch.compiler.is_compiling() or (is_in_torch_dispatch_mode() and get_proxy_mode() is not None)


class _Plan:
    """Owns a native plan handle and the host arrays it was created from."""

    def __init__(self, meta: Mapping, dtype: torch.dtype):
        lib = _native.library()
        specs = meta["generated_specs"]
        paths = (_native.UvuPath * len(specs))()
        ti, tj, tk, tc = [], [], [], []
        for record, spec in zip(paths, specs):
            record.x_offset = int(spec["x_offset"])
            record.y_offset = int(spec["y_offset"])
            record.out_offset = int(spec["out_offset"])
            record.weight_offset = int(spec["weight_offset"])
            record.weight_stride = int(spec.get("weight_stride", 1))
            record.channels = int(spec["channels"])
            record.l1, record.l2, record.l3 = int(spec["l1"]), int(spec["l2"]), int(spec["l3"])
            record.term_begin = len(ti)
            for i, j, k, c in spec["terms"]:
                ti.append(int(i))
                tj.append(int(j))
                tk.append(int(k))
                tc.append(float(c))
            record.term_end = len(ti)
        self._arrays = (
            paths,
            np.asarray(ti, dtype=np.int32), np.asarray(tj, dtype=np.int32), np.asarray(tk, dtype=np.int32),
            np.asarray(tc, dtype=np.float64),
        )
        as_ptr = lambda a, t: a.ctypes.data_as(ctypes.POINTER(t))
        desc = _native.UvuDesc(
            _native.dtype_code(dtype), int(meta["in1_dim"]), int(meta["in2_dim"]), int(meta["out_dim"]),
            int(meta["weight_numel"]), len(specs), paths, len(ti),
            as_ptr(self._arrays[1], ctypes.c_int32), as_ptr(self._arrays[2], ctypes.c_int32),
            as_ptr(self._arrays[3], ctypes.c_int32), as_ptr(self._arrays[4], ctypes.c_double),
        )
        handle = ctypes.c_void_p()
        _native.check(lib.luna_uvu_plan_create(ctypes.byref(desc), ctypes.byref(handle)))
        self.handle = handle
        self._destroy = lib.luna_uvu_plan_destroy

    def query(self, what: int) -> int:
        return int(_native.library().luna_uvu_plan_query(self.handle, what))

    def __del__(self):
        handle, self.handle = getattr(self, "handle", None), None
        if handle:
            try:
                self._destroy(handle)
            except Exception:  # interpreter shutdown
                pass


class LunaTPUVUConv:
    """Prepared UVU convolution for one path list and dtype."""

    mode = "uvu_conv"
    index_mode = "uvu_conv"

    def __init__(self, meta: Mapping, *, dtype: torch.dtype = torch.float32, index_bits: int = 32):
        if dtype not in (torch.float32, torch.float64):
            raise ValueError("LunaTP uvu_conv requires torch.float32 or torch.float64.")
        if not meta["generated_specs"] or any(int(s["channels"]) <= 0 for s in meta["generated_specs"]):
            raise ValueError("UVU convolution requires positive channels for every path")
        self.meta = dict(meta)
        self.compute_dtype = dtype
        self.index_bits = index_bits
        self.in1_dim = int(meta["in1_dim"])
        self.in2_dim = int(meta["in2_dim"])
        self.out_dim = int(meta["out_dim"])
        self.weight_numel = int(meta["weight_numel"])
        self.max_channels = int(meta.get("max_channels", max(int(s["channels"]) for s in meta["generated_specs"])))
        self.generated_specs = list(meta["generated_specs"])
        self.l0_offsets, self.l0_dim = l0_feature_layout(self.generated_specs)
        self._l0_operator = None
        self.lunatp_backend = "lunatp_uvuconv_fp64" if dtype == torch.float64 else "lunatp_uvuconv_fp32"
        self.lunatp_dtype = dtype
        self._plan = _Plan(self.meta, dtype)  # host-only; also validates the path list
        self._torch_config = None
        self.torch_config  # built now: a traced program reads it as a constant and must not run the encoder

    @property
    def torch_config(self) -> str:
        """Static description carried as a string constant through traced graphs."""
        if self._torch_config is None:
            meta = dict(self.meta)
            meta["generated_specs"] = [
                {k: ([list(t) for t in v] if k == "terms" else v) for k, v in spec.items()}
                for spec in self.generated_specs
            ]
            self._torch_config = json.dumps(
                dict(mode="uvu_conv", dtype=_DTYPE_NAMES[self.compute_dtype], index_bits=self.index_bits,
                     out_dim=self.out_dim, l0_dim=self.l0_dim, weight_mode="external", meta=meta),
                separators=(",", ":"),
            )
        return self._torch_config

    @property
    def l0_operator(self) -> "LunaTPUVUConv | None":
        """The operator whose output rows are the per-edge scalar features: this operator's paths into degree 0,
        each instruction writing its own block of ``channels`` columns (``None`` if there is no such path)."""
        if self.l0_dim == 0:
            return None
        if self._l0_operator is None:
            specs = [dict(spec, out_offset=self.l0_offsets[index])
                     for index, spec in enumerate(self.generated_specs) if index in self.l0_offsets]
            meta = dict(self.meta, out_dim=self.l0_dim, generated_specs=specs)
            self._l0_operator = LunaTPUVUConv(meta, dtype=self.compute_dtype, index_bits=self.index_bits)
        return self._l0_operator

    @property
    def uses_staged_kernels(self) -> bool:
        return bool(self._plan.query(0))

    @property
    def canonical_l2(self) -> int:
        """Highest edge-attribute degree if the path list is the full list of allowed couplings, else -1."""
        return self._plan.query(5)

    @property
    def uses_compiled_patterns(self) -> bool:
        """Whether the backward kernel with compiled-in coupling patterns applies."""
        return self._plan.query(6) > 0

    @property
    def backward_variant(self) -> str:
        """Which first-order backward kernel aligned inputs get: ``generic`` (table-driven), ``tables`` (staged,
        path list read from tables), ``row`` or ``units`` (compiled-in coupling patterns)."""
        return ("generic", "tables", "row", "units")[self._plan.query(7)]

    def check_status(self, device=None) -> None:
        """Raise ``RuntimeError`` if a kernel of this operator gave up a bounded wait since the last check.

        The staged kernels wait for their bulk copies with an iteration limit; a warp whose wait runs out records a
        code in the plan's device status word and returns, leaving its outputs partly written.  This call reads the
        word on the current stream of ``device`` (it synchronises that stream) and clears it.
        """
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        with torch.cuda.device(device):
            _native.check(_native.library().luna_uvu_check_status(self._plan.handle, _native.current_stream(device)))

    def force_generic(self, enabled: bool = True) -> None:
        """Route every call through the table-driven kernels (for comparisons and tests)."""
        _native.check(_native.library().luna_uvu_plan_set_generic(self._plan.handle, int(enabled)))

    def __getstate__(self):
        return dict(meta=self.meta, dtype=self.compute_dtype, index_bits=self.index_bits)

    def __setstate__(self, state):
        self.__init__(state["meta"], dtype=state["dtype"], index_bits=state["index_bits"])

    @staticmethod
    def run(op, x, edge_attr, weight, *, graph, env=None, return_l0_feat=False):
        return lunatp_uvu_conv_func(op, x, edge_attr, weight, graph=graph, env=env, return_l0_feat=return_l0_feat)


def l0_feature_layout(specs) -> tuple[dict, int]:
    """Column offset of every path into degree 0 and the total width of the per-edge scalar features.

    Blocks follow the order of the paths' output offsets; the specs one instruction was split into (several channels
    of the second input) share the instruction's block.
    """
    offsets, blocks, width = {}, {}, 0
    for index, spec in sorted(enumerate(specs), key=lambda item: int(item[1]["out_offset"])):
        if int(spec["l3"]) != 0:
            continue
        block = ("instruction", int(spec["l0_path"])) if "l0_path" in spec else ("path", index)
        if block not in blocks:
            blocks[block] = width
            width += int(spec["channels"])
        offsets[index] = blocks[block]
    return offsets, width


def edge_output_graph(graph: LunaTPGraph) -> LunaTPGraph:
    """The graph with the same sources in which edge ``e`` is destination ``e``: a convolution on it returns the
    messages themselves, one row per edge.  Built once per graph and kept with it."""
    cached = graph._tables.get("edge_output_graph")
    if cached is None:
        edges = graph.num_edges
        own = torch.arange(edges, device=graph.src.device, dtype=torch.int32)
        cached = make_graph(graph.src, own, edges, num_src_nodes=graph.source_rows)
        graph._tables["edge_output_graph"] = cached
    return cached


def create_uvu_conv_operator(official_tp_or_meta, *, dtype=None) -> LunaTPUVUConv:
    if dtype is None:
        dtype = torch.float32
    elif dtype is not torch.float32 and dtype is not torch.float64:
        raise ValueError("LunaTP uvu_conv requires torch.float32 or torch.float64.")
    if isinstance(official_tp_or_meta, Mapping):
        meta = official_tp_or_meta
        tp = None
    else:
        tp = TensorProductPaths.from_tensor_product(official_tp_or_meta)
        meta = build_uvu_conv_metadata(tp, dtype)
    op = LunaTPUVUConv(meta, dtype=dtype)
    if tp is not None:
        op.tp = tp
    return op


@lru_cache(maxsize=128)
def compiled_config(config: str) -> dict:
    return json.loads(config)


@lru_cache(maxsize=128)
def compiled_operator(config: str) -> LunaTPUVUConv:
    settings = compiled_config(config)
    if settings["mode"] != "uvu_conv":
        raise NotImplementedError(f"only uvu_conv operators are provided, got {settings['mode']!r}")
    return LunaTPUVUConv(settings["meta"], dtype=getattr(torch, settings["dtype"]), index_bits=settings["index_bits"])


# ----------------------------------------------------------------------------------------------- launch wrappers


def _require_cuda(tensor: torch.Tensor) -> None:
    if not tensor.is_cuda:
        raise RuntimeError("CUDA is required for SO3 LunaTP.")


def _prepared(tensor: torch.Tensor | None) -> torch.Tensor | None:
    """Contiguous and 16-byte aligned (offset views are cloned, as the reference does for vector loads,
    ``src/lunatp/uvu_conv/kernels/backward.py:623-628``)."""
    if tensor is None:
        return None
    tensor = tensor.contiguous()
    if tensor.data_ptr() % 16:
        tensor = tensor.clone()
    return tensor


def _check_inputs(op: LunaTPUVUConv, x, y, w, source_rows, num_edges, *, g=None, num_nodes=0, rx=None, ry=None,
                  rw=None) -> None:
    _require_cuda(x)
    for name, t, rows, cols in (("x", x, source_rows, op.in1_dim), ("edge_attr", y, num_edges, op.in2_dim),
                                ("weight", w, num_edges, op.weight_numel), ("grad_out", g, num_nodes, op.out_dim),
                                ("rx", rx, source_rows, op.in1_dim), ("ry", ry, num_edges, op.in2_dim),
                                ("rw", rw, num_edges, op.weight_numel)):
        if t is None:
            continue
        if t.dtype != op.compute_dtype:
            raise TypeError(f"{name} must be {op.compute_dtype}, got {t.dtype}")
        if t.device != x.device:
            raise ValueError("features, weights and graph must share one CUDA device")
        if t.ndim != 2 or t.shape[0] != rows or t.shape[1] != cols:
            raise ValueError(f"{name} must have shape ({rows}, {cols}), got {tuple(t.shape)}")


def _scratch(op: LunaTPUVUConv, num_nodes: int, num_edges: int, device) -> tuple[torch.Tensor | None, int]:
    size = int(_native.library().luna_uvu_conv_scratch_bytes(op._plan.handle, num_nodes, num_edges))
    if size <= 0:
        return None, 0
    return torch.empty(size, dtype=torch.uint8, device=device), size


class _GraphView:
    """Native graph struct built from a tensor table list (custom-op path) or a LunaTPGraph."""

    def __init__(self, tables, num_nodes: int):
        src, dst, dst_rowptr, src_rowptr, edge_ids_by_src = tables[:5]
        self.keep = (src, dst, dst_rowptr, src_rowptr, edge_ids_by_src)
        for t in self.keep:
            if t.dtype != torch.int32:
                raise OverflowError("this build supports int32 graph tables only")
        self.num_nodes = int(num_nodes)
        self.source_rows = int(src_rowptr.numel()) - 1
        self.num_edges = int(src.numel())
        self.struct = _native.Graph(self.num_nodes, self.source_rows, self.num_edges, src.data_ptr(), dst.data_ptr(),
                                    dst_rowptr.data_ptr(), src_rowptr.data_ptr(), edge_ids_by_src.data_ptr())


def _graph_struct(graph):
    """(native struct, destination rows, source rows, edges)"""
    if isinstance(graph, LunaTPGraph):
        return graph.native(), graph.num_nodes, graph.source_rows, graph.num_edges
    return graph.struct, graph.num_nodes, graph.source_rows, graph.num_edges


def _output(given, shape, like: torch.Tensor, name: str) -> torch.Tensor:
    """A caller-supplied output tensor (checked) or a fresh one."""
    if given is None:
        return torch.empty(shape, dtype=like.dtype, device=like.device)
    if tuple(given.shape) != tuple(shape) or given.dtype != like.dtype or given.device != like.device:
        raise ValueError(f"{name} must be a {like.dtype} tensor of shape {tuple(shape)} on {like.device}")
    if not given.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return given


def _split_of(graph):
    """The virtual-row form of a graph with very long rows (``LunaTPGraph.split_rows``), else ``None``."""
    return graph.split_rows() if isinstance(graph, LunaTPGraph) else None


def _deliver(value, given, add=False):
    """Hand a computed tensor over in the caller's tensor, if there is one."""
    if given is None or value is None:
        return value
    return given.add_(value) if add else given.copy_(value)


def run_forward(op: LunaTPUVUConv, x, y, w, graph, *, out=None) -> torch.Tensor:
    """``out`` may name the tensor to write (for example a row range of a larger one)."""
    split = _split_of(graph)
    if split is not None:  # long rows are walked as several virtual rows, then summed
        _check_inputs(op, x, y, w, graph.source_rows, graph.num_edges)
        virtual = run_forward(op, split.sources.gather(x), y, w, split.graph)
        return _deliver(split.destinations.reduce(virtual), out)
    struct, n, ns, e = _graph_struct(graph)
    _check_inputs(op, x, y, w, ns, e)
    x, y, w = _prepared(x), _prepared(y), _prepared(w)
    out = _output(out, (n, op.out_dim), x, "out")
    with torch.cuda.device(x.device):
        _native.check(_native.library().luna_uvu_conv_fwd(
            op._plan.handle, ctypes.byref(struct), x.data_ptr(), y.data_ptr(), w.data_ptr(), out.data_ptr(),
            _native.current_stream(x.device)))
    return out


def run_backward(op: LunaTPUVUConv, x, y, w, g, graph, needs=(True, True, True), *, out=(None, None, None),
                 add_gx=False):
    """``out`` may name the tensors to write (gx, gy, gw; each optional).  With ``add_gx`` the source-row gradient
    is added to ``out[0]`` instead of written: calls on pieces of one graph's edge list then sum up to the whole."""
    if add_gx and (not needs[0] or out[0] is None):
        raise ValueError("add_gx needs the tensor to add to as out[0]")
    split = _split_of(graph)
    if split is not None:
        _check_inputs(op, x, y, w, graph.source_rows, graph.num_edges, g=g, num_nodes=graph.num_nodes)
        gx, gy, gw = run_backward(op, split.sources.gather(x), y, w, split.destinations.gather(g), split.graph,
                                  needs, out=(None, out[1], out[2]))
        return _deliver(split.sources.reduce(gx), out[0], add_gx), gy, gw
    struct, n, ns, e = _graph_struct(graph)
    _check_inputs(op, x, y, w, ns, e, g=g, num_nodes=n)
    x, y, w, g = _prepared(x), _prepared(y), _prepared(w), _prepared(g)
    if not any(needs):
        return None, None, None
    gx = _output(out[0], x.shape, x, "gx") if needs[0] else None
    gy = _output(out[1], y.shape, y, "gy") if needs[1] else None
    gw = _output(out[2], w.shape, w, "gw") if needs[2] else None
    if e == 0 or n == 0:
        return tuple(None if t is None else (t if add_gx and t is gx else t.zero_()) for t in (gx, gy, gw))
    entry = _native.library().luna_uvu_conv_bwd_add_gx if add_gx else _native.library().luna_uvu_conv_bwd
    with torch.cuda.device(x.device):
        scratch, size = _scratch(op, n, e, x.device)
        _native.check(entry(
            op._plan.handle, ctypes.byref(struct), x.data_ptr(), y.data_ptr(), w.data_ptr(), g.data_ptr(),
            _native.pointer(gx), _native.pointer(gy), _native.pointer(gw), _native.pointer(scratch), size,
            _native.current_stream(x.device)))
    return gx, gy, gw


def run_double_backward(op: LunaTPUVUConv, x, y, w, g, rx, ry, rw, graph, needs=(True, True, True, True)):
    split = _split_of(graph)
    if split is not None:
        _check_inputs(op, x, y, w, graph.source_rows, graph.num_edges, g=g, num_nodes=graph.num_nodes, rx=rx, ry=ry,
                      rw=rw)
        gather_s, gather_d = split.sources.gather, split.destinations.gather
        hx, hy, hw, hg = run_double_backward(op, gather_s(x), y, w, gather_d(g), gather_s(rx), ry, rw, split.graph,
                                             needs)
        return split.sources.reduce(hx), hy, hw, split.destinations.reduce(hg)
    struct, n, ns, e = _graph_struct(graph)
    _check_inputs(op, x, y, w, ns, e, g=g, num_nodes=n, rx=rx, ry=ry, rw=rw)
    x, y, w, g = _prepared(x), _prepared(y), _prepared(w), _prepared(g)
    rx, ry, rw = _prepared(rx), _prepared(ry), _prepared(rw)
    if not any(needs):
        return None, None, None, None
    hx = torch.empty_like(x) if needs[0] else None
    hy = torch.empty_like(y) if needs[1] else None
    hw = torch.empty_like(w) if needs[2] else None
    hg = torch.empty_like(g) if needs[3] else None
    if e == 0 or n == 0:
        return tuple(None if t is None else t.zero_() for t in (hx, hy, hw, hg))
    with torch.cuda.device(x.device):
        scratch, size = _scratch(op, n, e, x.device)
        _native.check(_native.library().luna_uvu_conv_dbl_bwd(
            op._plan.handle, ctypes.byref(struct), x.data_ptr(), y.data_ptr(), w.data_ptr(), g.data_ptr(),
            _native.pointer(rx), _native.pointer(ry), _native.pointer(rw),
            _native.pointer(hx), _native.pointer(hy), _native.pointer(hw), _native.pointer(hg),
            _native.pointer(scratch), size, _native.current_stream(x.device)))
    return hx, hy, hw, hg


# ----------------------------------------------------------------------------------------------- eager autograd chain


def _engine_needs(needs) -> tuple:
    """Which gradients of the running autograd node's tensor inputs (``needs`` lists them in order) will be used.

    ``ctx.needs_input_grad`` only says which inputs require grad.  Under ``torch.autograd.grad(outputs, inputs)`` the
    engine also knows which of them lie on a path to the requested ``inputs``: a gradient whose consumer node will not
    run is dropped right after this node returns it.  The force-training step is the case that matters: the energy is
    differentiated with respect to the edge vectors only, yet the per-edge weights require grad for the later loss, so
    without this a weight-sized gradient would be computed and thrown away.  Any doubt (no engine information, a
    consumer the engine cannot be asked about, an API change) counts as "used".
    """
    needs = tuple(bool(n) for n in needs)
    try:
        consumers = torch._C._current_autograd_node().next_functions
        if len(consumers) != len(needs):  # one edge per tensor input; anything else is not understood
            return needs
    except Exception:
        return needs
    narrowed = []
    for need, (consumer, _) in zip(needs, consumers):
        if need and consumer is not None:
            try:
                need = bool(torch._C._will_engine_execute_node(consumer))
            except Exception:  # e.g. a leaf's accumulator cannot be queried under autograd.grad
                need = True
        narrowed.append(need and consumer is not None)
    return tuple(narrowed)


def _through_view(tensor):
    """A leaf that requires grad, seen through a no-copy view: the view's autograd node, unlike the leaf's own
    accumulator, can be asked whether the running backward pass will reach it (see ``_engine_needs``)."""
    if tensor is not None and tensor.requires_grad and tensor.is_leaf and torch.is_grad_enabled():
        return tensor.view_as(tensor)
    return tensor


class UVUConvForward(torch.autograd.Function):
    @staticmethod
    def forward(ctx, op, x, y, w, graph):
        ctx.op, ctx.graph = op, graph
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(x, y, w)
        return run_forward(op, x, y, w, graph)

    @staticmethod
    def backward(ctx, grad_out):
        x, y, w = ctx.saved_tensors
        op, graph = ctx.op, ctx.graph
        needs = ctx.needs_input_grad[1:4]
        if grad_out is None:
            return (None,) + tuple(torch.zeros_like(t) if need else None for t, need in zip((x, y, w), needs)) + (None,)
        needs = _engine_needs(needs)
        g = grad_out.contiguous()
        if torch.is_grad_enabled():
            gx, gy, gw = UVUConvBackward.apply(op, x, y, w, g, graph, needs)
        else:
            gx, gy, gw = run_backward(op, x, y, w, g, graph, needs=needs)
        return (None, gx, gy, gw, None)


class UVUConvBackward(torch.autograd.Function):
    """First-order gradients as a differentiable function of (x, y, w, g); ``needs`` selects the outputs."""

    @staticmethod
    def forward(ctx, op, x, y, w, g, graph, needs=(True, True, True)):
        ctx.op, ctx.graph = op, graph
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(x, y, w, g)
        return run_backward(op, x, y, w, g, graph, needs=tuple(needs))

    @staticmethod
    def backward(ctx, rx, ry, rw):
        x, y, w, g = ctx.saved_tensors
        needs = ctx.needs_input_grad[1:5]
        if rx is None and ry is None and rw is None:
            return (None,) * 7
        needs = _engine_needs(needs)
        if torch.is_grad_enabled():
            hx, hy, hw, hg = UVUConvDoubleBackward.apply(ctx.op, x, y, w, g, rx, ry, rw, ctx.graph, needs)
        else:
            hx, hy, hw, hg = run_double_backward(ctx.op, x, y, w, g, rx, ry, rw, ctx.graph, needs=needs)
        return (None, hx, hy, hw, hg, None, None)


class _Partial(torch.autograd.Function):
    """``dF/d(slot)`` of the four-linear form ``F(x, y, w, g)`` at the other three operands (slot 0..3 = x, y, w, g).

    The operand passed in the free slot only lends its shape.  ``<r, dF/ds(a, b, c)> = F(s=r, a, b, c)``, so the
    gradient with respect to operand ``a`` is ``dF/da`` with the cotangent ``r`` in slot ``s``: the backward of this
    function is this function again, which makes derivatives of any order available.
    """

    @staticmethod
    def forward(ctx, op, graph, slot, x, y, w, g):
        ctx.op, ctx.graph, ctx.slot = op, graph, slot
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(x, y, w, g)
        if slot == 3:
            return run_forward(op, x, y, w, graph)
        return run_backward(op, x, y, w, g, graph, needs=tuple(i == slot for i in range(3)))[slot]

    @staticmethod
    def backward(ctx, r):
        grads = [None] * 4
        if r is not None:
            operands = list(ctx.saved_tensors)
            operands[ctx.slot] = r.contiguous()
            for other in range(4):
                if other != ctx.slot and ctx.needs_input_grad[3 + other]:
                    grads[other] = _Partial.apply(ctx.op, ctx.graph, other, *operands)
        return (None, None, None, *grads)


def run_triple_backward(op, x, y, w, g, rx, ry, rw, bx, by, bw, bg, graph, needs=(True,) * 7):
    """Gradients of ``<bx,hx> + <by,hy> + <bw,hw> + <bg,hg>`` (the second-order outputs contracted with their
    cotangents) with respect to ``x, y, w, g, rx, ry, rw``; missing cotangents and tangents are skipped."""
    leaves = [None if t is None else t.detach().requires_grad_(bool(need))
              for t, need in zip((x, y, w, g, rx, ry, rw), needs)]
    X, Y, W, G, RX, RY, RW = leaves
    with torch.enable_grad():
        def partial(slot, a, b, c, d):
            return _Partial.apply(op, graph, slot, a, b, c, d)

        # second-order outputs as sums of partials (src/lunatp/utils/contractions.py:41-49)
        programs = (
            (bx, 0, ((X, RY, W, G), (X, Y, RW, G))),
            (by, 1, ((RX, Y, W, G), (X, Y, RW, G))),
            (bw, 2, ((RX, Y, W, G), (X, RY, W, G))),
            (bg, 3, ((RX, Y, W, G), (X, RY, W, G), (X, Y, RW, G))),
        )
        outputs, seeds = [], []
        for seed, slot, terms in programs:
            if seed is None:
                continue
            parts = [partial(slot, *operands) for operands in terms if all(o is not None for o in operands)]
            if parts:
                outputs.append(sum(parts[1:], parts[0]))
                seeds.append(seed.contiguous())
        wanted = [leaf for leaf, need in zip(leaves, needs) if leaf is not None and need]
        found = iter(torch.autograd.grad(outputs, wanted, seeds, allow_unused=True)) if outputs and wanted else iter(())
    result = []
    for leaf, need in zip(leaves, needs):
        value = next(found, None) if (leaf is not None and need) else None
        result.append(value)
    return tuple(result)


class UVUConvDoubleBackward(torch.autograd.Function):
    @staticmethod
    def forward(ctx, op, x, y, w, g, rx, ry, rw, graph, needs=(True, True, True, True)):
        ctx.op, ctx.graph = op, graph
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(x, y, w, g, rx, ry, rw)
        return run_double_backward(op, x, y, w, g, rx, ry, rw, graph, needs=tuple(needs))

    @staticmethod
    def backward(ctx, bx, by, bw, bg):
        if bx is None and by is None and bw is None and bg is None:
            return (None,) * 10
        x, y, w, g, rx, ry, rw = ctx.saved_tensors
        needs = _engine_needs(ctx.needs_input_grad[1:8])
        grads = run_triple_backward(ctx.op, x, y, w, g, rx, ry, rw, bx, by, bw, bg, ctx.graph, needs=needs)
        return (None, *grads, None, None)


# ----------------------------------------------------------------------------------------------- custom ops


@torch.library.custom_op(
    "lunatp::uvu_conv_forward", mutates_args=(),
    schema="(Tensor x, Tensor y, Tensor w, Tensor? env, Tensor?[] tables, SymInt num_nodes, bool return_l0, "
           "str config) -> (Tensor, Tensor?)")
def conv_forward(x, y, w, env, tables, num_nodes, return_l0, config):
    if env is not None or return_l0:
        # this library composes both outside the op (see lunatp_uvu_conv_func): the envelope as a product with the
        # edge attributes, the per-edge scalar features as a second call of this op
        raise NotImplementedError("pass env and return_l0_feat to the module or to lunatp_uvu_conv_func")
    op = compiled_operator(config)
    return run_forward(op, x, y, w, _GraphView(tables, num_nodes)), None


@conv_forward.register_fake
def _(x, y, w, env, tables, num_nodes, return_l0, config):
    dims = compiled_config(config)
    return x.new_empty((num_nodes, dims["out_dim"])), None


@torch.library.custom_op(
    "lunatp::uvu_conv_backward", mutates_args=(),
    schema="(Tensor x, Tensor y, Tensor w, Tensor? env, Tensor g, Tensor? gl0, Tensor?[] tables, SymInt num_nodes, "
           "bool[] needs, str config) -> (Tensor?, Tensor?, Tensor?, Tensor?)")
def conv_backward(x, y, w, env, g, gl0, tables, num_nodes, needs, config):
    op = compiled_operator(config)
    gx, gy, gw = run_backward(op, x, y, w, g, _GraphView(tables, num_nodes), needs=tuple(needs[:3]))
    return gx, gy, gw, None


@conv_backward.register_fake
def _(x, y, w, env, g, gl0, tables, num_nodes, needs, config):
    return tuple(torch.empty_like(v, memory_format=torch.contiguous_format) if need and v is not None else None
                 for v, need in zip((x, y, w, env), needs))


@torch.library.custom_op(
    "lunatp::uvu_conv_double_backward", mutates_args=(),
    schema="(Tensor x, Tensor y, Tensor w, Tensor? env, Tensor g, Tensor? gl0, Tensor? rx, Tensor? ry, Tensor? rw, "
           "Tensor? re, Tensor?[] tables, SymInt num_nodes, bool[] needs, str config) -> "
           "(Tensor?, Tensor?, Tensor?, Tensor?, Tensor?, Tensor?)")
def conv_double_backward(x, y, w, env, g, gl0, rx, ry, rw, re, tables, num_nodes, needs, config):
    op = compiled_operator(config)
    want = (needs[0], needs[1], needs[2], needs[4])
    hx, hy, hw, hg = run_double_backward(op, x, y, w, g, rx, ry, rw, _GraphView(tables, num_nodes), needs=want)
    return hx, hy, hw, None, hg, None


@conv_double_backward.register_fake
def _(x, y, w, env, g, gl0, rx, ry, rw, re, tables, num_nodes, needs, config):
    return tuple(torch.empty_like(v, memory_format=torch.contiguous_format) if need and v is not None else None
                 for v, need in zip((x, y, w, env, g, gl0), needs))


@torch.library.custom_op(
    "lunatp::uvu_conv_triple_backward", mutates_args=(),
    schema="(Tensor x, Tensor y, Tensor w, Tensor? env, Tensor g, Tensor? gl0, Tensor? rx, Tensor? ry, Tensor? rw, "
           "Tensor? re, Tensor? sx, Tensor? sy, Tensor? sw, Tensor? sg, Tensor? se, Tensor? sl0, Tensor?[] tables, "
           "SymInt num_nodes, bool[] needs, str config) -> (Tensor?, Tensor?, Tensor?, Tensor?, Tensor?, Tensor?, "
           "Tensor?, Tensor?, Tensor?, Tensor?)")
def conv_triple_backward(x, y, w, env, g, gl0, rx, ry, rw, re, sx, sy, sw, sg, se, sl0, tables, num_nodes, needs,
                         config):
    """Outputs in the reference's order (dx, dy, dw, de, dg, dl0, drx, dry, drw, dre); the envelope and scalar-feature
    slots are always None here."""
    op = compiled_operator(config)
    want = (needs[0], needs[1], needs[2], needs[4], needs[6], needs[7], needs[8])
    dx, dy, dw, dg, drx, dry, drw = run_triple_backward(op, x, y, w, g, rx, ry, rw, sx, sy, sw, sg,
                                                        _GraphView(tables, num_nodes), needs=want)
    return dx, dy, dw, None, dg, None, drx, dry, drw, None


@conv_triple_backward.register_fake
def _(x, y, w, env, g, gl0, rx, ry, rw, re, sx, sy, sw, sg, se, sl0, tables, num_nodes, needs, config):
    return tuple(torch.empty_like(v, memory_format=torch.contiguous_format) if need and v is not None else None
                 for v, need in zip((x, y, w, env, g, gl0, rx, ry, rw, re), needs))


def _setup_forward(ctx, inputs, output):
    x, y, w, env, tables, ctx.num_nodes, _, ctx.config = inputs
    ctx.save_for_backward(x, y, w, *tables)
    ctx.table_count = len(tables)
    ctx.set_materialize_grads(False)


def _forward_backward(ctx, g, gl0):
    x, y, w, *tables = ctx.saved_tensors
    table_grad = [None] * ctx.table_count
    if g is None:
        g = x.new_zeros((ctx.num_nodes, compiled_config(ctx.config)["out_dim"]))
    needs = list(ctx.needs_input_grad[:3]) + [False]
    gx, gy, gw, _ = conv_backward(x, y, w, None, g.contiguous(), None, tables, ctx.num_nodes, needs, ctx.config)
    return gx, gy, gw, None, table_grad, None, None, None


def _setup_backward(ctx, inputs, output):
    x, y, w, env, g, gl0, tables, ctx.num_nodes, _, ctx.config = inputs
    ctx.save_for_backward(x, y, w, g, *tables)
    ctx.table_count = len(tables)
    ctx.set_materialize_grads(False)


def _backward_backward(ctx, rx, ry, rw, re):
    x, y, w, g, *tables = ctx.saved_tensors
    table_grad = [None] * ctx.table_count
    if rx is None and ry is None and rw is None:
        return None, None, None, None, None, None, table_grad, None, None, None
    needs = [ctx.needs_input_grad[0], ctx.needs_input_grad[1], ctx.needs_input_grad[2], False,
             ctx.needs_input_grad[4], False]
    hx, hy, hw, _, hg, _ = conv_double_backward(x, y, w, None, g, None, rx, ry, rw, None, tables, ctx.num_nodes,
                                                needs, ctx.config)
    return hx, hy, hw, None, hg, None, table_grad, None, None, None


def _setup_double_backward(ctx, inputs, output):
    x, y, w, env, g, gl0, rx, ry, rw, re, tables, ctx.num_nodes, _, ctx.config = inputs
    ctx.save_for_backward(x, y, w, g, rx, ry, rw, *tables)
    ctx.table_count = len(tables)
    ctx.set_materialize_grads(False)


def _double_backward_backward(ctx, sx, sy, sw, se, sg, sl0):
    x, y, w, g, rx, ry, rw, *tables = ctx.saved_tensors
    table_grad = [None] * ctx.table_count
    if sx is None and sy is None and sw is None and sg is None:
        return (None,) * 10 + (table_grad, None, None, None)
    needs = [bool(n) for n in ctx.needs_input_grad[:10]]
    needs[3] = needs[5] = needs[9] = False  # envelope and scalar-feature slots
    dx, dy, dw, _, dg, _, drx, dry, drw, _ = conv_triple_backward(
        x, y, w, None, g, None, rx, ry, rw, None, sx, sy, sw, sg, None, None, tables, ctx.num_nodes, needs, ctx.config)
    return dx, dy, dw, None, dg, None, drx, dry, drw, None, table_grad, None, None, None


conv_forward.register_autograd(_forward_backward, setup_context=_setup_forward)
conv_backward.register_autograd(_backward_backward, setup_context=_setup_backward)
conv_double_backward.register_autograd(_double_backward_backward, setup_context=_setup_double_backward)


# ----------------------------------------------------------------------------------------------- functional entry


def _conv(op: LunaTPUVUConv, x, edge_attr, weight, graph: LunaTPGraph):
    if is_compiling():
        out, _ = torch.ops.lunatp.uvu_conv_forward.default(
            x.contiguous(), edge_attr.contiguous(), weight.contiguous(), None, graph.table_list(),
            graph.num_nodes, False, op.torch_config)
        return out
    return UVUConvForward.apply(op, _through_view(x), _through_view(edge_attr), _through_view(weight), graph)


def lunatp_uvu_conv_func(op: LunaTPUVUConv, x, edge_attr, weight, *, graph: LunaTPGraph, env=None,
                         return_l0_feat: bool = False):
    """Aggregate UVU edge messages by destination, differentiable to any order.

    ``x`` [num_nodes, in1_dim], ``edge_attr`` [num_edges, in2_dim], ``weight`` [num_edges, weight_numel] share one
    CUDA device and the operator's dtype; edge data follows the order of the graph's edge list.  ``env``
    ([num_edges] or [num_edges, 1]) scales each edge's message before aggregation.  With ``return_l0_feat`` the result
    is ``(out, l0_feat)``: ``l0_feat`` [num_edges, l0_dim] holds the raw per-edge contributions of the paths into
    degree 0 (one column per channel of each such instruction), without ``env``.
    """
    if weight is None:
        raise TypeError("UVU convolution requires explicit per-edge weights")
    if not isinstance(graph, LunaTPGraph):
        raise TypeError("graph must be a LunaTPGraph prepared with make_graph / create_graph")
    scaled = edge_attr
    if env is not None:
        if env.ndim == 1:
            env = env.unsqueeze(-1)
        if env.ndim != 2 or env.shape[0] != edge_attr.shape[0] or env.shape[1] != 1:
            raise ValueError(f"env must have shape ({edge_attr.shape[0]},) or ({edge_attr.shape[0]}, 1), "
                             f"got {tuple(env.shape)}")
        if env.dtype != edge_attr.dtype or env.device != edge_attr.device:
            raise TypeError("env must share the dtype and device of edge_attr")
        scaled = edge_attr * env  # the message is linear in the edge attributes
    out = _conv(op, x, scaled, weight, graph)
    if not return_l0_feat:
        return out
    scalar_op = op.l0_operator
    if scalar_op is None or graph.num_edges == 0:
        return out, edge_attr.new_zeros((graph.num_edges, op.l0_dim))
    return out, _conv(scalar_op, x, edge_attr, weight, edge_output_graph(graph))


__all__ = ["LunaTPUVUConv", "create_uvu_conv_operator", "lunatp_uvu_conv_func", "run_forward", "run_backward",
           "run_double_backward", "run_triple_backward", "l0_feature_layout", "edge_output_graph", "UVUConvForward", "UVUConvBackward", "UVUConvDoubleBackward"]
