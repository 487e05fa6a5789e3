"""``spherical_harmonics`` function, its configuration object and the recomputing autograd chain.

Follows the reference's ``src/o3/spherical_harmonics/interface.py``: ``parse_irreps`` (:27-55) for the accepted
forms of ``irreps_out`` / degree lists and their errors, ``SphericalHarmonicsConfig`` (:256-279), the eager chain
forward -> backward -> double-backward (:282-377, nothing but the inputs is saved; derivatives are recomputed from
``x``) and the custom ops ``lunaeq::spherical_harmonics_{forward,backward,double_backward}`` (:75-126).
CUDA float32/float64 inputs only: there is no CPU path in this library.
"""

from __future__ import annotations

import ctypes
import json
from functools import lru_cache

import torch

from . import _native
from .irreps import Irrep, Irreps, as_irreps

UNSET = object()
_NORMALIZATIONS = {"component": 0, "norm": 1, "integral": 2}


def parse_irreps(irreps_out, irreps_in=None):
    """Return ``(irreps_in, irreps_out, degrees)`` from irreps, a string, an int or a list of degrees."""
    is_irreps = isinstance(irreps_out, (str, Irreps, Irrep)) or hasattr(irreps_out, "ls")
    output = as_irreps(irreps_out) if is_irreps else None
    if irreps_in is None:
        odd_even = output is not None and any(ir.l % 2 and ir.p == 1 for _, ir in output)
        irreps_in = "1e" if odd_even else "1o"
    irreps_in = as_irreps(irreps_in)
    if irreps_in not in (Irreps("1o"), Irreps("1e")):
        raise ValueError("SphericalHarmonics input must be one vector (1o) or pseudovector (1e)")
    parity = irreps_in[0].ir.p
    if output is not None:
        if any(ir.p != parity ** ir.l for _, ir in output):
            raise ValueError("SphericalHarmonics output parity is inconsistent with input parity")
        degrees = tuple(ir.l for mul, ir in output for _ in range(mul))
    else:
        degrees = (irreps_out,) if isinstance(irreps_out, int) else tuple(irreps_out)
    if not degrees or any(not isinstance(l, int) or l < 0 for l in degrees):
        raise ValueError("SphericalHarmonics degrees must be nonempty nonnegative integers")
    if max(degrees) > 12:
        raise NotImplementedError("SphericalHarmonics supports degrees through 12")
    output = Irreps([(1, (l, parity ** l)) for l in degrees]).simplify()
    return irreps_in, output, degrees


class SphericalHarmonicsConfig:
    """Static description of one spherical-harmonics evaluation."""

    def __init__(self, degrees, normalize, normalization, dtype, index_bits=32, irreps_in=None):
        self.irreps_in, self.irreps_out, degrees = parse_irreps(degrees, irreps_in)
        if normalization not in _NORMALIZATIONS:
            raise ValueError("normalization must be component, norm or integral")
        self._ls_list = tuple(degrees)
        self._lmax = max(degrees)
        self.normalize, self.normalization = bool(normalize), normalization
        self.compute_dtype, self.index_bits = dtype, index_bits
        self.meta = dict(degrees=self._ls_list, normalize=self.normalize, normalization=normalization, dtype=dtype,
                         out_dim=self.irreps_out.dim)
        self.last_execution_backend = "uninitialized"
        self.backward_backend = None
        # encoded now: a traced program carries it as a string constant and must not run the encoder
        self._descriptor = json.dumps([list(self._ls_list), self.normalize, self.normalization, self.index_bits,
                                       str(self.compute_dtype).removeprefix("torch.")])

    @property
    def out_dim(self) -> int:
        return self.meta["out_dim"]

    def descriptor(self) -> str:
        return self._descriptor

    def native(self, dtype) -> "_native.ShDesc":
        if len(self._ls_list) > 32:
            raise NotImplementedError("at most 32 degree entries are supported")
        desc = _native.ShDesc()
        desc.dtype = _native.dtype_code(dtype)
        desc.num_degrees = len(self._ls_list)
        for index, degree in enumerate(self._ls_list):
            desc.degrees[index] = degree
        desc.normalize = int(self.normalize)
        desc.normalization = _NORMALIZATIONS[self.normalization]
        return desc


@lru_cache(maxsize=128)
def _config_from_descriptor(descriptor: str) -> SphericalHarmonicsConfig:
    degrees, normalize, normalization, index_bits, dtype = json.loads(descriptor)
    return SphericalHarmonicsConfig(tuple(degrees), normalize, normalization, getattr(torch, dtype), index_bits)


def _flat(x: torch.Tensor) -> torch.Tensor:
    return x.reshape(-1, x.shape[-1]).contiguous()


def _check(x: torch.Tensor) -> None:
    if not x.is_cuda:
        raise RuntimeError("CUDA is required for spherical harmonics in this library")
    if x.dtype not in (torch.float32, torch.float64):
        raise TypeError("spherical harmonics require float32 or float64 input")
    if x.ndim == 0 or x.shape[-1] != 3:
        raise ValueError("SphericalHarmonics input must have shape (...,3)")


def run_forward(op: SphericalHarmonicsConfig, x: torch.Tensor) -> torch.Tensor:
    _check(x)
    flat = _flat(x)
    out = torch.empty((flat.shape[0], op.out_dim), dtype=x.dtype, device=x.device)
    desc = op.native(x.dtype)
    with torch.cuda.device(x.device):
        _native.check(_native.library().luna_sh_fwd(ctypes.byref(desc), flat.data_ptr(), out.data_ptr(),
                                                    flat.shape[0], _native.current_stream(x.device)))
    return out.reshape(*x.shape[:-1], op.out_dim)


def run_backward(op: SphericalHarmonicsConfig, x: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    _check(x)
    flat, gflat = _flat(x), _flat(g)
    dx = torch.empty_like(flat)
    desc = op.native(x.dtype)
    with torch.cuda.device(x.device):
        _native.check(_native.library().luna_sh_bwd(ctypes.byref(desc), flat.data_ptr(), gflat.data_ptr(),
                                                    dx.data_ptr(), flat.shape[0], _native.current_stream(x.device)))
    return dx.reshape(x.shape)


def run_double_backward(op: SphericalHarmonicsConfig, x, g, rx, needs=(True, True)):
    _check(x)
    flat, gflat, rflat = _flat(x), _flat(g), _flat(rx)
    sx = torch.empty_like(flat) if needs[0] else None
    sg = torch.empty_like(gflat) if needs[1] else None
    desc = op.native(x.dtype)
    with torch.cuda.device(x.device):
        _native.check(_native.library().luna_sh_dbl_bwd(
            ctypes.byref(desc), flat.data_ptr(), gflat.data_ptr(), rflat.data_ptr(), _native.pointer(sx),
            _native.pointer(sg), flat.shape[0], _native.current_stream(x.device)))
    return (None if sx is None else sx.reshape(x.shape), None if sg is None else sg.reshape(g.shape))


class SphericalHarmonicsFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, op, x):
        ctx.op = op
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(x)
        return run_forward(op, x)

    @staticmethod
    def backward(ctx, g):
        if g is None or ctx.op._lmax == 0:
            return None, None
        (x,) = ctx.saved_tensors
        if torch.is_grad_enabled():
            return None, SphericalHarmonicsBackward.apply(ctx.op, x, g)
        return None, run_backward(ctx.op, x, g.contiguous())


class SphericalHarmonicsBackward(torch.autograd.Function):
    @staticmethod
    def forward(ctx, op, x, g):
        ctx.op = op
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(x, g)
        return run_backward(op, x, g.contiguous())

    @staticmethod
    def backward(ctx, rx):
        if rx is None:
            return None, None, None
        x, g = ctx.saved_tensors
        needs = ctx.needs_input_grad[1:3]
        if torch.is_grad_enabled():
            sx, sg = SphericalHarmonicsDoubleBackward.apply(ctx.op, x, g, rx)
        else:
            sx, sg = run_double_backward(ctx.op, x, g, rx.contiguous(), needs=needs)
        return None, sx if needs[0] else None, sg if needs[1] else None


class SphericalHarmonicsDoubleBackward(torch.autograd.Function):
    @staticmethod
    def forward(ctx, op, x, g, rx):
        ctx.set_materialize_grads(False)
        return run_double_backward(op, x, g, rx.contiguous(), needs=(True, True))

    @staticmethod
    def backward(ctx, bx, bg):
        if bx is None and bg is None:
            return None, None, None, None
        raise NotImplementedError("third-order derivatives of the spherical harmonics are not provided")


# ----------------------------------------------------------------------------------------------- custom ops


@torch.library.custom_op("lunaeq::spherical_harmonics_forward", mutates_args=())
def sh_forward_op(x: torch.Tensor, config: str) -> torch.Tensor:
    return run_forward(_config_from_descriptor(config), x)


@sh_forward_op.register_fake
def _(x, config):
    return x.new_empty((*x.shape[:-1], _config_from_descriptor(config).out_dim))


@torch.library.custom_op("lunaeq::spherical_harmonics_backward", mutates_args=(),
                         schema="(Tensor x, Tensor g, str config) -> Tensor")
def sh_backward_op(x, g, config):
    op = _config_from_descriptor(config)
    if not op._lmax:
        raise ValueError("Constant spherical harmonics have no input-gradient contribution")
    return run_backward(op, x, g.contiguous())


@sh_backward_op.register_fake
def _(x, g, config):
    return torch.empty_like(x, memory_format=torch.contiguous_format)


@torch.library.custom_op("lunaeq::spherical_harmonics_double_backward", mutates_args=(),
                         schema="(Tensor x, Tensor g, Tensor rx, bool[] needs, str config) -> (Tensor?, Tensor?)")
def sh_double_backward_op(x, g, rx, needs, config):
    return run_double_backward(_config_from_descriptor(config), x, g, rx.contiguous(), needs=tuple(needs))


@sh_double_backward_op.register_fake
def _(x, g, rx, needs, config):
    return tuple(torch.empty_like(v, memory_format=torch.contiguous_format) if need else None
                 for v, need in zip((x, g), needs))


def _sh_setup(ctx, inputs, output):
    ctx.config = inputs[-1]
    ctx.save_for_backward(*inputs[:-1])
    ctx.set_materialize_grads(False)


def _sh_forward_backward(ctx, g):
    if g is None or not _config_from_descriptor(ctx.config)._lmax:
        return None, None
    (x,) = ctx.saved_tensors
    return sh_backward_op(x, g, ctx.config), None


def _sh_backward_backward(ctx, rx):
    if rx is None:
        return None, None, None
    x, g = ctx.saved_tensors
    sx, sg = sh_double_backward_op(x, g, rx, list(ctx.needs_input_grad[:2]), ctx.config)
    return sx, sg, None


sh_forward_op.register_autograd(_sh_forward_backward, setup_context=_sh_setup)
sh_backward_op.register_autograd(_sh_backward_backward, setup_context=_sh_setup)


def spherical_harmonics(l, x, normalize, normalization="integral", *, config=None):
    """Evaluate the harmonics of the listed degrees (or irreps) for vectors ``x[..., 3]``."""
    if config is None or config.compute_dtype != x.dtype:
        if config is not None:
            degrees, irreps_in = tuple(config._ls_list), str(config.irreps_in)
            normalize, normalization = config.normalize, config.normalization
        else:
            degrees = l if isinstance(l, (int, str, Irreps, Irrep)) or hasattr(l, "ls") else tuple(l)
            irreps_in = None
        config = SphericalHarmonicsConfig(degrees, bool(normalize), normalization, x.dtype, irreps_in=irreps_in)
    if x.ndim == 0 or x.shape[-1] < 3:
        raise ValueError("SphericalHarmonics input must have shape (...,3)")
    _check(x)
    from .conv import is_compiling

    if is_compiling():
        return torch.ops.lunaeq.spherical_harmonics_forward.default(x, config.descriptor())
    config.last_execution_backend = "cuda_fused"
    tracked = torch.is_grad_enabled() and x.requires_grad and config._lmax > 0
    config.backward_backend = "cuda_fused_recompute" if tracked else None
    return SphericalHarmonicsFunction.apply(config, x) if tracked else run_forward(config, x)


# The composite op a traced or exported program can carry instead of the Python call; it decomposes into the ops
# above (same schema as the reference's fragment, ``src/o3/spherical_harmonics/interface.py:242-253``).
_FRAGMENT = torch.library.Library("lunaeq", "FRAGMENT")
_FRAGMENT.define("spherical_harmonics(Tensor x, int[] degrees, bool normalize, str normalization) -> Tensor")
_FRAGMENT.impl("spherical_harmonics",
               lambda x, degrees, normalize, normalization: spherical_harmonics(degrees, x, normalize, normalization),
               "CompositeImplicitAutograd")

__all__ = ["spherical_harmonics", "SphericalHarmonicsConfig", "parse_irreps", "UNSET"]
