"""SwiGLU of the FoX MLP: host-side mirror of upstream's ``swiglu`` / ``swiglu_linear``
(src/forgetting_transformer/model/forgetting_transformer/glu_linear.py:95-150), plus a packed form that
takes the (.., 2*I) projection output whole and returns its gradient in one buffer (no chunk / cat copies).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib

__all__ = ["swiglu", "swiglu_linear", "swiglu_linear_packed"]


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _rows(t: torch.Tensor) -> torch.Tensor:
    """2-D view (rows, cols) with unit inner stride whose row stride the kernels can use, else a packed copy."""
    t2 = t.reshape(-1, t.shape[-1])
    ok = t2.stride(1) == 1 and t2.stride(0) % 8 == 0 and t2.data_ptr() % 16 == 0
    return t2 if ok else t2.contiguous()


def _check(x):
    if not x.is_cuda:
        raise _lib.FoxError("swiglu needs CUDA tensors on an sm_100 device; there is no CPU path")
    assert x.dtype in (torch.float16, torch.bfloat16), "swiglu is built for 16-bit activations"
    assert x.shape[-1] % 8 == 0


def _fwd(x2, y2):
    lib = _lib.load()
    z = torch.empty((x2.shape[0], x2.shape[1]), dtype=x2.dtype, device=x2.device)
    _lib.check(lib.fox_swiglu_fwd(x2.device.index, _stream(), _lib.dtype_code(x2.dtype), x2.shape[0], x2.shape[1],
                                  x2.data_ptr(), x2.stride(0), y2.data_ptr(), y2.stride(0), z.data_ptr(), z.stride(0)),
               "fox_swiglu_fwd")
    return z


def _bwd(x2, y2, g2, dx, dy, z):
    lib = _lib.load()
    _lib.check(lib.fox_swiglu_bwd(x2.device.index, _stream(), _lib.dtype_code(x2.dtype), x2.shape[0], x2.shape[1],
                                  x2.data_ptr(), x2.stride(0), y2.data_ptr(), y2.stride(0), g2.data_ptr(), g2.stride(0),
                                  dx.data_ptr(), dx.stride(0), dy.data_ptr(), dy.stride(0), _lib.ptr(z),
                                  0 if z is None else z.stride(0)), "fox_swiglu_bwd")


class SwiGLUFunction(torch.autograd.Function):
    """z = swish(x) * y (glu_linear.py:95-113)."""

    @staticmethod
    def forward(ctx, x, y):
        _check(x)
        assert x.shape == y.shape and x.dtype == y.dtype
        with torch.cuda.device(x.device):
            x2, y2 = _rows(x), _rows(y)
            z = _fwd(x2, y2)
        ctx.save_for_backward(x2, y2)
        ctx.shape = x.shape
        return z.reshape(x.shape)

    @staticmethod
    def backward(ctx, dout):
        x2, y2 = ctx.saved_tensors
        with torch.cuda.device(x2.device):
            g2 = _rows(dout)
            dx, dy = torch.empty_like(g2, memory_format=torch.contiguous_format), torch.empty_like(g2, memory_format=torch.contiguous_format)
            _bwd(x2, y2, g2, dx, dy, None)
        return dx.reshape(ctx.shape), dy.reshape(ctx.shape)


def _linear_params(weight, bias):
    """Under autocast the product runs in the autocast dtype (upstream wraps these functions in
    custom_fwd / custom_bwd, glu_linear.py:116-119): the parameters are cast once here, so that forward and
    backward (where autocast is off) multiply in the same dtype; their gradients go back in the parameters' own."""
    if torch.is_autocast_enabled("cuda"):
        dt = torch.get_autocast_dtype("cuda")
        return weight.to(dt), None if bias is None else bias.to(dt)
    return weight, bias


class SwiGLULinearFunction(torch.autograd.Function):
    """(swish(x) * y) W^T + b without keeping the product (glu_linear.py:116-146)."""

    @staticmethod
    def forward(ctx, x, y, weight, bias):
        _check(x)
        with torch.cuda.device(x.device):
            x2, y2 = _rows(x), _rows(y)
            z = _fwd(x2, y2)
            ctx.param_dtypes = (weight.dtype, None if bias is None else bias.dtype)
            weight, bias = _linear_params(weight, bias)
            out = F.linear(z.to(weight.dtype), weight, bias)
        ctx.save_for_backward(x2, y2, weight)
        ctx.linear_bias_is_none = bias is None
        ctx.shape = x.shape
        return out.reshape(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dout, *args):
        x2, y2, weight = ctx.saved_tensors
        with torch.cuda.device(x2.device):
            dout = dout.reshape(-1, dout.shape[-1]).to(weight.dtype)
            dz = F.linear(dout, weight.t()).to(x2.dtype)
            dx, dy, z = torch.empty_like(dz), torch.empty_like(dz), torch.empty_like(dz)
            _bwd(x2, y2, _rows(dz), dx, dy, z)
            dlinear_weight = (dout.t() @ z.to(weight.dtype)).to(ctx.param_dtypes[0])
            dlinear_bias = None if ctx.linear_bias_is_none else dout.sum(0).to(ctx.param_dtypes[1])
        return dx.reshape(ctx.shape), dy.reshape(ctx.shape), dlinear_weight, dlinear_bias


class SwiGLULinearPackedFunction(torch.autograd.Function):
    """Same as SwiGLULinearFunction for xy = [x | y] packed along the last axis: the halves are read in place
    and the gradient is written as one [dx | dy] buffer."""

    @staticmethod
    def forward(ctx, xy, weight, bias):
        _check(xy)
        inter = xy.shape[-1] // 2
        assert xy.shape[-1] == 2 * inter and inter % 8 == 0
        with torch.cuda.device(xy.device):
            p = _rows(xy)
            z = _fwd(p[:, :inter], p[:, inter:])
            ctx.param_dtypes = (weight.dtype, None if bias is None else bias.dtype)
            weight, bias = _linear_params(weight, bias)
            out = F.linear(z.to(weight.dtype), weight, bias)
        ctx.save_for_backward(p, weight)
        ctx.linear_bias_is_none = bias is None
        ctx.shape = xy.shape
        return out.reshape(*xy.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dout, *args):
        p, weight = ctx.saved_tensors
        inter = p.shape[1] // 2
        with torch.cuda.device(p.device):
            dout = dout.reshape(-1, dout.shape[-1]).to(weight.dtype)
            dz = F.linear(dout, weight.t()).to(p.dtype)
            dxy = torch.empty_like(p, memory_format=torch.contiguous_format)
            z = torch.empty_like(dz)
            _bwd(p[:, :inter], p[:, inter:], _rows(dz), dxy[:, :inter], dxy[:, inter:], z)
            dlinear_weight = (dout.t() @ z.to(weight.dtype)).to(ctx.param_dtypes[0])
            dlinear_bias = None if ctx.linear_bias_is_none else dout.sum(0).to(ctx.param_dtypes[1])
        return dxy.reshape(ctx.shape), dlinear_weight, dlinear_bias


swiglu = SwiGLUFunction.apply
swiglu_linear = SwiGLULinearFunction.apply
swiglu_linear_packed = SwiGLULinearPackedFunction.apply
