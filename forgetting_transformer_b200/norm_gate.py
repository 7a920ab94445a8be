"""Fused per-head RMSNorm + sigmoid output gate of the FoX-Pro layer.

Host-side mirror of upstream's ``FusedGroupNormGated`` module and
``group_norm_gated`` function
(src/forgetting_transformer/model/forgetting_transformer/fuse_norm_gate.py:977-1002,
1389-1461) for the one configuration the FoX layer instantiates
(modeling_forgetting_transformer.py:243): ``is_rms_norm=True``,
``activation="sigmoid"``, a weight, no bias, no residual.  Everything else the
upstream class can do is rejected with NotImplementedError rather than routed
through another implementation.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from . import _lib

__all__ = ["group_norm_gated", "FusedGroupNormGated", "GroupRMSNormSigmoidGate", "group_norm", "GroupNorm",
           "rms_norm", "RMSNorm", "RowRMSNorm"]

_MAX_PARTIALS = 148 * 8


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class GroupRMSNormSigmoidGate(torch.autograd.Function):
    """y = rmsnorm_per_group(x) * weight * sigmoid(g); saves (x, g, weight, rstd) like
    upstream's LayerNormGatedFunction (fuse_norm_gate.py:726-822).  ``g=None`` leaves the gate
    out: upstream's LayerNormFunction (layernorm.py:523-620) in its per-head RMSNorm use."""

    @staticmethod
    def forward(ctx, x, g, weight, num_groups, eps):
        if not x.is_cuda:
            raise _lib.FoxError("group_norm_gated needs CUDA tensors on an sm_100 device; there is no CPU path")
        assert g is None or (x.shape == g.shape and x.dtype == g.dtype)
        assert x.dtype in (torch.float16, torch.bfloat16)
        hidden = x.shape[-1]
        assert hidden % num_groups == 0 and weight.shape == (hidden,)
        D = hidden // num_groups
        lib = _lib.load()
        shape = x.shape
        with torch.cuda.device(x.device):
            x2 = x.reshape(-1, hidden).contiguous()
            g2 = None if g is None else g.reshape(-1, hidden).contiguous()
            w32 = weight.detach().float().contiguous()
            tokens = x2.shape[0]
            y = torch.empty_like(x2)
            rstd = torch.empty(tokens * num_groups, dtype=torch.float32, device=x.device)
            _lib.check(lib.fox_normgate_fwd(x.device.index, _stream(), _lib.dtype_code(x.dtype), tokens,
                                            num_groups, D, x2.data_ptr(), _lib.ptr(g2), w32.data_ptr(),
                                            float(eps), y.data_ptr(), rstd.data_ptr()), "fox_normgate_fwd")
        ctx.save_for_backward(x2, g2, w32, rstd)
        ctx.shape = shape
        ctx.num_groups = num_groups
        ctx.w_dtype = weight.dtype
        return y.reshape(shape)

    @staticmethod
    def backward(ctx, dy):
        x2, g2, w32, rstd = ctx.saved_tensors
        hidden = x2.shape[-1]
        G = ctx.num_groups
        D = hidden // G
        tokens = x2.shape[0]
        lib = _lib.load()
        with torch.cuda.device(x2.device):
            dy2 = dy.reshape(-1, hidden).contiguous()
            dx = torch.empty_like(x2)
            dg = None if g2 is None else torch.empty_like(g2)
            n_part = min(tokens, _MAX_PARTIALS)
            dw_partial = torch.empty((n_part, hidden), dtype=torch.float32, device=x2.device)
            _lib.check(lib.fox_normgate_bwd(x2.device.index, _stream(), _lib.dtype_code(x2.dtype), tokens, G, D,
                                            x2.data_ptr(), _lib.ptr(g2), w32.data_ptr(), rstd.data_ptr(),
                                            dy2.data_ptr(), dx.data_ptr(), _lib.ptr(dg), dw_partial.data_ptr(),
                                            n_part), "fox_normgate_bwd")
            dw = dw_partial.sum(0).to(ctx.w_dtype)
        return dx.reshape(ctx.shape), None if dg is None else dg.reshape(ctx.shape), dw, None, None


def group_norm_gated(x, g, weight, bias=None, activation: str = "swish", residual=None, eps: float = 1e-5,
                     prenorm: bool = False, residual_in_fp32: bool = False, is_rms_norm: bool = False,
                     num_groups: int = 1):
    """Same argument list as upstream's ``group_norm_gated`` (fuse_norm_gate.py:977-1002)."""
    if bias is not None or residual is not None or prenorm or not is_rms_norm or activation != "sigmoid":
        raise NotImplementedError(
            "only the FoX-Pro configuration is built: is_rms_norm=True, activation='sigmoid', "
            "no bias, no residual, prenorm=False")
    if weight is None:
        raise NotImplementedError("elementwise_affine=False is not built")
    return GroupRMSNormSigmoidGate.apply(x, g, weight, num_groups, eps)


class FusedGroupNormGated(nn.Module):
    """Drop-in for upstream's module of the same name (fuse_norm_gate.py:1389-1461)."""

    def __init__(self, num_groups: int, hidden_size: int, elementwise_affine: bool = True, eps: float = 1e-5,
                 is_rms_norm: bool = False, activation: str = "swish", device=None, dtype=None):
        super().__init__()
        if hidden_size % num_groups != 0:
            raise ValueError("num_channels must be divisible by num_groups")
        if activation not in ["swish", "silu", "sigmoid"]:
            raise ValueError(f"Unsupported activation: {activation}")
        self.num_groups = num_groups
        self.hidden_size = hidden_size
        self.elementwise_affine = elementwise_affine
        self.eps = eps
        self.activation = activation
        self.is_rms_norm = is_rms_norm
        if elementwise_affine:
            self.weight = nn.Parameter(torch.empty(hidden_size, device=device, dtype=dtype))
        else:
            self.register_parameter("weight", None)
        self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self):
        if self.elementwise_affine:
            nn.init.ones_(self.weight)

    def extra_repr(self) -> str:
        return (f"{self.num_groups}, {self.hidden_size}, is_rms_norm={self.is_rms_norm}, eps={self.eps}, "
                f"activation={self.activation}")

    def forward(self, x: torch.Tensor, g: torch.Tensor, residual: Optional[torch.Tensor] = None,
                prenorm: bool = False, residual_in_fp32: bool = False) -> torch.Tensor:
        return group_norm_gated(x, g, self.weight, self.bias, self.activation, residual=residual, eps=self.eps,
                                prenorm=prenorm, residual_in_fp32=residual_in_fp32,
                                is_rms_norm=self.is_rms_norm, num_groups=self.num_groups)


def group_norm(x, weight, bias=None, residual=None, eps: float = 1e-5, prenorm: bool = False,
               residual_in_fp32: bool = False, is_rms_norm: bool = False, num_groups: int = 1):
    """Same argument list as upstream's ``group_norm`` / ``group_norm_fn`` (layernorm.py:706-792):
    the FoX layer's QK-norm is ``is_rms_norm=True`` with a weight and nothing else."""
    if bias is not None or residual is not None or prenorm or not is_rms_norm:
        raise NotImplementedError(
            "only the QK-norm configuration is built: is_rms_norm=True, no bias, no residual, prenorm=False")
    if weight is None:
        raise NotImplementedError("elementwise_affine=False is not built")
    return GroupRMSNormSigmoidGate.apply(x, None, weight, num_groups, eps)


class GroupNorm(nn.Module):
    """Drop-in for upstream's ``GroupNorm`` (layernorm.py:993-1051) as the FoX layer builds it for
    q and k (modeling_forgetting_transformer.py:264-265): per-head RMSNorm with a weight."""

    def __init__(self, num_groups: int, hidden_size: int, elementwise_affine: bool = True, bias: bool = False,
                 eps: float = 1e-5, is_rms_norm: bool = False, device=None, dtype=None):
        super().__init__()
        if hidden_size % num_groups != 0:
            raise ValueError("num_channels must be divisible by num_groups")
        if bias:
            raise NotImplementedError("bias=True is not built")
        self.num_groups = num_groups
        self.hidden_size = hidden_size
        self.elementwise_affine = elementwise_affine
        self.eps = eps
        self.is_rms_norm = is_rms_norm
        if elementwise_affine:
            self.weight = nn.Parameter(torch.empty(hidden_size, device=device, dtype=dtype))
        else:
            self.register_parameter("weight", None)
        self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self):
        if self.elementwise_affine:
            nn.init.ones_(self.weight)

    def extra_repr(self) -> str:
        return f"{self.num_groups}, {self.hidden_size}, is_rms_norm={self.is_rms_norm}, eps={self.eps}"

    def forward(self, x, residual=None, prenorm=False, residual_in_fp32=False):
        return group_norm(x, self.weight, self.bias, residual=residual, eps=self.eps, prenorm=prenorm,
                          residual_in_fp32=residual_in_fp32, is_rms_norm=self.is_rms_norm,
                          num_groups=self.num_groups)


class RowRMSNorm(torch.autograd.Function):
    """y = rmsnorm(x + residual) * weight over the last axis, optionally also returning the sum
    (prenorm); upstream's LayerNormFunction with is_rms_norm=True (layernorm.py:523-620)."""

    @staticmethod
    def forward(ctx, x, weight, residual, eps, prenorm):
        if not x.is_cuda:
            raise _lib.FoxError("rms_norm needs CUDA tensors on an sm_100 device; there is no CPU path")
        assert x.dtype in (torch.float16, torch.bfloat16)
        hidden = x.shape[-1]
        assert weight.shape == (hidden,)
        assert residual is None or (residual.shape == x.shape and residual.dtype == x.dtype)
        lib = _lib.load()
        shape = x.shape
        with torch.cuda.device(x.device):
            x2 = x.reshape(-1, hidden).contiguous()
            r2 = None if residual is None else residual.reshape(-1, hidden).contiguous()
            w32 = weight.detach().float().contiguous()
            rows = x2.shape[0]
            y = torch.empty_like(x2)
            z = None if r2 is None else torch.empty_like(x2)   # residual_out; without a residual z is x itself
            rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
            _lib.check(lib.fox_rmsnorm_fwd(x.device.index, _stream(), _lib.dtype_code(x.dtype), rows, hidden,
                                           x2.data_ptr(), _lib.ptr(r2), w32.data_ptr(), float(eps), y.data_ptr(),
                                           _lib.ptr(z), rstd.data_ptr()), "fox_rmsnorm_fwd")
        zs = x2 if z is None else z
        ctx.save_for_backward(zs, w32, rstd)
        ctx.shape, ctx.w_dtype = shape, weight.dtype
        ctx.has_residual, ctx.prenorm = residual is not None, prenorm
        y = y.reshape(shape)
        if not prenorm:
            return y
        return y, zs.reshape(shape)

    @staticmethod
    def backward(ctx, dy, *args):
        zs, w32, rstd = ctx.saved_tensors
        rows, hidden = zs.shape
        lib = _lib.load()
        dres_in = args[0] if (ctx.prenorm and len(args) > 0) else None
        with torch.cuda.device(zs.device):
            dy2 = dy.reshape(-1, hidden).contiguous()
            dr2 = None if dres_in is None else dres_in.reshape(-1, hidden).to(zs.dtype).contiguous()
            dx = torch.empty_like(zs)
            n_part = min((rows + 7) // 8, _MAX_PARTIALS)
            dw_partial = torch.empty((n_part, hidden), dtype=torch.float32, device=zs.device)
            _lib.check(lib.fox_rmsnorm_bwd(zs.device.index, _stream(), _lib.dtype_code(zs.dtype), rows, hidden,
                                           zs.data_ptr(), w32.data_ptr(), rstd.data_ptr(), dy2.data_ptr(),
                                           _lib.ptr(dr2), dx.data_ptr(), dw_partial.data_ptr(), n_part),
                       "fox_rmsnorm_bwd")
            dw = dw_partial.sum(0).to(ctx.w_dtype)
        dx = dx.reshape(ctx.shape)
        return dx, dw, (dx if ctx.has_residual else None), None, None


def rms_norm(x, weight, bias=None, residual=None, eps: float = 1e-5, prenorm: bool = False,
             residual_in_fp32: bool = False):
    """Same argument list as upstream's ``rms_norm`` (layernorm.py:841-859)."""
    if bias is not None or residual_in_fp32:
        raise NotImplementedError("only the FoX block's configuration is built: no bias, residual in the input dtype")
    if weight is None:
        raise NotImplementedError("elementwise_affine=False is not built")
    return RowRMSNorm.apply(x, weight, residual, eps, prenorm)


class RMSNorm(nn.Module):
    """Drop-in for upstream's ``RMSNorm`` (layernorm.py:1054-1101) as the FoX block builds it
    (attn_norm, mlp_norm: a weight, no bias)."""

    def __init__(self, hidden_size: int, elementwise_affine: bool = True, bias: bool = False, eps: float = 1e-5,
                 device=None, dtype=None):
        super().__init__()
        if bias:
            raise NotImplementedError("bias=True is not built")
        self.hidden_size = hidden_size
        self.elementwise_affine = elementwise_affine
        self.eps = eps
        if elementwise_affine:
            self.weight = nn.Parameter(torch.empty(hidden_size, device=device, dtype=dtype))
        else:
            self.register_parameter("weight", None)
        self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self):
        if self.elementwise_affine:
            nn.init.ones_(self.weight)

    def extra_repr(self) -> str:
        return f"{self.hidden_size}, eps={self.eps}"

    def forward(self, x, residual=None, prenorm=False, residual_in_fp32=False):
        return rms_norm(x, self.weight, self.bias, residual=residual, eps=self.eps, prenorm=prenorm,
                        residual_in_fp32=residual_in_fp32)
