"""Data-dependent token shift of the FoX-Pro key/value projections.

Host-side mirror of upstream's ``token_shift`` / ``TokenShift``
(src/forgetting_transformer/model/forgetting_transformer/token_shift.py:161-238), which
``ShiftLinear`` calls as ``token_shift(out_per_head, alpha, 1 - alpha)``
(modeling_forgetting_transformer.py:82):

    out[b, t, h, :] = x[b, t, h, :] * curr_weight[b, t, h] + x[b, t-1, h, :] * prev_weight[b, t, h]
"""
from __future__ import annotations

import torch

from . import _lib

__all__ = ["token_shift", "TokenShift"]


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _rows16(x: torch.Tensor) -> torch.Tensor:
    """A view the kernels can read: unit stride on D, 16-byte rows and base; else a packed copy."""
    ok = (x.stride(-1) == 1 and x.data_ptr() % 16 == 0 and all(s % 8 == 0 for s in x.stride()[:-1]))
    return x if ok else x.contiguous()


class TokenShift(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x: torch.Tensor, prev_weight: torch.Tensor, curr_weight: torch.Tensor):
        B, T, H, D = x.size()
        assert D in {16, 32, 64, 128}
        assert prev_weight.size() == curr_weight.size() == (B, T, H)
        if not x.is_cuda:
            raise _lib.FoxError("token_shift needs CUDA tensors on an sm_100 device; there is no CPU path")
        assert x.dtype in (torch.float16, torch.bfloat16), "token_shift is built for 16-bit activations"
        lib = _lib.load()
        w_dtype = prev_weight.dtype
        with torch.cuda.device(x.device):
            x = _rows16(x)
            pw = prev_weight.float()
            cw = curr_weight.float()
            if pw.stride() != cw.stride():
                pw, cw = pw.contiguous(), cw.contiguous()
            out = torch.empty_like(x)
            if out.stride() != x.stride():
                out = torch.empty_strided(x.size(), x.stride(), dtype=x.dtype, device=x.device)
            _lib.check(lib.fox_token_shift_fwd(x.device.index, _stream(), _lib.dtype_code(x.dtype), B, T, H, D,
                                               x.data_ptr(), x.stride(0), x.stride(1), x.stride(2), pw.data_ptr(),
                                               cw.data_ptr(), cw.stride(0), cw.stride(1), cw.stride(2),
                                               out.data_ptr()), "fox_token_shift_fwd")
        ctx.save_for_backward(x, pw, cw)
        ctx.w_dtype = w_dtype
        return out

    @staticmethod
    def backward(ctx, dout: torch.Tensor):
        x, pw, cw = ctx.saved_tensors
        B, T, H, D = x.size()
        lib = _lib.load()
        with torch.cuda.device(x.device):
            if dout.stride() != x.stride() or dout.data_ptr() % 16:
                d2 = torch.empty_strided(x.size(), x.stride(), dtype=x.dtype, device=x.device)
                d2.copy_(dout)
                dout = d2
            dx = torch.empty_strided(x.size(), x.stride(), dtype=x.dtype, device=x.device)
            dprev = torch.empty_strided(cw.size(), cw.stride(), dtype=torch.float32, device=x.device)
            dcurr = torch.empty_strided(cw.size(), cw.stride(), dtype=torch.float32, device=x.device)
            _lib.check(lib.fox_token_shift_bwd(x.device.index, _stream(), _lib.dtype_code(x.dtype), B, T, H, D,
                                               x.data_ptr(), x.stride(0), x.stride(1), x.stride(2), pw.data_ptr(),
                                               cw.data_ptr(), cw.stride(0), cw.stride(1), cw.stride(2),
                                               dout.data_ptr(), dx.data_ptr(), dprev.data_ptr(), dcurr.data_ptr()),
                       "fox_token_shift_bwd")
        return dx, dprev.to(ctx.w_dtype), dcurr.to(ctx.w_dtype)


def token_shift(x, prev_weight, curr_weight):
    """Same call as upstream's ``token_shift`` (token_shift.py:237-238): x (B, T, H, D) in
    fp16/bf16, weights (B, T, H); differentiable in all three."""
    return TokenShift.apply(x, prev_weight, curr_weight)
