"""Fused cross-entropy loss backed by the sm_100a kernels.

Host-side mirror of upstream's ``CrossEntropyLossFunction`` / ``cross_entropy_loss`` / ``FusedCrossEntropyLoss``
(src/forgetting_transformer/model/forgetting_transformer/fused_cross_entropy.py:137-401): same arguments,
defaults and returned (losses, z_losses), label smoothing, logit scale, z-loss, ``ignore_index`` and the
in-place backward the model's loss uses (modeling_forgetting_transformer.py:877-884).  With ``process_group`` the
classes are split over the group's ranks (upstream lines 150-151, 196-226): every rank passes its own (rows,
classes / world) slice of the logits and the full targets; the ranks' log-sum-exps are all-gathered and joined, the
loss parts all-reduced.  No CPU path.
"""
from __future__ import annotations

from typing import Any, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from . import _lib

__all__ = ["cross_entropy_loss", "CrossEntropyLossFunction", "FusedCrossEntropyLoss"]

_DTYPES = {torch.float16: _lib.FOX_DTYPE_FP16, torch.bfloat16: _lib.FOX_DTYPE_BF16, torch.float32: _lib.FOX_DTYPE_FP32}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _local_forward(logits, target, label_smoothing, logit_scale, lse_square_scale, ignore_index, total_classes,
                   class_start, split):
    """One rank's kernel launch: (losses or loss parts, z_losses or None, lse of this rank's classes)."""
    n_rows, n_cols = logits.shape
    lib = _lib.load()
    dev = logits.device
    with torch.cuda.device(dev):
        losses = torch.empty(n_rows, dtype=torch.float32, device=dev)
        lse = torch.empty(n_rows, dtype=torch.float32, device=dev)
        if split:
            _lib.check(lib.fox_cross_entropy_fwd_split(dev.index, _stream(), _DTYPES[logits.dtype], n_rows, n_cols,
                                                       logits.data_ptr(), logits.stride(0), target.data_ptr(),
                                                       float(label_smoothing), float(logit_scale), int(ignore_index),
                                                       int(total_classes), int(class_start), losses.data_ptr(),
                                                       lse.data_ptr()), "fox_cross_entropy_fwd_split")
            return losses, None, lse
        z_losses = torch.empty(n_rows, dtype=torch.float32, device=dev)
        _lib.check(lib.fox_cross_entropy_fwd(dev.index, _stream(), _DTYPES[logits.dtype], n_rows, n_cols,
                                             logits.data_ptr(), logits.stride(0), target.data_ptr(),
                                             float(label_smoothing), float(logit_scale), float(lse_square_scale),
                                             int(ignore_index), losses.data_ptr(), z_losses.data_ptr(),
                                             lse.data_ptr()), "fox_cross_entropy_fwd")
    return losses, z_losses, lse


def _local_backward(logits, target, lse, grad_losses, label_smoothing, logit_scale, lse_square_scale, ignore_index,
                    total_classes, class_start, dlogits):
    n_rows, n_cols = logits.shape
    lib = _lib.load()
    dev = logits.device
    with torch.cuda.device(dev):
        _lib.check(lib.fox_cross_entropy_bwd_split(dev.index, _stream(), _DTYPES[logits.dtype], n_rows, n_cols,
                                                   logits.data_ptr(), logits.stride(0), target.data_ptr(),
                                                   lse.data_ptr(), grad_losses.data_ptr(), grad_losses.stride(0),
                                                   label_smoothing, logit_scale, lse_square_scale, ignore_index,
                                                   int(total_classes), int(class_start), dlogits.data_ptr(),
                                                   dlogits.stride(0)), "fox_cross_entropy_bwd_split")
    return dlogits


def join_class_shards(loss_parts, lse_local, target, lse_square_scale, ignore_index, process_group):
    """Global (losses, z_losses, lse) from every rank's loss parts and local log-sum-exp (upstream lines 206-226)."""
    world = dist.get_world_size(process_group)
    gathered = torch.empty((world,) + tuple(lse_local.shape), dtype=lse_local.dtype, device=lse_local.device)
    dist.all_gather_into_tensor(gathered.view(-1), lse_local.contiguous(), group=process_group)
    handle = dist.all_reduce(loss_parts, op=dist.ReduceOp.SUM, group=process_group, async_op=True)
    lse = torch.logsumexp(gathered, dim=0)
    handle.wait()
    losses = loss_parts + lse
    if lse_square_scale != 0.0:
        z_losses = lse_square_scale * lse.square()
        z_losses.masked_fill_(target == ignore_index, 0.0)
        losses = losses + z_losses
    else:
        z_losses = torch.zeros_like(losses)
    losses.masked_fill_(target == ignore_index, 0.0)
    return losses, z_losses, lse


class CrossEntropyLossFunction(torch.autograd.Function):

    @staticmethod
    def forward(ctx, logits, target, label_smoothing=0.0, logit_scale=1.0, lse_square_scale=0.0, ignore_index=-100,
                inplace_backward=False, process_group=None):
        if not logits.is_cuda:
            raise _lib.FoxError("cross_entropy_loss needs CUDA tensors on an sm_100 device; there is no CPU path")
        n_rows, n_cols = logits.shape
        assert target.shape == (n_rows,)
        if logits.dtype not in _DTYPES:
            raise _lib.FoxError(f"unsupported logits dtype {logits.dtype}")
        world = 1 if process_group is None else dist.get_world_size(process_group)
        rank = 0 if process_group is None else dist.get_rank(process_group)
        total_classes, class_start = world * n_cols, rank * n_cols
        es = logits.element_size()
        if logits.stride(-1) != 1 or (logits.stride(0) * es) % 16 or logits.data_ptr() % 16:
            logits = logits.contiguous()
            if (logits.stride(0) * es) % 16:     # a class count whose rows cannot all start on 16 bytes: pad the stride
                pad = torch.empty((n_rows, -(-n_cols * es // 16) * 16 // es), dtype=logits.dtype, device=logits.device)
                pad[:, :n_cols] = logits
                logits = pad[:, :n_cols]
        target = target.to(torch.long).contiguous()
        losses, z_losses, lse = _local_forward(logits, target, label_smoothing, logit_scale, lse_square_scale,
                                               ignore_index, total_classes, class_start, world > 1)
        if world > 1:
            losses, z_losses, lse = join_class_shards(losses, lse, target, float(lse_square_scale), int(ignore_index),
                                                      process_group)
        ctx.save_for_backward(logits, lse, target)
        ctx.mark_non_differentiable(z_losses)
        ctx.args = (float(label_smoothing), float(logit_scale), float(lse_square_scale), int(ignore_index))
        ctx.classes = (total_classes, class_start)
        ctx.inplace_backward = inplace_backward
        return losses, z_losses

    @staticmethod
    def backward(ctx, grad_losses, grad_z_losses):
        del grad_z_losses  # z_losses are for logging only, as upstream
        logits, lse, target = ctx.saved_tensors
        label_smoothing, logit_scale, lse_square_scale, ignore_index = ctx.args
        # (same row stride as the saved logits: a re-laid class count keeps its 16-byte aligned rows)
        dlogits = logits if ctx.inplace_backward else torch.empty_strided(logits.shape, logits.stride(),
                                                                          dtype=logits.dtype, device=logits.device)
        _local_backward(logits, target, lse, grad_losses.float(), label_smoothing, logit_scale, lse_square_scale,
                        ignore_index, ctx.classes[0], ctx.classes[1], dlogits)
        return dlogits, None, None, None, None, None, None, None


def cross_entropy_loss(logits: torch.Tensor, target: torch.Tensor, label_smoothing: float = 0.0,
                       logit_scale: float = 1.0, lse_square_scale: float = 0.0, ignore_index=-100,
                       inplace_backward: bool = False, process_group=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """logits (rows, classes), target (rows,) -> (losses, z_losses), both fp32 (rows,); see upstream lines 275-312."""
    return CrossEntropyLossFunction.apply(logits, target, label_smoothing, logit_scale, lse_square_scale, ignore_index,
                                          inplace_backward, process_group)


class FusedCrossEntropyLoss(nn.Module):
    """Same constructor and forward contract as upstream's module (lines 315-401)."""

    def __init__(self, ignore_index: int = -100, reduction: str = "mean", label_smoothing: float = 0.0,
                 logit_scale: float = 1.0, lse_square_scale: float = 0.0, inplace_backward: bool = False,
                 process_group: Any = None, return_z_loss: bool = False):
        super().__init__()
        if reduction not in ["mean", "none", "sum"]:
            raise NotImplementedError("Only support reduction = 'mean' or 'none' or 'sum'")
        self.ignore_index = ignore_index
        self.reduction = reduction
        self.label_smoothing = label_smoothing
        self.logit_scale = logit_scale
        self.lse_square_scale = lse_square_scale
        self.inplace_backward = inplace_backward
        self.process_group = process_group
        self.return_z_loss = return_z_loss

    def forward(self, input, target):
        assert input.is_cuda and target.is_cuda, "Only support CUDA tensors"
        loss, z_loss = cross_entropy_loss(input, target, label_smoothing=self.label_smoothing,
                                          logit_scale=self.logit_scale, lse_square_scale=self.lse_square_scale,
                                          ignore_index=self.ignore_index, inplace_backward=self.inplace_backward,
                                          process_group=self.process_group)
        if self.reduction == "mean":
            loss = loss.sum() / (target != self.ignore_index).sum()
        elif self.reduction == "sum":
            loss = loss.sum()
        if not self.return_z_loss:
            return loss
        if self.reduction == "mean":
            z_loss = z_loss.sum() / (target != self.ignore_index).sum()
        elif self.reduction == "sum":
            z_loss = z_loss.sum()
        return loss, z_loss
