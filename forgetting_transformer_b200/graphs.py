"""CUDA-graph capture of the operator's forward and backward for launch-bound shapes.

A step of ``forgetting_attention`` at small sizes (B4 T512 H12 D64: ~0.29 ms) is 8-10 kernel launches
whose device time is a fraction of their launch cost.  Every entry point of the library launches on the
caller's current stream, allocates nothing and never synchronises, and the cached TMA descriptors are keyed
by (pointer, shape, strides), so a step can be captured once and replayed: ``make_graphed`` wraps
``torch.cuda.make_graphed_callables`` (static input / output buffers, one graph for the forward and one
for the backward) around the operator with its keyword arguments bound.
"""
from __future__ import annotations

from typing import Callable, Optional, Union

import torch

from .ops import forgetting_attention

__all__ = ["make_graphed"]


def make_graphed(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, log_fgate: torch.Tensor, *,
                 head_first: bool = False, seq_start: Optional[torch.Tensor] = None,
                 sm_scale: Optional[float] = None,
                 adaptive_threshold: Optional[Union[str, float, torch.Tensor]] = None,
                 num_warmup_iters: int = 3) -> Callable:
    """Returns ``f(q, k, v, log_fgate) -> out`` with the same autograd contract as ``forgetting_attention``
    for tensors of exactly the sample arguments' shapes, dtypes and ``requires_grad`` flags, replayed from CUDA
    graphs.  ``seq_start`` and a tensor ``adaptive_threshold`` are captured by reference: update them in place
    between calls.  The sample tensors are only used for warm-up and capture."""
    assert q.is_cuda, "CUDA graphs need CUDA tensors"

    def op(q_, k_, v_, lf_):
        return forgetting_attention(q_, k_, v_, lf_, head_first=head_first, seq_start=seq_start, sm_scale=sm_scale,
                                    adaptive_threshold=adaptive_threshold)

    return torch.cuda.make_graphed_callables(op, (q, k, v, log_fgate), num_warmup_iters=num_warmup_iters)
