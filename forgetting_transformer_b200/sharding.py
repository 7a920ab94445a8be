"""Multi-GPU partitioning of the Forgetting Attention hot path (one process per GPU,
``torch.distributed``; NCCL on GPUs, gloo in the CPU tests).

Two schemes, neither present upstream (which only knows data-parallel training):

* batch x head sharding -- every (batch, head) unit is independent in forward and
  backward (they are grid axes of every upstream kernel,
  src/forgetting_transformer/ops/forgetting_attention.py:186, 313, 366), so a rank takes a
  contiguous slice of the flattened units and no collective touches the data path.

* context parallel for long sequences -- the sequence is cut into 2P chunks and rank r owns
  chunks r and 2P-1-r ("zig-zag": causal work is balanced).  Keys, values and log gates are
  all-gathered once; each rank then calls the ordinary operator on its query chunk against the
  key prefix that chunk may attend to -- exactly the operator's ``seqlen_q <= seqlen_k``
  contract (queries are the last rows) -- and the gradients of the gathered tensors are
  reduce-scattered back to their owners.  Rows are complete on their owner, so no partial
  (max, sum, out) triples have to travel; the log-gate prefix is recomputed from the gathered
  gates by the operator's own prefix-sum kernel.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

__all__ = ["unit_slice", "shard_batch_heads", "zigzag_chunks", "ContextParallelAttention",
           "context_parallel_attention"]


# ----------------------------------------------------------------------------- batch x head
def unit_slice(n_units: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous [begin, end) of ``n_units`` flattened (batch, head) units owned by ``rank``;
    the first ``n_units % world`` ranks get one extra unit."""
    base, extra = divmod(n_units, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_batch_heads(q, k, v, log_fgate, seq_start=None, adaptive_threshold=None, *, world: int, rank: int):
    """Views of this rank's units of head-first tensors, reshaped to (units, 1, T, D) /
    (units, 1, T) so the unchanged operator can run on them; ``seq_start`` and a tensor
    threshold are expanded per unit.  No copies for contiguous inputs."""
    B, H, M, D = q.shape
    N = k.shape[2]
    u0, u1 = unit_slice(B * H, world, rank)
    qs = q.reshape(B * H, 1, M, D)[u0:u1]
    ks = k.reshape(B * H, 1, N, D)[u0:u1]
    vs = v.reshape(B * H, 1, N, D)[u0:u1]
    ls = log_fgate.reshape(B * H, 1, N)[u0:u1]
    ss = None
    if seq_start is not None:
        ss = seq_start.repeat_interleave(H)[u0:u1]
    thr = adaptive_threshold
    if isinstance(thr, torch.Tensor):
        thr = torch.broadcast_to(thr, (B, H)).reshape(B * H, 1)[u0:u1]
    return qs, ks, vs, ls, ss, thr


# --------------------------------------------------------------------------- context parallel
def zigzag_chunks(world: int, rank: int) -> Tuple[int, int]:
    """The two of 2*world equal sequence chunks owned by ``rank``."""
    return rank, 2 * world - 1 - rank


class _GatherSeq(torch.autograd.Function):
    """All-gather along the sequence axis in zig-zag chunk order -> full sequence in natural
    order; backward reduce-scatters (sums) the gradient back to the chunk owners."""

    @staticmethod
    def forward(ctx, local: torch.Tensor, seq_dim: int, group):
        world = dist.get_world_size(group)
        rank = dist.get_rank(group)
        ctx.seq_dim, ctx.group, ctx.world, ctx.rank = seq_dim, group, world, rank
        local = local.contiguous()
        parts = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(parts, local, group=group)
        tc = local.shape[seq_dim] // 2
        chunks: List[Optional[torch.Tensor]] = [None] * (2 * world)
        for r, p in enumerate(parts):
            a, b = zigzag_chunks(world, r)
            chunks[a] = p.narrow(seq_dim, 0, tc)
            chunks[b] = p.narrow(seq_dim, tc, tc)
        return torch.cat(chunks, dim=seq_dim)

    @staticmethod
    def backward(ctx, grad_full: torch.Tensor):
        world, seq_dim = ctx.world, ctx.seq_dim
        tc = grad_full.shape[seq_dim] // (2 * world)
        inputs = []
        for r in range(world):
            a, b = zigzag_chunks(world, r)
            inputs.append(torch.cat([grad_full.narrow(seq_dim, a * tc, tc), grad_full.narrow(seq_dim, b * tc, tc)],
                                    dim=seq_dim).contiguous())
        out = torch.empty_like(inputs[ctx.rank])
        dist.reduce_scatter(out, inputs, op=dist.ReduceOp.SUM, group=ctx.group)
        return out, None, None


def _reduce_scatter_fallback(out, inputs, group):  # gloo has no reduce_scatter: all_reduce + pick
    stacked = torch.stack(inputs)
    dist.all_reduce(stacked, group=group)
    out.copy_(stacked[dist.get_rank(group)])


class _GatherSeqGloo(_GatherSeq):
    @staticmethod
    def backward(ctx, grad_full: torch.Tensor):
        world, seq_dim = ctx.world, ctx.seq_dim
        tc = grad_full.shape[seq_dim] // (2 * world)
        inputs = []
        for r in range(world):
            a, b = zigzag_chunks(world, r)
            inputs.append(torch.cat([grad_full.narrow(seq_dim, a * tc, tc), grad_full.narrow(seq_dim, b * tc, tc)],
                                    dim=seq_dim).contiguous())
        out = torch.empty_like(inputs[ctx.rank])
        _reduce_scatter_fallback(out, inputs, ctx.group)
        return out, None, None


def context_parallel_attention(q, k, v, log_fgate, *, group=None, sm_scale: Optional[float] = None,
                               adaptive_threshold=None, attn_fn: Optional[Callable] = None):
    """Head-first forgetting attention over a sequence sharded in zig-zag chunks.

    Every rank passes its local shard: q, k, v (B, H, 2*Tc, D) and log_fgate (B, H, 2*Tc), the
    concatenation of its two chunks (``zigzag_chunks``) of a sequence of length 2*world*Tc.
    Returns the local shard of the output, same layout; differentiable (gradients of k, v and
    log_fgate are summed over ranks and returned to the owners).  ``seq_start`` is not supported
    here (left padding belongs to the first chunk only; pad on the host instead).

    ``attn_fn(q, k, v, log_fgate, head_first=True, sm_scale=..., adaptive_threshold=...)``
    defaults to the CUDA operator; the CPU tests inject the oracle.
    """
    if attn_fn is None:
        from .ops import forgetting_attention as attn_fn
    group = group if group is not None else dist.group.WORLD
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    gather = _GatherSeqGloo if dist.get_backend(group) == "gloo" else _GatherSeq
    tc = q.shape[2] // 2
    assert q.shape[2] == 2 * tc and k.shape[2] == 2 * tc and log_fgate.shape[2] == 2 * tc
    k_full = gather.apply(k, 2, group)
    v_full = gather.apply(v, 2, group)
    lf_full = gather.apply(log_fgate, 2, group)
    outs = []
    for idx, chunk in enumerate(zigzag_chunks(world, rank)):
        n = (chunk + 1) * tc  # keys this chunk may see: everything up to and including itself
        outs.append(attn_fn(q[:, :, idx * tc:(idx + 1) * tc], k_full[:, :, :n], v_full[:, :, :n],
                            lf_full[:, :, :n], head_first=True, sm_scale=sm_scale,
                            adaptive_threshold=adaptive_threshold))
    return torch.cat(outs, dim=2)


class ContextParallelAttention(torch.nn.Module):
    """Module form of :func:`context_parallel_attention` bound to a process group."""

    def __init__(self, group=None, attn_fn: Optional[Callable] = None):
        super().__init__()
        self.group, self.attn_fn = group, attn_fn

    def forward(self, q, k, v, log_fgate, sm_scale=None, adaptive_threshold=None):
        return context_parallel_attention(q, k, v, log_fgate, group=self.group, sm_scale=sm_scale,
                                          adaptive_threshold=adaptive_threshold, attn_fn=self.attn_fn)
