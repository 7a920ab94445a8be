"""Multi-GPU partitioning of the Forgetting Attention hot path (one process per GPU,
``torch.distributed``; NCCL on GPUs, gloo in the CPU tests).

Two schemes, neither present upstream (which only knows data-parallel training):

* batch x head sharding -- every (batch, head) unit is independent in forward and
  backward (they are grid axes of every upstream kernel,
  src/forgetting_transformer/ops/forgetting_attention.py:186, 313, 366), so a rank takes a
  contiguous slice of the flattened units and no collective touches the data path.

* context parallel for long sequences -- the sequence is cut into 2P chunks and rank r owns
  chunks r and 2P-1-r ("zig-zag": causal work is balanced).  Keys, values and log gates land in a
  sequence-major staging buffer (T', B, H, D) in two waves: the lower halves (chunks 0..P-1, one per rank,
  already in sequence order) by one all-gather per tensor, after which a rank's lower query chunk can already
  run, and the upper halves a rank may attend to (chunks P..2P-1-r), which travel while that first call
  computes -- point to point (batched NCCL sends / receives; causality halves this traffic) or as a second
  all-gather (``UPPER_EXCHANGE``).  Each query chunk is one call of the ordinary operator against the key prefix
  it may attend to -- exactly the operator's ``seqlen_q <= seqlen_k`` contract (queries are the last rows),
  reading the staging buffer through strided views, no reordering copies.  Rows are complete on their owner, so
  no partial (max, sum, out) triples have to travel; the log-gate prefix is recomputed from the gathered gates by
  the operator's own prefix-sum kernel.  Backward: both calls, then the partial key / value / gate gradients of
  the lower halves are reduce-scattered as they lie and those of the upper halves are sent to the chunk's owner,
  who sums in fp32.  The collectives run on a high-priority NCCL stream (``context_parallel_group``) so that they
  are not queued behind the attention kernels' thousands of CTAs.  Tiles are only ever read from this GPU's own
  memory.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

__all__ = ["unit_slice", "shard_batch_heads", "zigzag_chunks", "ContextParallelAttention",
           "context_parallel_attention", "context_parallel_threshold", "context_parallel_group"]


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


def _wait(work):
    if work is not None:
        work.wait()


# Optional stopwatch for the phases of a context-parallel step: when set to a list, (label, CUDA event) pairs are
# appended at the phase boundaries on the current stream (benchmark / profiling scripts read them back).
PHASE_TRACE = None


def _mark(label: str) -> None:
    if PHASE_TRACE is not None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        PHASE_TRACE.append((label, ev))


def _head_first(x: torch.Tensor) -> torch.Tensor:
    """View of a sequence-major (t, B, H, ...) buffer as (B, H, t, ...)."""
    return x.movedim(0, 2)


def context_parallel_group(ranks: Optional[Sequence[int]] = None, high_priority: bool = True):
    """A process group for :func:`context_parallel_attention` whose NCCL kernels run on a high-priority stream.

    The second wave of gathers and the first reduce-scatter travel while an attention kernel occupies every SM;
    on a stream of default priority the collective's few thread blocks queue behind thousands of attention
    blocks and a 0.3 ms transfer takes 3 ms (measured on two B200s).  With a high-priority stream they take
    the next SMs that become free.  Falls back to an ordinary group for other backends (gloo in the CPU tests).
    Collective call: every rank of the default group must call it."""
    if dist.get_backend() != "nccl":
        return dist.new_group(ranks=ranks)
    opts = dist.ProcessGroupNCCL.Options()
    opts.is_high_priority_stream = bool(high_priority)
    return dist.new_group(ranks=ranks, backend="nccl", pg_options=opts)


UPPER_EXCHANGE = None   # "p2p" | "collective"; None: $FOX_B200_CP_UPPER, else "p2p"


def _upper_half_mode(group) -> str:
    """How the upper halves travel: "p2p" (point to point, the causal subset only, straight into place) or
    "collective" (all-gather / reduce-scatter of all of them plus reordering copies).  Set
    ``sharding.UPPER_EXCHANGE`` (every rank alike) or FOX_B200_CP_UPPER; default p2p."""
    import os
    return UPPER_EXCHANGE or os.environ.get("FOX_B200_CP_UPPER", "p2p")


def _owner(chunk: int, world: int) -> int:
    """Rank that owns a chunk of the zig-zag split."""
    return chunk if chunk < world else 2 * world - 1 - chunk


def _exchange(ops_list):
    """Post a list of (kind, tensor, peer global rank, group) point-to-point operations as one batch; returns
    the requests to wait on.  Every tensor is a contiguous slab that is sent from / received into its final
    place, so nothing is reordered or copied around the transfer."""
    if not ops_list:
        return []
    return dist.batch_isend_irecv([dist.P2POp(dist.isend if kind == "send" else dist.irecv, t, peer, group)
                                   for kind, t, peer, group in ops_list])


class _ContextParallel(torch.autograd.Function):
    """Forward and backward of the zig-zag context-parallel attention as one autograd node, so that the
    transfers, the two operator calls per direction and their overlap are scheduled by hand.

    The lower halves (chunk j on rank j, needed by everyone) move by all-gather / reduce-scatter, which land
    them in natural order as they lie; the upper halves move point to point (one batched group of NCCL sends /
    receives), each slab straight between the staging buffer of its owner and of the ranks that attend to it --
    causality halves their traffic (rank r only ever sees chunks up to 2P-1-r)."""

    @staticmethod
    def forward(ctx, q, k, v, log_fgate, seq_start, sm_scale, threshold, group, attn_fn):
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        _mark("fwd begin")
        B, H, t2, D = q.shape
        tc = t2 // 2
        P = world
        T = 2 * P * tc
        lo_c, hi_c = zigzag_chunks(P, rank)
        n_lo, n_hi = (lo_c + 1) * tc, (hi_c + 1) * tc
        dev, dt = k.device, k.dtype
        peer = [dist.get_global_rank(group, j) for j in range(P)]
        # sequence-major staging of the keys this rank attends to: chunk j is the contiguous slab
        # [j*tc, (j+1)*tc); own chunks are copied in, the others received in place
        Kf = torch.empty((n_hi, B, H, D), dtype=dt, device=dev)
        Vf = torch.empty((n_hi, B, H, D), dtype=dt, device=dev)
        Gf = torch.empty((n_hi, B, H), dtype=log_fgate.dtype, device=dev)
        slab = lambda buf, c: buf.data[c * tc:(c + 1) * tc]     # (alias with its own version counter, see below)
        for buf, src in ((Kf, k), (Vf, v)):
            slab(buf, hi_c).copy_(src[:, :, tc:].movedim(2, 0))
        # wave 1: the lower halves -- chunk j < P lives on rank j and every rank attends to all of them, so an
        # all-gather lands them in natural order -- and the (small) gates of both halves;
        # wave 2: the upper halves this rank may attend to (chunks P .. hi_c, owned by the ranks above this one),
        # point to point
        k_lo, v_lo = k[:, :, :tc].movedim(2, 0).contiguous(), v[:, :, :tc].movedim(2, 0).contiguous()
        g_both = log_fgate.movedim(2, 0).contiguous().view(2, tc, B, H)
        g_all = torch.empty((P, 2, tc, B, H), dtype=log_fgate.dtype, device=dev)
        w1 = [dist.all_gather_into_tensor(g_all.view(P * 2, tc, B, H), g_both, group=group, async_op=True),
              dist.all_gather_into_tensor(Kf.data[:P * tc], k_lo, group=group, async_op=True),
              dist.all_gather_into_tensor(Vf.data[:P * tc], v_lo, group=group, async_op=True)]
        collective = _upper_half_mode(group) == "collective"
        wave2, w2, up = [], [], []
        if collective:
            # the upper halves by all-gather as well (every rank receives all of them, in rank order = reversed
            # chunk order); the slabs this rank attends to are copied into place afterwards
            for buf in (Kf, Vf):
                tmp = torch.empty((P * tc, B, H, D), dtype=dt, device=dev)
                w2.append(dist.all_gather_into_tensor(tmp, slab(buf, hi_c).clone(), group=group, async_op=True))
                up.append(tmp)
        else:
            for j in range(P):
                if j < rank:        # rank j attends to chunks up to 2P-1-j, which include this rank's upper chunk
                    for buf in (Kf, Vf):
                        wave2.append(("send", slab(buf, hi_c), peer[j], group))
                elif j > rank:      # and this rank to the upper chunk of every rank above it
                    for buf in (Kf, Vf):
                        wave2.append(("recv", slab(buf, 2 * P - 1 - j), peer[j], group))
        reqs2 = _exchange(wave2)

        def call(q_c, n):
            """The operator on one query chunk against keys [0, n), on views of the staging buffers."""
            leaves = [q_c.detach().requires_grad_(), _head_first(Kf[:n]).detach().requires_grad_(),
                      _head_first(Vf[:n]).detach().requires_grad_(), _head_first(Gf[:n]).detach().requires_grad_()]
            ss = None if seq_start is None else torch.clamp(seq_start, max=n)
            with torch.enable_grad():
                out = attn_fn(*leaves, head_first=True, seq_start=ss, sm_scale=sm_scale,
                              adaptive_threshold=threshold)
            return out, leaves

        _wait(w1[0])
        Gf.data[:P * tc].view(P, tc, B, H).copy_(g_all[:, 0])
        n_up = hi_c + 1 - P                                       # upper chunks P .. hi_c = ranks P-1 .. rank
        Gf.data[P * tc:].view(n_up, tc, B, H).copy_(g_all[rank:, 1].flip(0))
        _wait(w1[1])
        _wait(w1[2])
        _mark("lower halves gathered")
        out_lo, leaves_lo = call(q[:, :, :tc], n_lo)              # runs while wave 2 travels
        _mark("lower chunk forward")
        # (wave 2 lands in rows at and above P*tc of the same allocations, through aliases with their own version
        # counter: the lower call's saved views cover only rows below that, which stay as they are)
        for r_ in reqs2:
            r_.wait()
        for w, tmp, buf in zip(w2, up, (Kf, Vf)):
            _wait(w)
            buf.data[P * tc:].view(P - rank, tc, B, H, D).copy_(tmp.view(P, tc, B, H, D)[rank:].flip(0))
        _mark("upper halves gathered")
        out_hi, leaves_hi = call(q[:, :, tc:], n_hi)
        _mark("upper chunk forward")
        ctx.graph = (out_lo, leaves_lo, out_hi, leaves_hi)
        ctx.geom = (group, P, rank, B, H, D, tc)
        return torch.cat([out_lo.detach(), out_hi.detach()], dim=2)

    @staticmethod
    def backward(ctx, dout):
        out_lo, leaves_lo, out_hi, leaves_hi = ctx.graph
        group, P, rank, B, H, D, tc = ctx.geom
        ctx.graph = None
        lo_c, hi_c = zigzag_chunks(P, rank)
        n_lo = (lo_c + 1) * tc
        dev = dout.device
        collective = _upper_half_mode(group) == "collective"
        peer = [dist.get_global_rank(group, j) for j in range(P)]

        def seq_major_mem(g):
            """Gradient of a (B, H, n, ...) view of sequence-major memory, as (n, B, H, ...) contiguous."""
            g = g.movedim(2, 0)
            return g if g.is_contiguous() else g.contiguous()

        _mark("bwd begin")
        dq_hi, dk_hi, dv_hi, dg_hi = torch.autograd.grad(out_hi, leaves_hi, dout[:, :, tc:])
        _mark("upper chunk backward")
        dq_lo, dk_lo, dv_lo, dg_lo = torch.autograd.grad(out_lo, leaves_lo, dout[:, :, :tc])
        _mark("lower chunk backward")
        # Lower halves: chunk j belongs to rank j and every rank holds a partial for it: one reduce-scatter per
        # tensor over the first P slabs, as they lie.  Upper halves: rank r holds partials for chunks P .. 2P-1-r
        # only; each goes point to point from its slab to the chunk's owner, who sums what arrives in fp32.
        # Posted after both calls: ranks finish their first call at very different times, and a transfer posted
        # under the second call would spin on its SMs until the slowest rank arrives.
        works, ops_list, mine, recv, out_lo_hi = [], [], {}, {}, {}
        for name, g_hi, g_lo in (("k", dk_hi, dk_lo), ("v", dv_hi, dv_lo), ("g", dg_hi, dg_lo)):
            g_hi, g_lo = seq_major_mem(g_hi), seq_major_mem(g_lo)
            g_hi[:n_lo] += g_lo                                   # chunks both calls attended to
            tail = g_hi.shape[1:]
            final = torch.empty((2 * tc,) + tail, dtype=g_hi.dtype, device=dev)
            if dist.get_backend(group) == "gloo":                 # (no reduce-scatter in gloo: all-reduce, keep a slab)
                red = g_hi[:P * tc].clone()
                dist.all_reduce(red, group=group)
                final[:tc].copy_(red[rank * tc:(rank + 1) * tc])
            else:
                works.append(dist.reduce_scatter_tensor(final[:tc], g_hi[:P * tc], op=dist.ReduceOp.SUM, group=group,
                                                        async_op=True))
            if collective:
                # upper halves by reduce-scatter too: slab i of the input belongs to rank i, i.e. is chunk 2P-1-i;
                # this rank has partials for i >= rank only
                inp = torch.zeros((P, tc) + tail, dtype=g_hi.dtype, device=dev)
                inp[rank:].copy_(g_hi[P * tc:].view((P - rank, tc) + tail).flip(0))
                if dist.get_backend(group) == "gloo":
                    dist.all_reduce(inp, group=group)
                    final[tc:].copy_(inp[rank])
                else:
                    works.append(dist.reduce_scatter_tensor(final[tc:], inp, op=dist.ReduceOp.SUM, group=group,
                                                            async_op=True))
            else:
                # partials of this rank's upper chunk: its own (slot 0) and one from every rank below it
                recv[name] = torch.empty((rank + 1, tc) + tail, dtype=g_hi.dtype, device=dev)
                recv[name][0].copy_(g_hi[hi_c * tc:(hi_c + 1) * tc])
            mine[name], out_lo_hi[name] = g_hi, final
        for j in range(P):
            for name in ("k", "v", "g"):
                if collective:
                    break
                if j > rank:     # chunk 2P-1-j is below this rank's horizon 2P-1-rank: it has a partial for it
                    c = 2 * P - 1 - j
                    ops_list.append(("send", mine[name][c * tc:(c + 1) * tc], peer[j], group))
                elif j < rank:   # and the ranks below this one have partials for this rank's upper chunk
                    ops_list.append(("recv", recv[name][1 + j], peer[j], group))
        reqs = _exchange(ops_list)
        _mark("gradient exchange posted")
        for w in works:
            _wait(w)
        for r_ in reqs:
            r_.wait()
        _mark("gradients exchanged")
        grads = []
        for name in ("k", "v", "g"):
            if not collective:
                torch.sum(recv[name], dim=0, out=out_lo_hi[name][tc:])     # (16-bit sums accumulate in fp32)
            grads.append(_head_first(out_lo_hi[name]))
        dk, dv, dg = grads
        dq = torch.cat([dq_lo, dq_hi], dim=2)
        _mark("bwd end")
        return dq, dk, dv, dg, None, None, None, None, None


def context_parallel_threshold(q, k, sm_scale: float, seq_len: int, group, max_row_norm: Callable,
                               tolerance: float = -10.0) -> torch.Tensor:
    """``adaptive_threshold="auto"`` of the unsharded operator for a sharded sequence: the largest row norms
    of q and k over ALL ranks' rows (all-reduce MAX of the local maxima), rounded to the input dtype as
    ``torch.linalg.vector_norm`` of a 16-bit tensor rounds them, then upstream's expression
    (src/forgetting_transformer/ops/forgetting_attention.py:95-102) with the full sequence length."""
    import math
    nq, nk = max_row_norm(q).float(), max_row_norm(k).float()
    both = torch.stack([nq, nk])
    dist.all_reduce(both, op=dist.ReduceOp.MAX, group=group)
    bound = both[0].to(q.dtype) * both[1].to(q.dtype) * sm_scale
    return (-(2 * bound + math.log(seq_len)) + tolerance).float()


# side streams of the head-group pipeline, one per (device, group index)
_SIDE_STREAMS = {}
# how many head groups a context-parallel call is cut into (None: the environment's FOX_B200_CP_HEAD_GROUPS, else 1)
HEAD_GROUPS = None


def _head_groups(n_heads: int, is_cuda: bool) -> int:
    import os
    n = HEAD_GROUPS if HEAD_GROUPS is not None else int(os.environ.get("FOX_B200_CP_HEAD_GROUPS", "1"))
    n = max(1, min(n, n_heads))
    while n_heads % n:
        n -= 1
    return n


def context_parallel_attention(q, k, v, log_fgate, *, group=None, seq_start: Optional[torch.Tensor] = None,
                               sm_scale: Optional[float] = None, adaptive_threshold=None,
                               attn_fn: Optional[Callable] = None, max_row_norm: Optional[Callable] = None,
                               head_groups: Optional[int] = None):
    """Head-first forgetting attention over a sequence sharded in zig-zag chunks.

    Every rank passes its local shard: q, k, v (B, H, 2*Tc, D) and log_fgate (B, H, 2*Tc), the
    concatenation of its two chunks (``zigzag_chunks``) of a sequence of length 2*world*Tc.
    Returns the local shard of the output, same layout; differentiable (gradients of k, v and
    log_fgate are summed over ranks and returned to the owners).

    ``seq_start`` (B,) counts in positions of the whole sequence (left padding), the same tensor on
    every rank.  ``adaptive_threshold="auto"`` is evaluated once from the row norms of all ranks, so
    it is the threshold the unsharded call would use; a float or a (B, H)-broadcastable tensor is
    passed through.

    ``attn_fn(q, k, v, log_fgate, head_first=True, seq_start=..., sm_scale=..., adaptive_threshold=...)``
    defaults to the CUDA operator and ``max_row_norm(x) -> (B, H)`` to its row-norm kernel; the CPU
    tests inject the oracle.

    ``head_groups`` (default 1): heads are independent, so the call can be cut into that many groups of heads,
    each a complete context-parallel step on its own CUDA stream.  The first all-gather of a group and its final
    gradient exchange, which nothing of the same group can hide, then run under the other groups' kernels.
    Measured on B1 T65536 H24 D64 with two groups: 30.4 against 29.9 ms on 2 GPUs, 16.8 against 15.7 ms on 4, 10.8
    against 9.6 ms on 8 --
    the kernels of two streams share the SMs worse than the exposed collectives cost, so it is off by default.
    """
    if attn_fn is None:
        from .ops import forgetting_attention as attn_fn
    group = group if group is not None else dist.group.WORLD
    world = dist.get_world_size(group)
    tc = q.shape[2] // 2
    assert q.shape[2] == 2 * tc and k.shape[2] == 2 * tc and log_fgate.shape[2] == 2 * tc
    if sm_scale is None:
        sm_scale = q.shape[-1] ** -0.5
    if isinstance(adaptive_threshold, str):
        assert adaptive_threshold == "auto", f'adaptive_threshold must be either the string "auto", a float, or a Tensor, but got {adaptive_threshold}.'
        if max_row_norm is None:
            from .ops import max_row_norm
        with torch.no_grad():
            adaptive_threshold = context_parallel_threshold(q, k, sm_scale, 2 * world * tc, group, max_row_norm)
    B, H = q.shape[0], q.shape[1]
    n_groups = _head_groups(H, q.is_cuda) if head_groups is None else _head_groups_checked(head_groups, H)
    if n_groups == 1:
        return _ContextParallel.apply(q, k, v, log_fgate, seq_start, sm_scale, adaptive_threshold, group, attn_fn)
    hg = H // n_groups
    thr = adaptive_threshold
    if isinstance(thr, torch.Tensor) and thr.dim() > 0:
        thr = torch.broadcast_to(thr, (B, H))
    outs = []
    main = torch.cuda.current_stream() if q.is_cuda else None
    if main is not None:
        ready = torch.cuda.Event()     # the inputs are ready where the caller's stream stands now
        ready.record(main)
    for gi in range(n_groups):
        sl = slice(gi * hg, (gi + 1) * hg)
        thr_g = thr[:, sl] if (isinstance(thr, torch.Tensor) and thr.dim() > 0) else thr
        args = (q[:, sl], k[:, sl], v[:, sl], log_fgate[:, sl], seq_start, sm_scale, thr_g, group, attn_fn)
        if main is None or gi == 0:
            outs.append(_ContextParallel.apply(*args))      # (the first group stays on the caller's stream)
            continue
        key = (q.device.index, gi)
        side = _SIDE_STREAMS.get(key)
        if side is None:
            side = _SIDE_STREAMS[key] = torch.cuda.Stream(device=q.device)
        side.wait_event(ready)
        with torch.cuda.stream(side):
            o = _ContextParallel.apply(*args)
        o.record_stream(main)
        outs.append(o)
    if main is not None:
        for gi in range(1, n_groups):
            main.wait_stream(_SIDE_STREAMS[(q.device.index, gi)])
    return torch.cat(outs, dim=1)


def _head_groups_checked(n: int, n_heads: int) -> int:
    assert n >= 1 and n_heads % n == 0, f"head_groups={n} must divide the head count {n_heads}"
    return n


class ContextParallelAttention(torch.nn.Module):
    """Module form of :func:`context_parallel_attention` bound to a process group."""

    def __init__(self, group=None, attn_fn: Optional[Callable] = None):
        super().__init__()
        self.group, self.attn_fn = group, attn_fn

    def forward(self, q, k, v, log_fgate, seq_start=None, sm_scale=None, adaptive_threshold=None):
        return context_parallel_attention(q, k, v, log_fgate, group=self.group, seq_start=seq_start,
                                          sm_scale=sm_scale, adaptive_threshold=adaptive_threshold,
                                          attn_fn=self.attn_fn)
