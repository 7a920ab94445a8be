"""Forgetting Attention operator backed by the sm_100a kernels.

Host-side mirror of upstream's ``ForgettingAttention`` autograd function and
``forgetting_attention`` wrapper
(src/forgetting_transformer/ops/forgetting_attention.py:44-455): same argument
order, defaults, assertions and returned gradients, so it can be dropped in for
the Triton operator.  All device work goes through the C ABI of
``libfox_b200.so``; there is no Triton, no eager fallback and no CPU path.
"""
from __future__ import annotations

import math
import os
from typing import Literal, Optional, Union

import torch

from . import _lib

__all__ = ["forgetting_attention", "forgetting_attention_from_gate_logits", "ForgettingAttention", "make_graphed", "FWD_BLOCK",
           "BWD_BLOCK"]

# (BLOCK_M, BLOCK_N) of the kernels; pruning indices are defined on this grid.
_PADDED_HEAD_DIM = 64   # head dims 16 and 32 are zero-padded to this
# head dims whose backward runs as a key-side and a query-side kernel instead of the one-pass kernel
_TWO_KERNEL_BACKWARD_DIMS = set() if os.environ.get("FOX_B200_ONE_PASS_BWD", "0") == "1" else {128}
FWD_BLOCK = (128, 128)
BWD_BLOCK = (128, 128)

_DEBUG_SYNC = os.environ.get("FOX_B200_DEBUG_SYNC", "0") == "1"


class KernelTimer:
    """Optional CUDA-event stopwatch around each kernel launch of the operator (the
    counterpart of upstream's hidden ``record_time_key`` timers, lines 45-70).  Used by the
    benchmark to time the dominant kernel on the launching stream:

        with KernelTimer() as t: ...run steps...
        t.summary() -> {kernel name: (launches, mean milliseconds)}
    """
    active = None

    def __init__(self):
        self.events = []

    def __enter__(self):
        KernelTimer.active = self
        return self

    def __exit__(self, *exc):
        KernelTimer.active = None

    def summary(self):
        torch.cuda.synchronize()
        acc = {}
        for name, a, b in self.events:
            n, t = acc.get(name, (0, 0.0))
            acc[name] = (n + 1, t + a.elapsed_time(b))
        return {k: (n, t / n) for k, (n, t) in acc.items()}


def _call(name, fn, *args):
    """Launch one C-ABI entry point, timing it when a KernelTimer is active."""
    timer = KernelTimer.active
    if timer is None:
        _lib.check(fn(*args), name)
        return
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    _lib.check(fn(*args), name)
    b.record()
    timer.events.append((name, a, b))


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _tma_view(x: torch.Tensor) -> torch.Tensor:
    """Return ``x`` when TMA can address it, else a contiguous copy (upstream only
    insists on a unit inner stride, lines 35-38)."""
    return x if _lib.tma_ready(x) else x.contiguous()


def max_row_norm(x: torch.Tensor, keep_fp32: bool = False) -> torch.Tensor:
    """max_t ||x[b,h,t,:]||_2 in x's dtype, i.e.
    ``torch.linalg.vector_norm(x, dim=-1).max(dim=-1).values`` (upstream lines 95-96);
    ``keep_fp32`` returns the unrounded fp32 maxima."""
    lib = _lib.load()
    B, H, T, D = x.shape
    x = _tma_view(x)
    out = torch.zeros((B, H), dtype=torch.float32, device=x.device)
    _call("fox_max_row_norm", lib.fox_max_row_norm, x.device.index, _stream(), _lib.dtype_code(x.dtype), B, H, T,
          D, _lib.t4(x), out.data_ptr())
    return out if keep_fp32 else out.to(x.dtype)


def log_lambda_cumsum(log_fgate: torch.Tensor, seq_start: Optional[torch.Tensor],
                      carry_in: Optional[torch.Tensor] = None, return_total: bool = False):
    """fp32 inclusive prefix sum over the last axis of a (B,H,N) tensor of any
    strides with the gates left of ``seq_start`` treated as zero (upstream lines
    117-127).  ``carry_in`` (B,H) is added to every prefix (context-parallel
    chunks); ``return_total`` also returns the last prefix per (b,h)."""
    lib = _lib.load()
    B, H, N = log_fgate.shape
    out = torch.empty((B, H, N), dtype=torch.float32, device=log_fgate.device)
    total = torch.empty((B, H), dtype=torch.float32, device=log_fgate.device) if return_total else None
    _call("fox_cumsum_fwd", lib.fox_cumsum_fwd, log_fgate.device.index, _stream(), B, H, N, log_fgate.data_ptr(),
          log_fgate.stride(0), log_fgate.stride(1), log_fgate.stride(2), _lib.ptr(seq_start),
          _lib.ptr(carry_in), out.data_ptr(), _lib.ptr(total))
    return (out, total) if return_total else out


_GATE_DTYPES = {torch.float16: _lib.FOX_DTYPE_FP16, torch.bfloat16: _lib.FOX_DTYPE_BF16, torch.float32: _lib.FOX_DTYPE_FP32}


def gate_prefix_from_logits(fgate_logit: torch.Tensor, seq_start: Optional[torch.Tensor]) -> torch.Tensor:
    """fp32 prefix sum of log sigmoid(fgate_logit.float()) over the last axis of a (B,H,N) tensor of any strides
    and dtype fp16 / bf16 / fp32, gates left of ``seq_start`` treated as zero: upstream's
    ``F.logsigmoid(fgate_logit.float())`` (modeling_forgetting_transformer.py:343-346) and masked cumsum
    (forgetting_attention.py:117-127) in one kernel."""
    lib = _lib.load()
    B, H, N = fgate_logit.shape
    out = torch.empty((B, H, N), dtype=torch.float32, device=fgate_logit.device)
    _call("fox_gate_prefix_fwd", lib.fox_gate_prefix_fwd, fgate_logit.device.index, _stream(),
          _GATE_DTYPES[fgate_logit.dtype], B, H, N, fgate_logit.data_ptr(), fgate_logit.stride(0),
          fgate_logit.stride(1), fgate_logit.stride(2), _lib.ptr(seq_start), None, out.data_ptr())
    return out


def find_index(log_lambda: torch.Tensor, threshold: torch.Tensor, M: int, block_m: int, block_n: int,
               want_start: bool = True, want_end: bool = False):
    """Block-pruning index arrays (upstream lines 695-795) on a (block_m, block_n) grid."""
    lib = _lib.load()
    B, H, N = log_lambda.shape
    dev = log_lambda.device
    start = torch.empty((B, H, -(-M // block_m)), dtype=torch.long, device=dev) if want_start else None
    end = torch.empty((B, H, -(-N // block_n)), dtype=torch.long, device=dev) if want_end else None
    _call("fox_find_index", lib.fox_find_index, dev.index, _stream(), B, H, M, N, block_m, block_n,
          log_lambda.data_ptr(), threshold.data_ptr(), threshold.stride(0), threshold.stride(1),
          _lib.ptr(start), _lib.ptr(end))
    return start, end


class ForgettingAttention(torch.autograd.Function):
    """Same positional signature as upstream's autograd function (line 73); the three
    trailing timing arguments are accepted and ignored."""

    @staticmethod
    def forward(ctx, q, k, v, log_fgate, seq_start, causal, sm_scale, adaptive_threshold,
                return_log_normalizer=False, return_start_index=False, record_time_key=None,
                record_attention_time=False, record_find_index_time=False, gate_is_logit=False):
        """``gate_is_logit`` (not part of upstream's signature): ``log_fgate`` holds the gate LOGITS (fp16 / bf16 /
        fp32); log sigmoid and its derivative are folded into the prefix-sum kernels."""
        assert causal, "Only causal attention is supported"
        Dq, Dk, Dv = q.shape[-1], k.shape[-1], v.shape[-1]
        assert Dq == Dk == Dv, "feature size of q, k, v should be equal"
        assert Dk in {16, 32, 64, 128}, "We only support head dims in {16, 32, 64, 128}"

        B, H, M, D = q.shape
        N = k.shape[2]
        assert log_fgate.shape == (B, H, N)
        if gate_is_logit:
            assert log_fgate.dtype in _GATE_DTYPES, f"gate logits must be fp16, bf16 or fp32, but got {log_fgate.dtype}"
        else:
            assert log_fgate.dtype == torch.float32, "log_fgate must be in torch.float32. It is best to do this cast before logsigmoid, e.g., torch.nn.functional.logsigmoid(fgate_logit.float())."
        if sm_scale is None:
            sm_scale = 1. / math.sqrt(D)
        Hk, Hv = k.shape[1], v.shape[1]
        assert Hk == Hv, "num of heads in k and v should be equal"
        assert H == Hk, "groupped query attention has not been tested. You can uncomment this if you know what you are doing."
        assert not (M > N), "The key/value tensors must be longer than the query tensor"
        if isinstance(adaptive_threshold, str):
            assert adaptive_threshold == "auto", f'adaptive_threshold must be either the string "auto", a float, or a Tensor, but got {adaptive_threshold}.'
        if seq_start is not None:
            assert seq_start.shape == (B,)
        if not q.is_cuda:
            raise _lib.FoxError("forgetting_attention needs CUDA tensors on an sm_100 device; there is no CPU path")
        # Head dims 16 and 32 run through the D=64 kernels on zero-padded copies: zero columns change no
        # dot product, norm or output column, and their gradients are exactly zero and sliced off again.
        D_in = D
        if D in (16, 32):
            q, k, v = [torch.nn.functional.pad(t, (0, _PADDED_HEAD_DIM - D)) for t in (q, k, v)]
            D = _PADDED_HEAD_DIM

        lib = _lib.load()
        with torch.cuda.device(q.device):
            dev = q.device
            _lib.poll_status(dev)   # did a kernel of an earlier step give up on a wait? (no synchronisation)
            q, k, v = _tma_view(q), _tma_view(k), _tma_view(v)
            # largest key norm per (b,h): the forward kernel's bound that lets most tiles skip the row-maximum pass
            need_auto = isinstance(adaptive_threshold, str)
            k_norm_max = max_row_norm(k, keep_fp32=True) if ((N >= 8 * FWD_BLOCK[1] and M > 1) or need_auto) else None

            if adaptive_threshold is not None:
                if isinstance(adaptive_threshold, str):
                    assert adaptive_threshold == "auto", f'adaptive_threshold must be either the string "auto", a float, or a Tensor, but got {adaptive_threshold}.'
                    max_q_norm = max_row_norm(q)
                    max_k_norm = k_norm_max.to(k.dtype)
                    logit_upper_bound = max_q_norm * max_k_norm * sm_scale
                    tolerance = -10
                    adaptive_threshold = -(2 * logit_upper_bound + math.log(N)) + tolerance
                if isinstance(adaptive_threshold, torch.Tensor):
                    adaptive_threshold = adaptive_threshold.to(dtype=torch.float, device=dev)
                else:   # a fill kernel instead of a host-to-device copy: legal inside CUDA-graph capture
                    adaptive_threshold = torch.full((), float(adaptive_threshold), dtype=torch.float, device=dev)
                try:
                    adaptive_threshold = torch.broadcast_to(adaptive_threshold, (B, H))
                except RuntimeError:
                    raise RuntimeError(f'adaptive_threshold must be either the string "auto" or broadcastable to (batch_size, num_heads) = ({B}, {H}), but got {adaptive_threshold.size()}.')
                assert adaptive_threshold.size() == (B, H)

            if seq_start is not None:
                has_seq_start = True
                assert seq_start.shape == (B,)
                seq_start = seq_start.to(device=dev, dtype=torch.long).contiguous()
            else:
                has_seq_start = False

            log_lambda = (gate_prefix_from_logits(log_fgate, seq_start) if gate_is_logit
                          else log_lambda_cumsum(log_fgate, seq_start))

            start_index = None
            if adaptive_threshold is not None:
                start_index, _ = find_index(log_lambda, adaptive_threshold, M, *FWD_BLOCK)

            o = torch.empty_like(q)
            if not _lib.tma_ready(o):
                o = torch.empty(q.shape, dtype=q.dtype, device=dev)
            L = torch.empty((B, H, M), device=dev, dtype=torch.float32)
            if M == 1 and not any(ctx.needs_input_grad[:4]):
                # generation step: one query row against the cache, no gradients -> split-KV kernels
                splits = max(1, min((N + 511) // 512, (4 * 148 + B * H - 1) // (B * H), 256))
                work = torch.empty(lib.fox_attn_decode_workspace_floats(B, H, D, splits), device=dev,
                                   dtype=torch.float32)
                _call("fox_attn_decode", lib.fox_attn_decode, dev.index, _stream(), _lib.dtype_code(q.dtype), B, H, N,
                      D, _lib.t4(q), _lib.t4(k), _lib.t4(v), log_lambda.data_ptr(), _lib.ptr(seq_start),
                      _lib.ptr(start_index), float(sm_scale), _lib.t4(o), L.data_ptr(), work.data_ptr(), splits)
                out = o if D_in == D else o[..., :D_in].contiguous()
                if return_log_normalizer or return_start_index:
                    return (out, L if return_log_normalizer else None, start_index if return_start_index else None)
                return out
            status = _lib.status_buffer(dev)
            _call("fox_attn_fwd", lib.fox_attn_fwd, dev.index, _stream(), _lib.dtype_code(q.dtype), B, H, M, N, D,
                  _lib.t4(q), _lib.t4(k), _lib.t4(v), log_lambda.data_ptr(), _lib.ptr(seq_start),
                  _lib.ptr(start_index), float(sm_scale), _lib.t4(o), L.data_ptr(), _lib.ptr(k_norm_max),
                  status.data_ptr())
            if _DEBUG_SYNC:
                _lib.check_status(dev)

        ctx.save_for_backward(q, k, v, o, L, log_lambda, seq_start, adaptive_threshold)
        ctx.gate_logit = log_fgate if gate_is_logit else None    # (an input of the function: kept as it is)
        ctx.sm_scale = sm_scale
        ctx.has_seq_start = has_seq_start
        # the query-side backward kernel prunes by the same array when the two block grids agree (not an input or
        # output of the function, so it is kept on ctx rather than through save_for_backward)
        ctx.start_index = start_index if FWD_BLOCK == BWD_BLOCK else None
        ctx.head_dim = D_in
        out = o if D_in == D else o[..., :D_in].contiguous()
        if return_log_normalizer or return_start_index:
            ctx.mark_non_differentiable(*[t for t in (L, start_index) if t is not None])
            return (out, L if return_log_normalizer else None, start_index if return_start_index else None)
        return out

    @staticmethod
    def backward(ctx, do, *ignored):
        q, k, v, o, L, log_lambda, seq_start, adaptive_threshold = ctx.saved_tensors
        sm_scale = ctx.sm_scale
        B, H, M, D = q.shape
        N = k.shape[2]
        lib = _lib.load()
        # the autograd engine runs this on its own thread: select the device explicitly
        with torch.cuda.device(q.device):
            dev = q.device
            if ctx.head_dim != D:
                do = torch.nn.functional.pad(do, (0, D - ctx.head_dim))
            do = _tma_view(do)
            code = _lib.dtype_code(q.dtype)
            delta = torch.empty_like(L)
            _call("fox_bwd_delta", lib.fox_bwd_delta, dev.index, _stream(), code, B, H, M, D, _lib.t4(o),
                  _lib.t4(do), delta.data_ptr())
            end_index = None
            if adaptive_threshold is not None:
                _, end_index = find_index(log_lambda, adaptive_threshold, M, *BWD_BLOCK, want_start=False,
                                          want_end=True)
            dk = torch.empty_like(k)
            dv = torch.empty_like(v)
            dq = torch.empty_like(q)
            if not _lib.tma_ready(dk):
                dk = torch.empty(k.shape, dtype=k.dtype, device=dev)
            if not _lib.tma_ready(dv):
                dv = torch.empty(v.shape, dtype=v.dtype, device=dev)
            if not _lib.tma_ready(dq):
                dq = torch.empty(q.shape, dtype=q.dtype, device=dev)
            dlam_col = torch.empty((B, H, N), dtype=torch.float32, device=dev)
            status = _lib.status_buffer(dev)
            if D in _TWO_KERNEL_BACKWARD_DIMS:
                # key side (dk, dv, column sums) without a dQ product, query side as its own kernel: no fp32
                # dQ partials to add-reduce into L2, which is what bounds the one-pass kernel at this head dim
                start_index = None
                if adaptive_threshold is not None:
                    start_index = ctx.start_index
                    if start_index is None:
                        start_index, _ = find_index(log_lambda, adaptive_threshold, M, *BWD_BLOCK)
                dlam_row = torch.empty((B, H, M), dtype=torch.float32, device=dev)
                _call("fox_attn_bwd", lib.fox_attn_bwd, dev.index, _stream(), code, B, H, M, N, D, _lib.t4(q),
                      _lib.t4(k), _lib.t4(v), _lib.t4(do), log_lambda.data_ptr(), L.data_ptr(), delta.data_ptr(),
                      _lib.ptr(seq_start), _lib.ptr(end_index), float(sm_scale), None, None,
                      dlam_col.data_ptr(), _lib.t4(dk), _lib.t4(dv), status.data_ptr())
                _call("fox_attn_bwd_dq", lib.fox_attn_bwd_dq, dev.index, _stream(), code, B, H, M, N, D, _lib.t4(q),
                      _lib.t4(k), _lib.t4(v), _lib.t4(do), log_lambda.data_ptr(), L.data_ptr(), delta.data_ptr(),
                      _lib.ptr(seq_start), _lib.ptr(start_index), float(sm_scale), _lib.t4(dq), dlam_row.data_ptr(),
                      status.data_ptr())
                dlog_fgate = _gate_gradient(ctx, lib, dev, B, H, M, N, dlam_col, dlam_row)
                _lib.queue_status_readback(dev)
                if _DEBUG_SYNC:
                    _lib.check_status(dev)
                if ctx.head_dim != D:
                    dq, dk, dv = [t[..., :ctx.head_dim].contiguous() for t in (dq, dk, dv)]
                return dq, dk, dv, dlog_fgate, None, None, None, None, None, None, None, None, None, None
            # scratch: fp32 dQ accumulator and the query-side log-gate gradient (both reduced into)
            scratch = torch.zeros(B * H * M * (D + 1), dtype=torch.float32, device=dev)
            dq_accum = scratch[: B * H * M * D]
            dlam_row = scratch[B * H * M * D:]
            _call("fox_attn_bwd", lib.fox_attn_bwd, dev.index, _stream(), code, B, H, M, N, D, _lib.t4(q),
                  _lib.t4(k), _lib.t4(v), _lib.t4(do), log_lambda.data_ptr(), L.data_ptr(), delta.data_ptr(),
                  _lib.ptr(seq_start), _lib.ptr(end_index), float(sm_scale), dq_accum.data_ptr(),
                  dlam_row.data_ptr(), dlam_col.data_ptr(), _lib.t4(dk), _lib.t4(dv), status.data_ptr())
            _call("fox_dq_convert", lib.fox_dq_convert, dev.index, _stream(), code, B, H, M, D,
                  dq_accum.data_ptr(), float(sm_scale), _lib.t4(dq))
            dlog_fgate = _gate_gradient(ctx, lib, dev, B, H, M, N, dlam_col, dlam_row)
            _lib.queue_status_readback(dev)
            if _DEBUG_SYNC:
                _lib.check_status(dev)
        if ctx.head_dim != D:
            dq, dk, dv = [t[..., :ctx.head_dim].contiguous() for t in (dq, dk, dv)]
        return dq, dk, dv, dlog_fgate, None, None, None, None, None, None, None, None, None, None


def _gate_gradient(ctx, lib, dev, B, H, M, N, dlam_col, dlam_row):
    """Reverse prefix sum of the two halves of dlog_lambda (upstream lines 390-392); for gate logits also the
    chain rule through log sigmoid, in the logits' dtype and layout."""
    logit = getattr(ctx, "gate_logit", None)
    if logit is None:
        dlog_fgate = torch.empty((B, H, N), dtype=torch.float32, device=dev)
        _call("fox_revcumsum", lib.fox_revcumsum, dev.index, _stream(), B, H, M, N, dlam_col.data_ptr(),
              dlam_row.data_ptr(), None, dlog_fgate.data_ptr(), None)
        return dlog_fgate
    dlogit = torch.empty_strided(logit.shape, logit.stride(), dtype=logit.dtype, device=dev)
    _call("fox_gate_prefix_bwd", lib.fox_gate_prefix_bwd, dev.index, _stream(), _GATE_DTYPES[logit.dtype], B, H, M, N,
          dlam_col.data_ptr(), dlam_row.data_ptr(), logit.data_ptr(), logit.stride(0), logit.stride(1),
          logit.stride(2), dlogit.data_ptr())
    return dlogit


def forgetting_attention_from_gate_logits(q, k, v, fgate_logit, *, head_first: bool = False,
                                          seq_start: Optional[torch.Tensor] = None, sm_scale: Optional[float] = None,
                                          adaptive_threshold=None):
    """``forgetting_attention(q, k, v, F.logsigmoid(fgate_logit.float()), ...)`` with the log sigmoid folded into
    the operator's prefix-sum kernel and its derivative into the reverse prefix sum of the backward: the layer's
    gate projection output (fp16 / bf16 / fp32, (B, T, H) or (B, H, T) with ``head_first``, any strides) goes in as
    it is and receives its gradient in its own dtype (upstream forms the log gates with two elementwise kernels in
    front of the operator, modeling_forgetting_transformer.py:343-346).  Everything else as ``forgetting_attention``."""
    for name, entry in dict(q=q, k=k, v=v).items():
        assert entry.dtype in [torch.float16, torch.bfloat16], f"Only torch.float16 or torch.bfloat16 are supported for q/k/v, but got {entry.dtype} for {name}."
    if not head_first:
        q, k, v = [item.permute(0, 2, 1, 3) for item in (q, k, v)]
        fgate_logit = fgate_logit.permute(0, 2, 1)
    out = ForgettingAttention.apply(q, k, v, fgate_logit, seq_start, True, sm_scale, adaptive_threshold,
                                    False, False, None, False, False, True)
    if not head_first:
        out = out.permute(0, 2, 1, 3)
    return out


def forgetting_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    log_fgate: torch.Tensor,
    *,
    head_first: bool = False,
    seq_start: Optional[torch.Tensor] = None,
    sm_scale: Optional[float] = None,
    adaptive_threshold: Optional[Union[Literal["auto"], float, torch.Tensor]] = None,
):
    """Forgetting Attention (causal softmax attention with the decay bias
    ``cumsum(log_fgate)_i - cumsum(log_fgate)_j``), same contract as upstream's
    ``forgetting_transformer.forgetting_attention`` (lines 403-455):

    - q (B, Tq, H, D), k/v (B, Tk, H, D) in fp16/bf16 and log_fgate (B, Tk, H) in
      fp32, or with the H and T axes swapped when ``head_first=True``;
    - Tq <= Tk, causal, D in {16, 32, 64, 128} (16 and 32 run zero-padded through the D=64 kernels);
    - ``seq_start`` (B,) long: no attention to positions left of it (left padding);
    - ``sm_scale`` defaults to 1/sqrt(D);
    - ``adaptive_threshold``: "auto", a float or a tensor broadcastable to (B, H);
      whole KV blocks whose decay-bounded logits fall below it are skipped.

    Returns the output in q's layout; differentiable w.r.t. q, k, v and log_fgate.
    """
    for name, entry in dict(q=q, k=k, v=v).items():
        assert entry.dtype in [torch.float16, torch.bfloat16], f"Only torch.float16 or torch.bfloat16 are supported for q/k/v, but got {entry.dtype} for {name}."
    if not head_first:
        q, k, v = [item.permute(0, 2, 1, 3) for item in (q, k, v)]
        log_fgate = log_fgate.permute(0, 2, 1)
    out = ForgettingAttention.apply(q, k, v, log_fgate, seq_start, True, sm_scale, adaptive_threshold,
                                    False, False, None, False, False)
    if not head_first:
        out = out.permute(0, 2, 1, 3)
    return out


# ---- the FoX layer's glue in front of the operator (modeling_forgetting_transformer.py:366-396) ----

def seq_start_from_attention_mask(attention_mask: torch.Tensor) -> torch.Tensor:
    """``seq_start = T - attention_mask.sum(-1)`` for a left-padded (B, T) mask (upstream lines 392-396)."""
    assert attention_mask.dim() == 2
    return attention_mask.shape[-1] - attention_mask.sum(dim=-1)


def acp_threshold_from_qk_norm(q_norm_weight: torch.Tensor, k_norm_weight: torch.Tensor, num_heads: int,
                               head_dim: int, seq_len: int, log_pruning_tolerance: float,
                               share_param_across_head: bool = False) -> torch.Tensor:
    """Pruning threshold of a layer with QK-norm: after a per-head RMSNorm ||q|| <= max|w_q| sqrt(D), so
    the logit bound max|w_q| max|w_k| sqrt(D) needs no pass over the data (upstream lines 371-381).
    Returns a scalar (shared weights) or a (num_heads,) tensor for ``adaptive_threshold``."""
    with torch.no_grad():
        if share_param_across_head:
            assert q_norm_weight.size() == k_norm_weight.size() == (head_dim,)
            bound = q_norm_weight.abs().max() * k_norm_weight.abs().max() * math.sqrt(head_dim)
        else:
            assert q_norm_weight.size() == k_norm_weight.size() == (num_heads * head_dim,)
            bound = (q_norm_weight.view(num_heads, head_dim).abs().max(dim=-1).values
                     * k_norm_weight.view(num_heads, head_dim).abs().max(dim=-1).values * math.sqrt(head_dim))
        return -(2 * bound + math.log(seq_len)) + log_pruning_tolerance


def acp_threshold_from_data(q: torch.Tensor, k: torch.Tensor, log_pruning_tolerance: float) -> torch.Tensor:
    """Pruning threshold of a layer without QK-norm, from the largest row norms of head-first q, k
    (upstream lines 383-387); (B, H) tensor for ``adaptive_threshold``.  The norms come from
    ``fox_max_row_norm`` in the input dtype, as ``torch.linalg.vector_norm(...).max(...)`` gives them."""
    with torch.no_grad():
        D, T = q.shape[-1], k.shape[2]
        bound = max_row_norm(q) * max_row_norm(k) / math.sqrt(D)
        return -(2 * bound + math.log(T)) + log_pruning_tolerance


def make_graphed(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, log_fgate: torch.Tensor, *,
                 head_first: bool = False, seq_start: Optional[torch.Tensor] = None,
                 sm_scale: Optional[float] = None,
                 adaptive_threshold=None, num_warmup_iters: int = 3):
    """CUDA-graph replay of a step for launch-bound shapes (B4 T512 H12 D64: 7 launches whose device time is a
    fraction of their launch cost).  Returns ``f(q, k, v, log_fgate) -> out`` with the same autograd contract as
    ``forgetting_attention`` for tensors of exactly the sample arguments' shapes, dtypes and ``requires_grad``
    flags.  Every entry point of the library launches on the caller's current stream, allocates nothing and never
    synchronises, and the cached TMA descriptors are keyed by (pointer, shape, strides), so
    ``torch.cuda.make_graphed_callables`` can capture the forward and the backward once.  ``seq_start`` and a
    tensor ``adaptive_threshold`` are captured by reference: update them in place between calls.  The sample
    tensors are only used for warm-up and capture."""
    assert q.is_cuda, "CUDA graphs need CUDA tensors"

    def op(q_, k_, v_, lf_):
        return forgetting_attention(q_, k_, v_, lf_, head_first=head_first, seq_start=seq_start, sm_scale=sm_scale,
                                    adaptive_threshold=adaptive_threshold)

    return torch.cuda.make_graphed_callables(op, (q, k, v, log_fgate), num_warmup_iters=num_warmup_iters)
