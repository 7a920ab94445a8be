"""CPU oracle for the Forgetting Attention hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch/NumPy on the CPU, the arithmetic of the
upstream project's operator so that the CUDA kernels can be checked against it.
Nothing in the shipped package imports it: only the test-suite, the smoke entry
point and the benchmark's CPU-baseline leg do.

Parity pinning: the functions below are checked (tests/test_oracle.py) against
fixtures under tests/golden/ that were produced by importing the upstream
package itself and running its Triton kernels in Triton's CPU interpreter and
its in-file dense PyTorch formulation (tests/golden/make_golden.py).

Upstream citations use paths inside the upstream repository:
  OPS = src/forgetting_transformer/ops/forgetting_attention.py
  FNG = src/forgetting_transformer/model/forgetting_transformer/fuse_norm_gate.py
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch

LOG2E = 1.4426950408889634


# --------------------------------------------------------------------------
# log-gate prefix (OPS:111-127)
# --------------------------------------------------------------------------
def masked_log_fgate(log_fgate: torch.Tensor, seq_start: Optional[torch.Tensor]) -> torch.Tensor:
    """Zero the log gates left of ``seq_start`` (OPS:117-125).  (B, H, N) fp32."""
    lf = log_fgate.float()
    if seq_start is None:
        return lf
    N = lf.shape[-1]
    mask = torch.arange(N, device=lf.device)[None, None, :] < seq_start[:, None, None]
    return lf.masked_fill(mask, 0.0)


def log_lambda(log_fgate: torch.Tensor, seq_start: Optional[torch.Tensor]) -> torch.Tensor:
    """Inclusive prefix sum of the (masked) log gates, fp32 (OPS:127)."""
    return torch.cumsum(masked_log_fgate(log_fgate, seq_start), dim=-1, dtype=torch.float32)


def reverse_cumsum(dlog_lambda: torch.Tensor) -> torch.Tensor:
    """dlog_fgate_t = sum_{u >= t} dlog_lambda_u, written as upstream does (OPS:390-392)."""
    cs = torch.cumsum(dlog_lambda, dim=-1, dtype=dlog_lambda.dtype)
    return (dlog_lambda + cs[..., -1:] - cs).float()


# --------------------------------------------------------------------------
# dense formulation (upstream's in-file known-answer math, OPS:1380-1404)
# --------------------------------------------------------------------------
def dense_forgetting_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    log_fgate: torch.Tensor,
    seq_start: Optional[torch.Tensor] = None,
    sm_scale: Optional[float] = None,
    mask_gates: bool = False,
) -> torch.Tensor:
    """Head-first dense forgetting attention, differentiable through autograd.

    q (B,H,M,D); k, v (B,H,N,D); log_fgate (B,H,N) fp32.  Follows OPS:1380-1399
    line by line: logits in the input dtype, bias and softmax in fp32, the
    probabilities cast back to the input dtype before ``p @ v``, NaN rows
    (rows with nothing to attend to) set to zero.

    ``mask_gates=True`` additionally zeroes the gates left of ``seq_start``
    before the prefix sum, which is what the operator itself does (OPS:117-125);
    the upstream test leaves them in (the bias is a difference, so the result
    is the same up to rounding).
    """
    B, H, M, D = q.shape
    N = k.shape[2]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    P_SEQ = N - M
    dev = q.device
    mask = torch.tril(torch.ones((M, N), device=dev), diagonal=P_SEQ)
    p = torch.matmul(q, k.transpose(2, 3)) * sm_scale
    p = p.float()
    lf = masked_log_fgate(log_fgate, seq_start) if mask_gates else log_fgate
    lam = torch.cumsum(lf, dim=-1)
    decay_bias = lam[..., -M:, None] - lam[..., None, :]
    p = p + decay_bias
    p = p.masked_fill((mask == 0)[None, None], float("-inf"))
    if seq_start is not None:
        attention_mask = torch.arange(N, device=dev) < seq_start[:, None, None, None]
        p = torch.where(attention_mask, float("-inf"), p)
    p = torch.softmax(p.float(), dim=-1).to(q.dtype)
    p = torch.where(torch.isnan(p), torch.zeros_like(p), p)   # rows with no visible key
    return torch.matmul(p, v)


def dense_fwd_bwd(q, k, v, log_fgate, dout, seq_start=None, sm_scale=None, mask_gates=False):
    """Forward + autograd backward of the dense formulation.  Returns
    (out, dq, dk, dv, dlog_fgate)."""
    q, k, v, log_fgate = [t.detach().clone().requires_grad_() for t in (q, k, v, log_fgate)]
    out = dense_forgetting_attention(q, k, v, log_fgate, seq_start, sm_scale, mask_gates)
    out.backward(dout)
    return out.detach(), q.grad, k.grad, v.grad, log_fgate.grad


# --------------------------------------------------------------------------
# Adaptive Computation Pruning: threshold and block index scans
# --------------------------------------------------------------------------
def auto_threshold(q: torch.Tensor, k: torch.Tensor, sm_scale: float) -> torch.Tensor:
    """``adaptive_threshold="auto"`` (OPS:95-104).  The norms are evaluated in the
    input dtype (torch.linalg.vector_norm of a bf16 tensor returns bf16), then the
    result is cast to fp32.  q (B,H,M,D), k (B,H,N,D) -> (B,H) fp32."""
    N = k.shape[2]
    max_q_norm = torch.linalg.vector_norm(q, dim=-1).max(dim=-1).values
    max_k_norm = torch.linalg.vector_norm(k, dim=-1).max(dim=-1).values
    logit_upper_bound = max_q_norm * max_k_norm * sm_scale
    thr = -(2 * logit_upper_bound + math.log(N)) + (-10)
    return torch.as_tensor(thr, dtype=torch.float32)


def find_start_index(lam: np.ndarray, thr: np.ndarray, M: int, N: int, BM: int, BN: int) -> np.ndarray:
    """First KV column (a multiple of BN) each query block has to visit (OPS:695-745).

    lam (B,H,N) fp32, thr (B,H) fp32 -> int64 (B,H,ceil(M/BM)).  The scan position
    is carried from one query block to the next, exactly as upstream does.
    Thresholds must be <= 0 (otherwise upstream's loop does not terminate)."""
    lam = np.asarray(lam, dtype=np.float32)
    thr = np.asarray(thr, dtype=np.float32)
    B, H, _ = lam.shape
    P = N - M
    nmb = -(-M // BM)
    out = np.zeros((B, H, nmb), dtype=np.int64)
    for b in range(B):
        for h in range(H):
            row = lam[b, h]
            t = thr[b, h]
            s = 0
            for mb in range(nmb):
                lo = row[P + mb * BM]
                while np.float32(lo - row[min(N - 1, s + BN - 1)]) < t:
                    s += BN
                out[b, h, mb] = s
    return out


def find_end_index(lam: np.ndarray, thr: np.ndarray, M: int, N: int, BM: int, BN: int) -> np.ndarray:
    """First query row (block aligned, clipped to M) past which a KV block is pruned
    (OPS:747-795).  Note the row index carries no N-M offset upstream (OPS:783).
    -> int64 (B,H,ceil(N/BN))."""
    lam = np.asarray(lam, dtype=np.float32)
    thr = np.asarray(thr, dtype=np.float32)
    B, H, _ = lam.shape
    nnb = -(-N // BN)
    out = np.zeros((B, H, nnb), dtype=np.int64)
    for b in range(B):
        for h in range(H):
            row = lam[b, h]
            t = thr[b, h]
            e = 0
            for nb in range(nnb):
                li = row[min(N - 1, nb * BN + BN - 1)]
                while np.float32(row[min(e, M - 1)] - li) >= t and e < M:
                    e = min(e + BM, M)
                out[b, h, nb] = e
    return out


# --------------------------------------------------------------------------
# block-level restatement of the kernels (used when pruning is on)
# --------------------------------------------------------------------------
def _tile_masks(B, H, M, N, BM, BN, seq_start, start_index, end_index, bwd_kv_bm=None, bwd_kv_bn=None):
    """Element masks (B,H,M,N) of the tiles each kernel visits.

    forward / dQ pass (OPS:591-613, 1239-1261): columns >= floor(max(start_index,
    min(seq_start, hi))/BN)*BN and < hi.   dK/dV pass (OPS:1003-1049): rows
    < min(end_index, M), and nothing for KV blocks entirely left of seq_start-1.
    Causal/seq_start element masks are applied separately."""
    P = N - M
    rows = torch.arange(M)
    cols = torch.arange(N)
    fwd = torch.ones(B, H, M, N, dtype=torch.bool)
    if start_index is not None:
        si = torch.as_tensor(start_index)  # (B,H,nmb)
        lo = si.clone()
        if seq_start is not None:
            hi = torch.minimum(torch.tensor(N), P + (torch.arange(si.shape[-1]) + 1) * BM)
            lo = torch.maximum(lo, torch.minimum(seq_start[:, None, None], hi[None, None, :]))
        lo = (lo // BN) * BN
        lo_rows = lo[..., rows // BM]  # (B,H,M)
        fwd = cols[None, None, None, :] >= lo_rows[..., None]
    kv = torch.ones(B, H, M, N, dtype=torch.bool)
    if end_index is not None:
        bm = bwd_kv_bm or BM
        bn = bwd_kv_bn or BN
        ei = torch.clamp(torch.as_tensor(end_index), max=M)  # (B,H,nnb)
        hi_cols = ei[..., cols // bn]  # (B,H,N)
        if seq_start is not None:
            nb = cols // bn
            keep = (nb * bn + bn)[None, :] >= (seq_start[:, None] - 1)  # (B,N)
            hi_cols = torch.where(keep[:, None, :], hi_cols, torch.zeros_like(hi_cols))
        # rows are visited in blocks of bm starting at the causal lower bound; a row is
        # visited iff its block start < hi
        row_block_start = (rows // bm) * bm
        kv = row_block_start[None, None, :, None] < hi_cols[:, :, None, :]
    return fwd, kv


def blockwise_fwd_bwd(
    q, k, v, log_fgate, dout, seq_start=None, sm_scale=None,
    start_index=None, end_index=None, start_index_bwd=None,
    BM=128, BN=128, bwd_kv_bm=None, bwd_kv_bn=None, bwd_q_bm=None, bwd_q_bn=None,
    low_precision_matmul=True, lam=None, saved_out=None, saved_L=None,
):
    """Restatement of the kernels' arithmetic with block pruning (OPS:505-693,
    956-1344): the same formulas as the dense path, but tiles excluded by the
    index arrays contribute nothing, exactly as a skipped loop iteration.

    Returns dict(out, L, delta, dq, dk, dv, dlog_lambda, dlog_fgate).  All math in
    fp32 on the CPU; when ``low_precision_matmul`` the probabilities and dS are
    rounded to the input dtype before their matmuls as the kernels do
    (OPS:666, 1101, 1121, 1325).

    The backward is a function of what the forward saved (OPS:207): ``lam`` (the fp32 prefix sum), ``saved_out``
    (the 16-bit output, which delta is formed from, OPS:902-943) and ``saved_L`` (the log-normaliser the
    probabilities are recomputed with, OPS:1087, 1300).  When given, they replace the oracle's own values in the
    backward (and ``lam`` also in the forward), so that a backward kernel can be checked on exactly the inputs it
    was run on: two correct 16-bit forwards differ in the rounding of ``out`` (which enters every dS through
    delta) and, for long sequences, in the last bits of the fp32 prefix sum."""
    B, H, M, D = q.shape
    N = k.shape[2]
    P = N - M
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    dt = q.dtype
    qf, kf, vf, dof = q.float(), k.float(), v.float(), dout.float()
    lam = log_lambda(log_fgate, seq_start) if lam is None else lam.float()
    s = torch.matmul(qf, kf.transpose(2, 3)) * sm_scale + (lam[..., P:, None] - lam[..., None, :])
    rows = torch.arange(M)
    cols = torch.arange(N)
    elem = (P + rows)[:, None] >= cols[None, :]
    elem = elem[None, None].expand(B, H, M, N)
    if seq_start is not None:
        elem = elem & (cols[None, None, None, :] >= seq_start[:, None, None, None])
    fwd_mask, _ = _tile_masks(B, H, M, N, BM, BN, seq_start, start_index, None)
    _, kv_mask = _tile_masks(B, H, M, N, bwd_kv_bm or BM, bwd_kv_bn or BN, seq_start, None, end_index,
                             bwd_kv_bm, bwd_kv_bn)
    q_mask, _ = _tile_masks(B, H, M, N, bwd_q_bm or BM, bwd_q_bn or BN, seq_start,
                            start_index_bwd if start_index_bwd is not None else start_index, None)
    neg = torch.tensor(float("-inf"))
    s_f = torch.where(elem & fwd_mask, s, neg)
    L = torch.logsumexp(s_f, dim=-1)  # -inf on empty rows
    p_f = torch.exp(s_f - torch.where(torch.isinf(L), torch.zeros_like(L), L)[..., None])
    p_f = torch.where(elem & fwd_mask, p_f, torch.zeros_like(p_f))

    def lp(x):
        return x.to(dt).float() if low_precision_matmul else x

    out = torch.matmul(lp(p_f), vf)
    out_lp = out.to(dt)
    delta = ((out_lp if saved_out is None else saved_out).float() * dof).sum(-1)
    # backward: probabilities recomputed from the saved normaliser, no fwd tile mask
    Lb = L if saved_L is None else saved_L.float()
    Lz = torch.where(torch.isinf(Lb), torch.zeros_like(Lb), Lb)
    p = torch.exp(s - Lz[..., None])
    p = torch.where(elem & ~torch.isinf(Lb)[..., None], p, torch.zeros_like(p))
    dp = torch.matmul(dof, vf.transpose(2, 3))
    ds = p * (dp - delta[..., None])
    p_kv = torch.where(kv_mask, p, torch.zeros_like(p))
    ds_kv = torch.where(kv_mask, ds, torch.zeros_like(ds))
    ds_q = torch.where(q_mask, ds, torch.zeros_like(ds))
    dv = torch.matmul(lp(p_kv).transpose(2, 3), dof)
    dk = torch.matmul(lp(ds_kv).transpose(2, 3), qf) * sm_scale
    dq = torch.matmul(lp(ds_q), kf) * sm_scale
    dlam = -ds_kv.sum(dim=2)
    dlam[..., P:] += ds_q.sum(dim=3)
    if seq_start is not None:
        colmask = cols[None, None, :] >= seq_start[:, None, None]
        dk = dk * colmask[..., None]
        dv = dv * colmask[..., None]
    return dict(out=out_lp, L=L, delta=delta, dq=dq.to(dt), dk=dk.to(dt), dv=dv.to(dt), dlog_lambda=dlam,
                dlog_fgate=reverse_cumsum(dlam), log_lambda=lam)


def chunked_fwd_bwd(q, k, v, log_fgate, dout, seq_start=None, sm_scale=None, start_index=None, end_index=None,
                    BM=128, BN=128, row_chunk=1024, lam=None, saved_out=None, saved_L=None):
    """``blockwise_fwd_bwd`` for sequences too long to hold (M, N) matrices: the same formulas (OPS:505-693,
    956-1344) evaluated over chunks of ``row_chunk`` query rows with explicit gradients, in one pass for
    both the reference arithmetic (probabilities and dS rounded to the input dtype before their products,
    delta from the rounded output) and the unrounded fp32 path.  Pruning index arrays act on (BM, BN) tiles as
    in ``_tile_masks``; ``seq_start`` and pruning are not combined here.  M <= N.  ``lam``, ``saved_out``,
    ``saved_L``: as in ``blockwise_fwd_bwd`` (both evaluations then differentiate through the same saved tensors).

    Returns (rounded, fp32): two dicts with out, L, dq, dk, dv, dlog_fgate (out / dq / dk / dv of ``rounded``
    in the input dtype)."""
    B, H, M, D = q.shape
    N = k.shape[2]
    P = N - M
    assert row_chunk % BM == 0 and not (seq_start is not None and (start_index is not None or end_index is not None))
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    dt = q.dtype
    qf, kf, vf, dof = q.float(), k.float(), v.float(), dout.float()
    lam = log_lambda(log_fgate, seq_start) if lam is None else lam.float()
    cols = torch.arange(N)
    si = None if start_index is None else torch.as_tensor(start_index)
    ei = None if end_index is None else torch.clamp(torch.as_tensor(end_index), max=M)
    res = []
    for rounded in (True, False):
        res.append(dict(out=torch.zeros(B, H, M, D), L=torch.zeros(B, H, M), dq=torch.zeros(B, H, M, D),
                        dk=torch.zeros(B, H, N, D), dv=torch.zeros(B, H, N, D), dlam=torch.zeros(B, H, N)))
    for r0 in range(0, M, row_chunk):
        r1 = min(M, r0 + row_chunk)
        n1 = P + r1                                   # keys a row of this chunk may see
        rows = torch.arange(r0, r1)
        s = torch.matmul(qf[:, :, r0:r1], kf[:, :, :n1].transpose(2, 3)) * sm_scale
        s += lam[:, :, P + r0:P + r1, None] - lam[:, :, None, :n1]
        elem = ((P + rows)[:, None] >= cols[None, :n1])[None, None].expand(B, H, r1 - r0, n1)
        if seq_start is not None:
            elem = elem & (cols[None, None, None, :n1] >= seq_start[:, None, None, None])
        fwd_keep = kv_keep = None
        if si is not None:
            lo_rows = ((si // BN) * BN)[..., rows // BM]                       # (B,H,rows)
            fwd_keep = cols[None, None, None, :n1] >= lo_rows[..., None]
        if ei is not None:
            hi_cols = ei[..., cols[:n1] // BN]                                 # (B,H,n1)
            kv_keep = ((rows // BM) * BM)[None, None, :, None] < hi_cols[:, :, None, :]
        neg = torch.tensor(float("-inf"))
        s_f = torch.where(elem if fwd_keep is None else (elem & fwd_keep), s, neg)
        L = torch.logsumexp(s_f, dim=-1)
        empty = torch.isinf(L)
        Lz = torch.where(empty, torch.zeros_like(L), L)
        p_f = torch.where(torch.isinf(s_f), torch.zeros_like(s_f), torch.exp(s_f - Lz[..., None]))
        if saved_L is not None:
            Lb = saved_L[:, :, r0:r1].float()
            empty = torch.isinf(Lb)
            Lz = torch.where(empty, torch.zeros_like(Lb), Lb)
        p = torch.where(elem & ~empty[..., None], torch.exp(s - Lz[..., None]), torch.zeros_like(s))
        del s, s_f
        dp = torch.matmul(dof[:, :, r0:r1], vf[:, :, :n1].transpose(2, 3))
        for rounded, acc in zip((True, False), res):
            lp = (lambda x: x.to(dt).float()) if rounded else (lambda x: x)
            out = torch.matmul(lp(p_f), vf[:, :, :n1])
            out_used = lp(out)
            out_bwd = out_used if saved_out is None else saved_out[:, :, r0:r1].float()
            delta = (out_bwd * dof[:, :, r0:r1]).sum(-1)
            ds = p * (dp - delta[..., None])
            p_kv, ds_kv = (p, ds) if kv_keep is None else (p * kv_keep, ds * kv_keep)
            ds_q = ds if fwd_keep is None else ds * fwd_keep
            acc["out"][:, :, r0:r1] = out_used
            acc["L"][:, :, r0:r1] = L
            acc["dv"][:, :, :n1] += torch.matmul(lp(p_kv).transpose(2, 3), dof[:, :, r0:r1])
            acc["dk"][:, :, :n1] += torch.matmul(lp(ds_kv).transpose(2, 3), qf[:, :, r0:r1]) * sm_scale
            acc["dq"][:, :, r0:r1] = torch.matmul(lp(ds_q), kf[:, :, :n1]) * sm_scale
            acc["dlam"][:, :, :n1] -= ds_kv.sum(dim=2)
            acc["dlam"][:, :, P + r0:P + r1] += ds_q.sum(dim=3)
            del ds, ds_q, ds_kv, p_kv, out
    for rounded, acc in zip((True, False), res):
        if seq_start is not None:
            colmask = (cols[None, None, :] >= seq_start[:, None, None])[..., None]
            acc["dk"] *= colmask
            acc["dv"] *= colmask
        acc["dlog_fgate"] = reverse_cumsum(acc.pop("dlam"))
        if rounded:
            for n_ in ("out", "dq", "dk", "dv"):
                acc[n_] = acc[n_].to(dt)
    return res[0], res[1]


def pruned_tile_fraction(start_index: np.ndarray, M: int, N: int, BM: int, BN: int,
                         seq_start: Optional[np.ndarray] = None) -> float:
    """Fraction of causal (q-block, kv-block) tiles the forward skips because of the
    index array: sum(min(start_index, hi)//BN) / sum(ceil(hi/BN))."""
    P = N - M
    nmb = start_index.shape[-1]
    hi = np.minimum(N, P + (np.arange(nmb) + 1) * BM)
    total = np.ceil(hi / BN).sum() * start_index.shape[0] * start_index.shape[1]
    skipped = (np.minimum(start_index, hi[None, None, :]) // BN).sum()
    return float(skipped) / float(total)


# --------------------------------------------------------------------------
# fused RMSNorm + sigmoid output gate (FNG:18-53 with is_rms_norm, no bias/residual)
# --------------------------------------------------------------------------
def group_rmsnorm_gated(x: torch.Tensor, g: torch.Tensor, weight: torch.Tensor, num_groups: int,
                        eps: float = 1e-6, upcast: bool = True) -> torch.Tensor:
    """y = rmsnorm_per_group(x) * weight * sigmoid(g), cast back to x.dtype.
    x, g (..., G*D); weight (G*D,)."""
    dtype = x.dtype
    if upcast:
        x, g, weight = x.float(), g.float(), weight.float()
    shp = x.shape
    xg = x.reshape(*shp[:-1], num_groups, shp[-1] // num_groups)
    wg = weight.reshape(num_groups, -1)
    rstd = 1 / torch.sqrt(xg.square().mean(dim=-1, keepdim=True) + eps)
    out = (xg * rstd * wg).reshape(shp)
    out = out * torch.sigmoid(g)
    return out.to(dtype)


def group_rmsnorm_gated_fwd_bwd(x, g, weight, dy, num_groups, eps=1e-6):
    x, g, weight = [t.detach().clone().requires_grad_() for t in (x, g, weight)]
    y = group_rmsnorm_gated(x, g, weight, num_groups, eps)
    y.backward(dy)
    return y.detach(), x.grad, g.grad, weight.grad


def group_rmsnorm(x: torch.Tensor, weight: torch.Tensor, num_groups: int, eps: float = 1e-5,
                  upcast: bool = True) -> torch.Tensor:
    """y = rmsnorm_per_group(x) * weight, cast back to x.dtype: group_norm_ref with
    is_rms_norm=True, no bias, no residual (layernorm.py:77-110), the FoX layer's QK-norm."""
    dtype = x.dtype
    if upcast:
        x, weight = x.float(), weight.float()
    shp = x.shape
    xg = x.reshape(*shp[:-1], num_groups, shp[-1] // num_groups)
    rstd = 1 / torch.sqrt(xg.square().mean(dim=-1, keepdim=True) + eps)
    return (xg * rstd * weight.reshape(num_groups, -1)).reshape(shp).to(dtype)


def group_rmsnorm_fwd_bwd(x, weight, dy, num_groups, eps=1e-5):
    x, weight = [t.detach().clone().requires_grad_() for t in (x, weight)]
    y = group_rmsnorm(x, weight, num_groups, eps)
    y.backward(dy)
    return y.detach(), x.grad, weight.grad


def token_shift(x: torch.Tensor, prev_weight: torch.Tensor, curr_weight: torch.Tensor) -> torch.Tensor:
    """out[b,t,h,:] = x[b,t,h,:] curr[b,t,h] + x[b,t-1,h,:] prev[b,t,h] (x[b,-1] = 0), products in fp32,
    one rounding to x.dtype: the arithmetic of shift_fwd_kernel (token_shift.py:66-67)."""
    xf = x.float()
    x_prev = torch.nn.functional.pad(xf, (0, 0, 0, 0, 1, 0))[:, :-1]
    out = xf * curr_weight.float()[..., None] + x_prev * prev_weight.float()[..., None]
    return out.to(x.dtype)


def token_shift_fwd_bwd(x, prev_weight, curr_weight, dout):
    """Gradients with the kernel's roundings (token_shift.py:138-144): dx rounded to x.dtype from fp32
    products; weight gradients summed in fp32 from the 16-bit dout and x."""
    out = token_shift(x, prev_weight, curr_weight)
    df, xf = dout.float(), x.float()
    d_next = torch.nn.functional.pad(df, (0, 0, 0, 0, 0, 1))[:, 1:]
    p_next = torch.nn.functional.pad(prev_weight.float(), (0, 0, 0, 1))[:, 1:]
    dx = (df * curr_weight.float()[..., None] + d_next * p_next[..., None]).to(x.dtype)
    x_prev = torch.nn.functional.pad(xf, (0, 0, 0, 0, 1, 0))[:, :-1]
    dcurr = (df * xf).sum(-1)
    dprev = (df * x_prev).sum(-1)
    return out, dx, dprev, dcurr


def rms_norm(x, weight, residual=None, eps: float = 1e-5, prenorm: bool = False):
    """Row-wise RMSNorm with optional residual add as upstream's kernel computes it (layernorm.py:287-313):
    the sum x + residual is formed and normalised in fp32, its rounded copy is what prenorm returns."""
    z = x.float() if residual is None else x.float() + residual.float()
    rstd = 1 / torch.sqrt(z.square().mean(dim=-1, keepdim=True) + eps)
    y = (z * rstd * weight.float()).to(x.dtype)
    return (y, z.to(x.dtype)) if prenorm else y


def rms_norm_fwd_bwd(x, weight, residual, dy, dres, eps=1e-5):
    """Gradients as upstream's backward forms them (layernorm.py:380-416): from the saved, rounded sum."""
    y, zs = rms_norm(x, weight, residual, eps, prenorm=True)
    z = zs.float()
    rstd = 1 / torch.sqrt(z.square().mean(dim=-1, keepdim=True) + eps)
    xhat = z * rstd
    wdy = weight.float() * dy.float()
    c1 = (xhat * wdy).mean(dim=-1, keepdim=True)
    dx = (wdy - xhat * c1) * rstd
    if dres is not None:
        dx = dx + dres.float()
    dw = (dy.float() * xhat).reshape(-1, x.shape[-1]).sum(0)
    return y, zs, dx.to(x.dtype), dw


def fox_pro_block(x, weights: dict, num_heads: int, eps: float = 1e-6, attention_mask=None):
    """fp32 restatement of the FoX-Pro block's data flow (modeling_forgetting_transformer.py:44-95,
    300-430, 505-516, 565-588) from a dict of weights: attn_norm, q, k, k_shift, v, v_shift, q_norm, k_norm,
    fgate_w, fgate_b, ogate, out_norm, o, mlp_norm, gate, down.  Every operator is this module's own
    reference; the matrix products are plain fp32 matmuls."""
    W = {n: t.float() for n, t in weights.items()}
    x = x.float()
    B, T, C = x.shape
    H, D = num_heads, C // num_heads
    residual = x
    h = rms_norm(x, W["attn_norm"], None, eps)
    q = h @ W["q"].T

    def shifted(w, w_shift):
        out = (h @ w.T).view(B, T, H, D)
        alpha = torch.sigmoid(h @ w_shift.T)
        if attention_mask is not None:
            out = torch.where(attention_mask[:, :, None, None].bool(), out, 0.0)
        return token_shift(out, alpha, 1.0 - alpha).reshape(B, T, C)

    k = shifted(W["k"], W["k_shift"])
    v = shifted(W["v"], W["v_shift"])
    q = group_rmsnorm(q, W["q_norm"], H, 1e-5)
    k = group_rmsnorm(k, W["k_norm"], H, 1e-5)
    log_fgate = torch.nn.functional.logsigmoid(h @ W["fgate_w"].T + W["fgate_b"]).transpose(1, 2)
    qh, kh, vh = [t.view(B, T, H, D).transpose(1, 2) for t in (q, k, v)]
    seq_start = None if attention_mask is None else attention_mask.shape[-1] - attention_mask.sum(-1)
    o = dense_forgetting_attention(qh, kh, vh, log_fgate, seq_start=seq_start, sm_scale=1 / math.sqrt(D))
    o = o.transpose(1, 2).reshape(B, T, C)
    o = group_rmsnorm_gated(o, h @ W["ogate"].T, W["out_norm"], H, eps)
    attn_out = o @ W["o"].T
    h2, residual = rms_norm(attn_out, W["mlp_norm"], residual, eps, prenorm=True)
    gate, y = (h2 @ W["gate"].T).chunk(2, -1)
    return residual + (torch.nn.functional.silu(gate) * y) @ W["down"].T


def swiglu(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """z = x sigmoid(x) y in fp32, one rounding (glu_linear.py:64-68)."""
    xf = x.float()
    return (xf * y.float() / (1.0 + torch.exp(-xf))).to(x.dtype)


def swiglu_bwd(x, y, g):
    """dx, dy, z with upstream's expressions (glu_linear.py:78-86)."""
    xf, yf, gf = x.float(), y.float(), g.float()
    s = 1.0 / (1.0 + torch.exp(-xf))
    dx = s * (1 + xf * (1.0 - s)) * gf * yf
    dy = xf * s * gf
    return dx.to(x.dtype), dy.to(x.dtype), (xf * s * yf).to(x.dtype)


# --------------------------------------------------------------------------
# cross-entropy loss (fused_cross_entropy.py:24-134, without the tensor-parallel class split)
# --------------------------------------------------------------------------
def cross_entropy(logits: torch.Tensor, target: torch.Tensor, label_smoothing: float = 0.0, logit_scale: float = 1.0,
                  lse_square_scale: float = 0.0, ignore_index: int = -100):
    """(losses, z_losses), fp32 (rows,): lse - (1 - eps) z[label] - eps mean(z) + s lse^2 with z = logit_scale *
    logits in fp32; rows whose label is ``ignore_index`` give 0 (fused_cross_entropy.py:47-87)."""
    z = logits.float() * logit_scale
    lse = torch.logsumexp(z, dim=-1)
    keep = target != ignore_index
    safe = torch.where(keep, target, torch.zeros_like(target))
    zlab = z.gather(1, safe[:, None])[:, 0]
    loss = lse - (1.0 - label_smoothing) * zlab - label_smoothing * z.mean(dim=-1)
    zl = lse_square_scale * lse * lse
    zero = torch.zeros_like(loss)
    return torch.where(keep, loss + zl, zero), torch.where(keep, zl, zero)


def cross_entropy_class_shard(logits_shard: torch.Tensor, target: torch.Tensor, class_start: int, total_classes: int,
                              label_smoothing: float = 0.0, logit_scale: float = 1.0, ignore_index: int = -100):
    """What one rank contributes when the classes are split over ranks (fused_cross_entropy.py:84-92, 196-205):
    (loss_parts, lse_local) with loss_parts = -(1 - eps) z[label] [label on this rank] - eps sum(z) / total_classes,
    0 where the label is ``ignore_index``; the global loss is sum over ranks of loss_parts + logsumexp of the ranks'
    lse_local (+ the z-loss of that global lse)."""
    z = logits_shard.float() * logit_scale
    lse = torch.logsumexp(z, dim=-1)
    local = target - class_start
    mine = (target != ignore_index) & (local >= 0) & (local < z.shape[1])
    safe = torch.where(mine, local, torch.zeros_like(local))
    zlab = torch.where(mine, z.gather(1, safe[:, None])[:, 0], torch.zeros_like(lse))
    parts = -(1.0 - label_smoothing) * zlab - label_smoothing * z.sum(dim=-1) / total_classes
    return torch.where(target != ignore_index, parts, torch.zeros_like(parts)), lse


def cross_entropy_fwd_bwd(logits, target, dloss, **kw):
    """losses, z_losses and d(sum(losses * dloss)) / dlogits in fp32."""
    x = logits.detach().float().requires_grad_()
    losses, zl = cross_entropy(x, target, **kw)
    (losses * dloss).sum().backward()
    return losses.detach(), zl.detach(), x.grad
