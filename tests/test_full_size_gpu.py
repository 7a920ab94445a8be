"""Parity at the benchmark's full sequence lengths (B200): one or two (batch, head) units of the T = 16384 and
T = 65536 configurations through the C ABI against the CPU oracle evaluated in row chunks
(``oracle.chunked_fwd_bwd``: the dense formulation of forgetting_attention.py:1380-1404 with explicit gradients).

Every element of out, dq, dk, dv and dlog_fgate must lie within 2e-2 + 1e-2 |ref| of the reference arithmetic
(fp32 with upstream's roundings of P and dS to the input dtype); the backward is differentiated through the
tensors the forward saved (its 16-bit out, its log-normaliser, its fp32 prefix sum), as upstream's backward is.
The fp32 by-products: the prefix sum against a float64 prefix sum, the log-normaliser within 1e-4 relative of the
fp32 path on the same prefix sum (at T = 16384 with strong decay the prefix reaches -2.4e4, where one fp32 ulp is
2e-3: two fp32 prefix sums that add in different orders already move every logit by that much).  The measured
worst errors, and how far kernels and reference arithmetic are from the unrounded fp32 path, are printed
(pytest -s shows them).
"""
import math

import numpy as np
import pytest
import torch

import forgetting_transformer_b200 as fox
from forgetting_transformer_b200 import _lib, ops
from oracle import fox_oracle as orc
from test_attention_gpu import ATOL_BF16, RTOL_BF16, RTOL_FP32, _bars, _close, _no_worse_than

pytestmark = pytest.mark.gpu


def _unit(seed, H, M, N, D, mu, sigma, head_scale=None):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(1, H, M, D, generator=g)
    k = torch.randn(1, H, N, D, generator=g)
    v = torch.randn(1, H, N, D, generator=g)
    lf = torch.nn.functional.logsigmoid(torch.randn(1, H, N, generator=g) * sigma + mu)
    do = torch.randn(1, H, M, D, generator=g)
    if head_scale is not None:
        s = torch.tensor(head_scale).view(1, H, 1, 1)
        q, k, v = q * s, k * s, v * s
    return [t.bfloat16() for t in (q, k, v)] + [lf, do.bfloat16()]


def _gpu(q, k, v, lf, do, seq=None, thr=None):
    qq, kk, vv, ll = [t.cuda().requires_grad_() for t in (q, k, v, lf)]
    ss = None if seq is None else seq.cuda()
    out, L, si = ops.ForgettingAttention.apply(qq, kk, vv, ll, ss, True, None, thr, True, thr is not None, None,
                                               False, False)
    out.backward(do.cuda())
    lam = ops.log_lambda_cumsum(ll.detach(), ss)      # the same kernel call the forward made
    torch.cuda.synchronize()
    _lib.check_status()
    got = dict(out=out.detach().cpu(), L=L.cpu(), dq=qq.grad.cpu(), dk=kk.grad.cpu(), dv=vv.grad.cpu(),
               dlog_fgate=ll.grad.cpu(), lam=lam.cpu())
    return got, (None if si is None else si.cpu())


def _oracle(got, q, k, v, lf, do, **kw):
    """Reference arithmetic and fp32 path on the call's own prefix sum, backward through its saved out and L;
    also checks that prefix sum against a float64 one."""
    ref64 = torch.cumsum(orc.masked_log_fgate(lf, kw.get("seq_start")).double(), dim=-1)
    err = (got["lam"].double() - ref64).abs().max().item()
    print(f"prefix sum: max |Lambda| {ref64.abs().max().item():.1f}, max abs err vs float64 {err:.2e}")
    assert err <= 1e-5 * ref64.abs().max().item() + 1e-5
    return orc.chunked_fwd_bwd(q, k, v, lf, do, lam=got["lam"], saved_out=got["out"], saved_L=got["L"], **kw)


def _compare(label, got, rounded, fp32):
    report = {}
    for name in ("out", "dq", "dk", "dv", "dlog_fgate"):
        report[name] = dict(max_abs_err=(got[name].float() - rounded[name].float()).abs().max().item(),
                            bars=_bars(got[name], rounded[name]),
                            bars_from_fp32_path=_bars(got[name], fp32[name]),
                            reference_arithmetic_bars_from_fp32_path=_bars(rounded[name], fp32[name]))
    print(label, {n: {k_: round(v_, 4) for k_, v_ in r.items()} for n, r in report.items()})
    fin = torch.isfinite(fp32["L"])
    assert torch.equal(torch.isfinite(got["L"]), fin)
    _close(got["L"][fin], fp32["L"][fin], 1e-4, RTOL_FP32, "L")
    for name in ("out", "dq", "dk", "dv", "dlog_fgate"):
        _close(got[name], rounded[name], ATOL_BF16, RTOL_BF16, f"{label} {name}")
    _no_worse_than(got["out"], rounded["out"], fp32["out"], f"{label} out")


def test_long_context_unit_t16384_d64_with_seq_start():
    """One (batch, head) unit of the long-context configuration (B2 T16384 H24 D64, gate logits N(4,1),
    seq_start drawn in [0, 2048)), every query row."""
    q, k, v, lf, do = _unit(1003, 1, 16384, 16384, 64, 4.0, 1.0)
    seq = torch.tensor([1531])
    got, _ = _gpu(q, k, v, lf, do, seq)
    rounded, fp32 = _oracle(got, q, k, v, lf, do, seq_start=seq, row_chunk=2048)
    _compare("T16384 D64 seq_start", got, rounded, fp32)
    assert torch.all(got["out"][0, :, :1531] == 0) and torch.all(got["dk"][0, :, :1531] == 0)


@pytest.mark.parametrize("pruning", [None, "auto"])
def test_pruning_stress_unit_t16384_d128(pruning):
    """One (batch, head) unit of the pruning stress configuration (B4 T16384 H16 D128, gate logits
    N(-1,1.5), per-head input scales from [0.5, 2]), pruning off and with adaptive_threshold="auto"; with
    pruning the oracle skips exactly the tiles its own index arrays name, and those arrays must be the
    operator's."""
    q, k, v, lf, do = _unit(1004, 1, 16384, 16384, 128, -1.0, 1.5, head_scale=[0.8 if pruning is None else 1.7])
    got, si_gpu = _gpu(q, k, v, lf, do, thr=pruning)
    si = ei = None
    if pruning is not None:
        thr = orc.auto_threshold(q, k, 128 ** -0.5).numpy()
        lam = got["lam"].numpy()
        si = orc.find_start_index(lam, thr, 16384, 16384, 128, 128)
        ei = orc.find_end_index(lam, thr, 16384, 16384, 128, 128)
        frac = orc.pruned_tile_fraction(si, 16384, 16384, 128, 128)
        differing = int((si_gpu.numpy() != si).sum())
        print(f"pruned tile fraction {frac:.4f}; start_index entries differing from the oracle's: {differing} of {si.size}")
        assert frac > 0.9 and differing == 0
    rounded, fp32 = _oracle(got, q, k, v, lf, do, start_index=si, end_index=ei, row_chunk=2048)
    _compare(f"T16384 D128 pruning={pruning}", got, rounded, fp32)


def test_fox_pro_attention_unit_t65536_last_rows():
    """One head of the FoX-Pro block's attention shape (B1 T65536 H24 D64, gate logits N(5,1)): the last 2048
    query rows against all 65536 keys (seqlen_q < seqlen_k through the same kernels)."""
    q, k, v, lf, do = _unit(1005, 1, 2048, 65536, 64, 5.0, 1.0)
    got, _ = _gpu(q, k, v, lf, do)
    rounded, fp32 = _oracle(got, q, k, v, lf, do, row_chunk=1024)
    _compare("T65536 D64 last 2048 rows", got, rounded, fp32)
