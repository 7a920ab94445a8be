"""GPU parity tests (B200): the CUDA path, called through the C ABI, against the CPU
oracle on the same seeded inputs, against the golden fixtures produced by upstream's
own kernels, and through size-independent properties at the benchmark's full sizes."""
import math

import numpy as np
import pytest
import torch

import forgetting_transformer_b200 as fox
from forgetting_transformer_b200 import _lib, ops
from oracle import fox_oracle as orc

pytestmark = pytest.mark.gpu

# Tolerances.  fp16: upstream's own known-answer bar, atol 1e-2 on every element (forgetting_attention.py:1425).
# bf16: every element within |a - b| <= 2e-2 + 1e-2 |ref| of the reference arithmetic, i.e. the fp32 formulation with
# the roundings upstream's kernels make (probabilities and dS cast to the input dtype before their products,
# lines 666, 1101, 1121, 1325) -- ``blockwise_fwd_bwd`` with its default ``low_precision_matmul=True``.
# The backward is checked as the function of the forward's saved tensors that it is (lines 207, 241): the oracle
# differentiates through the 16-bit ``out`` and the log-normaliser the kernels themselves produced, and through
# their fp32 prefix sum.  Otherwise the comparison measures something else: any two correct 16-bit forwards round
# ``out`` differently, delta = rowsum(out * dout) carries that rounding (a few 1e-2 at these shapes) into every dS,
# and the gate gradient -- whose query-side half is exactly that residue -- differs by 2 to 4 bars between two
# correct implementations (upstream's Triton kernel against its own PyTorch path included).
# fp32 by-products (prefix sum, log-normaliser): 1e-4 relative to the fp32 path.
ATOL_FP16 = 1e-2
ATOL_BF16, RTOL_BF16 = 2e-2, 1e-2
RTOL_FP32 = 1e-4


def _close(a, b, atol, rtol=0.0, what=""):
    """Every element within atol + rtol * |reference element|."""
    a, b = a.float().cpu(), b.float().cpu()
    assert a.shape == b.shape
    assert not torch.isnan(a).any()
    if a.numel() == 0:
        return
    err = (a - b).abs()
    excess = err - (atol + rtol * b.abs())
    worst = int(excess.argmax())
    assert excess.flatten()[worst].item() <= 0, (
        f"{what} element {worst}: |{a.flatten()[worst].item():.5f} - {b.flatten()[worst].item():.5f}| = "
        f"{err.flatten()[worst].item():.3e} > {atol} + {rtol} * |ref|; max abs err {err.max().item():.3e}, "
        f"{int((excess > 0).sum())} of {a.numel()} elements over the bar")


def _bars(a, b, atol=ATOL_BF16, rtol=RTOL_BF16):
    """Largest error of any element in units of its own bar atol + rtol * |ref|."""
    a, b = a.float().cpu(), b.float().cpu()
    return ((a - b).abs() / (atol + rtol * b.abs())).max().item() if a.numel() else 0.0


def _no_worse_than(a, rounded_ref, fp32_ref, what=""):
    """Against the unrounded fp32 path the kernel may be as far off as the reference arithmetic itself is (plus
    half a bar for the different summation order), never more."""
    ours, theirs = _bars(a, fp32_ref), _bars(rounded_ref, fp32_ref)
    assert ours <= theirs + 0.5, f"{what}: {ours:.2f} bars from the fp32 path, reference arithmetic {theirs:.2f}"


class _Result(tuple):
    """(out, dq, dk, dv, dlog_fgate) of one call, plus what the forward saved: .L and .lam (CPU tensors)."""


def _run(q, k, v, lf, do, seq=None, sm_scale=None, thr=None):
    dev = "cuda"
    qq, kk, vv, ll = [t.to(dev).detach().requires_grad_() for t in (q, k, v, lf)]
    ss = None if seq is None else seq.to(dev)
    th = thr.to(dev) if isinstance(thr, torch.Tensor) else thr
    out, L, _ = ops.ForgettingAttention.apply(qq, kk, vv, ll, ss, True, sm_scale, th, True, False, None, False, False)
    out.backward(do.to(dev))
    lam = ops.log_lambda_cumsum(ll.detach(), ss)      # the same kernel call the forward made
    torch.cuda.synchronize()
    _lib.check_status()
    res = _Result((out.detach().cpu(), qq.grad.cpu(), kk.grad.cpu(), vv.grad.cpu(), ll.grad.cpu()))
    res.L, res.lam = L.cpu(), lam.cpu()
    return res


def _check_bf16(got, q, k, v, lf, do, seq=None, sm_scale=None, **prune):
    """One 16-bit call against the reference arithmetic, every element within the bar: the forward (out, and L
    against the fp32 path) on the call's own prefix sum, the backward through the call's own saved out and L."""
    r = orc.blockwise_fwd_bwd(q, k, v, lf, do, seq, sm_scale, lam=got.lam, saved_out=got[0], saved_L=got.L, **prune)
    atol, rtol = (ATOL_BF16, RTOL_BF16) if q.dtype == torch.bfloat16 else (ATOL_FP16, 0.0)
    fin = torch.isfinite(r["L"])
    assert torch.equal(torch.isfinite(got.L), fin)
    _close(got.L[fin], r["L"][fin], 1e-4, RTOL_FP32, "L")
    for name, a in zip(("out", "dq", "dk", "dv", "dlog_fgate"), got):
        _close(a, r[name], atol, rtol, name)
    if q.dtype == torch.bfloat16:
        f = orc.blockwise_fwd_bwd(q, k, v, lf, do, seq, sm_scale, low_precision_matmul=False, lam=got.lam, **prune)
        _no_worse_than(got[0], r["out"], f["out"], "out")
    return r


def _inputs(seed, B, H, M, N, D, dtype, mu=0.0, sigma=1.0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, H, M, D, generator=g) * std).to(dtype)
    k = (torch.randn(B, H, N, D, generator=g) * std).to(dtype)
    v = (torch.randn(B, H, N, D, generator=g) * std).to(dtype)
    lf = torch.nn.functional.logsigmoid(torch.randn(B, H, N, generator=g) * sigma + mu)
    do = torch.randn(B, H, M, D, generator=g).to(dtype)
    return q, k, v, lf, do


# ------------------------------------------------------------------ golden fixtures
def test_against_upstream_kernel_outputs(golden):
    """Same inputs as upstream's Triton kernels were run on (fp16): outputs, log-normaliser
    and all four gradients within upstream's own tolerance; pruning indices identical."""
    g = golden
    dev = "cuda"
    B, H, M, D = g["q"].shape
    N = g["k"].shape[2]
    qq, kk, vv, ll = [g[n].to(dev).requires_grad_() for n in ("q", "k", "v", "log_fgate")]
    ss = None if g["seq_start"] is None else g["seq_start"].to(dev)
    thr = None if g["threshold"] is None else g["threshold"].to(dev)
    out, L, si = ops.ForgettingAttention.apply(qq, kk, vv, ll, ss, True, g["sm_scale"], thr, True,
                                               thr is not None, None, False, False)
    out.backward(g["dout"].to(dev))
    torch.cuda.synchronize()
    _lib.check_status()
    _close(out, g["out"], 2e-3)
    fin = torch.isfinite(g["L"])
    assert torch.equal(torch.isfinite(L.cpu()), fin)
    _close(L.cpu()[fin], g["L"][fin], 1e-3, RTOL_FP32)
    _close(qq.grad, g["dq"], 4e-3)
    _close(kk.grad, g["dk"], 4e-3)
    _close(vv.grad, g["dv"], 4e-3)
    _close(ll.grad, g["dlog_fgate"], ATOL_FP16)
    if thr is not None:
        assert torch.equal(si.cpu(), g["start_index"])


# --------------------------------------------------- upstream's own known-answer grid
@pytest.mark.parametrize("Z,H,M,N,D", [(4, 2, 1020, 2098, 64), (4, 2, 1024, 2048, 128)])
@pytest.mark.parametrize("fgate_logit_range", [(0, 5), (5, 10)])
@pytest.mark.parametrize("has_seq_start", [True, False])
@pytest.mark.parametrize("adaptive_threshold", [-10.0, None, "per_head"])
def test_upstream_known_answer_grid(Z, H, M, N, D, fgate_logit_range, has_seq_start, adaptive_threshold):
    """The parametrisation of upstream's in-file test_op (forgetting_attention.py:1360-1425):
    fp16, q/k/v ~ N(0, 0.5^2), sm_scale 0.5, atol 1e-2, against the dense formulation."""
    g = torch.Generator().manual_seed(24)
    dtype = torch.float16
    q = torch.empty(Z, H, M, D).normal_(0.0, 0.5, generator=g).to(dtype)
    k = torch.empty(Z, H, N, D).normal_(0.0, 0.5, generator=g).to(dtype)
    v = torch.empty(Z, H, N, D).normal_(0.0, 0.5, generator=g).to(dtype)
    lf = torch.nn.functional.logsigmoid(torch.empty(Z, H, N).uniform_(*fgate_logit_range, generator=g))
    seq = torch.randint(0, N, (Z,), generator=g) if has_seq_start else None
    do = torch.randn(Z, H, M, D, generator=g).to(dtype)
    thr = torch.tensor([-1000.0, -100.0]) if adaptive_threshold == "per_head" else adaptive_threshold
    got = _run(q, k, v, lf, do, seq, 0.5, thr)
    out, dq, dk, dv, dlf = got
    ro, rdq, rdk, rdv, rdl = orc.dense_fwd_bwd(q.float(), k.float(), v.float(), lf, do.float(), seq, 0.5)
    _close(out, ro, ATOL_FP16)
    _close(dv, rdv, ATOL_FP16)
    _close(dk, rdk, ATOL_FP16)
    _close(dq, rdq, ATOL_FP16)
    _close(dlf, rdl, ATOL_FP16)


# ------------------------------------------------------------- benchmark configs 1, 2
def test_config1_fp32_reference_case():
    """B=2, T=256, H=4, D=64, seq_start=[0, 37], sm_scale=1/8: the CPU fp32 formulation
    against the fp16 kernels (4e-3 on every element), the reference arithmetic against the bf16 kernels."""
    q, k, v, lf, do = _inputs(1001, 2, 4, 256, 256, 64, torch.float16)
    seq = torch.tensor([0, 37])
    got = _run(q, k, v, lf, do, seq, 1 / 8)
    out, dq, dk, dv, dlf = got
    ro, rdq, rdk, rdv, rdl = orc.dense_fwd_bwd(q.float(), k.float(), v.float(), lf, do.float(), seq, 1 / 8, True)
    for a, b in [(out, ro), (dq, rdq), (dk, rdk), (dv, rdv)]:
        _close(a, b, 4e-3)
    _close(dlf, rdl, 8e-3)
    assert torch.all(out[1, :, :37] == 0)
    q, k, v, lf, do = _inputs(1001, 2, 4, 256, 256, 64, torch.bfloat16)
    got = _run(q, k, v, lf, do, seq, 1 / 8)
    _check_bf16(got, q, k, v, lf, do, seq, 1 / 8)
    assert torch.all(got[0][1, :, :37] == 0)


def test_config2_bf16_kernel_case():
    """B=4, T=512, H=12, D=64 bf16, no seq_start, no pruning (every element within 2e-2 + 1e-2 |ref|)."""
    q, k, v, lf, do = _inputs(1002, 4, 12, 512, 512, 64, torch.bfloat16)
    _check_bf16(_run(q, k, v, lf, do), q, k, v, lf, do)


def test_fp32_byproducts_match_fp32_path():
    """Prefix sum and log-normaliser are fp32 quantities: 1e-4 relative to the fp32 path."""
    q, k, v, lf, do = _inputs(5, 2, 3, 700, 700, 64, torch.bfloat16, mu=2.0)
    seq = torch.tensor([0, 300])
    lam = ops.log_lambda_cumsum(lf.cuda(), seq.cuda()).cpu()
    ref = orc.log_lambda(lf, seq)
    _close(lam, ref, 1e-5, RTOL_FP32)
    out, L, _ = ops.ForgettingAttention.apply(q.cuda(), k.cuda(), v.cuda(), lf.cuda(), seq.cuda(), True, None,
                                              None, True, False, None, False, False)
    r = orc.blockwise_fwd_bwd(q, k, v, lf, do, seq, low_precision_matmul=False)
    fin = torch.isfinite(r["L"])
    assert torch.equal(torch.isfinite(L.cpu()), fin)
    _close(L.cpu()[fin], r["L"][fin], 1e-4, RTOL_FP32)


# ---------------------------------------------------------------------- edge cases
@pytest.mark.parametrize("T", [1, 7, 127, 128, 129, 300])
@pytest.mark.parametrize("D", [64, 128])
def test_small_and_ragged_lengths(T, D):
    q, k, v, lf, do = _inputs(T + D, 2, 2, T, T, D, torch.bfloat16)
    got = _run(q, k, v, lf, do)
    out, dq, dk, dv, dlf = got
    _check_bf16(got, q, k, v, lf, do)


@pytest.mark.parametrize("D", [16, 32])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_small_head_dims(D, dtype):
    """Head dims 16 and 32 of upstream's contract (line 87): same results as the oracle at that D,
    default sm_scale = 1/sqrt(D), gradients of the input's own shape."""
    q, k, v, lf, do = _inputs(7 * D, 2, 3, 200, 333, D, dtype)
    seq = torch.tensor([0, 21])
    got = _run(q, k, v, lf, do, seq=seq)
    out, dq, dk, dv, dlf = got
    assert out.shape == q.shape and dq.shape == q.shape and dk.shape == k.shape and dv.shape == v.shape
    _check_bf16(got, q, k, v, lf, do, seq)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("two_kernel", [True, False])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_backward_formulations(D, two_kernel, dtype, monkeypatch):
    """The backward exists as one pass over (KV tile, query tile) pairs and as a key-side kernel plus a
    query-side kernel (upstream's split, forgetting_attention.py:956-1344); both forms at both head dims, with
    seqlen_q < seqlen_k, seq_start and pruning, against the same oracle and with upstream's 1e-2 on the gate
    gradient (the two halves of the gate gradient come from different kernels in the second form)."""
    monkeypatch.setattr(ops, "_TWO_KERNEL_BACKWARD_DIMS", {64, 128} if two_kernel else set())
    q, k, v, lf, do = _inputs(91 + D, 2, 2, 640, 1100, D, dtype, mu=2.0, std=0.5)
    seq = torch.tensor([0, 333])
    for thr in (None, -12.0):
        got = _run(q, k, v, lf, do, seq=seq, sm_scale=0.5, thr=thr)
        if dtype == torch.bfloat16:   # (what a threshold of -12 prunes carries less than e^-12 of a row's mass)
            _check_bf16(got, q, k, v, lf, do, seq, 0.5)
        else:
            ref = orc.dense_fwd_bwd(q.float(), k.float(), v.float(), lf, do.float(), seq, 0.5)
            for name, a, b in zip(("out", "dq", "dk", "dv", "dlog_fgate"), got, ref):
                _close(a, b, ATOL_FP16, 0.0, name)


def test_seq_start_extremes():
    """seq_start = 0, in the middle of a block, on a block boundary and at the last token."""
    B, H, T, D = 4, 2, 384, 64
    q, k, v, lf, do = _inputs(11, B, H, T, T, D, torch.bfloat16)
    seq = torch.tensor([0, 200, 256, T - 1])
    got = _run(q, k, v, lf, do, seq)
    out, dq, dk, dv, dlf = got
    _check_bf16(got, q, k, v, lf, do, seq)
    for b in range(B):
        s = int(seq[b])
        assert torch.all(out[b, :, :s] == 0) and torch.all(dk[b, :, :s] == 0) and torch.all(dv[b, :, :s] == 0)
    # the last row of batch 3 attends to itself only
    _close(out[3, :, T - 1], v[3, :, T - 1], 1e-2)


def test_seq_len_q_shorter_than_kv():
    q, k, v, lf, do = _inputs(12, 2, 2, 130, 517, 64, torch.bfloat16, mu=1.0)
    seq = torch.tensor([3, 400])
    got = _run(q, k, v, lf, do, seq)
    out, dq, dk, dv, dlf = got
    _check_bf16(got, q, k, v, lf, do, seq)


@pytest.mark.parametrize("N,D", [(777, 64), (1, 64), (4099, 128)])
def test_single_query_decode_step(N, D):
    """One new token against a cache of N keys (generation, OPS:148-153): seqlen_q = 1 goes through the
    same kernels; forward output and, for completeness, the gradients."""
    q, k, v, lf, do = _inputs(N + D, 2, 3, 1, N, D, torch.bfloat16, mu=2.0)
    seq = torch.tensor([0, min(5, N - 1)])
    got = _run(q, k, v, lf, do, seq)
    out, dq, dk, dv, dlf = got
    _check_bf16(got, q, k, v, lf, do, seq)


@pytest.mark.parametrize("N,D,dtype", [(1, 64, torch.bfloat16), (777, 64, torch.bfloat16), (5000, 128, torch.float16),
                                       (20000, 64, torch.bfloat16)])
@pytest.mark.parametrize("thr", [None, -15.0])
def test_decode_kernels_match_the_general_forward(N, D, dtype, thr):
    """Without gradients a single-query call takes the split-KV decode kernels; with gradients enabled the
    same call goes through the general forward kernel.  Both against the fp32 oracle and each other."""
    q, k, v, lf, _ = _inputs(N + D, 2, 5, 1, N, D, dtype, mu=3.0)
    seq = torch.tensor([0, min(9, N - 1)])
    qc, kc, vc, lc, sc = q.cuda(), k.cuda(), v.cuda(), lf.cuda(), seq.cuda()
    with torch.no_grad():
        out_d, L_d, si_d = ops.ForgettingAttention.apply(qc, kc, vc, lc, sc, True, None, thr, True, thr is not None,
                                                         None, False, False)
    out_g, L_g, _ = ops.ForgettingAttention.apply(qc.requires_grad_(), kc, vc, lc, sc, True, None, thr, True, False,
                                                  None, False, False)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = orc.dense_forgetting_attention(q.float(), k.float(), v.float(), lf, seq_start=seq)
    tol = ATOL_BF16 if dtype == torch.bfloat16 else ATOL_FP16
    if thr is None:
        _close(out_d, ref, tol)
    _close(out_d, out_g.detach(), tol)
    assert (L_d - L_g).abs().max().item() < 1e-3
    assert out_d.shape == q.shape and out_d.dtype == dtype


def test_layout_b_t_h_d_views_and_output_strides():
    """head_first=False hands the kernels permuted views; the output keeps q's layout."""
    B, T, H, D = 2, 320, 3, 64
    g = torch.Generator().manual_seed(13)
    q, k, v, do = [torch.randn(B, T, H, D, generator=g).bfloat16() for _ in range(4)]
    lf = torch.nn.functional.logsigmoid(torch.randn(B, T, H, generator=g) + 1)
    qq, kk, vv, ll = [t.cuda().requires_grad_() for t in (q, k, v, lf)]
    out = fox.forgetting_attention(qq, kk, vv, ll)
    assert out.shape == (B, T, H, D) and out.is_contiguous()
    out.backward(do.cuda())
    _lib.check_status()
    # the same call on head-first contiguous copies: same kernels, same tiles
    ref = _run(*[t.transpose(1, 2).contiguous() for t in (q, k, v)], lf.transpose(1, 2).contiguous(),
               do.transpose(1, 2).contiguous())
    _check_bf16(ref, *[t.transpose(1, 2) for t in (q, k, v)], lf.transpose(1, 2), do.transpose(1, 2))
    assert torch.equal(out.detach().cpu().transpose(1, 2), ref[0])
    assert torch.equal(kk.grad.cpu().transpose(1, 2), ref[2]) and torch.equal(vv.grad.cpu().transpose(1, 2), ref[3])
    # dq and the gate gradient come out of fp32 atomics whose order varies from run to run
    _close(qq.grad.transpose(1, 2), ref[1], 1e-2, 1e-2, "dq")
    _close(ll.grad.transpose(1, 2), ref[4], 1e-2, 1e-2, "dlog_fgate")
    assert ll.grad.shape == lf.shape


@pytest.mark.parametrize("D", [64, 128])
def test_pruned_call_on_b_t_h_d_views_equals_the_head_first_call(D):
    """With a threshold every output tile of the backward leaves through shared memory and TMA stores; on the
    permuted (B, T, H, D) views and a ragged length they must land where the head-first call puts them."""
    B, T, H = 2, 333, 3
    g = torch.Generator().manual_seed(17)
    q, k, v, do = [torch.randn(B, T, H, D, generator=g).bfloat16() for _ in range(4)]
    lf = torch.nn.functional.logsigmoid(torch.randn(B, T, H, generator=g))
    seq = torch.tensor([0, 70])
    outs = []
    for head_first in (False, True):
        args = [t.transpose(1, 2).contiguous() if head_first else t for t in (q, k, v, lf)]
        qq, kk, vv, ll = [t.cuda().requires_grad_() for t in args]
        out = fox.forgetting_attention(qq, kk, vv, ll, head_first=head_first, seq_start=seq.cuda(),
                                       adaptive_threshold=-8.0)
        out.backward((do.transpose(1, 2).contiguous() if head_first else do).cuda())
        _lib.check_status()
        res = [out.detach(), qq.grad, kk.grad, vv.grad, ll.grad]
        outs.append([t.transpose(1, 2) if not head_first else t for t in res])
    for name, a, b in zip(("out", "dq", "dk", "dv", "dlog_fgate"), *outs):
        if name in ("out", "dk", "dv") or D == 128:   # (the one-pass backward adds dq and the gate sums atomically)
            assert torch.equal(a, b), name
        else:
            _close(a, b, 1e-2, 1e-2, name)


def test_threshold_validation():
    q, k, v, lf, do = [t.cuda() for t in _inputs(14, 2, 2, 128, 128, 64, torch.bfloat16)]
    with pytest.raises(AssertionError, match="adaptive_threshold must be either"):
        fox.forgetting_attention(q, k, v, lf, head_first=True, adaptive_threshold="automatic")
    with pytest.raises(RuntimeError, match="broadcastable"):
        fox.forgetting_attention(q, k, v, lf, head_first=True, adaptive_threshold=torch.zeros(3, device="cuda"))


@pytest.mark.parametrize("D,dtype", [(64, torch.bfloat16), (128, torch.float32)])
def test_gate_logits_path_matches_the_log_gate_path(D, dtype):
    """``forgetting_attention_from_gate_logits`` (log sigmoid folded into the prefix-sum kernels) against
    ``forgetting_attention`` on ``F.logsigmoid(logit.float())`` with autograd through the log sigmoid, as upstream's
    layer does it (modeling_forgetting_transformer.py:343-346): the gate projection's (B, T, H) output as it is."""
    B, T, H = 2, 700, 3
    g = torch.Generator().manual_seed(31 + D)
    q, k, v, do = [torch.randn(B, T, H, D, generator=g).bfloat16().cuda() for _ in range(4)]
    logit = (torch.randn(B, T, H, generator=g) * 1.5 + 2).to(dtype).cuda()
    seq = torch.tensor([0, 129]).cuda()
    lam = ops.gate_prefix_from_logits(logit.permute(0, 2, 1), seq)
    ref_lam = orc.log_lambda(torch.nn.functional.logsigmoid(logit.float().cpu().double()).permute(0, 2, 1), seq.cpu())
    assert (lam.cpu().double() - ref_lam).abs().max().item() <= 1e-5 * ref_lam.abs().max().item() + 1e-5
    res = []
    for fused in (False, True):
        qq, kk, vv, ll = [t.detach().clone().requires_grad_() for t in (q, k, v, logit)]
        if fused:
            out = fox.forgetting_attention_from_gate_logits(qq, kk, vv, ll, seq_start=seq, adaptive_threshold=-15.0)
        else:
            out = fox.forgetting_attention(qq, kk, vv, torch.nn.functional.logsigmoid(ll.float()), seq_start=seq,
                                           adaptive_threshold=-15.0)
        out.backward(do)
        res.append((out.detach(), qq.grad, kk.grad, vv.grad, ll.grad))
    torch.cuda.synchronize()
    _lib.check_status()
    assert res[1][4].dtype == dtype and res[1][4].shape == logit.shape
    for name, a, b in zip(("out", "dq", "dk", "dv", "dlogit"), res[1], res[0]):
        _close(a, b, 1e-2, 1e-2, name)     # same kernels; the prefix sums differ in the last bits of log sigmoid


def test_expired_wait_is_reported_at_the_next_call():
    """A kernel that gives up on a bounded wait leaves a record in the device's status words; the operator copies
    them to pinned host memory after every backward and raises at the next call, without any synchronisation of
    its own.  The record is made here by writing the status words from the host (no kernel is made to hang)."""
    q, k, v, lf, do = [t.cuda() for t in _inputs(21, 1, 2, 256, 256, 64, torch.bfloat16)]
    dev = q.device
    for t in (q, k, v, lf):
        t.requires_grad_()
    fox.forgetting_attention(q, k, v, lf, head_first=True).backward(do)
    torch.cuda.synchronize()
    fox.forgetting_attention(q, k, v, lf, head_first=True)          # nothing to report
    _lib.status_buffer(dev).copy_(torch.tensor([34, 5, 96, 7], dtype=torch.int32))
    fox.forgetting_attention(q, k, v, lf, head_first=True).backward(do)   # queues the readback
    torch.cuda.synchronize()
    with pytest.raises(fox.FoxError, match="site=34 cta=5 thread=96 detail=7"):
        fox.forgetting_attention(q, k, v, lf, head_first=True)
    fox.forgetting_attention(q, k, v, lf, head_first=True).backward(do)   # the record was cleared
    torch.cuda.synchronize()
    fox.check_status()


def test_runs_under_autocast_and_checkpoint():
    from torch.utils.checkpoint import checkpoint
    q, k, v, lf, do = [t.cuda() for t in _inputs(15, 1, 2, 256, 256, 64, torch.bfloat16)]
    q.requires_grad_(); lf.requires_grad_()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = checkpoint(lambda *a: fox.forgetting_attention(*a, head_first=True), q, k, v, lf, use_reentrant=False)
    out.backward(do)
    _lib.check_status()
    ref = _run(q.detach().cpu(), k.cpu(), v.cpu(), lf.detach().cpu(), do.cpu())   # the plain call
    assert torch.equal(out.detach().cpu(), ref[0])
    _close(q.grad, ref[1], 1e-2, 1e-2, "dq")
    _close(lf.grad, ref[4], 1e-2, 1e-2, "dlog_fgate")


# ------------------------------------------------------------------------- pruning
@pytest.mark.parametrize("M,N", [(512, 512), (1020, 2098), (1000, 1000), (128, 128)])
def test_pruning_indices_bit_exact(M, N):
    rng = np.random.default_rng(M + N)
    B, H = 2, 3
    lf = -np.abs(rng.normal(0.05, 0.08, size=(B, H, N))).astype(np.float32)
    lam = np.cumsum(lf, axis=-1, dtype=np.float32)
    thr = np.array([[-1.0, -5.0, -20.0], [0.0, -3.0, -1000.0]], dtype=np.float32)
    for bm, bn in [(128, 128), (128, 64), (64, 64)]:
        si, ei = ops.find_index(torch.from_numpy(lam).cuda(), torch.from_numpy(thr).cuda(), M, bm, bn, True, True)
        assert np.array_equal(si.cpu().numpy(), orc.find_start_index(lam, thr, M, N, bm, bn))
        assert np.array_equal(ei.cpu().numpy(), orc.find_end_index(lam, thr, M, N, bm, bn))


def test_pruning_indices_bit_exact_against_upstream_scan_kernels():
    """fox_find_index against the index arrays upstream's own _find_start_index_kernel and
    _find_end_index_kernel produced (tests/golden/index_scans.npz), on the same torch.cumsum prefix; and
    how many entries change when the prefix comes from fox_cumsum_fwd instead (summation order differs)."""
    from conftest import load_index_golden
    for name, c in load_index_golden().items():
        B, H, M, N, bm, bn = c["shape"]
        lf = torch.from_numpy(c["log_fgate"])
        thr = torch.from_numpy(c["threshold"]).cuda()
        lam = torch.cumsum(lf, dim=-1).cuda()
        si, ei = ops.find_index(lam, thr, M, bm, bn, True, True)
        assert np.array_equal(si.cpu().numpy(), c["start_index"]), name
        assert np.array_equal(ei.cpu().numpy(), c["end_index"]), name
        lam_own = ops.log_lambda_cumsum(lf.cuda(), None)
        si2, ei2 = ops.find_index(lam_own, thr, M, bm, bn, True, True)
        differing = int((si2 != si).sum()) + int((ei2 != ei).sum())
        print(f"{name}: index entries that differ with the library's own prefix sum: {differing} of "
              f"{si.numel() + ei.numel()}")
        assert differing <= max(1, (si.numel() + ei.numel()) // 100), name


def test_auto_threshold_identical_to_upstream_expression():
    g = torch.Generator().manual_seed(16)
    for dtype in (torch.bfloat16, torch.float16):
        q = (torch.randn(2, 3, 333, 64, generator=g) * torch.rand(1, 3, 1, 1, generator=g) * 2).to(dtype)
        k = torch.randn(2, 3, 333, 64, generator=g).to(dtype)
        got_q = ops.max_row_norm(q.cuda()).cpu()
        assert torch.equal(got_q, torch.linalg.vector_norm(q, dim=-1).max(dim=-1).values)
        got_k = ops.max_row_norm(k.cuda()).cpu()
        thr = (-(2 * (got_q * got_k * 0.125) + math.log(333)) + (-10)).float()
        assert torch.equal(thr, orc.auto_threshold(q, k, 0.125))


def test_host_streamed_steps_equal_direct_calls():
    """The stream-pipelined host-buffer path returns, step by step, what direct calls return."""
    from forgetting_transformer_b200.host_pipeline import HostStreamedAttention
    seq = torch.tensor([0, 50]).cuda()
    pipe = HostStreamedAttention(torch.device("cuda", torch.cuda.current_device()), seq_start=seq)
    steps = []
    for i in range(5):                       # more steps than buffer sets
        q, k, v, lf, do = _inputs(40 + i, 2, 2, 384, 384, 64, torch.bfloat16)
        host = {n: t.pin_memory() for n, t in dict(q=q, k=k, v=v, log_fgate=lf, dout=do).items()}
        hout, ev = pipe.submit(host)
        ev.synchronize()
        steps.append((host, {n: t.clone() for n, t in hout.items()}))
    pipe.finish()
    for host, got in steps:
        qq, kk, vv, ll = [host[n].cuda().requires_grad_() for n in ("q", "k", "v", "log_fgate")]
        out = fox.forgetting_attention(qq, kk, vv, ll, head_first=True, seq_start=seq)
        out.backward(host["dout"].cuda())
        assert torch.equal(got["out"], out.detach().cpu()) and torch.equal(got["dk"], kk.grad.cpu())
        assert torch.equal(got["dv"], vv.grad.cpu())
        # dq and dlog_fgate come out of fp32 atomics whose order varies from run to run
        _close(got["dq"], qq.grad, 1e-2, 1e-2)
        _close(got["dlog_fgate"], ll.grad, 1e-2, 1e-2)


def test_layer_threshold_from_data_matches_auto():
    """acp_threshold_from_data with tolerance -10 is the operator's own "auto" threshold (OPS:95-102)."""
    q, k, v, lf, do = _inputs(5, 2, 3, 300, 300, 64, torch.bfloat16)
    thr = fox.acp_threshold_from_data(q.cuda(), k.cuda(), -10.0)
    ref = orc.auto_threshold(q, k, 1 / math.sqrt(64))
    assert thr.shape == (2, 3) and torch.equal(thr.float().cpu(), ref.float())


def test_pruned_attention_matches_block_oracle():
    """Strong decay + "auto": most KV blocks are pruned; outputs and gradients match the
    oracle that skips exactly the blocks named by the index arrays."""
    B, H, T, D = 2, 2, 1024, 128
    q, k, v, lf, do = _inputs(17, B, H, T, T, D, torch.bfloat16, mu=-1.0, sigma=1.5)
    got = _run(q, k, v, lf, do, thr="auto")
    out, dq, dk, dv, dlf = got
    thr = orc.auto_threshold(q, k, D ** -0.5).numpy()
    lam = got.lam.numpy()                       # the prefix sum the kernels pruned by
    si = orc.find_start_index(lam, thr, T, T, 128, 128)
    ei = orc.find_end_index(lam, thr, T, T, 128, 128)
    assert orc.pruned_tile_fraction(si, T, T, 128, 128) > 0.3
    _check_bf16(got, q, k, v, lf, do, start_index=si, end_index=ei)


# ----------------------------------------------- properties at the benchmark's full sizes
def test_full_size_properties_config3():
    """B=2, T=16384, H=24, D=64 (too big for the dense oracle): with v = 1 every non-empty
    row outputs exactly 1; with dout = 1 the column sums of dv count the non-empty rows;
    the gradient w.r.t. the first log gate vanishes; outputs are linear in v."""
    B, H, T, D = 2, 24, 16384, 64
    g = torch.Generator().manual_seed(1003)
    dev = "cuda"
    q = torch.randn(B, H, T, D, generator=g).bfloat16().to(dev)
    k = torch.randn(B, H, T, D, generator=g).bfloat16().to(dev)
    v1 = torch.randn(B, H, T, D, generator=g).bfloat16().to(dev)
    lf = torch.nn.functional.logsigmoid(torch.randn(B, H, T, generator=g) + 4).to(dev).requires_grad_()
    seq = torch.randint(0, 2048, (B,), generator=g).to(dev)
    ones = torch.ones_like(v1).requires_grad_()
    out = fox.forgetting_attention(q, k, ones, lf, head_first=True, seq_start=seq)
    out.backward(torch.ones_like(out))
    torch.cuda.synchronize()
    _lib.check_status()
    for b in range(B):
        s = int(seq[b])
        assert torch.all(out[b, :, :s] == 0)
        assert torch.all((out[b, :, s:].float() - 1).abs() < 1e-2)
        colsum = ones.grad[b].float().sum(dim=1)  # (H, D): sum_j dv_j = number of non-empty rows
        assert torch.all((colsum - (T - s)).abs() < 1e-3 * T)
    assert lf.grad[..., 0].abs().max().item() < 5e-2
    v2 = torch.randn(B, H, T, D, generator=g).bfloat16().to(dev)
    f = lambda vv: fox.forgetting_attention(q, k, vv, lf.detach(), head_first=True, seq_start=seq).float()
    lin = (f(v1) + f(v2) - f((v1.float() + v2.float()).bfloat16())).abs().max().item()
    assert lin < 8e-2


@pytest.mark.parametrize("D", [64, 128])
def test_cuda_graph_replay_is_bit_identical(D):
    """Forward and backward captured into CUDA graphs (``make_graphed``) and replayed on new input values:
    out, dk and dv bit-identical to the eager call (dq and the gate gradient up to the order of their fp32 atomic
    sums), with seq_start and pruning in the captured step."""
    q, k, v, lf, do = _inputs(300 + D, 2, 3, 384, 512, D, torch.bfloat16, mu=2.0)
    seq = torch.tensor([0, 77]).cuda()
    qs, ks, vs, ls = [t.cuda().requires_grad_() for t in (q, k, v, lf)]
    f = fox.make_graphed(qs, ks, vs, ls, head_first=True, seq_start=seq, adaptive_threshold=-12.0)
    q2, k2, v2, lf2, do2 = _inputs(400 + D, 2, 3, 384, 512, D, torch.bfloat16, mu=1.0)
    for a, b, c, l, g_ in ((q, k, v, lf, do), (q2, k2, v2, lf2, do2)):
        xe = [t.cuda().requires_grad_() for t in (a, b, c, l)]
        xg = [t.cuda().requires_grad_() for t in (a, b, c, l)]
        oe = fox.forgetting_attention(*xe, head_first=True, seq_start=seq, adaptive_threshold=-12.0)
        oe.backward(g_.cuda())
        og = f(*xg)
        og.backward(g_.cuda())
        torch.cuda.synchronize()
        _lib.check_status()
        assert torch.equal(oe, og)
        assert torch.equal(xe[1].grad, xg[1].grad) and torch.equal(xe[2].grad, xg[2].grad)
        # dq and the gate gradient are sums of fp32 atomics, whose order varies from launch to launch
        _close(xg[0].grad, xe[0].grad, 1e-2, 1e-2, "dq")
        _close(xg[3].grad, xe[3].grad, 1e-2, 1e-2, "dlog_fgate")
