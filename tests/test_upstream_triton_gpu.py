"""Head to head with the upstream project's own Triton kernels on the same GPU, natively in bf16 (B200).

Needs a copy of the upstream package (see ``conftest.upstream_ops``); skipped without one.  Upstream's block-size
hooks raise on sm_100 and are documented as overridable (forgetting_attention.py:459, 799): they are pinned to
128 x 128 tiles, the grid of the sm_100a kernels, so that ``start_index`` (upstream's hidden return, lines
223-229) can be compared entry by entry.

What is compared, every element with the bf16 bar |a - b| <= 2e-2 + 1e-2 |upstream|:
  * forward: out, and the log-normaliser to 1e-4.  The log gates are drawn on a binary grid fine enough for the
    distribution and coarse enough that every partial sum is exact in fp32, so both sides' prefix sums (upstream:
    torch.cumsum; here: fox_cumsum_fwd) are the same numbers whatever order they add in;
  * backward: this library's backward kernels run on the tensors UPSTREAM's forward saved (its out, its
    log-normaliser, its prefix sum; forgetting_attention.py:207) against upstream's backward on the same
    tensors: dq, dk, dv, dlog_fgate.  (The two forwards round ``out`` differently; delta = rowsum(out * dout)
    carries that into every dS, so gradients of two complete pipelines differ by the forwards' rounding, not by
    anything the backward kernels do.  That end-to-end difference is printed.)
"""
import types

import numpy as np
import pytest
import torch

from forgetting_transformer_b200 import _lib, ops
from conftest import upstream_ops
from test_attention_gpu import ATOL_BF16, RTOL_BF16, _bars, _close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def up():
    mod = upstream_ops()
    if mod is None:
        pytest.skip("no copy of the upstream package (FOX_REFERENCE_SRC or baseline/_ref)")
    return mod


def _upstream_prefix(lf, seq):
    """The prefix sum upstream's forward forms and saves (forgetting_attention.py:111-127)."""
    lf = lf.float()
    if seq is not None:
        mask = torch.arange(lf.shape[-1], device=lf.device)[None, None, :] < seq[:, None, None]
        lf = torch.where(mask, torch.zeros_like(lf), lf)
    return torch.cumsum(lf, dim=-1, dtype=lf.dtype).float()


def _both(up, q, k, v, lf, do, seq, sm_scale, thr):
    """(upstream's results, this library's results, this library's backward on upstream's saved tensors)."""
    res = []
    for fn in (up.ForgettingAttention, ops.ForgettingAttention):
        qq, kk, vv, ll = [t.detach().clone().requires_grad_() for t in (q, k, v, lf)]
        out, L, si = fn.apply(qq, kk, vv, ll, seq, True, sm_scale, thr, True, thr is not None, None, False, False)
        out.backward(do)
        torch.cuda.synchronize()
        res.append(dict(out=out.detach(), L=L, start_index=si, dq=qq.grad, dk=kk.grad, dv=vv.grad, dlog_fgate=ll.grad))
    theirs, ours = res
    B, H, M, D = q.shape
    thr_t = None
    if thr is not None:
        thr_t = ours_threshold(q, k, thr, sm_scale if sm_scale is not None else D ** -0.5)
    ctx = types.SimpleNamespace(
        saved_tensors=(q, k, v, theirs["out"], theirs["L"], _upstream_prefix(lf, seq), seq, thr_t),
        sm_scale=sm_scale if sm_scale is not None else D ** -0.5, has_seq_start=seq is not None, start_index=None,
        head_dim=D)
    grads = ops.ForgettingAttention.backward(ctx, do)
    torch.cuda.synchronize()
    _lib.check_status()
    on_theirs = dict(zip(("dq", "dk", "dv", "dlog_fgate"), grads[:4]))
    return theirs, ours, on_theirs


def ours_threshold(q, k, thr, sm_scale):
    """The (B, H) fp32 threshold tensor the operator saves for its backward."""
    B, H = q.shape[:2]
    if isinstance(thr, str):
        bound = ops.max_row_norm(q) * ops.max_row_norm(k) * sm_scale
        thr = -(2 * bound + float(np.log(k.shape[2]))) + (-10)
    t = thr.float().cuda() if isinstance(thr, torch.Tensor) else torch.full((), float(thr), device="cuda")
    return torch.broadcast_to(t, (B, H))


def _compare(label, theirs, ours, on_theirs):
    print(label, "complete pipelines, worst element in units of its bar:",
          {n: round(_bars(ours[n], theirs[n]), 3) for n in ("out", "dq", "dk", "dv", "dlog_fgate")},
          "| backward kernels on upstream's saved tensors:",
          {n: round(_bars(on_theirs[n], theirs[n]), 3) for n in ("dq", "dk", "dv", "dlog_fgate")})
    fin = torch.isfinite(theirs["L"])
    assert torch.equal(torch.isfinite(ours["L"]), fin)
    _close(ours["L"][fin], theirs["L"][fin], 1e-4, 1e-4, "L")
    _close(ours["out"], theirs["out"], ATOL_BF16, RTOL_BF16, f"{label} out")
    for n in ("dq", "dk", "dv", "dlog_fgate"):
        _close_two_roundings(on_theirs[n], theirs[n], f"{label} {n}")
    # end to end the value gradient does not depend on delta: it must agree as it is
    _close(ours["dv"], theirs["dv"], ATOL_BF16, RTOL_BF16, f"{label} dv (complete pipelines)")


def _close_two_roundings(a, b, what):
    """Two kernels that each round dS to 16 bits where the other does: their difference carries both roundings.
    Every element within 1.5 bars (2e-2 + 1e-2 |upstream|), and no more than ten per million over one bar."""
    a, b = a.float(), b.float()
    bars = (a - b).abs() / (ATOL_BF16 + RTOL_BF16 * b.abs())
    over = int((bars > 1.0).sum())
    assert bars.max().item() <= 1.5 and over <= max(1, a.numel() // 100000), (
        f"{what}: worst element {bars.max().item():.3f} bars, {over} of {a.numel()} over one bar")


def _inputs(seed, B, H, M, N, D, mu, sigma, std=1.0, uniform=None, grid=2.0 ** -12):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, H, M, D, generator=g) * std).bfloat16().cuda()
    k = (torch.randn(B, H, N, D, generator=g) * std).bfloat16().cuda()
    v = (torch.randn(B, H, N, D, generator=g) * std).bfloat16().cuda()
    logit = (torch.empty(B, H, N).uniform_(*uniform, generator=g) if uniform
             else torch.randn(B, H, N, generator=g) * sigma + mu)
    lf = torch.nn.functional.logsigmoid(logit)
    lf = torch.round(lf / grid) * grid          # every partial sum of N such terms is exact in fp32
    assert float(lf.abs().sum(-1).max()) / grid < 2 ** 24
    do = torch.randn(B, H, M, D, generator=g).bfloat16().cuda()
    return q, k, v, lf.cuda(), do


def test_kernel_level_config_b4_t512_h12_d64(up):
    q, k, v, lf, do = _inputs(1002, 4, 12, 512, 512, 64, 0.0, 1.0)
    _compare("B4 T512 H12 D64", *_both(up, q, k, v, lf, do, None, None, None))


@pytest.mark.parametrize("shape,seq,thr", [
    ((4, 2, 1020, 2098, 64), True, -10.0),
    ((4, 2, 1020, 2098, 64), False, None),
    ((4, 2, 1024, 2048, 128), True, "per_head"),
    ((4, 2, 1024, 2048, 128), False, -10.0),
])
def test_upstreams_own_test_grid_in_bf16(up, shape, seq, thr):
    """Shapes, input scales (std 0.5, sm_scale 0.5, gate logits U(0, 5)) and threshold kinds of upstream's
    in-file test (forgetting_attention.py:1360-1379), in bf16 instead of fp16."""
    B, H, M, N, D = shape
    q, k, v, lf, do = _inputs(24, B, H, M, N, D, 0, 0, std=0.5, uniform=(0, 5))
    seq_t = torch.tensor([7, 300, 1500, N - 1]).cuda() if seq else None
    thr_t = torch.tensor([-1000.0, -100.0]).cuda() if thr == "per_head" else thr
    theirs, ours, on_theirs = _both(up, q, k, v, lf, do, seq_t, 0.5, thr_t)
    _compare(f"{shape} seq_start={seq} thr={thr}", theirs, ours, on_theirs)
    if thr is not None:
        assert torch.equal(ours["start_index"], theirs["start_index"])


def test_long_context_slice_t16384_d64(up):
    """B=1, H=2 slice of the long-context configuration (gate logits N(4,1), seq_start in [0, 2048))."""
    q, k, v, lf, do = _inputs(1003, 1, 2, 16384, 16384, 64, 4.0, 1.0)
    _compare("T16384 D64", *_both(up, q, k, v, lf, do, torch.tensor([1531]).cuda(), None, None))


def test_pruning_stress_slice_t16384_d128_auto_threshold(up):
    """B=1, H=2 slice of the pruning stress configuration with adaptive_threshold="auto": the same KV blocks
    are pruned on both sides (start_index identical entry by entry, each side using its own prefix sum and its
    own evaluation of the threshold), and with them the pruned-tile fraction."""
    q, k, v, lf, do = _inputs(1004, 1, 2, 16384, 16384, 128, -1.0, 1.5, grid=2.0 ** -9)
    s = torch.tensor([0.8, 1.7]).view(1, 2, 1, 1).cuda()
    q, k, v = [(t.float() * s).bfloat16() for t in (q, k, v)]
    theirs, ours, on_theirs = _both(up, q, k, v, lf, do, None, None, "auto")
    differing = int((ours["start_index"] != theirs["start_index"]).sum())
    nmb = ours["start_index"].shape[-1]
    hi = torch.clamp((torch.arange(nmb, device="cuda") + 1) * 128, max=16384)
    frac = [float((torch.minimum(r["start_index"], hi) // 128).sum() / (torch.ceil(hi / 128).sum() * 2))
            for r in (theirs, ours)]
    print(f"pruned tile fraction upstream {frac[0]:.5f} ours {frac[1]:.5f}; differing start_index entries {differing}")
    assert differing == 0 and frac[0] == frac[1] and frac[0] > 0.9
    _compare("T16384 D128 auto", theirs, ours, on_theirs)
