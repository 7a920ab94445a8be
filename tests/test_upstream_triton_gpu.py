"""Head to head with the upstream project's own Triton kernels on the same GPU, natively in bf16 (B200).

Needs a copy of the upstream package (see ``conftest.upstream_ops``); skipped without one.  Upstream's block-size
hooks raise on sm_100 and are documented as overridable (forgetting_attention.py:459, 799): they are pinned to
128 x 128 tiles, the grid of the sm_100a kernels, so that ``start_index`` (upstream's hidden return, lines
223-229) can be compared entry by entry.

Both sides round probabilities and dS to bf16 before their products, so outputs and gradients are compared
element by element with the bf16 bar |a - b| <= 2e-2 + 1e-2 |upstream|.
"""
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


def _both(up, q, k, v, lf, do, seq, sm_scale, thr):
    res = []
    for fn in (up.ForgettingAttention, ops.ForgettingAttention):
        qq, kk, vv, ll = [t.detach().clone().requires_grad_() for t in (q, k, v, lf)]
        out, L, si = fn.apply(qq, kk, vv, ll, seq, True, sm_scale, thr, True, thr is not None, None, False, False)
        out.backward(do)
        torch.cuda.synchronize()
        res.append(dict(out=out.detach(), L=L, start_index=si, dq=qq.grad, dk=kk.grad, dv=vv.grad, dlog_fgate=ll.grad))
    _lib.check_status()
    return res


def _compare(label, theirs, ours):
    print(label, {n: round(_bars(ours[n], theirs[n]), 3) for n in ("out", "dq", "dk", "dv", "dlog_fgate")},
          "(worst element, in units of its bar)")
    fin = torch.isfinite(theirs["L"])
    assert torch.equal(torch.isfinite(ours["L"]), fin)
    _close(ours["L"][fin], theirs["L"][fin], 1e-4, 1e-4, "L")
    for n in ("out", "dq", "dk", "dv", "dlog_fgate"):
        _close(ours[n], theirs[n], ATOL_BF16, RTOL_BF16, f"{label} {n}")


def _inputs(seed, B, H, M, N, D, mu, sigma, std=1.0, uniform=None):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, H, M, D, generator=g) * std).bfloat16().cuda()
    k = (torch.randn(B, H, N, D, generator=g) * std).bfloat16().cuda()
    v = (torch.randn(B, H, N, D, generator=g) * std).bfloat16().cuda()
    logit = (torch.empty(B, H, N).uniform_(*uniform, generator=g) if uniform
             else torch.randn(B, H, N, generator=g) * sigma + mu)
    lf = torch.nn.functional.logsigmoid(logit).cuda()
    do = torch.randn(B, H, M, D, generator=g).bfloat16().cuda()
    return q, k, v, lf, do


def test_kernel_level_config_b4_t512_h12_d64(up):
    q, k, v, lf, do = _inputs(1002, 4, 12, 512, 512, 64, 0.0, 1.0)
    theirs, ours = _both(up, q, k, v, lf, do, None, None, None)
    _compare("B4 T512 H12 D64", theirs, ours)


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
    theirs, ours = _both(up, q, k, v, lf, do, seq_t, 0.5, thr_t)
    _compare(f"{shape} seq_start={seq} thr={thr}", theirs, ours)
    if thr is not None:
        assert torch.equal(ours["start_index"], theirs["start_index"])


def test_long_context_slice_t16384_d64(up):
    """B=1, H=2 slice of the long-context configuration (gate logits N(4,1), seq_start in [0, 2048))."""
    q, k, v, lf, do = _inputs(1003, 1, 2, 16384, 16384, 64, 4.0, 1.0)
    theirs, ours = _both(up, q, k, v, lf, do, torch.tensor([1531]).cuda(), None, None)
    _compare("T16384 D64", theirs, ours)


def test_pruning_stress_slice_t16384_d128_auto_threshold(up):
    """B=1, H=2 slice of the pruning stress configuration with adaptive_threshold="auto": the same KV blocks
    are pruned on both sides (start_index identical entry by entry, each side using its own prefix sum and its
    own evaluation of the threshold), and with them the pruned-tile fraction."""
    g = torch.Generator().manual_seed(7)
    q, k, v, lf, do = _inputs(1004, 1, 2, 16384, 16384, 128, -1.0, 1.5)
    s = torch.tensor([0.8, 1.7]).view(1, 2, 1, 1).cuda()
    q, k, v = [(t.float() * s).bfloat16() for t in (q, k, v)]
    theirs, ours = _both(up, q, k, v, lf, do, None, None, "auto")
    differing = int((ours["start_index"] != theirs["start_index"]).sum())
    nmb = ours["start_index"].shape[-1]
    hi = torch.clamp((torch.arange(nmb, device="cuda") + 1) * 128, max=16384)
    frac = [float((torch.minimum(r["start_index"], hi) // 128).sum() / (torch.ceil(hi / 128).sum() * 2))
            for r in (theirs, ours)]
    print(f"pruned tile fraction upstream {frac[0]:.5f} ours {frac[1]:.5f}; differing start_index entries {differing}")
    assert differing == 0 and frac[0] == frac[1] and frac[0] > 0.9
    _compare("T16384 D128 auto", theirs, ours)
