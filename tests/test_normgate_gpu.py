"""GPU parity tests of the fused per-head RMSNorm + sigmoid gate against the oracle's
restatement of upstream's reference function (fuse_norm_gate.py:18-53)."""
import pytest
import torch

import forgetting_transformer_b200 as fox
from oracle import fox_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens,G,D", [(1, 24, 64), (1000, 24, 64), (777, 16, 128), (4096, 3, 64)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_norm_gate_fwd_bwd(tokens, G, D, dtype):
    g = torch.Generator().manual_seed(tokens + G)
    hidden = G * D
    x = torch.randn(2, tokens, hidden, generator=g).to(dtype)
    gate = torch.randn(2, tokens, hidden, generator=g).to(dtype)
    w = (torch.rand(hidden, generator=g) + 0.5)
    dy = torch.randn(2, tokens, hidden, generator=g).to(dtype)
    m = fox.FusedGroupNormGated(G, hidden, is_rms_norm=True, eps=1e-6, activation="sigmoid").cuda()
    with torch.no_grad():
        m.weight.copy_(w)
    xc, gc = x.cuda().requires_grad_(), gate.cuda().requires_grad_()
    y = m(xc, gc)
    y.backward(dy.cuda())
    ry, rdx, rdg, rdw = orc.group_rmsnorm_gated_fwd_bwd(x, gate, w, dy, G, 1e-6)
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
    assert (y.cpu().float() - ry.float()).abs().max() < tol
    assert (xc.grad.cpu().float() - rdx.float()).abs().max() < 2 * tol
    assert (gc.grad.cpu().float() - rdg.float()).abs().max() < 2 * tol
    rel = (m.weight.grad.cpu().float() - rdw.float()).abs().max() / rdw.float().abs().max()
    assert rel < 2e-2
    assert y.dtype == dtype and m.weight.grad.dtype == torch.float32
