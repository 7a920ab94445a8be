"""The FoX-Pro block against the upstream project's own ``ForgettingTransformerBlock`` on the same GPU (B200).

Needs a copy of the upstream package (``conftest.upstream_ops``); skipped without one.  Three blocks share
one set of weights:

  * upstream's block as shipped: its Triton norms, token shift and attention (block-size hooks overridden, they
    raise on sm_100), its jiterator SwiGLU (modeling_forgetting_transformer.py:516-628);
  * ``FoxProBlock`` of this package;
  * upstream's block after the name patch a maintainer would apply (the snippet in INTEGRATION.md), i.e.
    upstream's module code calling this package's operators.

A block is a dozen 16-bit operators on each side and its output a residual sum of their results (an output of
0.2 can be the sum of a residual of -5.8 and an MLP output of 6.0 that was rounded to 16 bits at that magnitude),
so outputs are compared with the bf16 bar taken at the magnitude of the largest activation,
|a - b| <= 2e-2 + 1e-2 max|ref|, and together with the input and weight gradients by their relative error in the
Frobenius norm.
"""
import pytest
import torch

import forgetting_transformer_b200 as fox
from forgetting_transformer_b200 import _lib
from conftest import upstream_ops
from test_attention_gpu import ATOL_BF16, RTOL_BF16, _bars, _close

pytestmark = pytest.mark.gpu

HIDDEN, HEADS, INTER = 512, 8, 1024


@pytest.fixture(scope="module")
def upstream():
    ops_mod = upstream_ops()
    if ops_mod is None:
        pytest.skip("no copy of the upstream package (FOX_REFERENCE_SRC or baseline/_ref)")
    import forgetting_transformer.model.forgetting_transformer.modeling_forgetting_transformer as up_model
    from forgetting_transformer.model.forgetting_transformer.configuration_forgetting_transformer import (
        ForgettingTransformerConfig)
    cfg = ForgettingTransformerConfig(hidden_size=HIDDEN, num_heads=HEADS, use_output_gate=True, use_output_norm=True,
                                      qk_norm=True, use_k_shift=True, use_v_shift=True, intermediate_size=INTER,
                                      use_rope=False)
    return ops_mod, up_model, cfg


def _run(block, x, dy, mask, is_upstream):
    for p in block.parameters():
        p.grad = None
    xx = x.clone().requires_grad_()
    # upstream's layer computes in the autocast dtype and in fp32 without autocast (lines 289-295): bf16 autocast
    # over fp32 parameters, as its training configuration runs it (configs/config.py:22)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = block(xx, attention_mask=mask)
    out = out[0] if is_upstream else out
    out.backward(dy)
    torch.cuda.synchronize()
    _lib.check_status()
    return out.detach(), xx.grad, {n: p.grad.clone() for n, p in block.named_parameters()}


def _compare(label, ref, got, valid):
    (ro, rdx, rg), (go, gdx, gg) = ref, got
    v = valid[:, :, None]
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-6)).item()
    rels = {n: rel(gg[n], rg[n]) for n in rg}
    print(label, "out", round(_bars(go * v, ro * v), 3), "bars; relative errors: dx", round(rel(gdx * v, rdx * v), 4),
          "weights, worst", max(rels, key=rels.get), round(max(rels.values()), 4))
    assert ((go - ro) * v).abs().max().item() <= ATOL_BF16 + RTOL_BF16 * (ro * v).abs().max().item(), label + " out"
    assert rel(go * v, ro * v) < 1e-2, f"{label} out: relative error {rel(go * v, ro * v):.3e}"
    assert rel(gdx * v, rdx * v) < 2e-2, f"{label} dx: relative error {rel(gdx * v, rdx * v):.3e}"
    for n, r_ in rels.items():
        assert r_ < 3e-2, f"{label} grad of {n}: relative error {r_:.3e}"


@pytest.mark.parametrize("padded", [False, True])
def test_block_against_upstream_block_and_through_the_integration_patch(upstream, padded):
    ops_mod, up_model, cfg = upstream
    torch.manual_seed(5)
    dev = "cuda"
    B, T = 2, 384
    stock = up_model.ForgettingTransformerBlock(cfg, 0).to(dev)
    with torch.no_grad():
        for n, p in stock.named_parameters():
            if p.dim() == 2:
                p.normal_(0.0, 0.05)
            elif n.endswith("norm.weight"):
                p.uniform_(0.5, 1.5)
        stock.attn.fgate_proj.bias.fill_(3.0)
    ours = fox.FoxProBlock(HIDDEN, HEADS, INTER).to(dev)
    assert set(ours.state_dict()) == set(stock.state_dict())
    ours.load_state_dict(stock.state_dict())
    x = torch.randn(B, T, HIDDEN, device=dev).bfloat16()
    dy = torch.randn(B, T, HIDDEN, device=dev).bfloat16()
    mask = None
    valid = torch.ones(B, T, device=dev)
    if padded:
        mask = torch.ones(B, T, dtype=torch.long, device=dev)
        mask[1, :57] = 0            # left padding
        valid = mask.float()
        dy = dy * valid[:, :, None].bfloat16()
    ref = _run(stock, x, dy, mask, True)
    got = _run(ours, x, dy, mask, False)
    _compare("FoxProBlock vs upstream block", ref, got, valid)

    # the patch of INTEGRATION.md section 1, applied to upstream's modules and undone afterwards
    names = dict(forgetting_attention=fox.forgetting_attention, FusedGroupNormGated=fox.FusedGroupNormGated,
                 GroupNorm=fox.GroupNorm, token_shift=fox.token_shift, RMSNorm=fox.RMSNorm,
                 swiglu_linear=fox.swiglu_linear)
    saved = {n: getattr(up_model, n) for n in names}
    saved_op = ops_mod.forgetting_attention
    try:
        ops_mod.forgetting_attention = fox.forgetting_attention
        for n, obj in names.items():
            setattr(up_model, n, obj)
        patched = up_model.ForgettingTransformerBlock(cfg, 0).to(dev)
        patched.load_state_dict(stock.state_dict())
        via_patch = _run(patched, x, dy, mask, True)
    finally:
        ops_mod.forgetting_attention = saved_op
        for n, obj in saved.items():
            setattr(up_model, n, obj)
    _compare("patched upstream block vs upstream block", ref, via_patch, valid)
    _compare("patched upstream block vs FoxProBlock", got, via_patch, valid)
