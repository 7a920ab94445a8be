"""GPU parity tests of the operators around the attention in a FoX-Pro layer: the per-head RMSNorm
applied to q and k (upstream layernorm.py:993-1051 as built at modeling_forgetting_transformer.py:264-265)
and the data-dependent token shift (token_shift.py), against the oracle and against the fixtures
produced by upstream's own code (tests/golden/glue_refs.npz)."""
import pytest
import torch

import forgetting_transformer_b200 as fox
from forgetting_transformer_b200 import _lib
from conftest import load_glue_golden
from oracle import fox_oracle as orc

pytestmark = pytest.mark.gpu


def _oracle_weights(blk) -> dict:
    """The block's weights under the names the CPU oracle's restatement of the block uses."""
    a = blk.attn
    return {"attn_norm": blk.attn_norm.weight, "q": a.q_proj.weight, "k": a.k_proj.linear.weight,
            "k_shift": a.k_proj.shift_proj.weight, "v": a.v_proj.linear.weight,
            "v_shift": a.v_proj.shift_proj.weight, "q_norm": a.q_norm.weight, "k_norm": a.k_norm.weight,
            "fgate_w": a.fgate_proj.weight, "fgate_b": a.fgate_proj.bias, "ogate": a.ogate_proj.weight,
            "out_norm": a.output_norm.weight, "o": a.o_proj.weight, "mlp_norm": blk.mlp_norm.weight,
            "gate": blk.mlp.gate_proj.weight, "down": blk.mlp.down_proj.weight}


def _err(a, b):
    return (a.float().cpu() - b.float().cpu()).abs().max().item()


@pytest.mark.parametrize("tokens,G,D", [(1, 24, 64), (513, 24, 64), (300, 16, 128), (64, 5, 32)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_qk_norm_fwd_bwd(tokens, G, D, dtype):
    g = torch.Generator().manual_seed(tokens + D)
    hidden = G * D
    x = torch.randn(2, tokens, hidden, generator=g).to(dtype)
    w = torch.rand(hidden, generator=g) + 0.5
    dy = torch.randn(2, tokens, hidden, generator=g).to(dtype)
    m = fox.GroupNorm(G, hidden, is_rms_norm=True).cuda()
    with torch.no_grad():
        m.weight.copy_(w)
    xc = x.cuda().requires_grad_()
    y = m(xc)
    y.backward(dy.cuda())
    ry, rdx, rdw = orc.group_rmsnorm_fwd_bwd(x, w, dy, G, 1e-5)
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
    assert y.dtype == dtype and _err(y, ry) < tol
    assert _err(xc.grad, rdx) < 2 * tol
    assert _err(m.weight.grad, rdw) / rdw.abs().max().item() < 2e-2


def test_norms_against_upstream_reference_outputs():
    z = load_glue_golden()
    G = int(z["ng_groups"])
    x, gate, w, dy = [z[k].cuda() for k in ("ng_x", "ng_g", "ng_w", "ng_dy")]
    xc, gc, wc = x.clone().requires_grad_(), gate.clone().requires_grad_(), w.clone().requires_grad_()
    y = fox.group_norm_gated(xc, gc, wc, None, "sigmoid", eps=z["ng_eps"], is_rms_norm=True, num_groups=G)
    y.backward(dy)
    assert _err(y, z["ng_y"]) < 4e-3 and _err(xc.grad, z["ng_dx"]) < 8e-3 and _err(gc.grad, z["ng_dg"]) < 8e-3
    assert _err(wc.grad, z["ng_dw"]) / z["ng_dw"].abs().max().item() < 1e-2
    xc, wc = x.clone().requires_grad_(), w.clone().requires_grad_()
    y = fox.group_norm(xc, wc, None, eps=z["qk_eps"], is_rms_norm=True, num_groups=G)
    y.backward(dy)
    assert _err(y, z["qk_y"]) < 4e-3 and _err(xc.grad, z["qk_dx"]) < 8e-3
    assert _err(wc.grad, z["qk_dw"]) / z["qk_dw"].abs().max().item() < 1e-2


@pytest.mark.parametrize("rows,hidden", [(1, 256), (37, 768), (1000, 1536), (64, 2048)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("with_residual", [False, True])
def test_row_rms_norm_fwd_bwd(rows, hidden, dtype, with_residual):
    g = torch.Generator().manual_seed(rows + hidden)
    x = torch.randn(2, rows, hidden, generator=g).to(dtype)
    res = torch.randn(2, rows, hidden, generator=g).to(dtype) if with_residual else None
    w = torch.rand(hidden, generator=g) + 0.5
    dy = torch.randn(2, rows, hidden, generator=g).to(dtype)
    dres = torch.randn(2, rows, hidden, generator=g).to(dtype) if with_residual else None
    m = fox.RMSNorm(hidden).cuda()
    with torch.no_grad():
        m.weight.copy_(w)
    xc = x.cuda().requires_grad_()
    if with_residual:                      # the block's mlp_norm(hidden_states, residual, True)
        rc = res.cuda().requires_grad_()
        y, z = m(xc, rc, True)
        torch.autograd.backward([y, z], [dy.cuda(), dres.cuda()])
    else:                                  # the block's attn_norm(hidden_states)
        y = m(xc)
        y.backward(dy.cuda())
    ry, rz, rdx, rdw = orc.rms_norm_fwd_bwd(x, w, res, dy, dres, 1e-5)
    # one ulp of the 16-bit type at the tensor's largest magnitude (x + residual reaches 6-8)
    tol = (2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10)
    assert y.dtype == dtype and _err(y, ry) <= tol * max(1.0, ry.abs().max().item())
    assert _err(xc.grad, rdx) <= 2 * tol * max(1.0, rdx.abs().max().item())
    if with_residual:
        assert torch.equal(z.cpu(), rz) and torch.equal(rc.grad, xc.grad)
    assert _err(m.weight.grad, rdw) / rdw.abs().max().item() < 2e-2


def test_row_rms_norm_against_upstream_reference_outputs():
    z = load_glue_golden()
    x, res, w = z["rn_x"].cuda().requires_grad_(), z["rn_res"].cuda().requires_grad_(), z["rn_w"].cuda().requires_grad_()
    y, zs = fox.rms_norm(x, w, None, residual=res, eps=z["rn_eps"], prenorm=True)
    torch.autograd.backward([y, zs], [z["rn_dy"].cuda(), z["rn_dres"].cuda()])
    assert _err(y, z["rn_y"]) < 2e-3 and torch.equal(zs.cpu(), z["rn_z"].to(zs.dtype))
    assert _err(x.grad, z["rn_dx"]) < 8e-3 and _err(res.grad, z["rn_dr"]) < 8e-3
    assert _err(w.grad, z["rn_dw"]) / z["rn_dw"].abs().max().item() < 1e-2
    with pytest.raises(_lib.FoxError):
        fox.rms_norm(torch.randn(4, 384).half().cuda(), torch.ones(384).cuda())   # 384 is not a built row length


def test_token_shift_bit_exact_against_upstream_kernel_outputs():
    z = load_glue_golden()
    x = z["ts_x"].cuda().requires_grad_()
    pw = z["ts_prev"].cuda().requires_grad_()
    cw = z["ts_curr"].cuda().requires_grad_()
    out = fox.token_shift(x, pw, cw)
    out.backward(z["ts_dout"].cuda())
    torch.cuda.synchronize()
    # one fp32 multiply-add pair and one rounding per element on both sides
    assert torch.equal(out.cpu(), z["ts_out"]) and torch.equal(x.grad.cpu(), z["ts_dx"])
    assert _err(pw.grad, z["ts_dprev"]) < 1e-4 and _err(cw.grad, z["ts_dcurr"]) < 1e-4


@pytest.mark.parametrize("B,T,H,D", [(2, 1, 3, 64), (1, 257, 12, 64), (3, 100, 5, 16), (2, 129, 4, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_token_shift_shapes_and_strided_views(B, T, H, D, dtype):
    g = torch.Generator().manual_seed(T + D)
    # the layer passes a (B, T, H*D) projection viewed as (B, T, H, D); also try a head-first parent
    parent = torch.randn(B, H, T, D, generator=g).to(dtype)
    x = parent.permute(0, 2, 1, 3)
    alpha = torch.rand(B, T, H, generator=g)
    dout = torch.randn(B, T, H, D, generator=g).to(dtype)
    xc = x.cuda().requires_grad_()
    pw = alpha.cuda().requires_grad_()
    cw = (1.0 - alpha).cuda().requires_grad_()
    out = fox.token_shift(xc, pw, cw)
    out.backward(dout.cuda())
    ro, rdx, rdp, rdc = orc.token_shift_fwd_bwd(x, alpha, 1.0 - alpha, dout)
    assert out.shape == x.shape and torch.equal(out.cpu(), ro)
    assert torch.equal(xc.grad.cpu(), rdx)
    scale = max(rdp.abs().max().item(), 1.0)
    assert _err(pw.grad, rdp) < 1e-4 * scale and _err(cw.grad, rdc) < 1e-4 * scale


def test_token_shift_contract():
    x = torch.randn(1, 4, 2, 24).half()
    w = torch.rand(1, 4, 2)
    with pytest.raises(AssertionError):
        fox.token_shift(x.cuda(), w.cuda(), w.cuda())          # D not in {16, 32, 64, 128}
    with pytest.raises(_lib.FoxError):
        fox.token_shift(torch.randn(1, 4, 2, 16).half(), w, w)  # no CPU path


@pytest.mark.parametrize("with_mask", [False, True])
def test_fox_pro_block_against_oracle(with_mask):
    """The block composed from the package's operators against the oracle's fp32 restatement of its data
    flow, same weights: output and input gradient."""
    torch.manual_seed(3)
    B, T, C, H, I = 2, 300, 256, 4, 512
    blk = fox.FoxProBlock(C, H, I, fgate_bias=2.0).cuda().to(torch.bfloat16)
    with torch.no_grad():                       # non-trivial norm weights
        for m in (blk.attn_norm, blk.mlp_norm, blk.attn.q_norm, blk.attn.k_norm, blk.attn.output_norm):
            m.weight.uniform_(0.5, 1.5)
        for lin in (blk.attn.q_proj, blk.attn.k_proj.linear, blk.attn.v_proj.linear, blk.attn.o_proj,
                    blk.attn.ogate_proj, blk.mlp.gate_proj, blk.mlp.down_proj):
            lin.weight.normal_(0, 0.08)
    x = torch.randn(B, T, C, device="cuda").to(torch.bfloat16).requires_grad_()
    mask = None
    if with_mask:
        mask = torch.ones(B, T, dtype=torch.long, device="cuda")
        mask[1, :17] = 0                        # left padding
    y = blk(x, mask)
    dy = torch.randn_like(y)
    y.backward(dy)
    torch.cuda.synchronize()
    _lib.check_status()
    xr = x.detach().float().cpu().requires_grad_()
    w = {n: t.detach().float().cpu() for n, t in _oracle_weights(blk).items()}
    yr = orc.fox_pro_block(xr, w, H, eps=1e-6, attention_mask=None if mask is None else mask.cpu())
    yr.backward(dy.float().cpu())
    valid = slice(None) if mask is None else mask.bool().cpu()
    scale = yr.detach().abs().max().item()
    assert (y.detach().float().cpu() - yr.detach())[valid].abs().max().item() < 3e-2 * scale
    gscale = xr.grad.abs().max().item()
    assert (x.grad.float().cpu() - xr.grad)[valid].abs().max().item() < 5e-2 * gscale


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_swiglu_and_swiglu_linear(dtype):
    """SwiGLU kernels against upstream's expressions (glu_linear.py:64-86), in place on the halves of a
    packed projection, and the linear-fused forms against autograd through the eager composition."""
    g = torch.Generator().manual_seed(9)
    rows, inter, out_dim = 333, 256, 96
    xy = (torch.randn(3, rows, 2 * inter, generator=g) * 2).to(dtype).cuda()
    x, y = xy.chunk(2, -1)
    gout = torch.randn(3, rows, inter, generator=g).to(dtype).cuda()
    xr, yr = x.detach().clone().requires_grad_(), y.detach().clone().requires_grad_()
    z = fox.swiglu(xr, yr)
    z.backward(gout)
    rdx, rdy, rz = orc.swiglu_bwd(x.cpu(), y.cpu(), gout.cpu())
    ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    for a, b in ((z, rz), (xr.grad, rdx), (yr.grad, rdy)):          # __expf vs exp: at most one ulp apart
        assert _err(a, b) <= ulp * max(1.0, b.abs().max().item())
    w = (torch.randn(out_dim, inter, generator=g) * 0.1).to(dtype).cuda().requires_grad_()
    xy1 = xy.detach().clone().requires_grad_()
    out = fox.swiglu_linear_packed(xy1, w, None)
    dout = torch.randn_like(out)
    out.backward(dout)
    xy2, w2 = xy.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    a_, b_ = xy2.chunk(2, -1)
    ref = torch.nn.functional.linear(torch.nn.functional.silu(a_) * b_, w2)
    ref.backward(dout.float())
    assert _err(out, ref) < 3e-2 * ref.abs().max().item()
    assert _err(xy1.grad, xy2.grad) < 3e-2 * xy2.grad.abs().max().item()
    assert _err(w.grad, w2.grad) < 3e-2 * w2.grad.abs().max().item()
    x3, y3, w3 = x.detach().clone().requires_grad_(), y.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    out3 = fox.swiglu_linear(x3, y3, w3, None)
    out3.backward(dout)
    assert torch.equal(out3, out) and torch.equal(torch.cat([x3.grad, y3.grad], -1), xy1.grad)


@pytest.mark.parametrize("with_mask", [False, True])
def test_generation_with_cache_matches_full_forward(with_mask):
    """Prefill of T0 tokens followed by single-token steps through ``FgateCache`` (in-place growth, the
    ShiftLinear single-token branch of modeling_forgetting_transformer.py:83-86, the split-KV generation
    kernels) against the oracle's restatement of the block on the whole sequence, and against the block's own
    full-sequence forward."""
    torch.manual_seed(5)
    B, T0, steps, C, H, I = 2, 150, 6, 256, 4, 512
    T = T0 + steps
    blk = fox.FoxProBlock(C, H, I, fgate_bias=2.0).cuda().to(torch.bfloat16)
    with torch.no_grad():
        for m in (blk.attn_norm, blk.mlp_norm, blk.attn.q_norm, blk.attn.k_norm, blk.attn.output_norm):
            m.weight.uniform_(0.5, 1.5)
        for lin in (blk.attn.q_proj, blk.attn.k_proj.linear, blk.attn.v_proj.linear, blk.attn.o_proj,
                    blk.attn.ogate_proj, blk.mlp.gate_proj, blk.mlp.down_proj):
            lin.weight.normal_(0, 0.08)
    x = torch.randn(B, T, C, device="cuda").to(torch.bfloat16)
    mask = None
    if with_mask:
        mask = torch.ones(B, T, dtype=torch.long, device="cuda")
        mask[1, :9] = 0                         # left padding
    cache = fox.FgateCache(granule=128)
    st = blk.attn.init_shift_state(B)
    cache.update_shift_cache(st["key_shift"], st["value_shift"], 0)
    with torch.no_grad():
        full = blk(x, mask)
        outs = [blk(x[:, :T0], None if mask is None else mask[:, :T0], cache, 0)]
        ptr = cache[0][0].data_ptr()
        for t in range(T0, T):
            outs.append(blk(x[:, t:t + 1], None if mask is None else mask[:, :t + 1], cache, 0))
        gen = torch.cat(outs, dim=1)
    torch.cuda.synchronize()
    _lib.check_status()
    assert cache.get_seq_length() == T and cache.capacity(0) == 256
    assert cache[0][0].data_ptr() == ptr        # the steps wrote in place
    w = {n: t.detach().float().cpu() for n, t in _oracle_weights(blk).items()}
    yr = orc.fox_pro_block(x.float().cpu(), w, H, eps=1e-6, attention_mask=None if mask is None else mask.cpu())
    valid = slice(None) if mask is None else mask.bool().cpu()
    scale = yr.abs().max().item()
    assert (gen.float().cpu() - yr)[valid].abs().max().item() < 3e-2 * scale
    assert (gen.float().cpu() - full.float().cpu())[valid].abs().max().item() < 3e-2 * scale


@pytest.mark.parametrize("inplace", [False, True])
def test_cross_entropy_against_upstream_kernels_and_oracle(inplace):
    """fox_cross_entropy_fwd / _bwd through the module mirror: every fixture case of upstream's own kernels
    (fp32 and fp16 logits, 1003 classes: rows that do not start on 16 bytes are re-laid), then bf16 logits at a
    vocabulary-sized class count against the oracle, in place and out of place."""
    from conftest import load_ce_golden
    for name, c in load_ce_golden().items():
        ls, scale, zs = [float(x) for x in c["args"]]
        x = c["logits"].cuda().requires_grad_()
        losses, zl = fox.cross_entropy_loss(x, c["labels"].cuda(), ls, scale, zs, -100, False)
        (losses * c["dloss"].cuda()).sum().backward()
        # (with 16-bit logits upstream forms logit_scale * logits[label] and its (1 - smoothing) multiple in the
        # logits' dtype, fused_cross_entropy.py:65-72: its loss carries that one rounding)
        loss_tol = 2e-5 * max(1.0, c["losses"].abs().max().item()) if x.dtype == torch.float32 else 8e-3
        assert _err(losses, c["losses"].cuda()) < loss_tol, name
        assert _err(zl, c["z_losses"].cuda()) < 1e-6, name
        tol = 1e-6 if x.dtype == torch.float32 else 2e-3 * c["dlogits"].float().abs().max().item()
        assert _err(x.grad, c["dlogits"].cuda()) < tol, name
    g = torch.Generator().manual_seed(9)
    rows, cols = 300, 50304
    logits = (torch.randn(rows, cols, generator=g) * 2).bfloat16()
    labels = torch.randint(0, cols, (rows,), generator=g)
    labels[::7] = -100
    dloss = torch.rand(rows, generator=g)
    rl, rz, rd = orc.cross_entropy_fwd_bwd(logits, labels, dloss, lse_square_scale=1e-4)
    mod = fox.FusedCrossEntropyLoss(reduction="none", lse_square_scale=1e-4, inplace_backward=inplace, return_z_loss=True)
    x = logits.cuda().requires_grad_()
    xin = x.clone() if inplace else x          # (an in-place backward overwrites the tensor the function saved)
    losses, zl = mod(xin, labels.cuda())
    (losses * dloss.cuda()).sum().backward()
    assert _err(losses.cpu(), rl) < 1e-4 and _err(zl.cpu(), rz) < 1e-6
    assert _err(x.grad.cpu(), rd) < 4e-3 * rd.abs().max().item()     # one bf16 rounding of the gradient
    mean = fox.FusedCrossEntropyLoss()(logits.cuda(), labels.cuda())
    assert abs(mean.item() - (orc.cross_entropy(logits, labels)[0].sum() / (labels != -100).sum()).item()) < 1e-4
