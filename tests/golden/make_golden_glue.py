"""Generates the golden fixtures of the glue operators around the attention (per-head RMSNorm with and
without the sigmoid gate, token shift) from the upstream project itself.

Run once, in a container that has the upstream checkout (read-only) at
$FOX_REFERENCE_SRC (the directory that holds the ``forgetting_transformer`` package):

    FOX_REFERENCE_SRC=<upstream>/src TRITON_INTERPRET=1 python tests/golden/make_golden_glue.py

* norms: upstream's pure-PyTorch references ``group_norm_gated_ref`` (fuse_norm_gate.py:18-53) and
  ``group_norm_ref`` (layernorm.py:77-110), called on CPU with upcast=True in the FoX layer's
  configuration (is_rms_norm, sigmoid gate, weight, no bias); gradients by autograd through them.
* row RMSNorm with residual (the block's input norms): ``rms_norm_ref`` (layernorm.py:53-74), upcast=True,
  prenorm=True, gradients by autograd with a gradient flowing into both outputs.
* token shift: upstream's own Triton kernels (token_shift.py:21-157) in Triton's CPU interpreter, fp16,
  called through ``token_shift`` exactly as ShiftLinear does (alpha, 1 - alpha).  The kernels carry an
  autotuner, which needs a GPU to time its candidates; the generator pins the one tuned parameter
  (BLOCK_T = 64, one of upstream's own candidates) and calls the jitted functions underneath.
Inputs and outputs are stored in ``glue_refs.npz``; the tests never need the upstream checkout.
"""
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")
import numpy as np
import torch

REF = os.environ["FOX_REFERENCE_SRC"]
sys.path.insert(0, REF)
sys.dont_write_bytecode = True
from forgetting_transformer.model.forgetting_transformer.fuse_norm_gate import group_norm_gated_ref  # noqa: E402
from forgetting_transformer.model.forgetting_transformer.layernorm import group_norm_ref, rms_norm_ref  # noqa: E402
from forgetting_transformer.model.forgetting_transformer.token_shift import token_shift  # noqa: E402

import forgetting_transformer.model.forgetting_transformer.token_shift as ts_mod  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


class _Pinned:
    """Stands in for triton's Autotuner: same ``kernel[grid](...)`` call, BLOCK_T fixed."""

    def __init__(self, tuner, block_t=64):
        self.fn, self.block_t = tuner.fn, block_t

    def __getitem__(self, grid):
        g = grid({"BLOCK_T": self.block_t}) if callable(grid) else grid
        return lambda *a, **k: self.fn[g](*a, BLOCK_T=self.block_t, **k)


ts_mod.shift_fwd_kernel = _Pinned(ts_mod.shift_fwd_kernel)
ts_mod.shift_bwd_kernel = _Pinned(ts_mod.shift_bwd_kernel)


def main():
    rec = {}
    g = torch.Generator().manual_seed(11)
    # ---- norms: (B, T, G*D) with G heads of D channels ----
    B, T, G, D = 2, 37, 3, 64
    x = torch.randn(B, T, G * D, generator=g).half()
    gate = torch.randn(B, T, G * D, generator=g).half()
    w = (torch.rand(G * D, generator=g) + 0.5)
    dy = torch.randn(B, T, G * D, generator=g).half()
    xx, gg, ww = [t.clone().requires_grad_() for t in (x, gate, w)]
    y = group_norm_gated_ref(xx, gg, ww, None, num_groups=G, eps=1e-6, is_rms_norm=True,
                             upcast=True)
    y.backward(dy)
    rec.update(ng_x=x.numpy(), ng_g=gate.numpy(), ng_w=w.numpy(), ng_dy=dy.numpy(), ng_y=y.detach().numpy(),
               ng_dx=xx.grad.numpy(), ng_dg=gg.grad.numpy(), ng_dw=ww.grad.numpy(), ng_groups=np.int64(G),
               ng_eps=np.float64(1e-6))
    xx, ww = [t.clone().requires_grad_() for t in (x, w)]
    y = group_norm_ref(xx, ww, None, num_groups=G, eps=1e-5, is_rms_norm=True, upcast=True)
    y.backward(dy)
    rec.update(qk_y=y.detach().numpy(), qk_dx=xx.grad.numpy(), qk_dw=ww.grad.numpy(), qk_eps=np.float64(1e-5))
    # ---- row RMSNorm with residual, prenorm: (B, T, hidden) ----
    Bn, Tn, Hn = 2, 19, 768
    x = torch.randn(Bn, Tn, Hn, generator=g).half()
    res = torch.randn(Bn, Tn, Hn, generator=g).half()
    w = torch.rand(Hn, generator=g) + 0.5
    dy = torch.randn(Bn, Tn, Hn, generator=g).half()
    dres = torch.randn(Bn, Tn, Hn, generator=g).half()
    xx, rr, ww = [t.clone().requires_grad_() for t in (x, res, w)]
    y, z = rms_norm_ref(xx, ww, None, residual=rr, eps=1e-5, prenorm=True, upcast=True)
    torch.autograd.backward([y, z], [dy, dres.float()])
    rec.update(rn_x=x.numpy(), rn_res=res.numpy(), rn_w=w.numpy(), rn_dy=dy.numpy(), rn_dres=dres.numpy(),
               rn_y=y.detach().numpy(), rn_z=z.detach().numpy(), rn_dx=xx.grad.numpy(), rn_dr=rr.grad.numpy(),
               rn_dw=ww.grad.numpy(), rn_eps=np.float64(1e-5))
    # ---- token shift: (B, T, H, D), weights (B, T, H) fp32 ----
    B, T, H, D = 2, 70, 3, 32
    x = torch.randn(B, T, H, D, generator=g).half()
    alpha = torch.rand(B, T, H, generator=g)
    dout = torch.randn(B, T, H, D, generator=g).half()
    xx = x.clone().requires_grad_()
    pw = alpha.clone().requires_grad_()
    cw = (1.0 - alpha).clone().requires_grad_()
    out = token_shift(xx, pw, cw)
    out.backward(dout)
    rec.update(ts_x=x.numpy(), ts_prev=alpha.numpy(), ts_curr=(1.0 - alpha).numpy(), ts_dout=dout.numpy(),
               ts_out=out.detach().numpy(), ts_dx=xx.grad.numpy(), ts_dprev=pw.grad.numpy(),
               ts_dcurr=cw.grad.numpy())
    np.savez_compressed(os.path.join(HERE, "glue_refs.npz"), **rec)
    print({k: v.shape for k, v in rec.items()})


if __name__ == "__main__":
    main()
