"""Generates ``cross_entropy.npz`` from upstream's own fused cross-entropy kernels.

Run once, in a container that has the upstream checkout (read-only) at $FOX_REFERENCE_SRC:

    FOX_REFERENCE_SRC=<upstream>/src TRITON_INTERPRET=1 python tests/golden/make_golden_ce.py

Imports upstream's ``cross_entropy_loss`` (fused_cross_entropy.py:275-312) and runs its Triton kernels in
Triton's CPU interpreter on fp32 and fp16 logits: a class count that is not a power of two, labels with
``ignore_index`` entries, and the four argument sets plain / label smoothing / logit scale + z-loss / all three.
Stored per case: logits, labels, the upstream gradient of the losses, and upstream's losses, z_losses, dlogits.
"""
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")
import numpy as np
import torch

REF = os.environ["FOX_REFERENCE_SRC"]
sys.path.insert(0, REF)
sys.dont_write_bytecode = True
from forgetting_transformer.model.forgetting_transformer.fused_cross_entropy import cross_entropy_loss  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
# upstream selects the logits' CUDA device around its launches; there is none in the interpreter
import contextlib  # noqa: E402
torch.cuda.device = lambda *_a, **_k: contextlib.nullcontext()
ARGS = {
    "plain": dict(),
    "smoothing": dict(label_smoothing=0.1),
    "scale_zloss": dict(logit_scale=0.5, lse_square_scale=1e-3),
    "all": dict(label_smoothing=0.05, logit_scale=1.5, lse_square_scale=1e-4),
}


def main():
    rec = {}
    g = torch.Generator().manual_seed(77)
    rows, cols = 37, 1003
    for dt_name, dt in (("fp32", torch.float32), ("fp16", torch.float16)):
        logits = (torch.randn(rows, cols, generator=g) * 3).to(dt)
        labels = torch.randint(0, cols, (rows,), generator=g)
        labels[[3, 17]] = -100
        dloss = torch.randn(rows, generator=g)
        for name, kw in ARGS.items():
            x = logits.clone().requires_grad_()
            losses, z_losses = cross_entropy_loss(x, labels, **kw)
            (losses * dloss).sum().backward()
            key = f"{dt_name}_{name}"
            rec[key + "/logits"] = logits.numpy()
            rec[key + "/labels"] = labels.numpy()
            rec[key + "/dloss"] = dloss.numpy()
            rec[key + "/losses"] = losses.detach().numpy()
            rec[key + "/z_losses"] = z_losses.detach().numpy()
            rec[key + "/dlogits"] = x.grad.numpy()
            rec[key + "/args"] = np.asarray([kw.get("label_smoothing", 0.0), kw.get("logit_scale", 1.0),
                                             kw.get("lse_square_scale", 0.0)], dtype=np.float64)
            print(key, float(losses.sum()), flush=True)
    np.savez_compressed(os.path.join(HERE, "cross_entropy.npz"), **rec)


if __name__ == "__main__":
    main()
