"""Generates the golden fixtures in this directory from the upstream project itself.

Run once, in a container that has the upstream checkout (read-only) at
$FOX_REFERENCE_SRC (the directory that holds the ``forgetting_transformer`` package):

    FOX_REFERENCE_SRC=<upstream>/src TRITON_INTERPRET=1 python tests/golden/make_golden.py

It imports upstream's ``forgetting_transformer.ops.forgetting_attention`` and runs
its *own Triton kernels* in Triton's CPU interpreter (fp16 -- the interpreter has no
bf16), with the three block-size hooks upstream documents as overridable
(get_fwd_config / get_bwd_kv_config / get_bwd_q_config) pinned to 128x128 so that
the pruning index arrays live on the same block grid as the sm_100a kernels.  Inputs
and outputs (out, log-normaliser, start_index, dq, dk, dv, dlog_fgate) are stored as
compressed .npz files; the tests never need the upstream checkout.
"""
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")
import numpy as np
import torch

REF = os.environ["FOX_REFERENCE_SRC"]
sys.path.insert(0, REF)
sys.dont_write_bytecode = True
import forgetting_transformer.ops.forgetting_attention as ops  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
BLOCK = (128, 128, 1, 4)
ops.get_fwd_config = lambda *a, **k: BLOCK
ops.get_bwd_kv_config = lambda *a, **k: BLOCK
ops.get_bwd_q_config = lambda *a, **k: BLOCK

CASES = {
    # name: (B, H, M, N, D, gate mean, gate std, seq_start, threshold, sm_scale, input std)
    "cfg1_shape_seqstart": (2, 4, 256, 256, 64, 0.0, 1.0, [0, 37], None, None, 1.0),
    "acp_thr_m10": (1, 2, 512, 512, 64, -1.0, 1.5, None, -10.0, None, 1.0),
    "acp_per_head_thr_seqstart": (2, 2, 384, 384, 64, 0.0, 1.0, [130, 5], [-6.0, -40.0], 0.5, 0.5),
    "ragged_m_lt_n": (1, 2, 200, 328, 64, 2.5, 1.4, [0], None, 0.5, 0.5),
    "ragged_m_lt_n_seqstart_thr": (2, 1, 200, 328, 64, 0.0, 1.0, [40, 300], -8.0, 0.5, 0.5),
    "d128": (1, 2, 256, 256, 128, 1.0, 1.0, None, None, None, 1.0),
}


def make_inputs(seed, B, H, M, N, D, mu, sigma, std):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, H, M, D, generator=g) * std).half()
    k = (torch.randn(B, H, N, D, generator=g) * std).half()
    v = (torch.randn(B, H, N, D, generator=g) * std).half()
    log_fgate = torch.nn.functional.logsigmoid(torch.randn(B, H, N, generator=g) * sigma + mu)
    dout = torch.randn(B, H, M, D, generator=g).half()
    return q, k, v, log_fgate, dout


def main():
    for idx, (name, (B, H, M, N, D, mu, sigma, seq, thr, sm_scale, std)) in enumerate(CASES.items()):
        q, k, v, lf, dout = make_inputs(100 + idx, B, H, M, N, D, mu, sigma, std)
        seq_t = None if seq is None else torch.tensor(seq, dtype=torch.long)
        thr_t = None
        if thr is not None:
            thr_t = torch.tensor(thr, dtype=torch.float32) if isinstance(thr, list) else float(thr)
        qq, kk, vv, ll = [t.clone().requires_grad_() for t in (q, k, v, lf)]
        out, L, start_index = ops.ForgettingAttention.apply(
            qq, kk, vv, ll, seq_t, True, sm_scale, thr_t, True, thr is not None, None, False, False)
        out.backward(dout)
        rec = dict(
            q=q.numpy(), k=k.numpy(), v=v.numpy(), log_fgate=lf.numpy(), dout=dout.numpy(),
            out=out.detach().numpy(), L=L.detach().numpy(), dq=qq.grad.numpy(), dk=kk.grad.numpy(),
            dv=vv.grad.numpy(), dlog_fgate=ll.grad.numpy(),
            sm_scale=np.float64(sm_scale if sm_scale is not None else D ** -0.5),
        )
        if seq is not None:
            rec["seq_start"] = np.asarray(seq, dtype=np.int64)
        if thr is not None:
            rec["threshold"] = np.broadcast_to(np.asarray(thr, dtype=np.float32), (B, H)).copy()
            rec["start_index"] = start_index.numpy()
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
        print(name, "out", tuple(out.shape), "pruned start_index max",
              None if thr is None else int(start_index.max()), flush=True)


if __name__ == "__main__":
    main()
