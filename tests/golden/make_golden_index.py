"""Generates ``index_scans.npz``: the block-pruning index arrays of upstream's own scan kernels.

Run once, in a container that has the upstream checkout (read-only) at $FOX_REFERENCE_SRC
(the directory that holds the ``forgetting_transformer`` package):

    FOX_REFERENCE_SRC=<upstream>/src TRITON_INTERPRET=1 python tests/golden/make_golden_index.py

It launches upstream's ``_find_start_index_kernel`` and ``_find_end_index_kernel``
(forgetting_attention.py:695-795) directly, in Triton's CPU interpreter, with the argument lists
of upstream's own call sites (lines 163-172 and 289-298), on fp32 prefix sums formed by
``torch.cumsum`` exactly as upstream forms them (line 127).  Cases: the (M, N, BLOCK_M, BLOCK_N)
grid of small shapes, ragged and with seqlen_q < seqlen_k, at four thresholds per head, and one
full-length T = 16384 row set with the gate distribution of the pruning stress configuration
(logit ~ N(-1, 1.5)) and thresholds in the range its "auto" rule produces.  Stored per case:
the prefix sum's inputs (log gates), thresholds, and both index arrays.
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

# name: (B, H, M, N, BLOCK_M, BLOCK_N, gate mean, gate std, thresholds per head)
CASES = {
    "sq512_128x64": (2, 4, 512, 512, 128, 64, 2.0, 1.0, [-1.0, -5.0, -20.0, -1000.0]),
    "ragged_1020_2098_128x64": (2, 4, 1020, 2098, 128, 64, 2.5, 1.0, [0.0, -3.0, -12.0, -40.0]),
    "mltn_1024_2048_64x64": (1, 4, 1024, 2048, 64, 64, 3.0, 1.0, [-0.5, -2.0, -8.0, -30.0]),
    "ragged_500_32x128": (2, 4, 500, 500, 32, 128, 1.0, 1.0, [-1.0, -10.0, -25.0, -100.0]),
    "sq1000_128x128": (2, 4, 1000, 1000, 128, 128, 1.5, 1.2, [-2.0, -6.0, -18.0, -60.0]),
    "mltn_1020_2098_128x128": (2, 4, 1020, 2098, 128, 128, 2.5, 1.0, [0.0, -3.0, -12.0, -40.0]),
    # pruning stress configuration at full length (one batch row, four heads), 128x128 as the sm_100a kernels
    "stress_16384_128x128": (1, 4, 16384, 16384, 128, 128, -1.0, 1.5, [-28.0, -45.0, -90.0, -160.0]),
}


def run_scans(lam, thr, M, N, bm, bn):
    B, H, _ = lam.shape
    P = N - M
    start = torch.empty((B, H, -(-M // bm)), dtype=torch.long)
    end = torch.empty((B, H, -(-N // bn)), dtype=torch.long)
    common = dict(BLOCK_M=bm, BLOCK_N=bn, DIVISIBLE_M=M % bm == 0, DIVISIBLE_N=N % bn == 0, num_warps=1)
    ops._find_start_index_kernel[(H, B)](
        lam, start, thr, lam.stride(0), lam.stride(1), lam.stride(2), start.stride(0), start.stride(1),
        start.stride(2), thr.stride(0), thr.stride(1), B, H, M, N, P, **common)
    ops._find_end_index_kernel[(H, B)](
        lam, end, thr, lam.stride(0), lam.stride(1), lam.stride(2), end.stride(0), end.stride(1),
        end.stride(2), thr.stride(0), thr.stride(1), B, H, M, N, P, **common)
    return start, end


def main():
    rec = {}
    for idx, (name, (B, H, M, N, bm, bn, mu, sigma, thr)) in enumerate(CASES.items()):
        g = torch.Generator().manual_seed(700 + idx)
        lf = torch.nn.functional.logsigmoid(torch.randn(B, H, N, generator=g) * sigma + mu)
        lam = torch.cumsum(lf, dim=-1)
        thr_t = torch.tensor(thr, dtype=torch.float32).expand(B, H).contiguous()
        start, end = run_scans(lam, thr_t, M, N, bm, bn)
        rec[name + "/shape"] = np.asarray([B, H, M, N, bm, bn], dtype=np.int64)
        rec[name + "/log_fgate"] = lf.numpy()
        rec[name + "/threshold"] = thr_t.numpy()
        rec[name + "/start_index"] = start.numpy()
        rec[name + "/end_index"] = end.numpy()
        print(name, "start max", int(start.max()), "end min", int(end.min()), flush=True)
    np.savez_compressed(os.path.join(HERE, "index_scans.npz"), **rec)


if __name__ == "__main__":
    main()
