"""CPU tests: the oracle (oracle/fox_oracle.py) against the golden fixtures that were
produced by upstream's own Triton kernels (interpreter mode), plus its internal
consistency.  No GPU needed."""
import math

import numpy as np
import pytest
import torch

from oracle import fox_oracle as orc

# upstream's own known-answer tolerance (forgetting_attention.py:1416-1425): atol 1e-2, rtol 0, fp16
ATOL = 1e-2


def _err(a, b):
    return (a.float() - b.float()).abs().max().item()


def test_golden_fixtures_present():
    from conftest import golden_names
    assert len(golden_names()) >= 6


def test_dense_oracle_matches_upstream_kernels(golden):
    g = golden
    out, dq, dk, dv, dlf = orc.dense_fwd_bwd(g["q"].float(), g["k"].float(), g["v"].float(), g["log_fgate"],
                                             g["dout"].float(), g["seq_start"], g["sm_scale"], mask_gates=True)
    # pruning (where on) removes at most exp(threshold) of the mass: same tolerance
    assert _err(out, g["out"]) < ATOL
    assert _err(dq, g["dq"]) < ATOL
    assert _err(dk, g["dk"]) < ATOL
    assert _err(dv, g["dv"]) < ATOL
    assert _err(dlf, g["dlog_fgate"]) < ATOL


def test_blockwise_oracle_matches_upstream_kernels(golden):
    """The block-level restatement with pruning index arrays reproduces upstream's
    outputs, log-normaliser and gradients (tighter than the dense one when pruning is on)."""
    g = golden
    B, H, M, D = g["q"].shape
    N = g["k"].shape[2]
    si = ei = None
    if g["threshold"] is not None:
        lam = orc.log_lambda(g["log_fgate"], g["seq_start"]).numpy()
        si = orc.find_start_index(lam, g["threshold"].numpy(), M, N, 128, 128)
        ei = orc.find_end_index(lam, g["threshold"].numpy(), M, N, 128, 128)
    r = orc.blockwise_fwd_bwd(g["q"], g["k"], g["v"], g["log_fgate"], g["dout"], g["seq_start"], g["sm_scale"],
                              start_index=si, end_index=ei)
    assert _err(r["out"], g["out"]) < 2e-3
    Lg = g["L"]
    finite = torch.isfinite(Lg)
    assert torch.equal(finite, torch.isfinite(r["L"]))
    assert _err(r["L"][finite], Lg[finite]) < 2e-3
    assert _err(r["dq"], g["dq"]) < 4e-3
    assert _err(r["dk"], g["dk"]) < 4e-3
    assert _err(r["dv"], g["dv"]) < 4e-3
    assert _err(r["dlog_fgate"], g["dlog_fgate"]) < ATOL  # a sum over up to N terms of magnitude ~1


def test_find_start_index_bit_exact(golden):
    g = golden
    if g["threshold"] is None:
        pytest.skip("no pruning in this fixture")
    B, H, M, D = g["q"].shape
    N = g["k"].shape[2]
    # upstream computes log_lambda with torch.cumsum on the masked gates: same call here
    lam = orc.log_lambda(g["log_fgate"], g["seq_start"]).numpy()
    si = orc.find_start_index(lam, g["threshold"].numpy(), M, N, 128, 128)
    assert np.array_equal(si, g["start_index"].numpy())


def test_index_scans_bit_exact_against_upstream_scan_kernels():
    """Both carried scans (start and end index) against the arrays upstream's own scan kernels produced
    (tests/golden/index_scans.npz): small ragged grids at several block sizes, seqlen_q < seqlen_k, and a
    full-length T = 16384 case with the pruning stress configuration's gate distribution."""
    from conftest import load_index_golden
    cases = load_index_golden()
    assert "stress_16384_128x128" in cases and len(cases) >= 7
    for name, c in cases.items():
        B, H, M, N, bm, bn = c["shape"]
        lam = torch.cumsum(torch.from_numpy(c["log_fgate"]), dim=-1).numpy()
        si = orc.find_start_index(lam, c["threshold"], M, N, bm, bn)
        ei = orc.find_end_index(lam, c["threshold"], M, N, bm, bn)
        assert np.array_equal(si, c["start_index"]), name
        assert np.array_equal(ei, c["end_index"]), name
    stress = cases["stress_16384_128x128"]
    assert orc.pruned_tile_fraction(stress["start_index"], 16384, 16384, 128, 128) > 0.9


def test_some_fixture_actually_prunes():
    from conftest import load_golden
    assert int(load_golden("acp_thr_m10")["start_index"].max()) >= 128


def test_index_scans_monotone_equivalence():
    """With a non-increasing prefix the carried scans equal the per-tile predicate
    keep(mb, nb) = lam[P + mb*BM] - lam[last col of nb] >= thr."""
    rng = np.random.default_rng(0)
    for (M, N, BM, BN) in [(512, 512, 128, 128), (1020, 2098, 128, 64), (1024, 2048, 64, 64), (500, 500, 32, 128)]:
        lf = -np.abs(rng.normal(0.05, 0.05, size=(2, 3, N))).astype(np.float32)
        lam = np.cumsum(lf, axis=-1, dtype=np.float32)
        thr = np.array([[-1.0, -5.0, -20.0], [-0.5, -3.0, -1000.0]], dtype=np.float32)
        si = orc.find_start_index(lam, thr, M, N, BM, BN)
        ei = orc.find_end_index(lam, thr, M, N, BM, BN)
        P = N - M
        for b in range(2):
            for h in range(3):
                for mb in range(si.shape[-1]):
                    row = lam[b, h, P + mb * BM]
                    exp = 0
                    while np.float32(row - lam[b, h, min(N - 1, exp + BN - 1)]) < thr[b, h]:
                        exp += BN
                    assert si[b, h, mb] == exp
                assert np.all(np.diff(si[b, h]) >= 0) and np.all(np.diff(ei[b, h]) >= 0)
                assert ei[b, h].max() <= M


def test_auto_threshold_dtype_path():
    """The automatic threshold is evaluated in the input dtype (bf16) and only then cast
    to fp32 (upstream lines 95-104)."""
    g = torch.Generator().manual_seed(0)
    q = torch.randn(2, 3, 64, 64, generator=g).bfloat16()
    k = torch.randn(2, 3, 64, 64, generator=g).bfloat16()
    thr = orc.auto_threshold(q, k, 0.125)
    assert thr.dtype == torch.float32 and thr.shape == (2, 3)
    # every value is exactly representable in bf16
    assert torch.equal(thr, thr.bfloat16().float())
    ub = (q.float().norm(dim=-1).amax(-1) * k.float().norm(dim=-1).amax(-1) * 0.125)
    assert torch.allclose(thr, -(2 * ub + math.log(64)) - 10, rtol=2e-2)


def test_reverse_cumsum():
    x = torch.randn(2, 3, 100)
    ref = torch.flip(torch.cumsum(torch.flip(x, [-1]), -1), [-1])
    assert torch.allclose(orc.reverse_cumsum(x), ref, atol=1e-5)


def test_masked_prefix_ignores_gates_left_of_seq_start():
    lf = -torch.rand(2, 2, 50)
    ss = torch.tensor([0, 17])
    lam = orc.log_lambda(lf, ss)
    assert torch.all(lam[1, :, :17] == 0)
    assert torch.allclose(lam[0], torch.cumsum(lf[0], -1))
    lf2 = lf.clone()
    lf2[1, :, :17] = -100.0
    assert torch.equal(orc.log_lambda(lf2, ss), lam)


def test_rowsum_of_ds_vanishes_in_exact_arithmetic():
    """Softmax is shift invariant, so the query-side part of the log-gate gradient is
    pure rounding residue; the blockwise oracle in fp32 shows it is tiny."""
    g = torch.Generator().manual_seed(1)
    q, k, v, do = [torch.randn(1, 1, 96, 64, generator=g) for _ in range(4)]
    lf = torch.nn.functional.logsigmoid(torch.randn(1, 1, 96, generator=g))
    r = orc.blockwise_fwd_bwd(q, k, v, lf, do, low_precision_matmul=False)
    _, _, _, _, dlf = orc.dense_fwd_bwd(q, k, v, lf, do)
    assert _err(r["dlog_fgate"], dlf) < 1e-4


def test_norm_gate_reference_math():
    g = torch.Generator().manual_seed(2)
    x = torch.randn(2, 5, 4 * 64, generator=g)
    gate = torch.randn(2, 5, 4 * 64, generator=g)
    w = torch.rand(4 * 64, generator=g) + 0.5
    y = orc.group_rmsnorm_gated(x, gate, w, 4, eps=1e-6)
    xg = x.view(2, 5, 4, 64)
    ref = (xg / xg.pow(2).mean(-1, keepdim=True).add(1e-6).sqrt()).reshape(2, 5, -1) * w * torch.sigmoid(gate)
    assert torch.allclose(y, ref, atol=1e-5)


def test_glue_oracles_against_upstream_references():
    """Per-head RMSNorm with and without the gate against upstream's reference functions, token shift
    against upstream's own kernels (tests/golden/glue_refs.npz)."""
    from conftest import load_glue_golden
    z = load_glue_golden()
    G = int(z["ng_groups"])
    y, dx, dg, dw = orc.group_rmsnorm_gated_fwd_bwd(z["ng_x"], z["ng_g"], z["ng_w"], z["ng_dy"], G, z["ng_eps"])
    # upstream's reference function evaluates sigmoid(g) in g's 16-bit dtype, its kernel (and the oracle) in
    # fp32: outputs may differ by one fp16 ulp
    assert _err(y, z["ng_y"]) < 2e-3
    assert _err(dx, z["ng_dx"]) < 2e-3 and _err(dg, z["ng_dg"]) < 2e-3
    assert _err(dw, z["ng_dw"]) < 1e-3 * z["ng_dw"].abs().max()  # sums of 74 such terms
    y, dx, dw = orc.group_rmsnorm_fwd_bwd(z["ng_x"], z["ng_w"], z["ng_dy"], G, z["qk_eps"])
    assert torch.equal(y, z["qk_y"])
    assert _err(dx, z["qk_dx"]) < 2e-3
    assert _err(dw, z["qk_dw"]) < 1e-4 * z["qk_dw"].abs().max()
    out, dx, dprev, dcurr = orc.token_shift_fwd_bwd(z["ts_x"], z["ts_prev"], z["ts_curr"], z["ts_dout"])
    assert torch.equal(out, z["ts_out"]) and torch.equal(dx, z["ts_dx"])
    assert _err(dprev, z["ts_dprev"]) < 1e-4 and _err(dcurr, z["ts_dcurr"]) < 1e-4
    # row RMSNorm with residual, prenorm (upstream's reference keeps the sum in fp32; the kernel and the oracle
    # return it rounded to the input dtype, and differentiate through the rounded copy)
    y, zs, dx, dw = orc.rms_norm_fwd_bwd(z["rn_x"], z["rn_w"], z["rn_res"], z["rn_dy"], z["rn_dres"], z["rn_eps"])
    assert torch.equal(y, z["rn_y"]) and torch.equal(zs, z["rn_z"].to(zs.dtype))
    assert _err(dx, z["rn_dx"]) < 4e-3 and _err(dx, z["rn_dr"]) < 4e-3
    assert _err(dw, z["rn_dw"]) < 2e-3 * z["rn_dw"].abs().max()


def test_cross_entropy_oracle_against_upstream_kernels():
    """Losses, z-losses and the gradient of the logits against upstream's own fused cross-entropy kernels
    (tests/golden/cross_entropy.npz): fp32 and fp16 logits, 1003 classes, ignore_index rows, label smoothing,
    logit scale and z-loss."""
    from conftest import load_ce_golden
    cases = load_ce_golden()
    assert len(cases) == 8
    for name, c in cases.items():
        ls, scale, zs = [float(x) for x in c["args"]]
        losses, zl, dl = orc.cross_entropy_fwd_bwd(c["logits"], c["labels"], c["dloss"], label_smoothing=ls,
                                                   logit_scale=scale, lse_square_scale=zs)
        # (with 16-bit logits upstream forms logit_scale * logits[label] and its (1 - smoothing) multiple in the
        # logits' dtype, lines 65-72: its loss carries that one rounding of a value of magnitude <= 16)
        loss_tol = 2e-5 * max(1.0, c["losses"].abs().max().item()) if c["logits"].dtype == torch.float32 else 8e-3
        assert _err(losses, c["losses"]) < loss_tol, name
        assert _err(zl, c["z_losses"]) < 1e-6, name
        # upstream returns the gradient in the logits' dtype
        tol = 1e-6 if c["logits"].dtype == torch.float32 else 2e-3 * c["dlogits"].float().abs().max().item()
        assert _err(dl, c["dlogits"]) < tol, name
        assert torch.all(losses[c["labels"] == -100] == 0) and torch.all(dl[c["labels"] == -100] == 0)
