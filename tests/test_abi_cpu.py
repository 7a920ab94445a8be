"""CPU tests of the boundary: the C-ABI library loads and exports every symbol the
header declares, and the Python host mirrors upstream's argument checks.  No compute
call is made (there is no GPU here and no CPU path in the product)."""
import ctypes
import os
import re

import pytest
import torch

import forgetting_transformer_b200 as fox
from forgetting_transformer_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "fox_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fox_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    syms = _declared_symbols()
    for s in ["fox_attn_fwd", "fox_attn_bwd", "fox_cumsum_fwd", "fox_revcumsum", "fox_find_index",
              "fox_max_row_norm", "fox_bwd_delta", "fox_dq_convert", "fox_normgate_fwd", "fox_normgate_bwd",
              "fox_token_shift_fwd", "fox_token_shift_bwd", "fox_rmsnorm_fwd", "fox_rmsnorm_bwd",
              "fox_swiglu_fwd", "fox_swiglu_bwd", "fox_attn_decode", "fox_attn_bwd_dq"]:
        assert s in syms


def test_library_builds_and_exports_every_declared_symbol():
    path = build.build()
    lib = ctypes.CDLL(path)
    for s in _declared_symbols():
        assert hasattr(lib, s), f"{s} declared in include/fox_b200.h but not exported"
    lib.fox_version.restype = ctypes.c_char_p
    assert b"sm_100a" in lib.fox_version()


def test_library_exports_nothing_beyond_the_header():
    """The default build exports exactly the declared C ABI: no debug switches, no process-global hooks."""
    import subprocess
    path = build.build()
    out = subprocess.run(["nm", "-D", "--defined-only", path], capture_output=True, text=True, check=True).stdout
    exported = {line.split()[-1] for line in out.splitlines() if line.split()[-1].startswith("fox_")}
    assert exported == set(_declared_symbols()), exported ^ set(_declared_symbols())


def test_python_bindings_cover_every_declared_symbol():
    assert set(_declared_symbols()) <= set(_lib._SIGNATURES)


def _inputs(B=1, H=2, M=8, N=8, D=64, dtype=torch.bfloat16):
    q = torch.zeros(B, H, M, D, dtype=dtype)
    k = torch.zeros(B, H, N, D, dtype=dtype)
    v = torch.zeros(B, H, N, D, dtype=dtype)
    lf = torch.zeros(B, H, N, dtype=torch.float32)
    return q, k, v, lf


def test_dtype_assertions_match_upstream():
    q, k, v, lf = _inputs(dtype=torch.float32)
    with pytest.raises(AssertionError, match="Only torch.float16 or torch.bfloat16"):
        fox.forgetting_attention(q, k, v, lf, head_first=True)
    q, k, v, lf = _inputs()
    with pytest.raises(AssertionError, match="log_fgate must be in torch.float32"):
        fox.forgetting_attention(q, k, v, lf.half(), head_first=True)


def test_shape_assertions_match_upstream():
    q, k, v, lf = _inputs(D=48)
    with pytest.raises(AssertionError, match="head dims in"):
        fox.forgetting_attention(q, k, v, lf, head_first=True)
    q, k, v, lf = _inputs(M=16, N=8)
    with pytest.raises(AssertionError, match="longer than the query"):
        fox.forgetting_attention(q, k, v, lf, head_first=True)
    q, k, v, lf = _inputs()
    with pytest.raises(AssertionError):
        fox.forgetting_attention(q, k, v, lf[:, :1], head_first=True)
    with pytest.raises(AssertionError, match="groupped query attention"):
        fox.forgetting_attention(q, k[:, :1], v[:, :1], lf, head_first=True)


def test_no_cpu_fallback():
    q, k, v, lf = _inputs()
    with pytest.raises(_lib.FoxError, match="no CPU path"):
        fox.forgetting_attention(q, k, v, lf, head_first=True)
    with pytest.raises(_lib.FoxError, match="no CPU path"):
        fox.group_norm_gated(torch.zeros(2, 128, dtype=torch.bfloat16), torch.zeros(2, 128, dtype=torch.bfloat16),
                             torch.ones(128), is_rms_norm=True, activation="sigmoid", num_groups=2)


def test_norm_gate_rejects_unbuilt_configurations():
    x = torch.zeros(2, 128, dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError):
        fox.group_norm_gated(x, x, torch.ones(128), activation="swish", is_rms_norm=True, num_groups=2)
    with pytest.raises(NotImplementedError):
        fox.group_norm_gated(x, x, torch.ones(128), activation="sigmoid", is_rms_norm=False, num_groups=2)
    with pytest.raises(ValueError):
        fox.FusedGroupNormGated(3, 128)
    m = fox.FusedGroupNormGated(2, 128, is_rms_norm=True, eps=1e-6, activation="sigmoid")
    assert torch.all(m.weight == 1) and m.bias is None


def test_tma_ready_predicate():
    x = torch.zeros(2, 16, 4, 64, dtype=torch.bfloat16)
    assert _lib.tma_ready(x) and _lib.tma_ready(x.permute(0, 2, 1, 3))
    assert not _lib.tma_ready(x[..., 1:])            # base off by 2 bytes
    assert not _lib.tma_ready(x.transpose(2, 3))     # inner stride != 1
    y = torch.zeros(2, 16, 4, 68, dtype=torch.bfloat16)[..., :64]
    assert not _lib.tma_ready(y)                     # 136-byte row stride


def test_signature_matches_upstream():
    import inspect
    sig = inspect.signature(fox.forgetting_attention)
    names = list(sig.parameters)
    assert names == ["q", "k", "v", "log_fgate", "head_first", "seq_start", "sm_scale", "adaptive_threshold"]
    for n in names[4:]:
        assert sig.parameters[n].kind is inspect.Parameter.KEYWORD_ONLY
    assert sig.parameters["head_first"].default is False
    assert sig.parameters["seq_start"].default is None


def test_layer_glue_expressions():
    """The layer-side helpers restate upstream's expressions (modeling_forgetting_transformer.py:371-396)."""
    import math
    import forgetting_transformer_b200 as fox
    mask = torch.tensor([[0, 0, 1, 1, 1], [1, 1, 1, 1, 1]])
    assert fox.seq_start_from_attention_mask(mask).tolist() == [2, 0]
    g = torch.Generator().manual_seed(0)
    H, D, T, tol = 3, 64, 1000, -10.0
    wq, wk = torch.randn(H * D, generator=g), torch.randn(H * D, generator=g)
    thr = fox.acp_threshold_from_qk_norm(wq, wk, H, D, T, tol)
    ref = -(2 * wq.view(H, D).abs().max(-1).values * wk.view(H, D).abs().max(-1).values * math.sqrt(D)
            + math.log(T)) + tol
    assert thr.shape == (H,) and torch.equal(thr, ref)
    ws = fox.acp_threshold_from_qk_norm(wq[:D], wk[:D], H, D, T, tol, share_param_across_head=True)
    assert ws.dim() == 0 and ws.item() == (-(2 * wq[:D].abs().max() * wk[:D].abs().max() * math.sqrt(D)
                                              + math.log(T)) + tol).item()
