"""GPU test of ``fox_attn_bwd_noalloc``: the backward entry point for hosts that cannot
allocate device memory when they call (their own arena owns the GPU, or their thread may
not make a device-serialising call such as cudaMalloc).  Its dQ / gate-gradient scratch is a
fixed array inside the library instead of caller-allocated buffers.

The file name sorts last on purpose: should this test fail, a run that stops at the first
failure has already executed every other test.

Checked here, through the C ABI: two calls in a row (different upstream gradients, so stale
sums left in the shared array by the first call would show in the second) give the same dq,
dk, dv and dlog_fgate as the regular entry point, and a problem too large for the fixed
array is refused with FOX_ERR_TOO_LARGE.
"""
import ctypes

import pytest
import torch

from forgetting_transformer_b200 import _lib, ops

pytestmark = pytest.mark.gpu

ATOL_BF16, RTOL_BF16 = 2e-2, 1e-2


def _close(a, b, atol=ATOL_BF16, rtol=RTOL_BF16):
    """Every element within atol + rtol * |element of the regular entry point's result|."""
    err = (a.float() - b.float()).abs()
    over = err - (atol + rtol * b.float().abs())
    assert over.max().item() <= 0, f"max abs err {err.max().item():.3e}, {int((over > 0).sum())} elements over the bar"


def _noalloc_backward(lib, q, k, v, o, L, lam, do, seq, end_index, sm_scale):
    dev = q.device
    B, H, M, D = q.shape
    N = k.shape[2]
    code = _lib.dtype_code(q.dtype)
    stream = torch.cuda.current_stream().cuda_stream
    delta = torch.empty_like(L)
    _lib.check(lib.fox_bwd_delta(dev.index, stream, code, B, H, M, D, _lib.t4(o), _lib.t4(do), delta.data_ptr()),
               "fox_bwd_delta")
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    dlam_col = torch.empty((B, H, N), dtype=torch.float32, device=dev)
    dlog_fgate = torch.empty((B, H, N), dtype=torch.float32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    rc = lib.fox_attn_bwd_noalloc(dev.index, stream, code, B, H, M, N, D, _lib.t4(q), _lib.t4(k), _lib.t4(v),
                                  _lib.t4(do), lam.data_ptr(), L.data_ptr(), delta.data_ptr(), _lib.ptr(seq),
                                  _lib.ptr(end_index), float(sm_scale), _lib.t4(dq), _lib.t4(dk), _lib.t4(dv),
                                  dlam_col.data_ptr(), dlog_fgate.data_ptr(), status.data_ptr())
    _lib.check(rc, "fox_attn_bwd_noalloc")
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0
    return dq, dk, dv, dlog_fgate


@pytest.mark.parametrize("B,H,M,N,D,with_seq,thr", [(2, 3, 384, 384, 64, True, None), (1, 2, 200, 456, 128, False, -6.0)])
def test_noalloc_backward_matches_regular_entry_point(B, H, M, N, D, with_seq, thr):
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(B * 1000 + D)
    q = torch.randn(B, H, M, D, generator=g).bfloat16().to(dev)
    k = torch.randn(B, H, N, D, generator=g).bfloat16().to(dev)
    v = torch.randn(B, H, N, D, generator=g).bfloat16().to(dev)
    lf = torch.nn.functional.logsigmoid(torch.randn(B, H, N, generator=g)).to(dev)
    seq = torch.randint(0, N - 1, (B,), generator=g).to(dev) if with_seq else None
    sm_scale = D ** -0.5
    thr_t = None if thr is None else torch.full((B, H), thr, dtype=torch.float32, device=dev)
    lam = ops.log_lambda_cumsum(lf, seq)
    end_index = None
    if thr_t is not None:
        _, end_index = ops.find_index(lam, thr_t, M, *ops.BWD_BLOCK, want_start=False, want_end=True)
    for call in range(2):  # two calls in a row share the library's scratch array
        do = (torch.randn(B, H, M, D, generator=g) * (1.0 + 3.0 * call)).bfloat16().to(dev)
        qq, kk, vv, ll = [t.detach().clone().requires_grad_() for t in (q, k, v, lf)]
        out, L, _ = ops.ForgettingAttention.apply(qq, kk, vv, ll, seq, True, sm_scale, thr_t, True, False, None,
                                                  False, False)
        out.backward(do)
        torch.cuda.synchronize()
        _lib.check_status()
        dq, dk, dv, dlf = _noalloc_backward(lib, q, k, v, out.detach(), L, lam, do, seq, end_index, sm_scale)
        _close(dq, qq.grad)
        _close(dk, kk.grad)
        _close(dv, vv.grad)
        _close(dlf, ll.grad)


def test_noalloc_refuses_sizes_beyond_the_fixed_array():
    lib = _lib.load()
    cap = lib.fox_noalloc_scratch_floats()
    assert cap == 1 << 24
    dev = torch.device("cuda", 0)
    B, H, M, D = 1, 16, 16384, 64  # 16*16384*65 floats > 2^24
    assert B * H * M * (D + 1) > cap
    dummy = torch.zeros(16, dtype=torch.float32, device=dev)
    t4 = _lib.Tensor4(dummy.data_ptr(), 0, 0, 0)
    rc = lib.fox_attn_bwd_noalloc(0, torch.cuda.current_stream().cuda_stream, _lib.FOX_DTYPE_BF16, B, H, M, M, D,
                                  t4, t4, t4, t4, dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), None, None,
                                  0.125, t4, t4, t4, dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr())
    assert rc == -8  # FOX_ERR_TOO_LARGE, nothing was launched
    torch.cuda.synchronize()
