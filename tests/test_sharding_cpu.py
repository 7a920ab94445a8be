"""CPU tests (gloo, world_size 2) of the multi-GPU host logic: batch x head unit slicing and
the zig-zag context-parallel wrapper, with the oracle standing in for the CUDA operator."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from forgetting_transformer_b200 import sharding
from oracle import fox_oracle as orc


def test_unit_slices_cover_everything_once():
    for n, w in [(48, 1), (48, 2), (48, 8), (7, 4), (3, 8)]:
        got = []
        for r in range(w):
            a, b = sharding.unit_slice(n, w, r)
            got += list(range(a, b))
        assert got == list(range(n))


def test_shard_batch_heads_views_and_metadata():
    B, H, T, D = 2, 3, 8, 4
    q = torch.arange(B * H * T * D, dtype=torch.float32).reshape(B, H, T, D)
    lf = torch.zeros(B, H, T)
    seq = torch.tensor([1, 5])
    thr = torch.tensor([-1.0, -2.0, -3.0])
    pieces = []
    for r in range(4):
        qs, ks, vs, ls, ss, th = sharding.shard_batch_heads(q, q, q, lf, seq, thr, world=4, rank=r)
        assert qs.shape[1] == 1 and qs.shape[0] == ss.shape[0] == th.shape[0]
        assert qs.data_ptr() >= q.data_ptr()  # views, not copies
        pieces.append((qs, ss, th))
    assert torch.equal(torch.cat([p[0] for p in pieces]).reshape(B, H, T, D), q)
    assert torch.cat([p[1] for p in pieces]).tolist() == [1, 1, 1, 5, 5, 5]
    assert torch.cat([p[2] for p in pieces]).flatten().tolist() == [-1, -2, -3, -1, -2, -3]


def _oracle_attn(q, k, v, lf, head_first=True, seq_start=None, sm_scale=None, adaptive_threshold=None):
    _oracle_attn.thresholds.append(adaptive_threshold)
    if seq_start is not None:                  # the operator zeroes the gates left of seq_start (OPS:117-125)
        mask = torch.arange(lf.shape[-1])[None, None, :] < seq_start[:, None, None]
        lf = torch.where(mask, torch.zeros_like(lf), lf)
    return orc.dense_forgetting_attention(q, k, v, lf, seq_start, sm_scale)


_oracle_attn.thresholds = []


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _cp_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        B, H, D = 2, 2, 16
        tc = 8
        T = 2 * world * tc
        q, k, v, do = [torch.randn(B, H, T, D, dtype=torch.float64) for _ in range(4)]
        lf = torch.nn.functional.logsigmoid(torch.randn(B, H, T, dtype=torch.float64))
        a, b = sharding.zigzag_chunks(world, rank)
        idx = torch.cat([torch.arange(a * tc, (a + 1) * tc), torch.arange(b * tc, (b + 1) * tc)])
        worst = 0.0
        # no padding; left padding inside the first chunk and beyond it (whole lower chunks of rank 0 are empty)
        # (and the same cut into two head groups, which on CUDA run on their own streams)
        for seq, hg in ((None, 1), (torch.tensor([3, tc + 5]), 1), (torch.tensor([3, tc + 5]), 2)):
            ro, rdq, rdk, rdv, rdl = orc.dense_fwd_bwd(q, k, v, lf, do, seq, mask_gates=True)
            ql, kl, vl, ll = [t.index_select(2, idx).clone().requires_grad_() for t in (q, k, v, lf)]
            out = sharding.context_parallel_attention(ql, kl, vl, ll, seq_start=seq, attn_fn=_oracle_attn,
                                                      head_groups=hg)
            out.backward(do.index_select(2, idx))
            errs = [
                (out - ro.index_select(2, idx)).abs().max().item(),
                (ql.grad - rdq.index_select(2, idx)).abs().max().item(),
                (kl.grad - rdk.index_select(2, idx)).abs().max().item(),
                (vl.grad - rdv.index_select(2, idx)).abs().max().item(),
            ]
            # left of seq_start the dense formulation's gate gradient is rounding residue only
            keep = torch.ones(B, H, T, dtype=torch.bool) if seq is None else (
                torch.arange(T)[None, None, :] >= seq[:, None, None]).expand(B, H, T)
            errs.append(((ll.grad - rdl.index_select(2, idx)) * keep.index_select(2, idx)).abs().max().item())
            worst = max(worst, *errs)
        # "auto": one threshold from the row norms of every rank's rows = the unsharded call's
        _oracle_attn.thresholds.clear()
        row_norm_max = lambda x: torch.linalg.vector_norm(x, dim=-1).max(dim=-1).values
        qb, kb, vb = [t.detach().bfloat16() for t in (ql, kl, vl)]   # the norms are taken in the input dtype
        sharding.context_parallel_attention(qb, kb, vb, ll.detach().float(), adaptive_threshold="auto",
                                            attn_fn=_oracle_attn, max_row_norm=row_norm_max, head_groups=1)
        ref_thr = orc.auto_threshold(q.bfloat16(), k.bfloat16(), D ** -0.5)
        same = all(torch.equal(t.double(), ref_thr.double()) for t in _oracle_attn.thresholds)
        ret[rank] = (worst, same and len(_oracle_attn.thresholds) == 2)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(240)
@pytest.mark.parametrize("world", [2, 4])
def test_context_parallel_matches_unsharded(world):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_cp_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert len(ret) == world
    assert max(w for w, _ in ret.values()) < 1e-5  # the dense formulation does its softmax in fp32
    assert all(same for _, same in ret.values())


def _ce_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from forgetting_transformer_b200 import cross_entropy as ce
        g = torch.Generator().manual_seed(5)
        rows, classes = 37, 64 * world
        logits = torch.randn(rows, classes, generator=g) * 3
        target = torch.randint(0, classes, (rows,), generator=g)
        target[::7] = -100
        worst = 0.0
        for eps, scale, zsq in ((0.0, 1.0, 0.0), (0.1, 0.5, 1e-4)):
            n = classes // world
            parts, lse_local = orc.cross_entropy_class_shard(logits[:, rank * n:(rank + 1) * n], target, rank * n,
                                                                classes, label_smoothing=eps, logit_scale=scale)
            losses, z_losses, lse = ce.join_class_shards(parts, lse_local, target, zsq, -100, None)
            ref_l, ref_z = orc.cross_entropy(logits, target, label_smoothing=eps, logit_scale=scale,
                                                lse_square_scale=zsq)
            ref_lse = torch.logsumexp(logits.float() * scale, dim=-1)
            worst = max(worst, float((losses - ref_l).abs().max()), float((z_losses - ref_z).abs().max()),
                        float((lse - ref_lse).abs().max()))
        ret[rank] = worst
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_cross_entropy_class_shards_join_to_the_unsplit_loss(world):
    """Every rank's (loss part, local log-sum-exp) of its slice of the classes, joined over gloo by the host code the
    CUDA path uses, equals the loss over all classes (label smoothing, logit scale, z-loss, ignored rows)."""
    ret = mp.Manager().dict()
    mp.spawn(_ce_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert len(ret) == world and max(ret.values()) < 1e-5, dict(ret)
