"""GPU tests of the partitioning helpers: batch x head slices through the unchanged operator
(one GPU), and the zig-zag context-parallel wrapper over NCCL (needs two GPUs, else skipped)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import forgetting_transformer_b200 as fox
from forgetting_transformer_b200 import _lib, sharding

pytestmark = pytest.mark.gpu


def _inputs(B, H, T, D, seed=0):
    g = torch.Generator().manual_seed(seed)
    q, k, v, do = [torch.randn(B, H, T, D, generator=g).bfloat16() for _ in range(4)]
    lf = torch.nn.functional.logsigmoid(torch.randn(B, H, T, generator=g) + 2)
    return q, k, v, lf, do


def test_batch_head_shards_reproduce_the_full_call():
    B, H, T, D = 2, 3, 384, 64
    q, k, v, lf, do = [t.cuda() for t in _inputs(B, H, T, D)]
    seq = torch.tensor([0, 100]).cuda()
    thr = torch.tensor([-5.0, -20.0, -1000.0]).cuda()
    qq, kk, vv, ll = [t.detach().clone().requires_grad_() for t in (q, k, v, lf)]
    full = fox.forgetting_attention(qq, kk, vv, ll, head_first=True, seq_start=seq, adaptive_threshold=thr)
    full.backward(do)
    world = 4
    outs, dqs, dls = [], [], []
    for rank in range(world):
        qs, ks, vs, ls, ss, th = sharding.shard_batch_heads(q, k, v, lf, seq, thr, world=world, rank=rank)
        if qs.shape[0] == 0:
            continue
        qs, ks, vs, ls = [t.detach().clone().requires_grad_() for t in (qs, ks, vs, ls)]
        o = fox.forgetting_attention(qs, ks, vs, ls, head_first=True, seq_start=ss, adaptive_threshold=th)
        u0, u1 = sharding.unit_slice(B * H, world, rank)
        o.backward(do.reshape(B * H, 1, T, D)[u0:u1])
        outs.append(o.detach()); dqs.append(qs.grad); dls.append(ls.grad)
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(torch.cat(outs).reshape(B, H, T, D), full.detach())   # same kernels, same tiles: bit-equal
    assert torch.allclose(torch.cat(dqs).reshape(B, H, T, D).float(), qq.grad.float(), atol=2e-2)
    assert torch.allclose(torch.cat(dls).reshape(B, H, T), ll.grad, atol=2e-2, rtol=1e-2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _cp_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        B, H, D, tc = 2, 2, 64, 256
        T = 2 * world * tc
        q, k, v, lf, do = [t.cuda() for t in _inputs(B, H, T, D, seed=3)]
        a, b = sharding.zigzag_chunks(world, rank)
        idx = torch.cat([torch.arange(a * tc, (a + 1) * tc), torch.arange(b * tc, (b + 1) * tc)]).cuda()
        results = {}
        # plain; left padding inside and beyond the first chunk; pruning with the "auto" threshold
        # (and the plain case cut into two head groups, each a complete step on its own CUDA stream)
        for name, seq, thr in (("plain", None, None), ("seq_start", torch.tensor([40, tc + 77]).cuda(), None),
                               ("auto", None, "auto"), ("head_groups", None, None)):
            qq, kk, vv, ll = [t.detach().clone().requires_grad_() for t in (q, k, v, lf)]
            full = fox.forgetting_attention(qq, kk, vv, ll, head_first=True, seq_start=seq, adaptive_threshold=thr)
            full.backward(do)
            ql, kl, vl, l_l = [t.index_select(2, idx).contiguous().requires_grad_() for t in (q, k, v, lf)]
            out = sharding.context_parallel_attention(ql, kl, vl, l_l, seq_start=seq, adaptive_threshold=thr,
                                                      head_groups=2 if name == "head_groups" else 1)
            out.backward(do.index_select(2, idx).contiguous())
            torch.cuda.synchronize()
            _lib.check_status()
            results[name] = [
                (out.float() - full.detach().index_select(2, idx).float()).abs().max().item(),
                (ql.grad.float() - qq.grad.index_select(2, idx).float()).abs().max().item(),
                (kl.grad.float() - kk.grad.index_select(2, idx).float()).abs().max().item(),
                (vl.grad.float() - vv.grad.index_select(2, idx).float()).abs().max().item(),
                (l_l.grad - ll.grad.index_select(2, idx)).abs().max().item() / max(1.0, ll.grad.abs().max().item()),
            ]
        ret[rank] = results
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_context_parallel_over_nccl_matches_single_gpu():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_cp_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert len(ret) == world
    for results in ret.values():
        for name, errs in results.items():
            # k/v/gate gradients are sums of bf16 partial gradients from two calls and two ranks: more roundings
            # than the single call makes
            assert errs[0] < 2e-2 and errs[1] < 3e-2 and errs[2] < 6e-2 and errs[3] < 6e-2 and errs[4] < 3e-2, (name, errs)


def _ce_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        g = torch.Generator().manual_seed(11)
        rows, classes = 300, 4096 * world
        logits = (torch.randn(rows, classes, generator=g) * 3).bfloat16().cuda()
        target = torch.randint(0, classes, (rows,), generator=g)
        target[::9] = -100
        target = target.cuda()
        dloss = torch.randn(rows, generator=g).cuda()
        n = classes // world
        worst = {}
        for eps, scale, zsq in ((0.0, 1.0, 0.0), (0.1, 0.5, 1e-4)):
            full = logits.clone().requires_grad_()
            l_full, z_full = fox.cross_entropy_loss(full, target, label_smoothing=eps, logit_scale=scale,
                                                    lse_square_scale=zsq)
            (l_full * dloss).sum().backward()
            mine = logits[:, rank * n:(rank + 1) * n].contiguous().requires_grad_()
            l_tp, z_tp = fox.cross_entropy_loss(mine, target, label_smoothing=eps, logit_scale=scale,
                                                lse_square_scale=zsq, process_group=dist.group.WORLD)
            (l_tp * dloss).sum().backward()
            torch.cuda.synchronize()
            worst[(eps, scale, zsq)] = [
                (l_tp - l_full).abs().max().item(), (z_tp - z_full).abs().max().item(),
                (mine.grad.float() - full.grad[:, rank * n:(rank + 1) * n].float()).abs().max().item()]
        ret[rank] = worst
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_cross_entropy_with_classes_split_over_two_gpus():
    """The fused loss with the classes split over two ranks (process_group) against the same kernels on all classes:
    losses, z-losses and this rank's slice of the logit gradient."""
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_ce_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert len(ret) == world
    for worst in ret.values():
        for key, (dl, dz, dg) in worst.items():
            # fp32 losses from the same bf16 logits; gradients are rounded to bf16 on both sides
            assert dl < 2e-4 and dz < 1e-5 and dg < 4e-3, (key, dl, dz, dg)
