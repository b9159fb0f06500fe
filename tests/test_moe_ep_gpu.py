"""GPU tests of the expert-parallel MoE: the EP building blocks on one GPU must reproduce
b200dnn_moe_layer bit for bit (per-row arithmetic does not depend on placement), and two ranks on
two GPUs (NCCL all-to-all dispatch / combine) must reproduce the one-GPU result bit for bit."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _make(torch, dev, T, H, I, E, S, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    experts = []
    for _ in range(E + S):
        experts.append(dict(w13=torch.randint(-127, 128, (H, 2 * I), dtype=torch.int8, generator=g),
                            s13=torch.rand(2 * I, generator=g) * 2e-3 + 2e-4,
                            w2=torch.randint(-127, 128, (I, H), dtype=torch.int8, generator=g),
                            s2=torch.rand(H, generator=g) * 2e-3 + 2e-4))
    return x, logits, experts


def _to(dev, e):
    return {k: v.to(dev) for k, v in e.items()}


def _single_gpu_layer(capi, torch, dev, x, logits, experts, E, S, topk, H, I):
    ex = (capi.MoeExpert * (E + S))()
    keep = [_to(dev, e) for e in experts]
    for i, e in enumerate(keep):
        ex[i].w13, ex[i].ldb13, ex[i].w13_scale = e["w13"].data_ptr(), 2 * I, e["s13"].data_ptr()
        ex[i].w2, ex[i].ldb2, ex[i].w2_scale = e["w2"].data_ptr(), H, e["s2"].data_ptr()
    xd, ld = x.to(dev), logits.to(dev)
    out = torch.empty(x.shape[0], H, dtype=torch.bfloat16, device=dev)
    capi.check(capi.lib.b200dnn_moe_layer(xd.data_ptr(), H, ld.data_ptr(), x.shape[0], E, S, topk, ex, H, I, H, 0,
                                          capi.ACT["silu_and_mul"], out.data_ptr(), H, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return out, keep


@pytest.mark.parametrize("T,H,I,E,S,topk", [(300, 256, 128, 8, 0, 2), (257, 128, 96, 6, 2, 3)])
def test_ep_blocks_equal_fused_layer_on_one_gpu(T, H, I, E, S, topk):
    import torch
    from zendnn_b200 import capi, moe_ep
    dev = torch.device("cuda:0")
    x, logits, experts = _make(torch, dev, T, H, I, E, S, 0)
    ref, keep = _single_gpu_layer(capi, torch, dev, x, logits, experts, E, S, topk, H, I)
    ops = moe_ep.CapiOps(keep[:E], keep[E:], H, I, H)
    got = moe_ep.ep_moe_forward(x.to(dev), logits.to(dev), topk, E, S, ops)
    torch.cuda.synchronize()
    assert float(ref.float().abs().sum()) > 1e-3
    assert torch.equal(got, ref)
    capi.lib.b200dnn_clear_caches()


def _ep_worker(rank, world, port, T, H, I, E, S, topk, ret):
    import torch
    import torch.distributed as dist
    from zendnn_b200 import capi, moe_ep
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    x, logits, experts = _make(torch, dev, T, H, I, E, S, 0)
    ref, keep = _single_gpu_layer(capi, torch, dev, x, logits, experts, E, S, topk, H, I)
    mine = [keep[e] for e in moe_ep.experts_on_rank(rank, world, E)]
    ops = moe_ep.CapiOps(mine, keep[E:], H, I, H)
    lo, hi = rank * T // world, (rank + 1) * T // world
    got = moe_ep.ep_moe_forward(x[lo:hi].to(dev), logits[lo:hi].to(dev), topk, E, S, ops)
    torch.cuda.synchronize()
    ret[rank] = bool(torch.equal(got, ref[lo:hi]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpus_equal_one_gpu():
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_ep_worker, args=(2, port, 512, 256, 128, 8, 0, 2, ret), nprocs=2, join=True)
    assert ret[0] and ret[1]
