"""GPU tests of the expert-parallel MoE.  Per-row arithmetic does not depend on placement, so every form must
reproduce b200dnn_moe_layer bit for bit:
  - the library's expert-parallel layer with 1, 2, 4 and 8 ranks inside one process on one GPU (peer buffers are plain
    device pointers there): uneven token counts, a rank without tokens, expert counts that do not divide by the world
    size, shared experts, a load-aware placement map;
  - the same layer as one process per GPU over NCCL and CUDA IPC, at every world size the machine offers (2, 4, 8);
  - the building blocks under the torch.distributed all-to-all orchestration, on one GPU and on two."""
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


def _split(T, world, uneven):
    """Token ranges per rank: equal shares, or uneven ones with an empty rank in the middle."""
    if not uneven or world == 1:
        return [(r * T // world, (r + 1) * T // world) for r in range(world)]
    cuts = [0]
    for r in range(world):
        share = 0 if r == 1 else (2 if r % 2 == 0 else 1)
        cuts.append(cuts[-1] + share)
    return [(cuts[r] * T // cuts[-1], cuts[r + 1] * T // cuts[-1]) for r in range(world)]


def _placement(moe_ep, torch, logits, topk, E, world, planned):
    if not planned:
        return moe_ep.modulo_placement(E, world)
    ids = torch.topk(logits, topk, dim=1).indices.reshape(-1)
    return moe_ep.plan_expert_placement(torch.bincount(ids, minlength=E).tolist(), world)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("T,H,I,E,S,topk,uneven,planned", [(384, 256, 128, 8, 0, 2, False, False),
                                                           (300, 128, 96, 6, 2, 3, True, False),
                                                           (520, 256, 160, 20, 1, 4, True, True)])
def test_ep_layer_ranks_in_one_process_equal_fused_layer(world, T, H, I, E, S, topk, uneven, planned):
    """b200dnn_moe_layer_ep_local: all ranks' phases on one stream of one GPU."""
    import ctypes as C
    import torch
    from zendnn_b200 import capi, moe_ep
    dev = torch.device("cuda:0")
    st = torch.cuda.current_stream().cuda_stream
    x, logits, experts = _make(torch, dev, T, H, I, E, S, world)
    ref, keep = _single_gpu_layer(capi, torch, dev, x, logits, experts, E, S, topk, H, I)
    assert float(ref.float().abs().sum()) > 1e-3
    owner = _placement(moe_ep, torch, logits, topk, E, world, planned)
    parts = _split(T, world, uneven)
    layers = []
    for r in range(world):
        mine = [keep[e] for e in range(E) if owner[e] == r] + keep[E:]
        layers.append(moe_ep.EpLayer(r, world, E, S, topk, max(hi - lo for lo, hi in parts), H, I, H, mine, expert_rank=owner))
    handles = (C.c_void_p * world)(*[l.handle for l in layers])
    capi.check(capi.lib.b200dnn_ep_connect_local(handles, world))
    xs = [x[lo:hi].to(dev).contiguous() for lo, hi in parts]
    ls = [logits[lo:hi].to(dev).contiguous() for lo, hi in parts]
    outs = [torch.zeros(hi - lo, H, dtype=torch.bfloat16, device=dev) for lo, hi in parts]
    arr = lambda ts: (C.c_void_p * world)(*[t.data_ptr() for t in ts])
    Ts = (C.c_int32 * world)(*[hi - lo for lo, hi in parts])
    for _ in range(2):          # twice: the second call reuses every buffer
        capi.check(capi.lib.b200dnn_moe_layer_ep_local(handles, world, arr(xs), H, arr(ls), Ts, arr(outs), H, st))
        torch.cuda.synchronize()
        for r, (lo, hi) in enumerate(parts):
            assert torch.equal(outs[r], ref[lo:hi]), "rank %d of %d differs" % (r, world)
            assert layers[r].status() == capi.SUCCESS, capi.last_error()
        for o in outs:
            o.zero_()
    rows = layers[0].rows_per_rank()
    assert sum(rows) == T * (topk + S)
    for l in layers:
        l.close()
    capi.lib.b200dnn_clear_caches()


def test_ep_layer_reports_an_overflowing_receive_buffer():
    """capacity_rows below what the routing sends: the rows are dropped inside bounds and the status call says so."""
    import ctypes as C
    import torch
    from zendnn_b200 import capi, moe_ep
    dev = torch.device("cuda:0")
    T, H, I, E, S, topk, world = 256, 128, 96, 4, 0, 2, 2
    x, logits, experts = _make(torch, dev, T, H, I, E, S, 3)
    keep = [_to(dev, e) for e in experts]
    layers = [moe_ep.EpLayer(r, world, E, S, topk, T // world, H, I, H, [keep[e] for e in range(E) if e % world == r],
                             capacity_rows=8) for r in range(world)]
    handles = (C.c_void_p * world)(*[l.handle for l in layers])
    capi.check(capi.lib.b200dnn_ep_connect_local(handles, world))
    xs = [x[r * T // world:(r + 1) * T // world].to(dev).contiguous() for r in range(world)]
    ls = [logits[r * T // world:(r + 1) * T // world].to(dev).contiguous() for r in range(world)]
    outs = [torch.zeros(T // world, H, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    arr = lambda ts: (C.c_void_p * world)(*[t.data_ptr() for t in ts])
    Ts = (C.c_int32 * world)(*[T // world] * world)
    capi.check(capi.lib.b200dnn_moe_layer_ep_local(handles, world, arr(xs), H, arr(ls), Ts, arr(outs), H,
                                                   torch.cuda.current_stream().cuda_stream))
    assert layers[0].status() == capi.FAILURE
    for l in layers:
        l.close()
    capi.lib.b200dnn_clear_caches()


def _ep_layer_worker(rank, world, port, T, H, I, E, S, topk, planned, ret):
    import torch
    import torch.distributed as dist
    from zendnn_b200 import capi, moe_ep
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x, logits, experts = _make(torch, dev, T, H, I, E, S, 0)
    ref, keep = _single_gpu_layer(capi, torch, dev, x, logits, experts, E, S, topk, H, I)
    owner = _placement(moe_ep, torch, logits, topk, E, world, planned)
    parts = _split(T, world, True)
    lo, hi = parts[rank]
    mine = [keep[e] for e in range(E) if owner[e] == rank] + keep[E:]
    layer = moe_ep.EpLayer(rank, world, E, S, topk, max(b - a for a, b in parts), H, I, H, mine, expert_rank=owner)
    layer.connect()
    ok = True
    for _ in range(3):
        got = layer.forward(x[lo:hi].to(dev).contiguous(), logits[lo:hi].to(dev).contiguous())
        torch.cuda.synchronize()
        ok = ok and bool(torch.equal(got, ref[lo:hi])) and layer.status() == capi.SUCCESS
    ret[rank] = ok
    dist.barrier()
    layer.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("E,S,topk,planned", [(8, 0, 2, False), (20, 2, 4, True)])
def test_ep_layer_one_process_per_gpu_equals_one_gpu(world, E, S, topk, planned):
    """b200dnn_moe_layer_ep over NCCL + CUDA IPC at every world size the machine offers."""
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_ep_layer_worker, args=(world, port, 1000, 256, 128, E, S, topk, planned, ret), nprocs=world, join=True)
    assert all(ret[r] for r in range(world)), dict(ret)


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
