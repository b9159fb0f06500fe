"""Host logic of the expert-parallel MoE (zendnn_b200/moe_ep.py) on CPU ranks: two gloo processes run
the real orchestration (keys, stable sort, count exchange, all-to-all dispatch and combine, weighted
reduce) with a stand-in for the device kernels, and must reproduce a one-process run exactly.
A rank that never joins is covered too: the others see a process-group timeout, not a hang."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from zendnn_b200 import moe_ep


class CpuOps:
    """Stand-in for the CUDA kernels with the same interface; experts are cheap deterministic maps."""

    def __init__(self, expert_ids, shared_ids, H):
        self.ids = list(expert_ids) + list(shared_ids)
        self.n_local = len(expert_ids)
        self.H = H

    def route(self, logits, topk):
        p = torch.softmax(logits, dim=1)
        w, ids = torch.topk(p, topk, dim=1)
        return ids.to(torch.int32), (w / w.sum(1, keepdim=True)).float()

    def sort_slots(self, keys, nkeys):
        order = torch.argsort(keys.long(), stable=True)
        s2r = torch.empty_like(keys)
        s2r[order] = torch.arange(keys.numel(), dtype=keys.dtype)
        return torch.bincount(keys.long(), minlength=nkeys).to(torch.int32), s2r

    def quant_scatter(self, x, dst_rows, n_rows):
        rows = x.float()
        sc = rows.abs().amax(1).clamp_min(1e-10) / 127.0
        qv = torch.round(rows / sc[:, None]).to(torch.int8)
        q = torch.zeros(n_rows, x.shape[1], dtype=torch.int8)
        s = torch.zeros(n_rows)
        for j in range(dst_rows.shape[1]):
            q[dst_rows[:, j].long()] = qv
            s[dst_rows[:, j].long()] = sc
        return q, s

    def experts(self, q, s, group_rows, group_expert, out):
        r = 0
        for n, j in zip(group_rows, group_expert):
            if n:
                gid = self.ids[j]
                out[r:r + n] = (q[r:r + n].float() * s[r:r + n, None])[:, : self.H] * (gid + 1) + gid
            r += n

    def new_rows(self, n_rows, like):
        return torch.zeros(n_rows, self.H)

    def reduce_rows(self, rows, slot_rows, slot_w):
        return (rows[slot_rows.long()] * slot_w[:, :, None]).sum(1)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(T, K, E, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(T, K, generator=g), torch.randn(T, E, generator=g)


def _worker(rank, world, port, T, K, H, E, S, topk, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    x, logits = _inputs(T, K, E, 0)
    lo, hi = rank * T // world, (rank + 1) * T // world
    ops = CpuOps(moe_ep.experts_on_rank(rank, world, E), range(E, E + S), H)
    out = moe_ep.ep_moe_forward(x[lo:hi], logits[lo:hi], topk, E, S, ops)
    ret[rank] = out
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("E,S,topk", [(8, 0, 2), (6, 2, 3)])
def test_two_ranks_equal_one_process(E, S, topk):
    T, K, H, world = 64, 32, 32, 2
    ref_ops = CpuOps(range(E), range(E, E + S), H)
    x, logits = _inputs(T, K, E, 0)
    ref = moe_ep.ep_moe_forward(x, logits, topk, E, S, ref_ops)
    assert ref.abs().sum() > 1e-3
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), T, K, H, E, S, topk, ret), nprocs=world, join=True)
    got = torch.cat([ret[r] for r in range(world)], 0)
    assert torch.equal(got, ref)


def test_placement_helpers():
    assert moe_ep.experts_on_rank(1, 4, 10) == [1, 5, 9]
    ids = torch.tensor([0, 1, 2, 3, 4, 5, 6, 7])
    keys = moe_ep.dispatch_keys(ids, 4, 8)
    # destination rank major (e % 4), local index minor (e // 4)
    assert keys.tolist() == [0, 2, 4, 6, 1, 3, 5, 7]
    assert all(moe_ep.expert_owner(e, 4) == e % 4 and moe_ep.local_expert_index(e, 4) == e // 4 for e in range(8))


def test_planned_placement_balances_a_skewed_histogram():
    """Zipf-like loads: the planned map keeps the busiest rank near the mean, the modulo map does not; every rank gets at
    most ceil(E / world) experts; the map is a pure function of the histogram."""
    E, world = 64, 8
    hist = [int(100000 / (r + 1) ** 1.1) for r in range(E)]
    g = torch.Generator().manual_seed(5)
    perm = torch.randperm(E, generator=g).tolist()
    hist = [hist[perm[e]] for e in range(E)]
    owner = moe_ep.plan_expert_placement(hist, world)
    assert owner == moe_ep.plan_expert_placement(list(hist), world)
    load = [sum(h for h, o in zip(hist, owner) if o == r) for r in range(world)]
    naive = [sum(h for e, h in enumerate(hist) if e % world == r) for r in range(world)]
    mean = sum(hist) / world
    assert max(load) <= 1.1 * max(max(hist), mean)       # the busiest expert alone is a lower bound for any map
    assert max(naive) > 1.1 * max(load)
    assert max(owner.count(r) for r in range(world)) <= 8 and sorted(set(owner)) == list(range(world))
    assert moe_ep.modulo_placement(5, 2) == [0, 1, 0, 1, 0]


def _plan_worker(rank, world, port, E, topk, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    # every rank sees only its own tokens; the histogram is summed over the ranks before planning
    _, logits = _inputs(256, 8, E, 100 + rank)
    ids = torch.topk(logits, topk, dim=1).indices.reshape(-1)
    hist = torch.bincount(ids, minlength=E)
    dist.all_reduce(hist)
    ret[rank] = moe_ep.plan_expert_placement(hist.tolist(), world)
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_plan_the_same_placement():
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_plan_worker, args=(2, _free_port(), 12, 3, ret), nprocs=2, join=True)
    assert ret[0] == ret[1] and sorted(set(ret[0])) == [0, 1]


def _absent_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    if rank == 1:
        ret[rank] = "absent"          # this rank never joins the exchange
        return
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
        t = torch.zeros(4)
        dist.all_reduce(t)
        ret[rank] = "no error"
    except Exception as e:                      # rendezvous or collective timeout: reported, not hung
        ret[rank] = "error: " + type(e).__name__


def test_missing_rank_is_reported_not_hung():
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_absent_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert ret[1] == "absent" and ret[0].startswith("error")
