"""Expert-parallel fused MoE over several GPUs (one process per GPU, torch.distributed / NCCL).

The reference (a single-process CPU library) has no multi-device path; this module is the one place
where the W8A8 hot path has a real exchange step.  Placement: expert e lives on rank e % world (its
local index is e // world); tokens are data-parallel, every rank routes its own tokens.  Per layer:

  route local tokens -> sort (token,k) slots by (destination rank, local expert) -> quantise the
  gathered rows to s8 + one f32 scale per row (1 byte per element crosses NVLink instead of 2) ->
  all-to-all dispatch (rows, scales; counts exchanged first) -> grouped expert GEMMs on the received
  rows, one group per (source rank, local expert) -> all-to-all combine of the bf16 expert outputs ->
  weighted top-k reduce on the owning rank.  Shared experts are replicated and see the rank's tokens.

Per-row arithmetic does not depend on where a row is computed, so the result equals the single-GPU
result bit for bit.

The device work goes through an `ops` object.  `CapiOps` binds libb200dnn (CUDA); tests drive the
same orchestration on CPU ranks (gloo) with a stand-in `ops` to check the exchange logic.
"""
import ctypes as C

import torch
import torch.distributed as dist


def expert_owner(e, world):
    return e % world


def local_expert_index(e, world):
    return e // world


def dispatch_keys(ids, world, num_experts):
    """Sort key of every (token,k) slot: destination rank major, local expert minor."""
    e_local = (num_experts + world - 1) // world
    return ((ids % world) * e_local + ids // world).to(torch.int32)


def experts_on_rank(rank, world, num_experts):
    return list(range(rank, num_experts, world))


class CapiOps:
    """Device operations of the EP layer through the C ABI (CUDA tensors in, CUDA tensors out)."""

    def __init__(self, experts_local, shared, K, I, H, act="silu_and_mul"):
        from . import capi
        self.capi = capi
        self.K, self.I, self.H = K, I, H
        self.act = capi.ACT[act]
        self.n_local = len(experts_local)
        self.all = list(experts_local) + list(shared)      # local routed experts first, then shared
        self.struct = (capi.MoeExpert * max(1, len(self.all)))()
        for i, e in enumerate(self.all):
            s = self.struct[i]
            s.w13, s.ldb13, s.w13_scale = e["w13"].data_ptr(), 2 * I, e["s13"].data_ptr()
            s.w2, s.ldb2, s.w2_scale = e["w2"].data_ptr(), H, e["s2"].data_ptr()

    def _st(self):
        return torch.cuda.current_stream().cuda_stream

    def route(self, logits, topk):
        T, E = logits.shape
        ids = torch.empty(T, topk, dtype=torch.int32, device=logits.device)
        w = torch.empty(T, topk, dtype=torch.float32, device=logits.device)
        self.capi.check(self.capi.lib.b200dnn_moe_route(logits.data_ptr(), T, E, topk, 1, ids.data_ptr(), w.data_ptr(),
                                                        None, None, self._st()))
        return ids, w

    def sort_slots(self, keys, nkeys):
        n = keys.numel()
        counts = torch.empty(nkeys, dtype=torch.int32, device=keys.device)
        s2r = torch.empty(n, dtype=torch.int32, device=keys.device)
        self.capi.check(self.capi.lib.b200dnn_moe_sort_slots(keys.data_ptr(), n, nkeys, counts.data_ptr(), s2r.data_ptr(), self._st()))
        return counts, s2r

    def quant_gather(self, x, row_src, div, R):
        K = x.shape[1]
        Kq = (K + 15) // 16 * 16
        q = torch.empty(R, Kq, dtype=torch.int8, device=x.device)
        s = torch.empty(R, dtype=torch.float32, device=x.device)
        if R:
            self.capi.check(self.capi.lib.b200dnn_quant_per_token_gather(
                x.data_ptr(), self.capi.DT["bf16"], K, x.stride(0), row_src.data_ptr(), div, R, q.data_ptr(), Kq,
                s.data_ptr(), self._st()))
        return q, s

    def experts(self, q, s, group_rows, group_expert):
        R = q.shape[0]
        out = torch.empty(R, self.H, dtype=torch.bfloat16, device=q.device)
        if R:
            n = len(group_rows)
            gr = (C.c_int32 * n)(*[int(v) for v in group_rows])
            ge = (C.c_int32 * n)(*[int(v) for v in group_expert])
            self.capi.check(self.capi.lib.b200dnn_moe_experts_s8(
                q.data_ptr(), q.stride(0), s.data_ptr(), n, gr, ge, self.struct, self.K, self.I, self.H, 0, self.act,
                out.data_ptr(), self.H, self._st()))
        return out

    def reduce_rows(self, rows, slot_rows, slot_w):
        T, ns = slot_rows.shape
        out = torch.empty(T, self.H, dtype=torch.bfloat16, device=rows.device)
        self.capi.check(self.capi.lib.b200dnn_moe_weighted_reduce_rows(
            rows.data_ptr(), rows.stride(0), slot_rows.data_ptr(), slot_w.data_ptr(), T, ns, self.H, self.capi.DT["bf16"],
            out.data_ptr(), self.H, self._st()))
        return out


def ep_moe_forward(x, logits, topk, num_experts, num_shared, ops, group=None, timing=None):
    """One expert-parallel MoE layer for this rank's tokens.  x [T,K] bf16, logits [T,E] f32.
    `ops.all` holds this rank's routed experts (in local order) followed by the shared experts."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    T = x.shape[0]
    e_local = (num_experts + world - 1) // world
    ids, w = ops.route(logits, topk)
    keys = dispatch_keys(ids.reshape(-1).to(torch.int64), world, num_experts)
    counts, slot_to_row = ops.sort_slots(keys, world * e_local)
    R = T * topk
    row_to_slot = torch.empty(R, dtype=torch.int32, device=x.device)
    row_to_slot[slot_to_row.long()] = torch.arange(R, dtype=torch.int32, device=x.device)
    q, s = ops.quant_gather(x, row_to_slot, topk, R)

    counts_h = counts.view(world, e_local)
    if world > 1:
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts, group=group)          # [src rank][my local expert]
        send_split = counts_h.sum(1).tolist()
        recv_counts_h = recv_counts.view(world, e_local).cpu()
        recv_split = recv_counts_h.sum(1).tolist()
        R_recv = int(sum(recv_split))
        q_recv = torch.empty(R_recv, q.shape[1], dtype=q.dtype, device=q.device)
        s_recv = torch.empty(R_recv, dtype=s.dtype, device=s.device)
        dist.all_to_all_single(q_recv, q, recv_split, send_split, group=group)
        dist.all_to_all_single(s_recv, s, recv_split, send_split, group=group)
        group_rows = recv_counts_h.reshape(-1).tolist()
    else:
        q_recv, s_recv = q, s
        group_rows = counts.cpu().tolist()
        send_split = recv_split = None
    group_expert = [j for _ in range(world) for j in range(e_local)]
    # local experts that do not exist on this rank (num_experts not divisible by world) get no rows by construction
    n_local = getattr(ops, "n_local", e_local)
    group_expert = [min(j, max(n_local - 1, 0)) for j in group_expert]
    o_recv = ops.experts(q_recv, s_recv, group_rows, group_expert)

    if world > 1:
        o_back = torch.empty(R, o_recv.shape[1], dtype=o_recv.dtype, device=o_recv.device)
        dist.all_to_all_single(o_back, o_recv, send_split, recv_split, group=group)
    else:
        o_back = o_recv

    slot_rows = slot_to_row.view(T, topk)
    slot_w = w
    if num_shared:
        ident = torch.arange(T, dtype=torch.int32, device=x.device)
        qs, ss = ops.quant_gather(x, ident, 1, T)
        outs = [o_back]
        extra_rows = []
        for j in range(num_shared):
            outs.append(ops.experts(qs, ss, [T], [n_local + j]))
            extra_rows.append((R + j * T + ident).view(T, 1))
        o_back = torch.cat(outs, 0)
        slot_rows = torch.cat([slot_rows] + extra_rows, 1).contiguous()
        slot_w = torch.cat([w, torch.ones(T, num_shared, dtype=w.dtype, device=w.device)], 1).contiguous()
    return ops.reduce_rows(o_back, slot_rows.contiguous(), slot_w.contiguous())
