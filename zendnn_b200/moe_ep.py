"""Expert-parallel fused MoE over several GPUs (one process per GPU, torch.distributed / NCCL).

The reference (a single-process CPU library) has no multi-device path; this module is the one place
where the W8A8 hot path has a real exchange step.  Placement: expert e lives on rank e % world (its
local index is e // world); tokens are data-parallel, every rank routes its own tokens.  Per layer:

  route local tokens -> sort (token,k) slots by (destination rank, local expert) -> quantise every
  token once to s8 + one f32 scale and write it to the send rows of all its slots (1 byte per element
  crosses NVLink instead of 2) and, for the replicated shared experts, to their local rows ->
  all-to-all dispatch (rows, scales; counts exchanged first) -> ONE grouped expert computation over the
  received rows (one group per (source rank, local expert)) and the shared experts' rows -> all-to-all
  combine of the bf16 expert outputs -> weighted reduce on the owning rank.
  One buffer holds [received rows | shared-expert rows | send rows] (the same layout for the outputs), so
  the exchanges and the reduce work on views of it and nothing is concatenated or copied.

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
    ids = ids.to(torch.int32)                      # no-op for the router's int32 ids
    if world == 1:
        return ids
    return (ids % world) * e_local + torch.div(ids, world, rounding_mode="floor")


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

    def quant_scatter(self, x, dst_rows, n_rows):
        """Quantise every row of x once and write it to the rows dst_rows[t, :] of a [n_rows, Kq] buffer."""
        T, K = x.shape
        Kq = (K + 15) // 16 * 16
        q = torch.empty(n_rows, Kq, dtype=torch.int8, device=x.device)
        s = torch.empty(n_rows, dtype=torch.float32, device=x.device)
        self.capi.check(self.capi.lib.b200dnn_quant_per_token_scatter(
            x.data_ptr(), self.capi.DT["bf16"], K, x.stride(0), dst_rows.data_ptr(), dst_rows.shape[1], T, q.data_ptr(), Kq,
            s.data_ptr(), self._st()))
        return q, s

    def experts(self, q, s, group_rows, group_expert, out):
        """Grouped expert computation on the rows q/s (consecutive groups); results into out[:rows]."""
        R = q.shape[0]
        if R and sum(int(v) for v in group_rows):
            n = len(group_rows)
            gr = (C.c_int32 * n)(*[int(v) for v in group_rows])
            ge = (C.c_int32 * n)(*[int(v) for v in group_expert])
            self.capi.check(self.capi.lib.b200dnn_moe_experts_s8(
                q.data_ptr(), q.stride(0), s.data_ptr(), n, gr, ge, self.struct, self.K, self.I, self.H, 0, self.act,
                out.data_ptr(), out.stride(0), self._st()))

    def new_rows(self, n_rows, like):
        return torch.empty(n_rows, self.H, dtype=torch.bfloat16, device=like.device)

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

    def mark(name):
        # timing: a list that receives (phase name, CUDA event) pairs, for per-phase device times
        if timing is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            timing.append((name, ev))
    mark("start")
    T = x.shape[0]
    S = num_shared
    e_local = (num_experts + world - 1) // world
    ids, w = ops.route(logits, topk)
    keys = dispatch_keys(ids.reshape(-1), world, num_experts)
    counts, slot_to_row = ops.sort_slots(keys, world * e_local)
    R = T * topk
    mark("route+sort")

    if world > 1:
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts, group=group)          # [src rank][my local expert]
        both = torch.stack([counts.view(world, e_local), recv_counts.view(world, e_local)]).cpu()
        send_split = both[0].sum(1).tolist()
        recv_split = both[1].sum(1).tolist()
        group_rows = both[1].reshape(-1).tolist()
        R_recv = int(sum(recv_split))
        base_send = R_recv + S * T                                         # rows: [received | shared | send]
    else:
        group_rows = counts.cpu().tolist()
        R_recv, base_send = R, 0                                           # rows: [routed | shared]
    mark("counts exchange")
    base_shared = R_recv
    n_rows = base_shared + S * T + (R if world > 1 else 0)

    # where every token's quantised row goes: its topk routed slots, then one row per shared expert
    tok = torch.arange(T, dtype=torch.int32, device=x.device)
    cols = [slot_to_row.view(T, topk) + base_send] + [(base_shared + j * T + tok).view(T, 1) for j in range(S)]
    slot_rows = torch.cat(cols, 1).contiguous()
    slot_w = w if S == 0 else torch.cat([w, torch.ones(T, S, dtype=w.dtype, device=w.device)], 1).contiguous()
    q, s = ops.quant_scatter(x, slot_rows, n_rows)
    mark("quantise+scatter")

    if world > 1:
        dist.all_to_all_single(q[:R_recv], q[base_send:], recv_split, send_split, group=group)
        dist.all_to_all_single(s[:R_recv], s[base_send:], recv_split, send_split, group=group)

    mark("dispatch all-to-all")
    # one grouped computation: (source rank, local expert) groups over the received rows, then the shared experts
    n_local = getattr(ops, "n_local", e_local)
    # local experts that do not exist on this rank (num_experts not divisible by world) get no rows by construction
    group_expert = [min(j, max(n_local - 1, 0)) for _ in range(world) for j in range(e_local)]
    group_rows = list(group_rows) + [T] * S
    group_expert = group_expert + [n_local + j for j in range(S)]
    n_in = base_shared + S * T
    o = ops.new_rows(n_rows, x)
    ops.experts(q[:n_in], s[:n_in], group_rows, group_expert, o)
    mark("experts")

    if world > 1:
        dist.all_to_all_single(o[base_send:], o[:R_recv], send_split, recv_split, group=group)
    mark("combine all-to-all")
    y = ops.reduce_rows(o, slot_rows, slot_w)
    mark("reduce")
    return y
