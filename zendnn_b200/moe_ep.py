"""Expert-parallel fused MoE over several GPUs (one process per GPU).

Two layers live here.

`EpLayer` is the product path: a thin binding of the library's own expert-parallel entry point
(b200dnn_moe_layer_ep, include/b200dnn.h).  The whole layer runs inside the library on the caller's stream: tokens are
quantised once and stored straight into the receive buffers of the GPUs that own their experts (peer memory over
NVLink), the grouped GEMMs read only local memory, and the weighted reduce loads the output rows back from the owners.
NCCL carries the per-expert row counts and two barriers; torch.distributed is used once, to hand the communicator id
to the other ranks.  `plan_expert_placement` chooses which rank owns which expert from a histogram of routed rows.

`ep_moe_forward` below is the same exchange written over torch.distributed all-to-all calls with a pluggable `ops`
object.  It serves machines whose GPUs cannot map each other's memory and the CPU tests of the exchange logic
(gloo ranks with a stand-in `ops`).

The reference (a single-process CPU library) has no multi-device path.  Placement in `ep_moe_forward`: expert e lives
on rank e % world (local index e // world); every rank routes its own tokens, sorts the (token,k) slots by
(destination rank, local expert), quantises every token once into the send rows of all its slots, exchanges counts,
rows and scales with all-to-all calls, runs one grouped expert computation over (source rank, local expert) groups
and the shared experts' rows, returns the bf16 outputs with a second all-to-all and reduces on the owning rank.
Per-row arithmetic does not depend on where a row is computed, so both layers equal the single-GPU result bit for bit.
"""
import ctypes as C

import torch
import torch.distributed as dist


def plan_expert_placement(rows_per_expert, world, experts_per_rank=None):
    """Owner rank of every routed expert, balancing the rows each rank computes.

    rows_per_expert: how many (token,k) slots each expert received on a calibration batch (all ranks together).
    Longest-processing-time greedy: experts in descending load, each to the rank with the fewest rows so far among
    the ranks that still have room (experts_per_rank, default ceil(E / world), bounds the weights a rank holds).
    Ties go to the lower rank and the lower expert id, so every rank computes the same map from the same histogram.
    Returns a list of length E."""
    E = len(rows_per_expert)
    cap = experts_per_rank if experts_per_rank else (E + world - 1) // world
    assert cap * world >= E, "not enough room for %d experts on %d ranks" % (E, world)
    order = sorted(range(E), key=lambda e: (-int(rows_per_expert[e]), e))
    load, count, owner = [0] * world, [0] * world, [0] * E
    for e in order:
        r = min((r for r in range(world) if count[r] < cap), key=lambda r: (load[r], r))
        owner[e] = r
        load[r] += int(rows_per_expert[e])
        count[r] += 1
    return owner


def modulo_placement(num_experts, world):
    return [e % world for e in range(num_experts)]


class EpLayer:
    """One rank of the library's expert-parallel MoE layer (b200dnn_moe_layer_ep).

    experts: this rank's routed experts in ascending expert id, then the shared experts; each a dict with CUDA
    tensors w13 [K,2I] s8, s13 [2I] f32, w2 [I,H] s8, s2 [H] f32.  expert_rank: owner of every routed expert
    (default e % world).  With world > 1, `connect()` must be called by all ranks (it uses torch.distributed, any
    backend, only to broadcast the communicator id)."""

    def __init__(self, rank, world, num_experts, num_shared, topk, max_tokens, K, I, H, experts, expert_rank=None,
                 act="silu_and_mul", capacity_rows=0):
        from . import capi
        self.capi, self.rank, self.world = capi, rank, world
        self.K, self.I, self.H, self.E = K, I, H, num_experts
        cfg = capi.EpConfig()
        cfg.world, cfg.rank, cfg.num_experts, cfg.num_shared, cfg.topk = world, rank, num_experts, num_shared, topk
        cfg.max_tokens, cfg.K, cfg.I, cfg.H, cfg.transB, cfg.act = max_tokens, K, I, H, 0, capi.ACT[act]
        cfg.capacity_rows = capacity_rows
        self._map = None
        if expert_rank is not None:
            self._map = (C.c_int32 * num_experts)(*[int(r) for r in expert_rank])
            cfg.expert_rank = C.cast(self._map, C.c_void_p)
        self.handle = C.c_void_p()
        capi.check(capi.lib.b200dnn_ep_create(C.byref(cfg), C.byref(self.handle)))
        self.experts = list(experts)
        self.struct = (capi.MoeExpert * max(1, len(self.experts)))()
        for i, e in enumerate(self.experts):
            s = self.struct[i]
            s.w13, s.ldb13, s.w13_scale = e["w13"].data_ptr(), 2 * I, e["s13"].data_ptr()
            s.w2, s.ldb2, s.w2_scale = e["w2"].data_ptr(), H, e["s2"].data_ptr()
        capi.check(capi.lib.b200dnn_ep_set_experts(self.handle, self.struct, len(self.experts)))

    def connect(self, group=None):
        if self.world == 1:
            return
        ident = (C.c_uint8 * 128)()
        if self.rank == 0:
            self.capi.check(self.capi.lib.b200dnn_ep_nccl_unique_id(ident))
        box = [bytes(ident)]
        dist.broadcast_object_list(box, src=0, group=group)
        ident = (C.c_uint8 * 128).from_buffer_copy(box[0])
        self.capi.check(self.capi.lib.b200dnn_ep_connect_nccl(self.handle, ident, None))

    def forward(self, x, logits, out=None, stream=None):
        T = x.shape[0]
        if out is None:
            out = torch.empty(T, self.H, dtype=torch.bfloat16, device=x.device)
        st = stream if stream is not None else (torch.cuda.current_stream().cuda_stream if x.is_cuda else None)
        self.capi.check(self.capi.lib.b200dnn_moe_layer_ep(self.handle, x.data_ptr(), x.stride(0) if T else self.K,
                                                           logits.data_ptr(), T, out.data_ptr(), out.stride(0) if T else self.H, st))
        return out

    def rows_per_rank(self):
        rows = (C.c_int32 * self.world)()
        self.capi.check(self.capi.lib.b200dnn_ep_rows_per_rank(self.handle, rows, torch.cuda.current_stream().cuda_stream))
        return list(rows)

    def status(self):
        return self.capi.lib.b200dnn_ep_status(self.handle, torch.cuda.current_stream().cuda_stream)

    def close(self):
        if self.handle:
            self.capi.lib.b200dnn_ep_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


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
