#!/usr/bin/env python
"""Benchmark of the B200-native LowOHA W8A8 hot path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload decode|prefill|c1|moe] [--impl ours|reference]

Headline workload (default): the decode-shape W8A8 matmul_direct grid, M in {1,4,16} x
(K,N) in {(4096,4096),(4096,11008),(11008,4096)}, per-token s8 activations x per-channel s8
prepacked weights, bf16 output.  One step = every (M,K,N) combination once per rotating weight
copy; the copies of one shape total more than the 126 MB L2 so every launch streams its weights
from HBM.  Metric: algorithmic bytes (K*N + M*K + 4M + 4N + 2MN per GEMM) per second.

Prints ONE JSON line (rank 0).  `value` is measured with inputs resident in HBM (CUDA events on the
launching stream); `e2e` goes through the same C ABI with pinned HOST buffers, so every call carries
its host->device and device->host copies.  Multi-GPU: the decode path has no exchange step, each
rank runs an independent replica ("weak").  `--impl reference` times the CPU implementation of the
same path on the host cores (the oracle port; the reference's own default backend, AOCL-DLP, is not
part of the reference tree).
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

DECODE_MS = (1, 4, 16)
DECODE_KN = ((4096, 4096), (4096, 11008), (11008, 4096))


def decode_bytes(M, K, N):
    return K * N + M * K + 4 * M + 4 * N + 2 * M * N


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm=d.get("hbm_gbs", 6650.0), bf16=d.get("bf16_tflops", 1590.0), src="measured")
    return dict(hbm=6650.0, bf16=1590.0, src="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.idx = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        sm = sorted(int(float(r[1])) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit())
        mx = [int(float(r[2])) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) >= 9:
                for n, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        return dict(sm_mhz=sm[len(sm) // 2] if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


# ---------------------------------------------------------------------------------------------- inputs
def make_decode_inputs(rng, copies_bytes=140e6):
    """Quantised operands of every decode combination; `copies` distinct weights per shape."""
    from oracle import oracle as O  # only to quantise the synthetic inputs on the host (not timed)
    shapes = {}
    for K, N in DECODE_KN:
        copies = max(2, int(np.ceil(copies_bytes / (K * N))))
        ws, ss = [], []
        # weights ~ N(0, 0.02) quantised per channel (|q| = 127 at the column max).  One matrix is
        # drawn per shape; the other copies are row rotations of it (same distribution, distinct
        # buffers) to keep set-up time short.
        w = rng.standard_normal(size=(K, N), dtype=np.float32)
        amax = np.abs(w).max(axis=0)
        q0 = np.rint(w / (amax / 127.0)).astype(np.int8)
        s0 = (amax * 0.02 / 127.0).astype(np.float32)
        del w
        for i in range(copies):
            ws.append(np.ascontiguousarray(np.roll(q0, 17 * i, axis=0)))
            ss.append(s0)
        acts = {}
        for M in DECODE_MS:
            x = O.f32_to_bf16(rng.normal(size=(M, K)).astype(np.float32))
            qa, sa = O.quant_per_token(x)
            acts[M] = (qa, sa)
        shapes[(K, N)] = dict(w=ws, s=ss, acts=acts)
    return shapes


# ---------------------------------------------------------------------------------------------- ours
def run_ours(args, rank, world, local_rank):
    import torch
    from zendnn_b200 import capi
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    assert capi.lib.b200dnn_device_count() > 0
    rng = np.random.default_rng(1234 + rank)
    shapes = make_decode_inputs(rng)
    stream = torch.cuda.current_stream().cuda_stream

    # device-resident operands + prepacked weights
    calls = []      # (desc, bytes)
    keep = []
    for (K, N), sh in shapes.items():
        packed = []
        for q, s in zip(sh["w"], sh["s"]):
            size = capi.lib.b200dnn_prepack_size(K, N, 0)
            buf = torch.empty(size, dtype=torch.uint8, device=dev)
            qd = torch.from_numpy(q).to(dev)
            capi.check(capi.lib.b200dnn_prepack(qd.data_ptr(), K, N, N, 0, 0, buf.data_ptr(), stream))
            torch.cuda.synchronize()
            del qd
            packed.append((buf, torch.from_numpy(s).to(dev)))
        keep.append(packed)
        for M in DECODE_MS:
            qa, sa = sh["acts"][M]
            A, SA = torch.from_numpy(qa).to(dev), torch.from_numpy(sa).to(dev)
            out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            keep.append((A, SA, out))
            for buf, sw in packed:
                d = capi.make_matmul(M, N, K, A, buf, out, src_dt=capi.DT["s8"], dst_dt=capi.DT["bf16"], wei_format="r",
                                     src_scale=SA, wei_scale=sw, flags=capi.FLAG_STABLE_WEIGHTS)
                calls.append((d, decode_bytes(M, K, N)))
    step_bytes = sum(b for _, b in calls)

    def one_pass(stream_handle):
        for d, _ in calls:
            st = capi.matmul(d, stream_handle)
            if st != capi.SUCCESS:
                raise RuntimeError(capi.last_error())

    # One pass = every (M,K,N,weight copy) GEMM once.  The pass is captured in a CUDA graph (the calls
    # take device pointers, so the library only enqueues kernels) and a step replays it `inner` times:
    # this keeps host launch cost out of a loop of 10-microsecond kernels.
    inner = args.inner
    one_pass(stream)
    torch.cuda.synchronize()
    if world > 1:
        # the process group is created after the operands: the replicas exchange nothing, the group only
        # serves the barrier and the max over ranks
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    # one pass per graph by default; the host needs about 2.5 us to launch it (host_enqueue_ms_per_step in the output)
    per_graph = max(1, min(inner, args.passes_per_graph))
    while inner % per_graph:
        per_graph -= 1
    with torch.cuda.graph(graph, stream=side):
        for _ in range(per_graph):
            one_pass(torch.cuda.current_stream().cuda_stream)

    def step():
        for _ in range(inner // per_graph):
            graph.replay()

    step_bytes *= inner
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    t_host = time.perf_counter()
    for _ in range(args.steps):
        step()
    host_ms = (time.perf_counter() - t_host) * 1e3        # time the host needed to enqueue the timed region
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    launches = args.steps * inner * len(calls)     # one streaming-GEMM kernel per call in the graph
    clocks = sampler.stop()
    if world > 1:
        import torch.distributed as dist
        every = [torch.zeros(1, device=dev) for _ in range(world)]
        dist.all_gather(every, torch.tensor([ms], device=dev))
        ms_per_rank = [round(float(v.item()) / args.steps, 4) for v in every]
        ms = max(float(v.item()) for v in every)
    else:
        ms_per_rank = [round(ms / args.steps, 4)]

    # per-combination timing (device resident), for the breakdown
    per = {}
    for (K, N), sh in shapes.items():
        for M in DECODE_MS:
            sel = [(d, b) for d, b in calls if d.M == M and d.K == K and d.N == N]
            torch.cuda.synchronize()
            a, bt = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 20
            g2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g2, stream=side):
                for d, _ in sel:
                    capi.matmul(d, torch.cuda.current_stream().cuda_stream)
            g2.replay()
            torch.cuda.synchronize()
            a.record()
            for _ in range(reps):
                g2.replay()
            bt.record()
            torch.cuda.synchronize()
            t_ms = a.elapsed_time(bt) / (reps * len(sel))
            per["M%d_K%d_N%d" % (M, K, N)] = dict(us=round(t_ms * 1e3, 2), gbs=round(sel[0][1] / t_ms / 1e6, 1))

    # end-to-end through the C ABI with pinned host buffers (activations in, result out, every call)
    e2e_calls, h2d, d2h = [], 0, 0
    for (K, N), sh in shapes.items():
        for M in DECODE_MS:
            qa, sa = sh["acts"][M]
            A = torch.from_numpy(qa).pin_memory(); SA = torch.from_numpy(sa).pin_memory()
            out = torch.empty(M, N, dtype=torch.bfloat16).pin_memory()
            keep.append((A, SA, out))
            for buf, sw in keep[DECODE_KN.index((K, N)) * 4]:
                d = capi.make_matmul(M, N, K, A, buf, out, src_dt=capi.DT["s8"], dst_dt=capi.DT["bf16"], wei_format="r",
                                     src_scale=SA, wei_scale=sw, flags=capi.FLAG_STABLE_WEIGHTS)
                e2e_calls.append(d)
                h2d += M * K + 4 * M
                d2h += 2 * M * N
    for d in e2e_calls:
        capi.check(capi.matmul(d, stream))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e2e_passes = 5
    for _ in range(e2e_passes):
        for d in e2e_calls:
            capi.matmul(d, stream)
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / e2e_passes * inner      # scaled to one step (= inner passes)
    h2d *= inner
    d2h *= inner
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())

    peaks = measured_peaks()
    ms_per_step = ms / args.steps
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9
    n_launch_step = len(calls) * inner
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9     # per GPU: average over the launches of one step
    line = {
        "metric": "w8a8_decode_matmul_hbm_gbs", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "s8", "data": "synthetic",
        "config": {"workload": "decode W8A8 matmul_direct, M in {1,4,16} x (K,N) in {(4096,4096),(4096,11008),(11008,4096)}, "
                               "s8 per-token x s8 per-channel prepacked, bf16 out",
                   "gemm_launches_per_step": n_launch_step, "bytes_per_step": step_bytes,
                   "l2_policy": "weights rotate over >126 MB of distinct prepacked copies per shape",
                   "passes_per_step": inner, "launch": "CUDA graphs of %d passes of the grid" % per_graph,
                   "parallelism": "replicas" if world > 1 else "single"},
        "e2e": {"value": round(world * step_bytes / e2e_s / 1e9, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": int(launches), "ms_per_step_by_rank": ms_per_rank,
        "host_enqueue_ms_per_step": round(host_ms / args.steps, 3),
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm"], 4),
                     # DRAM bytes per launch: ncu measured 45.179 MB read + 0.001 MB written for the M=4 K=4096 N=11008 launch
                     # (algorithmic 45.239 MB, ratio 0.9987; profiles/decode_gemm_kernel_M4_K4096_N11008.md); traffic grows
                     # with K*N, so the average launch of this grid is scaled by the same ratio
                     "traffic": int(round(step_bytes / n_launch_step * 0.9987)), "traffic_source": "ncu capture of one shape, scaled by algorithmic bytes",
                     "achieved_def": "algorithmic bytes of one step / device time of the step (all launches are this kernel)",
                     "peak_source": peaks["src"],
                     "kernel": "decode_gemm_kernel (M = 4, 16 and the 16.8 MB weight at M = 1), decode_ring_kernel (M = 1, 45 MB weights)", "frac_of_8TBs": round(achieved / 8000.0, 4)},
        "per_shape": per,
    }
    # free the decode operands before the other workloads of the metric are measured
    del calls, e2e_calls, keep, graph
    capi.lib.b200dnn_clear_caches()
    torch.cuda.empty_cache()
    if not args.no_extras:
        line["also"] = run_extras(torch, capi, dev, rank, world, peaks)
    if rank == 0 and world == 1:
        # N = 1 only: at N > 1 the other ranks' host threads spin in the closing barrier and share the cores
        line["cpu_baseline"] = cpu_baseline_decode(shapes, budget_s=12.0)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        emit(line)


# ---------------------------------------------------------------------------------------------- other workloads
def _time_events(torch, fn, iters, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def run_extras(torch, capi, dev, rank, world, peaks):
    """The other two parts of the metric: prefill W8A8 TOPS (configurations 1 and 3) on one GPU and fused-MoE
    tokens/s (configurations 4 and 5), expert-parallel over all ranks when there are several (weak scaling:
    the tokens per rank stay fixed, the routed experts are sharded e % world, shared experts are replicated).
    Device-resident operands, CUDA-event timing."""
    st = torch.cuda.current_stream().cuda_stream
    out = {}
    int8_peak = 2.0 * peaks["bf16"]          # no measured int8 figure: twice the measured dense bf16 rate
    g = torch.Generator(device="cpu").manual_seed(7 + rank)

    def gemm(M, K, N, dyn, act, copies=1):
        # copies > 1: the calls rotate over that many prepacked weights (together larger than L2) and one pass over
        # them is replayed as a CUDA graph, as in the decode grid
        packs = []
        for _ in range(copies):
            W = torch.randint(-127, 128, (K, N), dtype=torch.int8, generator=g).to(dev)
            packed = torch.empty(capi.lib.b200dnn_prepack_size(K, N, 0), dtype=torch.uint8, device=dev)
            capi.check(capi.lib.b200dnn_prepack(W.data_ptr(), K, N, N, 0, 0, packed.data_ptr(), st))
            torch.cuda.synchronize()
            packs.append(packed)
            del W
        sw = (torch.rand(N, generator=g) * 0.009 + 0.001).to(dev)
        bias = torch.randn(N, generator=g).to(dev)
        o = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        if dyn:
            A = torch.randn(M, K, generator=g).to(torch.bfloat16).to(dev)
            ds = [capi.make_matmul(M, N, K, A, p, o, src_dt=capi.DT["bf16"], dst_dt=capi.DT["bf16"], wei_format="r",
                                   dynamic_quant=True, src_scale=capi.quant(None, count=M, dt=capi.DT["f32"]), wei_scale=sw,
                                   bias=bias, postops=[act]) for p in packs]
        else:
            A = torch.randint(0, 256, (M, K), dtype=torch.uint8, generator=g).to(dev)
            ss = torch.tensor([0.02], device=dev)
            zp = torch.tensor([128], dtype=torch.int32, device=dev)
            ds = [capi.make_matmul(M, N, K, A, p, o, src_dt=capi.DT["u8"], dst_dt=capi.DT["bf16"], wei_format="r",
                                   src_scale=ss, wei_scale=sw, src_zp=zp, bias=bias, postops=[act]) for p in packs]
        if copies == 1:
            ms = _time_events(torch, lambda: capi.check(capi.matmul(ds[0], st)), 20)
        else:
            for d in ds:
                capi.check(capi.matmul(d, st))
            torch.cuda.synchronize()
            side, graph = torch.cuda.Stream(), torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for d in ds:
                    capi.check(capi.matmul(d, torch.cuda.current_stream().cuda_stream))
            ms = _time_events(torch, graph.replay, 20) / copies
        tops = 2.0 * M * N * K / ms / 1e9
        r = {"us": round(ms * 1e3, 1), "tops": round(tops, 1), "frac_of_2x_measured_bf16": round(tops / int8_peak, 3)}
        if copies > 1:
            r["weights"] = "%d prepacked copies in turn (%.0f MB), CUDA graph" % (copies, copies * K * N / 1e6)
        return r

    if rank == 0:
        out["prefill_M2048_K4096_N14336_dynquant_bias_gelu_bf16"] = gemm(2048, 4096, 14336, True, "gelu_tanh")
        out["config1_M128_K4096_N4096_u8zp_bias_relu_bf16"] = gemm(128, 4096, 4096, False, "relu", copies=8)
    torch.cuda.synchronize()
    capi.lib.b200dnn_clear_caches()

    # fused MoE, configurations 4 (Mixtral-like) and 5 (fine-grained, Zipf-skewed routing, 2 shared experts):
    # tokens per rank fixed (weak scaling); one GPU runs b200dnn_moe_layer, several run the expert-parallel layer
    from zendnn_b200 import moe_ep
    for name, (T, H, I, E, topk, S, zipf) in (("moe_mixtral_like", (4096, 4096, 14336, 8, 2, 0, False)),
                                              ("moe_fine_grained", (16384, 2048, 1408, 64, 6, 2, True))):
        x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev)
        logits = torch.randn(T, E, generator=g)
        if zipf:
            gz = torch.Generator(device="cpu").manual_seed(5)
            pz = torch.arange(1, E + 1, dtype=torch.float64) ** -1.1
            logits = logits + torch.log(pz / pz.sum())[torch.randperm(E, generator=gz)].float()
        logits = logits.contiguous().to(dev)

        def expert(e):
            ge = torch.Generator(device="cpu").manual_seed(100 + e)
            return dict(w13=torch.randint(-127, 128, (H, 2 * I), dtype=torch.int8, generator=ge).to(dev),
                        s13=(torch.rand(2 * I, generator=ge) * 1e-3 + 1e-4).to(dev),
                        w2=torch.randint(-127, 128, (I, H), dtype=torch.int8, generator=ge).to(dev),
                        s2=(torch.rand(H, generator=ge) * 1e-3 + 1e-4).to(dev))
        shared = [expert(E + j) for j in range(S)]
        if world == 1:
            every = [expert(e) for e in range(E)] + shared
            ex = (capi.MoeExpert * len(every))()
            for i, w in enumerate(every):
                ex[i].w13, ex[i].ldb13, ex[i].w13_scale = w["w13"].data_ptr(), 2 * I, w["s13"].data_ptr()
                ex[i].w2, ex[i].ldb2, ex[i].w2_scale = w["w2"].data_ptr(), H, w["s2"].data_ptr()
            o = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
            ms = _time_events(torch, lambda: capi.check(capi.lib.b200dnn_moe_layer(
                x.data_ptr(), H, logits.data_ptr(), T, E, S, topk, ex, H, I, H, 0, capi.ACT["silu_and_mul"], o.data_ptr(), H, st)), 5)
            path = "single GPU, b200dnn_moe_layer"
            del every, ex, o
        else:
            mine = [expert(e) for e in moe_ep.experts_on_rank(rank, world, E)]
            ops = moe_ep.CapiOps(mine, shared, H, I, H)
            ms = _time_events(torch, lambda: moe_ep.ep_moe_forward(x, logits, topk, E, S, ops), 5)
            import torch.distributed as dist
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            path = "expert-parallel (expert e on rank e % N), NCCL all-to-all dispatch/combine"
            del ops, mine
        rows = T * (topk + S)
        ops_per_layer = 2.0 * rows * H * 2 * I + 2.0 * rows * I * H
        out[name] = {"tokens_per_s": round(world * T / ms * 1e3), "ms_per_layer": round(ms, 3), "n_gpus": world,
                     "tokens_per_rank": T, "experts": E, "topk": topk, "shared_experts": S, "scaling": "weak",
                     "tops_per_gpu": round(ops_per_layer / ms / 1e9, 1), "path": path}
        del shared, x, logits
        capi.lib.b200dnn_clear_caches()
        torch.cuda.empty_cache()
    return out


# ---------------------------------------------------------------------------------------------- CPU arm
def cpu_baseline_decode(shapes, budget_s=12.0, full=False):
    """The oracle port of the same GEMM + epilogue on the host cores over the same grid of shapes (every M of every
    (K,N), two rotating weights per (K,N)), weights packed outside the timed region (the reference caches its
    reordered weights after the first call).  Passes over the grid are repeated until the time budget is spent."""
    from oracle import oracle as O
    cores = os.cpu_count() or 1
    grid = []
    for (K, N) in DECODE_KN:
        sh = shapes[(K, N)]
        n_w = len(sh["w"]) if full else min(2, len(sh["w"]))
        grid.append((K, N, sh, [O.PackedB(w) for w in sh["w"][:n_w]]))
    t_total, nbytes, calls, passes = 0.0, 0, 0, 0
    t_start = time.perf_counter()
    while passes < 1 or (time.perf_counter() - t_start < budget_s and passes < 200):
        for K, N, sh, packed in grid:
            for M in DECODE_MS:
                qa, sa = sh["acts"][M]
                i = passes % len(packed)
                t0 = time.perf_counter()
                acc = packed[i].gemm_s32(qa)
                O.epilogue(acc, "bf16", sa, sh["s"][i])
                t_total += time.perf_counter() - t0
                nbytes += decode_bytes(M, K, N)
                calls += 1
        passes += 1
    return {"value": round(nbytes / t_total / 1e9, 2), "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": "%d passes over the grid (%d calls: M in %s x %s, 2 rotating weights each), oracle GEMM+epilogue, "
                      "OpenMP on %d threads" % (passes, calls, list(DECODE_MS), list(DECODE_KN), cores)}


def run_reference(args, rank, world):
    if rank != 0:
        return
    rng = np.random.default_rng(1234)
    shapes = make_decode_inputs(rng, copies_bytes=40e6)
    t0 = time.perf_counter()
    base = cpu_baseline_decode(shapes, budget_s=max(5.0, min(60.0, 4.0 * (args.steps + args.warmup))))
    line = {
        "impl": "reference", "metric": "w8a8_decode_matmul_hbm_gbs", "value": base["value"], "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round((time.perf_counter() - t0) * 1e3 / max(1, args.steps), 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "s8", "data": "synthetic",
        "config": {"workload": "decode W8A8 matmul_direct, M in {1,4,16} x (K,N) in {(4096,4096),(4096,11008),(11008,4096)}, "
                               "s8 per-token x s8 per-channel prepacked, bf16 out (CPU arm: repeated passes over the grid within a time budget)"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference default backend (AOCL-DLP) is not in the reference tree; this is the oracle port on the host cores",
    }
    emit(line)


_REAL_STDOUT = None


def emit(line):
    """The one JSON line, on the process's original stdout."""
    sys.stdout.flush()
    data = (json.dumps(line) + "\n").encode()
    if _REAL_STDOUT is None:
        sys.stdout.buffer.write(data)
        sys.stdout.flush()
    else:
        os.write(_REAL_STDOUT, data)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode"])
    ap.add_argument("--inner", type=int, default=100, help="passes over the decode grid per step")
    ap.add_argument("--passes-per-graph", type=int, default=1, help="passes captured in one CUDA graph")
    ap.add_argument("--no-extras", action="store_true", help="skip the prefill and MoE measurements reported under 'also'")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    # stdout carries exactly one JSON line: anything a library prints there (NCCL announces its version on
    # stdout) is sent to stderr instead, and the line is written to the saved descriptor at the end
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
    if rank == 0:
        # torchrun pins OMP_NUM_THREADS=1; the CPU baseline leg (rank 0 only) uses every host core
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
