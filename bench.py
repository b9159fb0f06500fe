#!/usr/bin/env python
"""Benchmark of the B200-native LowOHA W8A8 hot path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline (the part of the metric that is defined at 1/2/4/8 GPUs): fused-MoE tokens/s of group_matmul_direct's
dynamic-INT8 MoE block on the Mixtral-like configuration (hidden 4096, FFN 14336, 8 experts, top-2, SwiGLU; router,
per-token quantisation, two grouped W8A8 GEMMs, requantisation, weighted reduce), 4096 tokens per GPU.  One GPU runs
b200dnn_moe_layer; several GPUs run the library's expert-parallel layer (b200dnn_moe_layer_ep: experts sharded, tokens
exchanged inside the library's kernels over peer memory), tokens per GPU fixed ("weak").  One step = `--inner` layers
over the rank's batch.  The strong-scaling run of the same configuration (4096 tokens in total), the fine-grained
configuration (64 experts, top-6, 2 shared, Zipf-skewed routing) and, on one GPU, the decode-shape GEMM grid (HBM GB/s)
and the prefill GEMMs (TOPS) are reported under "also", each with its own roofline.

Prints ONE JSON line (rank 0).  `value` is measured with inputs resident in HBM (CUDA events on the launching stream, max
over ranks); `e2e` runs the same entry point from pinned HOST activations, logits and outputs, so every layer carries its
host->device and device->host copies (issued on three streams: neighbouring layers' copies overlap the computing layer; the
figure for one blocking call per layer with host pointers is reported beside it).  `--impl reference` times the CPU implementation of the same block on the
host cores (the oracle port; the reference's own default backend, AOCL-DLP, is not part of the reference tree).
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

MOE = {
    "c4": dict(T=4096, H=4096, I=14336, E=8, topk=2, S=0, zipf=False,
               text="fused MoE, Mixtral-like: hidden 4096, FFN 14336, 8 experts, top-2, SwiGLU, s8 per-channel weights, "
                    "per-token s8 activations on both GEMMs, bf16 out"),
    "c5": dict(T=16384, H=2048, I=1408, E=64, topk=6, S=2, zipf=True,
               text="fine-grained MoE: hidden 2048, expert FFN 1408, 64 routed experts top-6 + 2 shared, Zipf(1.1)-skewed "
                    "router bias, W8A8 SwiGLU experts"),
}
WORKLOAD = MOE["c4"]["text"] + "; 4096 tokens per GPU, experts sharded over the GPUs"
METRIC, UNIT = "w8a8_fused_moe_tokens_per_s", "tokens/s"


def decode_bytes(M, K, N):
    return K * N + M * K + 4 * M + 4 * N + 2 * M * N


def moe_ops(rows, H, I):
    """Operations of the two grouped GEMMs for `rows` (token, expert) rows: 2*rows*H*2I + 2*rows*I*H."""
    return 2.0 * rows * H * 2 * I + 2.0 * rows * I * H


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm=d.get("hbm_gbs", 6650.0), bf16=d.get("bf16_tflops", 1590.0),
                    bf16_sustained=d.get("bf16_tflops_sustained", 1400.0), src="measured")
    return dict(hbm=6650.0, bf16=1590.0, bf16_sustained=1400.0, src="fallback")


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
                                          "--format=csv,noheader,nounits", "-lms", "50"],
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
        pw = [float(r[3]) for r in self.rows if len(r) >= 9 and r[3].replace(".", "").isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) >= 9:
                for n, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        return dict(sm_mhz=sm[len(sm) // 2] if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm), power_w_max=max(pw) if pw else None)


# ---------------------------------------------------------------------------------------------- MoE on the GPU
def moe_inputs(torch, dev, cfg, T, seed):
    """Seeded synthetic activations N(0,1) in bf16 and router logits N(0,1) (+ log Zipf(1.1) bias over a seeded
    permutation of the experts for the fine-grained configuration), as the configuration text states."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(T, cfg["H"], generator=g).to(torch.bfloat16)
    logits = torch.randn(T, cfg["E"], generator=g)
    if cfg["zipf"]:
        gz = torch.Generator(device="cpu").manual_seed(5)
        pz = torch.arange(1, cfg["E"] + 1, dtype=torch.float64) ** -1.1
        logits = logits + torch.log(pz / pz.sum())[torch.randperm(cfg["E"], generator=gz)].float()
    return x.to(dev), logits.contiguous().to(dev)


def expert_weights(torch, dev, cfg, e):
    """s8 weights of expert e, the same on whichever rank owns it (seeded by the expert id), made on the GPU."""
    H, I = cfg["H"], cfg["I"]
    g = torch.Generator(device=dev).manual_seed(1000 + e)
    return dict(w13=torch.randint(-127, 128, (H, 2 * I), dtype=torch.int8, generator=g, device=dev),
                s13=torch.rand(2 * I, generator=g, device=dev) * 1e-3 + 1e-4,
                w2=torch.randint(-127, 128, (I, H), dtype=torch.int8, generator=g, device=dev),
                s2=torch.rand(H, generator=g, device=dev) * 1e-3 + 1e-4)


class MoeRunner:
    """One rank of the MoE block: b200dnn_moe_layer on one GPU, the expert-parallel layer on several."""

    def __init__(self, torch, capi, dev, cfg, rank, world, max_tokens, owner=None):
        self.torch, self.capi, self.cfg, self.world, self.rank = torch, capi, cfg, world, rank
        E, S, H, I = cfg["E"], cfg["S"], cfg["H"], cfg["I"]
        self.owner = owner
        if world == 1:
            self.weights = [expert_weights(torch, dev, cfg, e) for e in range(E + S)]
            self.ex = (capi.MoeExpert * (E + S))()
            for i, w in enumerate(self.weights):
                self.ex[i].w13, self.ex[i].ldb13, self.ex[i].w13_scale = w["w13"].data_ptr(), 2 * I, w["s13"].data_ptr()
                self.ex[i].w2, self.ex[i].ldb2, self.ex[i].w2_scale = w["w2"].data_ptr(), H, w["s2"].data_ptr()
            self.layer = None
        else:
            from zendnn_b200 import moe_ep
            mine = [e for e in range(E) if owner[e] == rank] + list(range(E, E + S))
            self.weights = [expert_weights(torch, dev, cfg, e) for e in mine]
            self.layer = moe_ep.EpLayer(rank, world, E, S, cfg["topk"], max_tokens, H, I, H, self.weights, expert_rank=owner)
            self.layer.connect()

    def forward(self, x, logits, out, stream):
        cfg, capi = self.cfg, self.capi
        T = x.shape[0]
        if self.layer is None:
            capi.check(capi.lib.b200dnn_moe_layer(x.data_ptr(), cfg["H"], logits.data_ptr(), T, cfg["E"], cfg["S"], cfg["topk"],
                                                  self.ex, cfg["H"], cfg["I"], cfg["H"], 0, capi.ACT["silu_and_mul"],
                                                  out.data_ptr(), cfg["H"], stream))
        else:
            self.layer.forward(x, logits, out, stream)

    def rows(self, T):
        if self.layer is None:
            return [T * (self.cfg["topk"] + self.cfg["S"])]
        return self.layer.rows_per_rank()

    def close(self):
        if self.layer is not None:
            self.layer.close()
        self.weights = None
        self.capi.lib.b200dnn_clear_caches()
        self.torch.cuda.empty_cache()


def time_layers(torch, dist, runner, x, logits, out, steps, warmup, inner, stream, dev, phases=True):
    """W warm-up steps, then K timed steps of `inner` layers, bracketed by barrier + synchronize; CUDA events on the
    launching stream; max over ranks.  Returns (ms per step, per-rank ms, mean phase ms per layer of this rank)."""
    capi = runner.capi
    for _ in range(warmup):
        for _ in range(inner):
            runner.forward(x, logits, out, stream)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    if phases:
        capi.check(capi.lib.b200dnn_phase_timing(stream, 1))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        for _ in range(inner):
            runner.forward(x, logits, out, stream)
    e1.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    ph = None
    if phases:
        buf, calls = (C.c_float * capi.PHASES)(), C.c_int32(0)
        capi.check(capi.lib.b200dnn_phase_times(stream, buf, capi.PHASES, C.byref(calls)))
        capi.check(capi.lib.b200dnn_phase_timing(stream, 0))
        ph = [float(v) for v in buf]
    per_rank = [ms / steps]
    if dist is not None:
        every = [torch.zeros(1, device=dev) for _ in range(dist.get_world_size())]
        dist.all_gather(every, torch.tensor([ms / steps], device=dev))
        per_rank = [float(v.item()) for v in every]
    return max(per_rank), per_rank, ph


def plan_owner(torch, dist, cfg, logits, world, dev):
    """Expert placement: e % world for the uniform configuration; for the skewed one a load-aware map from the histogram
    of a calibration batch (this step's own logits, summed over the ranks)."""
    from zendnn_b200 import moe_ep
    if world == 1:
        return None, "single"
    if not cfg["zipf"]:
        return moe_ep.modulo_placement(cfg["E"], world), "e % N"
    ids = torch.topk(logits, cfg["topk"], dim=1).indices.reshape(-1)
    hist = torch.bincount(ids, minlength=cfg["E"]).to(dev)
    dist.all_reduce(hist)
    return moe_ep.plan_expert_placement(hist.tolist(), world), "load-aware (greedy over the routed-row histogram, at most ceil(E/N) experts per rank)"


def phase_dict(capi, ph):
    return {n: round(v, 4) for n, v in zip(capi.PHASE_NAMES, ph)}


def run_moe(torch, dist, capi, dev, key, rank, world, T_rank, steps, warmup, inner, stream, peak_tops):
    """Times one MoE configuration at T_rank tokens per rank.  Returns (result dict, runner, tensors)."""
    cfg = MOE[key]
    x, logits = moe_inputs(torch, dev, cfg, T_rank, 7 + rank)
    owner, placement = plan_owner(torch, dist, cfg, logits, world, dev)
    runner = MoeRunner(torch, capi, dev, cfg, rank, world, T_rank, owner)
    out = torch.empty(T_rank, cfg["H"], dtype=torch.bfloat16, device=dev)
    ms, per_rank, ph = time_layers(torch, dist, runner, x, logits, out, steps, warmup, inner, stream, dev)
    rows = runner.rows(T_rank)
    my_rows = rows[rank] if world > 1 else rows[0]
    gemm_ms = ph[4] + ph[6]
    gemm_tops = moe_ops(my_rows, cfg["H"], cfg["I"]) / gemm_ms / 1e9 if gemm_ms > 0 else None
    if dist is not None:
        # the phase times of the slowest rank explain the step time: gather every rank's
        every = [None] * world
        dist.all_gather_object(every, dict(ph=ph, tops=gemm_tops, rows=my_rows))
        slow = max(range(world), key=lambda r: per_rank[r])
        ph_slow, by_rank = every[slow]["ph"], every
    else:
        ph_slow, by_rank, slow = ph, None, 0
    ms_layer = ms / inner
    res = {"tokens_per_s": round(world * T_rank / ms_layer * 1e3), "ms_per_layer": round(ms_layer, 4), "n_gpus": world,
           "tokens_per_rank": T_rank, "experts": cfg["E"], "topk": cfg["topk"], "shared_experts": cfg["S"],
           "placement": placement, "rows_per_rank": rows, "rows_max_over_mean": round(max(rows) / (sum(rows) / len(rows)), 3),
           "phase_ms_per_layer_slowest_rank": phase_dict(capi, ph_slow), "slowest_rank": slow,
           "grouped_gemm_tops_rank0": round(gemm_tops, 1) if gemm_tops else None,
           "grouped_gemm_frac_of_int8_peak_rank0": round(gemm_tops / peak_tops, 4) if gemm_tops and peak_tops else None,
           "ms_per_layer_by_rank": [round(v / inner, 4) for v in per_rank]}
    if by_rank is not None:
        res["grouped_gemm_tops_by_rank"] = [round(b["tops"], 1) if b["tops"] else None for b in by_rank]
    return res, runner, (x, logits, out), ph, my_rows


def measure_int8_peak(capi, stream):
    """Issue-bound tcgen05.mma kind::i8 rate: best of ten short runs (burst) and one run of about two seconds (under
    the power cap), in TOPS."""
    ms, ops = C.c_float(0), C.c_double(0)
    best = 0.0
    for _ in range(10):
        capi.check(capi.lib.b200dnn_measure_int8_peak(4096, 1, C.byref(ms), C.byref(ops), stream))
        best = max(best, ops.value / ms.value / 1e9)
    per_launch_ms = ops.value / (best * 1e9)
    launches = max(10, int(2000.0 / per_launch_ms))
    capi.check(capi.lib.b200dnn_measure_int8_peak(4096, launches, C.byref(ms), C.byref(ops), stream))
    return best, ops.value / ms.value / 1e9


def ep_parity(torch, dist, capi, dev, rank, world, stream):
    """Correctness evidence at N > 1: a small layer (16 experts, top-4, 1 shared, uneven tokens, load-aware map) through the
    expert-parallel entry point against b200dnn_moe_layer on the same tokens with all experts on this GPU."""
    from zendnn_b200 import moe_ep
    cfg = dict(T=0, H=512, I=256, E=16, topk=4, S=1, zipf=True)
    T = 640 + 64 * rank
    x, logits = moe_inputs(torch, dev, cfg, T, 99 + rank)
    ids = torch.topk(logits, cfg["topk"], dim=1).indices.reshape(-1)
    hist = torch.bincount(ids, minlength=cfg["E"]).to(dev)
    dist.all_reduce(hist)
    owner = moe_ep.plan_expert_placement(hist.tolist(), world)
    every = [expert_weights(torch, dev, cfg, e) for e in range(cfg["E"] + cfg["S"])]
    ex = (capi.MoeExpert * len(every))()
    for i, w in enumerate(every):
        ex[i].w13, ex[i].ldb13, ex[i].w13_scale = w["w13"].data_ptr(), 2 * cfg["I"], w["s13"].data_ptr()
        ex[i].w2, ex[i].ldb2, ex[i].w2_scale = w["w2"].data_ptr(), cfg["H"], w["s2"].data_ptr()
    ref = torch.empty(T, cfg["H"], dtype=torch.bfloat16, device=dev)
    capi.check(capi.lib.b200dnn_moe_layer(x.data_ptr(), cfg["H"], logits.data_ptr(), T, cfg["E"], cfg["S"], cfg["topk"], ex,
                                          cfg["H"], cfg["I"], cfg["H"], 0, capi.ACT["silu_and_mul"], ref.data_ptr(), cfg["H"], stream))
    mine = [every[e] for e in range(cfg["E"]) if owner[e] == rank] + every[cfg["E"]:]
    layer = moe_ep.EpLayer(rank, world, cfg["E"], cfg["S"], cfg["topk"], 640 + 64 * world, cfg["H"], cfg["I"], cfg["H"], mine,
                           expert_rank=owner)
    layer.connect()
    got = layer.forward(x, logits)
    torch.cuda.synchronize()
    bad = int((got != ref).any(dim=1).sum().item()) if float(ref.float().abs().sum()) > 0 else T
    ok_status = layer.status() == capi.SUCCESS
    t = torch.tensor([bad + (0 if ok_status else 1)], device=dev)
    dist.all_reduce(t)
    layer.close()
    capi.lib.b200dnn_clear_caches()
    n = int(t.item())
    return "bit-exact" if n == 0 else "%d rows differ" % n


def run_ours(args, rank, world, local_rank):
    import torch
    from zendnn_b200 import capi
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    assert capi.lib.b200dnn_device_count() > 0
    stream = torch.cuda.current_stream().cuda_stream
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    peaks = measured_peaks()
    cfg = MOE["c4"]
    T = cfg["T"]
    inner, steps, warmup = args.inner, args.steps, args.warmup

    # the denominator of the tensor roofline, measured on this GPU before anything else runs
    burst, sustained = measure_int8_peak(capi, stream)
    if dist is not None:
        t = torch.tensor([burst, sustained], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        burst, sustained = float(t[0].item()), float(t[1].item())

    launches0 = capi.lib.b200dnn_launch_count()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.2)
    head, runner, (x, logits, out), ph, my_rows = run_moe(torch, dist, capi, dev, "c4", rank, world, T, steps, warmup, inner,
                                                          stream, sustained)
    clocks = sampler.stop()
    n_calls = (steps + warmup) * inner
    launches_per_layer = (capi.lib.b200dnn_launch_count() - launches0) / n_calls
    ms_per_step = head["ms_per_layer"] * inner

    # the same layer timed alone after a pause (three layers, a few milliseconds): the GPU has no time to reach its power
    # cap, so this is the burst-clock figure that a single call sees; the headline above is the sustained one
    time.sleep(1.0)
    runner.forward(x, logits, out, stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    short_ms = _time_events(torch, lambda: runner.forward(x, logits, out, stream), 3, warm=0)
    if world > 1:
        t = torch.tensor([short_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        short_ms = float(t[0])
    head["short_run"] = {"ms_per_layer": round(short_ms, 4), "tokens_per_s": round(world * T / short_ms * 1e3),
                         "what": "three layers after a one-second pause: burst clocks, no power cap yet"}

    # end to end: the same entry point with pinned host activations, logits and outputs every layer
    xh, lh = x.cpu().pin_memory(), logits.cpu().pin_memory()
    oh = torch.empty(T, cfg["H"], dtype=torch.bfloat16).pin_memory()
    for _ in range(2):
        runner.forward(xh, lh, oh, stream)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    e2e_layers = 10
    t0 = time.perf_counter()
    for _ in range(e2e_layers):
        runner.forward(xh, lh, oh, stream)
    torch.cuda.synchronize()
    serial_s = (time.perf_counter() - t0) / e2e_layers
    # the same copies as a caller with three streams issues them: layer i+1's inputs go up and layer i-1's result comes
    # down while layer i computes (double-buffered device copies of the pinned host tensors; every layer still moves its
    # own inputs and its own result across the bus inside the timed region)
    s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.current_stream(), torch.cuda.Stream()   # compute stays on the stream used so far
    xd = [torch.empty_like(x) for _ in range(2)]
    ld = [torch.empty_like(logits) for _ in range(2)]
    od = [torch.empty(T, cfg["H"], dtype=torch.bfloat16, device=dev) for _ in range(2)]

    def pipeline(n):
        ev_in, ev_cmp, ev_out = {}, {}, {}
        for i in range(n):
            b = i % 2
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ev_cmp[i - 2])           # the buffer's previous layer has been computed
                xd[b].copy_(xh, non_blocking=True)
                ld[b].copy_(lh, non_blocking=True)
                ev_in[i] = torch.cuda.Event()
                ev_in[i].record(s_in)
            s_cmp.wait_event(ev_in[i])
            if i >= 2:
                s_cmp.wait_event(ev_out[i - 2])              # the buffer's previous result has left
            runner.forward(xd[b], ld[b], od[b], stream)
            ev_cmp[i] = torch.cuda.Event()
            ev_cmp[i].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp[i])
                oh.copy_(od[b], non_blocking=True)
                ev_out[i] = torch.cuda.Event()
                ev_out[i].record(s_out)
        torch.cuda.synchronize()
    pipeline(3)
    if dist is not None:
        dist.barrier()
    pipe_layers = max(3, steps) * inner     # as many layers as the device-timed figure ran, so that the GPU is at the same clocks
    t0 = time.perf_counter()
    pipeline(pipe_layers)
    e2e_s = (time.perf_counter() - t0) / pipe_layers
    if dist is not None:
        t = torch.tensor([e2e_s, serial_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s, serial_s = float(t[0].item()), float(t[1].item())
    h2d = inner * (T * cfg["H"] * 2 + T * cfg["E"] * 4)
    d2h = inner * T * cfg["H"] * 2

    gemm_ms = ph[4] + ph[6]
    achieved = moe_ops(my_rows, cfg["H"], cfg["I"]) / gemm_ms / 1e9
    line = {
        "metric": METRIC, "value": head["tokens_per_s"], "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s8",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "layers_per_step": inner, "tokens_per_gpu": T,
                   "entry_point": "b200dnn_moe_layer" if world == 1 else "b200dnn_moe_layer_ep",
                   "l2_policy": "every layer streams 1.4 GB of expert weights per GPU-set (inputs larger than the 126 MB L2)",
                   "parallelism": "single" if world == 1 else "expert-parallel ep%d, tokens data-parallel, placement %s" % (world, head["placement"])},
        "e2e": {"value": round(world * T / e2e_s), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "how": "pinned host activations, logits and outputs; per layer: copy up, b200dnn_moe_layer, copy down, issued on three "
                       "streams so that the copies of neighbouring layers overlap the layer that computes (wall clock over %d layers)" % pipe_layers,
                "one_call_per_layer_with_host_pointers": round(world * T / serial_s)},
        "gpu_launches": int(round(launches_per_layer * inner * steps)), "launches_per_layer": round(launches_per_layer, 1),
        "ms_per_step_by_rank": [round(v * inner, 4) for v in head["ms_per_layer_by_rank"]],
        "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": round(achieved, 1), "peak": round(sustained, 1), "unit": "TOP/s",
                     "frac": round(achieved / sustained, 4),
                     # DRAM bytes per launch from one ncu capture of a 4096-token single-GPU layer ((1.553 + 0.280 + 1.003 + 0.078) GB
                     # over the two launches), scaled by this rank's rows; the algorithmic bytes of such a launch are 0.93 GB
                     "traffic": int(round(1.457e9 * my_rows / 8192.0)),
                     "traffic_source": "ncu capture of the two grouped launches of one configuration-4 layer on one GPU "
                                       "(dram__bytes_read + dram__bytes_write, mean per launch), scaled by the rank's rows",
                     "kernel": "tc_gemm_kernel<false, true>, grouped two-CTA form: the two GEMM launches of a layer (gate|up with the gated epilogue, down)",
                     "achieved_def": "2*rows*H*2I + 2*rows*I*H operations of this rank's rows / mean device time of the two launches per layer "
                                     "(CUDA events recorded by the library on the launching stream inside the timed region)",
                     "peak_source": "int8 tensor rate measured in this run (b200dnn_measure_int8_peak, 2 s run under the power cap); "
                                    "MEASURED_PEAKS.json holds no int8 figure",
                     "int8_tops_measured": {"burst": round(burst, 1), "sustained": round(sustained, 1)},
                     "frac_of_burst": round(achieved / burst, 4),
                     "frac_of_2x_measured_bf16": round(achieved / (2 * peaks["bf16"]), 4), "bf16_peak_source": peaks["src"],
                     "frac_of_nominal_4500": round(achieved / 4500.0, 4)},
        "moe": head,
    }
    also = {}
    if not args.no_extras:
        # strong scaling of the same configuration: 4096 tokens in total
        if world > 1:
            Ts = T // world
            xs, ls, os_ = x[:Ts].contiguous(), logits[:Ts].contiguous(), out[:Ts]
            ms, per_rank, phs = time_layers(torch, dist, runner, xs, ls, os_, steps, warmup, inner, stream, dev)
            rows = runner.rows(Ts)
            also["moe_mixtral_like_strong"] = {"tokens_per_s": round(T / (ms / inner) * 1e3), "ms_per_layer": round(ms / inner, 4),
                                               "total_tokens": T, "tokens_per_rank": Ts, "scaling": "strong", "rows_per_rank": rows,
                                               "phase_ms_per_layer_rank0": phase_dict(capi, phs)}
    del x, logits, out, xh, lh, oh
    runner.close()
    if not args.no_extras:
        c5 = MOE["c5"]
        r5, runner5, tensors5, _, _ = run_moe(torch, dist, capi, dev, "c5", rank, world, c5["T"], max(2, steps // 4), warmup,
                                              max(1, inner // 2), stream, sustained)
        r5["scaling"] = "weak"
        also["moe_fine_grained"] = r5
        if world > 1:
            Ts = c5["T"] // world
            x5, l5, o5 = tensors5
            ms, per_rank, phs = time_layers(torch, dist, runner5, x5[:Ts].contiguous(), l5[:Ts].contiguous(), o5[:Ts],
                                            max(2, steps // 4), warmup, max(1, inner // 2), stream, dev)
            also["moe_fine_grained_strong"] = {"tokens_per_s": round(c5["T"] / (ms / max(1, inner // 2)) * 1e3),
                                               "ms_per_layer": round(ms / max(1, inner // 2), 4), "total_tokens": c5["T"],
                                               "tokens_per_rank": Ts, "scaling": "strong", "rows_per_rank": runner5.rows(Ts),
                                               "phase_ms_per_layer_rank0": phase_dict(capi, phs)}
        del tensors5
        runner5.close()
        if world > 1:
            line["ep_parity"] = ep_parity(torch, dist, capi, dev, rank, world, stream)
            also["nshard_prefill"] = run_nshard(torch, dist, capi, dev, rank, world, stream, sustained)
        else:
            also.update(run_single_gpu_extras(torch, capi, dev, peaks, sustained))
    line["also"] = also
    if rank == 0 and world == 1:
        # N = 1 only: at N > 1 the other ranks' host threads spin in the closing barrier and share the cores
        line["cpu_baseline"] = cpu_baseline_moe(budget_s=12.0)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        emit(line)


# ---------------------------------------------------------------------------------------------- decode and prefill (one GPU)
def make_decode_inputs(rng, copies_bytes=140e6):
    """Quantised operands of every decode combination; `copies` distinct weights per shape."""
    from oracle import oracle as O  # only to quantise the synthetic inputs on the host (not timed)
    shapes = {}
    for K, N in DECODE_KN:
        copies = max(2, int(np.ceil(copies_bytes / (K * N))))
        ws, ss = [], []
        # weights ~ N(0, 0.02) quantised per channel (|q| = 127 at the column max).  One matrix is drawn per shape; the
        # other copies are row rotations of it (same distribution, distinct buffers) to keep set-up time short.
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


def run_decode_grid(torch, capi, dev, peaks, passes=200):
    """The decode-shape W8A8 matmul_direct grid: M in {1,4,16} x (K,N) in {(4096,4096),(4096,11008),(11008,4096)}, per-token
    s8 x per-channel s8 prepacked, bf16 out.  Weights rotate over more than 126 MB of distinct prepacked copies per shape, so
    every launch streams from HBM; one pass of the grid is a CUDA graph.  Metric: algorithmic bytes per second."""
    rng = np.random.default_rng(1234)
    shapes = make_decode_inputs(rng)
    stream = torch.cuda.current_stream().cuda_stream
    calls, keep = [], []
    for (K, N), sh in shapes.items():
        packed = []
        for q, s in zip(sh["w"], sh["s"]):
            buf = torch.empty(capi.lib.b200dnn_prepack_size(K, N, 0), dtype=torch.uint8, device=dev)
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
    pass_bytes = sum(b for _, b in calls)
    side = torch.cuda.Stream()
    for d, _ in calls:
        capi.check(capi.matmul(d, stream))
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for d, _ in calls:
            capi.check(capi.matmul(d, torch.cuda.current_stream().cuda_stream))
    ms = _time_events(torch, graph.replay, passes, warm=20)
    gbs = pass_bytes / ms / 1e6
    per = {}
    for (K, N), sh in shapes.items():
        for M in DECODE_MS:
            sel = [(d, b) for d, b in calls if d.M == M and d.K == K and d.N == N]
            g2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g2, stream=side):
                for d, _ in sel:
                    capi.matmul(d, torch.cuda.current_stream().cuda_stream)
            t_ms = _time_events(torch, g2.replay, 20, warm=2) / len(sel)
            v = sel[0][1] / t_ms / 1e6
            per["M%d_K%d_N%d" % (M, K, N)] = dict(us=round(t_ms * 1e3, 2), gbs=round(v, 1), frac=round(v / peaks["hbm"], 3))
    # end to end through the C ABI with pinned host buffers (activations in, result out, every call)
    e2e_calls, h2d, d2h = [], 0, 0
    for (K, N), sh in shapes.items():
        for M in DECODE_MS:
            qa, sa = sh["acts"][M]
            A = torch.from_numpy(qa).pin_memory(); SA = torch.from_numpy(sa).pin_memory()
            out = torch.empty(M, N, dtype=torch.bfloat16).pin_memory()
            keep.append((A, SA, out))
            for buf, sw in keep[DECODE_KN.index((K, N)) * 4]:
                e2e_calls.append(capi.make_matmul(M, N, K, A, buf, out, src_dt=capi.DT["s8"], dst_dt=capi.DT["bf16"], wei_format="r",
                                                  src_scale=SA, wei_scale=sw, flags=capi.FLAG_STABLE_WEIGHTS))
                h2d += M * K + 4 * M
                d2h += 2 * M * N
    for d in e2e_calls:
        capi.check(capi.matmul(d, stream))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(5):
        for d in e2e_calls:
            capi.matmul(d, stream)
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / 5
    res = {"metric": "w8a8_decode_matmul_hbm_gbs", "value": round(gbs, 1), "unit": "GB/s", "launches_per_pass": len(calls),
           "bytes_per_pass": pass_bytes,
           "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm"], "unit": "GB/s", "frac": round(gbs / peaks["hbm"], 4),
                        "peak_source": peaks["src"], "frac_of_8TBs": round(gbs / 8000.0, 4),
                        "traffic": int(round(pass_bytes / len(calls) * 0.9987)),
                        "traffic_source": "ncu capture of the M=4 K=4096 N=11008 launch (DRAM bytes 0.9987 x algorithmic), scaled by algorithmic bytes"},
           "e2e": {"value": round(pass_bytes / e2e_s / 1e9, 2), "unit": "GB/s", "h2d_bytes_per_pass": h2d, "d2h_bytes_per_pass": d2h},
           "per_shape": per, "cpu_baseline": cpu_baseline_decode(shapes, budget_s=6.0)}
    del calls, e2e_calls, keep, graph
    capi.lib.b200dnn_clear_caches()
    torch.cuda.empty_cache()
    return res


def run_w4a8_grid(torch, capi, dev, peaks, decode_per_shape):
    """W4A8 on the decode shapes (the first "next" row of the scope): bf16 activations quantised per token by the library,
    packed s4 weights with {K/128, N} f32 scales, bf16 out.  Distinct weights per shape in turn (more than the L2 in total,
    prepared once by the library's weight cache), one pass per shape is a CUDA graph.  Weight bytes are K*N/2."""
    g = torch.Generator(device="cpu").manual_seed(99)
    stream = torch.cuda.current_stream().cuda_stream
    side = torch.cuda.Stream()
    gs, out = 128, {}
    for (K, N) in DECODE_KN:
        copies = max(2, int(140e6 // (K * N // 2)) + 1)
        ws = [torch.randint(0, 256, (K * N // 2,), dtype=torch.uint8, generator=g).to(dev) for _ in range(copies)]
        sw = (torch.rand(K // gs, N, generator=g) * 4e-3 + 1e-3).to(dev)
        for M in (1, 16):
            A = torch.randn(M, K, generator=g).to(torch.bfloat16).to(dev)
            o = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            ds = [capi.make_matmul(M, N, K, A, w, o, src_dt=capi.DT["bf16"], dst_dt=capi.DT["bf16"], wei_dt=capi.DT["s4"],
                                   dynamic_quant=True, src_scale=capi.quant(None, count=M, dt=capi.DT["f32"]),
                                   wei_scale=capi.quant(sw, count=(K // gs) * N, dt=capi.DT["f32"]), weights_const=True) for w in ws]
            for d in ds:
                capi.check(capi.matmul(d, stream))
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for d in ds:
                    capi.check(capi.matmul(d, torch.cuda.current_stream().cuda_stream))
            ms = _time_events(torch, graph.replay, 20, warm=3) / len(ds)
            key = "M%d_K%d_N%d" % (M, K, N)
            gbs = (K * N / 2) / ms / 1e6
            w8 = (decode_per_shape or {}).get(key, {}).get("us")
            out[key] = dict(us=round(ms * 1e3, 2), weight_gbs=round(gbs, 1), frac_of_hbm=round(gbs / peaks["hbm"], 3),
                            w8a8_us=w8, launches_per_call=2)
            del graph, ds, A, o
        del ws, sw
        capi.lib.b200dnn_clear_caches()
        torch.cuda.empty_cache()
    return {"what": "W4A8 matmul_direct (bf16 source quantised per token + group-scaled GEMM, group 128) on the decode shapes; "
                    "w8a8_us is the pre-quantised W8A8 call of the same shape from the decode grid", "per_shape": out}


def run_nshard(torch, dist, capi, dev, rank, world, stream, int8_peak):
    """One prefill GEMM of configuration 3 (M 2048, K 4096, N 14336; bf16 source quantised per token, f32 bias, GELU(tanh), bf16
    out) split by N columns over the ranks (b200dnn_matmul_nshard): every rank quantises the whole source and computes its
    column block; with gather = 1 every rank ends with the whole result.  Max over ranks of the device time per call; the
    sharded result is compared with the rank's own unsharded call."""
    import ctypes as C
    M, K, N = 2048, 4096, 14336
    g = torch.Generator(device="cpu").manual_seed(5)
    W = torch.randint(-127, 128, (K, N), dtype=torch.int8, generator=g).to(dev)
    sw = (torch.rand(N, generator=g) * 0.009 + 0.001).to(dev)
    bias = torch.randn(N, generator=g).to(dev)
    A = torch.randn(M, K, generator=g).to(torch.bfloat16).to(dev)
    box = [None]
    if rank == 0:
        ident = (C.c_uint8 * 128)()
        capi.check(capi.lib.b200dnn_ep_nccl_unique_id(ident))
        box[0] = bytes(ident)
    dist.broadcast_object_list(box, src=0)
    ident = (C.c_uint8 * 128).from_buffer_copy(box[0])
    h = C.c_void_p()
    capi.check(capi.lib.b200dnn_nshard_create(world, rank, ident, None, C.byref(h)))
    mk = lambda o: capi.make_matmul(M, N, K, A, W, o, src_dt=capi.DT["bf16"], dst_dt=capi.DT["bf16"], dynamic_quant=True,
                                    src_scale=capi.quant(None, count=M, dt=capi.DT["f32"]), wei_scale=sw, bias=bias,
                                    postops=["gelu_tanh"], weights_const=True)
    whole = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    capi.check(capi.matmul(mk(whole), stream))
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    d = mk(out)
    res = {}
    for gather in (0, 1):
        call = lambda: capi.check(capi.lib.b200dnn_matmul_nshard(h, C.byref(d), gather, stream))
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        dist.barrier()
        ms = _time_events(torch, call, 20, warm=0)
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res["gathered" if gather else "column_blocks"] = {"ms": round(float(t[0]), 4), "tops": round(2.0 * M * N * K / float(t[0]) / 1e9, 1)}
    torch.cuda.synchronize()
    same = torch.tensor([int(torch.equal(out, whole))], device=dev)
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    ms1 = _time_events(torch, lambda: capi.check(capi.matmul(mk(whole), stream)), 20, warm=2)
    res.update({"what": "configuration-3 GEMM (quantise + GEMM + bias + GELU) split by N columns over %d GPUs; ms = max over ranks per call" % world,
                "unsharded_ms_rank0": round(ms1, 4), "equals_unsharded": "bit-exact" if int(same[0]) else "differs",
                "frac_of_int8_peak_all_gpus": round(res["column_blocks"]["tops"] / (int8_peak * world), 4)})
    capi.check(capi.lib.b200dnn_nshard_destroy(h))
    capi.lib.b200dnn_clear_caches()
    return res


def run_single_gpu_extras(torch, capi, dev, peaks, int8_peak):
    """The other parts of the metric, on one GPU: decode HBM GB/s (configuration 2) and prefill TOPS (configurations 3, 1)."""
    st = torch.cuda.current_stream().cuda_stream
    out = {"decode_grid": run_decode_grid(torch, capi, dev, peaks)}
    out["w4a8_decode"] = run_w4a8_grid(torch, capi, dev, peaks, out["decode_grid"].get("per_shape"))
    g = torch.Generator(device="cpu").manual_seed(7)

    def gemm(M, K, N, dyn, act, copies=1):
        # copies > 1: the calls rotate over that many prepacked weights (together larger than L2), one pass is a CUDA graph
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
        r = {"us": round(ms * 1e3, 1), "tops": round(tops, 1),
             "roofline": {"bound": "tensor", "achieved": round(tops, 1), "peak": round(int8_peak, 1), "unit": "TOP/s",
                          "frac": round(tops / int8_peak, 4), "peak_source": "int8 tensor rate measured in this run"}}
        if copies > 1:
            r["weights"] = "%d prepacked copies in turn (%.0f MB), CUDA graph" % (copies, copies * K * N / 1e6)
            r["hbm_gbs"] = round((K * N + M * K + 2 * M * N) / ms / 1e6, 1)
        return r

    out["prefill_M2048_K4096_N14336_dynquant_bias_gelu_bf16"] = gemm(2048, 4096, 14336, True, "gelu_tanh")
    out["prefill_M8192_K4096_N14336_dynquant_bias_gelu_bf16"] = gemm(8192, 4096, 14336, True, "gelu_tanh")
    out["config1_M128_K4096_N4096_u8zp_bias_relu_bf16"] = gemm(128, 4096, 4096, False, "relu", copies=8)
    torch.cuda.synchronize()
    capi.lib.b200dnn_clear_caches()

    # ---- the non-quantised form of the same entry points (bf16:bf16:bf16, the dtype of the reference's MoE traces)
    bf = capi.DT["bf16"]
    bf16_peak = float(peaks["bf16"])

    def bf16_roof(tf):
        return {"bound": "tensor", "achieved": round(tf, 1), "peak": round(bf16_peak, 1), "unit": "TFLOP/s", "frac": round(tf / bf16_peak, 4),
                "peak_source": "bf16 GEMM burst rate, " + peaks["src"]}
    M, K, N = 2048, 4096, 14336
    A = torch.randn(M, K, generator=g).to(torch.bfloat16).to(dev)
    W = (torch.randn(K, N, generator=g) * 0.02).to(torch.bfloat16).to(dev)
    bias = torch.randn(N, generator=g).to(dev)
    o = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    d = capi.make_matmul(M, N, K, A, W, o, src_dt=bf, wei_dt=bf, dst_dt=bf, bias=bias, postops=["gelu_tanh"])
    ms = _time_events(torch, lambda: capi.check(capi.matmul(d, st)), 20)
    tf = 2.0 * M * N * K / ms / 1e9
    out["bf16_prefill_M2048_K4096_N14336_bias_gelu"] = {"us": round(ms * 1e3, 1), "tflops": round(tf, 1), "roofline": bf16_roof(tf)}
    del A, W, o
    cfg = MOE["c4"]
    T, H, I, E, k = cfg["T"], cfg["H"], cfg["I"], cfg["E"], cfg["topk"]
    gd = torch.Generator(device=dev).manual_seed(2000)
    keep, ex = [], (capi.MoeExpert * E)()
    for e in range(E):
        w13 = (torch.randn(H, 2 * I, generator=gd, device=dev) * 0.02).to(torch.bfloat16)
        w2 = (torch.randn(I, H, generator=gd, device=dev) * 0.02).to(torch.bfloat16)
        keep.append((w13, w2))
        ex[e].wei_dt = bf
        ex[e].w13, ex[e].ldb13, ex[e].w2, ex[e].ldb2 = w13.data_ptr(), 2 * I, w2.data_ptr(), H
    x, logits = moe_inputs(torch, dev, cfg, T, 11)
    o = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    ms = _time_events(torch, lambda: capi.check(capi.lib.b200dnn_moe_layer(x.data_ptr(), H, logits.data_ptr(), T, E, 0, k, ex, H, I, H, 0,
                                                                           capi.ACT["silu_and_mul"], o.data_ptr(), H, st)), 5)
    tf = moe_ops(T * k, H, I) / ms / 1e9
    out["moe_mixtral_like_bf16_weights"] = {"tokens_per_s": round(T / ms * 1e3), "ms_per_layer": round(ms, 4), "tflops": round(tf, 1),
                                            "roofline": bf16_roof(tf), "note": "same layer with bf16 experts, no quantisation"}
    del keep, ex, x, logits, o
    torch.cuda.synchronize()

    # ---- the operator in front of the block: fused-add RMSNorm whose result leaves as per-token s8 (and as bf16)
    import ctypes as C
    Rn, Dn = 16384, 4096
    copies = 3                                              # 3 x 134 MB of activations in turn: every call reads from HBM
    xs = [torch.randn(Rn, Dn, generator=gd, device=dev).to(torch.bfloat16) for _ in range(copies)]
    rs = [torch.randn(Rn, Dn, generator=gd, device=dev).to(torch.bfloat16) for _ in range(copies)]
    gamma = torch.randn(Dn, generator=gd, device=dev)
    y = torch.empty(Rn, Dn, dtype=torch.bfloat16, device=dev)
    q = torch.empty(Rn, Dn, dtype=torch.int8, device=dev)
    sc = torch.empty(Rn, dtype=torch.float32, device=dev)
    hbm = float(peaks["hbm"])

    def norm_case(kind, quant, out):
        ds = []
        for i in range(copies):
            d = capi.NormDesc()
            d.norm_type, d.batch, d.norm_size, d.epsilon, d.use_scale = capi.NORM[kind], Rn, Dn, 1e-6, 1
            d.src_dt = d.dst_dt = bf
            d.gamma_dt = d.beta_dt = capi.DT["f32"]
            d.input, d.gamma = xs[i].data_ptr(), gamma.data_ptr()
            d.output = y.data_ptr() if out else None
            if kind == "fused_add_rms_norm":
                d.residual = rs[i].data_ptr()
            if quant:
                d.quant_dst, d.quant_ld, d.quant_scale = q.data_ptr(), Dn, sc.data_ptr()
            ds.append(d)
        it = [0]

        def call():
            capi.check(capi.lib.b200dnn_normalization(C.byref(ds[it[0] % copies]), st))
            it[0] += 1
        ms = _time_events(torch, call, 12, warm=3)
        per = 2 + (2 if out else 0) + (4 if kind == "fused_add_rms_norm" else 0) + (1 if quant else 0)
        gbs = Rn * Dn * per / ms / 1e6
        return {"us": round(ms * 1e3, 1), "bytes_per_element": per, "gbs": round(gbs, 1),
                "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": round(hbm, 1), "unit": "GB/s", "frac": round(gbs / hbm, 4),
                             "peak_source": peaks["src"]}}
    out["norm_rows16384_cols4096_bf16"] = {
        "rms_norm": norm_case("rms_norm", False, True),
        "fused_add_rms_norm": norm_case("fused_add_rms_norm", False, True),
        "fused_add_rms_norm_with_s8_output": norm_case("fused_add_rms_norm", True, True),
        "rms_norm_s8_output_only": norm_case("rms_norm", True, False)}
    del xs, rs, y, q, sc
    torch.cuda.synchronize()

    # ---- attention beside the block (BMM form on the bf16 kernels: the scores pass through HBM)
    Bs, Hs, Ss, Ds = 1, 32, 2048, 128
    qkv = [torch.randn(Bs, Hs, Ss, Ds, generator=gd, device=dev).to(torch.bfloat16) for _ in range(3)]
    oa = torch.empty_like(qkv[0])
    sd = capi.SdpaDesc()
    sd.batch, sd.num_heads, sd.seq_len, sd.kv_seq_len, sd.head_dim = Bs, Hs, Ss, Ss, Ds
    for name in ("q_stride", "k_stride", "v_stride", "o_stride"):
        setattr(sd, name, (C.c_int64 * 4)(Hs * Ss * Ds, Ss * Ds, Ds, 1))
    sd.qkv_dt = sd.out_dt = bf
    sd.is_causal = 1
    sd.query, sd.key, sd.value, sd.output = qkv[0].data_ptr(), qkv[1].data_ptr(), qkv[2].data_ptr(), oa.data_ptr()
    ms = _time_events(torch, lambda: capi.check(capi.lib.b200dnn_sdpa(C.byref(sd), st)), 5)
    tf = 4.0 * Bs * Hs * Ss * Ss * Ds / ms / 1e9
    out["sdpa_bf16_H32_S2048_D128_causal"] = {"us": round(ms * 1e3, 1), "tflops_of_4BHSSD": round(tf, 1), "roofline": bf16_roof(tf),
                                              "note": "BMM form (scores, softmax, P V as separate steps): bound by the scores' HBM round trip"}
    del qkv, oa
    torch.cuda.synchronize()

    # ---- weight preparation at load time: bf16 checkpoint weight -> per-channel s8 in the packed layout
    Kw, Nw = 4096, 14336
    ws = [(torch.randn(Kw, Nw, generator=gd, device=dev) * 0.02).to(torch.bfloat16) for _ in range(2)]
    pk = torch.empty(capi.lib.b200dnn_prepack_size(Kw, Nw, 0), dtype=torch.uint8, device=dev)
    q8 = torch.empty(Kw, Nw, dtype=torch.int8, device=dev)
    sw = torch.empty(Nw, dtype=torch.float32, device=dev)
    it = [0]

    def one_call():
        w = ws[it[0] % 2]; it[0] += 1
        capi.check(capi.lib.b200dnn_quant_prepack(w.data_ptr(), bf, Kw, Nw, Nw, 0, 0, pk.data_ptr(), sw.data_ptr(), st))

    def two_calls():
        w = ws[it[0] % 2]; it[0] += 1
        capi.check(capi.lib.b200dnn_quant_dynamic(w.data_ptr(), bf, Kw, Nw, Nw, 1, q8.data_ptr(), Nw, sw.data_ptr(), st))
        capi.check(capi.lib.b200dnn_prepack(q8.data_ptr(), Kw, Nw, Nw, 0, 0, pk.data_ptr(), st))
    ms1 = _time_events(torch, one_call, 10, warm=3)
    ms2 = _time_events(torch, two_calls, 10, warm=3)
    gbs = Kw * Nw * 5 / ms1 / 1e6                          # the weight read twice (column maxima, then pack) + the s8 written
    out["weight_quant_prepack_K4096_N14336_bf16"] = {
        "one_call_us": round(ms1 * 1e3, 1), "quant_dynamic_then_prepack_us": round(ms2 * 1e3, 1), "bytes_per_element": 5,
        "gbs": round(gbs, 1),
        "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": round(hbm, 1), "unit": "GB/s", "frac": round(gbs / hbm, 4),
                     "peak_source": peaks["src"]}}
    del ws, pk, q8, sw
    torch.cuda.synchronize()
    capi.lib.b200dnn_clear_caches()
    torch.cuda.empty_cache()
    return out


# ---------------------------------------------------------------------------------------------- CPU arms
def cpu_baseline_decode(shapes, budget_s=6.0):
    """The oracle port of the decode GEMM + epilogue on the host cores over the same grid (two rotating weights per
    (K,N)), weights packed outside the timed region.  Best pass out of as many as fit the budget."""
    from oracle import oracle as O
    cores = os.cpu_count() or 1
    grid = [(K, N, shapes[(K, N)], [O.PackedB(w) for w in shapes[(K, N)]["w"][:2]]) for (K, N) in DECODE_KN]
    best, passes, t_start = None, 0, time.perf_counter()
    nbytes = sum(decode_bytes(M, K, N) for (K, N) in DECODE_KN for M in DECODE_MS)
    while passes < 2 or (time.perf_counter() - t_start < budget_s and passes < 200):
        t_pass = 0.0
        for K, N, sh, packed in grid:
            for M in DECODE_MS:
                qa, sa = sh["acts"][M]
                i = passes % len(packed)
                t0 = time.perf_counter()
                acc = packed[i].gemm_s32(qa)
                O.epilogue(acc, "bf16", sa, sh["s"][i])
                t_pass += time.perf_counter() - t0
        passes += 1
        best = t_pass if best is None else min(best, t_pass)
    return {"value": round(nbytes / best / 1e9, 2), "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": "best of %d passes over the nine shapes, 2 rotating weights each, oracle GEMM+epilogue, OpenMP on %d threads" % (passes, cores)}


def cpu_moe_sample(T=512, seed=7):
    """A token sample of the headline configuration for the CPU arm: the same distributions, all eight experts."""
    from oracle import oracle as O
    cfg = MOE["c4"]
    H, I, E = cfg["H"], cfg["I"], cfg["E"]
    rng = np.random.default_rng(seed)
    x = O.f32_to_bf16(rng.normal(size=(T, H)).astype(np.float32))
    logits = rng.normal(size=(T, E)).astype(np.float32)
    ids, w = O.router_topk(logits, cfg["topk"])
    w13, s13, w2, s2 = [], [], [], []
    base13 = rng.integers(-127, 128, (H, 2 * I), dtype=np.int8)
    base2 = rng.integers(-127, 128, (I, H), dtype=np.int8)
    for e in range(E):       # distinct buffers with the same distribution (rotations), to keep set-up short
        w13.append(O.PackedB(np.ascontiguousarray(np.roll(base13, 13 * e, axis=0))))
        w2.append(O.PackedB(np.ascontiguousarray(np.roll(base2, 13 * e, axis=0))))
        s13.append((rng.random(2 * I) * 1e-3 + 1e-4).astype(np.float32))
        s2.append((rng.random(H) * 1e-3 + 1e-4).astype(np.float32))
    return dict(x=x, ids=ids, w=w, w13=w13, s13=s13, w2=w2, s2=s2, T=T)


def cpu_moe_pass(s):
    """One pass of the fused MoE data flow on the host (oracle port, weights packed beforehand as the reference caches
    its reordered weights): per expert quantise -> GEMM -> gated activation -> bf16 -> quantise -> GEMM, then the weighted
    reduce.  Returns seconds."""
    from oracle import oracle as O
    k = s["ids"].shape[1]
    H = s["x"].shape[1]
    t0 = time.perf_counter()
    slot_out = np.zeros((s["T"] * k, H), dtype=np.uint16)
    flat = s["ids"].reshape(-1)
    for e in range(len(s["w13"])):
        slots = np.nonzero(flat == e)[0]
        if slots.size == 0:
            continue
        xe = np.ascontiguousarray(s["x"][slots // k])
        q1, sc1 = O.quant_per_token(xe)
        acc1 = s["w13"][e].gemm_s32(q1)
        I = acc1.shape[1] // 2
        y = O.epilogue(acc1, "f32", sc1, s["s13"][e])
        z = O.gated_act_f32_pairs(y[:, :I], y[:, I:], "silu_and_mul")
        q2, sc2 = O.quant_per_token(z)
        acc2 = s["w2"][e].gemm_s32(q2)
        slot_out[slots] = O.epilogue(acc2, "bf16", sc2, s["s2"][e])
    O.moe_weighted_reduce(slot_out, s["w"], k)
    return time.perf_counter() - t0


def cpu_baseline_moe(budget_s=12.0, passes_max=50):
    cores = os.cpu_count() or 1
    s = cpu_moe_sample()
    cpu_moe_pass(s)                                     # warm-up
    best, n, t_start = None, 0, time.perf_counter()
    while n < 2 or (time.perf_counter() - t_start < budget_s and n < passes_max):
        t = cpu_moe_pass(s)
        best = t if best is None else min(best, t)
        n += 1
    return {"value": round(s["T"] / best), "unit": UNIT, "cores": cores, "kind": "port",
            "sample": "best of %d passes over a %d-token sample of the same configuration (all 8 experts, about %d rows each), "
                      "oracle fused-MoE data flow, OpenMP on %d threads" % (n, s["T"], s["T"] * 2 // 8, cores)}


def run_reference(args, rank, world):
    if rank != 0:
        return
    t0 = time.perf_counter()
    base = cpu_baseline_moe(budget_s=max(5.0, min(60.0, 2.0 * (args.steps + args.warmup))))
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round((time.perf_counter() - t0) * 1e3 / max(1, args.steps), 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "s8", "data": "synthetic",
        "config": {"workload": WORKLOAD},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference default backend (AOCL-DLP) is not in the reference tree; this is the oracle port on the host cores, "
                "timed on a bounded token sample (see cpu_baseline.sample)",
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
    ap.add_argument("--inner", type=int, default=20, help="MoE layers per step")
    ap.add_argument("--no-extras", action="store_true", help="skip the measurements reported under 'also'")
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
        # torchrun pins OMP_NUM_THREADS=1; the CPU legs (rank 0 only) use every host core
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
