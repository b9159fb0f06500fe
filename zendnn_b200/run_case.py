"""Run one configured case of the library a few times on cuda:0 (for profilers and quick timing).

  python -m zendnn_b200.run_case matmul <auto|decode|tc> M K N [--copies C] [--reps R] [--act gelu_tanh] [--bias] [--dyn]
  python -m zendnn_b200.run_case moe <c4|c5> [--reps R] [--wdt s8|bf16]
  python -m zendnn_b200.run_case gs <w4a8|s8> M K N --gs G [--copies C] [--reps R]
  python -m zendnn_b200.run_case bf16 M K N [--copies C] [--reps R] [--act gelu_tanh] [--bias]
  python -m zendnn_b200.run_case norm <rms|fused_add_rms|layer> ROWS COLS [--quant] [--no-output] [--reps R]
  python -m zendnn_b200.run_case sdpa BATCH HEADS SEQ DIM [--causal] [--reps R]

matmul: s8 per-token activations x s8 per-channel prepacked weight -> bf16; `--copies` distinct prepacked
weights are used in turn (pick copies * K * N above the L2 size to keep the weight stream in HBM);
`--dyn` passes bf16 activations with dynamic_quant.  bf16: bf16 activations x bf16 weights (cached by the library
after the first call) -> bf16.  norm: normalization_direct over a bf16 [ROWS, COLS] matrix with an f32 gamma, optionally with
the fused per-token quantised output; buffers rotate so that every call reads from HBM.  moe: b200dnn_moe_layer at the shapes of the two MoE
configurations (c4: 4096 tokens, hidden 4096, FFN 14336, 8 experts top-2; c5: 16384 tokens, hidden 2048,
FFN 1408, 64 experts top-6 + 2 shared, Zipf-skewed routing).  Prints the mean time per call.
"""
import argparse
import time


def _matmul(args):
    import torch
    from . import capi
    dev = torch.device("cuda:0")
    st = torch.cuda.current_stream().cuda_stream
    M, K, N = args.M, args.K, args.N
    g = torch.Generator(device=dev).manual_seed(0)
    packed = []
    for _ in range(args.copies):
        W = torch.randint(-127, 128, (K, N), generator=g, dtype=torch.int8, device=dev)
        buf = torch.empty(capi.lib.b200dnn_prepack_size(K, N, 0), dtype=torch.uint8, device=dev)
        capi.check(capi.lib.b200dnn_prepack(W.data_ptr(), K, N, N, 0, 0, buf.data_ptr(), st))
        torch.cuda.synchronize()
        packed.append(buf)
        del W
    sw = torch.rand(N, generator=g, device=dev) * 4e-4 + 1e-4
    bias = torch.randn(N, generator=g, device=dev) if args.bias else None
    out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    force = {"auto": 0, "decode": 1, "tc": 2}[args.kernel]
    if args.dyn:
        A = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
        kw = dict(src_dt=capi.DT["bf16"], dynamic_quant=True, src_scale=capi.quant(None, M, capi.DT["f32"]))
    else:
        A = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8, device=dev)
        sa = torch.rand(M, generator=g, device=dev) * 0.04 + 0.01
        kw = dict(src_dt=capi.DT["s8"], src_scale=sa)
    descs = [capi.make_matmul(M, N, K, A, b, out, dst_dt=capi.DT["bf16"], wei_format="r", wei_scale=sw, bias=bias,
                              postops=[args.act] if args.act else [], force_kernel=force,
                              flags=capi.FLAG_STABLE_WEIGHTS, **kw) for b in packed]
    for d in descs:
        capi.check(capi.matmul(d, st))
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.reps):
        for d in descs:
            capi.check(capi.matmul(d, st))
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (args.reps * len(descs))
    print("matmul %s M%d K%d N%d: %.2f us per call (stream order, not graph-replayed)" % (args.kernel, M, K, N, us))


def _bf16(args):
    import torch
    from . import capi
    dev = torch.device("cuda:0")
    st = torch.cuda.current_stream().cuda_stream
    M, K, N = args.M, args.K, args.N
    g = torch.Generator(device=dev).manual_seed(0)
    weights = [(torch.randn(K, N, generator=g, device=dev) * 0.02).to(torch.bfloat16) for _ in range(args.copies)]
    A = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
    bias = torch.randn(N, generator=g, device=dev) if args.bias else None
    out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    bf = capi.DT["bf16"]
    descs = [capi.make_matmul(M, N, K, A, w, out, src_dt=bf, wei_dt=bf, dst_dt=bf, bias=bias,
                              postops=[args.act] if args.act else [], flags=capi.FLAG_STABLE_WEIGHTS) for w in weights]
    for d in descs:
        capi.check(capi.matmul(d, st))
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.reps):
        for d in descs:
            capi.check(capi.matmul(d, st))
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (args.reps * len(descs))
    print("bf16 M%d K%d N%d: %.2f us per call, %.0f TFLOP/s (stream order, not graph-replayed)" % (M, K, N, us, 2.0 * M * K * N / us / 1e6))


def _norm(args):
    import ctypes as C
    import torch
    from . import capi
    dev = torch.device("cuda:0")
    st = torch.cuda.current_stream().cuda_stream
    R, N = args.rows, args.cols
    copies = max(2, int(300e6 // (R * N * 2)) + 1)
    g = torch.Generator(device=dev).manual_seed(0)
    xs = [torch.randn(R, N, generator=g, device=dev).to(torch.bfloat16) for _ in range(copies)]
    res = [torch.randn(R, N, generator=g, device=dev).to(torch.bfloat16) for _ in range(copies)] if args.kind == "fused_add_rms" else None
    gamma = torch.randn(N, generator=g, device=dev)
    beta = torch.randn(N, generator=g, device=dev)
    out = torch.empty(R, N, dtype=torch.bfloat16, device=dev)
    q = torch.empty(R, N, dtype=torch.int8, device=dev)
    sc = torch.empty(R, dtype=torch.float32, device=dev)
    descs = []
    for i in range(copies):
        d = capi.NormDesc()
        d.norm_type = capi.NORM[{"rms": "rms_norm", "fused_add_rms": "fused_add_rms_norm", "layer": "layer_norm"}[args.kind]]
        d.batch, d.norm_size, d.epsilon, d.use_scale, d.use_shift = R, N, 1e-6, 1, int(args.kind == "layer")
        d.src_dt = d.dst_dt = capi.DT["bf16"]; d.gamma_dt = d.beta_dt = capi.DT["f32"]
        d.input, d.gamma, d.beta = xs[i].data_ptr(), gamma.data_ptr(), beta.data_ptr()
        d.output = None if args.no_output else out.data_ptr()
        if res is not None:
            d.residual = res[i].data_ptr()
        if args.quant:
            d.quant_dst, d.quant_ld, d.quant_scale = q.data_ptr(), N, sc.data_ptr()
        descs.append(d)
    for d in descs:
        capi.check(capi.lib.b200dnn_normalization(C.byref(d), st))
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.reps):
        for d in descs:
            capi.check(capi.lib.b200dnn_normalization(C.byref(d), st))
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (args.reps * copies)
    elem = 2 + (0 if args.no_output else 2) + (4 if res is not None else 0) + (1 if args.quant else 0)
    print("norm %s rows %d cols %d%s%s: %.2f us per call, %.0f GB/s (%d bytes per element)" %
          (args.kind, R, N, " +quant" if args.quant else "", " no bf16 output" if args.no_output else "", us, R * N * elem / us / 1e3, elem))


def _sdpa(args):
    import ctypes as C
    import torch
    from . import capi
    dev = torch.device("cuda:0")
    st = torch.cuda.current_stream().cuda_stream
    B, H, S, D = args.batch, args.heads, args.seq, args.dim
    g = torch.Generator(device=dev).manual_seed(0)
    q, k, v = (torch.randn(B, H, S, D, generator=g, device=dev).to(torch.bfloat16) for _ in range(3))
    o = torch.empty_like(q)
    d = capi.SdpaDesc()
    d.batch, d.num_heads, d.seq_len, d.kv_seq_len, d.head_dim = B, H, S, S, D
    for name in ("q_stride", "k_stride", "v_stride", "o_stride"):
        setattr(d, name, (C.c_int64 * 4)(H * S * D, S * D, D, 1))
    d.qkv_dt = d.out_dt = capi.DT["bf16"]
    d.is_causal = int(args.causal)
    d.query, d.key, d.value, d.output = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    for _ in range(2):
        capi.check(capi.lib.b200dnn_sdpa(C.byref(d), st))
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.reps):
        capi.check(capi.lib.b200dnn_sdpa(C.byref(d), st))
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / args.reps
    flops = 4.0 * B * H * S * S * D
    print("sdpa B%d H%d S%d D%d%s: %.1f us per call, %.0f TFLOP/s of 4*B*H*S*S*D (BMM form: the scores pass through HBM)" %
          (B, H, S, D, " causal" if args.causal else "", us, flops / us / 1e6))


def _gs(args):
    """Group-scaled forms: w4a8 = bf16 activations quantised per token by the library x packed s4 weights with {K/gs, N}
    scales; s8 = s8 activations with {M, K/gs} scales x s8 weights with {K/gs, N} scales.  Distinct weights in turn, cached
    by the library after the first call."""
    import torch
    from . import capi
    dev = torch.device("cuda:0")
    st = torch.cuda.current_stream().cuda_stream
    M, K, N, gs = args.M, args.K, args.N, args.gs
    G = K // gs
    g = torch.Generator(device=dev).manual_seed(0)
    w4 = args.form == "w4a8"
    weights = [torch.randint(0, 256, (K * N // 2,), generator=g, dtype=torch.uint8, device=dev) if w4 else
               torch.randint(-127, 128, (K, N), generator=g, dtype=torch.int8, device=dev) for _ in range(args.copies)]
    sw = torch.rand(G, N, generator=g, device=dev) * 4e-3 + 1e-3
    out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    if w4:
        A = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
        kw = dict(src_dt=capi.DT["bf16"], dynamic_quant=True, src_scale=capi.quant(None, M, capi.DT["f32"]), wei_dt=capi.DT["s4"])
    else:
        A = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8, device=dev)
        sa = torch.rand(M, G, generator=g, device=dev) * 0.04 + 0.01
        kw = dict(src_dt=capi.DT["s8"], src_scale=capi.quant(sa, M * G, capi.DT["f32"]))
    descs = [capi.make_matmul(M, N, K, A, w, out, dst_dt=capi.DT["bf16"], wei_scale=capi.quant(sw, G * N, capi.DT["f32"]),
                              weights_const=True, **kw) for w in weights]
    for d in descs:
        capi.check(capi.matmul(d, st))
    torch.cuda.synchronize()
    # one pass over the distinct weights as a CUDA graph: the timing is the device's, not the host's enqueue rate
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for d in descs:
            capi.check(capi.matmul(d, torch.cuda.current_stream().cuda_stream))
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (args.reps * len(descs))
    wbytes = K * N / (2 if w4 else 1)
    print("gs %s M%d K%d N%d group %d: %.2f us per call, weight stream %.0f GB/s, %.1f TOPS" %
          (args.form, M, K, N, gs, us, wbytes / us / 1e3, 2.0 * M * K * N / us / 1e6))


def _moe(args):
    import torch
    from . import capi
    dev = torch.device("cuda:0")
    st = torch.cuda.current_stream().cuda_stream
    T, H, I, E, k, S, zipf = dict(c4=(4096, 4096, 14336, 8, 2, 0, False), c5=(16384, 2048, 1408, 64, 6, 2, True))[args.config]
    g = torch.Generator(device=dev).manual_seed(0)
    G = E + S
    keep, ex = [], (capi.MoeExpert * G)()
    for e in range(G):
        if args.wdt == "bf16":
            w13 = (torch.randn(H, 2 * I, generator=g, device=dev) * 0.02).to(torch.bfloat16)
            w2 = (torch.randn(I, H, generator=g, device=dev) * 0.02).to(torch.bfloat16)
            keep.append((w13, w2))
            ex[e].wei_dt = capi.DT["bf16"]
            ex[e].w13, ex[e].ldb13, ex[e].w2, ex[e].ldb2 = w13.data_ptr(), 2 * I, w2.data_ptr(), H
            continue
        w13 = torch.randint(-127, 128, (H, 2 * I), generator=g, dtype=torch.int8, device=dev)
        w2 = torch.randint(-127, 128, (I, H), generator=g, dtype=torch.int8, device=dev)
        s13 = torch.rand(2 * I, generator=g, device=dev) * 4e-4 + 1e-4
        s2 = torch.rand(H, generator=g, device=dev) * 4e-4 + 1e-4
        keep.append((w13, w2, s13, s2))
        ex[e].w13, ex[e].ldb13, ex[e].w13_scale = w13.data_ptr(), 2 * I, s13.data_ptr()
        ex[e].w2, ex[e].ldb2, ex[e].w2_scale = w2.data_ptr(), H, s2.data_ptr()
    x = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, device=dev)
    if zipf:
        p = torch.arange(1, E + 1, device=dev, dtype=torch.float64) ** -1.1
        logits = (logits + torch.log(p / p.sum())[torch.randperm(E, generator=g, device=dev)].float()).contiguous()
    out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)

    def call():
        capi.check(capi.lib.b200dnn_moe_layer(x.data_ptr(), H, logits.data_ptr(), T, E, S, k, ex, H, I, H, 0,
                                              capi.ACT["silu_and_mul"], out.data_ptr(), H, st))
    call()
    call()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(args.reps):
        call()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.reps
    ops = 2 * T * (k + S) * (H * 2 * I + I * H)
    print("moe %s: %.1f us per layer, %.0f tokens/s, %.0f TOPS (wall %.1f us)" %
          (args.config, ms * 1e3, T / ms * 1e3, ops / ms / 1e9, (time.perf_counter() - t0) / args.reps * 1e6))
    # per-phase device times, recorded by the library itself
    import ctypes as C
    capi.check(capi.lib.b200dnn_phase_timing(st, 1))
    for _ in range(args.reps):
        call()
    buf = (C.c_float * capi.PHASES)()
    capi.check(capi.lib.b200dnn_phase_times(st, buf, capi.PHASES, None))
    capi.check(capi.lib.b200dnn_phase_timing(st, 0))
    rows = T * (k + S)
    print("  phases (us): " + ", ".join("%s %.1f" % (n, v * 1e3) for n, v in zip(capi.PHASE_NAMES, buf) if v > 0))
    print("  gemm1 %.0f TOPS, gemm2 %.0f TOPS" % (2.0 * rows * H * 2 * I / buf[4] / 1e9, 2.0 * rows * I * H / buf[6] / 1e9))


def _wprep(args):
    """Weight preparation: a bf16 [K,N] weight to per-channel s8 in the packed layout, one call."""
    import torch
    from . import capi
    dev = torch.device("cuda:0")
    st = torch.cuda.current_stream().cuda_stream
    K, N = args.K, args.N
    g = torch.Generator(device=dev).manual_seed(0)
    ws = [(torch.randn(K, N, generator=g, device=dev) * 0.02).to(torch.bfloat16) for _ in range(2)]
    if args.transB:
        ws = [w.t().contiguous() for w in ws]
    pk = torch.empty(capi.lib.b200dnn_prepack_size(K, N, 0), dtype=torch.uint8, device=dev)
    sw = torch.empty(N, dtype=torch.float32, device=dev)

    def call(i):
        capi.check(capi.lib.b200dnn_quant_prepack(ws[i % 2].data_ptr(), capi.DT["bf16"], K, N, K if args.transB else N,
                                                  int(args.transB), 0, pk.data_ptr(), sw.data_ptr(), st))
    call(0)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.reps):
        call(i + 1)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / args.reps
    print("wprep K%d N%d transB=%d: %.1f us per call, %.0f GB/s of 5 bytes per element" % (K, N, int(args.transB), us, 5.0 * K * N / us / 1e3))


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="what", required=True)
    m = sub.add_parser("matmul")
    m.add_argument("kernel", choices=["auto", "decode", "tc"])
    m.add_argument("M", type=int)
    m.add_argument("K", type=int)
    m.add_argument("N", type=int)
    m.add_argument("--copies", type=int, default=4)
    m.add_argument("--reps", type=int, default=3)
    m.add_argument("--act", default=None)
    m.add_argument("--bias", action="store_true")
    m.add_argument("--dyn", action="store_true")
    q = sub.add_parser("gs")
    q.add_argument("form", choices=["w4a8", "s8"])
    q.add_argument("M", type=int); q.add_argument("K", type=int); q.add_argument("N", type=int)
    q.add_argument("--gs", type=int, default=128)
    q.add_argument("--copies", type=int, default=4)
    q.add_argument("--reps", type=int, default=20)
    b = sub.add_parser("bf16")
    b.add_argument("M", type=int); b.add_argument("K", type=int); b.add_argument("N", type=int)
    b.add_argument("--copies", type=int, default=2)
    b.add_argument("--reps", type=int, default=5)
    b.add_argument("--act", default=None)
    b.add_argument("--bias", action="store_true")
    nm = sub.add_parser("norm")
    nm.add_argument("kind", choices=["rms", "fused_add_rms", "layer"])
    nm.add_argument("rows", type=int); nm.add_argument("cols", type=int)
    nm.add_argument("--quant", action="store_true")
    nm.add_argument("--no-output", action="store_true", dest="no_output")
    nm.add_argument("--reps", type=int, default=5)
    sd = sub.add_parser("sdpa")
    sd.add_argument("batch", type=int); sd.add_argument("heads", type=int); sd.add_argument("seq", type=int); sd.add_argument("dim", type=int)
    sd.add_argument("--causal", action="store_true")
    sd.add_argument("--reps", type=int, default=3)
    e = sub.add_parser("moe")
    e.add_argument("config", choices=["c4", "c5"])
    e.add_argument("--reps", type=int, default=3)
    e.add_argument("--wdt", choices=["s8", "bf16"], default="s8", help="expert weights: s8 (dynamic INT8) or bf16 (no quantisation)")
    wp = sub.add_parser("wprep")
    wp.add_argument("K", type=int); wp.add_argument("N", type=int)
    wp.add_argument("--transB", action="store_true")
    wp.add_argument("--reps", type=int, default=3)
    args = ap.parse_args()
    {"wprep": _wprep, "matmul": _matmul, "moe": _moe, "gs": _gs, "bf16": _bf16, "norm": _norm, "sdpa": _sdpa}[args.what](args)


if __name__ == "__main__":
    main()
