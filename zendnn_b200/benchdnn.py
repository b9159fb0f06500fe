"""Driver that accepts the reference benchmark's inputs (benchdnn, `--op=matmul` and `--op=grp_matmul`): the same
comma-separated input-file lines and, for matmul, the same command-line options, run through libb200dnn on cuda:0,
with a CSV result table in the reference's column order.

  python -m zendnn_b200.benchdnn --op=matmul --input_file=inputs.txt [--cache_mode=hot|warm] [--num_weight_buffers=N]
  python -m zendnn_b200.benchdnn --op=matmul --m=4096 --k=4096 --n=4096 --iters=100 --sdt=bf16 --wdt=s8 --ddt=bf16 \\
         --dynamic_quant=true --src_scale_granularity=per-token

Input-file fields (benchdnn/doc/matmul.md of the reference): m, k, n[:n2...], iters, src:wei:dst, bias, bias_dt,
post_ops (colon-separated), post_op_dt, kernel, is_weights_const, isTransA, isTransB, alpha, beta,
weight_scale_granularity, weight_group_size, weight_scale_dt, warmup_iters, src_dynamic_quant,
src_scale_granularity, src_group_size, src_scale_dt.  Lines starting with '#' and empty lines are skipped.

What runs: the INT8 path of matmul_direct (u8|s8 source with static per-tensor scale and zero point, or bf16|f32
source with src_dynamic_quant and per-token or per-tensor scales; s8 weights with per-channel or per-tensor scales;
bf16|f32|s32 destination) and the bf16 x bf16 path (bf16:bf16:bf16|f32, no quantisation).  Everything else (f32
weights, s4 weights, per-group scales,
alpha/beta other than 1/0, batched lines) is reported as `unimplemented`, which is the status the library returns
for it.  Multi-layer lines (n = a:b:c) run as a pipeline: layer i+1 consumes the bf16 output of layer i.
`--cache_mode=warm` rotates over `--num_weight_buffers` weight copies (default: enough to exceed the L2 size), `hot`
(default) reuses one; `cold` is accepted and treated as `warm` (there is no CPU cache to flush).

  python -m zendnn_b200.benchdnn --op=grp_matmul --input_file=trace.txt [--wdt_as=s8]

grp_matmul lines (benchdnn/doc/grp_matmul.md): num_ops, M (one value or a colon-separated list per expert), K, N, iters,
src:wei:dst, is_weights_const, warmup [, moe_topk [, gated_act [, N_down [, use_internal_alloc [, total_experts]]]]].
What runs: the full fused block (gated_act 1..3, N_down > 0) with s8 or bf16 weights and bf16 source and destination, i.e.
group_matmul_direct's fused MoE (dynamic INT8 with s8 weights, no quantisation with bf16 weights): gate|up GEMM ->
gated activation -> down GEMM, plus the weighted reduce when moe_topk > 0 (row pointers expert by expert, weights
1/topk, as the reference driver builds them).  The reference's shipped traces are bf16:bf16:bf16 and run as written;
`--wdt_as=s8` runs their shapes with s8 weights instead.  Other lines are reported `unimplemented`.

  python -m zendnn_b200.benchdnn --op=reorder --input_file=reorder_inputs.txt

reorder lines of the low-overhead API (benchdnn/doc/reorder.md): batch_size, rows, cols, iters, src_dtype, dst_dtype, algo,
scale_granularity, group_size, dynamic_quant [, num_threads [, warmup_iters]].  What runs (batch_size 1): dynamic
symmetric quantisation to s8 with one scale per row (`per_channel_row`, the per-token form), per column
(`per_channel_col`) or per tensor; static quantisation of f32|bf16 to s8|u8 and static dequantisation of s8|u8 to
f32|bf16 with per-tensor or per-column scales.  f16, per-group granularities, dynamic u8 and batches are reported
`unimplemented`.
"""
import argparse
import sys

FIELDS = ["m", "k", "n", "iters", "dt", "bias", "bias_dt", "post_ops", "post_op_dt", "kernel", "is_weights_const",
          "isTransA", "isTransB", "alpha", "beta", "weight_scale_granularity", "weight_group_size", "weight_scale_dt",
          "warmup_iters", "src_dynamic_quant", "src_scale_granularity", "src_group_size", "src_scale_dt"]
HEADER = ("M, K, N, Iterations, Data type, Bias Enabled, Bias Data type, Post Operation, PostOp Data type, Kernel name, "
          "isWeightsConst, isTransA, isTransB, Alpha, Beta, Weight Scale Granularity, Weight Group Size, "
          "Weight Scale Data type, Warmup iterations, Src Dynamic Quant, Src Scale Granularity, Src Group Size, "
          "Src Scale Data type, Total time (ms) (all iters),  Avg time (ms), GFLOPS, Status")
L2_BYTES = 126 << 20


def _bool(s, default=False):
    s = s.strip().lower()
    if s == "":
        return default
    return s in ("true", "1")


def _gran(s, default):
    s = s.strip().lower()
    table = {"per-channel": "per-channel", "channel": "per-channel", "per-group": "per-group", "group": "per-group",
             "per-tensor": "per-tensor", "tensor": "per-tensor", "per-token": "per-token", "token": "per-token"}
    return table.get(s, default)


def parse_line(line):
    """One input-file line -> config dict, or None for comments / blank lines.  Raises ValueError on a malformed line."""
    text = line.split("#", 1)[0].strip()          # whole-line and trailing comments
    if not text:
        return None
    parts = [p.strip() for p in text.split(",")]
    if len(parts) < 5:
        raise ValueError("expected at least m, k, n, iters, dt: %r" % line)
    parts += [""] * (len(FIELDS) - len(parts))
    f = dict(zip(FIELDS, parts))
    dts = f["dt"].split(":")
    if len(dts) != 3:
        raise ValueError("dt must be src:weights:dst: %r" % f["dt"])
    cfg = dict(
        m=int(f["m"]), k=int(f["k"]), n=[int(v) for v in f["n"].split(":")], iters=int(f["iters"]),
        sdt=dts[0], wdt=dts[1], ddt=dts[2], bias=_bool(f["bias"]), bias_dt=f["bias_dt"] or "f32",
        post_ops=[p for p in f["post_ops"].split(":") if p], post_op_dt=f["post_op_dt"] or "f32", kernel=f["kernel"],
        is_weights_const=_bool(f["is_weights_const"], True), transA=_bool(f["isTransA"]), transB=_bool(f["isTransB"]),
        alpha=float(f["alpha"] or 1.0), beta=float(f["beta"] or 0.0),
        wgran=_gran(f["weight_scale_granularity"], "per-channel"), wgroup=int(f["weight_group_size"] or 0),
        wscale_dt=f["weight_scale_dt"] or "f32", warmup=int(f["warmup_iters"] or 0),
        dyn=_bool(f["src_dynamic_quant"]), sgran=_gran(f["src_scale_granularity"], "per-tensor"),
        sgroup=int(f["src_group_size"] or 0), sscale_dt=f["src_scale_dt"] or "f32")
    if cfg["m"] <= 0 or cfg["k"] <= 0 or min(cfg["n"]) <= 0 or cfg["iters"] <= 0:
        raise ValueError("m, k, n, iters must be positive: %r" % line)
    return cfg


def parse_file(path):
    out = []
    with open(path) as fh:
        for no, line in enumerate(fh, 1):
            try:
                cfg = parse_line(line)
            except ValueError as e:
                raise ValueError("%s:%d: %s" % (path, no, e))
            if cfg:
                out.append(cfg)
    return out


def unsupported_reason(cfg):
    """None when the line is inside the subset the library computes, else why not."""
    bf16 = cfg["wdt"] == "bf16" and cfg["sdt"] == "bf16" and not cfg["dyn"]
    if cfg["wdt"] != "s8" and not bf16:
        return "weights %s with source %s (s8 weights, or bf16 x bf16)" % (cfg["wdt"], cfg["sdt"])
    if bf16:
        if cfg["ddt"] not in ("bf16", "f32"):
            return "destination %s" % cfg["ddt"]
        if len(cfg["n"]) > 1 and cfg["ddt"] != "bf16":
            return "pipeline lines need a bf16 destination between layers"
    elif cfg["dyn"]:
        if cfg["sdt"] not in ("bf16", "f32"):
            return "dynamic quantisation takes a bf16 or f32 source"
        if cfg["sgran"] == "per-group":
            return "per-group source scales"
    elif cfg["sdt"] not in ("u8", "s8"):
        return "source %s without src_dynamic_quant" % cfg["sdt"]
    if cfg["ddt"] not in ("bf16", "f32", "s32"):
        return "destination %s" % cfg["ddt"]
    if cfg["wgran"] == "per-group":
        return "per-group weight scales"
    if cfg["alpha"] != 1.0 or cfg["beta"] != 0.0:
        return "alpha/beta other than 1/0"
    known = {"relu", "gelu_tanh", "gelu_erf", "sigmoid", "swish", "tanh", "elu", "leaky_relu", "binary_add", "binary_mul"}
    for p in cfg["post_ops"]:
        if p not in known:
            return "post-op %s" % p
    if len(cfg["n"]) > 1 and cfg["ddt"] != "bf16" and not cfg["dyn"] and not bf16:
        return "pipeline lines need dynamic quantisation between layers"
    return None


def row(cfg, total_ms, status):
    n = ":".join(str(v) for v in cfg["n"])
    flops = 0.0
    k = cfg["k"]
    for nn in cfg["n"]:
        flops += 2.0 * cfg["m"] * k * nn
        k = nn
    avg = total_ms / cfg["iters"] if total_ms else 0.0
    gflops = flops / (avg * 1e6) if avg else 0.0
    vals = [cfg["m"], cfg["k"], n, cfg["iters"], "%s:%s:%s" % (cfg["sdt"], cfg["wdt"], cfg["ddt"]), str(cfg["bias"]).lower(),
            cfg["bias_dt"], ":".join(cfg["post_ops"]), cfg["post_op_dt"], cfg["kernel"], str(cfg["is_weights_const"]).lower(),
            str(cfg["transA"]).lower(), str(cfg["transB"]).lower(), "%.2f" % cfg["alpha"], "%.2f" % cfg["beta"], cfg["wgran"],
            cfg["wgroup"], cfg["wscale_dt"], cfg["warmup"], str(cfg["dyn"]).lower(), cfg["sgran"], cfg["sgroup"], cfg["sscale_dt"],
            "%.2f" % total_ms, "%.4f" % avg, "%.2f" % gflops, status]
    return ", ".join(str(v) for v in vals)


def run_config(cfg, cache_mode="hot", num_weight_buffers=0, capture=None):
    """Runs one line on cuda:0.  Returns (total_ms over iters, status string).  capture: a dict that receives host
    copies of the operands and results of the first weight set (for checks against a CPU statement of the line)."""
    why = unsupported_reason(cfg)
    if why:
        return 0.0, "unimplemented (%s)" % why
    import torch
    from . import capi
    dev = torch.device("cuda:0")
    st = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device=dev).manual_seed(0)
    M = cfg["m"]
    layers, k = [], cfg["k"]
    wbf16 = cfg["wdt"] == "bf16"
    tdt = {"bf16": torch.bfloat16, "f32": torch.float32, "s32": torch.int32}
    for li, n in enumerate(cfg["n"]):
        last = li == len(cfg["n"]) - 1
        copies = 1
        if cache_mode in ("warm", "cold"):
            copies = num_weight_buffers if num_weight_buffers > 0 else max(2, -(-L2_BYTES // (k * n)) + 1)
        shape = (n, k) if cfg["transB"] else (k, n)
        if wbf16:
            ws = [(torch.randn(shape, generator=g, device=dev) * 0.02).to(torch.bfloat16) for _ in range(copies)]
        else:
            ws = [torch.randint(-127, 128, shape, generator=g, dtype=torch.int8, device=dev) for _ in range(copies)]
        wn = n if cfg["wgran"] == "per-channel" else 1
        wscale = (torch.rand(wn, generator=g, device=dev) * 4e-4 + 1e-4)
        if cfg["wscale_dt"] == "bf16":
            wscale = wscale.to(torch.bfloat16)
        bias = None
        if cfg["bias"]:
            bias = torch.randn(n, generator=g, device=dev)
            if cfg["bias_dt"] == "bf16":
                bias = bias.to(torch.bfloat16)
        pos = []
        for p in cfg["post_ops"]:
            if p.startswith("binary"):
                b = torch.randn(M, n, generator=g, device=dev)
                pos.append(dict(type=p, buff=b.to(torch.bfloat16) if cfg["post_op_dt"] == "bf16" else b))
            else:
                pos.append(p)
        ddt = cfg["ddt"] if last else "bf16"
        out = torch.empty(M, n, dtype=tdt[ddt], device=dev)
        layers.append(dict(k=k, n=n, ws=ws, wscale=wscale, bias=bias, pos=pos, out=out, ddt=ddt))
        k = n
    if cfg["dyn"] or wbf16:
        x = torch.randn(M, cfg["k"], generator=g, device=dev)
        x = x.to(torch.bfloat16) if cfg["sdt"] == "bf16" else x
    else:
        lo, hi = (0, 256) if cfg["sdt"] == "u8" else (-127, 128)
        x = torch.randint(lo, hi, (M, cfg["k"]), generator=g, device=dev, dtype=torch.uint8 if cfg["sdt"] == "u8" else torch.int8)
    sscale = torch.tensor([0.02], device=dev)
    szp = torch.tensor([128], dtype=torch.int32, device=dev) if cfg["sdt"] == "u8" else None

    if cfg["transA"]:
        x = x.t().contiguous()                     # stored [K, M]: element (m, k) at k * M + m

    def descs(it):
        ds, src, src_dt = [], x, cfg["sdt"]
        for li, L in enumerate(layers):
            w = L["ws"][it % len(L["ws"])]
            dyn = (cfg["dyn"] or li > 0) and not wbf16
            kw = {}
            if wbf16:
                kw["wei_dt"] = capi.DT["bf16"]
            elif dyn:
                kw["src_scale"] = capi.quant(None, M if cfg["sgran"] == "per-token" or li > 0 else 1, capi.DT[cfg["sscale_dt"]])
            else:
                kw["src_scale"] = sscale
                if szp is not None:
                    kw["src_zp"] = szp
            ds.append(capi.make_matmul(M, L["n"], L["k"], src, w, L["out"], src_dt=capi.DT[src_dt], dst_dt=capi.DT[L["ddt"]],
                                       transB=cfg["transB"], transA=bool(cfg["transA"]) and li == 0, bias=L["bias"], weights_const=cfg["is_weights_const"],
                                       dynamic_quant=dyn, wei_scale=None if wbf16 else L["wscale"], postops=L["pos"], **kw))
            src, src_dt = L["out"], "bf16"
        return ds

    n_sets = max(len(L["ws"]) for L in layers)
    sets = [descs(i) for i in range(n_sets)]
    for d in sets[0]:
        stt = capi.matmul(d, st)
        if stt != capi.SUCCESS:
            return 0.0, ("unimplemented" if stt == capi.UNIMPLEMENTED else "failure") + " (%s)" % capi.last_error()
    for i in range(cfg["warmup"]):
        for d in sets[i % n_sets]:
            capi.matmul(d, st)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(cfg["iters"]):
        for d in sets[i % n_sets]:
            capi.matmul(d, st)
    e1.record()
    torch.cuda.synchronize()
    if capture is not None:
        for d in sets[0]:
            capi.matmul(d, st)
        torch.cuda.synchronize()

        def host(t):
            if t is None:
                return None
            return (t.view(torch.int16) if t.dtype == torch.bfloat16 else t).cpu().numpy()
        capture.update(x=host(x), sscale=host(sscale), szp=None if szp is None else 128,
                       layers=[dict(w=host(L["ws"][0]), wscale=host(L["wscale"]), bias=host(L["bias"]), out=host(L["out"]), ddt=L["ddt"],
                                    pos=[dict(p, buff=host(p["buff"])) if isinstance(p, dict) else p for p in L["pos"]])
                               for L in layers])
    capi.lib.b200dnn_clear_caches()
    return e0.elapsed_time(e1), "success"


# ------------------------------------------------------------------------------------------------ grp_matmul
GRP_HEADER = ("ops, M, K, N, iters, warmup, dtypes, moe, gated_act, N_down, total_experts, Total time (ms) (all iters), "
              "Avg time (ms), GFLOPS, Status")


def parse_grp_line(line):
    if not line.strip() or line.lstrip().startswith("#"):
        return None
    # the shipped traces end their rows with "# freq=N" (the reference's std::stoi stops at the blank before it)
    parts = [p.strip() for p in line.split("#", 1)[0].strip().split(",")]
    if len(parts) < 8:
        raise ValueError("expected num_ops, M, K, N, iters, dt, is_weights_const, warmup: %r" % line)
    parts += [""] * (13 - len(parts))
    ops = int(parts[0])
    ms = [int(v) for v in parts[1].split(":")]
    if len(ms) == 1:
        ms = ms * ops
    if len(ms) != ops:
        raise ValueError("M lists %d values for %d ops: %r" % (len(ms), ops, line))
    dts = parts[5].split(":")
    if len(dts) != 3:
        raise ValueError("dt must be src:weights:dst: %r" % parts[5])
    cfg = dict(ops=ops, M=ms, k=int(parts[2]), n=int(parts[3]), iters=int(parts[4]), sdt=dts[0], wdt=dts[1], ddt=dts[2],
               is_weights_const=_bool(parts[6], True), warmup=int(parts[7] or 0), topk=int(parts[8] or 0),
               act=int(parts[9] or 0), n_down=int(parts[10] or 0), internal_alloc=int(parts[11] or 0),
               total_experts=int(parts[12] or 0) or ops)
    if ops <= 0 or cfg["k"] <= 0 or cfg["n"] <= 0 or cfg["iters"] <= 0 or min(ms) < 0 or cfg["total_experts"] < ops:
        raise ValueError("bad sizes: %r" % line)
    return cfg


def grp_unsupported_reason(cfg):
    if cfg["wdt"] not in ("s8", "bf16"):
        return "weights %s (s8 or bf16)" % cfg["wdt"]
    if cfg["sdt"] != "bf16" or cfg["ddt"] != "bf16":
        return "source/destination other than bf16"
    if cfg["act"] not in (1, 2, 3) or cfg["n_down"] <= 0:
        return "only the fused gate/up -> activation -> down block"
    if cfg["n"] % 2:
        return "odd N"
    if cfg["topk"] > 0 and sum(cfg["M"]) % cfg["topk"]:
        return "total M not divisible by moe_topk"
    return None


def grp_row(cfg, total_ms, status):
    ms = cfg["M"]
    mtxt = str(ms[0]) if len(set(ms)) == 1 else "%d-%d(%d)" % (min(ms), max(ms), sum(ms) // len(ms))
    I = cfg["n"] // 2
    flops = sum(2.0 * m * cfg["k"] * cfg["n"] + 2.0 * m * I * cfg["n_down"] for m in ms)
    if cfg["topk"] > 0 and cfg["n_down"] > 0:
        flops += 2.0 * (sum(ms) // cfg["topk"]) * cfg["n_down"] * cfg["topk"]
    avg = total_ms / cfg["iters"] if total_ms else 0.0
    vals = [cfg["ops"], mtxt, cfg["k"], cfg["n"], cfg["iters"], cfg["warmup"], "%s:%s:%s" % (cfg["sdt"], cfg["wdt"], cfg["ddt"]),
            "topk=%d" % cfg["topk"] if cfg["topk"] else "off", cfg["act"], cfg["n_down"], cfg["total_experts"],
            "%.2f" % total_ms, "%.4f" % avg, "%.2f" % (flops / (avg * 1e6) if avg else 0.0), status]
    return ", ".join(str(v) for v in vals)


def run_grp_config(cfg):
    why = grp_unsupported_reason(cfg)
    if why:
        return 0.0, "unimplemented (%s)" % why
    import ctypes as C
    import torch
    from . import capi
    dev = torch.device("cuda:0")
    st = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device=dev).manual_seed(0)
    E, K, I, H = cfg["ops"], cfg["k"], cfg["n"] // 2, cfg["n_down"]
    wbf16 = cfg["wdt"] == "bf16"
    keep, ex = [], (capi.MoeExpert * E)()
    total = sum(cfg["M"])
    ptrs = (C.c_void_p * max(1, total))()
    slot = 0
    for e, m in enumerate(cfg["M"]):
        if wbf16:
            w13 = (torch.randn(K, 2 * I, generator=g, device=dev) * 0.02).to(torch.bfloat16)
            w2 = (torch.randn(I, H, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        else:
            w13 = torch.randint(-127, 128, (K, 2 * I), generator=g, dtype=torch.int8, device=dev)
            w2 = torch.randint(-127, 128, (I, H), generator=g, dtype=torch.int8, device=dev)
        s13 = torch.rand(2 * I, generator=g, device=dev) * 4e-4 + 1e-4
        s2 = torch.rand(H, generator=g, device=dev) * 4e-4 + 1e-4
        src = torch.randn(max(m, 1), K, generator=g, device=dev).to(torch.bfloat16)
        dst = torch.empty(max(m, 1), H, dtype=torch.bfloat16, device=dev)
        keep.append((w13, w2, s13, s2, src, dst))
        x = ex[e]
        x.M, x.src, x.lda = m, src.data_ptr(), K
        x.wei_dt = capi.DT["bf16"] if wbf16 else capi.DT["s8"]
        x.w13, x.ldb13, x.w13_scale = w13.data_ptr(), 2 * I, s13.data_ptr()
        x.w2, x.ldb2, x.w2_scale = w2.data_ptr(), H, s2.data_ptr()
        x.dst_down, x.ldc_down = dst.data_ptr(), H
        for r in range(m):      # row pointers expert by expert, as the reference driver builds them
            ptrs[slot] = dst.data_ptr() + r * H * 2
            slot += 1
    topk = cfg["topk"]
    T = total // topk if topk else 0
    if topk:
        w = torch.full((T, topk), 1.0 / topk, device=dev)
        out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        keep.append((w, out))

    def call():
        return capi.lib.b200dnn_fused_moe(E, ex, K, I, H, 0, cfg["act"], int(cfg["is_weights_const"]),
                                          ptrs if topk else None, w.data_ptr() if topk else None, T, topk,
                                          out.data_ptr() if topk else None, H, st)
    stt = call()
    if stt != capi.SUCCESS:
        return 0.0, ("unimplemented" if stt == capi.UNIMPLEMENTED else "failure") + " (%s)" % capi.last_error()
    for _ in range(cfg["warmup"]):
        call()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(cfg["iters"]):
        call()
    e1.record()
    torch.cuda.synchronize()
    capi.lib.b200dnn_clear_caches()
    return e0.elapsed_time(e1), "success"


# ------------------------------------------------------------------------------------------------ reorder
REORDER_HEADER = ("batch, rows, cols, iters, src_dtype, dst_dtype, algo, scale_granularity, group_size, dynamic_quant, "
                  "warmup_iters, Total time (ms) (all iters), Avg time (ms), GB/s, Status")


def parse_reorder_line(line):
    if not line.strip() or line.lstrip().startswith("#"):
        return None
    parts = [p.strip() for p in line.split("#", 1)[0].strip().split(",")]
    if len(parts) < 10:
        raise ValueError("expected batch, rows, cols, iters, src, dst, algo, granularity, group_size, dynamic_quant: %r" % line)
    parts += [""] * (12 - len(parts))
    cfg = dict(batch=int(parts[0]), rows=int(parts[1]), cols=int(parts[2]), iters=int(parts[3]), sdt=parts[4], ddt=parts[5],
               algo=parts[6], gran=parts[7].lower(), group=int(parts[8] or 0), dyn=_bool(parts[9]),
               threads=int(parts[10] or 0), warmup=int(parts[11]) if parts[11] else max(1, int(parts[3]) // 5))
    if min(cfg["batch"], cfg["rows"], cfg["cols"], cfg["iters"]) <= 0:
        raise ValueError("sizes must be positive: %r" % line)
    return cfg


def reorder_unsupported_reason(cfg):
    if cfg["batch"] != 1:
        return "batched reorder"
    if "f16" in (cfg["sdt"], cfg["ddt"]) and "bf16" not in (cfg["sdt"], cfg["ddt"]):
        return "f16"
    if cfg["gran"] not in ("per_tensor", "per_channel_row", "per_channel_col"):
        return "granularity %s" % cfg["gran"]
    quant = cfg["sdt"] in ("f32", "bf16") and cfg["ddt"] in ("s8", "u8")
    dequant = cfg["sdt"] in ("s8", "u8") and cfg["ddt"] in ("f32", "bf16")
    if not (quant or dequant):
        return "%s -> %s" % (cfg["sdt"], cfg["ddt"])
    if cfg["dyn"]:
        if not quant or cfg["ddt"] != "s8":
            return "dynamic quantisation writes s8 from f32|bf16"
    elif cfg["gran"] == "per_channel_row":
        return "static per-row scales"
    return None


def reorder_row(cfg, total_ms, status):
    esz = dict(f32=4, bf16=2, f16=2, s8=1, u8=1)
    avg = total_ms / cfg["iters"] if total_ms else 0.0
    bytes_moved = cfg["batch"] * cfg["rows"] * cfg["cols"] * (esz.get(cfg["sdt"], 0) + esz.get(cfg["ddt"], 0))
    vals = [cfg["batch"], cfg["rows"], cfg["cols"], cfg["iters"], cfg["sdt"], cfg["ddt"], cfg["algo"], cfg["gran"], cfg["group"],
            str(cfg["dyn"]).lower(), cfg["warmup"], "%.2f" % total_ms, "%.4f" % avg,
            "%.1f" % (bytes_moved / (avg * 1e6) if avg else 0.0), status]
    return ", ".join(str(v) for v in vals)


def run_reorder_config(cfg):
    why = reorder_unsupported_reason(cfg)
    if why:
        return 0.0, "unimplemented (%s)" % why
    import torch
    from . import capi
    dev = torch.device("cuda:0")
    st = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device=dev).manual_seed(0)
    M, N = cfg["rows"], cfg["cols"]
    tdt = dict(f32=torch.float32, bf16=torch.bfloat16, s8=torch.int8, u8=torch.uint8)
    L = capi.lib
    if cfg["sdt"] in ("f32", "bf16"):
        src = torch.randn(M, N, generator=g, device=dev).to(tdt[cfg["sdt"]])
    else:
        lo, hi = (0, 256) if cfg["sdt"] == "u8" else (-127, 128)
        src = torch.randint(lo, hi, (M, N), generator=g, device=dev, dtype=tdt[cfg["sdt"]])
    dst = torch.empty(M, N, dtype=tdt[cfg["ddt"]], device=dev)
    n_scale = N if cfg["gran"] == "per_channel_col" else 1
    if cfg["dyn"]:
        if cfg["gran"] == "per_channel_row":
            scale = torch.empty(M, device=dev)
            call = lambda: L.b200dnn_quant_per_token(src.data_ptr(), capi.DT[cfg["sdt"]], M, N, N, dst.data_ptr(), N,
                                                     scale.data_ptr(), capi.DT["f32"], st)
        else:
            scale = torch.empty(n_scale, device=dev)
            call = lambda: L.b200dnn_quant_dynamic(src.data_ptr(), capi.DT[cfg["sdt"]], M, N, N, int(n_scale > 1), dst.data_ptr(),
                                                   N, scale.data_ptr(), st)
    else:
        scale = torch.rand(n_scale, generator=g, device=dev) * 0.05 + 0.01
        zp = torch.full((1,), 128, dtype=torch.int32, device=dev) if "u8" in (cfg["sdt"], cfg["ddt"]) else None
        zp_ptr, n_zp = (zp.data_ptr(), 1) if zp is not None else (None, 0)
        if cfg["ddt"] in ("s8", "u8"):
            call = lambda: L.b200dnn_quant_static(src.data_ptr(), capi.DT[cfg["sdt"]], M, N, N, scale.data_ptr(), n_scale, zp_ptr,
                                                  n_zp, dst.data_ptr(), capi.DT[cfg["ddt"]], N, st)
        else:
            call = lambda: L.b200dnn_dequant_static(src.data_ptr(), capi.DT[cfg["sdt"]], M, N, N, scale.data_ptr(), n_scale, zp_ptr,
                                                    n_zp, dst.data_ptr(), capi.DT[cfg["ddt"]], N, st)
    stt = call()
    if stt != capi.SUCCESS:
        return 0.0, ("unimplemented" if stt == capi.UNIMPLEMENTED else "failure") + " (%s)" % capi.last_error()
    for _ in range(cfg["warmup"]):
        call()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(cfg["iters"]):
        call()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1), "success"


def config_from_args(a):
    line = ", ".join(str(v) for v in [
        a.m, a.k, a.n, a.iters, "%s:%s:%s" % (a.sdt, a.wdt, a.ddt), a.bias, a.bias_dt, a.post_ops, a.post_op_dt, a.kernel_name,
        a.is_weights_const, a.isTransA, a.isTransB, a.alpha, a.beta, a.weight_scale_granularity, a.weight_group_size,
        a.weight_scale_dt, a.warmup_iters, a.dynamic_quant, a.src_scale_granularity, a.src_group_size, a.src_scale_dt])
    return parse_line(line)


def main(argv=None):
    ap = argparse.ArgumentParser(description="benchdnn-style matmul driver over libb200dnn")
    ap.add_argument("--op", default="matmul")
    ap.add_argument("--input_file")
    ap.add_argument("--cache_mode", default="hot")
    ap.add_argument("--num_weight_buffers", type=int, default=0)
    ap.add_argument("--ndims", type=int, default=2)
    ap.add_argument("--lowoha", default="true")
    ap.add_argument("--wdt_as", default="", help="grp_matmul: run the lines with this weight type instead of the one in the file")
    for name, default in (("m", 0), ("k", 0), ("n", "0"), ("iters", 100), ("sdt", "f32"), ("wdt", "f32"), ("ddt", "f32"),
                          ("bias", "false"), ("bias_dt", "f32"), ("post_ops", ""), ("post_op_dt", "f32"), ("kernel_name", ""),
                          ("is_weights_const", "true"), ("isTransA", "false"), ("isTransB", "false"), ("alpha", 1.0),
                          ("beta", 0.0), ("weight_scale_granularity", "per-channel"), ("weight_group_size", 0),
                          ("weight_scale_dt", "f32"), ("warmup_iters", 0), ("dynamic_quant", "false"),
                          ("src_scale_granularity", "per-tensor"), ("src_group_size", 0), ("src_scale_dt", "f32")):
        ap.add_argument("--" + name, default=default)
    a = ap.parse_args(argv)
    if a.op == "grp_matmul":
        if not a.input_file:
            print("--op=grp_matmul needs --input_file", file=sys.stderr)
            return 2
        print(GRP_HEADER)
        with open(a.input_file) as fh:
            for line in fh:
                cfg = parse_grp_line(line)
                if cfg is None:
                    continue
                if a.wdt_as:
                    cfg["wdt"] = a.wdt_as
                total, status = run_grp_config(cfg)
                print(grp_row(cfg, total, status), flush=True)
        return 0
    if a.op == "reorder":
        if not a.input_file or a.lowoha.lower() != "true":
            print("--op=reorder needs --input_file and the low-overhead API (--lowoha=true)", file=sys.stderr)
            return 2
        print(REORDER_HEADER)
        with open(a.input_file) as fh:
            for line in fh:
                cfg = parse_reorder_line(line)
                if cfg is None:
                    continue
                total, status = run_reorder_config(cfg)
                print(reorder_row(cfg, total, status), flush=True)
        return 0
    if a.op != "matmul" or a.ndims != 2:
        print("only --op=matmul with --ndims=2, --op=grp_matmul and --op=reorder are in scope of this library", file=sys.stderr)
        return 2
    cfgs = parse_file(a.input_file) if a.input_file else [config_from_args(a)]
    print(HEADER)
    for cfg in cfgs:
        total, status = run_config(cfg, a.cache_mode.lower(), a.num_weight_buffers)
        print(row(cfg, total, status), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
