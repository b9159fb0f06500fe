"""CPU tests of the oracle: exact GEMM against numpy int64, the native-order epilogue against the
golden outputs of the reference's own INT8 tile kernel (bit-for-bit), and the other restated
formulas against independent numpy statements."""
import numpy as np
import pytest


def _cases(golden):
    i = 0
    while "c%d_meta" % i in golden:
        p = "c%d_" % i
        M, K, N, zp, fo, is_bf16, has_bias = [int(v) for v in golden[p + "meta"]]
        yield dict(A=golden[p + "A"], B=golden[p + "B"], ws=golden[p + "ws"], ss=float(golden[p + "ss"][0]),
                   bias=golden[p + "bias"] if has_bias else None, zp=zp, fo=fo,
                   dst="bf16" if is_bf16 else "f32", out=golden[p + "out"], M=M, K=K, N=N)
        i += 1


FUSED = {0: [], 1: ["relu"], 2: ["gelu_tanh"], 3: ["gelu_erf"], 4: ["sigmoid"], 5: ["swish"], 6: ["tanh"]}


def test_gemm_s32_exact(oracle):
    rng = np.random.default_rng(0)
    for M, K, N in [(1, 1, 1), (3, 5, 7), (17, 67, 33), (64, 1000, 48)]:
        A = rng.integers(0, 256, (M, K), dtype=np.uint8)
        B = rng.integers(-128, 128, (K, N), dtype=np.int8)
        ref = A.astype(np.int64) @ B.astype(np.int64)
        assert (oracle.gemm_s32(A, B) == ref).all()
        As = rng.integers(-128, 128, (M, K), dtype=np.int8)
        ref = As.astype(np.int64) @ B.astype(np.int64)
        assert (oracle.gemm_s32(As, B) == ref).all()
        assert (oracle.gemm_s32(As, np.ascontiguousarray(B.T), transB=True) == ref).all()


def test_gemm_s32_extremes(oracle):
    # largest magnitudes the configs reach stay exact (no float, no saturation)
    K = 11008
    A = np.full((2, K), -128, dtype=np.int8)
    B = np.full((K, 3), -128, dtype=np.int8)
    assert (oracle.gemm_s32(A, B) == 128 * 128 * K).all()
    Au = np.full((2, K), 255, dtype=np.uint8)
    assert (oracle.gemm_s32(Au, B) == -255 * 128 * K).all()


def test_native_order_matches_reference_golden(oracle, golden):
    """order=1 restates int8_brgemm_ukernel.cpp:91-129; fixtures are that kernel's outputs."""
    n = 0
    for c in _cases(golden):
        got = oracle.matmul_w8a8(c["A"], c["B"], c["dst"], src_scale=[c["ss"]], wei_scale=c["ws"], src_zp=c["zp"],
                                 bias=c["bias"], postops=FUSED[c["fo"]], order=1)
        if c["fo"] in (0, 1):
            assert (got == c["out"]).all(), "case M%d K%d N%d" % (c["M"], c["K"], c["N"])
        else:
            # the reference kernel uses polynomial tanh/sigmoid (~5e-5 relative)
            a = oracle.bf16_to_f32(got) if c["dst"] == "bf16" else got
            b = oracle.bf16_to_f32(c["out"]) if c["dst"] == "bf16" else c["out"]
            assert np.allclose(a, b, rtol=8e-3, atol=1e-4)
        n += 1
    assert n >= 8


def test_requested_order_within_one_ulp_of_reference(oracle, golden):
    """order=0 (exact s32 compensation, two multiplies) vs the reference kernel: <= 1 bf16 ulp."""
    for c in _cases(golden):
        if c["fo"] not in (0, 1):
            continue
        got = oracle.matmul_w8a8(c["A"], c["B"], c["dst"], src_scale=[c["ss"]], wei_scale=c["ws"], src_zp=c["zp"],
                                 bias=c["bias"], postops=FUSED[c["fo"]], order=0)
        if c["dst"] == "bf16":
            assert np.abs(got.astype(np.int32) - c["out"].astype(np.int32)).max() <= 1
        else:
            assert np.allclose(got, c["out"], rtol=1e-5, atol=1e-5)


def test_live_reference_kernel_if_present(oracle):
    if oracle.ref_lib() is None:
        pytest.skip("compiled reference kernel not available on this host")
    rng = np.random.default_rng(5)
    A = rng.integers(0, 256, (37, 200), dtype=np.uint8)
    B = rng.integers(-127, 128, (200, 64), dtype=np.int8)
    ws = rng.uniform(0.001, 0.01, 64).astype(np.float32)
    bias = rng.normal(size=64).astype(np.float32)
    ref = oracle.ref_int8_matmul(A, B, 128, 0.02, ws, bias, 1, "bf16")
    got = oracle.matmul_w8a8(A, B, "bf16", src_scale=[0.02], wei_scale=ws, src_zp=128, bias=bias, postops=["relu"], order=1)
    assert (ref == got).all()


def test_bf16_rne(oracle):
    x = np.array([1.0, 1.00390625, 1.005859375, -2.5, 3.1415927, 1e-30, 65504.0], dtype=np.float32)
    bits = oracle.f32_to_bf16(x)
    u = x.view(np.uint32).astype(np.uint64)
    exp = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    assert (bits == exp).all()
    assert (oracle.bf16_to_f32(bits).view(np.uint32) == (bits.astype(np.uint32) << 16)).all()


def test_quant_per_token(oracle):
    rng = np.random.default_rng(1)
    x = rng.normal(size=(9, 257)).astype(np.float32)
    x[3] = 0.0                      # all-zero row: scale clamps to 1e-10
    x[4, 5] = np.inf                # non-finite -> 0, ignored by absmax
    q, s = oracle.quant_per_token(x)
    fin = np.where(np.isfinite(x), np.abs(x), 0).max(axis=1)
    exp_s = np.maximum(np.maximum(fin, np.float32(1e-10)) / np.float32(127.0), np.float32(1e-10)).astype(np.float32)
    assert (s == exp_s).all()
    with np.errstate(invalid="ignore", over="ignore"):
        exp_q = np.where(np.isfinite(x), np.rint(x / exp_s[:, None]), 0).astype(np.int8)
    assert (q == exp_q).all()
    assert np.abs(q[np.isfinite(x)]).max() <= 127
    # bf16 input goes through f32
    xb = oracle.f32_to_bf16(x)
    qb, sb = oracle.quant_per_token(xb)
    q2, s2 = oracle.quant_per_token(oracle.bf16_to_f32(xb))
    assert (qb == q2).all() and (sb == s2).all()


def test_quant_weights_per_channel_roundtrip(oracle):
    rng = np.random.default_rng(2)
    w = (rng.normal(size=(300, 40)) * 0.02).astype(np.float32)
    q, s = oracle.quant_weights_per_channel(w)
    assert q.dtype == np.int8 and s.shape == (40,)
    assert (np.abs(q).max(axis=0) == 127).all()
    back = oracle.dequant_static(q, s)
    assert np.abs(back - w).max() <= s.max() * 0.5 + 1e-9


def test_gated_act_and_reduce(oracle):
    rng = np.random.default_rng(3)
    y = rng.normal(size=(5, 64)).astype(np.float32)
    z = oracle.gated_act(y, "silu_and_mul")
    g, u = y[:, :32], y[:, 32:]
    ref = (g * (1.0 / (1.0 + np.exp(-g.astype(np.float64))))).astype(np.float32) * u
    assert np.allclose(z, ref, rtol=1e-5, atol=1e-6)
    z3 = oracle.gated_act(y, "swiglu_oai_mul")
    g3, u3 = np.clip(y[:, 0::2], -7, 7), np.clip(y[:, 1::2], -7, 7)
    ref3 = (1 + u3) * g3 / (1 + np.exp(-1.702 * g3))
    assert np.allclose(z3, ref3, rtol=1e-5, atol=1e-6)
    rows = rng.normal(size=(12, 16)).astype(np.float32)
    w = rng.uniform(size=(4, 3)).astype(np.float32)
    out = oracle.moe_weighted_reduce(rows, w, 3)
    ref = (rows.reshape(4, 3, 16) * w[:, :, None]).sum(axis=1)
    assert np.allclose(out, ref, rtol=1e-5, atol=1e-6)


def test_router(oracle):
    rng = np.random.default_rng(4)
    l = rng.normal(size=(50, 8)).astype(np.float32)
    ids, w = oracle.router_topk(l, 2)
    p = np.exp(l - l.max(axis=1, keepdims=True))
    p /= p.sum(axis=1, keepdims=True)
    top = np.argsort(-p, axis=1, kind="stable")[:, :2]
    assert (ids == top).all()
    assert np.allclose(w.sum(axis=1), 1.0, atol=1e-6)


def test_fused_moe_flow_small(oracle):
    rng = np.random.default_rng(6)
    T, H, I, E, k = 24, 64, 32, 4, 2
    x = oracle.f32_to_bf16(rng.normal(size=(T, H)).astype(np.float32))
    ids, w = oracle.router_topk(rng.normal(size=(T, E)).astype(np.float32), k)
    w13, s13, w2, s2 = [], [], [], []
    for _ in range(E):
        q, s = oracle.quant_weights_per_channel((rng.normal(size=(H, 2 * I)) * 0.02).astype(np.float32))
        w13.append(q); s13.append(s)
        q, s = oracle.quant_weights_per_channel((rng.normal(size=(I, H)) * 0.02).astype(np.float32))
        w2.append(q); s2.append(s)
    out, _ = oracle.fused_moe(x, ids, w, w13, s13, w2, s2)
    out2, _ = oracle.fused_moe(x, ids, w, w13, s13, w2, s2, round_before_act=True)
    a, b = oracle.bf16_to_f32(out), oracle.bf16_to_f32(out2)
    assert np.abs(a).sum() > 1e-3            # anti-vacuity, as the reference's fused-MoE tests do
    assert np.allclose(a, b, rtol=0.05, atol=2e-3)


# ---- the reference's own quantisation, gated-activation and weighted-reduce code (tests/golden/make_golden_ref2.py)
ACTS = ["silu_and_mul", "gelu_and_mul", "swiglu_oai_mul"]


@pytest.fixture(scope="module")
def golden2():
    import os
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref2_cases.npz"))


def _as(oracle, a32, dt):
    return oracle.f32_to_bf16(a32) if dt == "bf16" else a32


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_quant_per_token_equals_reference_kernels(oracle, golden2, dt):
    """Scales and s8 values equal the reference's scalar kernel and its AVX-512 kernel bit for bit
    (rows with inf / nan entries and an all-zero row included)."""
    q, s = oracle.quant_per_token(_as(oracle, golden2["x32"], dt))
    for tag in ("scalar", "vec"):
        assert (s == golden2["quant_%s_%s_s" % (dt, tag)]).all(), tag
        assert (q == golden2["quant_%s_%s_q" % (dt, tag)]).all(), tag


@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("act", ACTS)
def test_gated_act_equals_reference_scalar_path(oracle, golden2, act, dt):
    """Bit-exact against the reference's scalar activation path; its AVX-512 path uses polynomial
    exponentials and stays within 2 bf16 ulp (relative 1e-4 in f32 away from cancellation)."""
    got = oracle.gated_act(_as(oracle, golden2["y32"], dt), act)
    assert (got == golden2["act_%s_%s_scalar" % (act, dt)]).all()
    vec = golden2["act_%s_%s_vec" % (act, dt)]
    if dt == "bf16":
        assert np.abs(got.astype(np.int32) - vec.astype(np.int32)).max() <= 2
    else:
        assert np.allclose(got, vec, rtol=2e-4, atol=2e-4)


@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("skip", [0, 1])
def test_weighted_reduce_equals_reference(oracle, golden2, dt, skip):
    """The oracle's fused form (multiply, then fused multiply-adds) is the reference's AVX-512 path, its unfused form
    the reference's scalar path: both bit for bit."""
    rows = _as(oracle, golden2["rows32"], dt)
    for tag, fused in (("vec", True), ("scalar", False)):
        got = oracle.moe_weighted_reduce(rows, golden2["w"], 3, skip_weighted=bool(skip), fused=fused)
        assert (got == golden2["reduce_%s_skip%d_%s" % (dt, skip, tag)]).all(), tag


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_dynamic_scales_and_static_quant_equal_reference(oracle, golden2, dt):
    """Per-channel / per-tensor dynamic scales (a column of zeros and an inf entry included), static quantise to s8 with
    per-channel scales and to u8 with a zero point, and dequantise: all bit for bit."""
    w = _as(oracle, golden2["w32"], dt)
    sc = oracle.dyn_scales(w, per_channel=True).astype(np.float32).reshape(-1)
    assert (sc == golden2["dyn_pc_" + dt]).all()
    assert (np.asarray(oracle.dyn_scales(w, per_channel=False)).reshape(-1) == golden2["dyn_pt_" + dt]).all()
    q = oracle.quant_static(w, sc.reshape(1, -1), None, "s8")
    assert (q == golden2["qs8_" + dt]).all()
    qu = oracle.quant_static(w, np.array([0.002], dtype=np.float32), np.array([13], dtype=np.int32), "u8")
    assert (qu == golden2["qu8_" + dt]).all()
    assert (oracle.dequant_static(q, sc.reshape(1, -1), None, dt) == golden2["deq_" + dt]).all()


def test_live_reference_quant_act_reduce_if_present(oracle):
    """Where oracle/_ref/libzendnn_ref2.so exists (built from a reference checkout) the same comparisons run live
    on fresh inputs."""
    if oracle.ref2_lib() is None:
        pytest.skip("libzendnn_ref2.so not built")
    rng = np.random.default_rng(5)
    x = oracle.f32_to_bf16((rng.normal(size=(9, 1000)) * 5).astype(np.float32))
    q, s = oracle.quant_per_token(x)
    for native in (False, True):
        r = oracle.ref2_quant_per_token(x, native=native)
        if r is not None:
            assert (r[0] == q).all() and (r[1] == s).all()
    rows = oracle.f32_to_bf16(rng.normal(size=(40, 200)).astype(np.float32))
    w = rng.uniform(0, 1, size=(10, 4)).astype(np.float32)
    assert (oracle.ref2_moe_reduce(rows, w, 4) == oracle.moe_weighted_reduce(rows, w, 4, fused=True)).all()
    y = oracle.f32_to_bf16((rng.normal(size=(8, 128)) * 2).astype(np.float32))
    for act in ACTS:
        d = np.abs(oracle.ref2_gated_act(y, act).astype(np.int32) - oracle.gated_act(y, act).astype(np.int32))
        assert d.max() <= 2


def _ukernel_inputs():
    # the same seeded inputs as tests/golden/make_golden_ref2.py::ukernel_inputs
    rng = np.random.default_rng(79)
    M, K, N = 21, 256, 128
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    B = rng.integers(-127, 128, (K, N), dtype=np.int8)
    sa = rng.uniform(0.01, 0.05, M).astype(np.float32)
    sw = rng.uniform(1e-4, 5e-4, N).astype(np.float32)
    bias = rng.normal(size=N).astype(np.float32)
    return A, B, sa, sw, bias


def _oracle_dq_int8(oracle, A, B, sa, sw, bias, act):
    """The oracle's statement of the group DQ-INT8 tile arithmetic: exact s32, x src scale, x weight scale, + bias
    (the order the GPU epilogues implement), then the gated activation on the f32 values, one rounding to bf16."""
    if act == "none":
        return oracle.matmul_w8a8(A, B, "bf16", src_scale=sa, wei_scale=sw, bias=bias)
    y = oracle.epilogue(oracle.gemm_s32(A, B), "f32", sa, sw, bias=bias)
    I = B.shape[1] // 2
    if act == "swiglu_oai_mul":
        return oracle.gated_act_f32_pairs(y[:, 0::2], y[:, 1::2], act)
    return oracle.gated_act_f32_pairs(y[:, :I], y[:, I:], act)


@pytest.mark.parametrize("act", ["none", "silu_and_mul", "gelu_and_mul", "swiglu_oai_mul"])
@pytest.mark.parametrize("has_bias", [0, 1])
def test_dq_int8_tile_arithmetic_equals_reference_microkernel(oracle, golden2, act, has_bias):
    """Outputs of the reference's own DQ-INT8 micro-kernel (matmul/group_matmul/custom_kernel/ukernel/int8_microkernel.cpp,
    driven by oracle/ref_driver2.cpp): the dequantisation order (exact s32 compensation, two multiplies, bias) is equal
    bit for bit; the gated forms, which the reference evaluates with polynomial exponentials, within 1 bf16 ulp
    (its gelu_and_mul is the tanh form, |gelu_tanh - gelu_erf| <= 1.5e-3: 2 ulp there)."""
    A, B, sa, sw, bias = _ukernel_inputs()
    ref = golden2["uk_%s_bias%d" % (act, has_bias)]
    got = _oracle_dq_int8(oracle, A, B, sa, sw, bias if has_bias else None, act)
    d = np.abs(got.astype(np.int32) - ref.astype(np.int32))
    if act == "none":
        assert d.max() == 0
    else:
        assert d.max() <= (2 if act == "gelu_and_mul" else 1)
        assert (d == 0).mean() > 0.99


def test_live_reference_microkernel_if_present(oracle):
    if oracle.ref2_lib() is None or oracle.ref2_int8_ukernel(*_ukernel_inputs()[:4]) is None:
        pytest.skip("reference micro-kernel not built or no AVX-512 VNNI on this host")
    rng = np.random.default_rng(11)
    M, K, N = 37, 512, 192
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    B = rng.integers(-127, 128, (K, N), dtype=np.int8)
    sa = rng.uniform(0.01, 0.05, M).astype(np.float32)
    sw = rng.uniform(1e-4, 5e-4, N).astype(np.float32)
    bias = rng.normal(size=N).astype(np.float32)
    assert (oracle.ref2_int8_ukernel(A, B, sa, sw, bias, "none") == _oracle_dq_int8(oracle, A, B, sa, sw, bias, "none")).all()
    ref = oracle.ref2_int8_ukernel(A, B, sa, sw, None, "silu_and_mul")
    got = _oracle_dq_int8(oracle, A, B, sa, sw, None, "silu_and_mul")
    assert np.abs(ref.astype(np.int32) - got.astype(np.int32)).max() <= 1


def _oracle_bf16_tile(oracle, A, B, bias, act):
    if act == "none":
        return oracle.matmul_bf16(A, B, "bf16", bias=bias)
    y = oracle.matmul_bf16(A, B, "f32", bias=bias)
    I = B.shape[1] // 2
    if act == "swiglu_oai_mul":
        return oracle.gated_act_f32_pairs(y[:, 0::2], y[:, 1::2], act)
    return oracle.gated_act_f32_pairs(y[:, :I], y[:, I:], act)


@pytest.mark.parametrize("act", ["none", "silu_and_mul", "gelu_and_mul", "swiglu_oai_mul"])
@pytest.mark.parametrize("has_bias", [0, 1])
def test_bf16_tile_arithmetic_against_reference_microkernel(oracle, golden2, act, has_bias):
    """Outputs of the reference's own bf16 micro-kernel (matmul/group_matmul/custom_kernel/ukernel/bf16_microkernel.cpp, driven
    by oracle/ref_driver2.cpp) against the oracle's bf16 GEMM (exact products summed in double) and gated activation on the
    f32 values.  The kernel sums in f32 in its own order and evaluates the activations with polynomial exponentials: at
    least 99 % of the elements are equal, none is further than 2 bf16 ulp."""
    from helpers import bf16_ulp_diff
    rng = np.random.default_rng(80)             # the same seeded inputs as tests/golden/make_golden_ref2.py::ukernel_bf16_inputs
    M, K, N = 21, 256, 128
    A = oracle.f32_to_bf16(rng.normal(size=(M, K)).astype(np.float32))
    B = oracle.f32_to_bf16((rng.normal(size=(K, N)) * 0.06).astype(np.float32))
    bias = rng.normal(size=N).astype(np.float32)
    ref = golden2["ukbf_%s_bias%d" % (act, has_bias)]
    got = _oracle_bf16_tile(oracle, A, B, bias if has_bias else None, act)
    d = bf16_ulp_diff(got, ref)
    assert d.max() <= 2 and (d == 0).mean() > 0.99, (int(d.max()), float((d == 0).mean()))


def _norm_inputs():
    # the same seeded inputs as tests/golden/make_golden_ref2.py::norm_inputs
    rng = np.random.default_rng(81)
    x = (rng.normal(size=(7, 300)) * 3 + 0.5).astype(np.float32)
    x[2] *= 100.0
    x[4] = 0.0
    gamma = rng.normal(size=300).astype(np.float32)
    beta = rng.normal(size=300).astype(np.float32)
    res = rng.normal(size=(7, 300)).astype(np.float32)
    xb = rng.normal(size=(3, 5, 11)).astype(np.float32)
    rm = rng.normal(size=5).astype(np.float32)
    rv = rng.uniform(0.5, 2.0, 5).astype(np.float32)
    return x, gamma, beta, res, xb, rm, rv


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_normalization_equals_reference_scalar_kernel(oracle, golden2, dt):
    """Outputs of the reference's own scalar normalization kernel (lowoha_operators/normalization/kernel/reference_kernel.cpp,
    driven by oracle/ref_driver2.cpp): LayerNorm with and without gamma / beta, RMSNorm, fused-add RMSNorm (output and the
    residual it updates in place) and BatchNorm, f32 and bf16 buffers: bit for bit."""
    x, gamma, beta, res, xb, rm, rv = _norm_inputs()
    cv = (lambda a: oracle.f32_to_bf16(a)) if dt == "bf16" else (lambda a: a)
    assert (oracle.normalization("layer_norm", cv(x), gamma, beta) == golden2["norm_layer_%s" % dt]).all()
    assert (oracle.normalization("layer_norm", cv(x)) == golden2["norm_layer_noaffine_%s" % dt]).all()
    assert (oracle.normalization("rms_norm", cv(x), gamma) == golden2["norm_rms_%s" % dt]).all()
    o, r = oracle.normalization("fused_add_rms_norm", cv(x), gamma, residual=cv(res))
    assert (o == golden2["norm_fused_%s" % dt]).all() and (r == golden2["norm_fused_res_%s" % dt]).all()
    got = oracle.normalization("batch_norm", cv(xb), gamma[:5], beta[:5], running_mean=rm, running_var=rv)
    assert (got == golden2["norm_batch_%s" % dt]).all()


def test_group_scaled_oracle_reduces_to_the_per_token_form(oracle):
    """With one group the per-group definition (operators/matmul/matmul_ref_kernel.cpp:961-1003) is the per-token
    epilogue order that the golden reference cases pin: (acc * src_scale[m]) * wei_scale[n] + bias."""
    rng = np.random.default_rng(0)
    M, K, N = 9, 96, 40
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    B = rng.integers(-128, 128, (K, N), dtype=np.int8)
    sa = rng.uniform(0.01, 0.05, M).astype(np.float32)
    sw = rng.uniform(1e-3, 5e-3, N).astype(np.float32)
    bias = rng.normal(size=N).astype(np.float32)
    for dst in ("bf16", "f32"):
        a = oracle.matmul_w8a8(A, B, dst, src_scale=sa, wei_scale=sw, bias=bias, postops=["gelu_tanh"])
        b = oracle.matmul_group_scaled(A, B, sa, sw[None, :], dst, bias=bias, postops=["gelu_tanh"])
        assert (a == b).all()
    # several groups: the same sums written with numpy, one f32 rounding per operation, groups in order
    G = 4
    sag = rng.uniform(0.01, 0.05, (M, G)).astype(np.float32)
    swg = rng.uniform(1e-3, 5e-3, (G, N)).astype(np.float32)
    ref = np.zeros((M, N), np.float32)
    for g in range(G):
        ks = slice(g * K // G, (g + 1) * K // G)
        acc = (A[:, ks].astype(np.int32) @ B[ks].astype(np.int32)).astype(np.float32)
        ref = ref + (acc * sag[:, g:g + 1]) * swg[g][None, :]
    assert (oracle.matmul_group_scaled(A, B, sag, swg, "f32") == ref).all()
    # a per-token source scale is the same scale in every group
    assert (oracle.matmul_group_scaled(A, B, sa, swg, "f32") ==
            oracle.matmul_group_scaled(A, B, np.repeat(sa[:, None], G, 1), swg, "f32")).all()


def test_s4_packing_follows_the_reference_index_rule(oracle):
    """Element (k,n) at physical index k*ldb+n (transB: n*ldb+k), even index in the low nibble, sign-extended on the way
    out (matmul/backends/aocl/aocl_kernel.cpp:33-42,145-160)."""
    W = np.array([[-8, 7, 1], [2, -1, 0], [3, -3, 5], [-7, 6, -2]], dtype=np.int8)     # K=4, N=3
    p = oracle.pack_s4(W)
    assert p[0] == ((7 & 0xF) << 4 | (-8 & 0xF)) and p[1] == ((2 & 0xF) << 4 | 1)
    assert (oracle.unpack_s4(p, 4, 3) == W).all()
    pt = oracle.pack_s4(W, transB=True)
    assert pt[0] == ((2 & 0xF) << 4 | (-8 & 0xF))
    assert (oracle.unpack_s4(pt, 4, 3, transB=True) == W).all()
    rng = np.random.default_rng(1)
    W = rng.integers(-8, 8, (64, 24), dtype=np.int8)
    assert (oracle.unpack_s4(oracle.pack_s4(W, ldb=30), 64, 24, ldb=30) == W).all()


def test_per_group_dynamic_quant_is_the_per_token_rule_on_each_group(oracle):
    rng = np.random.default_rng(2)
    x = oracle.f32_to_bf16(rng.normal(size=(6, 128)).astype(np.float32))
    q, s = oracle.quant_per_group(x, 4)
    for g in range(4):
        qg, sg = oracle.quant_per_token(np.ascontiguousarray(x[:, g * 32:(g + 1) * 32]))
        assert (q[:, g * 32:(g + 1) * 32] == qg).all() and (s[:, g] == sg).all()


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_per_group_dynamic_quant_equals_reference_kernel(oracle, golden2, dt):
    """The oracle's per-group quantisation against the reference's AVX-512 per-group kernel
    (reorder/reorder_data_type/dynamic_quant_impl/per_group_avx512_f32_fma_kernel.cpp), rows with inf / nan and an all-zero
    row included: scales and s8 codes bit for bit."""
    x = _as(oracle, golden2["x32"], dt)
    seen = 0
    for G in (2, 4, 8, 16):
        if "pg_%s_G%d_q" % (dt, G) not in golden2.files:
            continue
        q, s = oracle.quant_per_group(x, G)
        assert (s == golden2["pg_%s_G%d_s" % (dt, G)]).all(), G
        assert (q == golden2["pg_%s_G%d_q" % (dt, G)]).all(), G
        seen += 1
    assert seen >= 3


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_asymmetric_per_token_quant_equals_reference_kernels(oracle, golden2, dt):
    """u8 codes, f32 scales and s32 zero points equal the reference's scalar kernel and its AVX-512 kernel bit for bit
    (reorder/reorder_data_type/scalar_impl/dynamic_per_token_ref_kernel.cpp:38-56,128-183; rows with inf / nan entries and
    an all-zero row included)."""
    q, s, z = oracle.quant_per_token_asym(_as(oracle, golden2["x32"], dt))
    for tag in ("scalar", "vec"):
        assert (s == golden2["quantu8_%s_%s_s" % (dt, tag)]).all(), tag
        assert (z == golden2["quantu8_%s_%s_z" % (dt, tag)]).all(), tag
        assert (q == golden2["quantu8_%s_%s_q" % (dt, tag)]).all(), tag
