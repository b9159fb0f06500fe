"""GPU parity tests of the bf16 x bf16 form of b200dnn_matmul (matmul_direct with dtypes bf16:bf16:bf16|f32, the
reference's non-quantised path and the dtype of its MoE traces) against the CPU oracle, which sums the exact bf16
products in double.  Tolerance, stated per element: the f32 sum may differ from the exact one by the accumulation
error of the tensor core, bounded here by 2^-17 * sum_k |a||b| (the reference's own gtests allow K * 9.76e-4 + 1e-2*|ref|,
zendnnl/gtests/Readme.md "Tolerance Calculation"); a bf16 destination adds its rounding, 2^-8 * |ref|."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    from zendnn_b200 import capi as c
    assert c.lib.b200dnn_device_count() > 0, "no CUDA device"
    return c


@pytest.fixture(scope="module")
def golden2():
    import os
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref2_cases.npz"))


def make(oracle, rng, M, K, N, transB=False, wstd=1.0):
    A = oracle.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    W = oracle.f32_to_bf16((rng.standard_normal((N, K) if transB else (K, N)) * wstd).astype(np.float32))
    return A, W


def abs_dot(oracle, A, W, transB):
    a = np.abs(oracle.bf16_to_f32(A)).astype(np.float64)
    w = np.abs(oracle.bf16_to_f32(W)).astype(np.float64)
    return a @ (w.T if transB else w)


def run(capi, M, N, K, A, W, dst_dt, **kw):
    out = np.zeros((M, N), dtype={"bf16": np.uint16, "f32": np.float32}[dst_dt])
    d = capi.make_matmul(M, N, K, A, W, out, src_dt=capi.DT["bf16"], wei_dt=capi.DT["bf16"], dst_dt=capi.DT[dst_dt], **kw)
    st = capi.matmul(d)
    assert st == capi.SUCCESS, capi.last_error()
    return out


def check(oracle, got, ref_f32, bound, dst_dt, what):
    g = oracle.bf16_to_f32(got) if dst_dt == "bf16" else got
    tol = bound * 2.0 ** -17 + (np.abs(ref_f32) * 2.0 ** -8 if dst_dt == "bf16" else 0.0) + 1e-30
    err = np.abs(g.astype(np.float64) - ref_f32)
    assert (err <= tol).all(), "%s: %d of %d outside the bound, worst err/bound %.3g" % (
        what, int((err > tol).sum()), err.size, float((err / tol).max()))


SHAPES = [(1, 64, 16), (5, 100, 24), (16, 256, 64), (33, 260, 80), (130, 384, 200), (257, 1024, 264), (300, 4096, 1024)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dst", ["bf16", "f32"])
def test_plain_gemm(capi, oracle, shape, dst):
    M, K, N = shape
    rng = np.random.default_rng(M * 7 + K)
    for transB in (False, True):
        A, W = make(oracle, rng, M, K, N, transB)
        ref = oracle.matmul_bf16(A, W, "f32", transB=transB).astype(np.float64)
        got = run(capi, M, N, K, A, W, dst, weights_const=False, transB=transB)
        check(oracle, got, ref, abs_dot(oracle, A, W, transB), dst, "%s transB=%d" % (shape, transB))


@pytest.mark.parametrize("has_bias", [0, 1])
def test_against_reference_microkernel_outputs(capi, oracle, golden2, has_bias):
    """The committed outputs of the reference's own bf16 micro-kernel (tests/golden, generated from the compiled reference
    by tests/golden/make_golden_ref2.py): it sums in f32 in its own order, so at least 99 % of the elements are equal and none
    is further than 2 bf16 ulp, except where the sum nearly cancels (there: within 2^-16 * sum_k |a||b|)."""
    from helpers import bf16_ulp_diff
    rng = np.random.default_rng(80)             # the inputs of make_golden_ref2.py::ukernel_bf16_inputs
    M, K, N = 21, 256, 128
    A = oracle.f32_to_bf16(rng.normal(size=(M, K)).astype(np.float32))
    B = oracle.f32_to_bf16((rng.normal(size=(K, N)) * 0.06).astype(np.float32))
    bias = rng.normal(size=N).astype(np.float32)
    got = run(capi, M, N, K, A, B, "bf16", weights_const=False, bias=bias if has_bias else None)
    ref = golden2["ukbf_none_bias%d" % has_bias]
    d = bf16_ulp_diff(got, ref)
    # a result that nearly cancels carries both kernels' f32 accumulation errors: those elements are held to the stated bound
    near = np.abs(oracle.bf16_to_f32(got).astype(np.float64) - oracle.bf16_to_f32(ref)) <= 2.0 ** -16 * abs_dot(oracle, A, B, False)
    assert ((d <= 2) | near).all() and (d == 0).mean() > 0.99, (int(d.max()), float((d == 0).mean()))


@pytest.mark.parametrize("splits", [2, 3, 4])
def test_split_form(capi, oracle, monkeypatch, splits):
    """Clusters of 2-4 CTAs share one tile's K blocks and add their f32 partial sums in a fixed order (small-M GEMMs whose
    tiles do not fill the GPU): same tolerance as the unsplit kernel, and the same bytes on every call."""
    monkeypatch.setenv("B200DNN_TC_KSPLIT", str(splits))
    rng = np.random.default_rng(40 + splits)
    for M, K, N in [(16, 4096, 512), (128, 2048, 384), (200, 1100, 264)]:
        A, W = make(oracle, rng, M, K, N, wstd=0.05)
        bias = rng.standard_normal(N).astype(np.float32)
        ref = oracle.matmul_bf16(A, W, "f32", bias=bias).astype(np.float64)
        got = run(capi, M, N, K, A, W, "f32", weights_const=False, bias=bias)
        check(oracle, got, ref, abs_dot(oracle, A, W, False) + 1.0, "f32", "splits=%d %s" % (splits, (M, K, N)))
        again = run(capi, M, N, K, A, W, "f32", weights_const=False, bias=bias)
        assert (again == got).all()


@pytest.mark.parametrize("pair", [0, 1])
def test_pair_form_and_bias(capi, oracle, monkeypatch, pair):
    """Both tile forms (one CTA per 128-row tile, two CTAs per 256-row tile), f32 and bf16 bias."""
    monkeypatch.setenv("B200DNN_TC_PAIR", str(pair))
    rng = np.random.default_rng(3 + pair)
    for M, K, N in [(512, 512, 768), (700, 1000, 520)]:
        A, W = make(oracle, rng, M, K, N, wstd=0.05)
        for bias in (rng.standard_normal(N).astype(np.float32), oracle.f32_to_bf16(rng.standard_normal(N).astype(np.float32))):
            ref = oracle.matmul_bf16(A, W, "f32", bias=bias).astype(np.float64)
            got = run(capi, M, N, K, A, W, "bf16", weights_const=False, bias=bias)
            check(oracle, got, ref, abs_dot(oracle, A, W, False) + 1.0, "bf16", "pair=%d %s" % (pair, (M, K, N)))


@pytest.mark.parametrize("name", ["relu", "gelu_tanh", "gelu_erf", "sigmoid", "swish", "tanh", "elu", "leaky_relu", "mish"])
def test_eltwise_postops(capi, oracle, name):
    from helpers import assert_bf16_close
    rng = np.random.default_rng(11)
    M, K, N = 150, 256, 136
    A, W = make(oracle, rng, M, K, N, wstd=0.08)
    bias = rng.standard_normal(N).astype(np.float32)
    po = [dict(type=name, alpha=1.0)] if name == "elu" else [name]
    ref = oracle.matmul_bf16(A, W, "bf16", bias=bias, postops=po)
    got = run(capi, M, N, K, A, W, "bf16", weights_const=False, bias=bias, postops=po)
    assert_bf16_close(got, ref, 1, name, atol=2e-4)


def test_postop_chain_strides_and_cache(capi, oracle):
    from helpers import assert_bf16_close
    rng = np.random.default_rng(12)
    M, K, N, lda, ldc = 70, 192, 72, 200, 96
    Afull = oracle.f32_to_bf16(rng.standard_normal((M, lda)).astype(np.float32))
    A = np.ascontiguousarray(Afull[:, :K])
    W = oracle.f32_to_bf16((rng.standard_normal((K, N)) * 0.1).astype(np.float32))
    add = rng.normal(size=(1, N)).astype(np.float32)
    mul = rng.normal(size=(M, N)).astype(np.float32)
    po = [dict(type="binary_add", buff=add), "swish", dict(type="binary_mul", buff=mul), dict(type="clip", alpha=-0.5, beta=0.75)]
    ref = oracle.matmul_bf16(A, W, "bf16", postops=po)
    out = np.full((M, ldc), 0x4040, dtype=np.uint16)
    d = capi.make_matmul(M, N, K, Afull, W, out, src_dt=capi.DT["bf16"], wei_dt=capi.DT["bf16"], dst_dt=capi.DT["bf16"],
                         lda=lda, ldc=ldc, weights_const=True, postops=po)
    for _ in range(2):                         # the second call takes the cached pack
        out[:] = 0x4040
        assert capi.matmul(d) == capi.SUCCESS, capi.last_error()
        assert_bf16_close(out[:, :N], ref, 1, "chain", atol=2e-4)
        assert (out[:, N:] == 0x4040).all()


def test_contract(capi):
    M, K, N = 8, 64, 32
    A = np.zeros((M, K), dtype=np.uint16); W = np.zeros((K, N), dtype=np.uint16); out = np.zeros((M, N), dtype=np.uint16)
    bf = capi.DT["bf16"]
    one = np.ones(1, dtype=np.float32)
    d = capi.make_matmul(M, N, K, A, W, out, src_dt=bf, wei_dt=bf, dst_dt=bf, src_scale=one)
    assert capi.matmul(d) == capi.FAILURE and "only supported for INT8" in capi.last_error()
    d = capi.make_matmul(M, N, K, A, W, out, src_dt=bf, wei_dt=bf, dst_dt=capi.DT["s32"])
    assert capi.matmul(d) == capi.UNIMPLEMENTED
    d = capi.make_matmul(M, N, K, A, W, out, src_dt=bf, wei_dt=bf, dst_dt=bf, lda=K - 1)
    assert capi.matmul(d) == capi.FAILURE


# ---------------------------------------------------------------------------------- fused MoE, bf16 weights
def _bf16_experts(oracle, rng, E, H, I):
    w13 = [oracle.f32_to_bf16((rng.normal(size=(H, 2 * I)) * 0.05).astype(np.float32)) for _ in range(E)]
    w2 = [oracle.f32_to_bf16((rng.normal(size=(I, H)) * 0.05).astype(np.float32)) for _ in range(E)]
    return w13, w2


def _close(oracle, got, ref, what):
    """bf16 results of a chain of two GEMMs: a one-ulp difference of an intermediate Z element (its f32 value sits on a
    rounding boundary) moves a down-projection output by up to 2^-8 |z||w|; accepted: 2 bf16 ulp or 0.4 % of the row maximum."""
    from helpers import assert_bf16_close
    assert_bf16_close(got, ref, 2, what, row_atol_frac=4e-3)


@pytest.mark.parametrize("T,H,I,E,k,act", [(48, 128, 64, 4, 2, "silu_and_mul"), (300, 256, 160, 6, 2, "silu_and_mul"),
                                           (64, 136, 96, 3, 1, "gelu_and_mul"), (64, 128, 64, 4, 2, "swiglu_oai_mul")])
@pytest.mark.parametrize("pair", ["0", "1"])
def test_fused_moe_bf16_reference_contract(capi, oracle, monkeypatch, pair, T, H, I, E, k, act):
    """group_matmul_direct in fused-MoE mode with bf16:bf16:bf16 experts: rows gathered by the caller, per-expert dst_down,
    the activated first-GEMM output in dst_op1, row_ptrs + top-k weights."""
    monkeypatch.setenv("B200DNN_TC_PAIR", pair)
    rng = np.random.default_rng(T + I)
    x = oracle.f32_to_bf16(rng.normal(size=(T, H)).astype(np.float32))
    logits = rng.normal(size=(T, E)).astype(np.float32)
    logits[:, 1] = -1e4                      # expert 1 receives no token
    ids, w = oracle.router_topk(logits, k)
    w13, w2 = _bf16_experts(oracle, rng, E, H, I)
    b13 = [rng.normal(size=2 * I).astype(np.float32) * 0.2 for _ in range(E)]
    out_ref, slot_ref, z_ref = oracle.fused_moe_bf16(x, ids, w, w13, w2, act, b13=b13)
    flat = ids.reshape(-1)
    keep, dsts, zs, experts = [], [], [], (capi.MoeExpert * E)()
    ptrs = (C.c_void_p * (T * k))()
    for e in range(E):
        slots = np.nonzero(flat == e)[0]
        src = np.ascontiguousarray(x[slots // k]) if slots.size else np.zeros((1, H), dtype=np.uint16)
        dst = np.zeros((max(slots.size, 1), H), dtype=np.uint16)
        z = np.zeros((max(slots.size, 1), I), dtype=np.uint16)
        keep.append(src); dsts.append(dst); zs.append(z)
        ex = experts[e]
        ex.M = int(slots.size); ex.wei_dt = capi.DT["bf16"]; ex.src = src.ctypes.data; ex.lda = H
        ex.w13 = w13[e].ctypes.data; ex.ldb13 = 2 * I
        ex.w2 = w2[e].ctypes.data; ex.ldb2 = H
        ex.bias13 = b13[e].ctypes.data; ex.bias13_dt = capi.DT["f32"]
        ex.dst_down = dst.ctypes.data; ex.ldc_down = H
        ex.dst_op1 = z.ctypes.data; ex.ldc_op1 = I
        for r, s in enumerate(slots):
            ptrs[int(s)] = dst.ctypes.data + r * dst.strides[0]
    out = np.zeros((T, H), dtype=np.uint16)
    st = capi.lib.b200dnn_fused_moe(E, experts, H, I, H, 0, capi.ACT[act], 0, ptrs, capi.ptr(w), T, k, capi.ptr(out), H, None)
    assert st == capi.SUCCESS, capi.last_error()
    assert np.abs(oracle.bf16_to_f32(out)).sum() > 1e-3
    from helpers import assert_bf16_close
    for e in range(E):
        slots = np.nonzero(flat == e)[0]
        if slots.size:
            assert_bf16_close(zs[e][:slots.size], z_ref[slots], 1, "expert %d activated output" % e, atol=1e-4)
            _close(oracle, dsts[e][:slots.size], slot_ref[slots], "expert %d down output" % e)
    _close(oracle, out, out_ref, "moe output")
    capi.lib.b200dnn_clear_caches()


@pytest.mark.parametrize("T,H,I,E,k,S", [(256, 256, 128, 8, 2, 0), (512, 128, 96, 16, 4, 2), (1500, 256, 320, 4, 2, 1)])
def test_moe_layer_bf16_end_to_end(capi, oracle, T, H, I, E, k, S):
    """Router + permutation + bf16 fused MoE + un-permute on the device; shared experts see every token with weight 1."""
    rng = np.random.default_rng(E)
    x = oracle.f32_to_bf16(rng.normal(size=(T, H)).astype(np.float32))
    skew = np.log(np.arange(1, E + 1, dtype=np.float64) ** -1.1)
    logits = (rng.normal(size=(T, E)) + rng.permutation(skew)).astype(np.float32)
    w13, w2 = _bf16_experts(oracle, rng, E + S, H, I)
    b2 = [rng.normal(size=H).astype(np.float32) * 0.2 for _ in range(E + S)]
    ids, w = oracle.router_topk(logits, k)
    ids_all = np.concatenate([ids, np.tile(np.arange(E, E + S, dtype=np.int32), (T, 1))], axis=1)
    w_all = np.concatenate([w, np.ones((T, S), dtype=np.float32)], axis=1)
    out_ref, _, _ = oracle.fused_moe_bf16(x, ids_all, w_all, w13, w2, b2=b2)
    experts = (capi.MoeExpert * (E + S))()
    for e in range(E + S):
        ex = experts[e]
        ex.wei_dt = capi.DT["bf16"]
        ex.w13 = w13[e].ctypes.data; ex.ldb13 = 2 * I
        ex.w2 = w2[e].ctypes.data; ex.ldb2 = H
        ex.bias2 = b2[e].ctypes.data; ex.bias2_dt = capi.DT["f32"]
    out = np.zeros((T, H), dtype=np.uint16)
    st = capi.lib.b200dnn_moe_layer(capi.ptr(x), H, capi.ptr(logits), T, E, S, k, experts, H, I, H, 0, capi.ACT["silu_and_mul"],
                                    capi.ptr(out), H, None)
    assert st == capi.SUCCESS, capi.last_error()
    assert np.abs(oracle.bf16_to_f32(out)).sum() > 1e-3
    _close(oracle, out, out_ref, "moe layer")
    capi.lib.b200dnn_clear_caches()


# ---------------------------------------------------------------------------------- weight-only quantisation (s4 | u4)
@pytest.mark.parametrize("wei_dt,zp_kind", [("s4", None), ("u4", "s8"), ("u4", "bf16")])
@pytest.mark.parametrize("gran", ["tensor", "channel", "group"])
def test_weight_only_quantisation(capi, oracle, wei_dt, zp_kind, gran):
    """bf16 activations x packed 4-bit weights, no dynamic quantisation (TestMatmul WOQ cases of the reference,
    zendnnl/gtests/test_matmul.cpp:137 ff.): per-tensor, per-channel and per-group ({G,N}) scales in f32 or bf16 storage,
    u4 with an s8 or a bf16 zero point.  Against the reference's scalar definition: dequantise to bf16, then bf16 x bf16."""
    from helpers import assert_bf16_close
    rng = np.random.default_rng(sum(map(ord, wei_dt + str(zp_kind) + gran)))
    for M, K, N, gs, transB in [(40, 256, 136, 64, False), (200, 512, 264, 128, True)]:
        G = K // gs
        n_s = {"tensor": 1, "channel": N, "group": G * N}[gran]
        A = oracle.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
        if wei_dt == "s4":
            packed = oracle.pack_s4(rng.integers(-8, 8, (K, N), dtype=np.int8), transB)
        else:
            packed = oracle.pack_u4(rng.integers(0, 16, (K, N), dtype=np.uint8), transB)
        scale = rng.uniform(0.005, 0.02, n_s).astype(np.float32)
        if transB:
            scale = oracle.f32_to_bf16(scale)            # scales in bf16 storage
        zp = None
        if zp_kind == "s8":
            zp = rng.integers(5, 11, n_s, dtype=np.int8)
        elif zp_kind == "bf16":
            zp = oracle.f32_to_bf16(rng.uniform(-0.02, 0.02, n_s).astype(np.float32))
        bias = rng.standard_normal(N).astype(np.float32)
        ref = oracle.matmul_woq(A, packed, K, N, wei_dt, scale, zp, "bf16", transB=transB, bias=bias, postops=["gelu_tanh"])
        out = np.zeros((M, N), dtype=np.uint16)
        d = capi.make_matmul(M, N, K, A, packed, out, src_dt=capi.DT["bf16"], wei_dt=capi.DT[wei_dt], dst_dt=capi.DT["bf16"],
                             transB=transB, ldb=K if transB else N, weights_const=True, bias=bias, postops=["gelu_tanh"],
                             wei_scale=capi.quant(scale, count=n_s), wei_zp=None if zp is None else capi.quant(zp, count=n_s))
        for _ in range(2):                      # the second call takes the cached pack
            out[:] = 0
            assert capi.matmul(d) == capi.SUCCESS, capi.last_error()
            assert_bf16_close(out, ref, 1, "%s %s %s %s" % (wei_dt, zp_kind, gran, (M, K, N)), atol=2e-4)
    capi.lib.b200dnn_clear_caches()


def test_weight_only_quantisation_contract(capi, oracle):
    M, K, N = 8, 64, 32
    A = np.zeros((M, K), dtype=np.uint16); W4 = np.zeros(K * N // 2, dtype=np.uint8); out = np.zeros((M, N), dtype=np.uint16)
    bf, sc = capi.DT["bf16"], np.ones(N, dtype=np.float32)

    def mk(**kw):
        args = dict(src_dt=bf, wei_dt=capi.DT["s4"], dst_dt=bf, weights_const=True, wei_scale=sc)
        args.update(kw)
        return capi.make_matmul(M, N, K, A, W4, out, **args)
    assert capi.matmul(mk()) == capi.SUCCESS, capi.last_error()
    assert capi.matmul(mk(weights_const=False)) == capi.FAILURE and "constant weights" in capi.last_error()
    assert capi.matmul(mk(wei_scale=None)) == capi.FAILURE
    assert capi.matmul(mk(wei_dt=capi.DT["u4"])) == capi.FAILURE and "mandatory" in capi.last_error()
    assert capi.matmul(mk(wei_dt=capi.DT["u4"], wei_zp=np.zeros(N, dtype=np.float32))) == capi.FAILURE      # zero point must be s8 or bf16
    assert capi.matmul(mk(wei_scale=capi.quant(np.ones(3 * N, dtype=np.float32), count=3 * N))) == capi.FAILURE   # K % G != 0
    capi.lib.b200dnn_clear_caches()


# ---------------------------------------------------------------------------------- group_matmul_direct, plain mode, bf16 experts
def test_group_matmul_bf16_one_grouped_launch(capi, oracle, monkeypatch):
    """Plain (parallel) mode of group_matmul_direct with bf16 x bf16 experts of one shape: one grouped launch whose results are
    those of separate matmul calls (identical bytes), checked against the oracle per expert, with ragged and empty experts, a
    bias on some experts only and padded destinations."""
    from helpers import assert_bf16_close
    rng = np.random.default_rng(23)
    Ms, K, N, ldc = [200, 0, 37, 130, 1, 300], 264, 392, 400
    bf = capi.DT["bf16"]
    descs = (capi.MatmulDesc * len(Ms))()
    keep, outs, refs = [], [], []
    for g, M in enumerate(Ms):
        A = oracle.f32_to_bf16(rng.standard_normal((max(M, 1), K)).astype(np.float32))
        W = oracle.f32_to_bf16((rng.standard_normal((K, N)) * 0.06).astype(np.float32))
        bias = rng.standard_normal(N).astype(np.float32) if g % 2 == 0 else None
        out = np.zeros((max(M, 1), ldc), dtype=np.uint16)
        keep.append((A, W, bias)); outs.append(out)
        descs[g] = capi.make_matmul(M, N, K, A, W, out, src_dt=bf, wei_dt=bf, dst_dt=bf, ldc=ldc, bias=bias, postops=["swish"],
                                    weights_const=True)
        refs.append(oracle.matmul_bf16(A[:M], W, "bf16", bias=bias, postops=["swish"]) if M else None)
    capi.check(capi.lib.b200dnn_group_matmul(len(Ms), descs, None))          # packs the weights
    for o in outs:
        o[:] = 0
    n0 = capi.lib.b200dnn_launch_count()
    capi.check(capi.lib.b200dnn_group_matmul(len(Ms), descs, None))
    assert capi.lib.b200dnn_launch_count() - n0 == 1, "expected one grouped launch"
    grouped = [o.copy() for o in outs]
    for g, M in enumerate(Ms):
        if not M:
            assert not outs[g].any()
            continue
        assert_bf16_close(outs[g][:M, :N], refs[g], 1, "expert %d" % g, atol=2e-4)
        assert not outs[g][:, N:].any(), "padding columns of expert %d were written" % g
    monkeypatch.setenv("B200DNN_GROUPED_PLAIN", "0")
    for o in outs:
        o[:] = 0
    capi.check(capi.lib.b200dnn_group_matmul(len(Ms), descs, None))
    for g in range(len(Ms)):
        assert (outs[g] == grouped[g]).all(), "expert %d: grouped and separate calls differ" % g
    capi.lib.b200dnn_clear_caches()
