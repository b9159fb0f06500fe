"""GPU parity of the group-scaled INT8 matmul_direct forms against the CPU oracle: per-group source x weight scales
({M,G} x {G,N}; the reference's TestMatmul.INT8_SYM_QUANT_PER_GROUP_*, zendnnl/gtests/test_matmul.cpp:1049 ff.) and W4A8
(packed s4 weights, bf16 source quantised by the library per token or per group; TestMatmul.W4A8_BF16, :266 ff.).
The oracle restates the reference's scalar definition (operators/matmul/matmul_ref_kernel.cpp:961-1003).  Integer group
sums are exact; the f32 sum over the groups may associate differently when several warps share a row tile, so results
are compared within 1 bf16 ulp / rel 1e-5 -- and bit for bit where one warp owns the whole sum (M > 64)."""
import numpy as np
import pytest

from helpers import assert_bf16_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    from zendnn_b200 import capi as c
    assert c.lib.b200dnn_device_count() > 0, "no CUDA device"
    return c


def _call(capi, d):
    st = capi.matmul(d)
    assert st == capi.SUCCESS, capi.last_error()


SHAPES = [(1, 64, 16), (5, 128, 24), (16, 256, 72), (3, 1024, 40), (12, 2048, 200), (40, 192, 130), (100, 512, 264), (200, 1024, 96)]


@pytest.mark.parametrize("gs", [4, 8, 16, 32, 64, 128, 0], ids=lambda g: "gs%s" % (g or "K"))
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "M%d_K%d_N%d" % s)
def test_per_group_s8(capi, oracle, shape, gs):
    M, K, N = shape
    gs = gs or K
    if K % gs:
        pytest.skip("K not divisible")
    G = K // gs
    rng = np.random.default_rng(M * 7 + K + gs)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    W = rng.integers(-128, 128, (K, N), dtype=np.int8)
    sa = rng.uniform(0.01, 0.05, (M, G)).astype(np.float32)
    sw = rng.uniform(1e-4, 5e-4, (G, N)).astype(np.float32)
    bias = rng.normal(size=N).astype(np.float32)
    for dst, transB, po in (("bf16", False, ()), ("f32", True, ("gelu_tanh",)), ("bf16", True, ("relu",))):
        Wc = np.ascontiguousarray(W.T) if transB else W
        out = np.zeros((M, N), dtype=np.uint16 if dst == "bf16" else np.float32)
        d = capi.make_matmul(M, N, K, A, Wc, out, src_dt=capi.DT["s8"], dst_dt=capi.DT[dst], transB=transB, bias=bias,
                             src_scale=capi.quant(sa, count=M * G), wei_scale=capi.quant(sw, count=G * N), weights_const=False,
                             postops=po)
        if G == 1 and M > 1:
            continue    # {M,1} x {1,N} is the per-token form of the tcgen05 / decode kernels (tested elsewhere)
        _call(capi, d)
        ref = oracle.matmul_group_scaled(A, W, sa, sw, dst, bias=bias, postops=list(po))
        if dst == "bf16":
            if M > 64:
                assert (out == ref).all(), ("one warp per sum: bit-exact", shape, gs)
            assert_bf16_close(out, ref, 1, "per-group %s gs=%d" % (shape, gs), atol=1e-5)
        else:
            assert np.allclose(out, ref, rtol=2e-5, atol=1e-5), float(np.abs(out - ref).max())


@pytest.mark.parametrize("src_gran", ["token", "group"])
@pytest.mark.parametrize("gs", [4, 16, 32, 64, 128, 0], ids=lambda g: "gs%s" % (g or "K"))
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "M%d_K%d_N%d" % s)
def test_w4a8(capi, oracle, shape, gs, src_gran):
    """bf16 source, dynamic_quant, packed s4 weights with {G,N} scales; the source scale is {M,1} or {M,G}."""
    M, K, N = shape
    gs = gs or K
    if K % gs:
        pytest.skip("K not divisible")
    G = K // gs
    rng = np.random.default_rng(M * 11 + K + gs)
    X = oracle.f32_to_bf16(rng.normal(size=(M, K)).astype(np.float32))
    W = rng.integers(-8, 8, (K, N), dtype=np.int8)
    sw = rng.uniform(1e-3, 5e-3, (G, N)).astype(np.float32)
    bias = oracle.f32_to_bf16(rng.normal(size=N).astype(np.float32))
    if src_gran == "token":
        A, sa = oracle.quant_per_token(X)
        sa = sa.reshape(M, 1)
    else:
        A, sa = oracle.quant_per_group(X, G)
    for transB in (False, True):
        packed = oracle.pack_s4(W, transB)
        out = np.zeros((M, N), dtype=np.uint16)
        sc_out = np.zeros(sa.shape, dtype=np.float32)
        d = capi.make_matmul(M, N, K, X, packed, out, src_dt=capi.DT["bf16"], dst_dt=capi.DT["bf16"], transB=transB, bias=bias,
                             src_scale=capi.quant(sc_out, count=sa.size), wei_scale=capi.quant(sw, count=G * N),
                             weights_const=False, dynamic_quant=True, wei_dt=capi.DT["s4"], postops=("swish",))
        _call(capi, d)
        assert (sc_out == sa).all(), "dynamic source scales differ from the oracle's"
        ref = oracle.matmul_group_scaled(A, W, sa, sw, "bf16", bias=bias, postops=["swish"])
        assert_bf16_close(out, ref, 1, "w4a8 %s gs=%d %s" % (shape, gs, src_gran), atol=1e-5)


def test_w4a8_weight_cache_and_host_device_pointers(capi, oracle):
    """Constant weights are prepared once (second call launches fewer kernels) and device-resident operands work."""
    import torch
    M, K, N, gs = 8, 512, 256, 128
    G = K // gs
    rng = np.random.default_rng(3)
    X = oracle.f32_to_bf16(rng.normal(size=(M, K)).astype(np.float32))
    W = rng.integers(-8, 8, (K, N), dtype=np.int8)
    sw = rng.uniform(1e-3, 5e-3, (G, N)).astype(np.float32)
    A, sa = oracle.quant_per_token(X)
    ref = oracle.matmul_group_scaled(A, W, sa, sw, "bf16")
    dev = torch.device("cuda:0")
    Xd = torch.from_numpy(X.view(np.int16)).to(dev)
    Wd = torch.from_numpy(oracle.pack_s4(W)).to(dev)
    swd = torch.from_numpy(sw).to(dev)
    outd = torch.zeros((M, N), dtype=torch.int16, device=dev)
    d = capi.make_matmul(M, N, K, Xd, Wd, outd, src_dt=capi.DT["bf16"], dst_dt=capi.DT["bf16"],
                         src_scale=capi.quant(None, count=M), wei_scale=capi.quant(swd, count=G * N, dt=capi.DT["f32"]),
                         weights_const=True, dynamic_quant=True, wei_dt=capi.DT["s4"])
    n0 = capi.lib.b200dnn_launch_count()
    _call(capi, d)
    n1 = capi.lib.b200dnn_launch_count()
    _call(capi, d)
    n2 = capi.lib.b200dnn_launch_count()
    torch.cuda.synchronize()
    assert n2 - n1 < n1 - n0, "the second call prepared the weight again"
    got = outd.cpu().numpy().view(np.uint16)
    assert_bf16_close(got, ref, 1, "w4a8 device pointers", atol=1e-5)
    capi.lib.b200dnn_clear_caches()


def test_contract(capi, oracle):
    """The reference's refusals for these forms (matmul/lowoha_matmul_utils.cpp:72-178)."""
    M, K, N, G = 4, 64, 16, 4
    rng = np.random.default_rng(1)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    X = oracle.f32_to_bf16(rng.normal(size=(M, K)).astype(np.float32))
    W4 = oracle.pack_s4(rng.integers(-8, 8, (K, N), dtype=np.int8))
    sw = np.ones((G, N), dtype=np.float32)
    sa = np.ones((M, G), dtype=np.float32)
    out = np.zeros((M, N), dtype=np.uint16)
    outf = np.zeros((M, N), dtype=np.float32)
    mk = capi.make_matmul
    # pre-quantised s8 source with s4 weights
    d = mk(M, N, K, A, W4, out, src_dt=capi.DT["s8"], dst_dt=capi.DT["bf16"], src_scale=capi.quant(sa, count=M * G),
           wei_scale=capi.quant(sw, count=G * N), wei_dt=capi.DT["s4"], weights_const=False)
    assert capi.matmul(d) == capi.FAILURE
    # W4A8 with an f32 destination
    d = mk(M, N, K, X, W4, outf, src_dt=capi.DT["bf16"], dst_dt=capi.DT["f32"], src_scale=capi.quant(None, count=M),
           wei_scale=capi.quant(sw, count=G * N), wei_dt=capi.DT["s4"], dynamic_quant=True, weights_const=False)
    assert capi.matmul(d) == capi.FAILURE
    # K not divisible by the group count; group size not a multiple of 4
    d = mk(M, N, K, X, W4, out, src_dt=capi.DT["bf16"], dst_dt=capi.DT["bf16"], src_scale=capi.quant(None, count=M),
           wei_scale=capi.quant(np.ones((3, N), np.float32), count=3 * N), wei_dt=capi.DT["s4"], dynamic_quant=True, weights_const=False)
    assert capi.matmul(d) == capi.FAILURE
    d = mk(M, N, 40, X, W4, out, lda=K, src_dt=capi.DT["bf16"], dst_dt=capi.DT["bf16"], src_scale=capi.quant(None, count=M),
           wei_scale=capi.quant(np.ones((4, N), np.float32), count=4 * N), wei_dt=capi.DT["s4"], dynamic_quant=True, weights_const=False)
    assert capi.matmul(d) == capi.FAILURE      # group size 10
    # a source scale whose shape is neither {M,G} nor {M,1}
    d = mk(M, N, K, A, np.zeros((K, N), np.int8), out, src_dt=capi.DT["s8"], dst_dt=capi.DT["bf16"],
           src_scale=capi.quant(np.ones(M * 2, np.float32), count=M * 2), wei_scale=capi.quant(sw, count=G * N), weights_const=False)
    assert capi.matmul(d) == capi.FAILURE
    # zero points are refused
    d = mk(M, N, K, A, np.zeros((K, N), np.int8), out, src_dt=capi.DT["s8"], dst_dt=capi.DT["bf16"],
           src_scale=capi.quant(sa, count=M * G), wei_scale=capi.quant(sw, count=G * N), src_zp=np.array([3], np.int32), weights_const=False)
    assert capi.matmul(d) == capi.FAILURE


def test_decode_form_agrees_with_the_general_kernel(capi, oracle, monkeypatch):
    """The decode form (persistent CTAs, cp.async rings) and the general kernel on the same call: identical source scales,
    outputs within 1 bf16 ulp of each other and of the oracle."""
    M, K, N, gs = 7, 2048, 328, 128
    G = K // gs
    rng = np.random.default_rng(21)
    X = oracle.f32_to_bf16(rng.normal(size=(M, K)).astype(np.float32))
    X[2, 5] = 0x7FC0          # a NaN entry: ignored by the abs-max, quantised to 0
    W = rng.integers(-8, 8, (K, N), dtype=np.int8)
    sw = rng.uniform(1e-3, 5e-3, (G, N)).astype(np.float32)
    packed = oracle.pack_s4(W)
    A, sa = oracle.quant_per_token(X)
    ref = oracle.matmul_group_scaled(A, W, sa, sw, "bf16")
    outs = {}
    for name, env in (("decode", {}), ("general", {"B200DNN_GS_DECODE": "0"})):
        monkeypatch.delenv("B200DNN_GS_DECODE", raising=False)
        for k, v in env.items():
            monkeypatch.setenv(k, v)
        out = np.zeros((M, N), dtype=np.uint16)
        sc = np.zeros(M, dtype=np.float32)
        d = capi.make_matmul(M, N, K, X, packed, out, src_dt=capi.DT["bf16"], dst_dt=capi.DT["bf16"], src_scale=capi.quant(sc, count=M),
                             wei_scale=capi.quant(sw, count=G * N), weights_const=False, dynamic_quant=True, wei_dt=capi.DT["s4"])
        _call(capi, d)
        assert (sc == sa).all(), name
        assert_bf16_close(out, ref, 1, name, atol=1e-5)
        outs[name] = out
    assert_bf16_close(outs["general"], outs["decode"], 1, "general against decode form", atol=1e-5)


@pytest.mark.parametrize("shape", [(12, 2048, 200), (100, 512, 264)], ids=lambda s: "M%d_K%d_N%d" % s)
def test_w4a8_per_tensor_source_scale(capi, oracle, shape):
    """The third source granularity the reference's W4A8 contract allows, scale dims {1,1} (lowoha_matmul_utils.cpp:160-178):
    one dynamic scale for the whole source (abs-max / 127, then the static quantise), used for every group."""
    M, K, N = shape
    gs = 128
    G = K // gs
    rng = np.random.default_rng(M + N)
    X = oracle.f32_to_bf16(rng.normal(size=(M, K)).astype(np.float32))
    W = rng.integers(-8, 8, (K, N), dtype=np.int8)
    sw = rng.uniform(1e-3, 5e-3, (G, N)).astype(np.float32)
    s = oracle.dyn_scales(X, per_channel=False)
    A = oracle.quant_static(X, s)
    ref = oracle.matmul_group_scaled(A, W, np.repeat(s, M), sw, "bf16")
    out = np.zeros((M, N), dtype=np.uint16)
    sc = np.zeros(1, dtype=np.float32)
    packed = oracle.pack_s4(W)          # the descriptor holds only the address: the array must outlive the call
    d = capi.make_matmul(M, N, K, X, packed, out, src_dt=capi.DT["bf16"], dst_dt=capi.DT["bf16"], src_scale=capi.quant(sc, count=1),
                         wei_scale=capi.quant(sw, count=G * N), weights_const=False, dynamic_quant=True, wei_dt=capi.DT["s4"])
    _call(capi, d)
    assert (sc == s).all()
    assert_bf16_close(out, ref, 1, "w4a8 per-tensor source scale", atol=1e-5)
