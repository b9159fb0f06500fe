"""GPU parity tests of b200dnn_matmul (the matmul_direct INT8 path) against the CPU oracle and the
golden outputs of the reference's own kernel.  Mirrors the reference's TestMatmul.INT8,
INT8_SYM_QUANT_PER_TOKEN_* and INT8_DYNAMIC_GEMM_* cases (zendnnl/gtests/test_matmul.cpp:975-1650).
s32 results must be bit-exact; bf16 results within 1 bf16 ulp (rel <= 8e-3)."""
import ctypes as C

import numpy as np
import pytest

from helpers import assert_bf16_close, config1, decode_case

pytestmark = pytest.mark.gpu

STREAM, TC = 1, 2
TILED = 3   # the tiled split-K streaming kernel only (STREAM picks the persistent decode kernel when M <= 16)
KERNELS = [pytest.param(STREAM, id="stream"), pytest.param(TC, id="tc"), pytest.param(TILED, id="tiled")]


@pytest.fixture(scope="module")
def capi():
    from zendnn_b200 import capi as c
    assert c.lib.b200dnn_device_count() > 0, "no CUDA device"
    return c


def run(capi, M, N, K, A, W, dst_dt, **kw):
    out = np.zeros((M, N), dtype={"bf16": np.uint16, "f32": np.float32, "s32": np.int32, "s8": np.int8, "u8": np.uint8}[dst_dt])
    d = capi.make_matmul(M, N, K, A, W, out, src_dt=capi.dt_of(A) if "src_dt" not in kw else kw.pop("src_dt"),
                         dst_dt=capi.DT[dst_dt], **kw)
    st = capi.matmul(d)
    assert st == capi.SUCCESS, capi.last_error()
    return out


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("shape", [(1, 64, 16), (5, 100, 24), (16, 256, 64), (33, 260, 80), (128, 512, 128),
                                   (130, 384, 200), (257, 1024, 264)])
def test_s32_bit_exact_small(capi, oracle, kernel, shape):
    M, K, N = shape
    rng = np.random.default_rng(M * 131 + K)
    for src in ("u8", "s8"):
        A = rng.integers(0, 256, (M, K), dtype=np.uint8) if src == "u8" else rng.integers(-128, 128, (M, K), dtype=np.int8)
        W = rng.integers(-128, 128, (K, N), dtype=np.int8)
        if kernel == TC and K % 16 != 0:
            continue    # tcgen05 path needs 16-byte aligned rows; the dispatcher sends these to the streaming kernel
        got = run(capi, M, N, K, A, W, "s32", weights_const=False, force_kernel=kernel)
        assert (got == oracle.gemm_s32(A, W)).all(), (src, shape)
        # zero-point compensation stays exact in s32
        zp = np.array([37], dtype=np.int32)
        got = run(capi, M, N, K, A, W, "s32", weights_const=False, force_kernel=kernel, src_zp=zp)
        ref = oracle.epilogue(oracle.gemm_s32(A, W), "s32", src_zp=37, col_sum=oracle.colsum(W))
        assert (got == ref).all(), (src, shape, "zp")
        # transposed weight layout [N,K]
        Wt = np.ascontiguousarray(W.T)
        got = run(capi, M, N, K, A, Wt, "s32", weights_const=False, force_kernel=kernel, transB=True)
        assert (got == oracle.gemm_s32(A, W)).all(), (src, shape, "transB")


@pytest.mark.parametrize("kernel", KERNELS)
def test_golden_reference_cases(capi, oracle, golden, kernel):
    """Outputs of the reference's own INT8 tile kernel (tests/golden): <= 1 bf16 ulp."""
    fused = {0: [], 1: ["relu"], 2: ["gelu_tanh"], 3: ["gelu_erf"], 4: ["sigmoid"], 5: ["swish"], 6: ["tanh"]}
    i = 0
    while "c%d_meta" % i in golden:
        p = "c%d_" % i
        M, K, N, zp, fo, is_bf16, has_bias = [int(v) for v in golden[p + "meta"]]
        A, W, ws = golden[p + "A"], golden[p + "B"], golden[p + "ws"]
        i += 1
        if kernel == TC and K % 16 != 0:
            continue
        bias = golden[p + "bias"] if has_bias else None
        got = run(capi, M, N, K, A, W, "bf16" if is_bf16 else "f32", weights_const=False, force_kernel=kernel,
                  src_scale=golden[p + "ss"], wei_scale=ws, src_zp=np.array([zp], dtype=np.int32), bias=bias,
                  postops=fused[fo])
        ref = golden[p + "out"]
        if is_bf16:
            # the reference kernel evaluates tanh / sigmoid with ~5e-5-relative polynomials: its activation
            # cases are compared with an absolute floor, the linear ones to 1 ulp
            assert_bf16_close(got, ref, 1 if fo in (0, 1) else 2, "golden case %d" % (i - 1), atol=0.0 if fo in (0, 1) else 1e-4)
        else:
            assert np.allclose(got, ref, rtol=2e-4, atol=1e-4)


@pytest.mark.parametrize("kernel", KERNELS)
def test_config1_full_size(capi, oracle, kernel):
    """M128 K4096 N4096, u8 zp 128 scale .02, per-channel weight scales, f32 bias, ReLU, bf16 out, seed 0."""
    c = config1(oracle)
    M, K, N = 128, 4096, 4096
    acc = oracle.gemm_s32(c["A"], c["W"])
    if True:
        got = run(capi, M, N, K, c["A"], c["W"], "s32", force_kernel=kernel)
        assert (got == acc).all()
        got = run(capi, M, N, K, c["A"], c["W"], "bf16", force_kernel=kernel, src_scale=c["ss"], wei_scale=c["ws"],
                  src_zp=c["zp"], bias=c["bias"], postops=["relu"])
        ref = oracle.epilogue(acc, "bf16", c["ss"], c["ws"], 128, oracle.colsum(c["W"]), c["bias"], ["relu"])
        assert (got == ref).all(), "bf16 output differs from the oracle (same operation order): %d" % int((got != ref).sum())
        assert np.abs(oracle.bf16_to_f32(got)).sum() > 1e-3


@pytest.mark.parametrize("M", [1, 4, 16])
@pytest.mark.parametrize("KN", [(4096, 4096), (4096, 11008), (11008, 4096)])
def test_decode_shapes_prepacked(capi, oracle, M, KN):
    """Config 2: per-token s8 activations x per-channel s8 weights, prepacked, bf16 out."""
    K, N = KN
    c = decode_case(oracle, M, K, N, seed=M)
    size = capi.lib.b200dnn_prepack_size(K, N, 0)
    packed = np.zeros(size, dtype=np.uint8)
    assert capi.lib.b200dnn_prepack(capi.ptr(c["W"]), K, N, N, 0, 0, capi.ptr(packed), None) == capi.SUCCESS, capi.last_error()
    got = run(capi, M, N, K, c["A"], packed, "bf16", wei_format="r", src_scale=c["sa"], wei_scale=c["sw"])
    ref = oracle.matmul_w8a8(c["A"], c["W"], "bf16", src_scale=c["sa"], wei_scale=c["sw"])
    assert (got == ref).all(), int((got != ref).sum())
    # raw weights give the same bytes
    got2 = run(capi, M, N, K, c["A"], c["W"], "bf16", weights_const=False, src_scale=c["sa"], wei_scale=c["sw"])
    assert (got2 == ref).all()


@pytest.mark.parametrize("splits,bn", [("2", "128"), ("3", "256"), ("4", "128"), ("4", "256"), ("0", "0")])
@pytest.mark.parametrize("shape", [(100, 1024, 1000), (200, 2064, 520), (128, 4096, 264), (300, 640, 4096)])
def test_tc_split_form(capi, oracle, monkeypatch, splits, bn, shape):
    """Small plain GEMMs run as clusters whose CTAs split the K blocks of a tile and add their int32 partial sums through
    distributed shared memory: s32 bit-exact, and the float epilogue gives the bytes of the unsplit kernel."""
    M, K, N = shape
    if splits != "0":
        monkeypatch.setenv("B200DNN_TC_KSPLIT", splits)
        monkeypatch.setenv("B200DNN_TC_BN", bn)
    rng = np.random.default_rng(K + N)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    W = rng.integers(-128, 128, (K, N), dtype=np.int8)
    sa = rng.uniform(0.01, 0.05, M).astype(np.float32)
    sw = rng.uniform(1e-4, 5e-4, N).astype(np.float32)
    bias = rng.normal(size=N).astype(np.float32)
    acc = oracle.gemm_s32(A, W)
    got = run(capi, M, N, K, A, W, "s32", weights_const=False, force_kernel=TC)
    assert (got == acc).all()
    kw = dict(weights_const=False, force_kernel=TC, src_scale=sa, wei_scale=sw, bias=bias, postops=["gelu_tanh"])
    got = run(capi, M, N, K, A, W, "bf16", **kw)
    monkeypatch.setenv("B200DNN_TC_KSPLIT", "1")
    unsplit = run(capi, M, N, K, A, W, "bf16", **kw)
    assert (got == unsplit).all(), int((got != unsplit).sum())
    ref = oracle.matmul_w8a8(A, W, "bf16", src_scale=sa, wei_scale=sw, bias=bias, postops=["gelu_tanh"])
    assert_bf16_close(got, ref, 1, "split form", atol=1e-5)
    Au = rng.integers(0, 256, (M, K), dtype=np.uint8)
    monkeypatch.setenv("B200DNN_TC_KSPLIT", splits)
    got = run(capi, M, N, K, Au, W, "f32", weights_const=False, force_kernel=TC, src_scale=np.array([0.02], dtype=np.float32),
              wei_scale=sw, src_zp=np.array([128], dtype=np.int32), bias=bias, postops=["relu"])
    ref = oracle.epilogue(oracle.gemm_s32(Au, W), "f32", [0.02], sw, 128, oracle.colsum(W), bias, ["relu"])
    assert np.allclose(got, ref, rtol=2e-6, atol=1e-6)


ELTWISE = ["gelu_erf", "sigmoid", "tanh", "elu", "leaky_relu", "gelu_tanh", "swish", "relu"]


def _postop(name):
    if name == "elu":
        return dict(type="elu", alpha=1.0)
    if name == "leaky_relu":
        return dict(type="leaky_relu", alpha=0.01)
    return name


@pytest.mark.parametrize("kernel", KERNELS + [pytest.param("split", id="tc-split")])
@pytest.mark.parametrize("name", ELTWISE)
def test_eltwise_postops_single_and_chained(capi, oracle, monkeypatch, kernel, name):
    """Every element-wise post-op of the supported subset, alone (the specialised epilogue loops of the tcgen05 kernel)
    and inside a chain (the generic loop), on every kernel form: bf16 within 1 ulp of the oracle, f32 within rel 1e-5
    (the sigmoid family is evaluated with the fast exponential and reciprocal).  Reference definitions:
    operators/matmul/matmul_ref_kernel.cpp:694-761."""
    M, K, N = (200, 512, 264) if kernel in (TC, "split") else (12, 512, 264)
    if kernel == "split":
        monkeypatch.setenv("B200DNN_TC_KSPLIT", "2")
        monkeypatch.setenv("B200DNN_TC_BN", "128")
        kernel = TC
    rng = np.random.default_rng(len(name) * 7 + M)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    W = rng.integers(-128, 128, (K, N), dtype=np.int8)
    sa = rng.uniform(0.01, 0.05, M).astype(np.float32)
    sw = rng.uniform(1e-4, 5e-4, N).astype(np.float32)     # pre-activations of order +-3: both tails of every activation
    bias = rng.normal(size=N).astype(np.float32)
    add = rng.normal(size=(1, N)).astype(np.float32)
    for po in ([_postop(name)], [dict(type="binary_add", buff=add), _postop(name), dict(type="clip", alpha=-2.0, beta=2.0)]):
        kw = dict(weights_const=False, force_kernel=kernel, src_scale=sa, wei_scale=sw, bias=bias, postops=po)
        ref = oracle.matmul_w8a8(A, W, "bf16", src_scale=sa, wei_scale=sw, bias=bias, postops=po)
        got = run(capi, M, N, K, A, W, "bf16", **kw)
        assert_bf16_close(got, ref, 1, "%s x%d" % (name, len(po)), atol=1e-5)
        ref32 = oracle.matmul_w8a8(A, W, "f32", src_scale=sa, wei_scale=sw, bias=bias, postops=po)
        got32 = run(capi, M, N, K, A, W, "f32", **kw)
        assert np.allclose(got32, ref32, rtol=1e-5, atol=1e-5), (name, float(np.abs(got32 - ref32).max()))


@pytest.mark.parametrize("bn", ["0", "96", "128", "160", "224", "256"])
@pytest.mark.parametrize("shape", [(257, 1024, 264), (600, 512, 1000), (1024, 2048, 512), (130, 4096, 128), (900, 384, 2100)])
def test_tc_pair_form(capi, oracle, monkeypatch, bn, shape):
    """The two-CTA form of the tcgen05 kernel (cta_group::2: each CTA of a pair loads its 128 rows of A and half of the
    weight tile, the leader issues M256 MMAs for both): s32 bit-exact for ragged M and N, and the float epilogue gives the
    bytes of the single-CTA form."""
    M, K, N = shape
    monkeypatch.setenv("B200DNN_TC_PAIR", "1")
    monkeypatch.setenv("B200DNN_TC_BN", bn)
    rng = np.random.default_rng(M + N)
    W = rng.integers(-128, 128, (K, N), dtype=np.int8)
    for src in ("u8", "s8"):
        A = rng.integers(0, 256, (M, K), dtype=np.uint8) if src == "u8" else rng.integers(-128, 128, (M, K), dtype=np.int8)
        got = run(capi, M, N, K, A, W, "s32", weights_const=False, force_kernel=TC)
        assert (got == oracle.gemm_s32(A, W)).all(), (src, "pair form s32")
    sa = rng.uniform(0.01, 0.05, M).astype(np.float32)
    sw = rng.uniform(1e-4, 5e-4, N).astype(np.float32)
    bias = rng.normal(size=N).astype(np.float32)
    kw = dict(weights_const=False, force_kernel=TC, src_scale=sa, wei_scale=sw, bias=bias, postops=["gelu_tanh"])
    got = run(capi, M, N, K, A, W, "bf16", **kw)
    monkeypatch.setenv("B200DNN_TC_PAIR", "0")
    monkeypatch.setenv("B200DNN_TC_BN", "0")
    single = run(capi, M, N, K, A, W, "bf16", **kw)
    assert (got == single).all(), int((got != single).sum())
    got32 = run(capi, M, N, K, A, W, "f32", weights_const=False, force_kernel=TC, src_scale=sa, wei_scale=sw)
    assert np.array_equal(got32, oracle.matmul_w8a8(A, W, "f32", src_scale=sa, wei_scale=sw))


def test_scales_in_bf16_storage(capi, oracle):
    c = decode_case(oracle, 8, 512, 128, seed=3)
    sa16, sw16 = oracle.f32_to_bf16(c["sa"]), oracle.f32_to_bf16(c["sw"])
    got = run(capi, 8, 128, 512, c["A"], c["W"], "bf16", weights_const=False, src_scale=sa16, wei_scale=sw16)
    ref = oracle.matmul_w8a8(c["A"], c["W"], "bf16", src_scale=oracle.bf16_to_f32(sa16), wei_scale=oracle.bf16_to_f32(sw16))
    assert (got == ref).all()


@pytest.mark.parametrize("M,K,N", [(64, 512, 256), (300, 1024, 384)])
def test_dynamic_quant_gelu_tc(capi, oracle, M, K, N):
    """Config 3 family: bf16 activations quantised per token inside the call, bias, GELU(tanh), bf16 out."""
    rng = np.random.default_rng(M)
    x = oracle.f32_to_bf16(rng.normal(size=(M, K)).astype(np.float32))
    qw, sw = oracle.quant_weights_per_channel(oracle.f32_to_bf16((rng.normal(size=(K, N)) * 0.02).astype(np.float32)))
    bias = rng.normal(size=N).astype(np.float32)
    qa, sa = oracle.quant_per_token(x)
    ref = oracle.matmul_w8a8(qa, qw, "bf16", src_scale=sa, wei_scale=sw, bias=bias, postops=["gelu_tanh"])
    for with_buf in (False, True):
        scales = np.zeros(M, dtype=np.float32)
        ss = capi.quant(scales if with_buf else None, count=M, dt=capi.DT["f32"])
        got = run(capi, M, N, K, x, qw, "bf16", src_dt=capi.DT["bf16"], dynamic_quant=True, weights_const=False,
                  src_scale=ss, wei_scale=sw, bias=bias, postops=["gelu_tanh"])
        # the libm form 0.5*x*(1+tanh(u)) cancels for very negative u (outputs of order 1e-6): absolute floor there
        assert_bf16_close(got, ref, 1, "dynamic quant + gelu", atol=1e-5)
        if with_buf:
            assert (scales == sa).all()          # the library writes the scales it used


@pytest.mark.parametrize("kernel", KERNELS)
def test_postop_chain_and_strides(capi, oracle, kernel):
    rng = np.random.default_rng(9)
    M, K, N, lda, ldc = 40, 192, 72, 208, 96
    Afull = rng.integers(-128, 128, (M, lda), dtype=np.int8)
    A = Afull[:, :K]
    W = rng.integers(-64, 64, (K, N), dtype=np.int8)
    sw = rng.uniform(0.001, 0.01, N).astype(np.float32)
    add = rng.normal(size=(1, N)).astype(np.float32)
    mul = rng.normal(size=(M, N)).astype(np.float32)
    po = [dict(type="binary_add", buff=add), "swish", dict(type="binary_mul", buff=mul),
          dict(type="clip", alpha=-0.5, beta=0.75)]
    ref = oracle.matmul_w8a8(np.ascontiguousarray(A), W, "f32", src_scale=[0.05], wei_scale=sw, postops=po)
    out = np.full((M, ldc), 7.0, dtype=np.float32)
    ss = np.array([0.05], dtype=np.float32)         # the descriptor holds only the address: kept alive for the call
    if True:
        out[:] = 7.0
        d = capi.make_matmul(M, N, K, Afull, W, out, src_dt=capi.DT["s8"], dst_dt=capi.DT["f32"], lda=lda, ldc=ldc,
                             weights_const=False, src_scale=ss, wei_scale=sw, postops=po,
                             force_kernel=kernel)
        assert capi.matmul(d) == capi.SUCCESS, capi.last_error()
        assert np.allclose(out[:, :N], ref, rtol=2e-6, atol=1e-6)
        assert (out[:, N:] == 7.0).all()      # padding columns untouched


def test_device_pointers_and_weight_cache(capi, oracle):
    import torch
    c = decode_case(oracle, 4, 1024, 512, seed=11)
    dev = torch.device("cuda:0")
    A = torch.from_numpy(c["A"]).to(dev)
    W = torch.from_numpy(c["W"]).to(dev)
    sa, sw = torch.from_numpy(c["sa"]).to(dev), torch.from_numpy(c["sw"]).to(dev)
    out = torch.zeros(4, 512, dtype=torch.bfloat16, device=dev)
    d = capi.make_matmul(4, 512, 1024, A, W, out, src_dt=capi.DT["s8"], dst_dt=capi.DT["bf16"], src_scale=sa, wei_scale=sw)
    n0 = capi.lib.b200dnn_launch_count()
    assert capi.matmul(d, torch.cuda.current_stream().cuda_stream) == capi.SUCCESS, capi.last_error()
    n1 = capi.lib.b200dnn_launch_count()
    assert capi.matmul(d, torch.cuda.current_stream().cuda_stream) == capi.SUCCESS
    n2 = capi.lib.b200dnn_launch_count()
    torch.cuda.synchronize()
    assert n1 - n0 > n2 - n1 == 1          # second call hits the packed-weight cache: one GEMM launch
    ref = oracle.matmul_w8a8(c["A"], c["W"], "bf16", src_scale=c["sa"], wei_scale=c["sw"])
    got = out.view(torch.int16).cpu().numpy().view(np.uint16)
    assert (got == ref).all()
    assert capi.lib.b200dnn_clear_caches() == capi.SUCCESS


def test_host_inputs_with_device_output_back_to_back(capi, oracle):
    """Small host inputs travel in one pinned block per call; with a device output the call returns before that block
    has been read, and the next call must not overwrite it early: eight calls with different inputs, one sync."""
    import torch
    M, K, N = 4, 1024, 512
    dev = torch.device("cuda:0")
    cases = [decode_case(oracle, M, K, N, seed=20 + i) for i in range(8)]
    W = torch.from_numpy(cases[0]["W"]).to(dev)
    sw = torch.from_numpy(cases[0]["sw"]).to(dev)
    outs = [torch.zeros(M, N, dtype=torch.bfloat16, device=dev) for _ in cases]
    st = torch.cuda.current_stream().cuda_stream
    for c, out in zip(cases, outs):
        d = capi.make_matmul(M, N, K, c["A"], W, out, src_dt=capi.DT["s8"], dst_dt=capi.DT["bf16"], src_scale=c["sa"], wei_scale=sw)
        assert capi.matmul(d, st) == capi.SUCCESS, capi.last_error()
    torch.cuda.synchronize()
    for c, out in zip(cases, outs):
        ref = oracle.matmul_w8a8(c["A"], cases[0]["W"], "bf16", src_scale=c["sa"], wei_scale=cases[0]["sw"])
        assert (out.view(torch.int16).cpu().numpy().view(np.uint16) == ref).all()
    assert capi.lib.b200dnn_clear_caches() == capi.SUCCESS


def test_contract_violations(capi):
    """Boundary contract: failures and unimplemented features are reported, nothing is computed."""
    A = np.zeros((4, 64), dtype=np.int8); W = np.zeros((64, 16), dtype=np.int8); out = np.zeros((4, 16), dtype=np.float32)
    mk = lambda **kw: capi.make_matmul(4, 16, 64, A, W, out, **{**dict(src_dt=capi.DT["s8"], dst_dt=capi.DT["f32"]), **kw})
    d = mk(); d.src = None
    assert capi.matmul(d) == capi.FAILURE
    d = mk(); d.M = 0
    assert capi.matmul(d) == capi.FAILURE
    d = mk(); d.lda = 8
    assert capi.matmul(d) == capi.FAILURE
    d = mk(); d.wei_dt = capi.DT["s4"]
    assert capi.matmul(d) == capi.FAILURE                # s4 weights with a pre-quantised source: refused as in the reference
    d = mk(); d.wei_dt = capi.DT["u4"]
    assert capi.matmul(d) == capi.UNIMPLEMENTED
    d = mk(src_dt=capi.DT["f32"])
    assert capi.matmul(d) == capi.UNIMPLEMENTED          # float source without dynamic_quant
    d = mk(postops=["mish"])
    assert capi.matmul(d) == capi.FAILURE                # rejected on INT8, as the reference does
    d = mk(postops=["softmax"])
    assert capi.matmul(d) == capi.UNIMPLEMENTED
    # per-token source scale needs a per-channel weight scale of N elements
    d = mk(src_scale=np.ones(4, dtype=np.float32), wei_scale=np.ones(1, dtype=np.float32))
    assert capi.matmul(d) == capi.FAILURE
    # per-token source scale forbids a zero-point
    d = mk(src_scale=np.ones(4, dtype=np.float32), wei_scale=np.ones(16, dtype=np.float32), src_zp=np.array([3], dtype=np.int32))
    assert capi.matmul(d) == capi.FAILURE
    assert "zero-point" in capi.last_error()


def test_pinned_host_buffers(capi, oracle):
    """Pinned host operands: inputs are copied in, a small result is written straight into the pinned buffer."""
    import torch
    c = decode_case(oracle, 4, 1024, 512, seed=21)
    A = torch.from_numpy(c["A"]).pin_memory()
    sa, sw = torch.from_numpy(c["sa"]).pin_memory(), torch.from_numpy(c["sw"]).pin_memory()
    out = torch.zeros(4, 512, dtype=torch.bfloat16).pin_memory()
    d = capi.make_matmul(4, 512, 1024, A, c["W"], out, src_dt=capi.DT["s8"], dst_dt=capi.DT["bf16"], src_scale=sa, wei_scale=sw)
    assert capi.matmul(d) == capi.SUCCESS, capi.last_error()      # synchronous for host buffers: result is there on return
    ref = oracle.matmul_w8a8(c["A"], c["W"], "bf16", src_scale=c["sa"], wei_scale=c["sw"])
    assert (out.view(torch.int16).numpy().view(np.uint16) == ref).all()
    # a large pinned result takes the device-twin path
    M, K, N = 640, 256, 1024
    rng = np.random.default_rng(3)
    A2 = rng.integers(-128, 128, (M, K), dtype=np.int8); W2 = rng.integers(-128, 128, (K, N), dtype=np.int8)
    out2 = torch.zeros(M, N, dtype=torch.int32).pin_memory()
    d = capi.make_matmul(M, N, K, A2, W2, out2, src_dt=capi.DT["s8"], dst_dt=capi.DT["s32"], weights_const=False)
    assert capi.matmul(d) == capi.SUCCESS, capi.last_error()
    assert (out2.numpy() == oracle.gemm_s32(A2, W2)).all()
    capi.lib.b200dnn_clear_caches()


@pytest.mark.parametrize("form", ["1", "2", "3", "5"])
@pytest.mark.parametrize("shape", [(1, 64, 16), (2, 1000, 72), (3, 4096, 1184), (8, 300, 2368), (9, 2048, 4744), (16, 4224, 1000)])
def test_decode_kernel_forms(capi, oracle, monkeypatch, form, shape):
    """Both decode kernels (register-batch form, bulk-copy ring with 2..5 groups per stage) over all M <= 16,
    ragged K and N, u8 + zero point and s8 + per-token scale."""
    monkeypatch.setenv("B200DNN_DECODE_KERNEL", form)
    M, K, N = shape
    rng = np.random.default_rng(M * 7 + N)
    W = rng.integers(-128, 128, (K, N), dtype=np.int8)
    A = rng.integers(0, 256, (M, K), dtype=np.uint8)
    got = run(capi, M, N, K, A, W, "s32", weights_const=False, force_kernel=STREAM, src_zp=np.array([128], dtype=np.int32))
    assert (got == oracle.epilogue(oracle.gemm_s32(A, W), "s32", src_zp=128, col_sum=oracle.colsum(W))).all()
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    sa = rng.uniform(0.01, 0.05, M).astype(np.float32)
    sw = rng.uniform(1e-4, 5e-4, N).astype(np.float32)
    bias = rng.normal(size=N).astype(np.float32)
    got = run(capi, M, N, K, A, W, "bf16", weights_const=False, force_kernel=STREAM, src_scale=sa, wei_scale=sw, bias=bias,
              postops=["relu"])
    ref = oracle.matmul_w8a8(A, W, "bf16", src_scale=sa, wei_scale=sw, bias=bias, postops=["relu"])
    assert (got == ref).all()


@pytest.mark.parametrize("M", [1, 256])
def test_bounded_waits_leave_a_status_and_a_usable_context(capi, oracle, monkeypatch, M):
    """With the test hook that makes the producer issue no copies, every wait on data in the ring decode kernel (M = 1)
    and in the tcgen05 kernel (M = 256) runs into its limit of about a second: the kernel leaves without hanging,
    b200dnn_stream_status reports failure with the code, and the next call on the same context is correct."""
    import torch
    K, N = 512, 256
    rng = np.random.default_rng(M)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    W = rng.integers(-128, 128, (K, N), dtype=np.int8)
    dA, dW = torch.from_numpy(A).cuda(), torch.from_numpy(W).cuda()
    out = torch.zeros(M, N, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    d = capi.make_matmul(M, N, K, dA, dW, out, src_dt=capi.DT["s8"], dst_dt=capi.DT["s32"], weights_const=False)
    assert capi.lib.b200dnn_stream_status(st) == capi.SUCCESS
    monkeypatch.setenv("B200DNN_TEST_NO_LOADS", "1")
    monkeypatch.setenv("B200DNN_DECODE_KERNEL", "2")   # the ring form (by default only weights of 24 MB or more take it)
    assert capi.matmul(d, st) == capi.SUCCESS          # device pointers: the call only enqueues
    assert capi.lib.b200dnn_stream_status(st) == capi.FAILURE
    assert "gave up waiting" in capi.last_error()
    monkeypatch.delenv("B200DNN_TEST_NO_LOADS")
    assert capi.matmul(d, st) == capi.SUCCESS
    assert capi.lib.b200dnn_stream_status(st) == capi.SUCCESS
    assert (out.cpu().numpy() == oracle.gemm_s32(A, W)).all()
    capi.lib.b200dnn_clear_caches()


def test_two_host_threads_on_two_streams(capi, oracle):
    """The entry points are re-entrant like the reference's (lowoha_operators/matmul/lowoha_matmul.hpp:95-99): two host
    threads, each on its own stream, interleave dynamic-quantisation GEMMs (which use library workspace) and split-K
    streaming GEMMs (which use workspace and tile counters) without sharing scratch.  Every result is checked."""
    import threading
    import torch
    dev = torch.device("cuda:0")
    jobs = []
    for i, (M, K, N, kernel) in enumerate([(48, 1024, 512, 2), (7, 4096, 256, 3)]):
        rng = np.random.default_rng(40 + i)
        x = oracle.f32_to_bf16(rng.normal(size=(M, K)).astype(np.float32))
        qw, sw = oracle.quant_weights_per_channel(oracle.f32_to_bf16((rng.normal(size=(K, N)) * 0.02).astype(np.float32)))
        qa, sa = oracle.quant_per_token(x)
        ref = oracle.matmul_w8a8(qa, qw, "bf16", src_scale=sa, wei_scale=sw)
        jobs.append(dict(M=M, K=K, N=N, kernel=kernel, ref=ref, stream=torch.cuda.Stream(),
                         x=torch.from_numpy(x.view(np.int16)).to(dev), W=torch.from_numpy(qw).to(dev), sw=torch.from_numpy(sw).to(dev),
                         outs=[torch.zeros(M, N, dtype=torch.bfloat16, device=dev) for _ in range(40)], err=None))

    def work(j):
        try:
            st = j["stream"].cuda_stream
            for out in j["outs"]:
                d = capi.make_matmul(j["M"], j["N"], j["K"], j["x"], j["W"], out, src_dt=capi.DT["bf16"], dst_dt=capi.DT["bf16"],
                                     dynamic_quant=True, src_scale=capi.quant(None, count=j["M"], dt=capi.DT["f32"]), wei_scale=j["sw"],
                                     force_kernel=j["kernel"])
                if capi.matmul(d, st) != capi.SUCCESS:
                    raise RuntimeError(capi.last_error())
            if capi.lib.b200dnn_stream_status(st) != capi.SUCCESS:
                raise RuntimeError(capi.last_error())
        except Exception as e:      # reported by the main thread
            j["err"] = e

    torch.cuda.synchronize()
    threads = [threading.Thread(target=work, args=(j,)) for j in jobs]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    torch.cuda.synchronize()
    for j in jobs:
        assert j["err"] is None, j["err"]
        for out in j["outs"]:
            assert (out.view(torch.int16).cpu().numpy().view(np.uint16) == j["ref"]).all()
    capi.lib.b200dnn_clear_caches()


def test_two_devices_in_one_process(capi, oracle):
    """Library state belongs to the device that is current when a call starts: the same process calls on cuda:0 and on
    cuda:1 in turn (weights cached per device, scratch per device) and both results are right."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    c = decode_case(oracle, 4, 1024, 512, seed=31)
    ref = oracle.matmul_w8a8(c["A"], c["W"], "bf16", src_scale=c["sa"], wei_scale=c["sw"])
    M2, K2, N2 = 300, 512, 384
    rng = np.random.default_rng(32)
    A2 = rng.integers(-128, 128, (M2, K2), dtype=np.int8); W2 = rng.integers(-128, 128, (K2, N2), dtype=np.int8)
    for rnd in range(2):
        for dev_id in (0, 1):
            torch.cuda.set_device(dev_id)
            dev = torch.device("cuda", dev_id)
            A, W = torch.from_numpy(c["A"]).to(dev), torch.from_numpy(c["W"]).to(dev)
            sa, sw = torch.from_numpy(c["sa"]).to(dev), torch.from_numpy(c["sw"]).to(dev)
            out = torch.zeros(4, 512, dtype=torch.bfloat16, device=dev)
            d = capi.make_matmul(4, 512, 1024, A, W, out, src_dt=capi.DT["s8"], dst_dt=capi.DT["bf16"], src_scale=sa, wei_scale=sw,
                                 weights_const=False)
            st = torch.cuda.current_stream().cuda_stream
            assert capi.matmul(d, st) == capi.SUCCESS, capi.last_error()
            assert capi.lib.b200dnn_stream_status(st) == capi.SUCCESS, capi.last_error()
            assert (out.view(torch.int16).cpu().numpy().view(np.uint16) == ref).all(), (rnd, dev_id)
            # host buffers through the tcgen05 path on the same device
            got = run(capi, M2, N2, K2, A2, W2, "s32", weights_const=False, force_kernel=TC)
            assert (got == oracle.gemm_s32(A2, W2)).all(), (rnd, dev_id)
    torch.cuda.set_device(0)
    capi.lib.b200dnn_clear_caches()


def _group_case(capi, oracle, Ms, K, N, *, dyn, dst, bias_on, postops, rng, ldc_pad=0):
    """Build the descriptors of a plain grouped call; returns (array of descriptors, outputs, expected outputs, keepalive)."""
    G = len(Ms)
    descs = (capi.MatmulDesc * G)()
    outs, refs, keep = [], [], []
    for g, M in enumerate(Ms):
        W = rng.integers(-128, 128, (K, N), dtype=np.int8)
        sw = rng.uniform(1e-4, 5e-4, N).astype(np.float32)
        bias = rng.normal(size=N).astype(np.float32) if bias_on[g] else None
        rows = max(M, 1)
        ldc = N + ldc_pad
        out = np.zeros((rows, ldc), dtype=np.uint16 if dst == "bf16" else np.float32)
        if dyn:
            X = oracle.f32_to_bf16(rng.normal(size=(rows, K)).astype(np.float32))
            A, sa = oracle.quant_per_token(X)
            d = capi.make_matmul(M, N, K, X, W, out, src_dt=capi.DT["bf16"], dst_dt=capi.DT[dst], ldc=ldc, bias=bias,
                                 wei_scale=sw, dynamic_quant=True, weights_const=False, postops=postops)
            keep += [X]
        else:
            A = rng.integers(-128, 128, (rows, K), dtype=np.int8)
            sa = rng.uniform(0.01, 0.05, rows).astype(np.float32)
            d = capi.make_matmul(M, N, K, A, W, out, src_dt=capi.DT["s8"], dst_dt=capi.DT[dst], ldc=ldc, bias=bias,
                                 src_scale=capi.quant(sa, count=M), wei_scale=sw, weights_const=False, postops=postops)
        descs[g] = d
        keep += [A, sa, W, sw, bias]
        outs.append(out)
        refs.append(oracle.matmul_w8a8(A[:M], W, dst, src_scale=sa[:M], wei_scale=sw, bias=bias, postops=list(postops)) if M else None)
    return descs, outs, refs, keep


@pytest.mark.parametrize("dyn", [False, True], ids=["s8-rows", "bf16-dynamic"])
@pytest.mark.parametrize("dst", ["bf16", "f32"])
def test_group_matmul_one_grouped_launch(capi, oracle, dyn, dst):
    """The plain (parallel) mode of group_matmul_direct (reference: matmul/lowoha_matmul.hpp:204-223, experts with M == 0
    skipped, group_matmul_parallel_common.hpp:1240-1248): experts of one shape run as ONE grouped tcgen05 launch whose
    results are those of separate matmul calls -- checked against the oracle per expert, with ragged and empty experts, a
    bias on some experts only, padded destinations, and by the number of kernels launched."""
    rng = np.random.default_rng(17 + dyn)
    Ms, K, N = [200, 0, 37, 130, 1, 300], 256, 392
    bias_on = [True, False, False, True, True, False]
    po = ("relu",)
    descs, outs, refs, keep = _group_case(capi, oracle, Ms, K, N, dyn=dyn, dst=dst, bias_on=bias_on, postops=po, rng=rng, ldc_pad=8)
    for g in range(len(Ms)):
        descs[g].weights_const = 1          # packed once, on the first call
    capi.check(capi.lib.b200dnn_group_matmul(len(Ms), descs, None))
    for o in outs:
        o[:] = 0
    n0 = capi.lib.b200dnn_launch_count()
    capi.check(capi.lib.b200dnn_group_matmul(len(Ms), descs, None))
    launched = capi.lib.b200dnn_launch_count() - n0
    active = sum(1 for m in Ms if m)
    assert launched < active, "expected one grouped launch (plus one quantisation launch), saw %d launches" % launched
    capi.lib.b200dnn_clear_caches()
    for g, M in enumerate(Ms):
        if not M:
            assert not outs[g].any()
            continue
        got = outs[g][:M, :N]
        if dst == "bf16":
            assert_bf16_close(got, refs[g], 1, "expert %d" % g, atol=1e-5)
        else:
            assert np.allclose(got, refs[g], rtol=1e-5, atol=1e-5), g
        assert not outs[g][:, N:].any(), "padding columns of expert %d were written" % g


def test_group_matmul_equals_separate_calls_bit_for_bit(capi, oracle, monkeypatch):
    """Grouped launch against the same descriptors run one by one (B200DNN_GROUPED_PLAIN=0): identical bytes."""
    rng = np.random.default_rng(5)
    Ms, K, N = [129, 64, 0, 257], 512, 264
    descs, outs, refs, keep = _group_case(capi, oracle, Ms, K, N, dyn=False, dst="bf16", bias_on=[True] * 4, postops=(), rng=rng)
    capi.check(capi.lib.b200dnn_group_matmul(len(Ms), descs, None))
    grouped = [o.copy() for o in outs]
    for o in outs:
        o[:] = 0
    monkeypatch.setenv("B200DNN_GROUPED_PLAIN", "0")
    capi.check(capi.lib.b200dnn_group_matmul(len(Ms), descs, None))
    for g in range(len(Ms)):
        assert (grouped[g] == outs[g]).all(), g


def test_group_matmul_mixed_shapes_run_one_by_one(capi, oracle):
    """Experts that do not share one shape (here: differing N, and one decode-sized expert with a zero point) still
    compute, one launch each."""
    rng = np.random.default_rng(9)
    G = 3
    descs = (capi.MatmulDesc * G)()
    outs, refs, keep = [], [], []
    for g, (M, K, N) in enumerate([(40, 256, 128), (150, 256, 264), (3, 512, 136)]):
        A = rng.integers(-128, 128, (M, K), dtype=np.int8)
        W = rng.integers(-128, 128, (K, N), dtype=np.int8)
        sa = rng.uniform(0.01, 0.05, M).astype(np.float32)
        sw = rng.uniform(1e-4, 5e-4, N).astype(np.float32)
        out = np.zeros((M, N), dtype=np.uint16)
        descs[g] = capi.make_matmul(M, N, K, A, W, out, src_dt=capi.DT["s8"], dst_dt=capi.DT["bf16"], src_scale=sa, wei_scale=sw,
                                    weights_const=False)
        keep += [A, W, sa, sw]
        outs.append(out)
        refs.append(oracle.matmul_w8a8(A, W, "bf16", src_scale=sa, wei_scale=sw))
    capi.check(capi.lib.b200dnn_group_matmul(G, descs, None))
    for g in range(G):
        assert (outs[g] == refs[g]).all(), g
    # a negative M is refused
    descs[1].M = -1
    assert capi.lib.b200dnn_group_matmul(G, descs, None) == capi.FAILURE


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("dst", ["s8", "u8"])
def test_requantised_integer_destination(capi, oracle, kernel, dst):
    """s8 / u8 destinations: q = rne(clamp(x * dst_scale + dst_zp)) after bias and post-ops, as the reference's INT8
    cases with a quantised output tensor (zendnnl/gtests/test_matmul.cpp INT8; the definition is
    operators/matmul/matmul_ref_kernel.cpp:155-192,770-797).  A value whose f32 result sits within an ulp of a rounding
    boundary may land one step away: at most 0.2 % of the elements, never more than one step."""
    rng = np.random.default_rng(77)
    for M, K, N in [(4, 256, 136), (130, 384, 200), (300, 512, 1024)]:
        A = rng.integers(0, 256, (M, K), dtype=np.uint8)
        W = rng.integers(-128, 128, (K, N), dtype=np.int8)
        ss = np.array([0.02], dtype=np.float32)
        ws = rng.uniform(0.002, 0.01, N).astype(np.float32)
        bias = rng.standard_normal(N).astype(np.float32)
        zp_src = np.array([128], dtype=np.int32)
        ds = np.array([2.5], dtype=np.float32)
        dz = np.array([17 if dst == "u8" else -5], dtype=np.int32)
        for postops, use_zp, tol in (([], True, 1), (["relu"], False, 1), (["gelu_tanh"], True, 1)):
            x = oracle.matmul_w8a8(A, W, "f32", src_scale=ss, wei_scale=ws, src_zp=128, bias=bias, postops=postops)
            ref = oracle.requant_dst(x, dst, ds, dz if use_zp else None)
            got = run(capi, M, N, K, A, W, dst, weights_const=False, force_kernel=kernel, src_scale=ss, wei_scale=ws,
                      src_zp=zp_src, bias=bias, postops=postops, dst_scale=ds, dst_zp=dz if use_zp else None)
            diff = np.abs(got.astype(np.int32) - ref.astype(np.int32))
            assert diff.max() <= tol and (diff != 0).mean() < 2e-3, (M, K, N, postops, int(diff.max()), float((diff != 0).mean()))
            assert len(np.unique(got)) > 20       # the case covers the range, saturated ends included
    # strided destination, no scale (clamp and round only), device memory
    M, K, N, ldc = 33, 128, 72, 80
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    W = rng.integers(-128, 128, (K, N), dtype=np.int8)
    ws = np.full(1, 1e-3, dtype=np.float32)
    out = np.full((M, ldc), 99, dtype={"s8": np.int8, "u8": np.uint8}[dst])
    d = capi.make_matmul(M, N, K, A, W, out, src_dt=capi.DT["s8"], dst_dt=capi.DT[dst], ldc=ldc, weights_const=False,
                         force_kernel=kernel, wei_scale=ws)
    assert capi.matmul(d) == capi.SUCCESS, capi.last_error()
    ref = oracle.requant_dst(oracle.matmul_w8a8(A, W, "f32", wei_scale=ws), dst)
    assert np.abs(out[:, :N].astype(np.int32) - ref).max() <= 1 and (out[:, :N] != ref).mean() < 2e-3 and (out[:, N:] == 99).all()


def test_requantised_destination_contract(capi):
    M, K, N = 8, 64, 32
    A = np.zeros((M, K), dtype=np.int8); W = np.zeros((K, N), dtype=np.int8); out = np.zeros((M, N), dtype=np.int8)
    per_channel = np.ones(N, dtype=np.float32)
    d = capi.make_matmul(M, N, K, A, W, out, src_dt=capi.DT["s8"], dst_dt=capi.DT["s8"], weights_const=False, dst_scale=per_channel)
    assert capi.matmul(d) == capi.FAILURE and "per-tensor" in capi.last_error()
    d = capi.make_matmul(M, N, K, A, W, out, src_dt=capi.DT["s8"], dst_dt=capi.DT["s8"], weights_const=False,
                         dst_zp=np.zeros(1, dtype=np.int32))
    assert capi.matmul(d) == capi.UNIMPLEMENTED


def test_transposed_source(capi, oracle):
    """matmul_direct's transA: a source stored [K, lda] (element (m, k) at k * lda + m) gives the bytes of the untransposed
    call, on the INT8 path (u8 with a zero point, decode-sized and prefill-sized M) and on the bf16 path."""
    rng = np.random.default_rng(91)
    for M, K, N in [(4, 256, 136), (150, 328, 200)]:
        lda_t = M + 5
        A = rng.integers(0, 256, (M, K), dtype=np.uint8)
        At = np.zeros((K, lda_t), dtype=np.uint8); At[:, :M] = A.T
        W = rng.integers(-128, 128, (K, N), dtype=np.int8)
        ws = rng.uniform(0.002, 0.01, N).astype(np.float32)
        ss, zp = np.array([0.02], dtype=np.float32), np.array([128], dtype=np.int32)
        ref = run(capi, M, N, K, A, W, "bf16", weights_const=False, src_scale=ss, wei_scale=ws, src_zp=zp)
        got = run(capi, M, N, K, At, W, "bf16", weights_const=False, src_scale=ss, wei_scale=ws, src_zp=zp, transA=True, lda=lda_t,
                  src_dt=capi.DT["u8"])
        assert (got == ref).all(), (M, K, N)
        X = oracle.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
        Xt = np.zeros((K, lda_t), dtype=np.uint16); Xt[:, :M] = X.T
        Wb = oracle.f32_to_bf16((rng.standard_normal((K, N)) * 0.05).astype(np.float32))
        bf = capi.DT["bf16"]
        o0, o1 = np.zeros((M, N), dtype=np.uint16), np.zeros((M, N), dtype=np.uint16)
        assert capi.matmul(capi.make_matmul(M, N, K, X, Wb, o0, src_dt=bf, wei_dt=bf, dst_dt=bf, weights_const=False)) == capi.SUCCESS
        assert capi.matmul(capi.make_matmul(M, N, K, Xt, Wb, o1, src_dt=bf, wei_dt=bf, dst_dt=bf, weights_const=False, transA=True,
                                            lda=lda_t)) == capi.SUCCESS, capi.last_error()
        assert (o0 == o1).all() and o0.any()
