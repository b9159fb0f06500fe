"""GPU parity tests of the reorder_direct family (quantise / prepack) against the oracle.  The
reference checks these with quantise->dequantise round trips (zendnnl/gtests/reorder/
test_dynamic_quant.cpp:32,100, test_static_quant_dequant.cpp); here the s8 bytes and the scales
must equal the oracle's exactly, and the round-trip property is checked at full size."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    from zendnn_b200 import capi as c
    assert c.lib.b200dnn_device_count() > 0
    return c


@pytest.mark.parametrize("M,K", [(1, 16), (3, 100), (16, 4096), (33, 4097), (8, 14336), (5, 20000)])
@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_per_token_quant(capi, oracle, M, K, dt):
    rng = np.random.default_rng(M + K)
    x = rng.normal(size=(M, K)).astype(np.float32)
    if M > 2:
        x[1] = 0.0                     # all-zero row -> scale clamp 1e-10
        x[2, K // 2] = np.nan          # non-finite -> 0
        x[0, 0] = 1e30 if dt == "f32" else 3e38
    if dt == "bf16":
        x = oracle.f32_to_bf16(x)
    q_ref, s_ref = oracle.quant_per_token(x)
    q = np.zeros((M, K), dtype=np.int8); s = np.zeros(M, dtype=np.float32)
    st = capi.lib.b200dnn_quant_per_token(capi.ptr(x), capi.DT[dt], M, K, K, capi.ptr(q), K, capi.ptr(s), capi.DT["f32"], None)
    assert st == capi.SUCCESS, capi.last_error()
    assert (s == s_ref).all()
    assert (q == q_ref).all()
    # scales only (dst == NULL) and bf16 scale storage
    s16 = np.zeros(M, dtype=np.uint16)
    st = capi.lib.b200dnn_quant_per_token(capi.ptr(x), capi.DT[dt], M, K, K, None, 0, capi.ptr(s16), capi.DT["bf16"], None)
    assert st == capi.SUCCESS, capi.last_error()
    assert (s16 == oracle.f32_to_bf16(s_ref)).all()


def test_per_token_quant_strided(capi, oracle):
    rng = np.random.default_rng(0)
    M, K, ld, dld = 7, 120, 136, 128
    full = rng.normal(size=(M, ld)).astype(np.float32)
    q = np.full((M, dld), 99, dtype=np.int8); s = np.zeros(M, dtype=np.float32)
    st = capi.lib.b200dnn_quant_per_token(capi.ptr(full), capi.DT["f32"], M, K, ld, capi.ptr(q), dld, capi.ptr(s), capi.DT["f32"], None)
    assert st == capi.SUCCESS, capi.last_error()
    q_ref, s_ref = oracle.quant_per_token(np.ascontiguousarray(full[:, :K]))
    assert (q[:, :K] == q_ref).all() and (s == s_ref).all() and (q[:, K:] == 99).all()


def test_group_dynamic_quant(capi, oracle):
    """group_dynamic_quant: several tensors in one call, M == 0 groups skipped
    (zendnnl/gtests/group_matmul/test_quant.cpp:1284-1413)."""
    rng = np.random.default_rng(1)
    Ms = [0, 5, 1, 0, 17]
    K = 256
    xs = [oracle.f32_to_bf16(rng.normal(size=(max(m, 1), K)).astype(np.float32)) for m in Ms]
    qs = [np.zeros((max(m, 1), K), dtype=np.int8) for m in Ms]
    ss = [np.zeros(max(m, 1), dtype=np.float32) for m in Ms]
    G = len(Ms)
    arr = lambda xs_: (C.c_void_p * G)(*[x.ctypes.data for x in xs_])
    Mv = (C.c_int32 * G)(*Ms); Kv = (C.c_int32 * G)(*([K] * G)); ld = (C.c_int64 * G)(*([K] * G))
    st = capi.lib.b200dnn_group_quant_per_token(G, arr(xs), capi.DT["bf16"], Mv, Kv, ld, arr(qs), ld, arr(ss), capi.DT["f32"], None)
    assert st == capi.SUCCESS, capi.last_error()
    for m, x, q, s in zip(Ms, xs, qs, ss):
        if m == 0:
            assert not q.any() and not s.any()
            continue
        q_ref, s_ref = oracle.quant_per_token(x[:m])
        assert (q[:m] == q_ref).all() and (s[:m] == s_ref).all()


def test_group_dynamic_quant_with_differing_row_lengths(capi, oracle):
    """The reference lets K differ per group (lowoha_operators/reorder/lowoha_reorder.cpp:279-400): groups of one row
    length share a launch, every group gets its own K -- also when the first group is empty and a smaller group follows a
    larger one (a group must never be read or written with another group's row length)."""
    rng = np.random.default_rng(4)
    Ms, Ks = [0, 6, 4, 3, 5], [128, 256, 64, 256, 100]
    G = len(Ms)
    xs = [oracle.f32_to_bf16(rng.normal(size=(max(m, 1), k)).astype(np.float32)) for m, k in zip(Ms, Ks)]
    qs = [np.full((max(m, 1) + 1, k), 7, dtype=np.int8) for m, k in zip(Ms, Ks)]     # one guard row each
    ss = [np.full(max(m, 1) + 1, -1.0, dtype=np.float32) for m in Ms]
    arr = lambda xs_: (C.c_void_p * G)(*[x.ctypes.data for x in xs_])
    Mv = (C.c_int32 * G)(*Ms); Kv = (C.c_int32 * G)(*Ks); ld = (C.c_int64 * G)(*Ks)
    st = capi.lib.b200dnn_group_quant_per_token(G, arr(xs), capi.DT["bf16"], Mv, Kv, ld, arr(qs), ld, arr(ss), capi.DT["f32"], None)
    assert st == capi.SUCCESS, capi.last_error()
    for m, x, q, s in zip(Ms, xs, qs, ss):
        assert (q[m:] == 7).all() and (s[m:] == -1.0).all(), "rows beyond M were written"
        if m:
            q_ref, s_ref = oracle.quant_per_token(x[:m])
            assert (q[:m] == q_ref).all() and (s[:m] == s_ref).all()


@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("shape", [(1, 64), (7, 300), (33, 4096), (5, 11008)])
def test_asymmetric_per_token_quant(capi, oracle, shape, dt):
    """f32|bf16 -> u8 with one scale and one zero point per row, bit for bit against the oracle (itself pinned to both
    reference kernels): ordinary rows, a row with inf / nan entries, an all-zero row, a constant row, a strided source."""
    M, K = shape
    rng = np.random.default_rng(M + K)
    x32 = (rng.normal(size=(M, K)) * rng.uniform(0.01, 30, size=(M, 1)) + rng.normal(size=(M, 1))).astype(np.float32)
    if M > 4:
        x32[0, :3] = [np.inf, -np.inf, np.nan]
        x32[1, :] = 0
        x32[2, :] = 3.25
        x32[3, :] = np.abs(x32[3, :])          # a row without negative values
    x = oracle.f32_to_bf16(x32) if dt == "bf16" else x32
    ld = K + 8
    xs = np.zeros((M, ld), dtype=x.dtype); xs[:, :K] = x
    q = np.full((M, K), 99, dtype=np.uint8); s = np.zeros(M, dtype=np.float32); z = np.zeros(M, dtype=np.int32)
    st = capi.lib.b200dnn_quant_per_token_asym(capi.ptr(xs), capi.DT[dt], M, K, ld, capi.ptr(q), K, capi.ptr(s), capi.ptr(z), None)
    assert st == capi.SUCCESS, capi.last_error()
    q_ref, s_ref, z_ref = oracle.quant_per_token_asym(x)
    assert (s == s_ref).all() and (z == z_ref).all() and (q == q_ref).all()
    # scales and zero points only
    s2 = np.zeros(M, dtype=np.float32); z2 = np.zeros(M, dtype=np.int32)
    st = capi.lib.b200dnn_quant_per_token_asym(capi.ptr(xs), capi.DT[dt], M, K, ld, None, 0, capi.ptr(s2), capi.ptr(z2), None)
    assert st == capi.SUCCESS and (s2 == s_ref).all() and (z2 == z_ref).all()


@pytest.mark.parametrize("G", [2, 8, 32])
def test_per_group_dynamic_quant_through_the_per_token_entry(capi, oracle, G):
    """Per-group dynamic quantisation along K (scale layout {M,G}; reference kernel
    reorder/reorder_data_type/dynamic_quant_impl/per_group_avx512_f32_fma_kernel.cpp, to which the oracle is pinned): the
    C++ shims pass every (row, group) as a row of K/G elements."""
    rng = np.random.default_rng(G)
    M, K = 19, 256
    x = oracle.f32_to_bf16((rng.normal(size=(M, K)) * rng.uniform(0.01, 30, size=(M, 1))).astype(np.float32))
    x[3, 5] = 0x7F80     # +inf
    q = np.zeros((M, K), dtype=np.int8); s = np.zeros((M, G), dtype=np.float32)
    gs = K // G
    st = capi.lib.b200dnn_quant_per_token(capi.ptr(x), capi.DT["bf16"], M * G, gs, gs, capi.ptr(q), gs, capi.ptr(s), capi.DT["f32"], None)
    assert st == capi.SUCCESS, capi.last_error()
    q_ref, s_ref = oracle.quant_per_group(x, G)
    assert (q == q_ref).all() and (s == s_ref).all()


@pytest.mark.parametrize("K,N", [(64, 16), (300, 40), (4096, 1024)])
def test_per_channel_weight_quant(capi, oracle, K, N):
    rng = np.random.default_rng(K)
    w = oracle.f32_to_bf16((rng.normal(size=(K, N)) * 0.02).astype(np.float32))
    q_ref, s_ref = oracle.quant_weights_per_channel(w)
    q = np.zeros((K, N), dtype=np.int8); s = np.zeros(N, dtype=np.float32)
    st = capi.lib.b200dnn_quant_dynamic(capi.ptr(w), capi.DT["bf16"], K, N, N, 1, capi.ptr(q), N, capi.ptr(s), None)
    assert st == capi.SUCCESS, capi.last_error()
    assert (s == s_ref).all() and (q == q_ref).all()
    # per-tensor scale
    s1 = np.zeros(1, dtype=np.float32)
    st = capi.lib.b200dnn_quant_dynamic(capi.ptr(w), capi.DT["bf16"], K, N, N, 0, None, 0, capi.ptr(s1), None)
    assert st == capi.SUCCESS, capi.last_error()
    assert s1[0] == oracle.dyn_scales(w, per_channel=False)[0]


def test_static_quant_dequant_roundtrip(capi, oracle):
    rng = np.random.default_rng(2)
    M, N = 64, 96
    x = rng.uniform(-2, 2, size=(M, N)).astype(np.float32)
    scale = rng.uniform(0.01, 0.03, N).astype(np.float32)
    zp = rng.integers(-5, 5, N).astype(np.int32)
    q = np.zeros((M, N), dtype=np.int8)
    st = capi.lib.b200dnn_quant_static(capi.ptr(x), capi.DT["f32"], M, N, N, capi.ptr(scale), N, capi.ptr(zp), N, capi.ptr(q), capi.DT["s8"], N, None)
    assert st == capi.SUCCESS, capi.last_error()
    assert (q == oracle.quant_static(x, scale, zp)).all()
    back = np.zeros((M, N), dtype=np.float32)
    st = capi.lib.b200dnn_dequant_static(capi.ptr(q), capi.DT["s8"], M, N, N, capi.ptr(scale), N, capi.ptr(zp), N, capi.ptr(back), capi.DT["f32"], N, None)
    assert st == capi.SUCCESS, capi.last_error()
    assert (back == oracle.dequant_static(q, scale, zp)).all()
    unclipped = np.abs(np.rint(x / scale) + zp) < 127
    assert np.abs(back - x)[unclipped].max() <= scale.max() * 0.5 + 1e-6
    # u8 per-tensor
    qu = np.zeros((M, N), dtype=np.uint8)
    s1 = np.array([0.02], dtype=np.float32); z1 = np.array([128], dtype=np.int32)
    st = capi.lib.b200dnn_quant_static(capi.ptr(x), capi.DT["f32"], M, N, N, capi.ptr(s1), 1, capi.ptr(z1), 1, capi.ptr(qu), capi.DT["u8"], N, None)
    assert st == capi.SUCCESS, capi.last_error()
    assert (qu == oracle.quant_static(x, s1, z1, "u8")).all()


def _unblock(flat, Np, Kp):
    """Packed weight bytes Wt[Np/8][Kp/128][8][128] (rows interleaved eight at a time in 128-byte
    pieces) back to a plain [Np, Kp] row-major matrix."""
    return flat.reshape(Np // 8, Kp // 128, 8, 128).transpose(0, 2, 1, 3).reshape(Np, Kp)


@pytest.mark.parametrize("transB", [False, True])
@pytest.mark.parametrize("K,N", [(64, 16), (130, 200), (512, 384)])
def test_prepack_layout(capi, oracle, K, N, transB):
    """Packed form: header, column sums, K-major zero-padded rows."""
    rng = np.random.default_rng(K + N)
    W = rng.integers(-128, 128, (K, N), dtype=np.int8)
    src = np.ascontiguousarray(W.T) if transB else W
    size = capi.lib.b200dnn_prepack_size(K, N, 0)
    buf = np.zeros(size, dtype=np.uint8)
    st = capi.lib.b200dnn_prepack(capi.ptr(src), K, N, K if transB else N, int(transB), 0, capi.ptr(buf), None)
    assert st == capi.SUCCESS, capi.last_error()
    Kp, Np = -(-K // 128) * 128, -(-N // 128) * 128
    hdr = buf[:48].view(np.int64)
    assert int(buf[:4].view(np.uint32)[0]) == 0x38573242 and list(hdr[1:5]) == [K, N, Kp, Np]
    colsum = buf[256:256 + 4 * Np].view(np.int32)
    wt = _unblock(buf[256 + 4 * Np:256 + 4 * Np + Np * Kp].view(np.int8), Np, Kp)
    assert (wt[:N, :K] == W.T).all() and not wt[N:].any() and not wt[:, K:].any()
    assert (colsum[:N] == W.astype(np.int32).sum(axis=0)).all() and not colsum[N:].any()


def test_prepack_gated_interleave(capi):
    rng = np.random.default_rng(5)
    K, I = 128, 64
    W = rng.integers(-128, 128, (K, 2 * I), dtype=np.int8)
    size = capi.lib.b200dnn_prepack_size(K, 2 * I, 1)
    buf = np.zeros(size, dtype=np.uint8)
    assert capi.lib.b200dnn_prepack(capi.ptr(W), K, 2 * I, 2 * I, 0, 1, capi.ptr(buf), None) == capi.SUCCESS, capi.last_error()
    Np = 128
    wt = _unblock(buf[256 + 4 * Np:256 + 4 * Np + Np * 128].view(np.int8), Np, 128)
    # packed rows: g[0:32] u[0:32] g[32:64] u[32:64]
    exp = np.concatenate([W[:, 0:32], W[:, I:I + 32], W[:, 32:64], W[:, I + 32:I + 64]], axis=1).T
    assert (wt == exp).all()


@pytest.mark.parametrize("gated", [0, 1, 2])
@pytest.mark.parametrize("transB", [False, True])
@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("K,N", [(64, 64), (300, 192), (1024, 4096)])
def test_quant_prepack_one_call(capi, oracle, K, N, dt, transB, gated):
    """Float weight -> per-channel s8 -> packed layout in one call: the scales are the oracle's, and the packed buffer is
    byte for byte the one that per-channel quantisation followed by the prepack writes."""
    rng = np.random.default_rng(K * 3 + N + gated)
    wf = (rng.normal(size=(K, N)) * rng.uniform(0.005, 0.05, size=(1, N))).astype(np.float32)
    wf[:, 3] = 0.0                                   # an all-zero channel
    w = oracle.f32_to_bf16(wf) if dt == "bf16" else wf
    q_ref, s_ref = oracle.quant_weights_per_channel(w)
    src = np.ascontiguousarray(w.T) if transB else w
    ldb = K if transB else N
    size = capi.lib.b200dnn_prepack_size(K, N, gated)
    one = np.zeros(size, dtype=np.uint8)
    s = np.zeros(N, dtype=np.float32)
    st = capi.lib.b200dnn_quant_prepack(capi.ptr(src), capi.DT[dt], K, N, ldb, int(transB), gated, capi.ptr(one), capi.ptr(s), None)
    assert st == capi.SUCCESS, capi.last_error()
    assert (s == s_ref).all()
    # the two calls it replaces
    q = np.zeros((K, N), dtype=np.int8); s2 = np.zeros(N, dtype=np.float32)
    st = capi.lib.b200dnn_quant_dynamic(capi.ptr(w), capi.DT[dt], K, N, N, 1, capi.ptr(q), N, capi.ptr(s2), None)
    assert st == capi.SUCCESS, capi.last_error()
    assert (q == q_ref).all()
    two = np.zeros(size, dtype=np.uint8)
    assert capi.lib.b200dnn_prepack(capi.ptr(q), K, N, N, 0, gated, capi.ptr(two), None) == capi.SUCCESS, capi.last_error()
    Np = -(-N // 128) * 128
    assert (one[:256] == two[:256]).all(), "header"
    assert (one[256:256 + 4 * Np] == two[256:256 + 4 * Np]).all(), "column sums"
    assert (one == two).all(), int((one != two).sum())


@pytest.mark.parametrize("transB", [False, True])
@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("K,N,pad", [(130, 100, 0), (70, 13, 0), (96, 40, 3)])
def test_quant_prepack_ragged(capi, oracle, K, N, pad, dt, transB):
    """Shapes that are no multiple of the tile or of a 16-byte load, and a padded leading dimension."""
    rng = np.random.default_rng(K + N)
    wf = (rng.normal(size=(K, N)) * 0.02).astype(np.float32)
    w = oracle.f32_to_bf16(wf) if dt == "bf16" else wf
    q_ref, s_ref = oracle.quant_weights_per_channel(w)
    lay = np.ascontiguousarray(w.T) if transB else w
    ldb = lay.shape[1] + pad
    src = np.zeros((lay.shape[0], ldb), dtype=lay.dtype)
    src[:, :lay.shape[1]] = lay
    size = capi.lib.b200dnn_prepack_size(K, N, 0)
    one = np.zeros(size, dtype=np.uint8); two = np.zeros(size, dtype=np.uint8)
    s = np.zeros(N, dtype=np.float32)
    st = capi.lib.b200dnn_quant_prepack(capi.ptr(src), capi.DT[dt], K, N, ldb, int(transB), 0, capi.ptr(one), capi.ptr(s), None)
    assert st == capi.SUCCESS, capi.last_error()
    assert (s == s_ref).all()
    assert capi.lib.b200dnn_prepack(capi.ptr(q_ref), K, N, N, 0, 0, capi.ptr(two), None) == capi.SUCCESS, capi.last_error()
    assert (one == two).all(), int((one != two).sum())


@pytest.mark.parametrize("transB", [False, True])
def test_quant_prepack_non_finite(capi, transB):
    """inf and nan in the weight: ignored by the channel maxima, and coded as the two separate calls code them."""
    rng = np.random.default_rng(9)
    K, N = 192, 128
    w = (rng.normal(size=(K, N)) * 0.02).astype(np.float32)
    w[3, 5], w[100, 5], w[7, 64], w[191, 127] = np.inf, -np.inf, np.nan, np.inf
    src = np.ascontiguousarray(w.T) if transB else w
    size = capi.lib.b200dnn_prepack_size(K, N, 0)
    one = np.zeros(size, dtype=np.uint8); two = np.zeros(size, dtype=np.uint8)
    s1 = np.zeros(N, dtype=np.float32); s2 = np.zeros(N, dtype=np.float32)
    st = capi.lib.b200dnn_quant_prepack(capi.ptr(src), capi.DT["f32"], K, N, K if transB else N, int(transB), 0, capi.ptr(one), capi.ptr(s1), None)
    assert st == capi.SUCCESS, capi.last_error()
    q = np.zeros((K, N), dtype=np.int8)
    st = capi.lib.b200dnn_quant_dynamic(capi.ptr(w), capi.DT["f32"], K, N, N, 1, capi.ptr(q), N, capi.ptr(s2), None)
    assert st == capi.SUCCESS, capi.last_error()
    assert capi.lib.b200dnn_prepack(capi.ptr(q), K, N, N, 0, 0, capi.ptr(two), None) == capi.SUCCESS, capi.last_error()
    assert np.isfinite(s1).all() and (s1 == s2).all()
    assert (one == two).all(), int((one != two).sum())


def test_quant_prepack_feeds_matmul(capi, oracle):
    """The buffer of the one-call form is a prepacked weight: matmul_direct on it gives the oracle's bytes for the
    quantised weight and its scales."""
    rng = np.random.default_rng(77)
    M, K, N = 48, 512, 384
    w = oracle.f32_to_bf16((rng.normal(size=(K, N)) * 0.03).astype(np.float32))
    q_ref, s_ref = oracle.quant_weights_per_channel(w)
    packed = np.zeros(capi.lib.b200dnn_prepack_size(K, N, 0), dtype=np.uint8)
    sw = np.zeros(N, dtype=np.float32)
    st = capi.lib.b200dnn_quant_prepack(capi.ptr(w), capi.DT["bf16"], K, N, N, 0, 0, capi.ptr(packed), capi.ptr(sw), None)
    assert st == capi.SUCCESS, capi.last_error()
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    sa = rng.uniform(0.01, 0.05, M).astype(np.float32)
    dst = np.zeros((M, N), dtype=np.uint16)
    d = capi.make_matmul(M, N, K, A, packed, dst, src_dt=capi.DT["s8"], dst_dt=capi.DT["bf16"], wei_format="r",
                         src_scale=sa, wei_scale=sw)
    assert capi.matmul(d) == capi.SUCCESS, capi.last_error()
    ref = oracle.matmul_w8a8(A, q_ref, "bf16", src_scale=sa, wei_scale=s_ref)
    assert (dst == ref).all()


def test_quant_prepack_contract(capi):
    w = np.zeros((64, 64), dtype=np.float32)
    buf = np.zeros(capi.lib.b200dnn_prepack_size(64, 64, 0), dtype=np.uint8)
    s = np.zeros(64, dtype=np.float32)
    f = capi.lib.b200dnn_quant_prepack
    assert f(None, capi.DT["f32"], 64, 64, 64, 0, 0, capi.ptr(buf), capi.ptr(s), None) == capi.FAILURE
    assert f(capi.ptr(w), capi.DT["f32"], 64, 64, 32, 0, 0, capi.ptr(buf), capi.ptr(s), None) == capi.FAILURE
    assert f(capi.ptr(w), capi.DT["s8"], 64, 64, 64, 0, 0, capi.ptr(buf), capi.ptr(s), None) == capi.UNIMPLEMENTED
    assert f(capi.ptr(w), capi.DT["f32"], 64, 48, 64, 0, 1, capi.ptr(buf), capi.ptr(s), None) == capi.UNIMPLEMENTED
