"""GPU parity tests of b200dnn_sdpa (sdpa_direct: softmax(Q K^T * scale + mask) V) against the CPU oracle, which follows the
steps of the reference's BMM backend with exact dot products.  Tolerance: 2 bf16 ulp, or 1e-3 of the largest |V| entry
absolute (an output is a convex combination of V rows; probabilities are rounded to bf16 on both sides, sums differ in
their f32 order)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    from zendnn_b200 import capi as c
    assert c.lib.b200dnn_device_count() > 0, "no CUDA device"
    return c


def strides_of(a):
    return [s // a.itemsize for s in a.strides]


def run(capi, q, k, v, mask=None, scale=0.0, causal=False, out=None):
    B, H, S, D = q.shape
    KV = k.shape[2]
    if out is None:
        out = np.zeros((B, H, S, D), dtype=np.uint16)
    d = capi.SdpaDesc()
    d.batch, d.num_heads, d.seq_len, d.kv_seq_len, d.head_dim = B, H, S, KV, D
    for name, arr in (("q_stride", q), ("k_stride", k), ("v_stride", v), ("o_stride", out)):
        setattr(d, name, (C.c_int64 * 4)(*strides_of(arr)))
    d.qkv_dt = d.out_dt = capi.DT["bf16"]
    d.scale, d.dropout_p, d.is_causal = scale, 0.0, int(causal)
    if mask is not None:
        d.mask_ndims = mask.ndim
        d.mask_sizes = (C.c_int64 * 4)(*(list(mask.shape) + [0] * (4 - mask.ndim)))
        d.mask_strides = (C.c_int64 * 4)(*(strides_of(mask) + [0] * (4 - mask.ndim)))
        d.mask_dt = capi.dt_of(mask)
        d.attn_mask = mask.ctypes.data
    d.query, d.key, d.value, d.output = q.ctypes.data, k.ctypes.data, v.ctypes.data, out.ctypes.data
    st = capi.lib.b200dnn_sdpa(C.byref(d), None)
    return st, out


def close(oracle, got, ref, v, what):
    from helpers import bf16_ulp_diff
    dd = bf16_ulp_diff(got, ref)
    g, r = oracle.bf16_to_f32(got), oracle.bf16_to_f32(ref)
    ok = (dd <= 2) | (np.abs(g - r) <= 1e-3 * np.abs(oracle.bf16_to_f32(v)).max())
    assert ok.all(), "%s: %d of %d elements off (max %d ulp)" % (what, int((~ok).sum()), ok.size, int(dd.max()))
    assert (dd == 0).mean() > 0.9, (what, float((dd == 0).mean()))


def make(oracle, rng, B, H, S, KV, D):
    q = oracle.f32_to_bf16(rng.standard_normal((B, H, S, D)).astype(np.float32))
    k = oracle.f32_to_bf16(rng.standard_normal((B, H, KV, D)).astype(np.float32))
    v = oracle.f32_to_bf16(rng.standard_normal((B, H, KV, D)).astype(np.float32))
    return q, k, v


@pytest.mark.parametrize("shape", [(1, 1, 8, 8, 16), (2, 3, 50, 50, 64), (1, 4, 300, 300, 128), (2, 2, 17, 260, 80), (1, 2, 256, 100, 64)])
@pytest.mark.parametrize("causal", [False, True])
def test_plain_and_causal(capi, oracle, shape, causal):
    B, H, S, KV, D = shape
    rng = np.random.default_rng(S + KV + D)
    q, k, v = make(oracle, rng, B, H, S, KV, D)
    st, out = run(capi, q, k, v, causal=causal)
    assert st == capi.SUCCESS, capi.last_error()
    close(oracle, out, oracle.sdpa(q, k, v, causal=causal), v, (shape, causal))


def test_head_by_head_form_on_contiguous_tensors(capi, oracle, monkeypatch):
    """Contiguous [batch, head, seq, dim] tensors take the grouped launches; the head-by-head form must give the same answer
    (to the tolerance), here with a 4-D mask and the causal mask together."""
    monkeypatch.setenv("B200DNN_SDPA_GROUPED", "0")
    rng = np.random.default_rng(8)
    B, H, S, KV, D = 2, 2, 130, 130, 64
    q, k, v = make(oracle, rng, B, H, S, KV, D)
    m4 = rng.standard_normal((B, H, S, KV)).astype(np.float32)
    st, out = run(capi, q, k, v, mask=m4, causal=True)
    assert st == capi.SUCCESS, capi.last_error()
    close(oracle, out, oracle.sdpa(q, k, v, m4, causal=True), v, "head by head")
    monkeypatch.setenv("B200DNN_SDPA_GROUPED", "1")
    st, out2 = run(capi, q, k, v, mask=m4, causal=True)
    assert st == capi.SUCCESS, capi.last_error()
    close(oracle, out2, oracle.sdpa(q, k, v, m4, causal=True), v, "grouped")


def test_masks_scale_and_strides(capi, oracle):
    rng = np.random.default_rng(5)
    B, H, S, KV, D = 2, 3, 70, 90, 64
    # [batch, seq, head, dim] storage seen through [b, h, s, d] strides
    def bshd(n):
        base = oracle.f32_to_bf16(rng.standard_normal((B, n, H, D)).astype(np.float32))
        return base.transpose(0, 2, 1, 3)
    q, k, v = bshd(S), bshd(KV), bshd(KV)
    out = np.zeros((B, S, H, D), dtype=np.uint16).transpose(0, 2, 1, 3)
    m2 = rng.standard_normal((S, KV)).astype(np.float32)
    m2[:, 5] = -np.inf                                            # a key nobody may attend to
    st, got = run(capi, q, k, v, mask=m2, scale=0.2, out=out)
    assert st == capi.SUCCESS, capi.last_error()
    close(oracle, np.ascontiguousarray(got), oracle.sdpa(np.ascontiguousarray(q), np.ascontiguousarray(k), np.ascontiguousarray(v), m2, 0.2),
          np.ascontiguousarray(v), "2-D mask, scale, strided tensors")
    # 4-D masks: per batch and head, and a padding mask broadcast over heads and queries (bf16 storage)
    m4 = rng.standard_normal((B, H, S, KV)).astype(np.float32)
    st, got = run(capi, q, k, v, mask=m4, out=out)
    assert st == capi.SUCCESS, capi.last_error()
    close(oracle, np.ascontiguousarray(got), oracle.sdpa(np.ascontiguousarray(q), np.ascontiguousarray(k), np.ascontiguousarray(v), m4),
          np.ascontiguousarray(v), "4-D mask")
    pad = np.zeros((B, 1, 1, KV), dtype=np.float32)
    pad[0, :, :, 60:] = -np.inf
    pad[1, :, :, 33:] = -np.inf
    pad_bf = oracle.f32_to_bf16(pad)
    st, got = run(capi, q, k, v, mask=pad_bf, causal=True, out=out)
    assert st == capi.SUCCESS, capi.last_error()
    close(oracle, np.ascontiguousarray(got), oracle.sdpa(np.ascontiguousarray(q), np.ascontiguousarray(k), np.ascontiguousarray(v), pad, causal=True),
          np.ascontiguousarray(v), "padding mask + causal")


def test_contract(capi, oracle):
    rng = np.random.default_rng(1)
    q, k, v = make(oracle, rng, 1, 1, 8, 8, 16)
    d_ok, _ = run(capi, q, k, v)
    assert d_ok == capi.SUCCESS
    m = np.zeros((8, 8), dtype=np.float32)
    d = capi.SdpaDesc()
    d.batch = d.num_heads = 1
    d.seq_len = d.kv_seq_len = 8
    d.head_dim = 16
    for name in ("q_stride", "k_stride", "v_stride", "o_stride"):
        setattr(d, name, (C.c_int64 * 4)(128, 128, 16, 1))
    out = np.zeros((1, 1, 8, 16), dtype=np.uint16)
    d.query, d.key, d.value, d.output = q.ctypes.data, k.ctypes.data, v.ctypes.data, out.ctypes.data
    d.qkv_dt = d.out_dt = capi.DT["bf16"]
    d.dropout_p = 0.1
    assert capi.lib.b200dnn_sdpa(C.byref(d), None) == capi.FAILURE and "dropout" in capi.last_error()
    d.dropout_p = 0.0
    d.attn_mask = m.ctypes.data
    assert capi.lib.b200dnn_sdpa(C.byref(d), None) == capi.FAILURE and "mask_ndims" in capi.last_error()
    d.attn_mask = None
    d.qkv_dt = d.out_dt = capi.DT["f32"]
    assert capi.lib.b200dnn_sdpa(C.byref(d), None) == capi.UNIMPLEMENTED
    d.qkv_dt = capi.DT["bf16"]
    assert capi.lib.b200dnn_sdpa(C.byref(d), None) == capi.FAILURE and "out_dt" in capi.last_error()
    d.out_dt = capi.DT["bf16"]
    d.q_stride = (C.c_int64 * 4)(128, 128, 16, 2)
    assert capi.lib.b200dnn_sdpa(C.byref(d), None) == capi.FAILURE
