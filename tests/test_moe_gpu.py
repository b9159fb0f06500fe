"""GPU parity tests of the fused-MoE path (group_matmul_direct with fused_moe + gated_act +
moe_postop) against the oracle's statement of the reference data flow.  Mirrors
TestGatedAct.Correctness / TestMoEPostop.Correctness (zendnnl/gtests/group_matmul/test_basic.cpp:464,655)
and TestFusedMoEQuantDynINT8.BothPasses (test_fused_moe.cpp:2491-2721), including M_e = 0 experts,
skewed M_e and the sum|out| > 1e-3 anti-vacuity guard."""
import ctypes as C

import numpy as np
import pytest

from helpers import assert_bf16_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    from zendnn_b200 import capi as c
    assert c.lib.b200dnn_device_count() > 0
    return c


@pytest.mark.parametrize("act", ["silu_and_mul", "gelu_and_mul", "swiglu_oai_mul"])
@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_gated_act(capi, oracle, act, dt):
    rng = np.random.default_rng(1)
    M, N, ldc = 9, 600, 640
    y = (rng.normal(size=(M, ldc)) * 3).astype(np.float32)
    if dt == "bf16":
        y = oracle.f32_to_bf16(y)
    ref = oracle.gated_act(np.ascontiguousarray(y[:, :N]), act)
    buf = y.copy()
    st = capi.lib.b200dnn_gated_act(capi.ptr(buf), capi.DT[dt], M, N, ldc, capi.ACT[act], None)
    assert st == capi.SUCCESS, capi.last_error()
    got = buf[:, :N // 2]
    if dt == "bf16":
        assert_bf16_close(got, ref, 1, act, atol=1e-5)
    else:
        assert np.allclose(got, ref, rtol=1e-5, atol=1e-6)
    assert (buf[:, N:] == y[:, N:]).all()


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_weighted_reduce(capi, oracle, dt):
    rng = np.random.default_rng(2)
    T, k, D = 37, 3, 264
    rows = rng.normal(size=(T * k, D)).astype(np.float32)
    if dt == "bf16":
        rows = oracle.f32_to_bf16(rows)
    w = rng.uniform(size=(T, k)).astype(np.float32)
    perm = rng.permutation(T * k)          # rows live anywhere: row_ptrs gathers them
    ptrs = (C.c_void_p * (T * k))(*[rows.ctypes.data + int(perm[i]) * rows.strides[0] for i in range(T * k)])
    out = np.zeros((T, D), dtype=rows.dtype)
    st = capi.lib.b200dnn_moe_weighted_reduce(ptrs, capi.ptr(w), T, k, D, 0, capi.DT[dt], capi.ptr(out), D, None)
    assert st == capi.SUCCESS, capi.last_error()
    ref = oracle.moe_weighted_reduce(rows[perm], w, k, fused=True)
    assert (out == ref).all()
    st = capi.lib.b200dnn_moe_weighted_reduce(ptrs, None, T, k, D, 1, capi.DT[dt], capi.ptr(out), D, None)
    assert st == capi.SUCCESS, capi.last_error()
    assert (out == oracle.moe_weighted_reduce(rows[perm], w, k, skip_weighted=True, fused=True)).all()


@pytest.mark.parametrize("T,E,k", [(64, 8, 2), (1000, 64, 6)])
def test_router(capi, oracle, T, E, k):
    rng = np.random.default_rng(3)
    logits = rng.normal(size=(T, E)).astype(np.float32)
    ids = np.zeros((T, k), dtype=np.int32); w = np.zeros((T, k), dtype=np.float32)
    cnt = np.zeros(E, dtype=np.int32); s2r = np.zeros((T, k), dtype=np.int32)
    st = capi.lib.b200dnn_moe_route(capi.ptr(logits), T, E, k, 1, capi.ptr(ids), capi.ptr(w), capi.ptr(cnt), capi.ptr(s2r), None)
    assert st == capi.SUCCESS, capi.last_error()
    ids_ref, w_ref = oracle.router_topk(logits, k)
    assert (ids == ids_ref).all()
    assert np.allclose(w, w_ref, rtol=2e-6, atol=1e-8)
    assert (cnt == np.bincount(ids.reshape(-1), minlength=E)).all()
    # stable expert-sorted order
    order = np.argsort(ids.reshape(-1), kind="stable")
    exp = np.empty(T * k, dtype=np.int32); exp[order] = np.arange(T * k)
    assert (s2r.reshape(-1) == exp).all()


def _experts(oracle, rng, E, H, I):
    w13, s13, w2, s2 = [], [], [], []
    for _ in range(E):
        q, s = oracle.quant_weights_per_channel(oracle.f32_to_bf16((rng.normal(size=(H, 2 * I)) * 0.02).astype(np.float32)))
        w13.append(q); s13.append(s)
        q, s = oracle.quant_weights_per_channel(oracle.f32_to_bf16((rng.normal(size=(I, H)) * 0.02).astype(np.float32)))
        w2.append(q); s2.append(s)
    return w13, s13, w2, s2


@pytest.mark.parametrize("T,H,I,E,k,act", [(48, 128, 64, 4, 2, "silu_and_mul"), (300, 256, 160, 6, 2, "silu_and_mul"),
                                           (64, 128, 96, 3, 1, "gelu_and_mul"), (64, 128, 64, 4, 2, "swiglu_oai_mul")])
@pytest.mark.parametrize("pair", ["0", "1"])
def test_fused_moe_reference_contract(capi, oracle, monkeypatch, pair, T, H, I, E, k, act):
    """Rows gathered by the caller, per-expert dst_down, row_ptrs + top-k weights: the group_matmul_direct contract.
    pair: the grouped GEMMs run in the single-CTA form or in the two-CTA (cta_group::2) form."""
    monkeypatch.setenv("B200DNN_TC_PAIR", pair)
    rng = np.random.default_rng(T + I)
    x = oracle.f32_to_bf16(rng.normal(size=(T, H)).astype(np.float32))
    logits = rng.normal(size=(T, E)).astype(np.float32)
    logits[:, 1] = -1e4                      # expert 1 receives no token: M_e = 0
    ids, w = oracle.router_topk(logits, k)
    w13, s13, w2, s2 = _experts(oracle, rng, E, H, I)
    out_ref, slot_ref = oracle.fused_moe(x, ids, w, w13, s13, w2, s2, act)
    flat = ids.reshape(-1)
    srcs, dsts, experts = [], [], (capi.MoeExpert * E)()
    ptrs = (C.c_void_p * (T * k))()
    for e in range(E):
        slots = np.nonzero(flat == e)[0]
        src = np.ascontiguousarray(x[slots // k]) if slots.size else np.zeros((1, H), dtype=np.uint16)
        dst = np.zeros((max(slots.size, 1), H), dtype=np.uint16)
        srcs.append(src); dsts.append(dst)
        ex = experts[e]
        ex.M = int(slots.size); ex.src = src.ctypes.data; ex.lda = H
        ex.w13 = w13[e].ctypes.data; ex.ldb13 = 2 * I; ex.w13_scale = s13[e].ctypes.data
        ex.w2 = w2[e].ctypes.data; ex.ldb2 = H; ex.w2_scale = s2[e].ctypes.data
        ex.dst_down = dst.ctypes.data; ex.ldc_down = H
        for r, s in enumerate(slots):
            ptrs[int(s)] = dst.ctypes.data + r * dst.strides[0]
    out = np.zeros((T, H), dtype=np.uint16)
    st = capi.lib.b200dnn_fused_moe(E, experts, H, I, H, 0, capi.ACT[act], 0, ptrs, capi.ptr(w), T, k, capi.ptr(out), H, None)
    assert st == capi.SUCCESS, capi.last_error()
    assert np.abs(oracle.bf16_to_f32(out)).sum() > 1e-3
    for e in range(E):
        slots = np.nonzero(flat == e)[0]
        if slots.size:
            assert_bf16_close(dsts[e][:slots.size], slot_ref[slots], 1, "expert %d down output" % e)
    assert_bf16_close(out, out_ref, 1, "moe output")
    capi.lib.b200dnn_clear_caches()


@pytest.mark.parametrize("T,H,I,E,k,S", [(256, 256, 128, 8, 2, 0), (512, 128, 96, 16, 4, 2), (1500, 256, 320, 4, 2, 1)])
@pytest.mark.parametrize("pair", ["0", "1"])
def test_moe_layer_end_to_end(capi, oracle, monkeypatch, pair, T, H, I, E, k, S):
    """Router + permutation + fused MoE + un-permute on the device; shared experts see every token with weight 1."""
    monkeypatch.setenv("B200DNN_TC_PAIR", pair)
    rng = np.random.default_rng(E)
    x = oracle.f32_to_bf16(rng.normal(size=(T, H)).astype(np.float32))
    bias = np.log(np.arange(1, E + 1, dtype=np.float64) ** -1.1)      # skewed load
    logits = (rng.normal(size=(T, E)) + rng.permutation(bias)).astype(np.float32)
    w13, s13, w2, s2 = _experts(oracle, rng, E + S, H, I)
    ids, w = oracle.router_topk(logits, k)
    ids_all = np.concatenate([ids, np.tile(np.arange(E, E + S, dtype=np.int32), (T, 1))], axis=1)
    w_all = np.concatenate([w, np.ones((T, S), dtype=np.float32)], axis=1)
    out_ref, _ = oracle.fused_moe(x, ids_all, w_all, w13, s13, w2, s2)
    experts = (capi.MoeExpert * (E + S))()
    for e in range(E + S):
        ex = experts[e]
        ex.w13 = w13[e].ctypes.data; ex.ldb13 = 2 * I; ex.w13_scale = s13[e].ctypes.data
        ex.w2 = w2[e].ctypes.data; ex.ldb2 = H; ex.w2_scale = s2[e].ctypes.data
    out = np.zeros((T, H), dtype=np.uint16)
    st = capi.lib.b200dnn_moe_layer(capi.ptr(x), H, capi.ptr(logits), T, E, S, k, experts, H, I, H, 0, capi.ACT["silu_and_mul"],
                                    capi.ptr(out), H, None)
    assert st == capi.SUCCESS, capi.last_error()
    assert np.abs(oracle.bf16_to_f32(out)).sum() > 1e-3
    assert_bf16_close(out, out_ref, 1, "moe layer")
    capi.lib.b200dnn_clear_caches()


@pytest.mark.parametrize("pair", ["0", "1"])
def test_moe_layer_with_biases(capi, oracle, monkeypatch, pair):
    """Biases on both GEMMs of the fused block (the reference's bias[] and fused.bias_down[]): added after the
    dequantisation, before the gated activation / to the down projection."""
    monkeypatch.setenv("B200DNN_TC_PAIR", pair)
    T, H, I, E, k = 700, 256, 192, 5, 2
    rng = np.random.default_rng(77)
    x = oracle.f32_to_bf16(rng.normal(size=(T, H)).astype(np.float32))
    logits = rng.normal(size=(T, E)).astype(np.float32)
    w13, s13, w2, s2 = _experts(oracle, rng, E, H, I)
    b13 = [rng.normal(size=2 * I).astype(np.float32) * 0.3 for _ in range(E)]
    b2 = [rng.normal(size=H).astype(np.float32) * 0.3 for _ in range(E)]
    ids, w = oracle.router_topk(logits, k)
    out_ref, _ = oracle.fused_moe(x, ids, w, w13, s13, w2, s2, b13=b13, b2=b2)
    experts = (capi.MoeExpert * E)()
    for e in range(E):
        ex = experts[e]
        ex.w13 = w13[e].ctypes.data; ex.ldb13 = 2 * I; ex.w13_scale = s13[e].ctypes.data
        ex.w2 = w2[e].ctypes.data; ex.ldb2 = H; ex.w2_scale = s2[e].ctypes.data
        ex.bias13 = b13[e].ctypes.data; ex.bias13_dt = capi.DT["f32"]
        ex.bias2 = b2[e].ctypes.data; ex.bias2_dt = capi.DT["f32"]
    out = np.zeros((T, H), dtype=np.uint16)
    st = capi.lib.b200dnn_moe_layer(capi.ptr(x), H, capi.ptr(logits), T, E, 0, k, experts, H, I, H, 0, capi.ACT["silu_and_mul"],
                                    capi.ptr(out), H, None)
    assert st == capi.SUCCESS, capi.last_error()
    assert_bf16_close(out, out_ref, 1, "moe layer with biases")
    capi.lib.b200dnn_clear_caches()
