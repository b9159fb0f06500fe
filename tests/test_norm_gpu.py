"""GPU parity tests of b200dnn_normalization (normalization_direct: LayerNorm, RMSNorm, fused-add RMSNorm, BatchNorm) against
the CPU oracle, which equals the reference's scalar kernel bit for bit (tests/test_oracle.py), and against that kernel's
committed outputs.  The device adds the row sums in a tree, the reference sequentially: f32 results agree to a few f32 ulp
of the row scale ((2e-6 + 2.4e-7 * sqrt(n)) * (|ref| + max|row|): the sequential sum's own error grows with the row
length), bf16 results within 1 bf16 ulp with at least 99.5 % of them equal.
The fused quantised output (no reference counterpart) must equal the per-token quantisation of the SAME call's bf16 output
bit for bit."""
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


def run(capi, kind, x, gamma=None, beta=None, residual=None, rm=None, rv=None, eps=1e-5, dst_dt=None, quant=False, want_output=True):
    x = np.ascontiguousarray(x)
    dst_dt = dst_dt or ("bf16" if x.dtype == np.uint16 else "f32")
    d = capi.NormDesc()
    d.norm_type = capi.NORM[kind]
    if kind == "batch_norm":
        d.batch, d.num_channels, d.norm_size = x.shape[0], x.shape[1], int(np.prod(x.shape[2:]))
    else:
        d.batch, d.norm_size = int(np.prod(x.shape[:-1])), x.shape[-1]
    d.epsilon = eps
    d.use_scale, d.use_shift = int(gamma is not None), int(beta is not None)
    d.src_dt, d.dst_dt = capi.dt_of(x), capi.DT[dst_dt]
    d.gamma_dt = capi.dt_of(gamma) if gamma is not None else capi.DT["f32"]
    d.beta_dt = capi.dt_of(beta) if beta is not None else capi.DT["f32"]
    out = np.zeros(x.shape, dtype={"bf16": np.uint16, "f32": np.float32}[dst_dt])
    res = None if residual is None else np.array(residual, copy=True, order="C")
    d.input = x.ctypes.data
    d.output = out.ctypes.data if want_output else None
    keep = [np.ascontiguousarray(a) if a is not None else None for a in (gamma, beta, rm, rv)]
    d.gamma, d.beta, d.running_mean, d.running_var = [None if a is None else a.ctypes.data for a in keep]
    d.residual = None if res is None else res.ctypes.data
    q = s = None
    if quant:
        q = np.zeros((d.batch, d.norm_size), dtype=np.int8)
        s = np.zeros(d.batch, dtype=np.float32)
        d.quant_dst, d.quant_ld, d.quant_scale = q.ctypes.data, d.norm_size, s.ctypes.data
    st = capi.lib.b200dnn_normalization(C.byref(d), None)
    return st, out, res, q, s


def close(oracle, got, ref, what):
    # the reference's sequential f32 sum over n terms carries about sqrt(n) * 2^-22 of relative error itself
    n = ref.shape[-1]
    tol = 2e-6 + 2.4e-7 * np.sqrt(n)
    if got.dtype == np.uint16:
        from helpers import bf16_ulp_diff
        dd = bf16_ulp_diff(got, ref)
        g, r = oracle.bf16_to_f32(got), oracle.bf16_to_f32(ref)
        # x - mean nearly cancels for elements beside the mean: those are held to the f32 bound on the row's scale
        small = np.abs(g - r) <= tol * np.abs(r).max(axis=-1, keepdims=True)
        assert ((dd <= 1) | small).all() and (dd == 0).mean() > 0.995, (what, int(dd.max()), float((dd == 0).mean()))
    else:
        scale = np.abs(ref).max(axis=-1, keepdims=True)
        assert (np.abs(got - ref) <= tol * (np.abs(ref) + scale) + 1e-30).all(), what


SHAPES = [(1, 8), (5, 33), (64, 300), (300, 4096), (9, 5000), (2, 60000)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_layer_rms_and_fused_add(capi, oracle, shape, dt):
    rng = np.random.default_rng(shape[0] + shape[1])
    x32 = (rng.normal(size=shape) * 2 + 0.3).astype(np.float32)
    r32 = rng.normal(size=shape).astype(np.float32)
    cv = (lambda a: oracle.f32_to_bf16(a)) if dt == "bf16" else (lambda a: a)
    x, res = cv(x32), cv(r32)
    gamma = rng.normal(size=shape[1]).astype(np.float32)
    beta = oracle.f32_to_bf16(rng.normal(size=shape[1]).astype(np.float32))       # beta in bf16 storage
    for kind, g, b in (("layer_norm", gamma, beta), ("layer_norm", None, None), ("rms_norm", gamma, None), ("rms_norm", None, None)):
        st, out, _, _, _ = run(capi, kind, x, g, b)
        assert st == capi.SUCCESS, capi.last_error()
        close(oracle, out, oracle.normalization(kind, x, g, b), (kind, shape, dt))
    st, out, res_out, _, _ = run(capi, "fused_add_rms_norm", x, gamma, residual=res)
    assert st == capi.SUCCESS, capi.last_error()
    ref, ref_res = oracle.normalization("fused_add_rms_norm", x, gamma, residual=res)
    assert (res_out == ref_res).all()                       # one addition and one rounding: bit for bit
    close(oracle, out, ref, ("fused", shape, dt))
    # f32 source into a bf16 destination
    if dt == "f32":
        st, out, _, _, _ = run(capi, "rms_norm", x, gamma, dst_dt="bf16")
        assert st == capi.SUCCESS, capi.last_error()
        close(oracle, out, oracle.normalization("rms_norm", x, gamma, dst_dt="bf16"), ("rms f32->bf16", shape))


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_reference_kernel_outputs_and_batch_norm(capi, oracle, golden2, dt):
    rng = np.random.default_rng(81)             # the inputs of tests/golden/make_golden_ref2.py::norm_inputs
    x = (rng.normal(size=(7, 300)) * 3 + 0.5).astype(np.float32)
    x[2] *= 100.0
    x[4] = 0.0
    gamma = rng.normal(size=300).astype(np.float32)
    beta = rng.normal(size=300).astype(np.float32)
    res = rng.normal(size=(7, 300)).astype(np.float32)
    xb = rng.normal(size=(3, 5, 11)).astype(np.float32)
    rm = rng.normal(size=5).astype(np.float32)
    rv = rng.uniform(0.5, 2.0, 5).astype(np.float32)
    cv = (lambda a: oracle.f32_to_bf16(a)) if dt == "bf16" else (lambda a: a)
    for key, kind, g, b in (("norm_layer_", "layer_norm", gamma, beta), ("norm_layer_noaffine_", "layer_norm", None, None),
                            ("norm_rms_", "rms_norm", gamma, None)):
        st, out, _, _, _ = run(capi, kind, cv(x), g, b)
        assert st == capi.SUCCESS, capi.last_error()
        close(oracle, out, golden2[key + dt], key)
    st, out, res_out, _, _ = run(capi, "fused_add_rms_norm", cv(x), gamma, residual=cv(res))
    assert st == capi.SUCCESS and (res_out == golden2["norm_fused_res_" + dt]).all()
    close(oracle, out, golden2["norm_fused_" + dt], "fused")
    st, out, _, _, _ = run(capi, "batch_norm", cv(xb), gamma[:5], beta[:5], rm=rm, rv=rv)
    assert st == capi.SUCCESS, capi.last_error()
    assert (out == golden2["norm_batch_" + dt]).all()        # element-wise: bit for bit


@pytest.mark.parametrize("kind", ["rms_norm", "fused_add_rms_norm", "layer_norm"])
def test_fused_per_token_quantisation(capi, oracle, kind):
    """norm -> bf16 -> per-token s8 in one pass: codes and scales equal the oracle's per-token quantisation of the bf16 output
    that the same call wrote; without an output buffer the codes are the same."""
    rng = np.random.default_rng(17)
    for shape in [(40, 256), (300, 4096), (7, 1000)]:
        x = oracle.f32_to_bf16((rng.normal(size=shape) * 2).astype(np.float32))
        gamma = oracle.f32_to_bf16(rng.normal(size=shape[1]).astype(np.float32))
        res = oracle.f32_to_bf16(rng.normal(size=shape).astype(np.float32)) if kind == "fused_add_rms_norm" else None
        beta = rng.normal(size=shape[1]).astype(np.float32) if kind == "layer_norm" else None
        st, out, _, q, s = run(capi, kind, x, gamma, beta, residual=res, quant=True)
        assert st == capi.SUCCESS, capi.last_error()
        qr, sr = oracle.quant_per_token(out)
        assert (q == qr).all() and (s == sr).all(), (kind, shape)
        st, _, _, q2, s2 = run(capi, kind, x, gamma, beta, residual=res, quant=True, want_output=False)
        assert st == capi.SUCCESS and (q2 == q).all() and (s2 == s).all()


def test_device_buffers(capi, oracle):
    torch = pytest.importorskip("torch")
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(3)
    x = oracle.f32_to_bf16(rng.normal(size=(512, 2048)).astype(np.float32))
    g = rng.normal(size=2048).astype(np.float32)
    xd = torch.from_numpy(x.view(np.int16)).to(dev); gd = torch.from_numpy(g).to(dev)
    od = torch.zeros_like(xd)
    d = capi.NormDesc()
    d.norm_type, d.batch, d.norm_size, d.epsilon, d.use_scale = capi.NORM["rms_norm"], 512, 2048, 1e-6, 1
    d.src_dt = d.dst_dt = capi.DT["bf16"]; d.gamma_dt = capi.DT["f32"]; d.beta_dt = capi.DT["f32"]
    d.input, d.output, d.gamma = xd.data_ptr(), od.data_ptr(), gd.data_ptr()
    assert capi.lib.b200dnn_normalization(C.byref(d), torch.cuda.current_stream().cuda_stream) == capi.SUCCESS, capi.last_error()
    torch.cuda.synchronize()
    close(oracle, od.cpu().numpy().view(np.uint16), oracle.normalization("rms_norm", x, g, eps=1e-6), "device buffers")


def test_contract(capi):
    x = np.zeros((4, 16), dtype=np.float32)
    assert run(capi, "rms_norm", x, eps=0.0)[0] == capi.FAILURE and "epsilon" in capi.last_error()
    assert run(capi, "fused_add_rms_norm", x)[0] == capi.FAILURE and "residual" in capi.last_error()
    assert run(capi, "batch_norm", np.zeros((2, 3, 4), dtype=np.float32))[0] == capi.FAILURE and "running_mean" in capi.last_error()
    d = capi.NormDesc()
    d.norm_type, d.batch, d.norm_size, d.epsilon = capi.NORM["rms_norm"], 4, 16, 1e-5
    d.src_dt, d.dst_dt = 2, 2                                  # f16
    out = np.zeros((4, 16), dtype=np.uint16)
    d.input, d.output = x.ctypes.data, out.ctypes.data
    assert capi.lib.b200dnn_normalization(C.byref(d), None) == capi.UNIMPLEMENTED
    d.src_dt, d.dst_dt = capi.DT["bf16"], 2
    assert capi.lib.b200dnn_normalization(C.byref(d), None) == capi.FAILURE and "cross-mixing" in capi.last_error()
    d.src_dt = d.dst_dt = capi.DT["f32"]; d.use_scale = 1
    assert capi.lib.b200dnn_normalization(C.byref(d), None) == capi.FAILURE and "gamma" in capi.last_error()
    d.use_scale = 0; d.norm_type = -1
    assert capi.lib.b200dnn_normalization(C.byref(d), None) == capi.FAILURE
