"""Shared helpers for the GPU parity tests: seeded inputs shaped like the benchmark configs and
comparison rules.  bf16 tensors are numpy uint16 bit patterns on the host."""
import numpy as np


def bf16_ulp_diff(a_bits, b_bits):
    """Distance in bf16 units of last place between two bit-pattern arrays (sign-magnitude aware)."""
    def key(x):
        x = x.astype(np.int32)
        return np.where(x & 0x8000, -(x & 0x7FFF), x & 0x7FFF)
    return np.abs(key(a_bits) - key(b_bits))


def assert_bf16_close(got, ref, max_ulp=1, what="", row_atol_frac=0.0, atol=0.0):
    """Within max_ulp bf16 ulp, or within rel 8e-3 of the reference value (the stated tolerance).
    row_atol_frac > 0 additionally accepts |diff| <= frac * max|ref row|: used where an output is
    a sum of terms that cancel (the MoE weighted reduce), so that a one-ulp change of one term is
    not measured against a near-zero result.  atol accepts small absolute differences where the
    formula itself cancels (1 + erf(x) or 1 + tanh(x) for very negative x: both sides are correct to
    f32 precision of the transcendental, the tiny product is not)."""
    d = bf16_ulp_diff(got, ref)
    bad = d > max_ulp
    if bad.any():
        g = (got.astype(np.uint32) << 16).view(np.float32)
        r = (ref.astype(np.uint32) << 16).view(np.float32)
        tol = 8e-3 * np.abs(r) + 1e-30 + atol
        if row_atol_frac > 0:
            tol = np.maximum(tol, row_atol_frac * np.abs(r).max(axis=-1, keepdims=True))
        bad &= ~(np.abs(g - r) <= tol)
    assert not bad.any(), "%s: %d of %d elements differ by more than %d bf16 ulp (max %d)" % (
        what, int(bad.sum()), bad.size, max_ulp, int(d.max()))


def config1(oracle, M=128, K=4096, N=4096, seed=0):
    rng = np.random.default_rng(seed)
    A = rng.integers(0, 256, (M, K), dtype=np.uint8)
    W = rng.integers(-127, 128, (K, N), dtype=np.int8)
    ws = rng.uniform(0.001, 0.01, N).astype(np.float32)
    bias = rng.normal(size=N).astype(np.float32)
    return dict(A=A, W=W, ws=ws, bias=bias, zp=np.array([128], dtype=np.int32), ss=np.array([0.02], dtype=np.float32))


def decode_case(oracle, M, K, N, seed=0):
    """bf16 activations N(0,1) quantised per token, bf16 weights N(0,0.02) quantised per channel."""
    rng = np.random.default_rng(seed)
    x = oracle.f32_to_bf16(rng.normal(size=(M, K)).astype(np.float32))
    w = oracle.f32_to_bf16((rng.normal(size=(K, N)) * 0.02).astype(np.float32))
    qa, sa = oracle.quant_per_token(x)
    qw, sw = oracle.quant_weights_per_channel(w)
    return dict(x=x, w=w, A=qa, sa=sa, W=qw, sw=sw)
