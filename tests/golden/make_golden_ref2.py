"""Generates tests/golden/ref2_cases.npz from more of the REFERENCE's own code: the dynamic per-token
quantisation kernels, the gated activations (AVX-512 and scalar paths), the MoE weighted reduce, the per-channel /
per-tensor dynamic scales and the static quantise / dequantise.

Run in a container that has the reference checkout (its location: the ZENDNN_REFERENCE_ROOT variable) and AVX-512:
    python tests/golden/make_golden_ref2.py
It builds oracle/_ref/libzendnn_ref2.so from the reference sources (oracle/Makefile, oracle/ref_driver2.cpp),
runs the reference functions on seeded inputs and stores inputs and outputs.  The scalar paths are produced by
a child process started with ORACLE_REF_SCALAR=1.  The fixtures travel with the repository; the reference
does not.
"""
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

ACTS = ["silu_and_mul", "gelu_and_mul", "swiglu_oai_mul"]


def inputs():
    rng = np.random.default_rng(77)
    x32 = (rng.normal(size=(12, 520)) * rng.uniform(0.01, 30, size=(12, 1))).astype(np.float32)
    x32[0, :3] = [np.inf, -np.inf, np.nan]
    x32[2, :] = 0
    y32 = (rng.normal(size=(16, 256)) * 3).astype(np.float32)
    rows32 = rng.normal(size=(16 * 3, 136)).astype(np.float32)
    w = rng.uniform(0, 1, size=(16, 3)).astype(np.float32)
    return x32, y32, rows32, w


def weight_input():
    rng = np.random.default_rng(78)
    w32 = (rng.normal(size=(70, 45)) * 0.05).astype(np.float32)
    w32[3, 4] = np.inf
    w32[:, 7] = 0
    return w32


def ukernel_inputs():
    """Inputs of the group DQ-INT8 micro-kernel cases: s8 activations with per-token scales, s8 weights with per-channel
    scales, an f32 bias.  M is not a multiple of the kernel's row block, K and N are the smallest legal multiples."""
    rng = np.random.default_rng(79)
    M, K, N = 21, 256, 128
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    B = rng.integers(-127, 128, (K, N), dtype=np.int8)
    sa = rng.uniform(0.01, 0.05, M).astype(np.float32)
    sw = rng.uniform(1e-4, 5e-4, N).astype(np.float32)
    bias = rng.normal(size=N).astype(np.float32)
    return A, B, sa, sw, bias


def ukernel_bf16_inputs():
    """Inputs of the group bf16 micro-kernel cases: bf16 activations and weights (bit patterns), an f32 bias."""
    rng = np.random.default_rng(80)
    M, K, N = 21, 256, 128
    A = O.f32_to_bf16(rng.normal(size=(M, K)).astype(np.float32))
    B = O.f32_to_bf16((rng.normal(size=(K, N)) * 0.06).astype(np.float32))
    bias = rng.normal(size=N).astype(np.float32)
    return A, B, bias


def norm_inputs():
    """Inputs of the normalization cases: a [7, 300] matrix with an offset and a wide row, gamma / beta, a residual, and a
    [3, 5, 11] tensor with running statistics for BatchNorm."""
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


PG_GROUPS = [2, 4, 8, 16]
UK_ACTS = ["none", "silu_and_mul", "gelu_and_mul", "swiglu_oai_mul"]


def run(tag):
    x32, y32, rows32, w = inputs()
    out = {}
    for dt in ("bf16", "f32"):
        x = O.f32_to_bf16(x32) if dt == "bf16" else x32
        y = O.f32_to_bf16(y32) if dt == "bf16" else y32
        rows = O.f32_to_bf16(rows32) if dt == "bf16" else rows32
        native = tag == "vec"
        q, s = O.ref2_quant_per_token(x, native=native)
        out["quant_%s_%s_q" % (dt, tag)], out["quant_%s_%s_s" % (dt, tag)] = q, s
        r = O.ref2_quant_per_token_asym(x, native=native)
        assert r is not None
        out["quantu8_%s_%s_q" % (dt, tag)], out["quantu8_%s_%s_s" % (dt, tag)], out["quantu8_%s_%s_z" % (dt, tag)] = r
        for a in ACTS:
            out["act_%s_%s_%s" % (a, dt, tag)] = O.ref2_gated_act(y, a)
        for skip in (0, 1):
            out["reduce_%s_skip%d_%s" % (dt, skip, tag)] = O.ref2_moe_reduce(rows, w, 3, bool(skip), threads=2)
    if tag == "vec":     # these reference functions have a single (scalar) implementation
        w32 = weight_input()
        for dt in ("bf16", "f32"):
            wv = O.f32_to_bf16(w32) if dt == "bf16" else w32
            sc = O.ref2_dyn_scales(wv, True)
            out["dyn_pc_" + dt], out["dyn_pt_" + dt] = sc, O.ref2_dyn_scales(wv, False)
            q = O.ref2_granular(wv, "s8", sc.reshape(1, -1))
            out["qs8_" + dt] = q
            out["qu8_" + dt] = O.ref2_granular(wv, "u8", np.array([[0.002]], dtype=np.float32), np.array([13], dtype=np.int32))
            out["deq_" + dt] = O.ref2_granular(q, dt, sc.reshape(1, -1))
        out["w32"] = w32
        # per-group dynamic quantisation along K (the reference has the AVX-512 kernel only); x32 has K = 96 ... use G that divides it
        for dt in ("bf16", "f32"):
            x = O.f32_to_bf16(x32) if dt == "bf16" else x32
            for G in PG_GROUPS:
                if x.shape[1] % G:
                    continue
                r = O.ref2_quant_per_group(x, G)
                assert r is not None, "the reference per-group kernel needs AVX-512"
                out["pg_%s_G%d_q" % (dt, G)], out["pg_%s_G%d_s" % (dt, G)] = r
        A, B, sa, sw, bias = ukernel_inputs()
        for a in UK_ACTS:
            for hb in (0, 1):
                r = O.ref2_int8_ukernel(A, B, sa, sw, bias if hb else None, a)
                assert r is not None, "the reference micro-kernel needs AVX-512 VNNI"
                out["uk_%s_bias%d" % (a, hb)] = r
        x, gamma, beta, res, xb, rm, rv = norm_inputs()
        for dt in ("f32", "bf16"):
            cv = (lambda a: O.f32_to_bf16(a)) if dt == "bf16" else (lambda a: a)
            out["norm_layer_%s" % dt] = O.ref2_normalization("layer_norm", cv(x), gamma, beta)
            out["norm_layer_noaffine_%s" % dt] = O.ref2_normalization("layer_norm", cv(x))
            out["norm_rms_%s" % dt] = O.ref2_normalization("rms_norm", cv(x), gamma)
            o, r = O.ref2_normalization("fused_add_rms_norm", cv(x), gamma, residual=cv(res))
            out["norm_fused_%s" % dt], out["norm_fused_res_%s" % dt] = o, r
            out["norm_batch_%s" % dt] = O.ref2_normalization("batch_norm", cv(xb), gamma[:5], beta[:5], running_mean=rm, running_var=rv)
        A, B, bias = ukernel_bf16_inputs()
        for a in UK_ACTS:
            for hb in (0, 1):
                r = O.ref2_bf16_ukernel(A, B, bias if hb else None, a)
                assert r is not None, "the reference bf16 micro-kernel needs AVX512-BF16"
                out["ukbf_%s_bias%d" % (a, hb)] = r
    return out


def main():
    O.build()
    assert O.ref2_lib() is not None, "libzendnn_ref2.so unavailable (needs a reference checkout)"
    here = os.path.dirname(os.path.abspath(__file__))
    if len(sys.argv) > 1 and sys.argv[1] == "--scalar-child":
        np.savez_compressed(sys.argv[2], **run("scalar"))
        return
    out = run("vec")
    tmp = os.path.join(here, "_scalar_tmp.npz")
    subprocess.check_call([sys.executable, os.path.abspath(__file__), "--scalar-child", tmp],
                          env=dict(os.environ, ORACLE_REF_SCALAR="1"))
    out.update(dict(np.load(tmp)))
    os.remove(tmp)
    x32, y32, rows32, w = inputs()
    out.update(x32=x32, y32=y32, rows32=rows32, w=w)
    path = os.path.join(here, "ref2_cases.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
