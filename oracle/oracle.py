"""numpy front end of the CPU oracle (oracle/w8a8_oracle.c) and of the compiled reference
tile kernel (oracle/_ref/libzendnn_ref.so).

TEST INFRASTRUCTURE ONLY.  Imported by tests/, by __graft_entry__.smoke() and by the CPU
baseline legs of bench.py; the product package never imports it.

bf16 tensors are carried as numpy uint16 arrays holding the bit patterns.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

# dtype / post-op codes of the reference (common/data_types.hpp:44-58,
# operators/common/post_op.hpp:36-57)
DT = dict(none=0, f32=1, f16=2, bf16=3, s32=4, s64=5, s16=6, s8=7, s4=8, u32=9, u16=10, u8=11, u4=12)
PO = dict(none=0, elu=1, relu=2, leaky_relu=3, gelu_tanh=4, gelu_erf=5, sigmoid=6, swish=7, tanh=8,
          softmax=9, pooling=10, square=11, abs=12, sqrt=13, exp=14, log=15, clip=16, binary_add=17,
          binary_mul=18, mish=19)
ACT = dict(none=0, silu_and_mul=1, gelu_and_mul=2, swiglu_oai_mul=3)


def build(force=False):
    """Compile liboracle.so (always possible) and, if a reference checkout exists, _ref."""
    lib = os.path.join(_HERE, "liboracle.so")
    if force or not os.path.exists(lib) or os.path.getmtime(lib) < os.path.getmtime(
            os.path.join(_HERE, "w8a8_oracle.c")):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    ref_root = os.environ.get("ZENDNN_REFERENCE_ROOT", "/root/reference")
    ref = os.path.join(_HERE, "_ref", "libzendnn_ref.so")
    ref2 = os.path.join(_HERE, "_ref", "libzendnn_ref2.so")
    if os.path.isdir(ref_root) and (force or not os.path.exists(ref) or not os.path.exists(ref2)):
        subprocess.check_call(["make", "-C", _HERE, "-s", "ref", "REF=" + ref_root])


class _PostOp(C.Structure):
    _fields_ = [("type", C.c_int32), ("dt", C.c_int32), ("buff", C.c_void_p), ("ld", C.c_int64),
                ("alpha", C.c_float), ("beta", C.c_float)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        _lib = C.CDLL(path)
        _lib.orc_gemm_s32.restype = C.c_int
        _lib.orc_epilogue.restype = C.c_int
        _lib.orc_group_scaled_gemm.restype = C.c_int
    return _lib


_ref = None


def ref_lib():
    """The compiled reference tile kernel, or None when absent / the host lacks AVX-512 VNNI+BF16."""
    global _ref
    if _ref is None:
        path = os.path.join(_HERE, "_ref", "libzendnn_ref.so")
        if not os.path.exists(path):
            _ref = False
        else:
            try:
                l = C.CDLL(path)
                _ref = l if l.ref_available() else False
            except OSError:
                _ref = False
    return _ref or None


_ref2 = None


def ref2_lib():
    """The reference's per-token quantisation kernels, gated activations and MoE weighted reduce compiled from the
    reference tree (oracle/ref_driver2.cpp), or None when absent.  The environment variable ORACLE_REF_SCALAR=1,
    set before the first call, makes the reference take its scalar code paths."""
    global _ref2
    if _ref2 is None:
        path = os.path.join(_HERE, "_ref", "libzendnn_ref2.so")
        try:
            _ref2 = C.CDLL(path) if os.path.exists(path) else False
        except OSError:
            _ref2 = False
    return _ref2 or None


def ref2_quant_per_token(x, native=False):
    """Reference dynamic per-token quantisation (scalar kernel, or the AVX-512 one).  None if unavailable."""
    r = ref2_lib()
    x = np.ascontiguousarray(x)
    M, K = x.shape
    q = np.zeros((M, K), dtype=np.int8)
    s = np.zeros(M, dtype=np.float32)
    if r is None or (native and not r.ref2_avx512()):
        return None
    rc = r.ref2_quant_per_token(_p(x), int(x.dtype == np.uint16), _p(q), _p(s), C.c_int64(M), C.c_int64(K), int(native))
    return (q, s) if rc == 0 else None


def ref2_quant_per_group(x, G):
    """Reference per-group dynamic quantisation (AVX-512 kernel), scale layout {M,G}.  None if unavailable."""
    r = ref2_lib()
    x = np.ascontiguousarray(x)
    M, K = x.shape
    if r is None or not r.ref2_avx512() or not hasattr(r, "ref2_quant_per_group"):
        return None
    q = np.zeros((M, K), dtype=np.int8)
    s = np.zeros((M, G), dtype=np.float32)
    rc = r.ref2_quant_per_group(_p(x), int(x.dtype == np.uint16), _p(q), _p(s), C.c_int64(M), C.c_int64(K), C.c_int64(G))
    return (q, s) if rc == 0 else None


def ref2_gated_act(y, act):
    """Reference gated activation (in place in the reference; here on a copy).  y [M, 2I] f32 or bf16 bits."""
    r = ref2_lib()
    if r is None:
        return None
    buf = np.ascontiguousarray(y).copy()
    M, N = buf.shape
    r.ref2_gated_act(ACT[act], _p(buf), M, N, N, DT["bf16"] if buf.dtype == np.uint16 else DT["f32"])
    return np.ascontiguousarray(buf[:, : N // 2])


def ref2_moe_reduce(rows, weights, topk, skip_weighted=False, threads=1):
    """Reference MoE weighted reduce over rows [T*topk, D] (f32 or bf16 bits), weights [T, topk]."""
    r = ref2_lib()
    if r is None:
        return None
    rows = np.ascontiguousarray(rows)
    T, D = rows.shape[0] // topk, rows.shape[1]
    w = np.ascontiguousarray(weights, dtype=np.float32)
    ptrs = (C.c_void_p * (T * topk))(*[rows.ctypes.data + i * rows.strides[0] for i in range(T * topk)])
    out = np.zeros((T, D), dtype=rows.dtype)
    rc = r.ref2_moe_reduce(ptrs, _p(w), int(skip_weighted), T, topk, D, DT["bf16"] if rows.dtype == np.uint16 else DT["f32"],
                           _p(out), D, threads)
    return out if rc == 1 else None


def ref2_dyn_scales(x, per_channel=True):
    """Reference dynamic scales (compute_dynamic_quant_params) of a [M,N] matrix, symmetric s8 target."""
    r = ref2_lib()
    if r is None:
        return None
    x = np.ascontiguousarray(x)
    M, N = x.shape
    s = np.zeros(N if per_channel else 1, dtype=np.float32)
    rc = r.ref2_dyn_scales(_p(x), DT["bf16"] if x.dtype == np.uint16 else DT["f32"], C.c_int64(M), C.c_int64(N),
                           int(per_channel), _p(s))
    return s if rc == 1 else None


def ref2_granular(src, dst_dt, scale, zp=None):
    """Reference static quantise / dequantise (scalar granular implementation).  scale [sr,sc] f32, zp [zr,zc] s32."""
    r = ref2_lib()
    if r is None:
        return None
    src = np.ascontiguousarray(src)
    M, N = src.shape
    names = {np.dtype(np.uint16): "bf16", np.dtype(np.float32): "f32", np.dtype(np.int8): "s8", np.dtype(np.uint8): "u8"}
    dst = np.zeros((M, N), dtype={"s8": np.int8, "u8": np.uint8, "f32": np.float32, "bf16": np.uint16}[dst_dt])
    sc = np.ascontiguousarray(np.asarray(scale, dtype=np.float32).reshape(np.asarray(scale).shape if np.asarray(scale).ndim == 2 else (1, -1)))
    z = None if zp is None else np.ascontiguousarray(np.asarray(zp, dtype=np.int32).reshape(1, -1))
    r.ref2_granular(_p(src), DT[names[src.dtype]], _p(dst), DT[dst_dt], C.c_int64(M), C.c_int64(N), _p(sc),
                    C.c_int64(sc.shape[0]), C.c_int64(sc.shape[1]), _p(z), C.c_int64(1 if z is not None else 0),
                    C.c_int64(z.shape[1] if z is not None else 0))
    return dst


def ref2_int8_ukernel(A, B, src_scale, wei_scale, bias=None, act="none"):
    """The reference's group DQ-INT8 micro-kernel (custom_kernel/ukernel/int8_microkernel.cpp) over A s8 [M,K] x
    B s8 [K,N]: exact s32 compensation, x src scale, x weight scale, + bias, optional gated activation, bf16 out
    ([M,N], or [M,N/2] for the gated forms).  None if unavailable."""
    r = ref2_lib()
    if r is None or not hasattr(r, "ref2_int8_ukernel"):
        return None
    A = np.ascontiguousarray(A, dtype=np.int8); B = np.ascontiguousarray(B, dtype=np.int8)
    M, K = A.shape
    N = B.shape[1]
    kind = {"none": 0, "swiglu_oai_mul": 1, "silu_and_mul": 2, "gelu_and_mul": 3}[act]
    sa = np.ascontiguousarray(src_scale, dtype=np.float32); sw = np.ascontiguousarray(wei_scale, dtype=np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    out = np.zeros((M, N if kind == 0 else N // 2), dtype=np.uint16)
    rc = r.ref2_int8_ukernel(_p(A), _p(B), M, N, K, _p(sa), _p(sw), _p(b), kind, _p(out))
    return out if rc == 0 else None


def ref2_bf16_ukernel(A, B, bias=None, act="none"):
    """The reference's group bf16 micro-kernel (custom_kernel/ukernel/bf16_microkernel.cpp) over A bf16 [M,K] x B bf16 [K,N]
    (bit patterns): f32 accumulation, + bias, optional gated activation, bf16 out ([M,N], or [M,N/2] gated).
    None if unavailable (library not built, or no AVX512-BF16 on this host)."""
    r = ref2_lib()
    if r is None or not hasattr(r, "ref2_bf16_ukernel"):
        return None
    A = np.ascontiguousarray(A, dtype=np.uint16); B = np.ascontiguousarray(B, dtype=np.uint16)
    M, K = A.shape
    N = B.shape[1]
    kind = {"none": 0, "swiglu_oai_mul": 1, "silu_and_mul": 2, "gelu_and_mul": 3}[act]
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    out = np.zeros((M, N if kind == 0 else N // 2), dtype=np.uint16)
    rc = r.ref2_bf16_ukernel(_p(A), _p(B), M, N, K, _p(b), kind, _p(out))
    return out if rc == 0 else None


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def f32_to_bf16(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f32_to_bf16(_p(x), _p(out), C.c_int64(x.size))
    return out


def bf16_to_f32(x):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    return (x.astype(np.uint32) << 16).view(np.float32)


def _dt_of(a):
    return {np.dtype(np.float32): DT["f32"], np.dtype(np.uint16): DT["bf16"], np.dtype(np.int32): DT["s32"],
            np.dtype(np.int8): DT["s8"], np.dtype(np.uint8): DT["u8"]}[a.dtype]


def gemm_s32(A, B, transB=False):
    """Exact int32 accumulators.  A [M,K] u8|s8; B [K,N] s8, or [N,K] when transB."""
    A = np.ascontiguousarray(A)
    B = np.ascontiguousarray(B)
    M, K = A.shape
    N = B.shape[0] if transB else B.shape[1]
    out = np.empty((M, N), dtype=np.int32)
    rc = lib().orc_gemm_s32(_p(A), int(A.dtype == np.uint8), C.c_int64(K), _p(B), C.c_int64(B.shape[1]),
                            int(transB), M, N, K, _p(out), C.c_int64(N))
    assert rc == 0
    return out


class PackedB:
    """Weight packed once for repeated oracle GEMMs (CPU-baseline timing)."""

    def __init__(self, B, transB=False):
        B = np.ascontiguousarray(B)
        self.K, self.N = (B.shape[1], B.shape[0]) if transB else B.shape
        lib().orc_pack_b.restype = C.c_void_p
        self.h = C.c_void_p(lib().orc_pack_b(_p(B), C.c_int64(B.shape[1]), int(transB), self.K, self.N))

    def gemm_s32(self, A, out=None):
        A = np.ascontiguousarray(A)
        M = A.shape[0]
        if out is None:
            out = np.empty((M, self.N), dtype=np.int32)
        rc = lib().orc_gemm_s32_packed(_p(A), int(A.dtype == np.uint8), C.c_int64(A.shape[1]), self.h, M, _p(out),
                                       C.c_int64(self.N))
        assert rc == 0
        return out

    def __del__(self):
        try:
            lib().orc_free_b(self.h)
        except Exception:
            pass


def colsum(B, transB=False):
    B = np.ascontiguousarray(B)
    K, N = (B.shape[1], B.shape[0]) if transB else B.shape
    out = np.empty(N, dtype=np.int32)
    lib().orc_colsum(_p(B), C.c_int64(B.shape[1]), int(transB), K, N, _p(out))
    return out


def _postops(postops, keep):
    arr = (_PostOp * max(1, len(postops)))()
    for i, po in enumerate(postops):
        if isinstance(po, str):
            po = dict(type=po)
        arr[i].type = PO[po["type"]]
        arr[i].alpha = po.get("alpha", 0.0)
        arr[i].beta = po.get("beta", 0.0)
        b = po.get("buff")
        if b is not None:
            b = np.ascontiguousarray(b)
            keep.append(b)
            arr[i].buff = b.ctypes.data
            arr[i].dt = _dt_of(b)
            arr[i].ld = 0 if (b.ndim == 1 or b.shape[0] == 1) else b.shape[1]
    return arr


def epilogue(acc, dst_dt="bf16", src_scale=None, wei_scale=None, src_zp=0, col_sum=None, bias=None,
             postops=(), order=0):
    """Dequantising epilogue over s32 accumulators; returns f32 / bf16-bits(uint16) / s32 array."""
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    M, N = acc.shape
    keep = []
    ss = None if src_scale is None else np.ascontiguousarray(np.asarray(src_scale, dtype=np.float32).reshape(-1))
    ws = None if wei_scale is None else np.ascontiguousarray(np.asarray(wei_scale, dtype=np.float32).reshape(-1))
    cs = None if col_sum is None else np.ascontiguousarray(col_sum, dtype=np.int32)
    b = None if bias is None else np.ascontiguousarray(bias)
    po = _postops(list(postops), keep)
    out = np.empty((M, N), dtype={"bf16": np.uint16, "f32": np.float32, "s32": np.int32}[dst_dt])
    rc = lib().orc_epilogue(_p(acc), C.c_int64(N), M, N, order, _p(ss), 0 if ss is None else ss.size,
                            _p(ws), 0 if ws is None else ws.size, C.c_int32(int(src_zp)), _p(cs),
                            _p(b), 0 if b is None else _dt_of(b), po, len(postops),
                            _p(out), DT[dst_dt], C.c_int64(N))
    assert rc == 0
    return out


def matmul_w8a8(A, B, dst_dt="bf16", transB=False, src_scale=None, wei_scale=None, src_zp=0, bias=None,
                postops=(), order=0):
    """matmul_direct INT8 semantics: exact GEMM then epilogue."""
    acc = gemm_s32(A, B, transB)
    cs = colsum(B, transB) if src_zp != 0 else None
    return epilogue(acc, dst_dt, src_scale, wei_scale, src_zp, cs, bias, postops, order)


def matmul_bf16(A, B, dst_dt="bf16", transB=False, bias=None, postops=()):
    """bf16 x bf16 matmul_direct: A [M,K] and B [K,N] ([N,K] with transB) as bf16 bit patterns (uint16); exact
    products summed in double, one rounding to f32, bias, post-ops, RNE to dst."""
    A = np.ascontiguousarray(A, dtype=np.uint16)
    B = np.ascontiguousarray(B, dtype=np.uint16)
    M, K = A.shape
    N = B.shape[0] if transB else B.shape[1]
    keep = []
    b = None if bias is None else np.ascontiguousarray(bias)
    po = _postops(list(postops), keep)
    out = np.empty((M, N), dtype={"bf16": np.uint16, "f32": np.float32}[dst_dt])
    rc = lib().orc_matmul_bf16(_p(A), C.c_int64(K), _p(B), C.c_int64(B.shape[1]), int(bool(transB)), M, N, K,
                               _p(b), 0 if b is None else _dt_of(b), po, len(postops), _p(out), DT[dst_dt], C.c_int64(N))
    assert rc == 0
    return out


def requant_dst(x, dst_dt, dst_scale=None, dst_zp=None):
    """Requantised matmul destination over the f32 epilogue result: x * dst_scale + dst_zp in f32
    (operators/matmul/matmul_ref_kernel.cpp:770-797), clamp to the range of the type and nearbyint (:155-192)."""
    x = np.asarray(x, dtype=np.float32)
    if dst_scale is not None:
        x = x * np.float32(np.asarray(dst_scale, dtype=np.float32).reshape(-1)[0])
    if dst_zp is not None:
        x = x + np.float32(int(np.asarray(dst_zp).reshape(-1)[0]))
    lo, hi, t = (0.0, 255.0, np.uint8) if dst_dt == "u8" else (-128.0, 127.0, np.int8)
    x = np.where(x < lo, np.float32(lo), np.where(x > hi, np.float32(hi), x))
    return np.rint(np.nan_to_num(x, nan=0.0)).astype(t)


def matmul_group_scaled(A, B, src_scale, wei_scale, dst_dt="bf16", bias=None, postops=()):
    """Per-group symmetric INT8 matmul_direct (and W4A8 after the s4 -> s8 widening), the reference's scalar formula
    (operators/matmul/matmul_ref_kernel.cpp:961-1003): A s8 [M,K], B s8 [K,N], src_scale f32 [M,G] or [M] / [M,1]
    (per-token, broadcast over the groups), wei_scale f32 [G,N]."""
    A = np.ascontiguousarray(A, dtype=np.int8)
    B = np.ascontiguousarray(B, dtype=np.int8)
    M, K = A.shape
    N = B.shape[1]
    ws = np.ascontiguousarray(np.asarray(wei_scale, dtype=np.float32).reshape(-1, N))
    G = ws.shape[0]
    ss = np.ascontiguousarray(np.asarray(src_scale, dtype=np.float32).reshape(M, -1))
    keep = []
    b = None if bias is None else np.ascontiguousarray(bias)
    po = _postops(list(postops), keep)
    out = np.empty((M, N), dtype={"bf16": np.uint16, "f32": np.float32}[dst_dt])
    rc = lib().orc_group_scaled_gemm(_p(A), C.c_int64(K), _p(B), C.c_int64(N), M, N, K, G, _p(ss), ss.shape[1], _p(ws),
                                     _p(b), 0 if b is None else _dt_of(b), po, len(postops), _p(out), DT[dst_dt], C.c_int64(N))
    assert rc == 0, "bad group count"
    return out


def pack_s4(W, transB=False, ldb=None):
    """Signed 4-bit weights as the reference stores them (matmul/backends/aocl/aocl_kernel.cpp:145-160): element (k,n)
    lives at physical index k*ldb+n (transB: n*ldb+k), two per byte, even index in the low nibble.  W int8 [K,N] with
    values in [-8,7] -> uint8 bytes."""
    W = np.asarray(W, dtype=np.int8)
    assert W.min() >= -8 and W.max() <= 7
    K, N = W.shape
    P = W.T if transB else W                       # physical rows
    rows, cols = P.shape
    ldb = cols if ldb is None else ldb
    flat = np.zeros(rows * ldb + (rows * ldb) % 2, dtype=np.uint8)
    idx = (np.arange(rows)[:, None] * ldb + np.arange(cols)[None, :]).reshape(-1)
    flat[idx] = P.reshape(-1).astype(np.uint8) & 0xF
    return (flat[0::2] | (flat[1::2] << 4)).astype(np.uint8)


def unpack_s4(packed, K, N, transB=False, ldb=None):
    """Inverse of pack_s4: sign-extended nibble codes, int8 [K,N] (the reference's cvt_s4_to_s8)."""
    rows, cols = (N, K) if transB else (K, N)
    ldb = cols if ldb is None else ldb
    b = np.asarray(packed, dtype=np.uint8)
    flat = np.empty(b.size * 2, dtype=np.uint8)
    flat[0::2] = b & 0xF
    flat[1::2] = b >> 4
    idx = np.arange(rows)[:, None] * ldb + np.arange(cols)[None, :]
    v = flat[idx].astype(np.int8)
    v = np.where(v & 8, v | np.int8(-16), v).astype(np.int8)
    return np.ascontiguousarray(v.T) if transB else v


def pack_u4(W, transB=False, ldb=None):
    """Unsigned 4-bit weights, same placement as pack_s4; W uint8 [K,N] with values in [0,15]."""
    W = np.asarray(W, dtype=np.uint8)
    assert W.max() <= 15
    return pack_s4((W.astype(np.int16) - 16 * (W > 7)).astype(np.int8), transB, ldb)


def woq_dequant(packed, K, N, wei_dt, scale, zp=None, transB=False, ldb=None):
    """Weight-only quantisation, the reference's scalar definition (operators/matmul/matmul_ref_kernel.cpp:359-489): every
    4-bit weight becomes a bf16 value; s4, or u4 with an integer (s8) zero point: w = bf16((q - zp) * scale) (zp = 0 for s4);
    u4 with a bf16 zero point (uint16 bits): w = bf16((q - 8) * scale + zp).  scale (f32, or bf16 bits) and zp have 1, N or
    G*N elements ({G,N}: group g = k // (K/G)).  Returns bf16 bits [K,N]."""
    q = unpack_s4(packed, K, N, transB, ldb).astype(np.int32)
    if wei_dt == "u4":
        q = q & 0xF

    def expand(v):
        v = np.asarray(v)
        v = bf16_to_f32(v) if v.dtype == np.uint16 else v.astype(np.float32)
        v = v.reshape(-1)
        if v.size == 1:
            return np.full((K, N), v[0], dtype=np.float32)
        if v.size == N:
            return np.broadcast_to(v[None, :], (K, N)).astype(np.float32)
        G = v.size // N
        return np.repeat(v.reshape(G, N), K // G, axis=0).astype(np.float32)
    s = expand(scale)
    qf = q.astype(np.float32)
    if wei_dt == "u4" and zp is not None and np.asarray(zp).dtype == np.uint16:
        w = (qf - np.float32(8)) * s + expand(zp)
    elif wei_dt == "u4":
        w = (qf - expand(np.asarray(zp).astype(np.float32))) * s
    else:
        w = qf * s
    return f32_to_bf16(w.astype(np.float32))


def matmul_woq(A, packed, K, N, wei_dt, scale, zp=None, dst_dt="bf16", transB=False, ldb=None, bias=None, postops=()):
    """matmul_direct with bf16 activations and s4 | u4 weights, no quantisation of the activations: the weights are
    dequantised to bf16 (woq_dequant), then the bf16 x bf16 product."""
    return matmul_bf16(A, woq_dequant(packed, K, N, wei_dt, scale, zp, transB, ldb), dst_dt, bias=bias, postops=postops)


def quant_per_token_asym(x):
    """Asymmetric per-token dynamic quantisation: x [M,K] f32 or bf16-bits -> (u8 [M,K], f32 scales [M], s32 zero points [M])."""
    x = np.ascontiguousarray(x)
    M, K = x.shape
    q = np.empty((M, K), dtype=np.uint8)
    s = np.empty(M, dtype=np.float32)
    z = np.empty(M, dtype=np.int32)
    lib().orc_quant_per_token_asym(_p(x), _dt_of(x), C.c_int64(M), C.c_int64(K), C.c_int64(K), _p(q), C.c_int64(K), _p(s), _p(z))
    return q, s, z


def ref2_quant_per_token_asym(x, native=False):
    """Reference asymmetric per-token quantisation (scalar kernel, or the AVX-512 one).  None if unavailable."""
    r = ref2_lib()
    x = np.ascontiguousarray(x)
    M, K = x.shape
    if r is None or (native and not r.ref2_avx512()) or not hasattr(r, "ref2_quant_per_token_u8"):
        return None
    q = np.zeros((M, K), dtype=np.uint8)
    s = np.zeros(M, dtype=np.float32)
    z = np.zeros(M, dtype=np.int32)
    rc = r.ref2_quant_per_token_u8(_p(x), int(x.dtype == np.uint16), _p(q), _p(s), _p(z), C.c_int64(M), C.c_int64(K), int(native))
    return (q, s, z) if rc == 0 else None


def quant_per_group(x, G):
    """Dynamic symmetric quantisation with G groups along K per row (scale buffer {M,G}): the per-token rule applied to
    every group of K/G elements (reorder/lowoha_reorder.cpp:318-390).  Returns (s8 [M,K], f32 [M,G])."""
    x = np.ascontiguousarray(x)
    M, K = x.shape
    assert K % G == 0
    q, s = quant_per_token(x.reshape(M * G, K // G))
    return q.reshape(M, K), s.reshape(M, G)


def quant_per_token(x, scales_only=False):
    """x [M,K] f32 or bf16-bits.  Returns (s8 [M,K] or None, f32 scales [M])."""
    x = np.ascontiguousarray(x)
    M, K = x.shape
    q = None if scales_only else np.empty((M, K), dtype=np.int8)
    s = np.empty(M, dtype=np.float32)
    lib().orc_quant_per_token(_p(x), _dt_of(x), C.c_int64(M), C.c_int64(K), C.c_int64(K), _p(q),
                              C.c_int64(K), _p(s))
    return q, s


def dyn_scales(x, per_channel=True):
    x = np.ascontiguousarray(x)
    M, N = x.shape
    s = np.empty(N if per_channel else 1, dtype=np.float32)
    lib().orc_dyn_scales(_p(x), _dt_of(x), C.c_int64(M), C.c_int64(N), C.c_int64(N), int(per_channel), _p(s))
    return s


def quant_static(x, scale, zp=None, dst_dt="s8"):
    x = np.ascontiguousarray(x)
    M, N = x.shape
    scale = np.ascontiguousarray(np.asarray(scale, dtype=np.float32).reshape(-1))
    z = None if zp is None else np.ascontiguousarray(np.asarray(zp, dtype=np.int32).reshape(-1))
    out = np.empty((M, N), dtype=np.uint8 if dst_dt == "u8" else np.int8)
    lib().orc_quant_static(_p(x), _dt_of(x), C.c_int64(M), C.c_int64(N), C.c_int64(N), _p(scale),
                           C.c_int64(scale.size), _p(z), C.c_int64(0 if z is None else z.size), _p(out),
                           DT[dst_dt], C.c_int64(N))
    return out


def dequant_static(q, scale, zp=None, dst_dt="f32"):
    q = np.ascontiguousarray(q)
    M, N = q.shape
    scale = np.ascontiguousarray(np.asarray(scale, dtype=np.float32).reshape(-1))
    z = None if zp is None else np.ascontiguousarray(np.asarray(zp, dtype=np.int32).reshape(-1))
    out = np.empty((M, N), dtype=np.uint16 if dst_dt == "bf16" else np.float32)
    lib().orc_dequant_static(_p(q), _dt_of(q), C.c_int64(M), C.c_int64(N), C.c_int64(N), _p(scale),
                             C.c_int64(scale.size), _p(z), C.c_int64(0 if z is None else z.size), _p(out),
                             DT[dst_dt], C.c_int64(N))
    return out


def quant_weights_per_channel(w):
    """The reference tests' weight quantisation (gtests/gtest_utils.cpp:4269-4369): dynamic
    per-column scale, then static quantise.  w [K,N] f32 or bf16-bits -> (s8 [K,N], f32 [N])."""
    s = dyn_scales(w, per_channel=True)
    return quant_static(w, s), s


def gated_act(y, act="silu_and_mul"):
    """In-place semantics on a copy: y [M, 2I] f32 or bf16-bits -> [M, I]."""
    y = np.array(y, copy=True, order="C")
    M, N = y.shape
    lib().orc_gated_act(_p(y), _dt_of(y), C.c_int64(M), C.c_int64(N), C.c_int64(N), ACT[act])
    return np.ascontiguousarray(y[:, : N // 2])


def gated_act_f32_pairs(g, u, act="silu_and_mul", dst_dt="bf16"):
    g = np.ascontiguousarray(g, dtype=np.float32)
    u = np.ascontiguousarray(u, dtype=np.float32)
    out = np.empty(g.shape, dtype=np.uint16 if dst_dt == "bf16" else np.float32)
    lib().orc_gated_act_f32_pairs(_p(g), _p(u), C.c_int64(g.size), ACT[act], DT[dst_dt], _p(out))
    return out


def moe_weighted_reduce(rows, weights, topk, skip_weighted=False, fused=False):
    """rows [T*topk, D] (slot order t*topk+k) f32 or bf16-bits; weights [T,topk] f32."""
    rows = np.ascontiguousarray(rows)
    T = rows.shape[0] // topk
    D = rows.shape[1]
    ptrs = (C.c_void_p * (T * topk))(*[rows.ctypes.data + i * rows.strides[0] for i in range(T * topk)])
    w = np.ascontiguousarray(weights, dtype=np.float32)
    out = np.empty((T, D), dtype=rows.dtype)
    lib().orc_moe_weighted_reduce(ptrs, _p(w), T, topk, D, int(skip_weighted), _dt_of(rows), _p(out),
                                  C.c_int64(D), int(fused))
    return out


def router_topk(logits, k, renorm=True):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    T, E = logits.shape
    ids = np.empty((T, k), dtype=np.int32)
    w = np.empty((T, k), dtype=np.float32)
    lib().orc_router_topk(_p(logits), T, E, k, int(renorm), _p(ids), _p(w))
    return ids, w


def fused_moe(x_bf16, ids, weights, w13, s13, w2, s2, act="silu_and_mul", round_before_act=False, b13=None, b2=None):
    """Dynamic-INT8 fused MoE data flow of group_matmul_direct
    (group_matmul/group_matmul_fused_moe.cpp:906-1078; test convention
    gtests/group_matmul/test_fused_moe.cpp:2565-2676).

    x_bf16 [T,H] bf16-bits; ids/weights [T,k]; w13[e] s8 [H,2I] ([gate|up]) with scales s13[e] [2I];
    w2[e] s8 [I,H] with s2[e] [H].  Rows are gathered per expert in token order (stable), each
    expert runs quant -> GEMM -> act -> bf16 -> quant -> GEMM -> bf16, then the top-k weighted
    reduce.  round_before_act selects the separate-pass form (Op1 output rounded to bf16 before
    the activation, group_matmul_moe_act.cpp:110-117); default is the fused-epilogue form
    (group_matmul_act_avx512.hpp:62-70).  Returns (out [T,H] bf16-bits, expert row outputs
    [T*k, H] in slot order).  b13[e] [2I] / b2[e] [H]: optional f32 biases, added after the dequantisation and before
    the activation (group_matmul/custom_kernel/ukernel/int8_microkernel.cpp:161-177) / to the down projection
    (grp_matmul_fused_moe_params::bias_down)."""
    T, H = x_bf16.shape
    k = ids.shape[1]
    E = len(w13)
    slot_out = np.zeros((T * k, H), dtype=np.uint16)
    flat = ids.reshape(-1)
    for e in range(E):
        slots = np.nonzero(flat == e)[0]
        if slots.size == 0:
            continue
        xe = np.ascontiguousarray(x_bf16[slots // k])
        q1, sc1 = quant_per_token(xe)
        acc1 = gemm_s32(q1, w13[e])
        I = acc1.shape[1] // 2
        if round_before_act:
            y = epilogue(acc1, "bf16", sc1, s13[e], bias=None if b13 is None else b13[e])
            z = gated_act(y, act)
        else:
            y = epilogue(acc1, "f32", sc1, s13[e], bias=None if b13 is None else b13[e])
            if act == "swiglu_oai_mul":
                z = gated_act_f32_pairs(y[:, 0::2], y[:, 1::2], act)
            else:
                z = gated_act_f32_pairs(y[:, :I], y[:, I:], act)
        q2, sc2 = quant_per_token(z)
        o = matmul_w8a8(q2, w2[e], "bf16", src_scale=sc2, wei_scale=s2[e], bias=None if b2 is None else b2[e])
        slot_out[slots] = o
    out = moe_weighted_reduce(slot_out, weights, k)
    return out, slot_out


def fused_moe_bf16(x_bf16, ids, weights, w13, w2, act="silu_and_mul", b13=None, b2=None):
    """bf16:bf16:bf16 fused MoE of group_matmul_direct (no quantisation): per expert Y = X·W13 (+bias) in f32, gated
    activation on the f32 pairs, Z rounded to bf16, O = bf16(Z·W2 (+bias)), then the top-k weighted reduce
    (group_matmul/custom_kernel/ukernel/bf16_microkernel.hpp: activation in registers on the f32 accumulators).
    w13[e] bf16 bits [H,2I] ([gate|up]; element-interleaved for swiglu_oai_mul), w2[e] bf16 bits [I,H].
    Returns (out [T,H], expert row outputs [T*k,H] in slot order, Z rows [T*k,I])."""
    T, H = x_bf16.shape
    k = ids.shape[1]
    E = len(w13)
    I = w13[0].shape[1] // 2
    slot_out = np.zeros((T * k, H), dtype=np.uint16)
    slot_z = np.zeros((T * k, I), dtype=np.uint16)
    flat = ids.reshape(-1)
    for e in range(E):
        slots = np.nonzero(flat == e)[0]
        if slots.size == 0:
            continue
        xe = np.ascontiguousarray(x_bf16[slots // k])
        y = matmul_bf16(xe, w13[e], "f32", bias=None if b13 is None else b13[e])
        if act == "swiglu_oai_mul":
            z = gated_act_f32_pairs(y[:, 0::2], y[:, 1::2], act)
        else:
            z = gated_act_f32_pairs(y[:, :I], y[:, I:], act)
        slot_z[slots] = z
        slot_out[slots] = matmul_bf16(z, w2[e], "bf16", bias=None if b2 is None else b2[e])
    out = moe_weighted_reduce(slot_out, weights, k)
    return out, slot_out, slot_z


NORM = dict(layer_norm=0, batch_norm=1, rms_norm=2, fused_add_rms_norm=3)


def _norm_call(fn, kind, x, gamma, beta, residual, running_mean, running_var, eps, dst_dt, channels):
    x = np.ascontiguousarray(x)
    if kind == "batch_norm":
        batch, n = x.shape[0], int(np.prod(x.shape[2:], dtype=np.int64))
    else:
        batch, n = int(np.prod(x.shape[:-1], dtype=np.int64)), x.shape[-1]
    out = np.empty(x.shape, dtype={"bf16": np.uint16, "f32": np.float32}[dst_dt])
    g = None if gamma is None else np.ascontiguousarray(gamma)
    bt = None if beta is None else np.ascontiguousarray(beta)
    rm = None if running_mean is None else np.ascontiguousarray(running_mean, dtype=np.float32)
    rv = None if running_var is None else np.ascontiguousarray(running_var, dtype=np.float32)
    res = None if residual is None else np.array(residual, copy=True, order="C")
    rc = fn(NORM[kind], _p(x), _p(out), _p(g), _p(bt), _p(rm), _p(rv), _p(res), C.c_int64(batch), C.c_int64(n), C.c_int64(channels),
            C.c_float(eps), int(g is not None), int(bt is not None), _dt_of(x), DT[dst_dt], DT["f32"] if g is None else _dt_of(g),
            DT["f32"] if bt is None else _dt_of(bt))
    assert rc == 0, rc
    return (out, res) if kind == "fused_add_rms_norm" else out


def normalization(kind, x, gamma=None, beta=None, residual=None, running_mean=None, running_var=None, eps=1e-5, dst_dt=None):
    """normalization_direct as the reference's scalar kernel defines it (kernel/reference_kernel.cpp, f32 accumulation):
    kind in NORM; x f32 or bf16 bits, normalised over the last axis (batch_norm: x is [N, C, ...] with per-channel running
    statistics).  fused_add_rms_norm returns (output, updated residual)."""
    dst_dt = dst_dt or ("bf16" if np.asarray(x).dtype == np.uint16 else "f32")
    ch = np.asarray(x).shape[1] if kind == "batch_norm" else 0
    return _norm_call(lib().orc_normalization, kind, x, gamma, beta, residual, running_mean, running_var, eps, dst_dt, ch)


def ref2_normalization(kind, x, gamma=None, beta=None, residual=None, running_mean=None, running_var=None, eps=1e-5, dst_dt=None):
    """The reference's own scalar normalization kernel (normalization_reference_wrapper, compiled into libzendnn_ref2.so).
    None if unavailable."""
    r = ref2_lib()
    if r is None or not hasattr(r, "ref2_normalization"):
        return None
    dst_dt = dst_dt or ("bf16" if np.asarray(x).dtype == np.uint16 else "f32")
    ch = np.asarray(x).shape[1] if kind == "batch_norm" else 0
    return _norm_call(r.ref2_normalization, kind, x, gamma, beta, residual, running_mean, running_var, eps, dst_dt, ch)


def sdpa(q, k, v, mask=None, scale=0.0, causal=False):
    """softmax(Q K^T * scale + mask) V per (batch, head), the steps of the reference's BMM backend
    (lowoha_operators/sdpa/bmm_sdpa/lowoha_sdpa_bmm.cpp): scores from the exact bf16 products (summed in double, rounded to
    f32), scale (0: 1/sqrt(head_dim)), additive mask and causal mask (key j > query i) on the f32 scores, softmax in f32,
    probabilities rounded to bf16, P V summed in double, rounded to f32 and then to bf16.  q [B,H,S,D], k / v [B,H,KV,D] as
    bf16 bits; mask f32 broadcastable to [B,H,S,KV].  Returns bf16 bits [B,H,S,D]."""
    qf, kf, vf = (bf16_to_f32(a).astype(np.float64) for a in (q, k, v))
    B, H, S, D = qf.shape
    KV = kf.shape[2]
    sc = np.float32(1.0 / np.sqrt(np.float32(D))) if scale == 0.0 else np.float32(scale)
    s = np.einsum("bhsd,bhkd->bhsk", qf, kf).astype(np.float32) * sc
    if mask is not None:
        s = s + np.broadcast_to(np.asarray(mask, dtype=np.float32), s.shape)
    if causal:
        s = np.where(np.arange(KV)[None, :] > np.arange(S)[:, None], np.float32(-np.inf), s)
    m = s.max(axis=-1, keepdims=True)
    m = np.where(np.isfinite(m), m, np.float32(0))
    e = np.exp((s - m).astype(np.float32)).astype(np.float32)
    tot = e.sum(axis=-1, keepdims=True, dtype=np.float32)
    p = np.where(tot > 0, e / np.where(tot > 0, tot, 1), 0).astype(np.float32)
    pb = bf16_to_f32(f32_to_bf16(p)).astype(np.float64)
    return f32_to_bf16(np.einsum("bhsk,bhkd->bhsd", pb, vf).astype(np.float32))


def ref_int8_matmul(A_u8, B_s8, src_zp, src_scale, wei_scale, bias=None, fused_op=0, dst_dt="bf16"):
    """Runs the compiled reference tile kernel (per-tensor src scale/zp).  None if unavailable."""
    r = ref_lib()
    if r is None:
        return None
    A = np.ascontiguousarray(A_u8, dtype=np.uint8)
    B = np.ascontiguousarray(B_s8, dtype=np.int8)
    M, K = A.shape
    N = B.shape[1]
    ws = np.ascontiguousarray(np.asarray(wei_scale, dtype=np.float32).reshape(-1))
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    out = np.empty((M, N), dtype=np.uint16 if dst_dt == "bf16" else np.float32)
    rc = r.ref_int8_matmul(_p(A), K, _p(B), N, M, N, K, C.c_int32(int(src_zp)), C.c_float(float(src_scale)),
                           _p(ws), int(ws.size), _p(b), int(fused_op),
                           _p(out) if dst_dt == "bf16" else None, _p(out) if dst_dt == "f32" else None, N)
    return out if rc == 0 else None
