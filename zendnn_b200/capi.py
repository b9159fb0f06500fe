"""ctypes binding of libb200dnn.so (include/b200dnn.h).

Buffers may be numpy arrays (host memory) or torch tensors (host or CUDA); only their address
is passed on.  There is no fallback: if the shared library is missing, importing this module
raises, and every compute call fails when no CUDA device is present.
"""
import ctypes as C
import os

import numpy as np

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libb200dnn.so")

SUCCESS, FAILURE, UNIMPLEMENTED = 1, 0, -1
DT = dict(none=0, f32=1, f16=2, bf16=3, s32=4, s64=5, s16=6, s8=7, s4=8, u32=9, u16=10, u8=11, u4=12)
PO = dict(none=0, elu=1, relu=2, leaky_relu=3, gelu_tanh=4, gelu_erf=5, sigmoid=6, swish=7, tanh=8,
          softmax=9, pooling=10, square=11, abs=12, sqrt=13, exp=14, log=15, clip=16, binary_add=17,
          binary_mul=18, mish=19)
ACT = dict(none=0, silu_and_mul=1, gelu_and_mul=2, swiglu_oai_mul=3)
MAX_POSTOPS = 8


class Quant(C.Structure):
    _fields_ = [("buff", C.c_void_p), ("dt", C.c_int32), ("reserved", C.c_int32), ("count", C.c_int64)]


class PostOp(C.Structure):
    _fields_ = [("type", C.c_int32), ("dt", C.c_int32), ("buff", C.c_void_p), ("ld", C.c_int64),
                ("alpha", C.c_float), ("beta", C.c_float)]


class MatmulDesc(C.Structure):
    _fields_ = [("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32), ("transB", C.c_int32),
                ("src_dt", C.c_int32), ("wei_dt", C.c_int32), ("dst_dt", C.c_int32), ("bias_dt", C.c_int32),
                ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64),
                ("src", C.c_void_p), ("weight", C.c_void_p), ("bias", C.c_void_p), ("dst", C.c_void_p),
                ("wei_format", C.c_int32), ("weights_const", C.c_int32), ("dynamic_quant", C.c_int32),
                ("n_postops", C.c_int32),
                ("src_scale", Quant), ("wei_scale", Quant), ("src_zp", Quant),
                ("postops", PostOp * MAX_POSTOPS),
                ("force_kernel", C.c_int32), ("flags", C.c_int32),
                ("dst_scale", Quant), ("dst_zp", Quant), ("wei_zp", Quant), ("transA", C.c_int32), ("reserved_a", C.c_int32)]

FLAG_STABLE_WEIGHTS = 1


class MoeExpert(C.Structure):
    _fields_ = [("M", C.c_int32), ("wei_dt", C.c_int32), ("src", C.c_void_p), ("lda", C.c_int64),
                ("w13", C.c_void_p), ("ldb13", C.c_int64), ("w13_scale", C.c_void_p),
                ("w2", C.c_void_p), ("ldb2", C.c_int64), ("w2_scale", C.c_void_p),
                ("dst_down", C.c_void_p), ("ldc_down", C.c_int64),
                ("bias13", C.c_void_p), ("bias13_dt", C.c_int32), ("reserved2", C.c_int32),
                ("bias2", C.c_void_p), ("bias2_dt", C.c_int32), ("reserved3", C.c_int32),
                ("dst_op1", C.c_void_p), ("ldc_op1", C.c_int64)]


class NormDesc(C.Structure):
    _fields_ = [("norm_type", C.c_int32), ("use_scale", C.c_int32), ("use_shift", C.c_int32), ("epsilon", C.c_float),
                ("batch", C.c_int64), ("norm_size", C.c_int64), ("num_channels", C.c_int64),
                ("src_dt", C.c_int32), ("dst_dt", C.c_int32), ("gamma_dt", C.c_int32), ("beta_dt", C.c_int32),
                ("input", C.c_void_p), ("output", C.c_void_p), ("gamma", C.c_void_p), ("beta", C.c_void_p),
                ("running_mean", C.c_void_p), ("running_var", C.c_void_p), ("residual", C.c_void_p),
                ("quant_dst", C.c_void_p), ("quant_ld", C.c_int64), ("quant_scale", C.c_void_p)]


NORM = dict(layer_norm=0, batch_norm=1, rms_norm=2, fused_add_rms_norm=3)


class SdpaDesc(C.Structure):
    _fields_ = [("batch", C.c_int64), ("num_heads", C.c_int64), ("seq_len", C.c_int64), ("kv_seq_len", C.c_int64), ("head_dim", C.c_int64),
                ("q_stride", C.c_int64 * 4), ("k_stride", C.c_int64 * 4), ("v_stride", C.c_int64 * 4), ("o_stride", C.c_int64 * 4),
                ("mask_ndims", C.c_int32), ("is_causal", C.c_int32), ("mask_sizes", C.c_int64 * 4), ("mask_strides", C.c_int64 * 4),
                ("qkv_dt", C.c_int32), ("out_dt", C.c_int32), ("mask_dt", C.c_int32), ("reserved", C.c_int32),
                ("scale", C.c_double), ("dropout_p", C.c_double),
                ("query", C.c_void_p), ("key", C.c_void_p), ("value", C.c_void_p), ("attn_mask", C.c_void_p), ("output", C.c_void_p)]


class EpConfig(C.Structure):
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("num_experts", C.c_int32), ("num_shared", C.c_int32),
                ("topk", C.c_int32), ("max_tokens", C.c_int32), ("K", C.c_int32), ("I", C.c_int32), ("H", C.c_int32),
                ("transB", C.c_int32), ("act", C.c_int32), ("capacity_rows", C.c_int32), ("expert_rank", C.c_void_p)]


PHASES = 9
PHASE_NAMES = ["route+rank", "count exchange", "quantise+dispatch", "barrier after dispatch", "gemm1+act", "requantise", "gemm2",
               "barrier before combine", "combine+reduce"]

EXPORTS = ["b200dnn_last_error", "b200dnn_version", "b200dnn_device_count", "b200dnn_launch_count",
           "b200dnn_matmul", "b200dnn_matmul_static_scratch", "b200dnn_static_scratch_query", "b200dnn_prepack_size", "b200dnn_prepack", "b200dnn_quant_per_token",
           "b200dnn_group_quant_per_token", "b200dnn_quant_per_token_asym", "b200dnn_quant_dynamic", "b200dnn_quant_prepack", "b200dnn_quant_static",
           "b200dnn_dequant_static", "b200dnn_gated_act", "b200dnn_moe_weighted_reduce", "b200dnn_fused_moe", "b200dnn_group_matmul", "b200dnn_nshard_range", "b200dnn_nshard_create", "b200dnn_nshard_destroy", "b200dnn_matmul_nshard",
           "b200dnn_moe_route", "b200dnn_moe_layer", "b200dnn_clear_caches", "b200dnn_stream_status", "b200dnn_moe_sort_slots",
           "b200dnn_quant_per_token_gather", "b200dnn_quant_per_token_scatter", "b200dnn_moe_experts_s8",
           "b200dnn_moe_weighted_reduce_rows", "b200dnn_ep_create", "b200dnn_ep_destroy", "b200dnn_ep_local_expert_count",
           "b200dnn_ep_set_experts", "b200dnn_ep_nccl_unique_id", "b200dnn_ep_connect_nccl", "b200dnn_ep_connect_local",
           "b200dnn_moe_layer_ep", "b200dnn_moe_layer_ep_local", "b200dnn_ep_rows_per_rank", "b200dnn_ep_status",
           "b200dnn_phase_timing", "b200dnn_phase_times", "b200dnn_measure_int8_peak", "b200dnn_normalization", "b200dnn_sdpa"]

if not os.path.exists(LIB_PATH):
    raise ImportError(
        "zendnn_b200: %s is missing. Build it with `python -m zendnn_b200.build`; there is no "
        "Python or CPU fallback for the kernels." % LIB_PATH)

lib = C.CDLL(LIB_PATH)
lib.b200dnn_last_error.restype = C.c_char_p
lib.b200dnn_prepack_size.restype = C.c_size_t
lib.b200dnn_prepack_size.argtypes = [C.c_int64, C.c_int64, C.c_int32]
lib.b200dnn_launch_count.restype = C.c_int64
i32, i64, vp = C.c_int32, C.c_int64, C.c_void_p
lib.b200dnn_matmul.argtypes = [C.POINTER(MatmulDesc), vp]
lib.b200dnn_matmul_static_scratch.argtypes = [C.POINTER(MatmulDesc), vp]
lib.b200dnn_static_scratch_query.argtypes = [i32, i32, i32, i32, C.POINTER(C.c_size_t)]
lib.b200dnn_prepack.argtypes = [vp, i64, i64, i64, i32, i32, vp, vp]
lib.b200dnn_quant_prepack.argtypes = [vp, i32, i64, i64, i64, i32, i32, vp, vp, vp]
lib.b200dnn_quant_per_token.argtypes = [vp, i32, i64, i64, i64, vp, i64, vp, i32, vp]
lib.b200dnn_group_quant_per_token.argtypes = [i32, vp, i32, vp, vp, vp, vp, vp, vp, i32, vp]
lib.b200dnn_quant_dynamic.argtypes = [vp, i32, i64, i64, i64, i32, vp, i64, vp, vp]
lib.b200dnn_quant_static.argtypes = [vp, i32, i64, i64, i64, vp, i64, vp, i64, vp, i32, i64, vp]
lib.b200dnn_dequant_static.argtypes = [vp, i32, i64, i64, i64, vp, i64, vp, i64, vp, i32, i64, vp]
lib.b200dnn_gated_act.argtypes = [vp, i32, i64, i64, i64, i32, vp]
lib.b200dnn_moe_weighted_reduce.argtypes = [vp, vp, i32, i32, i32, i32, i32, vp, i64, vp]
lib.b200dnn_quant_per_token_asym.argtypes = [vp, i32, i64, i64, i64, vp, i64, vp, vp, vp]
lib.b200dnn_normalization.argtypes = [C.POINTER(NormDesc), C.c_void_p]
lib.b200dnn_sdpa.argtypes = [C.POINTER(SdpaDesc), C.c_void_p]
lib.b200dnn_nshard_range.argtypes = [i64, i32, i32, C.POINTER(i64), C.POINTER(i64), C.POINTER(i32)]
lib.b200dnn_nshard_create.argtypes = [i32, i32, vp, vp, C.POINTER(vp)]
lib.b200dnn_nshard_destroy.argtypes = [vp]
lib.b200dnn_matmul_nshard.argtypes = [vp, C.POINTER(MatmulDesc), i32, vp]
lib.b200dnn_group_matmul.argtypes = [i32, C.POINTER(MatmulDesc), vp]
lib.b200dnn_fused_moe.argtypes = [i32, C.POINTER(MoeExpert), i32, i32, i32, i32, i32, i32, vp, vp, i32, i32, vp, i64, vp]
lib.b200dnn_moe_route.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp, vp, vp]
lib.b200dnn_moe_layer.argtypes = [vp, i64, vp, i32, i32, i32, i32, C.POINTER(MoeExpert), i32, i32, i32, i32, i32, vp, i64, vp]


lib.b200dnn_stream_status.argtypes = [vp]
lib.b200dnn_moe_sort_slots.argtypes = [vp, i32, i32, vp, vp, vp]
lib.b200dnn_quant_per_token_gather.argtypes = [vp, i32, i64, i64, vp, i32, i64, vp, i64, vp, vp]
lib.b200dnn_quant_per_token_scatter.argtypes = [vp, i32, i64, i64, vp, i32, i64, vp, i64, vp, vp]
lib.b200dnn_moe_experts_s8.argtypes = [vp, i64, vp, i32, vp, vp, C.POINTER(MoeExpert), i32, i32, i32, i32, i32, vp, i64, vp]
lib.b200dnn_moe_weighted_reduce_rows.argtypes = [vp, i64, vp, vp, i32, i32, i32, i32, vp, i64, vp]


lib.b200dnn_ep_create.argtypes = [C.POINTER(EpConfig), C.POINTER(vp)]
lib.b200dnn_ep_destroy.argtypes = [vp]
lib.b200dnn_ep_local_expert_count.argtypes = [vp, C.POINTER(i32)]
lib.b200dnn_ep_set_experts.argtypes = [vp, C.POINTER(MoeExpert), i32]
lib.b200dnn_ep_nccl_unique_id.argtypes = [vp]
lib.b200dnn_ep_connect_nccl.argtypes = [vp, vp, vp]
lib.b200dnn_ep_connect_local.argtypes = [C.POINTER(vp), i32]
lib.b200dnn_moe_layer_ep.argtypes = [vp, vp, i64, vp, i32, vp, i64, vp]
lib.b200dnn_moe_layer_ep_local.argtypes = [C.POINTER(vp), i32, C.POINTER(vp), i64, C.POINTER(vp), C.POINTER(i32), C.POINTER(vp), i64, vp]
lib.b200dnn_ep_rows_per_rank.argtypes = [vp, C.POINTER(i32), vp]
lib.b200dnn_ep_status.argtypes = [vp, vp]
lib.b200dnn_phase_timing.argtypes = [vp, i32]
lib.b200dnn_phase_times.argtypes = [vp, C.POINTER(C.c_float), i32, C.POINTER(i32)]
lib.b200dnn_measure_int8_peak.argtypes = [i32, i32, C.POINTER(C.c_float), C.POINTER(C.c_double), vp]


class B200DNNError(RuntimeError):
    def __init__(self, status, text):
        super().__init__("b200dnn status %d: %s" % (status, text))
        self.status = status


def last_error():
    return lib.b200dnn_last_error().decode()


def check(status):
    if status != SUCCESS:
        raise B200DNNError(status, last_error())
    return status


def ptr(buf):
    """Address of a numpy array, torch tensor, raw int or None."""
    if buf is None:
        return None
    if isinstance(buf, int):
        return buf
    if isinstance(buf, np.ndarray):
        return buf.ctypes.data
    if hasattr(buf, "data_ptr"):
        return buf.data_ptr()
    raise TypeError("unsupported buffer type %r" % type(buf))


def dt_of(buf, bf16_bits=True):
    """dtype code of a numpy / torch buffer; uint16 numpy arrays and int16 tensors carry bf16 bits."""
    name = str(buf.dtype).replace("torch.", "")
    table = {"float32": "f32", "bfloat16": "bf16", "uint16": "bf16", "int16": "bf16", "int32": "s32",
             "int8": "s8", "uint8": "u8"}
    return DT[table[name]]


def quant(buf, count=None, dt=None):
    q = Quant()
    if buf is None and not count:
        return q
    q.buff = ptr(buf)
    q.dt = dt if dt is not None else (dt_of(buf) if buf is not None else DT["f32"])
    q.count = int(count if count is not None else buf.size if isinstance(buf, np.ndarray) else buf.numel())
    return q


def make_matmul(M, N, K, src, weight, dst, *, src_dt, dst_dt, lda=None, ldb=None, ldc=None, transB=False,
                bias=None, bias_dt=None, wei_format="n", weights_const=True, dynamic_quant=False,
                src_scale=None, wei_scale=None, src_zp=None, postops=(), force_kernel=0, flags=0, wei_dt=None,
                dst_scale=None, dst_zp=None, wei_zp=None, transA=False):
    d = MatmulDesc()
    d.M, d.N, d.K, d.transB = M, N, K, int(transB)
    d.transA = int(transA)
    d.src_dt, d.wei_dt, d.dst_dt = src_dt, (DT["s8"] if wei_dt is None else wei_dt), dst_dt
    d.bias_dt = bias_dt if bias_dt is not None else (dt_of(bias) if bias is not None else 0)
    d.lda = lda if lda is not None else (M if transA else K)
    d.ldb = ldb if ldb is not None else (K if transB else N)
    d.ldc = ldc if ldc is not None else N
    d.src, d.weight, d.bias, d.dst = ptr(src), ptr(weight), ptr(bias), ptr(dst)
    d.wei_format = ord(wei_format)
    d.weights_const = int(weights_const)
    d.dynamic_quant = int(dynamic_quant)
    if isinstance(src_scale, Quant):
        d.src_scale = src_scale
    elif src_scale is not None:
        d.src_scale = quant(src_scale)
    if isinstance(wei_scale, Quant):
        d.wei_scale = wei_scale
    elif wei_scale is not None:
        d.wei_scale = quant(wei_scale)
    if isinstance(src_zp, Quant):
        d.src_zp = src_zp
    elif src_zp is not None:
        d.src_zp = quant(src_zp)
    d.n_postops = len(postops)
    for i, po in enumerate(postops):
        if isinstance(po, str):
            po = dict(type=po)
        d.postops[i].type = PO[po["type"]]
        d.postops[i].alpha = po.get("alpha", 0.0)
        d.postops[i].beta = po.get("beta", 0.0)
        b = po.get("buff")
        if b is not None:
            d.postops[i].buff = ptr(b)
            d.postops[i].dt = dt_of(b)
            shape = tuple(b.shape)
            d.postops[i].ld = po.get("ld", 0 if (len(shape) == 1 or shape[0] == 1) else shape[-1])
    d.force_kernel = force_kernel
    d.flags = flags
    if dst_scale is not None:
        d.dst_scale = dst_scale if isinstance(dst_scale, Quant) else quant(dst_scale)
    if dst_zp is not None:
        d.dst_zp = dst_zp if isinstance(dst_zp, Quant) else quant(dst_zp)
    if wei_zp is not None:
        d.wei_zp = wei_zp if isinstance(wei_zp, Quant) else quant(wei_zp)
    return d


def matmul(desc, stream=None):
    return lib.b200dnn_matmul(C.byref(desc), stream)
