// Shared device/host helpers of libb200dnn: dtype codes, bf16 conversion, the dequantising
// epilogue used by every GEMM kernel, and small launch utilities.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

enum : int32_t { DT_NONE = 0, DT_F32 = 1, DT_F16 = 2, DT_BF16 = 3, DT_S32 = 4, DT_S8 = 7, DT_U8 = 11 };
enum : int32_t { PO_NONE = 0, PO_ELU = 1, PO_RELU = 2, PO_LEAKY_RELU = 3, PO_GELU_TANH = 4, PO_GELU_ERF = 5,
                 PO_SIGMOID = 6, PO_SWISH = 7, PO_TANH = 8, PO_CLIP = 16, PO_BINARY_ADD = 17,
                 PO_BINARY_MUL = 18, PO_MISH = 19 };
enum : int32_t { ACT_NONE = 0, ACT_SILU_MUL = 1, ACT_GELU_MUL = 2, ACT_SWIGLU_OAI = 3 };

constexpr int kNumSMs = 148;

// bf16 <-> f32 on the bit pattern, round-to-nearest-even exactly as the reference does it
// (common/bfloat16.cpp:68-82: bias 0x7FFF + lsb, no NaN special case).
__host__ __device__ __forceinline__ float bf16_bits_to_f32(uint16_t h) {
#ifdef __CUDA_ARCH__
  return __uint_as_float((uint32_t)h << 16);
#else
  union { uint32_t u; float f; } c; c.u = (uint32_t)h << 16; return c.f;
#endif
}
__host__ __device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
#ifdef __CUDA_ARCH__
  uint32_t u = __float_as_uint(f);
#else
  union { uint32_t u; float f; } c; c.f = f; uint32_t u = c.u;
#endif
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

__device__ __forceinline__ float load_as_f32(const void *p, int32_t dt, int64_t i) {
  switch (dt) {
  case DT_F32: return ((const float *)p)[i];
  case DT_BF16: return bf16_bits_to_f32(((const uint16_t *)p)[i]);
  case DT_S32: return (float)((const int32_t *)p)[i];
  case DT_S8: return (float)((const int8_t *)p)[i];
  case DT_U8: return (float)((const uint8_t *)p)[i];
  default: return 0.f;
  }
}

// ---- element-wise post-ops (formulas: operators/matmul/matmul_ref_kernel.cpp:694-761,
// constants matmul_ref_kernel.hpp:31-33; LowOHA mapping backends/aocl/aocl_postop.cpp:404-441).
// Every multiply/add that the reference performs as a separate f32 operation is written with
// the non-contracting intrinsics so that nvcc does not fuse it into an FMA.
__device__ __forceinline__ float act_sigmoid(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x))); }
__device__ __forceinline__ float po_gelu_tanh(float x) {
  const float c = 0.79788458347320556640625f, f = 0.044715f;
  float inner = __fmul_rn(__fmul_rn(c, x), __fadd_rn(1.0f, __fmul_rn(__fmul_rn(f, x), x)));
  float v = tanhf(inner);
  return __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, v));
}
__device__ __forceinline__ float po_gelu_erf(float x) {
  float v = __fmul_rn(x, 0.707106769084930419921875f);
  return __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, erff(v)));
}

struct PostOp {
  int32_t type;
  int32_t dt;
  const void *buff;
  int64_t ld;
  float alpha, beta;
};

// Everything a GEMM epilogue needs.  Passed by value as a kernel parameter.
struct EpiParams {
  const void *src_scale; int32_t src_scale_dt; int32_t src_scale_n;  // n: 0 none, 1 per-tensor, else per-row
  const void *wei_scale; int32_t wei_scale_dt; int32_t wei_scale_n;  // n: 0 none, 1 per-tensor, else per-column
  const void *src_zp; int32_t src_zp_dt; int32_t has_zp;
  const int32_t *colsum;   // per packed column: sum_k W[k,n]
  const void *bias; int32_t bias_dt; int32_t n_po;
  void *dst; int64_t ldc; int32_t dst_dt;
  int32_t gated_act;       // != 0: columns come as (gate,up) pairs, output is act(g)*u, I columns wide
  int32_t gated_I;         // I for the gated form
  uint32_t *row_absmax;    // gated form: per-row max |bf16(z)| as float bits (atomicMax)
  PostOp po[8];
};

__device__ __forceinline__ float apply_postop(const PostOp &p, float x, int m, int n) {
  switch (p.type) {
  case PO_RELU: return x > 0.f ? x : 0.f;
  case PO_LEAKY_RELU: return x > 0.f ? x : __fmul_rn(0.01f, x);
  case PO_ELU: return x > 0.f ? x : __fmul_rn(p.alpha, __fadd_rn(expf(x), -1.0f));
  case PO_GELU_TANH: return po_gelu_tanh(x);
  case PO_GELU_ERF: return po_gelu_erf(x);
  case PO_SIGMOID: return act_sigmoid(x);
  case PO_SWISH: return __fmul_rn(x, act_sigmoid(x));
  case PO_TANH: return tanhf(x);
  case PO_MISH: return __fmul_rn(x, tanhf(__fadd_rn(fmaxf(x, 0.0f), log1pf(expf(-fabsf(x))))));   // x * tanh(softplus(x))
  case PO_CLIP: { float lo = p.alpha, hi = p.beta; x = x > lo ? x : lo; return x > hi ? hi : x; }
  case PO_BINARY_ADD: return __fadd_rn(x, load_as_f32(p.buff, p.dt, p.ld ? (int64_t)m * p.ld + n : n));
  case PO_BINARY_MUL: return __fmul_rn(x, load_as_f32(p.buff, p.dt, p.ld ? (int64_t)m * p.ld + n : n));
  default: return x;
  }
}

__device__ __forceinline__ int32_t load_zp(const EpiParams &e) {
  if (!e.has_zp) return 0;
  switch (e.src_zp_dt) {
  case DT_S32: return *(const int32_t *)e.src_zp;
  case DT_S8: return *(const int8_t *)e.src_zp;
  case DT_U8: return *(const uint8_t *)e.src_zp;
  default: return 0;
  }
}

__device__ __forceinline__ bool finite_f32(float v) { return (__float_as_uint(v) & 0x7F800000u) != 0x7F800000u; }

// Per-row / per-group view of the epilogue operands (the grouped GEMM swaps these per expert).
struct EpiCtx {
  const void *wei_scale;
  const int32_t *colsum;
  const void *bias;
  void *dst;
  int64_t ldc;
  float s_src;   // src scale of this row (1 when absent)
};
__device__ __forceinline__ EpiCtx epi_ctx(const EpiParams &e, int m_scale) {
  EpiCtx c;
  c.wei_scale = e.wei_scale; c.colsum = e.colsum; c.bias = e.bias; c.dst = e.dst; c.ldc = e.ldc;
  c.s_src = e.src_scale_n ? load_as_f32(e.src_scale, e.src_scale_dt, e.src_scale_n > 1 ? m_scale : 0) : 1.0f;
  return c;
}
// s32 accumulator -> dequantised f32 (before bias): exact s32 zero-point compensation, then
// x*src_scale, then *wei_scale[n] as two separate multiplies
// (backends/aocl/aocl_postop.cpp:1339-1395; group custom kernel int8_microkernel.cpp:161-177).
// `pn` indexes colsum (packed column), `n` the caller's column.
__device__ __forceinline__ float epi_dequant(const EpiParams &e, const EpiCtx &c, int32_t acc, int32_t zp, int n, int pn) {
  if (zp != 0) acc -= zp * c.colsum[pn];
  float x = (float)acc;
  if (e.src_scale_n) x = __fmul_rn(x, c.s_src);
  if (e.wei_scale_n) x = __fmul_rn(x, load_as_f32(c.wei_scale, e.wei_scale_dt, e.wei_scale_n > 1 ? n : 0));
  return x;
}
__device__ __forceinline__ float epi_finish(const EpiParams &e, const EpiCtx &c, float x, int m, int n) {
  if (c.bias) x = __fadd_rn(x, load_as_f32(c.bias, e.bias_dt, n));
  for (int i = 0; i < e.n_po; ++i) x = apply_postop(e.po[i], x, m, n);
  return x;
}
// gated activations on f32 (g,u): group_matmul/group_matmul_moe_act.cpp:88-145
__device__ __forceinline__ float gated_f32(int act, float g, float u) {
  if (act == ACT_SILU_MUL) return __fmul_rn(__fmul_rn(g, act_sigmoid(g)), u);
  if (act == ACT_GELU_MUL)
    return __fmul_rn(__fmul_rn(__fmul_rn(g, 0.5f), __fadd_rn(1.0f, erff(__fmul_rn(g, 0.70710678118654752440f)))), u);
  g = fmaxf(-7.0f, fminf(g, 7.0f)); u = fmaxf(-7.0f, fminf(u, 7.0f));
  return __fmul_rn(__fmul_rn(__fadd_rn(1.0f, u), g), act_sigmoid(__fmul_rn(g, 1.702f)));
}

}  // namespace b200
