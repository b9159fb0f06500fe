// Test-only driver around more of the REFERENCE's own code on the path: the dynamic per-token
// quantisation kernels (scalar and AVX-512), the gated activations and the MoE weighted reduce.
// oracle/Makefile compiles those reference files where they lie (together with the reference's common/
// sources they depend on) and links them with this driver into oracle/_ref/libzendnn_ref2.so; no
// reference source is copied.  Every function below only forwards its arguments.
//
//   reorder/reorder_data_type/scalar_impl/dynamic_per_token_ref_kernel.cpp
//   reorder/reorder_data_type/dynamic_quant_impl/per_token_avx512_f32_fma_kernel.cpp
//   matmul/group_matmul/group_matmul_moe_act.cpp
//   matmul/group_matmul/group_matmul_moe_postop.cpp
//   reorder/lowoha_reorder_utils.cpp (compute_dynamic_quant_params: per-channel / per-tensor dynamic scales)
//   reorder/reorder_data_type/scalar_impl/scalar_granular_impl.cpp (static quantise / dequantise with granular scales)
//   matmul/group_matmul/custom_kernel/ukernel/int8_microkernel.cpp (the DQ-INT8 tile micro-kernel of group_matmul_direct:
//     VNNI GEMM, exact s32 compensation, x src scale, x weight scale, + bias, gated activation in registers)
//   normalization/kernel/reference_kernel.cpp (the scalar LayerNorm / BatchNorm / RMSNorm / fused-add RMSNorm)
//   matmul/group_matmul/custom_kernel/ukernel/bf16_microkernel.cpp (the bf16 tile micro-kernel of group_matmul_direct:
//     VDPBF16PS GEMM with f32 accumulators, + bias, gated activation in registers)
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "lowoha_operators/matmul/group_matmul/custom_kernel/ukernel/int8_microkernel.hpp"
#include "lowoha_operators/matmul/group_matmul/custom_kernel/ukernel/bf16_microkernel.hpp"

#include "lowoha_operators/normalization/kernel/reference_kernel.hpp"
#include "lowoha_operators/matmul/group_matmul/group_matmul_direct.hpp"
#include "lowoha_operators/reorder/lowoha_reorder_utils.hpp"
#include "lowoha_operators/reorder/reorder_data_type/scalar_impl/scalar_kernels.hpp"
#include "lowoha_operators/reorder/reorder_data_type/dynamic_quant_impl/dynamic_kernels.hpp"

namespace zendnnl { namespace lowoha { namespace reorder {
void dynamic_per_token_quant_bf16_s8_ref(const uint16_t *, int8_t *, float *, int64_t, int64_t);
void dynamic_per_token_quant_f32_s8_ref(const float *, int8_t *, float *, int64_t, int64_t);
void dynamic_per_token_quant_bf16_s8_native(const uint16_t *, int8_t *, float *, int64_t, int64_t);
void dynamic_per_token_quant_f32_s8_native(const float *, int8_t *, float *, int64_t, int64_t);
}}}

#define API extern "C" __attribute__((visibility("default")))

API int ref2_avx512() {
  __builtin_cpu_init();
  return __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw") && __builtin_cpu_supports("avx512vl");
}

// src: [M,K] contiguous, bf16 bits (is_bf16) or f32; dst s8 [M,K]; scale f32 [M].  native: the AVX-512 kernel.
API int ref2_quant_per_token(const void *src, int is_bf16, int8_t *dst, float *scale, int64_t M, int64_t K, int native) {
  using namespace zendnnl::lowoha::reorder;
  if (native && !ref2_avx512()) return -1;
  if (is_bf16) {
    if (native) dynamic_per_token_quant_bf16_s8_native((const uint16_t *)src, dst, scale, M, K);
    else dynamic_per_token_quant_bf16_s8_ref((const uint16_t *)src, dst, scale, M, K);
  } else {
    if (native) dynamic_per_token_quant_f32_s8_native((const float *)src, dst, scale, M, K);
    else dynamic_per_token_quant_f32_s8_ref((const float *)src, dst, scale, M, K);
  }
  return 0;
}

// Asymmetric per-token quantisation to u8 with one f32 scale and one s32 zero point per row.
API int ref2_quant_per_token_u8(const void *src, int is_bf16, uint8_t *dst, float *scale, int32_t *zp, int64_t M, int64_t K, int native) {
  using namespace zendnnl::lowoha::reorder;
  if (native && !ref2_avx512()) return -1;
  if (is_bf16) {
    if (native) dynamic_per_token_quant_bf16_u8_native((const uint16_t *)src, dst, scale, zp, M, K);
    else dynamic_per_token_quant_bf16_u8_ref((const uint16_t *)src, dst, scale, zp, M, K);
  } else {
    if (native) dynamic_per_token_quant_f32_u8_native((const float *)src, dst, scale, zp, M, K);
    else dynamic_per_token_quant_f32_u8_ref((const float *)src, dst, scale, zp, M, K);
  }
  return 0;
}

// Per-group dynamic quantisation along K (scale layout {M,G}), the reference's AVX-512 kernel
// (reorder/reorder_data_type/dynamic_quant_impl/per_group_avx512_f32_fma_kernel.cpp).
API int ref2_quant_per_group(const void *src, int is_bf16, int8_t *dst, float *scale, int64_t M, int64_t K, int64_t G) {
  using namespace zendnnl::lowoha::reorder;
  if (!ref2_avx512()) return -1;
  if (is_bf16) dynamic_per_group_quant_bf16_s8_native((const uint16_t *)src, dst, scale, M, K, G);
  else dynamic_per_group_quant_f32_s8_native((const float *)src, dst, scale, M, K, G);
  return 0;
}

// In place on buf [M, N = 2I] (row stride ldc elements); dt: 1 f32, 3 bf16 (data_type_t values).
API int ref2_gated_act(int act, void *buf, int M, int N, int ldc, int dt) {
  using namespace zendnnl::lowoha::matmul;
  apply_gated_act_inplace((grp_matmul_gated_act_t)act, buf, 0, M, N, ldc, (zendnnl::common::data_type_t)dt);
  return 0;
}

// rows: [T*topk] pointers to D-wide rows; weights [T*topk] (null with skip_weighted); out [T, ld_out].
API int ref2_moe_reduce(const void **row_ptrs, const float *weights, int skip_weighted, int T, int topk, int D, int dt,
                        void *out, int ld_out, int num_threads) {
  using namespace zendnnl::lowoha::matmul;
  group_matmul_moe_postop_params p;
  p.num_tokens = T; p.topk = topk; p.output = out; p.ldc_output = ld_out; p.topk_weights = weights;
  p.skip_weighted = skip_weighted != 0; p.row_ptrs = row_ptrs;
  return (int)group_matmul_moe_postop_execute(&p, D, num_threads, (zendnnl::common::data_type_t)dt);
}

// Dynamic scales of a [M,N] matrix (f32 or bf16 bits, contiguous): per_channel -> scale[N] (dims {1,N}), else one
// scale (dims {1,1}); symmetric s8 target.  Returns the reference's status_t.
API int ref2_dyn_scales(const void *src, int src_dt, int64_t M, int64_t N, int per_channel, float *scale) {
  using namespace zendnnl::lowoha::reorder;
  reorder_params_t p;
  p.src_dtype = (zendnnl::common::data_type_t)src_dt; p.dst_dtype = zendnnl::common::data_type_t::s8;
  p.src_shape = {M, N}; p.dst_shape = {M, N}; p.dynamic_quant = true; p.num_threads = 1;
  p.quant_params.scale.buff = scale; p.quant_params.scale.dt = zendnnl::common::data_type_t::f32;
  p.quant_params.scale.dims = per_channel ? std::vector<int64_t>{1, N} : std::vector<int64_t>{1, 1};
  return (int)compute_dynamic_quant_params(src, p);
}

// Static quantise (src f32/bf16 -> dst s8/u8) or dequantise (src s8/u8 -> dst f32/bf16) of a contiguous [M,N]
// matrix with scale dims {sr, sc} (f32) and optional zero point dims {zr, zc} (s32), through the reference's
// scalar granular implementation.
API int ref2_granular(const void *src, int src_dt, void *dst, int dst_dt, int64_t M, int64_t N, float *scale, int64_t sr,
                      int64_t sc, int32_t *zp, int64_t zr, int64_t zc) {
  using namespace zendnnl::lowoha::reorder;
  reorder_params_t p;
  p.src_dtype = (zendnnl::common::data_type_t)src_dt; p.dst_dtype = (zendnnl::common::data_type_t)dst_dt;
  p.src_shape = {M, N}; p.dst_shape = {M, N}; p.num_threads = 1;
  p.quant_params.scale.buff = scale; p.quant_params.scale.dt = zendnnl::common::data_type_t::f32;
  p.quant_params.scale.dims = {sr, sc};
  if (zp) {
    p.quant_params.zero_point.buff = zp; p.quant_params.zero_point.dt = zendnnl::common::data_type_t::s32;
    p.quant_params.zero_point.dims = {zr, zc};
  }
  reorder_granular_scaler_impl_2d(src, dst, p);
  return 0;
}

// The reference's DQ-INT8 micro-kernel (s8 symmetric source) over a whole [M,K] x [K,N] problem.  The driver does what
// the kernel's contract asks of its caller (custom_kernel/pack.hpp:212-232): per block of 32 packed columns, the weight
// bytes as [K/4][32][4] followed by the 32 int32 column sums; for silu_and_mul / gelu_and_mul the caller's split halves
// [gate | up] are re-ordered into (g0,u0,g1,u1,...) pairs, and the per-column scales and bias follow the same order.
// act: the kernel's ActKind (0 none, 1 swiglu_oai_mul, 2 silu_and_mul, 3 gelu_and_mul).  K % 4 == 0, N % 32 == 0.
// out: bf16 bits, [M,N] for act 0, else [M,N/2].  Returns 0 on success.
API int ref2_int8_ukernel(const int8_t *A, const int8_t *B, int M, int N, int K, const float *src_scale, const float *wei_scale,
                          const float *bias, int act, uint16_t *out) {
  using namespace zendnnl::lowoha::matmul::custom_kernel;
  if (!avx512vnni_available() || K % 4 != 0 || N % 32 != 0 || M <= 0) return -1;
  const int NR = 32, I = N / 2, kq = K / 4;
  auto src_col = [&](int p) { return (act == 2 || act == 3) ? ((p & 1) ? I + p / 2 : p / 2) : p; };
  const size_t slab_bytes = (size_t)kq * NR * 4 + NR * sizeof(int32_t);
  int8_t *slab = static_cast<int8_t *>(aligned_alloc(64, (slab_bytes + 63) / 64 * 64));
  std::vector<float> ws(NR), bs(NR);
  for (int ob = 0; ob < N / NR; ++ob) {
    int32_t *comp = reinterpret_cast<int32_t *>(slab + (size_t)kq * NR * 4);
    for (int c = 0; c < NR; ++c) {
      const int sc = src_col(ob * NR + c);
      int32_t sum = 0;
      for (int k = 0; k < K; ++k) { const int8_t v = B[(size_t)k * N + sc]; slab[((size_t)(k / 4) * NR + c) * 4 + (k % 4)] = v; sum += v; }
      comp[c] = sum; ws[c] = wei_scale[sc]; bs[c] = bias ? bias[sc] : 0.f;
    }
    for (int m = 0; m < M;) {
      const int MR = M - m >= 8 ? 8 : M - m;
      int8_ukernel_fn_t fn = select_int8_ukernel(MR, 2, IntCompute::kS8_Sym, static_cast<ActKind>(act), DstDt::kBf16);
      if (!fn) { free(slab); return -2; }
      void *full = act == 0 ? out + (size_t)m * N + ob * NR : nullptr;
      void *tight = act == 0 ? nullptr : out + (size_t)m * I + ob * (NR / 2);
      fn(reinterpret_cast<const uint8_t *>(A) + (size_t)m * K, K, slab, src_scale + m, nullptr, ws.data(), ScaleKind::kF32,
         bias ? bs.data() : nullptr, bias ? BiasKind::fp32 : BiasKind::none, full, act == 0 ? N : 0, tight, act == 0 ? 0 : I, K);
      m += MR;
    }
  }
  free(slab);
  return 0;
}

// The group bf16 micro-kernel over A bf16 [M,K] x B bf16 [K,N] (row-major, caller's column order: [gate | up] halves for
// act 2 and 3, element-interleaved pairs for act 1), f32 bias [N] or null.  B is packed here as the kernel reads it:
// 32-column slabs, K-pair-major, element (k, c) at ((k/2)*32 + c)*2 + k%2; the gated forms that take split halves get their
// columns interleaved by the pack, as the reference's prepack does.  act: 0 none, 1 swiglu_oai_mul, 2 silu_and_mul,
// 3 gelu_and_mul.  K % 2 == 0, N % 32 == 0.  out: bf16 bits, [M,N] for act 0, else [M,N/2].
API int ref2_bf16_ukernel(const uint16_t *A, const uint16_t *B, int M, int N, int K, const float *bias, int act, uint16_t *out) {
  using namespace zendnnl::lowoha::matmul::custom_kernel;
  using zendnnl::common::bfloat16_t;
  if (!avx512bf16_available() || K % 2 != 0 || N % 32 != 0 || M <= 0) return -1;
  const int NR = 32, I = N / 2, kp = K / 2;
  auto src_col = [&](int p) { return (act == 2 || act == 3) ? ((p & 1) ? I + p / 2 : p / 2) : p; };
  uint16_t *slab = static_cast<uint16_t *>(aligned_alloc(64, ((size_t)kp * NR * 2 * 2 + 63) / 64 * 64));
  std::vector<float> bs(NR);
  for (int ob = 0; ob < N / NR; ++ob) {
    for (int c = 0; c < NR; ++c) {
      const int sc = src_col(ob * NR + c);
      for (int k = 0; k < K; ++k) slab[((size_t)(k / 2) * NR + c) * 2 + (k % 2)] = B[(size_t)k * N + sc];
      bs[c] = bias ? bias[sc] : 0.f;
    }
    for (int m = 0; m < M;) {
      const int MR = M - m >= 8 ? 8 : M - m;
      ukernel_fn_t fn = select_ukernel(MR, 2, static_cast<ActKind>(act), DstDt::kBf16);
      if (!fn) { free(slab); return -2; }
      void *full = act == 0 ? out + (size_t)m * N + ob * NR : nullptr;
      void *tight = act == 0 ? nullptr : out + (size_t)m * I + ob * (NR / 2);
      fn(reinterpret_cast<const bfloat16_t *>(A) + (size_t)m * K, K, reinterpret_cast<const bfloat16_t *>(slab),
         bias ? bs.data() : nullptr, bias ? BiasKind::fp32 : BiasKind::none, full, act == 0 ? N : 0, tight, act == 0 ? 0 : I, K);
      m += MR;
    }
  }
  free(slab);
  return 0;
}

// The reference's scalar normalization kernel.  Same argument list as the oracle's orc_normalization; dtype codes are
// data_type_t values.  type: 0 layer, 1 batch, 2 rms, 3 fused-add rms.
API int ref2_normalization(int type, const void *x, void *y, const void *gamma, const void *beta, const float *run_mean,
                           const float *run_var, void *residual, int64_t batch, int64_t n, int64_t channels, float eps,
                           int use_scale, int use_shift, int src_dt, int dst_dt, int gamma_dt, int beta_dt) {
  using namespace zendnnl::lowoha::normalization;
  using zendnnl::common::data_type_t;
  norm_params p;
  p.norm_type = static_cast<norm_type_t>(type);
  p.batch = (uint64_t)batch; p.norm_size = (uint64_t)n; p.num_channels = (uint64_t)channels;
  p.epsilon = eps; p.use_scale = use_scale != 0; p.use_shift = use_shift != 0;
  p.src_dt = static_cast<data_type_t>(src_dt); p.dst_dt = static_cast<data_type_t>(dst_dt);
  p.gamma_dt = static_cast<data_type_t>(gamma_dt); p.beta_dt = static_cast<data_type_t>(beta_dt);
  p.num_threads = 1;
  return normalization_reference_wrapper(x, y, gamma, beta, run_mean, run_var, residual, p) == zendnnl::error_handling::status_t::success ? 0 : -1;
}
