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
#include <cstdint>
#include <vector>

#include "lowoha_operators/matmul/group_matmul/group_matmul_direct.hpp"

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
