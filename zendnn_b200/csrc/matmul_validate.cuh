// Contract checks of the INT8 matmul_direct path, shared by b200dnn_matmul and b200dnn_matmul_static_scratch.
// They restate the INT8 rules of the reference's validator (matmul/lowoha_matmul_utils.cpp:180-420) for the
// supported subset; everything outside it is reported as unimplemented, never computed differently.
// ZENDNNL_DIAGNOSTICS_ENABLE=0 switches the rich contract checks off as in the reference
// (common/operator_instrumentation.hpp:49-66); the memory-safety guards and the unimplemented-feature checks stay.
#pragma once
#include <cmath>
#include <cstdlib>
#include "runtime.cuh"
#include "common.cuh"

namespace b200 {

inline bool diagnostics_enabled() {
  static const bool dynamic = [] { const char *e = getenv("B200DNN_ENV_DYNAMIC"); return e && atoi(e) != 0; }();
  static const bool cached = [] { const char *e = getenv("ZENDNNL_DIAGNOSTICS_ENABLE"); return !e || atoi(e) != 0; }();
  if (!dynamic) return cached;
  const char *e = getenv("ZENDNNL_DIAGNOSTICS_ENABLE");
  return !e || atoi(e) != 0;
}

inline int32_t validate_matmul_desc(const b200dnn_matmul_t *d) {
  const int M = d->M, N = d->N, K = d->K;
  const bool diag = diagnostics_enabled();
  // ---- always-on guards
  B2_CHECK(d->src && d->weight && d->dst, B200DNN_FAILURE, "null src, weight or dst");
  B2_CHECK(M > 0 && N > 0 && K > 0, B200DNN_FAILURE, "M, N, K must be positive (got %d, %d, %d)", M, N, K);
  B2_CHECK(d->lda >= K && d->ldc >= N, B200DNN_FAILURE, "lda/ldc smaller than the row length");
  B2_CHECK(d->wei_format == 'r' || d->ldb >= (d->transB ? K : N), B200DNN_FAILURE, "ldb smaller than the row length");
  B2_CHECK(d->wei_dt == B200DNN_S8, B200DNN_UNIMPLEMENTED, "only s8 weights are implemented (wei dtype %d)", d->wei_dt);
  const bool int_dst = d->dst_dt == B200DNN_S8 || d->dst_dt == B200DNN_U8;
  B2_CHECK(d->dst_dt == B200DNN_BF16 || d->dst_dt == B200DNN_F32 || d->dst_dt == B200DNN_S32 || int_dst, B200DNN_UNIMPLEMENTED,
           "dst dtype %d is not implemented for the INT8 path", d->dst_dt);
  if (int_dst) {
    // requantised destination: per-tensor scale (matmul/lowoha_matmul_utils.cpp:307-309), optional per-tensor zero point
    // (without a scale the result is clamped and rounded as it is)
    B2_CHECK(!d->dst_scale.buff || d->dst_scale.count == 1, B200DNN_FAILURE, "Destination quant scale supports only per-tensor");
    B2_CHECK(!d->dst_scale.buff || d->dst_scale.dt == B200DNN_F32, B200DNN_UNIMPLEMENTED, "dst_scale must be f32");
    B2_CHECK(d->dst_scale.buff || !d->dst_zp.buff, B200DNN_UNIMPLEMENTED, "a destination zero point needs a destination scale");
    B2_CHECK(!d->dst_zp.buff || (d->dst_zp.count == 1 && d->dst_zp.dt == B200DNN_S32), B200DNN_UNIMPLEMENTED, "dst zero point must be one s32 value");
  }
  B2_CHECK(d->n_postops >= 0 && d->n_postops <= B200DNN_MAX_POSTOPS, B200DNN_FAILURE, "too many post-ops");
  const bool dyn = d->dynamic_quant != 0;
  if (dyn) {
    B2_CHECK(d->src_dt == B200DNN_BF16 || d->src_dt == B200DNN_F32, B200DNN_UNIMPLEMENTED, "dynamic quantisation takes a bf16 or f32 source");
    B2_CHECK(d->src_scale.count == M || (M == 1 && d->src_scale.count == 1) || d->src_scale.count == 0, B200DNN_UNIMPLEMENTED,
             "dynamic quantisation is per-token only (src scale count %lld, M %d)", (long long)d->src_scale.count, M);
    B2_CHECK(d->src_zp.buff == nullptr, B200DNN_UNIMPLEMENTED, "asymmetric dynamic quantisation is not implemented");
  } else {
    B2_CHECK(d->src_dt == B200DNN_S8 || d->src_dt == B200DNN_U8, B200DNN_UNIMPLEMENTED, "src dtype %d without dynamic_quant", d->src_dt);
    B2_CHECK(d->src_scale.count == 0 || d->src_scale.buff, B200DNN_FAILURE, "src scale buffer is null");
    B2_CHECK(d->src_scale.count == 0 || d->src_scale.count == 1 || d->src_scale.count == M, B200DNN_UNIMPLEMENTED,
             "src scale must be per-tensor or per-token");
  }
  const bool per_token = d->src_scale.count > 1 || (dyn && M > 1);
  if (per_token && diag) {
    // per-token rules: symmetric source, float destination, per-channel weight scale of N elements
    // (matmul/lowoha_matmul_utils.cpp:252-292)
    B2_CHECK(d->src_zp.buff == nullptr, B200DNN_FAILURE, "per-token source scale does not allow a zero-point");
    B2_CHECK(dyn || d->src_dt == B200DNN_S8, B200DNN_FAILURE, "per-token source scale needs a symmetric s8 source");
    B2_CHECK(d->dst_dt != B200DNN_S32, B200DNN_FAILURE, "per-token source scale needs an f32 or bf16 destination");
    B2_CHECK(d->wei_scale.count == N, B200DNN_FAILURE, "per-token source scale needs a per-channel weight scale of N elements");
  }
  B2_CHECK(d->wei_scale.count == 0 || d->wei_scale.count == 1 || d->wei_scale.count == N, B200DNN_UNIMPLEMENTED,
           "weight scale must be per-tensor or per-channel");
  B2_CHECK(d->wei_scale.count == 0 || d->wei_scale.buff, B200DNN_FAILURE, "weight scale buffer is null");
  B2_CHECK(d->src_zp.buff == nullptr || d->src_zp.count <= 1, B200DNN_UNIMPLEMENTED, "src zero-point must be per-tensor");
  auto scale_dt_ok = [](int32_t dt) { return dt == B200DNN_F32 || dt == B200DNN_BF16; };
  B2_CHECK(d->src_scale.count == 0 || !d->src_scale.buff || scale_dt_ok(d->src_scale.dt), B200DNN_UNIMPLEMENTED, "src scale dtype");
  B2_CHECK(d->wei_scale.count == 0 || scale_dt_ok(d->wei_scale.dt), B200DNN_UNIMPLEMENTED, "weight scale dtype");
  B2_CHECK(!d->bias || scale_dt_ok(d->bias_dt), B200DNN_UNIMPLEMENTED, "bias dtype %d", d->bias_dt);
  if (d->dst_dt == B200DNN_S32)
    B2_CHECK(d->src_scale.count == 0 && d->wei_scale.count == 0 && !d->bias && d->n_postops == 0, B200DNN_UNIMPLEMENTED,
             "s32 destination returns raw compensated accumulators: no scales, bias or post-ops");
  for (int i = 0; i < d->n_postops; ++i) {
    const b200dnn_postop_t &p = d->postops[i];
    switch (p.type) {
    case PO_RELU: case PO_LEAKY_RELU: case PO_GELU_TANH: case PO_GELU_ERF: case PO_SIGMOID: case PO_SWISH: case PO_TANH: case PO_ELU: break;
    case PO_CLIP: B2_CHECK(!diag || (std::isfinite(p.alpha) && std::isfinite(p.beta)), B200DNN_FAILURE, "clip bounds must be finite"); break;
    case PO_BINARY_ADD: case PO_BINARY_MUL:
      B2_CHECK(p.buff && (p.dt == B200DNN_F32 || p.dt == B200DNN_BF16), B200DNN_FAILURE, "binary post-op needs an f32 or bf16 operand");
      B2_CHECK(p.ld == 0 || p.ld >= N, B200DNN_FAILURE, "binary post-op leading dimension");
      break;
    case PO_MISH: return fail(B200DNN_FAILURE, "mish is rejected on the INT8 path");
    default: return fail(B200DNN_UNIMPLEMENTED, "post-op %d is not implemented", p.type);
    }
  }

  if (d->src_zp.buff)
    B2_CHECK(d->src_zp.dt == B200DNN_S32 || d->src_zp.dt == B200DNN_S8 || d->src_zp.dt == B200DNN_U8, B200DNN_UNIMPLEMENTED, "src zero-point dtype");
  return B200DNN_SUCCESS;
}

}  // namespace b200
