// C++ shims with the reference's LowOHA signatures (include/zendnnl_b200/lowoha.hpp) over the C ABI
// of libb200dnn.  Each function flattens the reference's parameter structs into the plain
// descriptors of b200dnn.h; all arithmetic happens in the CUDA library.  What the reference does
// at this level and is kept: argument checks that need the C++ containers, the active/total
// expert contract, the choice between fused-MoE and plain grouped execution.
//
// Reference entry points: lowoha_operators/matmul/lowoha_matmul.cpp:278 (matmul_direct),
// lowoha_operators/matmul/group_matmul_direct.cpp:747 (group_matmul_direct),
// lowoha_operators/reorder/lowoha_reorder.cpp:43,279 (reorder_direct, group_dynamic_quant),
// lowoha_operators/reorder/prepack/lowoha_prepack.cpp:285,315 (weight_prepack_size / _into).
#include "zendnnl_b200/lowoha.hpp"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <sstream>

#include "b200dnn.h"

namespace zendnnl {
namespace lowoha {

namespace {
using zendnnl::common::data_type_t;
using zendnnl::error_handling::status_t;

thread_local std::string g_shim_error;
thread_local void *g_stream = nullptr;   // the calling thread's CUDA stream (b200::set_stream)

status_t shim_fail(status_t s, const char *msg) { g_shim_error = msg; return s; }
status_t from_c(int32_t rc) {
  if (rc != B200DNN_SUCCESS) g_shim_error = b200dnn_last_error();
  return static_cast<status_t>(rc);
}
int64_t nelem(const std::vector<int64_t> &d) {
  if (d.empty()) return 0;
  int64_t n = 1;
  for (auto v : d) n *= v;
  return n;
}
template <class Q> b200dnn_quant_t flat_quant(const Q &q) {
  b200dnn_quant_t o{};
  o.buff = q.buff; o.dt = static_cast<int32_t>(q.dt);
  const int64_t n = nelem(q.dims);
  o.count = n > 0 ? n : (q.buff ? 1 : 0);
  return o;
}

// The reference's log knobs (common/config_manager.cpp:273-330, levels common/logging_support.hpp:31-38):
// ZENDNNL_API_LOG_LEVEL >= 3 (or "info" / "verbose") prints one line per call, ZENDNNL_ENABLE_PROFILER=1 with
// ZENDNNL_PROFILE_LOG_LEVEL >= 4 (or "verbose") adds the call's host time.  Read once.
int env_level(const char *name) {
  const char *e = std::getenv(name);
  if (!e || !*e) return 0;
  if (!std::strcmp(e, "error")) return 1;
  if (!std::strcmp(e, "warning")) return 2;
  if (!std::strcmp(e, "info")) return 3;
  if (!std::strcmp(e, "verbose")) return 4;
  return std::atoi(e);
}
bool apilog_info() { static const bool v = env_level("ZENDNNL_API_LOG_LEVEL") >= 3; return v; }
bool profile_on() {
  static const bool v = [] { const char *e = std::getenv("ZENDNNL_ENABLE_PROFILER"); return e && std::atoi(e) != 0 && env_level("ZENDNNL_PROFILE_LOG_LEVEL") >= 4; }();
  return v;
}
const char *dt_name(data_type_t d) {
  switch (d) {
  case data_type_t::f32: return "f32"; case data_type_t::bf16: return "bf16"; case data_type_t::s32: return "s32";
  case data_type_t::s8: return "s8"; case data_type_t::u8: return "u8"; case data_type_t::s4: return "s4";
  case data_type_t::u4: return "u4"; case data_type_t::f16: return "f16"; case data_type_t::none: return "none";
  default: return "other";
  }
}
struct CallTimer {
  std::chrono::steady_clock::time_point t0 = std::chrono::steady_clock::now();
  double ms() const { return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count(); }
};
// one line in the shape of the reference's (lowoha_operators/matmul/lowoha_matmul.cpp:472-506)
void log_call(const std::string &text, status_t st, const CallTimer &t, const void *weight = nullptr) {
  if (apilog_info()) std::fprintf(stderr, "[ZENDNNL API INFO] %s, kernel=b200dnn, status=%d\n", text.c_str(), static_cast<int>(st));
  if (profile_on()) std::fprintf(stderr, "[ZENDNNL PROFILE] %s, kernel=b200dnn, weight_address=%p, time=%.4f ms (host time of the call; device-pointer calls only enqueue)\n", text.c_str(), weight, t.ms());
}
}  // namespace

namespace b200 {
void set_stream(void *cuda_stream) { g_stream = cuda_stream; }
void *get_stream() { return g_stream; }
}  // namespace b200

// =========================================================================================== matmul
namespace matmul {

const char *last_error() { return g_shim_error.c_str(); }

namespace {
// Flattens one matmul_direct call.  Returns success when `d` is filled, otherwise the status to return.
status_t flatten(const char layout, const bool transA, const bool transB, const int M, const int N, const int K,
                 const float alpha, const void *src, const int lda, const void *weight, const int ldb, const void *bias,
                 const float beta, void *dst, const int ldc, const bool is_weights_const,
                 const matmul_batch_params_t &bp, const matmul_params &p, b200dnn_matmul_t *d) {
  if (layout != 'r' && layout != 'R') return shim_fail(status_t::unimplemented, "only row-major layout is implemented");
  if (bp.Batch_A != 1 || bp.Batch_B != 1) return shim_fail(status_t::unimplemented, "batched matmul is not implemented");
  if (alpha != 1.0f || beta != 0.0f) return shim_fail(status_t::unimplemented, "only alpha = 1, beta = 0 is implemented");
  if (p.packing.pack_format_b != 0) return shim_fail(status_t::unimplemented, "GGML-packed weights are not implemented");
  const bool int_dst = p.dtypes.dst == data_type_t::s8 || p.dtypes.dst == data_type_t::u8;
  if (!int_dst && (p.quant_params.dst_scale.buff || p.quant_params.dst_zp.buff))
    return shim_fail(status_t::unimplemented, "a destination scale or zero point is implemented for s8/u8 destinations only");
  const bool woq_u4 = p.dtypes.wei == data_type_t::u4 && p.dtypes.src == data_type_t::bf16 && !p.dynamic_quant;
  if (p.quant_params.wei_zp.buff && !woq_u4)
    return shim_fail(status_t::unimplemented, "weight zero-points are implemented for u4 weight-only quantisation");
  if (p.postop_.size() > B200DNN_MAX_POSTOPS) return shim_fail(status_t::failure, "too many post-ops");
  // W4A8 (s4 weights, bf16 source quantised by the library): the reference wants s8 compute and 2-D scale dims
  // (lowoha_matmul_utils.cpp:101-145); the remaining rules are checked behind the C ABI
  if (p.dynamic_quant && p.dtypes.wei == data_type_t::s4 && p.dtypes.src == data_type_t::bf16) {
    if (p.dtypes.compute != data_type_t::s8) return shim_fail(status_t::failure, "W4A8 dynamic quantization requires s8 compute");
    if (p.quant_params.wei_scale.dims.size() != 2) return shim_fail(status_t::failure, "W4A8 requires weight scale dims {G,N}");
    if (p.quant_params.src_scale.dims.size() != 2) return shim_fail(status_t::failure, "W4A8 requires source scale dims {1,1}, {M,1}, or {M,G}");
  }
  std::memset(d, 0, sizeof *d);
  d->M = M; d->N = N; d->K = K; d->transB = transB ? 1 : 0; d->transA = transA ? 1 : 0;
  d->src_dt = static_cast<int32_t>(p.dtypes.src); d->wei_dt = static_cast<int32_t>(p.dtypes.wei);
  d->dst_dt = static_cast<int32_t>(p.dtypes.dst); d->bias_dt = static_cast<int32_t>(p.dtypes.bias);
  d->lda = lda; d->ldb = ldb; d->ldc = ldc;
  d->src = src; d->weight = weight; d->bias = bias; d->dst = dst;
  d->wei_format = p.mem_format_b;
  d->weights_const = (is_weights_const && p.weight_cache_type != 0) ? 1 : 0;
  d->dynamic_quant = p.dynamic_quant ? 1 : 0;
  d->src_scale = flat_quant(p.quant_params.src_scale);
  d->wei_scale = flat_quant(p.quant_params.wei_scale);
  d->src_zp = flat_quant(p.quant_params.src_zp);
  if (!p.quant_params.src_zp.buff) d->src_zp.count = 0;
  if (woq_u4) d->wei_zp = flat_quant(p.quant_params.wei_zp);
  if (int_dst) {
    d->dst_scale = flat_quant(p.quant_params.dst_scale);
    d->dst_zp = flat_quant(p.quant_params.dst_zp);
    if (!p.quant_params.dst_zp.buff) d->dst_zp.count = 0;
  }
  d->n_postops = static_cast<int32_t>(p.postop_.size());
  for (int i = 0; i < d->n_postops; ++i) {
    const matmul_post_op &po = p.postop_[i];
    b200dnn_postop_t &o = d->postops[i];
    o.type = static_cast<int32_t>(po.po_type); o.dt = static_cast<int32_t>(po.dtype); o.buff = po.buff;
    o.alpha = po.alpha; o.beta = po.beta;
    const bool row_broadcast = po.dims.size() == 2 && po.dims[0] == 1;
    const bool vec_broadcast = po.dims.size() == 1;
    o.ld = (row_broadcast || vec_broadcast) ? 0 : (po.leading_dim > 0 ? po.leading_dim : N);   // default leading dim N
    if (po.po_type == zendnnl::ops::post_op_type_t::clip && o.alpha > o.beta) std::swap(o.alpha, o.beta);
  }
  return status_t::success;
}
}  // namespace

status_t matmul_direct(const char layout, const bool transA, const bool transB, const int M, const int N, const int K,
                       const float alpha, const void *src, const int lda, const void *weight, const int ldb,
                       const void *bias, const float beta, void *dst, const int ldc, const bool is_weights_const,
                       const matmul_batch_params_t &batch_params, const matmul_params &params) {
  b200dnn_matmul_t d;
  const CallTimer timer;
  status_t st = flatten(layout, transA, transB, M, N, K, alpha, src, lda, weight, ldb, bias, beta, dst, ldc, is_weights_const,
                        batch_params, params, &d);
  if (st == status_t::success) st = from_c(b200dnn_matmul(&d, g_stream));
  if (apilog_info() || profile_on()) {
    std::ostringstream ss;
    ss << "LOWOHA matmul_direct: M=" << M << ", N=" << N << ", K=" << K << ", alpha=" << alpha << ", beta=" << beta << ", lda=" << lda
       << ", ldb=" << ldb << ", ldc=" << ldc << ", transA=" << (transA ? "true" : "false") << ", transB=" << (transB ? "true" : "false")
       << ", input_dtype=" << dt_name(params.dtypes.src) << ", weight_dtype=" << dt_name(params.dtypes.wei)
       << ", output_dtype=" << dt_name(params.dtypes.dst) << ", bias_dtype=" << dt_name(params.dtypes.bias)
       << ", bias=" << (bias ? "true" : "false") << ", is_weights_const=" << (is_weights_const ? "true" : "false")
       << ", post_ops=" << params.postop_.size() << ", Batch_A=" << batch_params.Batch_A << ", Batch_B=" << batch_params.Batch_B
       << ", plugin_op=" << params.plugin_op << ", dynamic_quant=" << (params.dynamic_quant ? "true" : "false");
    log_call(ss.str(), st, timer, weight);
  }
  return st;
}

status_t group_matmul_moe_act_execute(const grp_matmul_gated_act_params *act_params, const std::vector<void *> &dst,
                                      const std::vector<int> &M, const std::vector<int> &N, const std::vector<int> &ldc,
                                      data_type_t dst_dtype, int /*num_threads*/) {
  if (!act_params || act_params->act == grp_matmul_gated_act_t::none) return status_t::success;
  if (dst.size() != M.size() || N.size() != M.size() || ldc.size() != M.size())
    return shim_fail(status_t::failure, "gated activation: vector sizes differ");
  for (size_t i = 0; i < M.size(); ++i) {
    if (M[i] <= 0) continue;
    if (!dst[i]) return shim_fail(status_t::failure, "gated activation: null dst");
    status_t st = from_c(b200dnn_gated_act(dst[i], static_cast<int32_t>(dst_dtype), M[i], N[i], ldc[i],
                                           static_cast<int32_t>(act_params->act), g_stream));
    if (st != status_t::success) return st;
  }
  return status_t::success;
}

status_t group_matmul_moe_postop_execute(const group_matmul_moe_postop_params *p, int D, int /*num_threads*/,
                                         data_type_t dst_elem) {
  if (!p) return status_t::success;
  if (p->num_tokens <= 0 || p->topk <= 0 || !p->output || !p->row_ptrs || D <= 0 || p->ldc_output < D)
    return shim_fail(status_t::failure, "moe post-op: bad argument");
  if (!p->skip_weighted && !p->topk_weights) return shim_fail(status_t::failure, "moe post-op: topk_weights is null");
  return from_c(b200dnn_moe_weighted_reduce(p->row_ptrs, p->topk_weights, p->num_tokens, p->topk, D, p->skip_weighted ? 1 : 0,
                                            static_cast<int32_t>(dst_elem), p->output, p->ldc_output, g_stream));
}

void clear_fused_moe_scratch() { b200dnn_clear_caches(); }

static status_t group_matmul_impl(const std::vector<char> &layout, const std::vector<bool> &transA, const std::vector<bool> &transB,
                             const std::vector<int> &M, const std::vector<int> &N, const std::vector<int> &K,
                             const std::vector<float> &alpha, const std::vector<const void *> &src, const std::vector<int> &lda,
                             const std::vector<const void *> &weight, const std::vector<int> &ldb,
                             const std::vector<const void *> &bias, const std::vector<float> &beta,
                             const std::vector<void *> &dst, const std::vector<int> &ldc,
                             const std::vector<bool> &is_weights_const, const std::vector<matmul_params> &params,
                             const group_matmul_moe_postop_params *moe_postop, const grp_matmul_gated_act_params *gated_act,
                             const grp_matmul_fused_moe_params *fused) {
  // always-on guards (group_matmul_direct.cpp:812-1063): non-empty, consistent vector lengths
  if (M.empty() || params.empty()) return shim_fail(status_t::failure, "group_matmul_direct: empty M or params");
  // active/total contract: only params[0] is read; compute the leading `active` experts (lowoha_common.hpp:169-214)
  size_t num_ops = M.size();
  if (params[0].active_matmul > 0) {
    if (params[0].total_matmul > 0 && params[0].active_matmul > params[0].total_matmul)
      return shim_fail(status_t::failure, "group_matmul_direct: active_matmul > total_matmul");
    num_ops = std::min<size_t>(params[0].active_matmul, M.size());
  }
  auto at_least = [&](size_t n) { return n >= num_ops; };
  if (!at_least(layout.size()) || !at_least(transA.size()) || !at_least(transB.size()) || !at_least(N.size()) ||
      !at_least(K.size()) || !at_least(alpha.size()) || !at_least(lda.size()) || !at_least(weight.size()) ||
      !at_least(ldb.size()) || !at_least(bias.size()) || !at_least(beta.size()) || !at_least(ldc.size()) ||
      !at_least(is_weights_const.size()) || !at_least(params.size()))
    return shim_fail(status_t::failure, "group_matmul_direct: a per-expert vector is shorter than the number of operations");
  const grp_matmul_gated_act_t act = gated_act ? gated_act->act : grp_matmul_gated_act_t::none;
  if (src.size() == 1 && num_ops > 1) {
    // ---- sequential chain (group_matmul_direct.cpp:424-456 rules, :1138-1163 dispatch): layer i + 1 reads layer i's
    // destination with its leading dimension; M is constant and K[i] == N[i-1]
    if (moe_postop) return shim_fail(status_t::failure, "group_matmul_direct: moe_postop is only supported in parallel mode (src.size() == num_ops)");
    if (act != grp_matmul_gated_act_t::none) return shim_fail(status_t::failure, "group_matmul_direct: gated_act is only supported in parallel mode (src.size() == num_ops)");
    if (fused) return shim_fail(status_t::failure, "group_matmul_direct: fused_moe is only supported in parallel mode (src.size() == num_ops)");
    if (!at_least(dst.size())) return shim_fail(status_t::failure, "group_matmul_direct: dst vector too short");
    if (!src[0]) return shim_fail(status_t::failure, "group_matmul sequential: null src pointer");
    for (size_t i = 0; i < num_ops; ++i) {
      if (!weight[i] || !dst[i]) return shim_fail(status_t::failure, "group_matmul sequential: null pointer at an operation");
      if (M[i] <= 0 || N[i] <= 0 || K[i] <= 0) return shim_fail(status_t::failure, "group_matmul sequential: invalid dimensions at an operation");
      if (i && M[i] != M[0]) return shim_fail(status_t::failure, "group_matmul sequential: M must be constant across layers");
      if (i && K[i] != N[i - 1]) return shim_fail(status_t::failure, "group_matmul sequential: dimension mismatch between layers (K[i] != N[i-1])");
    }
    const matmul_batch_params_t bp;
    for (size_t i = 0; i < num_ops; ++i) {
      b200dnn_matmul_t d;
      status_t st = flatten(layout[i], transA[i], transB[i], M[i], N[i], K[i], alpha[i], i ? dst[i - 1] : src[0], i ? ldc[i - 1] : lda[0],
                            weight[i], ldb[i], bias[i], beta[i], dst[i], ldc[i], is_weights_const[i], bp, params[i], &d);
      if (st == status_t::success) st = from_c(b200dnn_matmul(&d, g_stream));
      if (st != status_t::success) return st;
    }
    return status_t::success;
  }
  if (!at_least(src.size())) return shim_fail(status_t::failure, "group_matmul_direct: src vector too short");

  if (fused) {
    // ---- fused MoE: Op1 (gate|up) -> gated activation -> per-token requantisation -> Op2 (down) [-> weighted reduce]
    if (act == grp_matmul_gated_act_t::none) return shim_fail(status_t::failure, "fused MoE needs a gated activation");
    const bool wants_scales = !params.empty() && params[0].dtypes.wei == data_type_t::s8;
    if (fused->down_weight.size() < num_ops || fused->N_down.size() < num_ops || fused->ldb_down.size() < num_ops ||
        (wants_scales && fused->down_scale.size() < num_ops))
      return shim_fail(status_t::failure, "fused MoE: down-projection vectors are shorter than the number of experts");
    // mode (1): caller-allocated dst_down; mode (2), dst_down empty: the result is written back into src[]
    // (group_matmul_direct.hpp:500-566: matched src/dst precision and lda >= N_down are preconditions)
    const bool reuse_src = fused->dst_down.empty();
    if (!reuse_src && (fused->dst_down.size() < num_ops || fused->ldc_down.size() < num_ops))
      return shim_fail(status_t::failure, "fused MoE: dst_down / ldc_down are shorter than the number of experts");
    bool any_bias_down = false;
    for (size_t i = 0; i < num_ops && i < fused->bias_down.size(); ++i) any_bias_down |= fused->bias_down[i] != nullptr;
    if (any_bias_down && fused->bias_dt_down == data_type_t::none)
      return shim_fail(status_t::failure, "fused MoE: bias_down given without bias_dt_down");
    const matmul_params &p0 = params[0];
    const bool moe_int8 = p0.dynamic_quant && p0.dtypes.src == data_type_t::bf16 && p0.dtypes.wei == data_type_t::s8 &&
                          p0.dtypes.dst == data_type_t::bf16;
    const bool moe_bf16 = !p0.dynamic_quant && p0.dtypes.src == data_type_t::bf16 && p0.dtypes.wei == data_type_t::bf16 &&
                          p0.dtypes.dst == data_type_t::bf16;
    if (!moe_int8 && !moe_bf16)
      return shim_fail(status_t::unimplemented,
                       "fused MoE is implemented for dynamic per-token INT8 (bf16 src, s8 weights, bf16 dst) and for bf16:bf16:bf16");
    std::vector<b200dnn_moe_expert_t> ex(num_ops);
    for (size_t i = 0; i < num_ops; ++i) {
      if (N[i] != N[0] || K[i] != K[0] || fused->N_down[i] != fused->N_down[0] || transB[i] != transB[0])
        return shim_fail(status_t::unimplemented, "fused MoE: experts must share K, N, N_down and transB");
      if (layout[i] != 'r' && layout[i] != 'R') return shim_fail(status_t::failure, "fused MoE requires row-major layout");
      if (transA[i] || alpha[i] != 1.0f || beta[i] != 0.0f) return shim_fail(status_t::unimplemented, "fused MoE: transA / alpha / beta");
      if (reuse_src && lda[i] < fused->N_down[i]) return shim_fail(status_t::failure, "fused MoE: src-reuse mode needs lda >= N_down");
      const auto &ws = params[i].quant_params.wei_scale;
      if (moe_int8 && (!ws.buff || ws.dt != data_type_t::f32 || nelem(ws.dims) != N[i]))
        return shim_fail(status_t::failure, "fused MoE: per-channel f32 weight scale of N elements required");
      static const grp_matmul_fused_moe_params::down_weight_quant_t no_scale{};
      const auto &ds = moe_int8 ? fused->down_scale[i] : no_scale;
      if (moe_int8 && (!ds.buff || ds.dt != data_type_t::f32 || nelem(ds.dims) != fused->N_down[i]))
        return shim_fail(status_t::failure, "fused MoE: per-channel f32 down_scale of N_down elements required");
      b200dnn_moe_expert_t &e = ex[i];
      std::memset(&e, 0, sizeof e);
      e.M = M[i]; e.src = src[i]; e.lda = lda[i];
      e.wei_dt = moe_bf16 ? B200DNN_BF16 : B200DNN_S8;
      e.w13 = weight[i]; e.ldb13 = ldb[i]; e.w13_scale = moe_int8 ? static_cast<const float *>(ws.buff) : nullptr;
      e.w2 = fused->down_weight[i]; e.ldb2 = fused->ldb_down[i]; e.w2_scale = moe_int8 ? static_cast<const float *>(ds.buff) : nullptr;
      if (!reuse_src) { e.dst_down = fused->dst_down[i]; e.ldc_down = fused->ldc_down[i]; }
      e.bias13 = bias[i]; e.bias13_dt = static_cast<int32_t>(params[i].dtypes.bias);
      if (i < fused->bias_down.size()) { e.bias2 = fused->bias_down[i]; e.bias2_dt = static_cast<int32_t>(fused->bias_dt_down); }
      // mode (1): the activated output of the first GEMM stays visible in the caller's dst[] (group_matmul_direct.hpp:489-497)
      if (!reuse_src && i < dst.size() && dst[i] && i < ldc.size()) { e.dst_op1 = dst[i]; e.ldc_op1 = ldc[i]; }
    }
    const bool wconst = is_weights_const[0] && p0.weight_cache_type != 0;
    return from_c(b200dnn_fused_moe(static_cast<int32_t>(num_ops), ex.data(), K[0], N[0] / 2, fused->N_down[0], transB[0] ? 1 : 0,
                                    static_cast<int32_t>(act), wconst ? 1 : 0,
                                    moe_postop ? reinterpret_cast<const void *const *>(moe_postop->row_ptrs) : nullptr,
                                    moe_postop ? moe_postop->topk_weights : nullptr, moe_postop ? moe_postop->num_tokens : 0,
                                    moe_postop ? moe_postop->topk : 0, moe_postop ? moe_postop->output : nullptr,
                                    moe_postop ? moe_postop->ldc_output : 0, g_stream));
  }

  // ---- plain grouped mode: every expert's GEMM, experts with M == 0 skipped (group_matmul_parallel_common.hpp:1240-1248)
  if (!at_least(dst.size())) return shim_fail(status_t::failure, "group_matmul_direct: dst vector too short");
  // one C call for the whole group: experts of one shape share a grouped launch, the rest run one by one
  {
    const matmul_batch_params_t bp;
    std::vector<b200dnn_matmul_t> descs(num_ops);
    for (size_t i = 0; i < num_ops; ++i) {
      if (M[i] == 0) { std::memset(&descs[i], 0, sizeof descs[i]); continue; }
      status_t st = flatten(layout[i], transA[i], transB[i], M[i], N[i], K[i], alpha[i], src[i], lda[i], weight[i], ldb[i], bias[i],
                            beta[i], dst[i], ldc[i], is_weights_const[i], bp, params[i], &descs[i]);
      if (st != status_t::success) return st;
    }
    status_t st = from_c(b200dnn_group_matmul(static_cast<int32_t>(num_ops), descs.data(), g_stream));
    if (st != status_t::success) return st;
  }
  if (act != grp_matmul_gated_act_t::none) {
    std::vector<void *> d(dst.begin(), dst.begin() + num_ops);
    std::vector<int> m(M.begin(), M.begin() + num_ops), n(N.begin(), N.begin() + num_ops), l(ldc.begin(), ldc.begin() + num_ops);
    status_t st = group_matmul_moe_act_execute(gated_act, d, m, n, l, params[0].dtypes.dst, 0);
    if (st != status_t::success) return st;
  }
  if (moe_postop) {
    const int D = act != grp_matmul_gated_act_t::none ? N[0] / 2 : N[0];
    return group_matmul_moe_postop_execute(moe_postop, D, 0, params[0].dtypes.dst);
  }
  return status_t::success;
}

status_t group_matmul_direct(const std::vector<char> &layout, const std::vector<bool> &transA, const std::vector<bool> &transB,
                             const std::vector<int> &M, const std::vector<int> &N, const std::vector<int> &K,
                             const std::vector<float> &alpha, const std::vector<const void *> &src, const std::vector<int> &lda,
                             const std::vector<const void *> &weight, const std::vector<int> &ldb,
                             const std::vector<const void *> &bias, const std::vector<float> &beta,
                             const std::vector<void *> &dst, const std::vector<int> &ldc,
                             const std::vector<bool> &is_weights_const, const std::vector<matmul_params> &params,
                             const group_matmul_moe_postop_params *moe_postop, const grp_matmul_gated_act_params *gated_act,
                             const grp_matmul_fused_moe_params *fused) {
  const CallTimer timer;
  const status_t st = group_matmul_impl(layout, transA, transB, M, N, K, alpha, src, lda, weight, ldb, bias, beta, dst, ldc, is_weights_const,
                                        params, moe_postop, gated_act, fused);
  if (apilog_info() || profile_on()) {
    long rows = 0;
    for (int m : M) rows += m;
    std::ostringstream ss;
    ss << "LOWOHA group_matmul_direct: num_ops=" << M.size() << ", total_M=" << rows << ", N=" << (N.empty() ? 0 : N[0])
       << ", K=" << (K.empty() ? 0 : K[0]) << ", input_dtype=" << (params.empty() ? "none" : dt_name(params[0].dtypes.src))
       << ", weight_dtype=" << (params.empty() ? "none" : dt_name(params[0].dtypes.wei))
       << ", output_dtype=" << (params.empty() ? "none" : dt_name(params[0].dtypes.dst))
       << ", active_matmul=" << (params.empty() ? 0 : params[0].active_matmul)
       << ", mode=" << (fused ? "fused_moe" : (src.size() == 1 && M.size() > 1 ? "sequential" : "parallel"))
       << ", gated_act=" << (gated_act ? "true" : "false") << ", moe_postop=" << (moe_postop ? "true" : "false");
    log_call(ss.str(), st, timer, weight.empty() ? nullptr : weight[0]);
  }
  return st;
}
}  // namespace matmul

// =========================================================================================== reorder
namespace reorder {

size_t weight_prepack_size(const reorder_params_t &params) {
  const prepack_params_t &pp = params.prepack;
  if (pp.K <= 0 || pp.N <= 0 || pp.wei_dtype != data_type_t::s8) return 0;
  if (pp.cached_size == 0) pp.cached_size = b200dnn_prepack_size(pp.K, pp.N, 0);
  return pp.cached_size;
}

status_t weight_prepack_into(const void *weights, const reorder_params_t &params, void *dst) {
  const prepack_params_t &pp = params.prepack;
  if (!weights || !dst) return shim_fail(status_t::failure, "prepack: null pointer");
  if (pp.wei_dtype != data_type_t::s8) return shim_fail(status_t::unimplemented, "prepack: only s8 weights are implemented");
  if (pp.sym_group_size != 0 && pp.sym_group_size != pp.K)
    return shim_fail(status_t::unimplemented, "prepack: per-group symmetric quantisation is not implemented");
  return from_c(b200dnn_prepack(weights, pp.K, pp.N, pp.ldb > 0 ? pp.ldb : (pp.transposed ? pp.K : pp.N), pp.transposed ? 1 : 0, 0,
                                dst, g_stream));
}

static status_t reorder_impl(const void *src, void *dst, reorder_params_t &params) {
  if (params.is_prepack) return weight_prepack_into(src, params, dst);
  if (!src) return shim_fail(status_t::failure, "reorder: null src");
  if (!params.is_2d()) return shim_fail(status_t::unimplemented, "reorder: only 2-D shapes are implemented");
  const int64_t M = params.M(), N = params.N();
  if (M <= 0 || N <= 0) return shim_fail(status_t::failure, "reorder: non-positive shape");
  if (!params.dst_shape.empty() && params.dst_shape != params.src_shape) return shim_fail(status_t::failure, "reorder: shapes differ");
  int64_t src_ld = N;
  if (params.has_src_strides()) {
    if (params.src_strides.size() != 2 || params.src_strides[1] != 1) return shim_fail(status_t::unimplemented, "reorder: source must be row-strided");
    src_ld = params.src_strides[0];
  }
  const auto &sc = params.quant_params.scale;
  const auto &zp = params.quant_params.zero_point;
  const int32_t sdt = static_cast<int32_t>(params.src_dtype), ddt = static_cast<int32_t>(params.dst_dtype);
  const bool src_float = params.src_dtype == data_type_t::f32 || params.src_dtype == data_type_t::bf16;
  const int64_t ns = nelem(sc.dims) > 0 ? nelem(sc.dims) : 1;
  const bool per_token = sc.dims.size() == 2 && sc.dims[0] == M && sc.dims[1] == 1 && M > 1;
  const bool per_channel = sc.dims.size() == 2 && sc.dims[0] == 1 && sc.dims[1] == N && N > 1;
  if (params.dynamic_quant) {
    // the caller owns the scale buffer (lowoha_reorder_utils.cpp:524-528); dst == null computes scales only
    if (!sc.buff) return shim_fail(status_t::failure, "reorder: dynamic quantisation needs a scale buffer");
    if (zp.buff) {
      // asymmetric: f32|bf16 -> u8, one scale and one s32 zero point per token (scale and zero-point dims {M,1})
      if (!src_float || (dst && params.dst_dtype != data_type_t::u8)) return shim_fail(status_t::unimplemented, "reorder: asymmetric dynamic quantisation is f32|bf16 -> u8");
      const bool tok = per_token || (ns == M && M == 1);
      if (!tok || zp.dims != sc.dims) return shim_fail(status_t::unimplemented, "reorder: asymmetric dynamic quantisation is implemented per token");
      if (sc.dt != data_type_t::f32 || zp.dt != data_type_t::s32) return shim_fail(status_t::unimplemented, "reorder: asymmetric scales are f32, zero points s32");
      return from_c(b200dnn_quant_per_token_asym(src, sdt, M, N, src_ld, dst, N, static_cast<float *>(sc.buff), static_cast<int32_t *>(zp.buff), g_stream));
    }
    if (!src_float || (dst && params.dst_dtype != data_type_t::s8)) return shim_fail(status_t::unimplemented, "reorder: dynamic quantisation is f32|bf16 -> s8");
    if (per_token || (ns == M && M == 1 && N > 1 && sc.dims.size() == 2 && sc.dims[1] == 1))
      return from_c(b200dnn_quant_per_token(src, sdt, M, N, src_ld, dst, N, sc.buff, static_cast<int32_t>(sc.dt), g_stream));
    if (sc.dt != data_type_t::f32) return shim_fail(status_t::unimplemented, "reorder: per-channel / per-tensor scales are f32");
    if (per_channel) return from_c(b200dnn_quant_dynamic(src, sdt, M, N, src_ld, 1, dst, N, static_cast<float *>(sc.buff), g_stream));
    if (ns == 1) return from_c(b200dnn_quant_dynamic(src, sdt, M, N, src_ld, 0, dst, N, static_cast<float *>(sc.buff), g_stream));
    // per-group along K: scale dims {M, G}; every (row, group) is quantised like a token
    // (reorder/reorder_data_type/dynamic_quant_impl/dynamic_dispatch.cpp:255-353)
    if (sc.dims.size() == 2 && sc.dims[0] == M && sc.dims[1] > 1 && N % sc.dims[1] == 0) {
      if (src_ld != N) return shim_fail(status_t::unimplemented, "reorder: per-group dynamic quantisation needs contiguous rows");
      const int64_t G = sc.dims[1], gs = N / G;
      if (sc.dt != data_type_t::f32 && sc.dt != data_type_t::bf16) return shim_fail(status_t::unimplemented, "reorder: per-group scales are f32 or bf16");
      return from_c(b200dnn_quant_per_token(src, sdt, M * G, gs, gs, dst, gs, sc.buff, static_cast<int32_t>(sc.dt), g_stream));
    }
    return shim_fail(status_t::unimplemented, "reorder: this scale granularity is not implemented for dynamic quantisation");
  }
  if (!dst) return shim_fail(status_t::failure, "reorder: null dst");
  if (!sc.buff || sc.dt != data_type_t::f32) return shim_fail(status_t::unimplemented, "reorder: static (de)quantisation needs an f32 scale");
  if (!(ns == 1 || per_channel)) return shim_fail(status_t::unimplemented, "reorder: scale must be per-tensor or per-channel");
  int64_t nz = 0;
  if (zp.buff) {
    if (zp.dt != data_type_t::s32) return shim_fail(status_t::unimplemented, "reorder: zero-point must be s32");
    nz = nelem(zp.dims) > 0 ? nelem(zp.dims) : 1;
    if (!(nz == 1 || nz == N)) return shim_fail(status_t::unimplemented, "reorder: zero-point granularity");
  }
  const bool dst_int = params.dst_dtype == data_type_t::s8 || params.dst_dtype == data_type_t::u8;
  const bool src_int = params.src_dtype == data_type_t::s8 || params.src_dtype == data_type_t::u8;
  if (src_float && dst_int)
    return from_c(b200dnn_quant_static(src, sdt, M, N, src_ld, static_cast<const float *>(sc.buff), ns,
                                       static_cast<const int32_t *>(zp.buff), nz, dst, ddt, N, g_stream));
  if (src_int && (params.dst_dtype == data_type_t::f32 || params.dst_dtype == data_type_t::bf16))
    return from_c(b200dnn_dequant_static(src, sdt, M, N, src_ld, static_cast<const float *>(sc.buff), ns,
                                         static_cast<const int32_t *>(zp.buff), nz, dst, ddt, N, g_stream));
  return shim_fail(status_t::unimplemented, "reorder: dtype combination is not implemented");
}

status_t reorder_direct(const void *src, void *dst, reorder_params_t &params) {
  const CallTimer timer;
  const status_t st = reorder_impl(src, dst, params);
  if (apilog_info() || profile_on()) {
    std::ostringstream ss;
    ss << "LOWOHA reorder_direct" << (params.is_prepack ? " (Prepack)" : params.dynamic_quant ? "" : " (Static_Quantize)")
       << ": M=" << (params.is_2d() ? params.M() : 0) << ", K=" << (params.is_2d() ? params.N() : 0)
       << ", src_dtype=" << dt_name(params.src_dtype) << ", dst_dtype=" << dt_name(params.dst_dtype)
       << ", dynamic_quant=" << (params.dynamic_quant ? "true" : "false");
    log_call(ss.str(), st, timer, src);
  }
  return st;
}

status_t group_dynamic_quant(const std::vector<const void *> &src, const std::vector<int> &M, const std::vector<int> &K,
                             const std::vector<std::vector<int64_t>> &src_strides, const std::vector<void *> &dst,
                             const std::vector<std::vector<int64_t>> &dst_strides, const std::vector<void *> &scale,
                             const group_dynamic_quant_params_t &params) {
  // one entry per expert; params.num_groups is the GRANULARITY: <= 1 per token, > 1 that many groups along K with a
  // {M_i, G} scale buffer (reorder/lowoha_reorder_common.hpp:335-360, checks reorder/lowoha_reorder.cpp:279-372)
  const size_t num_ops = M.size();
  if (num_ops == 0) return shim_fail(status_t::failure, "group_dynamic_quant: M vector is empty");
  if (src.size() != num_ops || K.size() != num_ops || dst.size() != num_ops || scale.size() != num_ops ||
      (!src_strides.empty() && src_strides.size() != num_ops) || (!dst_strides.empty() && dst_strides.size() != num_ops))
    return shim_fail(status_t::failure, "group_dynamic_quant: vector size mismatch");
  if (params.dst_dtype != data_type_t::s8) return shim_fail(status_t::failure, "group_dynamic_quant: only s8 destination is supported");
  if (params.src_dtype != data_type_t::bf16 && params.src_dtype != data_type_t::f32)
    return shim_fail(status_t::failure, "group_dynamic_quant: only bf16/f32 source is supported");
  if (params.scale_dtype != data_type_t::f32 && params.scale_dtype != data_type_t::bf16)
    return shim_fail(status_t::failure, "group_dynamic_quant: scale dtype must be f32 or bf16");
  const int64_t G = params.num_groups;
  const bool per_group = G > 1;
  std::vector<int32_t> m(num_ops), k(num_ops);
  std::vector<int64_t> sld(num_ops), dld(num_ops);
  for (size_t i = 0; i < num_ops; ++i) {
    int64_t s_ld = K[i], d_ld = K[i];
    if (!src_strides.empty() && !src_strides[i].empty()) {
      if (src_strides[i].size() != 2 || src_strides[i][1] != 1) return shim_fail(status_t::failure, "group_dynamic_quant: src_strides must be empty or {row_stride, 1}");
      s_ld = src_strides[i][0];
    }
    if (!dst_strides.empty() && !dst_strides[i].empty()) {
      if (dst_strides[i].size() != 2 || dst_strides[i][1] != 1) return shim_fail(status_t::failure, "group_dynamic_quant: dst_strides must be empty or {row_stride, 1}");
      d_ld = dst_strides[i][0];
    }
    if (M[i] < 0 || K[i] <= 0 || s_ld < K[i] || d_ld < K[i]) return shim_fail(status_t::failure, "group_dynamic_quant: invalid shape or stride");
    m[i] = M[i]; k[i] = K[i]; sld[i] = s_ld; dld[i] = d_ld;
    if (M[i] == 0) continue;      // experts without rows are not validated further, as in the reference
    if (per_group && K[i] % G != 0) return shim_fail(status_t::failure, "group_dynamic_quant: per-group requires K % num_groups == 0");
    if (!src[i] || !dst[i] || !scale[i]) return shim_fail(status_t::failure, "group_dynamic_quant: null active buffer");
    if (per_group) {
      // every (row, group) becomes a row of K/G elements; that view needs rows without gaps
      if (s_ld != K[i] || d_ld != K[i]) return shim_fail(status_t::unimplemented, "group_dynamic_quant: per-group needs contiguous rows");
      m[i] = static_cast<int32_t>(M[i] * G); k[i] = static_cast<int32_t>(K[i] / G); sld[i] = k[i]; dld[i] = k[i];
    }
  }
  return from_c(b200dnn_group_quant_per_token(static_cast<int32_t>(num_ops), src.data(), static_cast<int32_t>(params.src_dtype), m.data(),
                                              k.data(), sld.data(), dst.data(), dld.data(), scale.data(),
                                              static_cast<int32_t>(params.scale_dtype), g_stream));
}

}  // namespace reorder
}  // namespace lowoha
}  // namespace zendnnl

// ------------------------------------------------------------------------------------------------ normalization
namespace zendnnl { namespace lowoha { namespace normalization {

status_t normalization_direct(const void *input, void *output, const void *gamma, const void *beta, const void *running_mean,
                              const void *running_var, void *residual, norm_params &params) {
  b200dnn_norm_t d;
  std::memset(&d, 0, sizeof d);
  d.norm_type = static_cast<int32_t>(params.norm_type);
  d.use_scale = params.use_scale ? 1 : 0; d.use_shift = params.use_shift ? 1 : 0;
  d.epsilon = params.epsilon;
  d.batch = static_cast<int64_t>(params.batch); d.norm_size = static_cast<int64_t>(params.norm_size);
  d.num_channels = static_cast<int64_t>(params.num_channels);
  d.src_dt = static_cast<int32_t>(params.src_dt); d.dst_dt = static_cast<int32_t>(params.dst_dt);
  d.gamma_dt = static_cast<int32_t>(params.gamma_dt); d.beta_dt = static_cast<int32_t>(params.beta_dt);
  d.input = input; d.output = output; d.gamma = gamma; d.beta = beta;
  d.running_mean = static_cast<const float *>(running_mean); d.running_var = static_cast<const float *>(running_var);
  d.residual = residual;
  return from_c(b200dnn_normalization(&d, g_stream));
}

}}}  // namespace zendnnl::lowoha::normalization

// ------------------------------------------------------------------------------------------------ sdpa
namespace zendnnl { namespace lowoha { namespace sdpa {

status_t sdpa_direct(const void *query, const void *key, const void *value, const void *attn_mask, void *output, sdpa_params &p) {
  b200dnn_sdpa_t d;
  std::memset(&d, 0, sizeof d);
  d.batch = p.batch; d.num_heads = p.num_heads; d.seq_len = p.seq_len; d.kv_seq_len = p.kv_seq_len; d.head_dim = p.head_dim;
  const int64_t qs[4] = {p.q_stride_b, p.q_stride_h, p.q_stride_s, p.q_stride_d}, ks[4] = {p.k_stride_b, p.k_stride_h, p.k_stride_s, p.k_stride_d};
  const int64_t vs[4] = {p.v_stride_b, p.v_stride_h, p.v_stride_s, p.v_stride_d}, os[4] = {p.o_stride_b, p.o_stride_h, p.o_stride_s, p.o_stride_d};
  for (int i = 0; i < 4; ++i) {
    d.q_stride[i] = qs[i]; d.k_stride[i] = ks[i]; d.v_stride[i] = vs[i]; d.o_stride[i] = os[i];
    d.mask_sizes[i] = p.mask_sizes[i]; d.mask_strides[i] = p.mask_strides[i];
  }
  d.mask_ndims = p.mask_ndims; d.is_causal = p.is_causal ? 1 : 0;
  d.qkv_dt = static_cast<int32_t>(p.qkv_dt); d.out_dt = static_cast<int32_t>(p.out_dt); d.mask_dt = static_cast<int32_t>(p.mask_dt);
  d.scale = p.scale; d.dropout_p = p.dropout_p;
  d.query = query; d.key = key; d.value = value; d.attn_mask = attn_mask; d.output = output;
  return from_c(b200dnn_sdpa(&d, g_stream));
}

}}}  // namespace zendnnl::lowoha::sdpa
