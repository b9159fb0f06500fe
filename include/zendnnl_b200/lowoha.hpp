// C++ interface of the B200-native LowOHA W8A8 path: the reference's namespaces, type names,
// field names, enum values and function signatures, so that code written against the reference
// headers compiles against this one.  Implemented in zendnn_b200/csrc/lowoha_host.cpp as thin
// callers of the C ABI (b200dnn.h).
//
// Reference declarations mirrored here (paths inside the reference checkout, zendnnl/src/):
//   common/data_types.hpp:44-58 (data_type_t)       common/error_status.hpp:34-58 (status_t)
//   operators/common/post_op.hpp:36-57               operators/matmul/matmul_config.hpp:37-52
//   lowoha_operators/matmul/lowoha_common.hpp:38-227 lowoha_operators/matmul/lowoha_matmul.hpp:104-223
//   lowoha_operators/matmul/group_matmul/group_matmul_direct.hpp:96-171,406-577
//   lowoha_operators/reorder/lowoha_reorder_common.hpp:38-360
//   lowoha_operators/reorder/prepack/lowoha_prepack.hpp:75-165
//   lowoha_operators/reorder/lowoha_reorder.hpp:103-128
// Pointers may be host or device memory.  Features outside the supported W8A8 subset return
// status_t::unimplemented.
#ifndef ZENDNNL_B200_LOWOHA_HPP
#define ZENDNNL_B200_LOWOHA_HPP

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#if defined(__GNUC__)
#define ZENDNNL_B200_API __attribute__((visibility("default")))
#else
#define ZENDNNL_B200_API
#endif

namespace zendnnl {

namespace common {
enum class data_type_t : uint8_t { none, f32, f16, bf16, s32, s64, s16, s8, s4, u32, u16, u8, u4 };
}  // namespace common

namespace error_handling {
enum class status_t : int32_t {
  success = 1, failure = 0, unimplemented = -1, bad_object = -2, op_bad_context = -3, op_bad_io = -4,
  op_bad_forced_kernel = -5, utils_bad_module_name = -6, utils_bad_dynamic_module = -7, memory_bad_size = -8,
  memory_bad_aligned_size = -9, memory_bad_order = -10, memory_bad_stride = -11, memory_bad_base = -12,
  memory_bad_index = -13, memory_bad_storage = -14, config_bad_json_file = -15, memory_bad_meta = -16,
  memory_bad_quant = -17, lru_node_not_found = -18, lru_node_exists = -19, bad_hash_object = -20,
  isa_unsupported = -21
};
}  // namespace error_handling

namespace ops {
using zendnnl::common::data_type_t;
enum class post_op_type_t {
  none, elu, relu, leaky_relu, gelu_tanh, gelu_erf, sigmoid, swish, tanh, softmax, pooling, square, abs, sqrt, exp,
  log, clip, binary_add, binary_mul, mish
};
enum class matmul_algo_t : int32_t {
  none = -1, dynamic_dispatch = 0, aocl_dlp_blocked = 1, onednn_blocked = 2, libxsmm_blocked = 3, aocl_dlp = 4,
  onednn = 5, libxsmm = 6, batched_sgemm = 7, auto_tuner = 8, reference = 9, native_gemm = 10, native_brgemm = 11,
  algo_count
};
}  // namespace ops

namespace memory {
using zendnnl::common::data_type_t;
using zendnnl::error_handling::status_t;
}  // namespace memory

namespace interface {
using data_type_t = zendnnl::common::data_type_t;
using status_t = zendnnl::error_handling::status_t;
using post_op_type_t = zendnnl::ops::post_op_type_t;
}  // namespace interface

namespace lowoha {

// ------------------------------------------------------------------------------------------ reorder
namespace reorder {
using zendnnl::memory::data_type_t;
using zendnnl::memory::status_t;
using zendnnl::ops::matmul_algo_t;

struct prepack_params_t {
  matmul_algo_t algo = matmul_algo_t::none;
  data_type_t wei_dtype = data_type_t::none;
  data_type_t src_dtype = data_type_t::none;
  int64_t K = 0, N = 0, ldb = 0;
  bool transposed = false;
  int sym_group_size = 0;
  mutable size_t cached_size = 0;
};

enum class reorder_algo_t : int { none = -1, DT = 0, native = 1, reference = 2, algo_count };

struct reorder_quant_params_t {
  struct quant_t {
    void *buff = nullptr;
    data_type_t dt = data_type_t::none;
    std::vector<int64_t> dims;
  };
  quant_t scale;
  quant_t zero_point;
};

struct reorder_params_t {
  data_type_t src_dtype = data_type_t::none;
  data_type_t dst_dtype = data_type_t::none;
  reorder_quant_params_t quant_params;
  reorder_algo_t algo = reorder_algo_t::DT;
  int32_t num_threads = 0;
  std::vector<int64_t> src_shape, dst_shape, src_strides, dst_strides;
  bool dynamic_quant = false;
  bool is_prepack = false;
  prepack_params_t prepack;

  bool is_1d() const { return src_shape.size() == 1; }
  bool is_2d() const { return src_shape.size() == 2; }
  bool is_3d() const { return src_shape.size() == 3; }
  int64_t M() const { return is_3d() ? src_shape[1] : (src_shape.empty() ? 0 : src_shape[0]); }
  int64_t N() const { return is_1d() ? 1 : (is_2d() ? src_shape[1] : (is_3d() ? src_shape[2] : 0)); }
  int64_t nelems() const { int64_t n = src_shape.empty() ? 0 : 1; for (auto d : src_shape) n *= d; return n; }
  bool has_src_strides() const { return !src_strides.empty(); }
};

struct group_dynamic_quant_params_t {
  data_type_t src_dtype = data_type_t::none;
  data_type_t dst_dtype = data_type_t::none;
  data_type_t scale_dtype = data_type_t::f32;
  int32_t num_threads = 0;
  int32_t num_groups = 0;
};

ZENDNNL_B200_API size_t weight_prepack_size(const reorder_params_t &params);
ZENDNNL_B200_API status_t weight_prepack_into(const void *weights, const reorder_params_t &params, void *dst);
ZENDNNL_B200_API status_t reorder_direct(const void *src, void *dst, reorder_params_t &params);
ZENDNNL_B200_API status_t group_dynamic_quant(const std::vector<const void *> &src, const std::vector<int> &M,
                                              const std::vector<int> &K,
                                              const std::vector<std::vector<int64_t>> &src_strides,
                                              const std::vector<void *> &dst,
                                              const std::vector<std::vector<int64_t>> &dst_strides,
                                              const std::vector<void *> &scale,
                                              const group_dynamic_quant_params_t &params);
}  // namespace reorder

// ------------------------------------------------------------------------------------------ normalization
// Mirrors lowoha_operators/normalization/lowoha_normalization_common.hpp:63-153 (enum values, field order, defaults) and
// lowoha_normalization.hpp:98-107.
namespace normalization {
using zendnnl::memory::data_type_t;
using zendnnl::memory::status_t;

enum class norm_type_t : int { NONE = -1, LAYER_NORM = 0, BATCH_NORM = 1, RMS_NORM = 2, FUSED_ADD_RMS_NORM = 3 };
enum class norm_algo_t : int { none = -1, dynamic_dispatch = 0, reference = 1 };

struct norm_params {
  norm_type_t norm_type = norm_type_t::NONE;
  uint64_t batch = 0, norm_size = 0, num_channels = 0;
  float epsilon = 1e-5f;
  bool use_scale = false, use_shift = false;
  data_type_t src_dt = data_type_t::none, dst_dt = data_type_t::none, gamma_dt = data_type_t::f32, beta_dt = data_type_t::f32;
  norm_algo_t algorithm = norm_algo_t::none;
  int32_t num_threads = 0;
  data_type_t accum_type = data_type_t::f32;
};

ZENDNNL_B200_API status_t normalization_direct(const void *input, void *output, const void *gamma, const void *beta,
                                               const void *running_mean, const void *running_var, void *residual,
                                               norm_params &params);
}  // namespace normalization

// ------------------------------------------------------------------------------------------ sdpa
// Mirrors lowoha_operators/sdpa/lowoha_sdpa_common.hpp:31-103 (field order and defaults) and lowoha_sdpa.hpp:48-55.
namespace sdpa {
using zendnnl::memory::data_type_t;
using zendnnl::memory::status_t;

enum class mask_type_t { none = 0, causal = 1, custom = 2 };

struct sdpa_params {
  int64_t batch = 1, num_heads = 1, seq_len = 0, kv_seq_len = 0, head_dim = 0;
  int64_t q_stride_b = 0, q_stride_h = 0, q_stride_s = 0, q_stride_d = 1;
  int64_t k_stride_b = 0, k_stride_h = 0, k_stride_s = 0, k_stride_d = 1;
  int64_t v_stride_b = 0, v_stride_h = 0, v_stride_s = 0, v_stride_d = 1;
  int64_t o_stride_b = 0, o_stride_h = 0, o_stride_s = 0, o_stride_d = 1;
  int mask_ndims = 0;
  int64_t mask_sizes[4] = {0, 0, 0, 0};
  int64_t mask_strides[4] = {0, 0, 0, 0};
  mask_type_t mask_type = mask_type_t::none;
  int64_t mask_dims[3] = {0, 0, 0};
  data_type_t qkv_dt = data_type_t::none, out_dt = data_type_t::none, mask_dt = data_type_t::none;
  double scale = 0.0;
  bool is_causal = false;
  double dropout_p = 0.0;
  int32_t num_threads = 0;
};

ZENDNNL_B200_API status_t sdpa_direct(const void *query, const void *key, const void *value, const void *attn_mask, void *output,
                                      sdpa_params &params);
}  // namespace sdpa

// ------------------------------------------------------------------------------------------ matmul
namespace matmul {
using namespace zendnnl::memory;
using namespace zendnnl::ops;

struct matmul_data_types {
  data_type_t src = data_type_t::none, wei = data_type_t::none, dst = data_type_t::none, bias = data_type_t::none,
              compute = data_type_t::none;
};

struct matmul_post_op {
  post_op_type_t po_type = post_op_type_t::none;
  void *buff = nullptr;              // operand of binary_add / binary_mul
  data_type_t dtype = data_type_t::none;
  std::vector<int64_t> dims;         // {1,N}: row broadcast; otherwise dense [M, leading_dim]
  float alpha = 0.0f, beta = 0.0f;   // clip: alpha = lower, beta = upper
  int leading_dim = -1;
};

struct matmul_quantization_params_t {
  struct matmul_quant_t {
    const void *buff = nullptr;
    data_type_t dt = data_type_t::none;
    std::vector<int64_t> dims;       // {} or {1}: per-tensor; {M,1}: per-token; {1,N}: per-channel
  };
  matmul_quant_t src_scale, wei_scale, dst_scale, src_zp, wei_zp, dst_zp;
};

struct matmul_batch_params_t {
  int Batch_A = 1, Batch_B = 1;
  size_t batch_stride_src = static_cast<size_t>(-1), batch_stride_wei = static_cast<size_t>(-1),
         batch_stride_dst = static_cast<size_t>(-1);
};

struct pack_format { int pack_format_b = 0; };

struct matmul_params {
  matmul_data_types dtypes;
  std::vector<matmul_post_op> postop_;
  matmul_quantization_params_t quant_params;
  char mem_format_a = 'n';
  char mem_format_b = 'n';           // 'r': weight buffer written by reorder_direct(is_prepack)
  matmul_algo_t lowoha_algo = matmul_algo_t::none;   // accepted and ignored: there is one backend
  int32_t num_threads = 0;           // accepted and ignored
  std::string plugin_op;
  bool dynamic_quant = false;
  pack_format packing;
  uint32_t total_matmul = 0, active_matmul = 0;
  int32_t weight_cache_type = 2;     // 0 disables caching of packed weights for this call
};

struct group_matmul_moe_postop_params {
  int num_tokens = 0;
  int topk = 0;
  void *output = nullptr;
  int ldc_output = 0;
  const float *topk_weights = nullptr;
  bool skip_weighted = false;
  const void **row_ptrs = nullptr;
};

enum class grp_matmul_gated_act_t : int { none = 0, silu_and_mul = 1, gelu_and_mul = 2, swiglu_oai_mul = 3 };
struct grp_matmul_gated_act_params { grp_matmul_gated_act_t act = grp_matmul_gated_act_t::none; };

struct grp_matmul_fused_moe_params {
  std::vector<const void *> down_weight;
  std::vector<int> N_down, ldb_down;
  std::vector<const void *> bias_down;
  data_type_t bias_dt_down = data_type_t::none;
  struct down_weight_quant_t {
    const void *buff = nullptr;
    data_type_t dt = data_type_t::none;
    std::vector<int64_t> dims;
  };
  std::vector<down_weight_quant_t> down_scale, down_zp;
  std::vector<void *> dst_down;
  std::vector<int> ldc_down;
};

ZENDNNL_B200_API status_t matmul_direct(const char layout, const bool transA, const bool transB, const int M, const int N,
                                        const int K, const float alpha, const void *src, const int lda, const void *weight,
                                        const int ldb, const void *bias, const float beta, void *dst, const int ldc,
                                        const bool is_weights_const, const matmul_batch_params_t &batch_params,
                                        const matmul_params &params);

ZENDNNL_B200_API status_t group_matmul_direct(
    const std::vector<char> &layout, const std::vector<bool> &transA, const std::vector<bool> &transB,
    const std::vector<int> &M, const std::vector<int> &N, const std::vector<int> &K, const std::vector<float> &alpha,
    const std::vector<const void *> &src, const std::vector<int> &lda, const std::vector<const void *> &weight,
    const std::vector<int> &ldb, const std::vector<const void *> &bias, const std::vector<float> &beta,
    const std::vector<void *> &dst, const std::vector<int> &ldc, const std::vector<bool> &is_weights_const,
    const std::vector<matmul_params> &params, const group_matmul_moe_postop_params *moe_postop = nullptr,
    const grp_matmul_gated_act_params *gated_act = nullptr, const grp_matmul_fused_moe_params *fused_moe = nullptr);

ZENDNNL_B200_API status_t group_matmul_moe_act_execute(const grp_matmul_gated_act_params *act_params,
                                                       const std::vector<void *> &dst, const std::vector<int> &M,
                                                       const std::vector<int> &N, const std::vector<int> &ldc,
                                                       data_type_t dst_dtype, int num_threads);
ZENDNNL_B200_API status_t group_matmul_moe_postop_execute(const group_matmul_moe_postop_params *postop, int D,
                                                          int num_threads, data_type_t dst_elem);
ZENDNNL_B200_API void clear_fused_moe_scratch();
// text of the last failure on the calling thread
ZENDNNL_B200_API const char *last_error();
}  // namespace matmul

// Not in the reference (a CPU library has no streams).  The CUDA stream (a cudaStream_t passed as void*) on which the
// calling thread's matmul_direct / group_matmul_direct / reorder_direct calls enqueue their work; nullptr, the default,
// is the legacy default stream.  Per thread: two threads with two streams run concurrently and share no scratch.
// Calls whose buffers are all device memory return as soon as the work is enqueued.
namespace b200 {
ZENDNNL_B200_API void set_stream(void *cuda_stream);
ZENDNNL_B200_API void *get_stream();
}  // namespace b200
}  // namespace lowoha
}  // namespace zendnnl

#endif  // ZENDNNL_B200_LOWOHA_HPP
