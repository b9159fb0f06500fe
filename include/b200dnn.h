/*
 * b200dnn.h -- C ABI of the B200-native LowOHA W8A8 hot path (libb200dnn.so).
 *
 * Plain C, plain pointers and sizes.  Every entry point names the reference (amd/ZenDNN)
 * interface it stands in for; paths are relative to the reference root,
 * zendnnl/src/lowoha_operators/ unless stated.  The C++ shims that keep the reference's
 * own signatures (include/zendnnl_b200/lowoha.hpp) are thin callers of these functions.
 *
 * Conventions
 *  - Return value: the reference's status_t as int32 (common/error_status.hpp:34-58):
 *    1 success, 0 failure (contract violation or CUDA error), -1 unimplemented.
 *    b200dnn_last_error() gives the text for the calling thread.
 *  - Data pointers may be host or device pointers, independently; each is classified with
 *    cudaPointerGetAttributes.  Host buffers are staged through library-owned device
 *    workspace (inputs copied in, outputs copied back before the call returns).  With device
 *    pointers the call only enqueues work on `stream` and returns.
 *  - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 *  - dtype codes are the reference's data_type_t (common/data_types.hpp:44-58):
 *    1 f32, 3 bf16, 4 s32, 7 s8, 11 u8.  Post-op codes are post_op_type_t
 *    (../operators/common/post_op.hpp:36-57).
 *  - There is no CPU fallback anywhere: without a usable CUDA device every compute entry
 *    point returns failure.
 */
#ifndef B200DNN_H
#define B200DNN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define B200DNN_API __attribute__((visibility("default")))
#else
#define B200DNN_API
#endif

#define B200DNN_SUCCESS 1
#define B200DNN_FAILURE 0
#define B200DNN_UNIMPLEMENTED (-1)

enum { B200DNN_F32 = 1, B200DNN_BF16 = 3, B200DNN_S32 = 4, B200DNN_S8 = 7, B200DNN_S4 = 8, B200DNN_U8 = 11, B200DNN_U4 = 12 };
enum { B200DNN_MAX_POSTOPS = 8 };
/* b200dnn_matmul_t::flags.  STABLE_WEIGHTS: the (prepacked or cached) weight was written before
 * any work still pending on the stream, so the decode kernel may start streaming it while the
 * previous kernel of the stream is still finishing (programmatic dependent launch).  Activations,
 * scales and outputs are never touched early.  Do not set it when the weight buffer is produced
 * by work enqueued just before the call. */
enum { B200DNN_FLAG_STABLE_WEIGHTS = 1 };

/* One scale / zero-point tensor: matmul_quantization_params_t::matmul_quant_t
 * (matmul/lowoha_common.hpp:67-86).  count = number of elements: 1 per-tensor,
 * M per-token ({M,1}), N per-channel ({1,N}); 0 = absent.  Per-group forms: M*G for a source scale of dims {M,G},
 * G*N for a weight scale of dims {G,N} (G groups along K; the library derives G from the counts). */
typedef struct b200dnn_quant_t {
  const void *buff;
  int32_t dt;
  int32_t reserved;
  int64_t count;
} b200dnn_quant_t;

/* One post-op: matmul_post_op (matmul/lowoha_common.hpp:53-65).  For binary_add/mul,
 * ld == 0 means a {1,N} row broadcast, ld > 0 a dense [M,ld] operand.  clip: alpha = lower,
 * beta = upper (matmul/backends/aocl/aocl_postop.cpp:424-433). */
typedef struct b200dnn_postop_t {
  int32_t type;
  int32_t dt;
  const void *buff;
  int64_t ld;
  float alpha;
  float beta;
} b200dnn_postop_t;

/* Flat form of the arguments of matmul_direct (matmul/lowoha_matmul.hpp:104-108) plus the
 * fields of matmul_params it reads on the INT8 path (matmul/lowoha_common.hpp:142-227). */
typedef struct b200dnn_matmul_t {
  int32_t M, N, K;
  int32_t transB;        /* 0: weight is [K,ldb]; 1: weight is [N,ldb] */
  int32_t src_dt;        /* u8 | s8, or bf16 | f32 together with dynamic_quant */
  int32_t wei_dt;        /* s8 */
  int32_t dst_dt;        /* bf16 | f32 | s32, or s8 | u8 with dst_scale (requantised destination) */
  int32_t bias_dt;       /* f32 | bf16; ignored when bias == NULL */
  int64_t lda, ldb, ldc; /* in elements */
  const void *src;
  const void *weight;    /* raw s8 weights, or a buffer written by b200dnn_prepack when wei_format=='r' */
  const void *bias;
  void *dst;
  int32_t wei_format;    /* 'n' raw | 'r' prepacked: matmul_params::mem_format_b */
  int32_t weights_const; /* is_weights_const: raw weights are packed once and cached by address */
  int32_t dynamic_quant; /* matmul_params::dynamic_quant: per-token s8 quantisation of a bf16/f32 src */
  int32_t n_postops;
  b200dnn_quant_t src_scale; /* with dynamic_quant: buff may be NULL; if not, the M scales are written there */
  b200dnn_quant_t wei_scale;
  b200dnn_quant_t src_zp;    /* per-tensor; dt s32 | s8 | u8 */
  b200dnn_postop_t postops[B200DNN_MAX_POSTOPS];
  int32_t force_kernel;  /* for tests: 0 auto, 1 weight-streaming kernels, 2 tcgen05 kernel, 3 tiled streaming kernel only */
  int32_t flags;         /* B200DNN_FLAG_* */
  /* requantised integer destination (dst_dt s8 | u8): after bias and post-ops, q = rne(clamp(x * dst_scale + dst_zp)), the
   * last step of the reference's epilogue chain (matmul/backends/aocl/aocl_postop.cpp:1339-1453; definition
   * operators/matmul/matmul_ref_kernel.cpp:155-192,770-797).  dst_scale: per-tensor f32 (count 1; absent = 1); dst_zp:
   * optional, per-tensor s32.  Ignored for float and s32 destinations. */
  b200dnn_quant_t dst_scale;
  b200dnn_quant_t dst_zp;
  /* weight zero points, read for u4 weights only (weight-only quantisation: bf16 source, s4 | u4 weights, no dynamic_quant;
   * lowoha_matmul_utils.cpp:319-331): s8 or bf16, count 1, N or G*N like wei_scale.  w = bf16((q - zp) * scale) with an s8
   * zero point, bf16((q - 8) * scale + zp) with a bf16 one (operators/matmul/matmul_ref_kernel.cpp:466-474). */
  b200dnn_quant_t wei_zp;
  int32_t transA;        /* != 0: the source is stored transposed, element (m, k) at src[k * lda + m] with lda >= M (matmul_direct's
                          * transA, lowoha_matmul.hpp:95-99); it is transposed into the workspace first */
  int32_t reserved_a;
} b200dnn_matmul_t;

B200DNN_API const char *b200dnn_last_error(void);
B200DNN_API int32_t b200dnn_version(void);
/* Number of CUDA devices the library can use; 0 when there is none (no compute possible). */
B200DNN_API int32_t b200dnn_device_count(void);
/* Kernels launched by this library in the calling process so far (for benchmark accounting). */
B200DNN_API int64_t b200dnn_launch_count(void);

/* matmul_direct, INT8 path (matmul/lowoha_matmul.cpp:278): C = postops(dequant(A*B) + bias). */
B200DNN_API int32_t b200dnn_matmul(const b200dnn_matmul_t *desc, void *stream);

/* group_matmul_direct, plain parallel mode (matmul/lowoha_matmul.hpp:204-223; dispatch
 * matmul/group_matmul/group_matmul_parallel_common.hpp:1240-1248): num_ops independent GEMMs, each with its own source,
 * weight, bias and destination; descriptors with M == 0 are skipped.  The result is that of num_ops b200dnn_matmul
 * calls.  When the active descriptors share K, N, the dtypes, the quantisation form (s8 rows with per-token f32 scales,
 * or bf16 / f32 rows with dynamic_quant and no caller-side scale buffer), per-channel f32 weight scales and the same
 * element-wise post-ops, all of them run in ONE grouped tcgen05 launch; otherwise one launch per descriptor. */
B200DNN_API int32_t b200dnn_group_matmul(int32_t num_ops, const b200dnn_matmul_t *descs, void *stream);

/* No counterpart in the reference.  The same W8A8 matmul for callers that cannot allocate device
 * memory at call time (a server whose own pool already holds all free memory, a latency-bound loop
 * that cannot risk a blocking cudaMalloc): it never allocates.  The split-K scratch is a fixed
 * 8 MiB + 16 KiB device array inside the library, held by every GPU that uses it until the process
 * exits; split shapes that need more are rejected with failure (shapes that are not split over K use
 * no scratch and are never rejected for it).  Restrictions, all checked: every pointer is a device
 * pointer, the weight is a buffer written by b200dnn_prepack for this K and N (wei_format 'r'), no
 * dynamic_quant.  The first call on a device is a warm-up: it loads the module that holds the array
 * and resolves the array's address, so make it before the application's pool takes the remaining
 * memory and before any stream capture.  All calls share the array: calls that overlap on the GPU
 * race, so keep them on one stream or otherwise serialised. */
B200DNN_API int32_t b200dnn_matmul_static_scratch(const b200dnn_matmul_t *desc, void *stream);
/* No counterpart in the reference.  Bytes of the fixed array that b200dnn_matmul_static_scratch would use for this
 * shape on a device with sm_count SMs (0 = the current device); 0 bytes for shapes that are not split.  Returns
 * failure when the shape would be rejected.  Host arithmetic only. */
B200DNN_API int32_t b200dnn_static_scratch_query(int32_t M, int32_t N, int32_t K, int32_t sm_count, size_t *bytes);

/* weight_prepack_size (reorder/prepack/lowoha_prepack.cpp:285): bytes of the packed form of a
 * K x N s8 weight (multiple of 64).  gated != 0 selects the gate/up interleaved form used by
 * the fused MoE first GEMM (N = 2*I, I a multiple of 32). */
B200DNN_API size_t b200dnn_prepack_size(int64_t K, int64_t N, int32_t gated);
/* reorder_direct with is_prepack (reorder/lowoha_reorder.cpp:43 -> prepack/lowoha_prepack.cpp:315):
 * writes the packed weight (K-major rows padded for TMA, column sums appended) into dst. */
B200DNN_API int32_t b200dnn_prepack(const void *weight, int64_t K, int64_t N, int64_t ldb, int32_t transB,
                        int32_t gated, void *dst, void *stream);
/* The two reorder_direct calls that prepare an INT8 weight from a float one, as one call: per-channel dynamic
 * quantisation (reorder/lowoha_reorder.cpp:186, scale dims {1,N}) and the prepack reorder
 * (reorder/prepack/lowoha_prepack.cpp:315).  weight [K,N] (or [N,K] with transB) in bf16|f32 -> dst in the layout
 * b200dnn_prepack writes (b200dnn_prepack_bytes(K,N) bytes) and N f32 scales, indexed by the caller's column.  The
 * bytes and the scales are those of b200dnn_quant_dynamic followed by b200dnn_prepack; the s8 matrix in the caller's
 * layout is never written. */
B200DNN_API int32_t b200dnn_quant_prepack(const void *weight, int32_t wei_dt, int64_t K, int64_t N, int64_t ldb,
                        int32_t transB, int32_t gated, void *dst, float *scale, void *stream);

/* reorder_direct, dynamic per-token symmetric quantisation (reorder/lowoha_reorder.cpp:119-136):
 * src [M,K] f32|bf16 with row stride src_ld -> dst s8 [M,K] (row stride dst_ld; dst may be NULL:
 * scales only) and M scales (scale_dt f32|bf16). */
B200DNN_API int32_t b200dnn_quant_per_token(const void *src, int32_t src_dt, int64_t M, int64_t K, int64_t src_ld,
                                void *dst, int64_t dst_ld, void *scale, int32_t scale_dt, void *stream);
/* Per-token ASYMMETRIC dynamic quantisation, f32|bf16 -> u8 with one f32 scale and one s32 zero point per row
 * (reorder_direct with a zero-point buffer; reorder/reorder_data_type/scalar_impl/dynamic_per_token_ref_kernel.cpp:38-56,128-183).
 * dst may be NULL (scales and zero points only). */
B200DNN_API int32_t b200dnn_quant_per_token_asym(const void *src, int32_t src_dt, int64_t M, int64_t K, int64_t src_ld, void *dst,
                                                 int64_t dst_ld, float *scale, int32_t *zero_point, void *stream);

/* group_dynamic_quant (reorder/lowoha_reorder.cpp:279): the same over num_groups tensors;
 * groups with M[i]==0 are skipped. */
B200DNN_API int32_t b200dnn_group_quant_per_token(int32_t num_groups, const void *const *src, int32_t src_dt,
                                      const int32_t *M, const int32_t *K, const int64_t *src_ld,
                                      void *const *dst, const int64_t *dst_ld, void *const *scale,
                                      int32_t scale_dt, void *stream);
/* reorder_direct, dynamic symmetric scales at per-channel ({1,N}, per_channel=1) or per-tensor
 * granularity followed by the static quantise (reorder/lowoha_reorder_utils.cpp:591, 708-766,
 * 908-935): src [M,N] f32|bf16 -> dst s8 [M,N] (may be NULL) + f32 scales. */
B200DNN_API int32_t b200dnn_quant_dynamic(const void *src, int32_t src_dt, int64_t M, int64_t N, int64_t src_ld,
                              int32_t per_channel, void *dst, int64_t dst_ld, float *scale, void *stream);
/* reorder_direct, static quantise / dequantise (reorder/lowoha_reorder.cpp:211-267):
 * q = clamp(rne(x/s)+zp), x = (q-zp)*s; n_scale and n_zp are 1 or N; zp may be NULL. */
B200DNN_API int32_t b200dnn_quant_static(const void *src, int32_t src_dt, int64_t M, int64_t N, int64_t src_ld,
                             const float *scale, int64_t n_scale, const int32_t *zp, int64_t n_zp,
                             void *dst, int32_t dst_dt, int64_t dst_ld, void *stream);
B200DNN_API int32_t b200dnn_dequant_static(const void *src, int32_t src_dt, int64_t M, int64_t N, int64_t src_ld,
                               const float *scale, int64_t n_scale, const int32_t *zp, int64_t n_zp,
                               void *dst, int32_t dst_dt, int64_t dst_ld, void *stream);

/* group_matmul_moe_act_execute (matmul/group_matmul/group_matmul_moe_act.cpp:728): in place on
 * buf [M, N=2I] (row stride ldc), result in the first I columns.  act: 1 silu_and_mul,
 * 2 gelu_and_mul, 3 swiglu_oai_mul (matmul/group_matmul/group_matmul_direct.hpp:153-158). */
B200DNN_API int32_t b200dnn_gated_act(void *buf, int32_t dt, int64_t M, int64_t N, int64_t ldc, int32_t act, void *stream);

/* group_matmul_moe_postop_execute (matmul/group_matmul/group_matmul_moe_postop.cpp:506):
 * out[t,0:D] = sum_k w[t,k] * row_ptrs[t*topk+k][0:D].  row_ptrs is an array of T*topk
 * pointers (host array; the rows themselves may be host or device memory, all alike). */
B200DNN_API int32_t b200dnn_moe_weighted_reduce(const void *const *row_ptrs, const float *topk_weights,
                                    int32_t num_tokens, int32_t topk, int32_t D, int32_t skip_weighted,
                                    int32_t dt, void *out, int64_t ld_out, void *stream);

/* Flat form of one expert of group_matmul_direct in fused-MoE mode
 * (matmul/lowoha_matmul.hpp:204-223, matmul/group_matmul/group_matmul_direct.hpp:406-577). */
typedef struct b200dnn_moe_expert_t {
  int32_t M;             /* rows routed to this expert (0 allowed: skipped) */
  int32_t wei_dt;        /* 0 or B200DNN_S8: s8 weights with scales, both GEMMs on dynamically quantised rows;
                          * B200DNN_BF16: bf16 weights, no quantisation and no scales (the reference's bf16:bf16:bf16 fused
                          * MoE, matmul/group_matmul/custom_kernel/ukernel/bf16_microkernel.hpp).  One value for all experts. */
  const void *src;       /* [M,K] bf16 rows gathered by the caller, row stride lda */
  int64_t lda;
  const void *w13;       /* s8 | bf16 [K, 2I] = [gate | up] (transB: [2I, K]) */
  int64_t ldb13;
  const float *w13_scale; /* [2I] (s8 weights) */
  const void *w2;        /* s8 | bf16 [I, H] (transB: [H, I]) */
  int64_t ldb2;
  const float *w2_scale; /* [H] (s8 weights) */
  void *dst_down;        /* [M,H] bf16, row stride ldc_down.  NULL (b200dnn_fused_moe only): the result is written back
                          * into `src` with row stride lda, the reference's src-reuse mode
                          * (matmul/group_matmul/group_matmul_direct.hpp:500-566); lda >= H then */
  int64_t ldc_down;
  const void *bias13;    /* optional bias of the first GEMM, [2I] in the caller's column order, added before the activation
                          * (matmul/group_matmul/custom_kernel/ukernel/int8_microkernel.cpp:161-177) */
  int32_t bias13_dt;     /* f32 | bf16 */
  int32_t reserved2;
  const void *bias2;     /* optional bias of the second GEMM, [H] (grp_matmul_fused_moe_params::bias_down) */
  int32_t bias2_dt;
  int32_t reserved3;
  void *dst_op1;         /* optional (b200dnn_fused_moe only): the activated output of the first GEMM, [M,I] bf16 with row
                          * stride ldc_op1, which the reference leaves in the caller's dst[] (group_matmul_direct.hpp:489-497) */
  int64_t ldc_op1;
} b200dnn_moe_expert_t;

/* group_matmul_direct with fused_moe + gated_act (+ optional moe_postop), dynamic per-token INT8
 * on both GEMMs (matmul/group_matmul/group_matmul_fused_moe.cpp:1131, data flow :906-1078):
 * per expert  quant(src) -> GEMM(w13) -> gated act -> bf16 -> quant -> GEMM(w2) -> dst_down,
 * then, if row_ptrs != NULL, the weighted top-k reduce into `out`.
 * K = hidden size, I = expert FFN width (N of the first GEMM is 2*I), H = output width. */
B200DNN_API int32_t b200dnn_fused_moe(int32_t num_experts, const b200dnn_moe_expert_t *experts, int32_t K, int32_t I,
                          int32_t H, int32_t transB, int32_t act, int32_t weights_const,
                          const void *const *row_ptrs, const float *topk_weights, int32_t num_tokens,
                          int32_t topk, void *out, int64_t ld_out, void *stream);

/* Router + permutation front end.  Has NO counterpart in the reference: the reference's callers do
 * this themselves before group_matmul_direct (examples/lowoha_group_matmul_example.cpp:273-300).
 * logits [T,E] f32 -> softmax -> top-k (ties to the lower expert id) -> renormalised weights;
 * also returns the per-expert row counts and, per (token,k) slot, the row index inside the
 * stable expert-sorted order.  All outputs may be NULL except ids. */
B200DNN_API int32_t b200dnn_moe_route(const float *logits, int32_t T, int32_t E, int32_t topk, int32_t renorm,
                          int32_t *ids, float *weights, int32_t *expert_counts, int32_t *slot_to_row,
                          void *stream);

/* End-to-end MoE layer on one GPU built from the pieces above, with the token gather fused into
 * the first quantisation and the un-permute fused into the weighted reduce:
 * x [T,K] bf16, logits [T,E] f32, per-expert weights as in b200dnn_moe_expert_t (M/src/dst_down
 * ignored), optional shared experts appended after the E routed ones (applied to every token with
 * weight 1).  out [T,H] bf16. */
B200DNN_API int32_t b200dnn_moe_layer(const void *x, int64_t ldx, const float *logits, int32_t T, int32_t E,
                          int32_t num_shared, int32_t topk, const b200dnn_moe_expert_t *experts,
                          int32_t K, int32_t I, int32_t H, int32_t transB, int32_t act, void *out,
                          int64_t ld_out, void *stream);

/* ---- Building blocks of the expert-parallel MoE (experts sharded over GPUs).  No counterpart in the
 * reference, which is a single-process CPU library; the exchange of tokens between GPUs (NCCL
 * all-to-all) happens in the caller between these calls.  Device pointers only. ---- */

/* Stable counting sort of (token,k) slots by an integer key in [0,nkeys): counts per key and, for
 * every slot, its row in key-sorted order.  With key = (destination rank, local expert) this gives
 * the send order of the dispatch. */
B200DNN_API int32_t b200dnn_moe_sort_slots(const int32_t *keys, int32_t nslots, int32_t nkeys, int32_t *counts,
                                           int32_t *slot_to_row, void *stream);
/* Per-token quantisation (as b200dnn_quant_per_token) of gathered rows: output row r is source row
 * row_src[r] / row_div of src [*, K] (row stride src_ld). */
B200DNN_API int32_t b200dnn_quant_per_token_gather(const void *src, int32_t src_dt, int64_t K, int64_t src_ld,
                                                   const int32_t *row_src, int32_t row_div, int64_t R, void *dst,
                                                   int64_t dst_ld, float *scale, void *stream);
/* Per-token quantisation of T source rows, each written to several output rows: source row t goes to the
 * rows dst_rows[t*n_dst + j], j < n_dst, of dst and scale (entries < 0 are skipped).  A token that is routed
 * to several experts is quantised once. */
B200DNN_API int32_t b200dnn_quant_per_token_scatter(const void *src, int32_t src_dt, int64_t K, int64_t src_ld,
                                                    const int32_t *dst_rows, int32_t n_dst, int64_t T, void *dst,
                                                    int64_t dst_ld, float *scale, void *stream);
/* Expert computation of the fused MoE on rows that arrive already quantised (s8 [R,lda] + f32 scale
 * per row): first GEMM + gated activation + requantisation + second GEMM, out bf16 [R,H].  Rows are
 * grouped: group g has group_rows[g] consecutive rows and uses experts[group_expert[g]] (host arrays). */
B200DNN_API int32_t b200dnn_moe_experts_s8(const void *rows_s8, int64_t lda, const float *row_scale, int32_t n_groups,
                                           const int32_t *group_rows, const int32_t *group_expert,
                                           const b200dnn_moe_expert_t *experts, int32_t K, int32_t I, int32_t H,
                                           int32_t transB, int32_t act, void *out, int64_t ld_out, void *stream);
/* Weighted reduce with row indices instead of pointers: out[t] = sum_j slot_weights[t,j] * rows[slot_rows[t,j]]. */
B200DNN_API int32_t b200dnn_moe_weighted_reduce_rows(const void *rows, int64_t ld_rows, const int32_t *slot_rows,
                                                     const float *slot_weights, int32_t num_tokens, int32_t nslots,
                                                     int32_t D, int32_t dt, void *out, int64_t ld_out, void *stream);

/* ---- N-column sharding of one large matmul_direct over the GPUs of a node (one process per GPU; no counterpart in
 * the reference).  Rank r computes the column block [n0, n1) of dst from its column block of the weight, the matching
 * slices of the per-channel weight scales, the bias and the binary post-op operands, and the whole (replicated) source:
 * no reduction, so every output element is the one a single GPU computes.  A GEMM narrower than 8 tiles of 256 columns
 * is not split (sharded = 0: every rank computes all of it).  Blocks are whole 128-column tiles. ---- */
B200DNN_API int32_t b200dnn_nshard_range(int64_t N, int32_t world, int32_t rank, int64_t *n0, int64_t *n1, int32_t *sharded);
/* id128: the bytes of b200dnn_ep_nccl_unique_id made on one rank, or nccl_comm: an existing ncclComm_t; both NULL: no
 * communicator (enough when the blocks are not gathered). */
B200DNN_API int32_t b200dnn_nshard_create(int32_t world, int32_t rank, const void *id128, void *nccl_comm, void **handle);
B200DNN_API int32_t b200dnn_nshard_destroy(void *handle);
/* desc describes the WHOLE problem, weights in the caller's layout ('n').  gather != 0: afterwards every rank holds the whole
 * dst (device memory; collective over the communicator, enqueued on `stream`). */
B200DNN_API int32_t b200dnn_matmul_nshard(void *handle, const b200dnn_matmul_t *desc, int32_t gather, void *stream);

/* ---- Expert-parallel fused MoE across the GPUs of one node, one process per GPU (or several handles in one process).
 * No counterpart in the reference (a single-process CPU library); the per-expert contract is group_matmul_direct's
 * (matmul/lowoha_matmul.hpp:204-223: independent experts, M_e = 0 allowed).  Routed expert e lives on rank expert_rank[e],
 * shared experts are replicated, tokens are data-parallel.  The token exchange is part of the library's own kernels
 * (stores and loads over peer memory); NCCL carries only the per-expert row counts and two barriers per layer.  The
 * result equals b200dnn_moe_layer on the same tokens bit for bit. ---- */
typedef struct b200dnn_ep_config_t {
  int32_t world, rank;          /* 1 <= world <= 8 */
  int32_t num_experts;          /* routed experts over all ranks (<= 256) */
  int32_t num_shared;           /* shared experts, applied to every token with weight 1 */
  int32_t topk;
  int32_t max_tokens;           /* largest T of a call on any rank: sizes the exchange buffers */
  int32_t K, I, H;              /* hidden size, expert FFN width, output width */
  int32_t transB, act;          /* as b200dnn_fused_moe */
  int32_t capacity_rows;        /* rows one rank accepts from one source rank; 0 = max_tokens * topk, which can never overflow */
  const int32_t *expert_rank;   /* host array [num_experts], owner of each routed expert; NULL = e % world */
} b200dnn_ep_config_t;
/* Allocates this rank's buffers on the current device (the only allocation of the layer).  All ranks must use the
 * same configuration apart from `rank`. */
B200DNN_API int32_t b200dnn_ep_create(const b200dnn_ep_config_t *cfg, void **handle);
B200DNN_API int32_t b200dnn_ep_destroy(void *handle);
B200DNN_API int32_t b200dnn_ep_local_expert_count(void *handle, int32_t *n_local);
/* Weights of this rank: its routed experts in ascending expert id, then the shared experts (M/src/dst_down ignored;
 * device or host weights, device scales).  Packed once and cached by address like every constant weight. */
B200DNN_API int32_t b200dnn_ep_set_experts(void *handle, const b200dnn_moe_expert_t *experts, int32_t n);
/* One process per GPU: rank 0 makes an id (128 bytes, an ncclUniqueId), the application carries it to the other ranks,
 * every rank connects (collective: creates the communicator unless nccl_comm, an ncclComm_t, is given, and opens the
 * peers' buffers through CUDA IPC). */
B200DNN_API int32_t b200dnn_ep_nccl_unique_id(void *id128);
B200DNN_API int32_t b200dnn_ep_connect_nccl(void *handle, const void *id128, void *nccl_comm);
/* All ranks in one process (handles[r] is rank r; same device, or devices with peer access). */
B200DNN_API int32_t b200dnn_ep_connect_local(void *const *handles, int32_t world);
/* One MoE layer for this rank's T tokens (collective over the ranks; T may differ per rank and may be 0):
 * x [T,K] bf16, logits [T,num_experts] f32 -> out [T,H] bf16.  Enqueues on `stream` and returns (device buffers). */
B200DNN_API int32_t b200dnn_moe_layer_ep(void *handle, const void *x, int64_t ldx, const float *logits, int32_t T, void *out,
                                         int64_t ld_out, void *stream);
/* The same for handles that share a process: every rank's phases in turn on one stream (no NCCL). */
B200DNN_API int32_t b200dnn_moe_layer_ep_local(void *const *handles, int32_t world, const void *const *x, int64_t ldx,
                                               const float *const *logits, const int32_t *T, void *const *out, int64_t ld_out,
                                               void *stream);
/* Rows every rank received in the last layer (routed + shared): the load imbalance as numbers.  Synchronises. */
B200DNN_API int32_t b200dnn_ep_rows_per_rank(void *handle, int32_t *rows, void *stream);
/* Waits for `stream`; failure when a kernel gave up a bounded wait, rows were dropped (capacity_rows too small) or
 * the communicator reports an asynchronous error (a rank that died). */
B200DNN_API int32_t b200dnn_ep_status(void *handle, void *stream);

/* Per-phase device times of b200dnn_moe_layer and b200dnn_moe_layer_ep calls on `stream` (CUDA events recorded by the
 * library itself; off by default).  b200dnn_phase_times waits for the stream and returns the mean milliseconds per call
 * over the calls made since timing was switched on (their number in *calls, which may be NULL): index 0 route + slot ranks, 1 count exchange, 2 quantise + dispatch, 3 barrier, 4 first GEMM with the gated
 * activation, 5 requantisation, 6 second GEMM, 7 barrier, 8 combine + weighted reduce. */
enum { B200DNN_PHASES = 9 };
B200DNN_API int32_t b200dnn_phase_timing(void *stream, int32_t enable);
B200DNN_API int32_t b200dnn_phase_times(void *stream, float *ms, int32_t n, int32_t *calls);

/* Measurement aid, no reference counterpart: the issue-bound rate of the int8 tensor-core instruction the GEMM
 * kernels use (tcgen05.mma kind::i8, M128 x N256 x K32, operands resident in shared memory, no global loads), on every
 * SM at once.  `launches` launches of `iters` K-blocks each run back to back; *ms is their device time, *ops the
 * operations performed (2 per multiply-add), so ops / ms / 1e9 is TOPS.  A short run gives the burst rate, a run of
 * seconds the rate under the power cap. */
B200DNN_API int32_t b200dnn_measure_int8_peak(int32_t iters, int32_t launches, float *ms, double *ops, void *stream);

/* Drops every cached packed weight / staged buffer: the counterpart of the reference's cache
 * clearing between tests (gtests/gtest_utils.cpp:77-118) and clear_fused_moe_scratch()
 * (matmul/group_matmul/group_matmul_direct.hpp:683). */
B200DNN_API int32_t b200dnn_clear_caches(void);

/* Calls that take device pointers only enqueue work and return before it has run.  This waits for `stream` and
 * reports whether any kernel of this library, since the last check, gave up on one of its bounded waits (it
 * then left without writing its outputs): success, or failure with the code in b200dnn_last_error().  Calls with
 * host buffers synchronise anyway and make this check themselves.  No reference counterpart (the reference is
 * synchronous). */
B200DNN_API int32_t b200dnn_stream_status(void *stream);

/* ---- normalization_direct (lowoha_operators/normalization/lowoha_normalization.hpp:98-107, norm_params in
 * lowoha_normalization_common.hpp:96-153): the operators on either side of the quantised GEMMs in a decoder layer.
 * The input is a [batch, norm_size] matrix (BatchNorm: [batch, num_channels, norm_size]); f32 and bf16 buffers (f16:
 * unimplemented); every pointer may be host or device memory.  norm_type uses the reference's values. ---- */
enum { B200DNN_NORM_LAYER = 0, B200DNN_NORM_BATCH = 1, B200DNN_NORM_RMS = 2, B200DNN_NORM_FUSED_ADD_RMS = 3 };
typedef struct b200dnn_norm_t {
  int32_t norm_type;
  int32_t use_scale, use_shift;   /* gamma / beta applied (beta is ignored by the two RMS forms) */
  float epsilon;
  int64_t batch, norm_size, num_channels;
  int32_t src_dt, dst_dt, gamma_dt, beta_dt;
  const void *input;
  void *output;                   /* may be NULL when only the quantised form is wanted */
  const void *gamma, *beta;
  const float *running_mean, *running_var;   /* BatchNorm */
  void *residual;                 /* fused-add RMSNorm: updated in place to residual + input (rounded to src_dt) */
  /* No counterpart in the reference: the normalised row, rounded to dst_dt, also leaves as per-token symmetric s8 with
   * one f32 scale per row (the arithmetic of b200dnn_quant_per_token), in the same pass.  Both NULL: off. */
  void *quant_dst; int64_t quant_ld; float *quant_scale;
} b200dnn_norm_t;
B200DNN_API int32_t b200dnn_normalization(const b200dnn_norm_t *desc, void *stream);

/* ---- sdpa_direct (lowoha_operators/sdpa/lowoha_sdpa.hpp:48-55, sdpa_params in lowoha_sdpa_common.hpp:57-103):
 * output = softmax(Q K^T * scale + mask) V per (batch, head); bf16 tensors with [batch, head, seq, dim] strides (dim stride
 * 1), optional additive mask (f32 | bf16, 2-D [seq, kv] or 4-D broadcastable), causal masking (key j > query i), scale 0 =
 * 1/sqrt(head_dim).  Computed in the form of the reference's BMM backend (scores, softmax, P V as three steps per head). ---- */
typedef struct b200dnn_sdpa_t {
  int64_t batch, num_heads, seq_len, kv_seq_len, head_dim;
  int64_t q_stride[4], k_stride[4], v_stride[4], o_stride[4];   /* elements, order b, h, s, d */
  int32_t mask_ndims; int32_t is_causal;
  int64_t mask_sizes[4], mask_strides[4];                        /* the first mask_ndims entries */
  int32_t qkv_dt, out_dt, mask_dt; int32_t reserved;
  double scale, dropout_p;
  const void *query, *key, *value, *attn_mask;
  void *output;
} b200dnn_sdpa_t;
B200DNN_API int32_t b200dnn_sdpa(const b200dnn_sdpa_t *desc, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* B200DNN_H */
