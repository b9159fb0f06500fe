// Host side of the group-scaled INT8 matmul (per-group scales, W4A8): detection, the reference's contract checks
// (matmul/lowoha_matmul_utils.cpp:72-178), weight preparation with the weight cache, source quantisation and the launch
// of gs_gemm_kernel.  Included by b200dnn.cu in front of the C ABI.
#pragma once
#include "gs_gemm.cuh"

namespace {

// weight-cache layout codes stored in the `gated` slot of the cache key
constexpr int kGsLayoutS8 = 16, kGsLayoutS4 = 17;

// A descriptor takes this path when its weights are 4-bit or one of its scales has more than one value per row /
// column ({M,G} source scales, {G,N} weight scales).
inline bool is_group_scaled(const b200dnn_matmul_t *d) {
  if (d->wei_dt == B200DNN_S4) return true;
  if (d->N > 0 && d->wei_scale.count > d->N) return true;
  if (d->M > 0 && d->src_scale.count > d->M) return true;
  return false;
}

struct GsPlan { int G; int gs; bool w4; bool dyn; int src_cols; bool src_per_tensor; };

int32_t validate_group_scaled(const b200dnn_matmul_t *d, GsPlan *p) {
  const int M = d->M, N = d->N, K = d->K;
  B2_CHECK(d->src && d->weight && d->dst, B200DNN_FAILURE, "null src, weight or dst");
  B2_CHECK(M > 0 && N > 0 && K > 0, B200DNN_FAILURE, "M, N, K must be positive (got %d, %d, %d)", M, N, K);
  B2_CHECK(d->lda >= K && d->ldc >= N && d->ldb >= (d->transB ? K : N), B200DNN_FAILURE, "leading dimension smaller than the row length");
  B2_CHECK(d->wei_dt == B200DNN_S8 || d->wei_dt == B200DNN_S4, B200DNN_UNIMPLEMENTED, "weight dtype %d (s8 and s4 are implemented)", d->wei_dt);
  B2_CHECK(d->wei_format == 'n' || d->wei_format == 0, B200DNN_UNIMPLEMENTED, "prepacked weights are not implemented for per-group scales / s4 weights");
  B2_CHECK(d->n_postops >= 0 && d->n_postops <= B200DNN_MAX_POSTOPS, B200DNN_FAILURE, "too many post-ops");
  const bool w4 = d->wei_dt == B200DNN_S4, dyn = d->dynamic_quant != 0;
  if (w4) {
    // W4A8 contract, in the reference's words (lowoha_matmul_utils.cpp:72-100)
    B2_CHECK(d->src_dt != B200DNN_S8, B200DNN_FAILURE, "W4A8 requires bf16 source with dynamic_quant=true (pre-quantized s8 source is not supported)");
    B2_CHECK(d->src_dt != B200DNN_U8, B200DNN_FAILURE, "S4 weights do not support u8 source; W4A8 requires bf16 source with dynamic_quant=true");
    B2_CHECK(dyn && d->src_dt == B200DNN_BF16, B200DNN_UNIMPLEMENTED, "s4 weights are implemented for W4A8 only (bf16 source, dynamic_quant)");
    B2_CHECK(d->dst_dt == B200DNN_BF16, B200DNN_FAILURE, "W4A8 dynamic quantization requires bf16 output");
  } else if (dyn) {
    B2_CHECK(d->src_dt == B200DNN_BF16 || d->src_dt == B200DNN_F32, B200DNN_UNIMPLEMENTED, "dynamic quantisation takes a bf16 or f32 source");
  } else {
    B2_CHECK(d->src_dt == B200DNN_S8, B200DNN_FAILURE, "per-group source scales need a symmetric s8 source");
  }
  B2_CHECK(d->dst_dt == B200DNN_BF16 || d->dst_dt == B200DNN_F32, B200DNN_UNIMPLEMENTED, "per-group scales need a bf16 or f32 destination");
  B2_CHECK(!d->src_zp.buff, B200DNN_FAILURE, "per-group / W4A8 supports symmetric quantization only");
  // weight scales {G,N}
  const auto &ws = d->wei_scale;
  B2_CHECK(ws.buff, B200DNN_FAILURE, "per-group / W4A8 requires quant_params.wei_scale.buff");
  B2_CHECK(ws.dt == B200DNN_F32 || ws.dt == B200DNN_BF16, B200DNN_FAILURE, "weight scale supports only f32 or bf16 data type");
  B2_CHECK(ws.count >= N && ws.count % N == 0, B200DNN_FAILURE, "weight scale dims must be {G,N} (count %lld, N %d)", (long long)ws.count, N);
  const int64_t G = ws.count / N;
  B2_CHECK(K % G == 0, B200DNN_FAILURE, "K must be divisible by the weight group count (K=%d, G=%lld)", K, (long long)G);
  const int64_t gs = K / G;
  B2_CHECK(gs % 4 == 0, B200DNN_FAILURE, "K/G must be a multiple of 4 (got group_size=%lld)", (long long)gs);
  B2_CHECK(gs == 4 || gs == 8 || gs == 16 || gs % 32 == 0, B200DNN_UNIMPLEMENTED,
           "group sizes 4, 8, 16 and multiples of 32 are implemented (got %lld)", (long long)gs);
  // source scales {M,G}, or {M,1} when the library quantises per token
  const auto &ss = d->src_scale;
  int src_cols;
  bool per_tensor = false;
  if (ss.count == (int64_t)M * G) src_cols = (int)G;
  else if (dyn && (ss.count == M || ss.count == 0)) src_cols = 1;
  else if (dyn && ss.count == 1) { src_cols = 1; per_tensor = true; }      // {1,1}: one scale for the whole source
  else return fail(B200DNN_FAILURE, "source scale dims must be {M,G}%s (count %lld, M %d, G %lld)", dyn ? " or {M,1}" : "", (long long)ss.count, M, (long long)G);
  if (!dyn) B2_CHECK(ss.buff && ss.dt == B200DNN_F32, ss.buff ? B200DNN_UNIMPLEMENTED : B200DNN_FAILURE, "per-group source scales: an f32 buffer is required");
  else B2_CHECK(!ss.buff || ss.dt == B200DNN_F32, B200DNN_UNIMPLEMENTED, "dynamic per-group source scales are written as f32");
  B2_CHECK(!d->bias || d->bias_dt == B200DNN_F32 || d->bias_dt == B200DNN_BF16, B200DNN_UNIMPLEMENTED, "bias dtype %d", d->bias_dt);
  for (int i = 0; i < d->n_postops; ++i) {
    const b200dnn_postop_t &po = d->postops[i];
    switch (po.type) {
    case PO_RELU: case PO_LEAKY_RELU: case PO_GELU_TANH: case PO_GELU_ERF: case PO_SIGMOID: case PO_SWISH: case PO_TANH: case PO_ELU: case PO_CLIP: break;
    case PO_BINARY_ADD: case PO_BINARY_MUL:
      B2_CHECK(po.buff && (po.dt == B200DNN_F32 || po.dt == B200DNN_BF16), B200DNN_FAILURE, "binary post-op needs an f32 or bf16 operand");
      B2_CHECK(po.ld == 0 || po.ld >= N, B200DNN_FAILURE, "binary post-op leading dimension");
      break;
    case PO_MISH: return fail(B200DNN_FAILURE, "mish is rejected on the INT8 path");
    default: return fail(B200DNN_UNIMPLEMENTED, "post-op %d is not implemented", po.type);
    }
  }
  p->G = (int)G; p->gs = (int)gs; p->w4 = w4; p->dyn = dyn; p->src_cols = src_cols; p->src_per_tensor = per_tensor;
  return B200DNN_SUCCESS;
}

// blocked s8 / s4 copy of the weight (layout in gs_gemm.cuh), cached per (pointer, shape, layout) like the packed tcgen05 weights.
int32_t resolve_gs_weight(const b200dnn_matmul_t *d, bool w4, int64_t Kp, cudaStream_t st, PackedWeight *pw) {
  DeviceShared &D = *rt().shared;
  const int K = d->K, N = d->N;
  auto key = std::make_tuple(d->weight, (int64_t)K, (int64_t)N, (int64_t)d->ldb, (int)d->transB, w4 ? kGsLayoutS4 : kGsLayoutS8);
  const bool cache = d->weights_const && env_int("ZENDNNL_MATMUL_WEIGHT_CACHE", 1) != 0;
  std::unique_lock<std::mutex> lk(D.cache_mu, std::defer_lock);
  if (cache) {
    lk.lock();
    auto it = D.wcache.find(key);
    if (it != D.wcache.end()) { B2_TRY(wait_ready(it->second, st)); *pw = it->second; return B200DNN_SUCCESS; }
  }
  const int64_t wrows = d->transB ? N : K, wcols = d->transB ? K : N;
  const size_t src_bytes = w4 ? (size_t)(((wrows - 1) * d->ldb + wcols + 1) / 2) : span_bytes(wrows, wcols, d->ldb, B200DNN_S8);
  const void *w_dev = nullptr;
  B2_TRY(stage_in(d->weight, src_bytes, st, &w_dev));
  const int64_t np8 = (N + 7) / 8 * 8;
  const size_t bytes = (size_t)np8 * (w4 ? Kp / 2 : Kp);
  void *buf = nullptr;
  if (cache) B2_CUDA(cudaMalloc(&buf, bytes));
  else { buf = rt().ws.alloc(bytes); B2_CHECK(buf, B200DNN_FAILURE, "workspace allocation failed"); }
  const int64_t threads = (Kp / 2) * np8;
  gs_pack_weight_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>((const uint8_t *)w_dev, d->ldb, d->transB, w4 ? 1 : 0, K, N, (int)Kp, (uint8_t *)buf);
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  *pw = PackedWeight{};
  pw->wt = (const int8_t *)buf; pw->K = K; pw->N = N; pw->Kp = Kp; pw->Np = N; pw->gated = w4 ? kGsLayoutS4 : kGsLayoutS8;
  if (cache) { pw->owned = buf; B2_TRY(mark_ready(*pw, st)); D.wcache.emplace(key, *pw); }
  return B200DNN_SUCCESS;
}

// one f32 value replicated n times (a per-tensor source scale as the per-row scales the kernels read)
__global__ void gs_fill_f32_kernel(float *dst, const float *value, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = *value;
}

template <int NT, int CH>
int32_t launch_gs_t(const GsGemmArgs &a, const EpiParams &epi, cudaStream_t st) {
  dim3 grid((unsigned)((a.N + NT * 8 - 1) / (NT * 8)), (unsigned)((a.M + a.MT * 16 - 1) / (a.MT * 16)));
  if (a.w4) gs_gemm_kernel<NT, CH, true><<<grid, kGsWarps * 32, 0, st>>>(a, epi);
  else gs_gemm_kernel<NT, CH, false><<<grid, kGsWarps * 32, 0, st>>>(a, epi);
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  return B200DNN_SUCCESS;
}

// The decode form: M <= 16, at least eight groups of a multiple of 32 elements, f32 weight scales, even N, activations
// that leave room for a ring of at least four slots per lane in shared memory.
template <int CH, bool W4, int R>
int32_t launch_gs_decode_r(const GsDecodeArgs &da, const EpiParams &epi, size_t smem, int grid, cudaStream_t st) {
  B2_TRY(ensure_max_smem((const void *)gs_decode_kernel<CH, W4, R>, (int)smem));
  gs_decode_kernel<CH, W4, R><<<grid, kGsWarps * 32, smem, st>>>(da, epi);
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  return B200DNN_SUCCESS;
}
template <int CH, bool W4>
int32_t launch_gs_decode_t(const GsGemmArgs &a, const EpiParams &epi, cudaStream_t st, bool *done) {
  *done = false;
  GsDecodeArgs da{};
  da.g = a;
  da.rows_staged = a.M;
  // row stride of the staged activations: the lanes of a quarter warp (16-byte loads) or half warp (8-byte loads) read
  // distinct bank groups when the stride is 64 (32) bytes off a multiple of 128
  da.a_stride = CH == 128 ? a.Kp + 16 : (CH == 64 ? (a.Kp % 128 == 64 ? a.Kp : a.Kp + 64) : a.Kp + 32);   // (128-k chunks: two 16-byte loads, 32 bytes apart per lane)
  constexpr int slot_w = 32 * 2 * (W4 ? CH / 8 : CH / 4), slot_s = 32 * 2 * 8;     // bytes per warp and ring slot (see the kernel)
  const int chunks = a.gs / CH;
  const size_t fixed = (size_t)da.rows_staged * da.a_stride + (size_t)((da.rows_staged * a.sa_cols + 3) & ~3) * 4 +
                       (size_t)2 * kGsWarps * 16 * 17 * 4;
  // ring depth and CTAs per SM: whatever keeps the most copies in flight per SM (ties: more CTAs, which also evens out the tiles)
  const size_t sm_bytes = (size_t)226 * 1024;     // per SM, with 1 KiB per CTA reserved by the system
  int best_r = 0, best_ctas = 0, best_score = -1;
  size_t best_smem = 0;
  const int items_per_tile = ((a.G + kGsWarps - 1) / kGsWarps) * chunks;      // of one warp: more in flight than that spans tiles
  for (int r : {16, 12, 8, 6, 4}) {
    const int rs = (r + chunks - 1) / chunks + 1;
    const size_t smem = fixed + (size_t)kGsWarps * ((size_t)r * slot_w + (size_t)rs * slot_s);
    if (smem > (size_t)224 * 1024) continue;
    int ctas = (int)(sm_bytes / (smem + 1024));
    if (ctas > (CH == 128 ? 2 : 3)) ctas = CH == 128 ? 2 : 3;      // 72-88 registers x 256 threads (87-96 with 128-k chunks)
    const int score = ctas * ((r - 1) < items_per_tile ? (r - 1) : items_per_tile);
    if (score > best_score || (score == best_score && ctas > best_ctas)) { best_score = score; best_r = r; best_ctas = ctas; best_smem = smem; }
  }
  if (best_r == 0) return B200DNN_SUCCESS;        // the general kernel takes it
  da.scale_slots = (best_r + chunks - 1) / chunks + 1;
  const size_t smem = best_smem;
  const int tiles = (a.N + 15) / 16;
  // persistent CTAs (one tile per CTA, left to the hardware's scheduler, measured slower: 18.3 against 15.4 us at M = 1, K = 4096, N = 11008)
  const int slots = rt().sm_count * best_ctas;
  const int grid = tiles < slots ? tiles : slots;
  switch (best_r) {
  case 16: B2_TRY((launch_gs_decode_r<CH, W4, 16>(da, epi, smem, grid, st))); break;
  case 12: B2_TRY((launch_gs_decode_r<CH, W4, 12>(da, epi, smem, grid, st))); break;
  case 8: B2_TRY((launch_gs_decode_r<CH, W4, 8>(da, epi, smem, grid, st))); break;
  case 6: B2_TRY((launch_gs_decode_r<CH, W4, 6>(da, epi, smem, grid, st))); break;
  default: B2_TRY((launch_gs_decode_r<CH, W4, 4>(da, epi, smem, grid, st))); break;
  }
  *done = true;
  return B200DNN_SUCCESS;
}

// The whole call; the caller holds the call guard (B2_ENTER) and has checked is_group_scaled().
int32_t matmul_group_scaled(const b200dnn_matmul_t *d, cudaStream_t st) {
  Runtime &R = rt();
  GsPlan p;
  B2_TRY(validate_group_scaled(d, &p));
  const int M = d->M, N = d->N, K = d->K;
  const int64_t Kp = round_up(K, 64);
  PackedWeight pw;
  B2_TRY(resolve_gs_weight(d, p.w4, Kp, st, &pw));

  // ---- epilogue operands
  EpiParams epi;
  fill_epi(d, &epi);
  const void *ws_dev = nullptr;
  B2_TRY(stage_in(d->wei_scale.buff, (size_t)d->wei_scale.count * dt_size(d->wei_scale.dt), st, &ws_dev));
  if (d->bias) { const void *b; B2_TRY(stage_in(d->bias, (size_t)N * dt_size(d->bias_dt), st, &b)); epi.bias = b; }
  for (int i = 0; i < d->n_postops; ++i) {
    const b200dnn_postop_t &po = d->postops[i];
    epi.po[i].type = po.type; epi.po[i].dt = po.dt; epi.po[i].ld = po.ld; epi.po[i].alpha = po.alpha; epi.po[i].beta = po.beta;
    epi.po[i].buff = nullptr;
    if (po.type == PO_BINARY_ADD || po.type == PO_BINARY_MUL) {
      const void *b;
      B2_TRY(stage_in(po.buff, po.ld ? span_bytes(M, N, po.ld, po.dt) : (size_t)N * dt_size(po.dt), st, &b));
      epi.po[i].buff = b;
    }
  }
  Staged o_dst;
  B2_TRY(stage_out(d->dst, span_bytes(M, N, d->ldc, d->dst_dt), st, &o_dst, d->ldc != N));
  epi.dst = o_dst.dev;

  const void *src_dev = nullptr;
  B2_TRY(stage_in(d->src, span_bytes(M, K, d->lda, d->src_dt), st, &src_dev));
  Staged o_scale; o_scale.copy_back = false;
  if (p.dyn) B2_TRY(stage_out(const_cast<void *>(d->src_scale.buff), (size_t)(p.src_per_tensor ? 1 : M * p.src_cols) * 4, st, &o_scale));

  GsGemmArgs a{};
  a.sa_cols = p.src_cols;
  a.W = (const uint8_t *)pw.wt; a.w4 = p.w4 ? 1 : 0;
  a.sw = ws_dev; a.sw_dt = d->wei_scale.dt;
  a.M = M; a.N = N; a.K = K; a.Kp = (int)Kp; a.gs = p.gs; a.G = p.G;
  a.MT = M <= 16 ? 1 : (M <= 32 ? 2 : (M <= 64 ? 4 : 8));
  const bool ch64 = p.gs % 64 == 0;

  // ---- source rows for the kernels that do not quantise themselves: s8 [M][Kp], zero padded, and f32 scales [M][src_cols]
  auto prepare_source = [&]() -> int32_t {
    int8_t *A = (int8_t *)R.ws.alloc((size_t)M * Kp);
    B2_CHECK(A, B200DNN_FAILURE, "workspace allocation failed");
    if (Kp != K) B2_CUDA(cudaMemsetAsync(A, 0, (size_t)M * Kp, st));
    const float *sa = nullptr;
    if (p.dyn && p.src_per_tensor) {
      // one dynamic scale for the whole source (the reference's per-tensor rule: abs-max over the finite values / 127, then
      // the static quantise; reorder/lowoha_reorder_utils.cpp:708-766), replicated per row for the kernels
      uint32_t *amax = (uint32_t *)R.ws.alloc(4);
      float *s1 = (float *)o_scale.dev;
      if (!s1) s1 = (float *)R.ws.alloc(4);
      float *sc = (float *)R.ws.alloc((size_t)M * 4);
      B2_CHECK(amax && s1 && sc, B200DNN_FAILURE, "workspace allocation failed");
      B2_CUDA(cudaMemsetAsync(amax, 0, 4, st));
      dim3 grid((unsigned)((K + 255) / 256), (unsigned)(M < 64 ? 1 : (M / 64 > 256 ? 256 : M / 64)));
      dim3 g2((unsigned)((K + 255) / 256), (unsigned)(M > 1024 ? 1024 : M));
      if (d->src_dt == B200DNN_BF16) {
        absmax_cols_kernel<uint16_t><<<grid, 256, 0, st>>>((const uint16_t *)src_dev, M, K, d->lda, 0, amax);
        scales_from_absmax_kernel<<<1, 32, 0, st>>>(amax, 1, s1);
        quant_static_kernel<uint16_t><<<g2, 256, 0, st>>>((const uint16_t *)src_dev, M, K, d->lda, s1, 1, nullptr, 0, A, B200DNN_S8, Kp);
      } else {
        absmax_cols_kernel<float><<<grid, 256, 0, st>>>((const float *)src_dev, M, K, d->lda, 0, amax);
        scales_from_absmax_kernel<<<1, 32, 0, st>>>(amax, 1, s1);
        quant_static_kernel<float><<<g2, 256, 0, st>>>((const float *)src_dev, M, K, d->lda, s1, 1, nullptr, 0, A, B200DNN_S8, Kp);
      }
      gs_fill_f32_kernel<<<(unsigned)((M + 255) / 256), 256, 0, st>>>(sc, s1, M);
      B2_LAUNCHED(); B2_LAUNCHED(); B2_LAUNCHED(); B2_LAUNCHED();
      B2_CUDA(cudaGetLastError());
      sa = sc;
    } else if (p.dyn) {
      const int64_t n_sc = (int64_t)M * p.src_cols;
      float *sc = (float *)o_scale.dev;
      if (!sc) { sc = (float *)R.ws.alloc((size_t)n_sc * 4); B2_CHECK(sc, B200DNN_FAILURE, "workspace allocation failed"); }
      RowQuantArgs qa{};
      qa.gather_div = 1; qa.scale = sc; qa.scale_dt = B200DNN_F32;
      if (p.src_cols == 1) {
        qa.src = src_dev; qa.src_ld = d->lda; qa.dst = A; qa.dst_ld = Kp; qa.K = K;
        B2_TRY(launch_quant_rows(qa, d->src_dt, M, st));
      } else {
        // every (row, group) is a row of gs elements; needs rows that follow each other without gaps
        const size_t esz = dt_size(d->src_dt);
        const void *xs = src_dev;
        if (d->lda != K) {
          void *x = R.ws.alloc((size_t)M * K * esz);
          B2_CHECK(x, B200DNN_FAILURE, "workspace allocation failed");
          B2_CUDA(cudaMemcpy2DAsync(x, (size_t)K * esz, src_dev, (size_t)d->lda * esz, (size_t)K * esz, (size_t)M, cudaMemcpyDeviceToDevice, st));
          xs = x;
        }
        int8_t *q = A;
        if (Kp != K) { q = (int8_t *)R.ws.alloc((size_t)M * K); B2_CHECK(q, B200DNN_FAILURE, "workspace allocation failed"); }
        qa.src = xs; qa.src_ld = p.gs; qa.dst = q; qa.dst_ld = p.gs; qa.K = p.gs;
        B2_TRY(launch_quant_rows(qa, d->src_dt, (int64_t)M * p.G, st));
        if (q != A) B2_CUDA(cudaMemcpy2DAsync(A, (size_t)Kp, q, (size_t)K, (size_t)K, (size_t)M, cudaMemcpyDeviceToDevice, st));
      }
      sa = sc;
    } else {
      B2_CUDA(cudaMemcpy2DAsync(A, (size_t)Kp, src_dev, (size_t)d->lda, (size_t)K, (size_t)M, cudaMemcpyDefault, st));
      const void *sp = nullptr;
      B2_TRY(stage_in(d->src_scale.buff, (size_t)M * p.src_cols * 4, st, &sp));
      sa = (const float *)sp;
    }
    a.A = A; a.lda = Kp; a.sa = sa;
    return B200DNN_SUCCESS;
  };

  // (the decode form addresses the weight and the scales with 32-bit offsets)
  if (M <= 16 && p.G >= kGsWarps && p.gs % 32 == 0 && d->wei_scale.dt == B200DNN_F32 && N % 2 == 0 &&
      (int64_t)(N + 8) * Kp < (int64_t)1 << 32 && (int64_t)p.G * N < (int64_t)1 << 30 &&
      (reinterpret_cast<uintptr_t>(ws_dev) & 7) == 0 && env_int("B200DNN_GS_DECODE", 1) != 0) {
    B2_TRY(prepare_source());
    bool done = false;
    int32_t rcd;
    const bool ch128 = p.gs % 128 == 0 && env_int("B200DNN_GS_CH128", 1) != 0;     // fewer, larger items per group
    if (p.w4) rcd = ch128 ? launch_gs_decode_t<128, true>(a, epi, st, &done) : ch64 ? launch_gs_decode_t<64, true>(a, epi, st, &done) : launch_gs_decode_t<32, true>(a, epi, st, &done);
    else rcd = ch128 ? launch_gs_decode_t<128, false>(a, epi, st, &done) : ch64 ? launch_gs_decode_t<64, false>(a, epi, st, &done) : launch_gs_decode_t<32, false>(a, epi, st, &done);
    B2_TRY(rcd);
    if (done) return finish_out({&o_dst, &o_scale}, st);
  } else B2_TRY(prepare_source());
  // few rows: narrower CTAs, so that a call with few rows still has a few CTAs per SM
  int32_t rc;
  if (M <= 16) rc = ch64 ? launch_gs_t<2, 64>(a, epi, st) : launch_gs_t<2, 32>(a, epi, st);
  else rc = ch64 ? launch_gs_t<4, 64>(a, epi, st) : launch_gs_t<4, 32>(a, epi, st);   // (eight column tiles per warp need a CTA's whole register file)
  B2_TRY(rc);
  return finish_out({&o_dst, &o_scale}, st);
}

}  // namespace
