// Fused MoE entry points: b200dnn_fused_moe (the reference's group_matmul_direct contract, rows
// gathered by the caller) and b200dnn_moe_layer (router + permutation in front, un-permute
// behind).  Included at the end of b200dnn.cu.
//
// Data flow per expert, as in the reference's dynamic-INT8 two-pass semantics
// (matmul/group_matmul/group_matmul_fused_moe.cpp:906-1078):
//   A1 = quant_per_token(src)                          one kernel over all experts' rows
//   Z  = bf16( act( dequant(A1 x W13) ) )              grouped tcgen05 GEMM, gated epilogue,
//                                                      per-row max |Z| collected with atomicMax
//   A2 = quant_per_token(Z) using that max             one kernel, Z read once
//   O  = bf16( dequant(A2 x W2) )                      grouped tcgen05 GEMM
//   out[t] = sum_k w[t,k] * O[row(t,k)]                weighted reduce
#pragma once

namespace {

int32_t grouped_gemm(const uint8_t *A, int64_t lda, int R, int N, int K, const std::vector<PackedWeight> &pws,
                     const int32_t *row_off_dev, const int32_t *tile_prefix_dev, const TcGroupDesc *groups_dev,
                     int m_tiles_bound, EpiParams epi, bool shared_dst, cudaStream_t st, int tile_rows = kTcBM, bool f16 = false) {
  Runtime &Rt = rt();
  const int G = (int)pws.size();
  TcGemmArgs ta{};
  ta.pair = tile_rows > kTcBM ? 1 : 0;  // tile_prefix_dev and m_tiles_bound count tiles of tile_rows rows
  ta.f16 = f16 ? 1 : 0;                 // bf16 form: lda and K count bytes, pws hold bf16 packs
  ta.shared_dst = shared_dst ? 1 : 0;   // no group carries its own destination
  ta.n_groups = G; ta.row_off = row_off_dev; ta.tile_prefix = tile_prefix_dev; ta.groups = groups_dev;
  // one tensor map per expert, in device memory
  const PackedWeight &p0 = pws[0];
  const int BN = pick_bn(m_tiles_bound, N, Rt.sm_count, p0.gated, ta.pair);
  std::vector<CUtensorMap> maps(G);
  for (int g = 0; g < G; ++g) {
    B2_CHECK(pws[g].Kp == p0.Kp && pws[g].Np == p0.Np && pws[g].gated == p0.gated, B200DNN_UNIMPLEMENTED,
             "experts of one grouped GEMM must share K and N");
    B2_TRY(make_map_wt(&maps[g], pws[g].wt, (uint64_t)p0.Kp, (uint64_t)p0.Np, (uint32_t)(ta.pair ? BN / 2 : BN)));
  }
  void *maps_dev = nullptr;
  B2_TRY(cached_blob(maps.data(), sizeof(CUtensorMap) * G, st, &maps_dev));
  ta.maps_b = (const CUtensorMap *)maps_dev;
  // launch_tc picks the same BN from the same inputs
  return launch_tc(A, lda, false, R, N, K, p0, ta, epi, m_tiles_bound, st);
}

struct ExpertWeightsIn {
  const void *w13; int64_t ldb13; const float *s13; const void *w2; int64_t ldb2; const float *s2;
  const void *b13 = nullptr; int32_t b13_dt = 0; const void *b2 = nullptr; int32_t b2_dt = 0;   // optional biases
  int32_t wei_dt = 0;
};
inline ExpertWeightsIn expert_in(const b200dnn_moe_expert_t &e) {
  ExpertWeightsIn w{e.w13, e.ldb13, e.w13_scale, e.w2, e.ldb2, e.w2_scale};
  w.b13 = e.bias13; w.b13_dt = e.bias13_dt; w.b2 = e.bias2; w.b2_dt = e.bias2_dt;
  w.wei_dt = e.wei_dt;
  return w;
}

// rows of a bf16 matrix copied to their slots: source row r goes to the rows scatter[r*n + j] of dst (entries < 0 skipped),
// or, gather form, output row r comes from source row gather[r] / div.  One CTA per source (scatter) or output (gather) row.
__global__ void __launch_bounds__(256) moe_place_rows_bf16_kernel(const uint16_t *src, int64_t src_ld, const int32_t *scatter, int n,
                                                                  const int32_t *gather, int div, uint16_t *dst, int64_t dst_ld, int K) {
  const int r = blockIdx.x;
  const uint16_t *s;
  if (gather) {
    const int g = gather[r];
    if (g < 0) return;
    s = src + (int64_t)(g / div) * src_ld;
    uint16_t *d = dst + (int64_t)r * dst_ld;
    for (int k = threadIdx.x; k < K; k += blockDim.x) d[k] = s[k];
    return;
  }
  s = src + (int64_t)r * src_ld;
  const bool vec = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0 && src_ld % 8 == 0 && dst_ld % 8 == 0 && K % 8 == 0;
  if (vec) {
    for (int k = threadIdx.x; k < K / 8; k += blockDim.x) {
      const uint4 v = reinterpret_cast<const uint4 *>(s)[k];
      for (int j = 0; j < n; ++j) {
        const int row = scatter[r * n + j];
        if (row >= 0) reinterpret_cast<uint4 *>(dst + (int64_t)row * dst_ld)[k] = v;
      }
    }
  } else {
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
      const uint16_t v = s[k];
      for (int j = 0; j < n; ++j) {
        const int row = scatter[r * n + j];
        if (row >= 0) dst[(int64_t)row * dst_ld + k] = v;
      }
    }
  }
}

// bf16 weights: no quantisation.  X (rows in expert order, bf16) -> GEMM(w13) + gated activation -> Z bf16 -> GEMM(w2) -> O,
// both GEMMs on the tcgen05 kernel's bf16 form with f32 accumulation
// (reference: matmul/group_matmul/custom_kernel/ukernel/bf16_microkernel.hpp, gated epilogue on the f32 accumulators).
int32_t moe_core_bf16(int G, const std::vector<ExpertWeightsIn> &ew, int K, int I, int H, int transB, int act, int weights_const,
                      RowQuantArgs qa, int32_t src_dt, int R, const int32_t *row_off_dev, const int32_t *tile_prefix_dev,
                      int m_tiles_bound, const std::vector<void *> *dst_down_dev, const std::vector<int64_t> *ldc_down,
                      void **O_out, int64_t *ldO_out, cudaStream_t st, void *O_given, int tile_rows, const uint16_t **Z_out) {
  Runtime &Rt = rt();
  B2_CHECK(src_dt == B200DNN_BF16, B200DNN_UNIMPLEMENTED, "bf16 experts take bf16 rows");
  B2_CHECK(!qa.scatter_peer && !qa.n_rows_dev, B200DNN_UNIMPLEMENTED, "the expert-parallel exchange is built for s8 experts");
  const int gated = act == ACT_SWIGLU_OAI ? 2 : 1;
  std::vector<PackedWeight> p13(G), p2(G);
  std::vector<TcGroupDesc> g13(G), g2(G);
  int32_t b13_dt = 0, b2_dt = 0;
  for (int g = 0; g < G; ++g) {
    B2_CHECK(ew[g].w13 && ew[g].w2, B200DNN_FAILURE, "expert %d: null weight", g);
    B2_TRY(resolve_bf16_weight(ew[g].w13, K, 2 * (int64_t)I, ew[g].ldb13, transB, gated, weights_const, st, &p13[g]));
    B2_TRY(resolve_bf16_weight(ew[g].w2, I, H, ew[g].ldb2, transB, 0, weights_const, st, &p2[g]));
    const void *b13 = nullptr, *b2 = nullptr;
    if (ew[g].b13) {
      B2_CHECK(ew[g].b13_dt == B200DNN_F32 || ew[g].b13_dt == B200DNN_BF16, B200DNN_UNIMPLEMENTED, "expert %d: bias dtype %d", g, ew[g].b13_dt);
      B2_CHECK(b13_dt == 0 || b13_dt == ew[g].b13_dt, B200DNN_UNIMPLEMENTED, "the experts' first-GEMM biases must share one dtype");
      b13_dt = ew[g].b13_dt;
      B2_TRY(stage_in(ew[g].b13, (size_t)2 * I * dt_size(b13_dt), st, &b13));
    }
    if (ew[g].b2) {
      B2_CHECK(ew[g].b2_dt == B200DNN_F32 || ew[g].b2_dt == B200DNN_BF16, B200DNN_UNIMPLEMENTED, "expert %d: down bias dtype %d", g, ew[g].b2_dt);
      B2_CHECK(b2_dt == 0 || b2_dt == ew[g].b2_dt, B200DNN_UNIMPLEMENTED, "the experts' second-GEMM biases must share one dtype");
      b2_dt = ew[g].b2_dt;
      B2_TRY(stage_in(ew[g].b2, (size_t)H * dt_size(b2_dt), st, &b2));
    }
    g13[g] = TcGroupDesc{nullptr, nullptr, b13, nullptr, 0};
    g2[g] = TcGroupDesc{nullptr, nullptr, b2, dst_down_dev ? (*dst_down_dev)[g] : nullptr, ldc_down ? (*ldc_down)[g] : 0};
  }
  void *g13_dev, *g2_dev;
  B2_TRY(cached_blob(g13.data(), sizeof(TcGroupDesc) * G, st, &g13_dev));
  if (dst_down_dev) B2_TRY(upload_blob(g2.data(), sizeof(TcGroupDesc) * G, st, &g2_dev));
  else B2_TRY(cached_blob(g2.data(), sizeof(TcGroupDesc) * G, st, &g2_dev));

  // 1. rows in expert order, at a pitch the copy engine accepts
  const int64_t Kq = round_up(K, 8);
  const uint16_t *X = (const uint16_t *)qa.src; int64_t ldx = qa.src_ld;
  const bool placed = qa.scatter || qa.gather;
  if (placed || ldx % 8 != 0 || (reinterpret_cast<uintptr_t>(X) & 15) != 0) {
    uint16_t *Xs = (uint16_t *)Rt.ws.alloc((size_t)R * Kq * 2);
    B2_CHECK(Xs, B200DNN_FAILURE, "workspace allocation failed");
    if (qa.scatter)
      moe_place_rows_bf16_kernel<<<(unsigned)qa.scatter_rows, 256, 0, st>>>(X, ldx, qa.scatter, qa.scatter_n, nullptr, 1, Xs, Kq, K);
    else if (qa.gather)
      moe_place_rows_bf16_kernel<<<(unsigned)R, 256, 0, st>>>(X, ldx, nullptr, 0, qa.gather, qa.gather_div, Xs, Kq, K);
    else B2_CUDA(cudaMemcpy2DAsync(Xs, (size_t)Kq * 2, X, (size_t)ldx * 2, (size_t)K * 2, (size_t)R, cudaMemcpyDeviceToDevice, st));
    if (placed) { B2_LAUNCHED(); B2_CUDA(cudaGetLastError()); }
    X = Xs; ldx = Kq;
  }
  rt().mark(2);

  // 2. first GEMM with the gated epilogue -> Z (bf16, [R, I])
  uint16_t *Z = (uint16_t *)Rt.ws.alloc((size_t)R * I * 2);
  B2_CHECK(Z, B200DNN_FAILURE, "workspace allocation failed");
  EpiParams e1{};
  e1.dst = Z; e1.ldc = I; e1.dst_dt = B200DNN_BF16; e1.gated_act = act; e1.gated_I = I; e1.bias_dt = b13_dt;
  B2_TRY(grouped_gemm((const uint8_t *)X, ldx * 2, R, 2 * I, 2 * K, p13, row_off_dev, tile_prefix_dev, (const TcGroupDesc *)g13_dev,
                      m_tiles_bound, e1, true, st, tile_rows, true));
  rt().mark(4);

  // 3. second GEMM reads Z as it is -> O
  uint16_t *O = (uint16_t *)O_given;
  if (!dst_down_dev && !O) { O = (uint16_t *)Rt.ws.alloc((size_t)R * H * 2); B2_CHECK(O, B200DNN_FAILURE, "workspace allocation failed"); }
  EpiParams e2{};
  e2.dst = O; e2.ldc = H; e2.dst_dt = B200DNN_BF16; e2.bias_dt = b2_dt;
  B2_TRY(grouped_gemm((const uint8_t *)Z, (int64_t)I * 2, R, H, 2 * I, p2, row_off_dev, tile_prefix_dev, (const TcGroupDesc *)g2_dev,
                      m_tiles_bound, e2, dst_down_dev == nullptr, st, tile_rows, true));
  rt().mark(6);
  if (Z_out) *Z_out = Z;
  if (O_out) { *O_out = O; *ldO_out = H; }
  return B200DNN_SUCCESS;
}

// Shared core: rows already laid out expert by expert in device memory as the gather described by qa.
int32_t moe_core(int G, const std::vector<ExpertWeightsIn> &ew, int K, int I, int H, int transB, int act, int weights_const,
                 RowQuantArgs qa, int32_t src_dt, int R, const int32_t *row_off_dev, const int32_t *tile_prefix_dev,
                 int m_tiles_bound, const std::vector<void *> *dst_down_dev, const std::vector<int64_t> *ldc_down,
                 void **O_out, int64_t *ldO_out, cudaStream_t st, void *O_given = nullptr, int tile_rows = kTcBM,
                 const uint16_t **Z_out = nullptr) {
  Runtime &Rt = rt();
  B2_CHECK(act >= 1 && act <= 3, B200DNN_UNIMPLEMENTED, "fused MoE needs a gated activation (got %d)", act);
  B2_CHECK(I % kGateGranule == 0, B200DNN_UNIMPLEMENTED, "expert FFN width must be a multiple of %d", kGateGranule);
  const int gated = act == ACT_SWIGLU_OAI ? 2 : 1;
  const bool wbf16 = ew[0].wei_dt == B200DNN_BF16;
  for (int g = 0; g < G; ++g)
    B2_CHECK((ew[g].wei_dt == B200DNN_BF16) == wbf16 && (wbf16 || ew[g].wei_dt == 0 || ew[g].wei_dt == B200DNN_S8), B200DNN_UNIMPLEMENTED,
             "expert %d: weight dtype %d (all experts s8, or all bf16)", g, ew[g].wei_dt);
  if (wbf16) return moe_core_bf16(G, ew, K, I, H, transB, act, weights_const, qa, src_dt, R, row_off_dev, tile_prefix_dev, m_tiles_bound,
                                  dst_down_dev, ldc_down, O_out, ldO_out, st, O_given, tile_rows, Z_out);
  std::vector<PackedWeight> p13(G), p2(G);
  std::vector<TcGroupDesc> g13(G), g2(G);
  int32_t b13_dt = 0, b2_dt = 0;
  for (int g = 0; g < G; ++g) {
    B2_CHECK(ew[g].w13 && ew[g].w2 && ew[g].s13 && ew[g].s2, B200DNN_FAILURE, "expert %d: null weight or scale", g);
    B2_TRY(resolve_weight(ew[g].w13, 'n', K, 2 * (int64_t)I, ew[g].ldb13, transB, gated, weights_const, st, &p13[g]));
    B2_TRY(resolve_weight(ew[g].w2, 'n', I, H, ew[g].ldb2, transB, 0, weights_const, st, &p2[g]));
    const void *s13, *s2, *b13 = nullptr, *b2 = nullptr;
    B2_TRY(stage_in(ew[g].s13, (size_t)2 * I * 4, st, &s13));
    B2_TRY(stage_in(ew[g].s2, (size_t)H * 4, st, &s2));
    // biases: one dtype per GEMM (the reference has one bias dtype per pass); an expert may have none
    if (ew[g].b13) {
      B2_CHECK(ew[g].b13_dt == B200DNN_F32 || ew[g].b13_dt == B200DNN_BF16, B200DNN_UNIMPLEMENTED, "expert %d: bias dtype %d", g, ew[g].b13_dt);
      B2_CHECK(b13_dt == 0 || b13_dt == ew[g].b13_dt, B200DNN_UNIMPLEMENTED, "the experts' first-GEMM biases must share one dtype");
      b13_dt = ew[g].b13_dt;
      B2_TRY(stage_in(ew[g].b13, (size_t)2 * I * dt_size(b13_dt), st, &b13));
    }
    if (ew[g].b2) {
      B2_CHECK(ew[g].b2_dt == B200DNN_F32 || ew[g].b2_dt == B200DNN_BF16, B200DNN_UNIMPLEMENTED, "expert %d: down bias dtype %d", g, ew[g].b2_dt);
      B2_CHECK(b2_dt == 0 || b2_dt == ew[g].b2_dt, B200DNN_UNIMPLEMENTED, "the experts' second-GEMM biases must share one dtype");
      b2_dt = ew[g].b2_dt;
      B2_TRY(stage_in(ew[g].b2, (size_t)H * dt_size(b2_dt), st, &b2));
    }
    g13[g] = TcGroupDesc{s13, p13[g].colsum, b13, nullptr, 0};
    g2[g] = TcGroupDesc{s2, p2[g].colsum, b2, dst_down_dev ? (*dst_down_dev)[g] : nullptr, ldc_down ? (*ldc_down)[g] : 0};
  }
  void *g13_dev, *g2_dev;
  B2_TRY(cached_blob(g13.data(), sizeof(TcGroupDesc) * G, st, &g13_dev));
  if (dst_down_dev) B2_TRY(upload_blob(g2.data(), sizeof(TcGroupDesc) * G, st, &g2_dev));   // carries the caller's output pointers: not cached
  else B2_TRY(cached_blob(g2.data(), sizeof(TcGroupDesc) * G, st, &g2_dev));

  const int64_t Kq = round_up(K, 16), Iq = round_up(I, 16);
  int8_t *A1 = (int8_t *)Rt.ws.alloc((size_t)R * Kq);
  float *s1 = (float *)Rt.ws.alloc((size_t)R * 4);
  uint16_t *Z = (uint16_t *)Rt.ws.alloc((size_t)R * I * 2);
  uint32_t *zmax = (uint32_t *)Rt.ws.alloc((size_t)R * 4);
  int8_t *A2 = (int8_t *)Rt.ws.alloc((size_t)R * Iq);
  float *s2v = (float *)Rt.ws.alloc((size_t)R * 4);
  B2_CHECK(A1 && s1 && Z && zmax && A2 && s2v, B200DNN_FAILURE, "workspace allocation failed");
  B2_CUDA(cudaMemsetAsync(zmax, 0, (size_t)R * 4, st));

  // 1. quantise the gathered rows (src_dt == s8: the caller hands over rows that are already quantised,
  //    qa.src = s8 [R, qa.src_ld], qa.scale = their f32 scales -- the expert-parallel path after dispatch)
  const uint8_t *A1_in = (const uint8_t *)A1; int64_t lda1 = Kq; const float *s1_in = s1;
  if (src_dt == B200DNN_S8) {
    B2_CHECK(qa.src && qa.scale && qa.src_ld % 16 == 0 && (reinterpret_cast<uintptr_t>(qa.src) & 15) == 0, B200DNN_FAILURE,
             "pre-quantised rows must be 16-byte aligned with a row stride that is a multiple of 16");
    A1_in = (const uint8_t *)qa.src; lda1 = qa.src_ld; s1_in = (const float *)qa.scale;
  } else {
    qa.dst = A1; qa.dst_ld = Kq; qa.scale = s1; qa.scale_dt = B200DNN_F32; qa.K = K;
    B2_TRY(launch_quant_rows(qa, src_dt, qa.scatter ? qa.scatter_rows : R, st));
  }
  rt().mark(2);

  // 2. first GEMM with the gated epilogue -> Z (bf16, [R, I]) and per-row max |Z|
  EpiParams e1{};
  e1.src_scale = s1_in; e1.src_scale_dt = B200DNN_F32; e1.src_scale_n = R > 1 ? R : 2;  // always per-row
  e1.wei_scale_dt = B200DNN_F32; e1.wei_scale_n = 2 * I;
  e1.dst = Z; e1.ldc = I; e1.dst_dt = B200DNN_BF16; e1.gated_act = act; e1.gated_I = I; e1.row_absmax = zmax;
  e1.bias_dt = b13_dt;
  B2_TRY(grouped_gemm(A1_in, lda1, R, 2 * I, K, p13, row_off_dev, tile_prefix_dev, (const TcGroupDesc *)g13_dev,
                      m_tiles_bound, e1, true, st, tile_rows));
  rt().mark(4);

  // 3. re-quantise the activated rows (from their bf16 values, as the reference does)
  RowQuantArgs q2{};
  q2.src = Z; q2.src_ld = I; q2.dst = A2; q2.dst_ld = Iq; q2.scale = s2v; q2.scale_dt = B200DNN_F32; q2.K = I;
  q2.absmax_bits = zmax; q2.gather_div = 1;
  B2_TRY(launch_quant_rows(q2, B200DNN_BF16, R, st));
  rt().mark(5);

  // 4. second GEMM -> O
  uint16_t *O = (uint16_t *)O_given;     // dense [R, H] rows of the caller, when given
  if (!dst_down_dev && !O) { O = (uint16_t *)Rt.ws.alloc((size_t)R * H * 2); B2_CHECK(O, B200DNN_FAILURE, "workspace allocation failed"); }
  EpiParams e2{};
  e2.src_scale = s2v; e2.src_scale_dt = B200DNN_F32; e2.src_scale_n = R > 1 ? R : 2;
  e2.wei_scale_dt = B200DNN_F32; e2.wei_scale_n = H;
  e2.dst = O; e2.ldc = H; e2.dst_dt = B200DNN_BF16; e2.bias_dt = b2_dt;
  B2_TRY(grouped_gemm((const uint8_t *)A2, Iq, R, H, I, p2, row_off_dev, tile_prefix_dev, (const TcGroupDesc *)g2_dev,
                      m_tiles_bound, e2, dst_down_dev == nullptr, st, tile_rows));
  rt().mark(6);
  if (Z_out) *Z_out = Z;
  if (O_out) { *O_out = O; *ldO_out = H; }
  return B200DNN_SUCCESS;
}

}  // namespace

extern "C" int32_t b200dnn_fused_moe(int32_t G, const b200dnn_moe_expert_t *ex, int32_t K, int32_t I, int32_t H,
                                     int32_t transB, int32_t act, int32_t weights_const, const void *const *row_ptrs,
                                     const float *topk_weights, int32_t T, int32_t topk, void *out, int64_t ld_out,
                                     void *stream) {
  B2_ENTER(stream);
  Runtime &Rt = rt();
  B2_CHECK(G > 0 && ex && K > 0 && I > 0 && H > 0, B200DNN_FAILURE, "bad argument");
  std::vector<int32_t> row_off(G + 1, 0), tile_prefix(G + 1, 0);
  long long rows_all = 0;
  for (int g = 0; g < G; ++g) rows_all += ex[g].M > 0 ? ex[g].M : 0;
  const int tile_rows = tc_tile_rows(rows_all, H < 2 * I ? H : 2 * I);
  for (int g = 0; g < G; ++g) {
    B2_CHECK(ex[g].M >= 0, B200DNN_FAILURE, "expert %d: negative M", g);
    row_off[g + 1] = row_off[g] + ex[g].M;
    tile_prefix[g + 1] = tile_prefix[g] + (ex[g].M + tile_rows - 1) / tile_rows;
    if (ex[g].M > 0) {
      B2_CHECK(ex[g].src, B200DNN_FAILURE, "expert %d: null src", g);
      // dst_down == NULL: the reference's src-reuse mode, the result goes back into src with row stride lda
      B2_CHECK(ex[g].lda >= K && (ex[g].dst_down ? ex[g].ldc_down >= H : ex[g].lda >= H), B200DNN_FAILURE,
               "expert %d: leading dimension too small", g);
      B2_CHECK(!ex[g].dst_op1 || ex[g].ldc_op1 >= I, B200DNN_FAILURE, "expert %d: ldc_op1 too small", g);
    }
  }
  const int R = row_off[G];
  if (R == 0) return B200DNN_SUCCESS;
  // stage per-expert sources / destinations and build the device tables
  std::vector<const void *> src_dev(G, nullptr);
  std::vector<void *> dst_dev(G, nullptr);
  std::vector<int64_t> src_ld(G), ldc_down(G);
  std::vector<Staged> outs(G);
  for (int g = 0; g < G; ++g) {
    src_ld[g] = ex[g].lda; ldc_down[g] = ex[g].dst_down ? ex[g].ldc_down : ex[g].lda;
    outs[g].copy_back = false;
    if (ex[g].M == 0) continue;
    B2_TRY(stage_in(ex[g].src, span_bytes(ex[g].M, K, ex[g].lda, B200DNN_BF16), st, &src_dev[g]));
    // the rows are copied out of src and quantised before the second GEMM runs, so src may take the result
    void *dst_host = ex[g].dst_down ? ex[g].dst_down : const_cast<void *>(ex[g].src);
    B2_TRY(stage_out(dst_host, span_bytes(ex[g].M, H, ldc_down[g], B200DNN_BF16), st, &outs[g], ldc_down[g] != H));
    dst_dev[g] = outs[g].dev;
  }
  // blob: src ptrs | src ld | row_off | tile_prefix
  const size_t o_ptr = 0, o_ld = o_ptr + sizeof(void *) * G, o_ro = o_ld + sizeof(int64_t) * G,
               o_tp = o_ro + sizeof(int32_t) * (G + 1), total = o_tp + sizeof(int32_t) * (G + 1);
  std::vector<uint8_t> blob((total + 15) & ~size_t(15));
  memcpy(blob.data() + o_ptr, src_dev.data(), sizeof(void *) * G);
  memcpy(blob.data() + o_ld, src_ld.data(), sizeof(int64_t) * G);
  memcpy(blob.data() + o_ro, row_off.data(), sizeof(int32_t) * (G + 1));
  memcpy(blob.data() + o_tp, tile_prefix.data(), sizeof(int32_t) * (G + 1));
  void *bd;
  B2_TRY(upload_blob(blob.data(), blob.size(), st, &bd));
  uint8_t *b = (uint8_t *)bd;
  const int32_t *row_off_dev = (const int32_t *)(b + o_ro), *tile_prefix_dev = (const int32_t *)(b + o_tp);

  std::vector<ExpertWeightsIn> ew(G);
  for (int g = 0; g < G; ++g) ew[g] = expert_in(ex[g]);

  // the experts' rows are first laid back to back in one bf16 slab, then quantised in one launch
  RowQuantArgs qa{};
  qa.gather_div = 1;
  uint16_t *X = (uint16_t *)Rt.ws.alloc((size_t)R * K * 2);
  B2_CHECK(X, B200DNN_FAILURE, "workspace allocation failed");
  for (int g = 0; g < G; ++g) {
    if (ex[g].M == 0) continue;
    B2_CUDA(cudaMemcpy2DAsync(X + (size_t)row_off[g] * K, (size_t)K * 2, src_dev[g], (size_t)ex[g].lda * 2, (size_t)K * 2,
                              (size_t)ex[g].M, cudaMemcpyDeviceToDevice, st));
  }
  qa.src = X; qa.src_ld = K;

  const uint16_t *Z = nullptr;
  B2_TRY(moe_core(G, ew, K, I, H, transB, act, weights_const, qa, B200DNN_BF16, R, row_off_dev, tile_prefix_dev,
                  tile_prefix[G], &dst_dev, &ldc_down, nullptr, nullptr, st, nullptr, tile_rows, &Z));
  // the activated output of the first GEMM, for callers that want it (the reference leaves it in dst[])
  std::vector<Staged> op1_outs;
  for (int g = 0; g < G; ++g) {
    if (ex[g].M == 0 || !ex[g].dst_op1) continue;
    Staged o1;
    B2_TRY(stage_out(ex[g].dst_op1, span_bytes(ex[g].M, I, ex[g].ldc_op1, B200DNN_BF16), st, &o1, ex[g].ldc_op1 != I));
    B2_CUDA(cudaMemcpy2DAsync(o1.dev, (size_t)ex[g].ldc_op1 * 2, Z + (size_t)row_off[g] * I, (size_t)I * 2, (size_t)I * 2,
                              (size_t)ex[g].M, cudaMemcpyDefault, st));
    op1_outs.push_back(o1);
  }

  Staged o_out; o_out.copy_back = false;
  if (row_ptrs) {
    B2_CHECK(out && T > 0 && topk > 0 && ld_out >= H, B200DNN_FAILURE, "weighted reduce: bad argument");
    B2_CHECK(topk_weights, B200DNN_FAILURE, "weighted reduce: topk_weights is null");
    B2_CHECK(!is_device_ptr(row_ptrs), B200DNN_UNIMPLEMENTED,
             "weighted reduce: row_ptrs is an array in host memory (as in the reference); a device array is not accepted");
    const size_t ns = (size_t)T * topk;
    // translate the caller's row pointers (into dst_down buffers) to device addresses
    std::vector<const void *> dev_rows(ns);
    for (size_t i = 0; i < ns; ++i) {
      const uint8_t *p = (const uint8_t *)row_ptrs[i];
      B2_CHECK(p, B200DNN_FAILURE, "row_ptrs[%zu] is null", i);
      const void *dp = nullptr;
      for (int g = 0; g < G && !dp; ++g) {
        if (ex[g].M == 0) continue;
        const uint8_t *lo = (const uint8_t *)(ex[g].dst_down ? ex[g].dst_down : ex[g].src);
        const uint8_t *hi = lo + span_bytes(ex[g].M, H, ldc_down[g], B200DNN_BF16);
        if (p >= lo && p < hi) dp = (const uint8_t *)dst_dev[g] + (p - lo);
      }
      B2_CHECK(dp, B200DNN_FAILURE, "row_ptrs[%zu] does not point into any expert's output buffer", i);
      dev_rows[i] = dp;
    }
    void *tab, *w_dev;
    B2_TRY(upload_blob(dev_rows.data(), ns * sizeof(void *), st, &tab));
    const void *wd;
    B2_TRY(stage_in(topk_weights, ns * 4, st, &wd));
    w_dev = const_cast<void *>(wd);
    B2_TRY(stage_out(out, span_bytes(T, H, ld_out, B200DNN_BF16), st, &o_out, ld_out != H));
    ReduceArgs ra{};
    ra.row_ptrs = (const void *const *)tab; ra.w = (const float *)w_dev; ra.nslots = topk; ra.D = H; ra.dt = B200DNN_BF16;
    ra.out = o_out.dev; ra.ld_out = ld_out;
    moe_reduce_kernel<<<(unsigned)T, 256, (sizeof(void *) + 4) * topk, st>>>(ra);
    B2_LAUNCHED();
    B2_CUDA(cudaGetLastError());
  }
  bool any = o_out.copy_back || o_out.sync;
  for (auto &s : outs) if (s.sync) any = true;
  for (auto &s : op1_outs) {
    if (s.sync) any = true;
    if (s.copy_back) { B2_CUDA(cudaMemcpyAsync(s.host, s.dev, s.bytes, cudaMemcpyDeviceToHost, st)); any = true; }
  }
  for (auto &s : outs) if (s.copy_back) { B2_CUDA(cudaMemcpyAsync(s.host, s.dev, s.bytes, cudaMemcpyDeviceToHost, st)); any = true; }
  if (o_out.copy_back) B2_CUDA(cudaMemcpyAsync(o_out.host, o_out.dev, o_out.bytes, cudaMemcpyDeviceToHost, st));
  if (any) { B2_CUDA(cudaStreamSynchronize(st)); B2_TRY(check_tc_status(st)); }
  return B200DNN_SUCCESS;
}

extern "C" int32_t b200dnn_moe_layer(const void *x, int64_t ldx, const float *logits, int32_t T, int32_t E, int32_t S,
                                     int32_t topk, const b200dnn_moe_expert_t *ex, int32_t K, int32_t I, int32_t H,
                                     int32_t transB, int32_t act, void *out, int64_t ld_out, void *stream) {
  B2_ENTER(stream);
  Runtime &Rt = rt();
  B2_CHECK(x && logits && ex && out && T > 0 && E > 0 && S >= 0 && topk > 0 && topk <= E && topk <= kMaxTopk, B200DNN_FAILURE, "bad argument");
  B2_CHECK(ldx >= K && ld_out >= H, B200DNN_FAILURE, "leading dimension too small");
  const int G = E + S, ns = topk + S, R = T * ns;
  const void *x_dev, *l_dev;
  B2_TRY(stage_in(x, span_bytes(T, K, ldx, B200DNN_BF16), st, &x_dev));
  B2_TRY(stage_in(logits, (size_t)T * E * 4, st, &l_dev));
  int32_t *ids = (int32_t *)Rt.ws.alloc((size_t)T * topk * 4);
  float *w = (float *)Rt.ws.alloc((size_t)T * topk * 4);
  int32_t *rank = (int32_t *)Rt.ws.alloc((size_t)T * topk * 4);
  int32_t *cnt = (int32_t *)Rt.ws.alloc((size_t)E * 4);
  int32_t *row_off = (int32_t *)Rt.ws.alloc((size_t)(G + 1) * 4);
  int32_t *tile_prefix = (int32_t *)Rt.ws.alloc((size_t)(G + 1) * 4);
  int32_t *slot_rows = (int32_t *)Rt.ws.alloc((size_t)R * 4);
  float *slot_w = (float *)Rt.ws.alloc((size_t)R * 4);
  int32_t *row_token = (int32_t *)Rt.ws.alloc((size_t)R * 4);
  B2_CHECK(ids && w && rank && cnt && row_off && tile_prefix && slot_rows && slot_w && row_token, B200DNN_FAILURE, "workspace allocation failed");
  rt().mark(-1);
  B2_TRY(launch_route_topk((const float *)l_dev, T, E, topk, 1, ids, w, st));
  B2_TRY(launch_expert_rank(ids, T * topk, E, rank, cnt, st));
  const int tile_rows = tc_tile_rows(R, H < 2 * I ? H : 2 * I);
  expert_offsets_kernel<<<1, 32, 0, st>>>(cnt, E, S, T, row_off, tile_prefix, tile_rows);
  B2_LAUNCHED();
  build_maps_kernel<<<(unsigned)((R + 255) / 256), 256, 0, st>>>(ids, rank, w, row_off, T, topk, E, S, slot_rows, slot_w, row_token);
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  rt().mark(0);

  std::vector<ExpertWeightsIn> ew(G);
  for (int g = 0; g < G; ++g) ew[g] = expert_in(ex[g]);
  RowQuantArgs qa{};
  // every token is quantised once and written to the rows of all its slots (routed and shared experts)
  qa.src = x_dev; qa.src_ld = ldx; qa.gather_div = 1;
  if (ns <= 32) { qa.scatter = slot_rows; qa.scatter_n = ns; qa.scatter_rows = T; }
  else qa.gather = row_token;
  void *O = nullptr; int64_t ldO = 0;
  const int m_tiles_bound = (R + tile_rows - 1) / tile_rows + G;
  B2_TRY(moe_core(G, ew, K, I, H, transB, act, 1, qa, B200DNN_BF16, R, row_off, tile_prefix, m_tiles_bound, nullptr, nullptr, &O, &ldO, st,
                  nullptr, tile_rows));

  Staged o_out;
  B2_TRY(stage_out(out, span_bytes(T, H, ld_out, B200DNN_BF16), st, &o_out, ld_out != H));
  ReduceArgs ra{};
  ra.base = O; ra.ld = ldO; ra.slot_rows = slot_rows; ra.w = slot_w; ra.nslots = ns; ra.D = H; ra.dt = B200DNN_BF16;
  ra.out = o_out.dev; ra.ld_out = ld_out;
  moe_reduce_kernel<<<(unsigned)T, 256, (sizeof(void *) + 4) * ns, st>>>(ra);
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  rt().mark(8);
  return finish_out({&o_out}, st);
}

// ------------------------------------------------------------------------------------------------
// Building blocks of the expert-parallel MoE (token dispatch between GPUs happens outside, over
// NCCL): stable sort positions of (token,k) slots by an integer key, gather + per-token
// quantisation into send order, and the expert computation on rows that arrive already quantised.
namespace {
__global__ void slot_rows_kernel(const int32_t *keys, const int32_t *rank, const int32_t *off, int n, int32_t *slot_to_row) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) slot_to_row[i] = off[keys[i]] + rank[i];
}
}  // namespace

extern "C" int32_t b200dnn_moe_sort_slots(const int32_t *keys, int32_t nslots, int32_t nkeys, int32_t *counts,
                                          int32_t *slot_to_row, void *stream) {
  B2_ENTER(stream);
  Runtime &Rt = rt();
  B2_CHECK(keys && counts && slot_to_row && nslots > 0 && nkeys > 0, B200DNN_FAILURE, "bad argument");
  const void *k_dev;
  B2_TRY(stage_in(keys, (size_t)nslots * 4, st, &k_dev));
  Staged o_cnt, o_s2r;
  B2_TRY(stage_out(counts, (size_t)nkeys * 4, st, &o_cnt));
  B2_TRY(stage_out(slot_to_row, (size_t)nslots * 4, st, &o_s2r));
  int32_t *rank = (int32_t *)Rt.ws.alloc((size_t)nslots * 4);
  int32_t *off = (int32_t *)Rt.ws.alloc((size_t)(nkeys + 1) * 4);
  B2_CHECK(rank && off, B200DNN_FAILURE, "workspace allocation failed");
  B2_TRY(launch_expert_rank((const int32_t *)k_dev, nslots, nkeys, rank, (int32_t *)o_cnt.dev, st));
  expert_offsets_kernel<<<1, 32, 0, st>>>((const int32_t *)o_cnt.dev, nkeys, 0, 0, off);
  B2_LAUNCHED();
  slot_rows_kernel<<<(unsigned)((nslots + 255) / 256), 256, 0, st>>>((const int32_t *)k_dev, rank, off, nslots, (int32_t *)o_s2r.dev);
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  return finish_out({&o_cnt, &o_s2r}, st);
}

extern "C" int32_t b200dnn_quant_per_token_gather(const void *src, int32_t src_dt, int64_t K, int64_t src_ld,
                                                  const int32_t *row_src, int32_t row_div, int64_t R, void *dst,
                                                  int64_t dst_ld, float *scale, void *stream) {
  B2_ENTER(stream);
  B2_CHECK(src && row_src && dst && scale && K > 0 && R > 0 && src_ld >= K && dst_ld >= K && row_div > 0, B200DNN_FAILURE, "bad argument");
  B2_CHECK(is_device_ptr(src) && is_device_ptr(row_src) && is_device_ptr(dst) && is_device_ptr(scale), B200DNN_UNIMPLEMENTED,
           "gathered quantisation takes device pointers only");
  RowQuantArgs a{};
  a.src = src; a.src_ld = src_ld; a.gather = row_src; a.gather_div = row_div; a.dst = (int8_t *)dst; a.dst_ld = dst_ld;
  a.scale = scale; a.scale_dt = B200DNN_F32; a.K = (int32_t)K;
  return launch_quant_rows(a, src_dt, R, st);
}

extern "C" int32_t b200dnn_quant_per_token_scatter(const void *src, int32_t src_dt, int64_t K, int64_t src_ld,
                                                   const int32_t *dst_rows, int32_t n_dst, int64_t T, void *dst,
                                                   int64_t dst_ld, float *scale, void *stream) {
  B2_ENTER(stream);
  B2_CHECK(src && dst_rows && dst && scale && K > 0 && T > 0 && src_ld >= K && dst_ld >= K && n_dst > 0 && n_dst <= 32,
           B200DNN_FAILURE, "bad argument");
  B2_CHECK(is_device_ptr(src) && is_device_ptr(dst_rows) && is_device_ptr(dst) && is_device_ptr(scale), B200DNN_UNIMPLEMENTED,
           "scattered quantisation takes device pointers only");
  RowQuantArgs a{};
  a.src = src; a.src_ld = src_ld; a.gather_div = 1; a.dst = (int8_t *)dst; a.dst_ld = dst_ld;
  a.scale = scale; a.scale_dt = B200DNN_F32; a.K = (int32_t)K;
  a.scatter = dst_rows; a.scatter_n = n_dst; a.scatter_rows = (int32_t)T;
  return launch_quant_rows(a, src_dt, T, st);
}

extern "C" int32_t b200dnn_moe_experts_s8(const void *rows_s8, int64_t lda, const float *row_scale, int32_t n_groups,
                                          const int32_t *group_rows, const int32_t *group_expert,
                                          const b200dnn_moe_expert_t *experts, int32_t K, int32_t I, int32_t H,
                                          int32_t transB, int32_t act, void *out, int64_t ld_out, void *stream) {
  B2_ENTER(stream);
  Runtime &Rt = rt();
  B2_CHECK(rows_s8 && row_scale && group_rows && group_expert && experts && out && n_groups > 0, B200DNN_FAILURE, "bad argument");
  B2_CHECK(is_device_ptr(rows_s8) && is_device_ptr(row_scale) && is_device_ptr(out), B200DNN_UNIMPLEMENTED,
           "the expert-parallel building block takes device buffers only");
  B2_CHECK(ld_out == H, B200DNN_UNIMPLEMENTED, "output rows must be dense (ld_out == H)");
  std::vector<int32_t> row_off(n_groups + 1, 0), tile_prefix(n_groups + 1, 0);
  std::vector<ExpertWeightsIn> ew(n_groups);
  long long rows_all = 0;
  for (int g = 0; g < n_groups; ++g) rows_all += group_rows[g] > 0 ? group_rows[g] : 0;
  const int tile_rows = tc_tile_rows(rows_all, H < 2 * I ? H : 2 * I);
  for (int g = 0; g < n_groups; ++g) {
    B2_CHECK(group_rows[g] >= 0 && group_expert[g] >= 0, B200DNN_FAILURE, "group %d: negative row count or expert id", g);
    row_off[g + 1] = row_off[g] + group_rows[g];
    tile_prefix[g + 1] = tile_prefix[g] + (group_rows[g] + tile_rows - 1) / tile_rows;
    const b200dnn_moe_expert_t &e = experts[group_expert[g]];
    ew[g] = expert_in(e);
  }
  const int R = row_off[n_groups];
  if (R == 0) return B200DNN_SUCCESS;
  std::vector<int32_t> blob(2 * (n_groups + 1));
  memcpy(blob.data(), row_off.data(), sizeof(int32_t) * (n_groups + 1));
  memcpy(blob.data() + n_groups + 1, tile_prefix.data(), sizeof(int32_t) * (n_groups + 1));
  void *bd;
  B2_TRY(upload_blob(blob.data(), blob.size() * 4, st, &bd));
  const int32_t *row_off_dev = (const int32_t *)bd, *tile_prefix_dev = row_off_dev + n_groups + 1;
  RowQuantArgs qa{};
  qa.src = rows_s8; qa.src_ld = lda; qa.scale = const_cast<float *>(row_scale);
  void *O = nullptr; int64_t ldO = 0;
  // the second GEMM writes the caller's dense rows directly
  return moe_core(n_groups, ew, K, I, H, transB, act, 1, qa, B200DNN_S8, R, row_off_dev, tile_prefix_dev, tile_prefix[n_groups],
                  nullptr, nullptr, &O, &ldO, st, out, tile_rows);
}

extern "C" int32_t b200dnn_moe_weighted_reduce_rows(const void *rows, int64_t ld_rows, const int32_t *slot_rows,
                                                    const float *slot_weights, int32_t num_tokens, int32_t nslots, int32_t D,
                                                    int32_t dt, void *out, int64_t ld_out, void *stream) {
  B2_ENTER(stream);
  B2_CHECK(rows && slot_rows && slot_weights && out && num_tokens > 0 && nslots > 0 && D > 0 && ld_rows >= D && ld_out >= D,
           B200DNN_FAILURE, "bad argument");
  B2_CHECK(dt == B200DNN_BF16 || dt == B200DNN_F32, B200DNN_UNIMPLEMENTED, "weighted reduce on f32 or bf16 only");
  B2_CHECK(is_device_ptr(rows) && is_device_ptr(slot_rows) && is_device_ptr(slot_weights) && is_device_ptr(out), B200DNN_UNIMPLEMENTED,
           "device pointers only");
  ReduceArgs ra{};
  ra.base = rows; ra.ld = ld_rows; ra.slot_rows = slot_rows; ra.w = slot_weights; ra.nslots = nslots; ra.D = D; ra.dt = dt;
  ra.out = out; ra.ld_out = ld_out;
  moe_reduce_kernel<<<(unsigned)num_tokens, 256, (sizeof(void *) + 4) * nslots, st>>>(ra);
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  return B200DNN_SUCCESS;
}
