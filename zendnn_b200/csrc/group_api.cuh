// b200dnn_group_matmul: the plain (parallel) mode of the reference's group_matmul_direct -- every expert an
// independent GEMM with its own source, weight, bias and destination
// (lowoha_operators/matmul/group_matmul/group_matmul_parallel_common.hpp:1240-1248: experts with M == 0 are skipped).
// Experts that share one problem shape run as ONE grouped tcgen05 launch (the same kernel as the fused MoE's second
// GEMM: one tensor map per expert, per-expert epilogue pointers), W8A8 experts and bf16 x bf16 experts alike; anything else
// runs expert by expert through
// b200dnn_matmul, so the results are those of G separate calls either way.  Included at the end of b200dnn.cu.
#pragma once

namespace {

// Can the active experts share one grouped launch?  Pure host logic on the descriptors.
bool group_is_uniform(int G, const b200dnn_matmul_t *d) {
  const b200dnn_matmul_t *f = nullptr;
  long long rows = 0;
  int active = 0, bias_dt = 0;
  for (int g = 0; g < G; ++g) {
    const b200dnn_matmul_t &x = d[g];
    if (x.M <= 0) { if (x.M < 0) return false; continue; }
    ++active; rows += x.M;
    if (!f) f = &x;
    if (x.bias) {           // experts with a bias share its dtype; an expert may have none
      if (bias_dt && x.bias_dt != bias_dt) return false;
      bias_dt = x.bias_dt;
    }
    if (x.transA) return false;             // transposed sources go through b200dnn_matmul one by one
    if (x.K != f->K || x.N != f->N || x.transB != f->transB || x.wei_format != f->wei_format || x.src_dt != f->src_dt ||
        x.wei_dt != f->wei_dt || x.dst_dt != f->dst_dt || x.dynamic_quant != f->dynamic_quant ||
        x.weights_const != f->weights_const || x.n_postops != f->n_postops || x.force_kernel != 0)
      return false;
    if (x.wei_dt != B200DNN_S8 || (x.dst_dt != B200DNN_BF16 && x.dst_dt != B200DNN_F32)) return false;
    if (x.src_zp.buff || x.src_zp.count > 0) return false;
    if (!x.wei_scale.buff || x.wei_scale.dt != B200DNN_F32 || x.wei_scale.count != x.N) return false;
    if (x.dynamic_quant) {
      // the library quantises the rows; a caller-side scale buffer (an output then) takes the one-by-one path
      if ((x.src_dt != B200DNN_BF16 && x.src_dt != B200DNN_F32) || x.src_scale.buff) return false;
    } else {
      if (x.src_dt != B200DNN_S8 || !x.src_scale.buff || x.src_scale.dt != B200DNN_F32 || x.src_scale.count != x.M) return false;
    }
    for (int i = 0; i < x.n_postops; ++i) {
      const b200dnn_postop_t &p = x.postops[i], &q = f->postops[i];
      if (p.type == PO_BINARY_ADD || p.type == PO_BINARY_MUL) return false;   // per-expert operand matrices
      if (p.type != q.type || p.alpha != q.alpha || p.beta != q.beta) return false;
    }
  }
  // fewer than two experts, or so few rows that the weight-streaming kernels are the better choice per expert
  return active >= 2 && rows > 16ll * active && f->K % 16 == 0;
}

int32_t group_matmul_grouped(int G, const b200dnn_matmul_t *d, void *stream) {
  B2_ENTER(stream);
  Runtime &Rt = rt();
  const b200dnn_matmul_t *f = nullptr;
  std::vector<int32_t> row_off(G + 1, 0), tile_prefix(G + 1, 0);
  long long rows_all = 0;
  for (int g = 0; g < G; ++g) if (d[g].M > 0) { rows_all += d[g].M; if (!f) f = &d[g]; }
  const int K = f->K, N = f->N;
  const int tile_rows = tc_tile_rows(rows_all, N);
  for (int g = 0; g < G; ++g) {
    const int m = d[g].M > 0 ? d[g].M : 0;
    if (m) B2_TRY(validate_matmul_desc(&d[g]));
    row_off[g + 1] = row_off[g] + m;
    tile_prefix[g + 1] = tile_prefix[g] + (m + tile_rows - 1) / tile_rows;
  }
  const int R = row_off[G];
  const bool dyn = f->dynamic_quant != 0;
  const int64_t Kq = round_up(K, 16);

  // weights, epilogue tables and destinations per expert
  std::vector<PackedWeight> pws(G);
  std::vector<TcGroupDesc> gd(G);
  std::vector<Staged> outs(G);
  std::vector<const void *> src_dev(G, nullptr);
  int first = -1;
  for (int g = 0; g < G; ++g) {
    outs[g].copy_back = false;
    if (d[g].M <= 0) continue;
    if (first < 0) first = g;
    B2_TRY(resolve_weight(d[g].weight, d[g].wei_format, K, N, d[g].ldb, d[g].transB, 0, d[g].weights_const, st, &pws[g]));
    const void *ws = nullptr, *b = nullptr;
    B2_TRY(stage_in(d[g].wei_scale.buff, (size_t)N * 4, st, &ws));
    if (d[g].bias) B2_TRY(stage_in(d[g].bias, (size_t)N * dt_size(d[g].bias_dt), st, &b));
    B2_TRY(stage_in(d[g].src, span_bytes(d[g].M, K, d[g].lda, d[g].src_dt), st, &src_dev[g]));
    B2_TRY(stage_out(d[g].dst, span_bytes(d[g].M, N, d[g].ldc, d[g].dst_dt), st, &outs[g], d[g].ldc != N));
    gd[g] = TcGroupDesc{ws, pws[g].colsum, b, outs[g].dev, d[g].ldc};
  }
  // an expert without rows still needs a valid tensor map: it borrows the first active expert's weight (never read)
  for (int g = 0; g < G; ++g) if (d[g].M <= 0) { pws[g] = pws[first]; gd[g] = TcGroupDesc{gd[first].wei_scale, gd[first].colsum, nullptr, nullptr, 0}; }
  void *gd_dev = nullptr;
  B2_TRY(upload_blob(gd.data(), sizeof(TcGroupDesc) * G, st, &gd_dev));   // carries the caller's output pointers: not cached

  // rows of all experts back to back: [R, Kq] s8 and R f32 scales
  int8_t *A = (int8_t *)Rt.ws.alloc((size_t)R * Kq);
  float *sc = (float *)Rt.ws.alloc((size_t)R * 4);
  B2_CHECK(A && sc, B200DNN_FAILURE, "workspace allocation failed");
  if (dyn) {
    // one quantisation launch over all experts' rows (the group form of the per-token kernel)
    std::vector<void *> q_dev(G, nullptr), s_dev(G, nullptr);
    std::vector<int64_t> sld(G, 0), dld(G, Kq);
    for (int g = 0; g < G; ++g) {
      sld[g] = d[g].lda;
      if (d[g].M > 0) { q_dev[g] = A + (size_t)row_off[g] * Kq; s_dev[g] = sc + row_off[g]; }
    }
    const size_t tb = sizeof(void *) * G;
    std::vector<uint8_t> host(3 * tb + 2 * sizeof(int64_t) * G + sizeof(int32_t) * (G + 1));
    uint8_t *h = host.data();
    memcpy(h, src_dev.data(), tb); memcpy(h + tb, q_dev.data(), tb); memcpy(h + 2 * tb, s_dev.data(), tb);
    memcpy(h + 3 * tb, sld.data(), sizeof(int64_t) * G);
    memcpy(h + 3 * tb + sizeof(int64_t) * G, dld.data(), sizeof(int64_t) * G);
    memcpy(h + 3 * tb + 2 * sizeof(int64_t) * G, row_off.data(), sizeof(int32_t) * (G + 1));
    void *tab = nullptr;
    B2_TRY(upload_blob(h, host.size(), st, &tab));
    uint8_t *t = (uint8_t *)tab;
    RowQuantArgs a{};
    a.n_groups = G; a.K = K; a.scale_dt = B200DNN_F32; a.gather_div = 1;
    a.g_src = (const void *const *)t; a.g_dst = (void *const *)(t + tb); a.g_scale = (void *const *)(t + 2 * tb);
    a.g_src_ld = (const int64_t *)(t + 3 * tb); a.g_dst_ld = (const int64_t *)(t + 3 * tb + sizeof(int64_t) * G);
    a.row_off = (const int32_t *)(t + 3 * tb + 2 * sizeof(int64_t) * G);
    B2_TRY(launch_quant_rows(a, f->src_dt, R, st));
  } else {
    for (int g = 0; g < G; ++g) {
      if (d[g].M <= 0) continue;
      const void *s = nullptr;
      B2_TRY(stage_in(d[g].src_scale.buff, (size_t)d[g].M * 4, st, &s));
      B2_CUDA(cudaMemcpy2DAsync(A + (size_t)row_off[g] * Kq, (size_t)Kq, src_dev[g], (size_t)d[g].lda, (size_t)K, (size_t)d[g].M,
                                cudaMemcpyDefault, st));
      B2_CUDA(cudaMemcpyAsync(sc + row_off[g], s, (size_t)d[g].M * 4, cudaMemcpyDefault, st));
    }
  }

  void *tabs = nullptr;
  std::vector<int32_t> both(2 * (G + 1));
  memcpy(both.data(), row_off.data(), sizeof(int32_t) * (G + 1));
  memcpy(both.data() + G + 1, tile_prefix.data(), sizeof(int32_t) * (G + 1));
  B2_TRY(upload_blob(both.data(), both.size() * sizeof(int32_t), st, &tabs));
  const int32_t *row_off_dev = (const int32_t *)tabs, *tile_prefix_dev = row_off_dev + G + 1;

  EpiParams e{};
  e.src_scale = sc; e.src_scale_dt = B200DNN_F32; e.src_scale_n = R > 1 ? R : 2;   // always per row
  e.wei_scale_dt = B200DNN_F32; e.wei_scale_n = N;
  e.dst = nullptr; e.ldc = N; e.dst_dt = f->dst_dt;
  for (int g = 0; g < G; ++g) if (d[g].M > 0 && d[g].bias) e.bias_dt = d[g].bias_dt;
  e.n_po = f->n_postops;
  for (int i = 0; i < f->n_postops; ++i) {
    const b200dnn_postop_t &p = f->postops[i];
    e.po[i].type = p.type; e.po[i].dt = p.dt; e.po[i].ld = 0; e.po[i].alpha = p.alpha; e.po[i].beta = p.beta; e.po[i].buff = nullptr;
  }
  B2_TRY(grouped_gemm((const uint8_t *)A, Kq, R, N, K, pws, row_off_dev, tile_prefix_dev, (const TcGroupDesc *)gd_dev, tile_prefix[G], e,
                      false, st, tile_rows));
  bool any = false;
  for (auto &s : outs) {
    if (s.copy_back) { B2_CUDA(cudaMemcpyAsync(s.host, s.dev, s.bytes, cudaMemcpyDeviceToHost, st)); any = true; }
    else if (s.sync) any = true;
  }
  if (any) B2_TRY(check_tc_status(st));
  return B200DNN_SUCCESS;
}

// bf16 x bf16 experts of one shape (no quantisation, no scales): the same grouped launch on the kernel's bf16 form
bool group_is_uniform_bf16(int G, const b200dnn_matmul_t *d) {
  const b200dnn_matmul_t *f = nullptr;
  long long rows = 0;
  int active = 0, bias_dt = 0;
  for (int g = 0; g < G; ++g) {
    const b200dnn_matmul_t &x = d[g];
    if (x.M <= 0) { if (x.M < 0) return false; continue; }
    ++active; rows += x.M;
    if (!f) f = &x;
    if (!is_bf16_matmul(&x) || (x.dst_dt != B200DNN_BF16 && x.dst_dt != B200DNN_F32)) return false;
    if (x.bias) {
      if (bias_dt && x.bias_dt != bias_dt) return false;
      bias_dt = x.bias_dt;
    }
    if (x.transA) return false;
    if (x.K != f->K || x.N != f->N || x.transB != f->transB || x.dst_dt != f->dst_dt || x.weights_const != f->weights_const ||
        x.n_postops != f->n_postops || x.force_kernel != 0 || (x.wei_format != 'n' && x.wei_format != 0))
      return false;
    for (int i = 0; i < x.n_postops; ++i) {
      const b200dnn_postop_t &p = x.postops[i], &q = f->postops[i];
      if (p.type == PO_BINARY_ADD || p.type == PO_BINARY_MUL) return false;
      if (p.type != q.type || p.alpha != q.alpha || p.beta != q.beta) return false;
    }
  }
  return active >= 2 && rows > 16ll * active;
}

int32_t group_matmul_grouped_bf16(int G, const b200dnn_matmul_t *d, void *stream) {
  B2_ENTER(stream);
  Runtime &Rt = rt();
  const b200dnn_matmul_t *f = nullptr;
  std::vector<int32_t> row_off(G + 1, 0), tile_prefix(G + 1, 0);
  long long rows_all = 0;
  for (int g = 0; g < G; ++g) if (d[g].M > 0) { rows_all += d[g].M; if (!f) f = &d[g]; }
  const int K = f->K, N = f->N;
  const int tile_rows = tc_tile_rows(rows_all, N);
  for (int g = 0; g < G; ++g) {
    const int m = d[g].M > 0 ? d[g].M : 0;
    if (m) B2_TRY(validate_bf16_matmul(&d[g]));
    row_off[g + 1] = row_off[g] + m;
    tile_prefix[g + 1] = tile_prefix[g] + (m + tile_rows - 1) / tile_rows;
  }
  const int R = row_off[G];
  const int64_t Kq = round_up(K, 8);
  std::vector<PackedWeight> pws(G);
  std::vector<TcGroupDesc> gd(G);
  std::vector<Staged> outs(G);
  uint16_t *X = (uint16_t *)Rt.ws.alloc((size_t)R * Kq * 2);
  B2_CHECK(X, B200DNN_FAILURE, "workspace allocation failed");
  int first = -1;
  for (int g = 0; g < G; ++g) {
    outs[g].copy_back = false;
    if (d[g].M <= 0) continue;
    if (first < 0) first = g;
    B2_TRY(resolve_bf16_weight(d[g].weight, K, N, d[g].ldb, d[g].transB, 0, d[g].weights_const, st, &pws[g]));
    const void *b = nullptr, *src = nullptr;
    if (d[g].bias) B2_TRY(stage_in(d[g].bias, (size_t)N * dt_size(d[g].bias_dt), st, &b));
    B2_TRY(stage_in(d[g].src, span_bytes(d[g].M, K, d[g].lda, B200DNN_BF16), st, &src));
    B2_TRY(stage_out(d[g].dst, span_bytes(d[g].M, N, d[g].ldc, d[g].dst_dt), st, &outs[g], d[g].ldc != N));
    gd[g] = TcGroupDesc{nullptr, nullptr, b, outs[g].dev, d[g].ldc};
    // the experts' rows back to back at a pitch the copy engine accepts
    B2_CUDA(cudaMemcpy2DAsync(X + (size_t)row_off[g] * Kq, (size_t)Kq * 2, src, (size_t)d[g].lda * 2, (size_t)K * 2, (size_t)d[g].M,
                              cudaMemcpyDefault, st));
  }
  for (int g = 0; g < G; ++g) if (d[g].M <= 0) { pws[g] = pws[first]; gd[g] = TcGroupDesc{nullptr, nullptr, nullptr, nullptr, 0}; }
  void *gd_dev = nullptr, *tabs = nullptr;
  B2_TRY(upload_blob(gd.data(), sizeof(TcGroupDesc) * G, st, &gd_dev));
  std::vector<int32_t> both(2 * (G + 1));
  memcpy(both.data(), row_off.data(), sizeof(int32_t) * (G + 1));
  memcpy(both.data() + G + 1, tile_prefix.data(), sizeof(int32_t) * (G + 1));
  B2_TRY(upload_blob(both.data(), both.size() * sizeof(int32_t), st, &tabs));
  const int32_t *row_off_dev = (const int32_t *)tabs, *tile_prefix_dev = row_off_dev + G + 1;
  EpiParams e{};
  e.dst = nullptr; e.ldc = N; e.dst_dt = f->dst_dt;
  for (int g = 0; g < G; ++g) if (d[g].M > 0 && d[g].bias) e.bias_dt = d[g].bias_dt;
  e.n_po = f->n_postops;
  for (int i = 0; i < f->n_postops; ++i) {
    const b200dnn_postop_t &p = f->postops[i];
    e.po[i].type = p.type; e.po[i].dt = p.dt; e.po[i].ld = 0; e.po[i].alpha = p.alpha; e.po[i].beta = p.beta; e.po[i].buff = nullptr;
  }
  B2_TRY(grouped_gemm((const uint8_t *)X, Kq * 2, R, N, 2 * K, pws, row_off_dev, tile_prefix_dev, (const TcGroupDesc *)gd_dev, tile_prefix[G], e,
                      false, st, tile_rows, true));
  bool any = false;
  for (auto &s : outs) {
    if (s.copy_back) { B2_CUDA(cudaMemcpyAsync(s.host, s.dev, s.bytes, cudaMemcpyDeviceToHost, st)); any = true; }
    else if (s.sync) any = true;
  }
  if (any) B2_TRY(check_tc_status(st));
  return B200DNN_SUCCESS;
}

}  // namespace

extern "C" int32_t b200dnn_group_matmul(int32_t G, const b200dnn_matmul_t *d, void *stream) {
  B2_CHECK(G > 0 && d, B200DNN_FAILURE, "group matmul: bad argument");
  if (group_is_uniform(G, d) && env_int("B200DNN_GROUPED_PLAIN", 1) != 0) return group_matmul_grouped(G, d, stream);
  if (group_is_uniform_bf16(G, d) && env_int("B200DNN_GROUPED_PLAIN", 1) != 0) return group_matmul_grouped_bf16(G, d, stream);
  for (int g = 0; g < G; ++g) {
    B2_CHECK(d[g].M >= 0, B200DNN_FAILURE, "group matmul: expert %d has negative M", g);
    if (d[g].M == 0) continue;
    B2_TRY(b200dnn_matmul(&d[g], stream));
  }
  return B200DNN_SUCCESS;
}
