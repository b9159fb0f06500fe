// bf16 x bf16 matmul_direct: the reference's non-quantised path for the same entry point (lowoha_matmul.cpp:278 with
// dtypes bf16:bf16:bf16|f32; its micro-kernel for grouped GEMMs is matmul/group_matmul/custom_kernel/ukernel/
// bf16_microkernel.cpp), here on the same tcgen05 kernel as the INT8 path in its bf16 form: kind::f16 MMAs with f32
// accumulators over the same 128-byte K tiles, C = post_ops(A·B + bias), bf16 or f32 out.  No scales and no zero points:
// the reference refuses source / destination quantisation parameters outside INT8 and W4A8
// (lowoha_matmul_utils.cpp:227-233).  Included by b200dnn.cu before the C ABI.
#pragma once

namespace {

constexpr int kLayoutBf16 = 32;    // weight-cache layout code of a bf16 pack (added to the gated code)

inline bool is_bf16_matmul(const b200dnn_matmul_t *d) {
  return d->src_dt == B200DNN_BF16 && d->wei_dt == B200DNN_BF16 && !d->dynamic_quant;
}

inline size_t pack_bytes_bf16(int64_t K, int64_t N) {
  const int64_t Kp = round_up(2 * K, 128), Np = round_up(N, 128);
  return (size_t)Np * Kp;
}

// weight [K,N] (or [N,K] with transB) in bf16 -> cached tile layout; Kp counts bytes
int32_t resolve_bf16_weight(const void *weight, int64_t K, int64_t N, int64_t ldb, int transB, int gated, int weights_const,
                            cudaStream_t st, PackedWeight *pw) {
  DeviceShared &D = *rt().shared;
  auto key = std::make_tuple(weight, K, N, ldb, transB, gated + kLayoutBf16);
  const bool cache = weights_const && env_int("ZENDNNL_MATMUL_WEIGHT_CACHE", 1) != 0;
  std::unique_lock<std::mutex> lk(D.cache_mu, std::defer_lock);
  if (cache) {
    lk.lock();
    auto it = D.wcache.find(key);
    if (it != D.wcache.end()) { B2_TRY(wait_ready(it->second, st)); *pw = it->second; return B200DNN_SUCCESS; }
  }
  const int64_t I = gated ? N / 2 : 0;
  if (gated) B2_CHECK(N % 2 == 0 && I % kGateGranule == 0, B200DNN_UNIMPLEMENTED,
                      "gated weights need N = 2*I with I a multiple of %d (N=%lld)", kGateGranule, (long long)N);
  const int64_t wrows = transB ? N : K, wcols = transB ? K : N;
  const void *w_dev = nullptr;
  B2_TRY(stage_in(weight, span_bytes(wrows, wcols, ldb, B200DNN_BF16), st, &w_dev));
  const int64_t Kp = round_up(2 * K, 128), Np = round_up(N, 128);
  void *buf = nullptr;
  if (cache) B2_CUDA(cudaMalloc(&buf, pack_bytes_bf16(K, N)));
  else { buf = rt().ws.alloc(pack_bytes_bf16(K, N)); B2_CHECK(buf, B200DNN_FAILURE, "workspace allocation failed"); }
  dim3 grid((unsigned)(Kp / 128), (unsigned)(Np / 32));
  pack_weight_bf16_kernel<<<grid, 256, 0, st>>>((const uint16_t *)w_dev, ldb, transB, K, N, Kp, gated, I, (uint8_t *)buf);
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  *pw = PackedWeight{};
  pw->wt = (const int8_t *)buf; pw->K = K; pw->N = N; pw->Kp = Kp; pw->Np = Np; pw->gated = gated; pw->I = I;
  if (cache) { pw->owned = buf; B2_TRY(mark_ready(*pw, st)); D.wcache.emplace(key, *pw); }
  return B200DNN_SUCCESS;
}

// rows of 2-byte elements copied to a pitch the copy engine accepts (16-byte multiple, 16-byte aligned base)
__global__ void repitch_rows_u16_kernel(const uint16_t *src, int64_t src_ld, uint16_t *dst, int64_t dst_ld, int64_t rows, int64_t cols) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * dst_ld) return;
  const int64_t r = i / dst_ld, c = i - r * dst_ld;
  dst[i] = c < cols ? src[r * src_ld + c] : (uint16_t)0;
}

int32_t validate_bf16_matmul(const b200dnn_matmul_t *d) {
  const int M = d->M, N = d->N, K = d->K;
  B2_CHECK(d->src && d->weight && d->dst, B200DNN_FAILURE, "null src, weight or dst");
  B2_CHECK(M > 0 && N > 0 && K > 0, B200DNN_FAILURE, "M, N, K must be positive (got %d, %d, %d)", M, N, K);
  B2_CHECK(d->lda >= K && d->ldc >= N, B200DNN_FAILURE, "lda/ldc smaller than the row length");
  B2_CHECK(d->ldb >= (d->transB ? K : N), B200DNN_FAILURE, "ldb smaller than the row length");
  B2_CHECK(d->wei_format == 'n' || d->wei_format == 0, B200DNN_UNIMPLEMENTED, "prepacked bf16 weights are not implemented: pass the caller's layout, the library caches its pack");
  B2_CHECK(d->dst_dt == B200DNN_BF16 || d->dst_dt == B200DNN_F32, B200DNN_UNIMPLEMENTED, "bf16 matmul writes bf16 or f32 (dst dtype %d)", d->dst_dt);
  B2_CHECK(!d->src_scale.buff && !d->src_zp.buff && !d->dst_scale.buff && !d->dst_zp.buff, B200DNN_FAILURE,
           "Source/destination quantization params are only supported for INT8 (u8/s8 src + s8 weights) or W4A8 (bf16 src + s4 wei)");
  B2_CHECK(!d->wei_scale.buff, B200DNN_UNIMPLEMENTED, "weight scales on a bf16 weight are not implemented");
  B2_CHECK(!d->bias || d->bias_dt == B200DNN_F32 || d->bias_dt == B200DNN_BF16, B200DNN_UNIMPLEMENTED, "bias dtype %d", d->bias_dt);
  B2_CHECK(d->n_postops >= 0 && d->n_postops <= B200DNN_MAX_POSTOPS, B200DNN_FAILURE, "too many post-ops");
  for (int i = 0; i < d->n_postops; ++i) {
    const b200dnn_postop_t &p = d->postops[i];
    switch (p.type) {
    case PO_RELU: case PO_LEAKY_RELU: case PO_GELU_TANH: case PO_GELU_ERF: case PO_SIGMOID: case PO_SWISH: case PO_TANH: case PO_ELU:
    case PO_MISH: break;
    case PO_CLIP: B2_CHECK(!diagnostics_enabled() || (std::isfinite(p.alpha) && std::isfinite(p.beta)), B200DNN_FAILURE, "clip bounds must be finite"); break;
    case PO_BINARY_ADD: case PO_BINARY_MUL:
      B2_CHECK(p.buff && (p.dt == B200DNN_F32 || p.dt == B200DNN_BF16), B200DNN_FAILURE, "binary post-op needs an f32 or bf16 operand");
      B2_CHECK(p.ld == 0 || p.ld >= N, B200DNN_FAILURE, "binary post-op leading dimension");
      break;
    default: return fail(B200DNN_UNIMPLEMENTED, "post-op %d is not implemented", p.type);
    }
  }
  return B200DNN_SUCCESS;
}

// the GEMM over a weight that already sits in the tile layout as bf16 (a packed bf16 weight, or 4-bit weights dequantised
// at pack time)
int32_t matmul_bf16_packed(const b200dnn_matmul_t *d, const PackedWeight &pw, cudaStream_t st) {
  Runtime &R = rt();
  const int M = d->M, N = d->N, K = d->K;
  EpiParams epi;
  fill_epi(d, &epi);
  const void *src_dev = nullptr;
  B2_TRY(stage_in(d->src, span_bytes(M, K, d->lda, B200DNN_BF16), st, &src_dev, &R.small));
  if (d->bias) { const void *p; B2_TRY(stage_in(d->bias, (size_t)N * dt_size(d->bias_dt), st, &p, &R.small)); epi.bias = p; }
  for (int i = 0; i < d->n_postops; ++i) {
    const b200dnn_postop_t &p = d->postops[i];
    epi.po[i].type = p.type; epi.po[i].dt = p.dt; epi.po[i].ld = p.ld; epi.po[i].alpha = p.alpha; epi.po[i].beta = p.beta;
    epi.po[i].buff = nullptr;
    if (p.type == PO_BINARY_ADD || p.type == PO_BINARY_MUL) {
      const void *b;
      B2_TRY(stage_in(p.buff, p.ld ? span_bytes(M, N, p.ld, p.dt) : (size_t)N * dt_size(p.dt), st, &b, &R.small));
      epi.po[i].buff = b;
    }
  }
  Staged o_dst;
  B2_TRY(stage_out(d->dst, span_bytes(M, N, d->ldc, d->dst_dt), st, &o_dst, d->ldc != N));
  epi.dst = o_dst.dev;
  B2_TRY(R.small.flush(st, o_dst.copy_back || o_dst.sync));

  // the copy engine wants 16-byte aligned rows: other sources are copied to such a pitch first
  const uint8_t *A = (const uint8_t *)src_dev;
  int64_t lda = d->lda;
  if ((reinterpret_cast<uintptr_t>(A) & 15) != 0 || (lda * 2) % 16 != 0) {
    const int64_t ld2 = round_up(K, 8);
    uint16_t *tmp = (uint16_t *)R.ws.alloc((size_t)M * ld2 * 2);
    B2_CHECK(tmp, B200DNN_FAILURE, "workspace allocation failed");
    const int64_t n = (int64_t)M * ld2;
    repitch_rows_u16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>((const uint16_t *)src_dev, d->lda, tmp, ld2, M, K);
    B2_LAUNCHED();
    B2_CUDA(cudaGetLastError());
    A = (const uint8_t *)tmp; lda = ld2;
  }
  TcGemmArgs ta{};
  const int tile_rows = tc_tile_rows(M, N);
  ta.pair = tile_rows > kTcBM ? 1 : 0;
  ta.f16 = 1;
  ta.n_groups = 1; ta.m_tiles_plain = (M + tile_rows - 1) / tile_rows; ta.shared_dst = 1;
  B2_TRY(launch_tc(A, lda * 2, false, M, N, 2 * K, pw, ta, epi, ta.m_tiles_plain, st));
  return finish_out({&o_dst}, st);
}

int32_t matmul_bf16(const b200dnn_matmul_t *d, cudaStream_t st) {
  B2_TRY(validate_bf16_matmul(d));
  PackedWeight pw;
  B2_TRY(resolve_bf16_weight(d->weight, d->K, d->N, d->ldb, d->transB, 0, d->weights_const, st, &pw));
  return matmul_bf16_packed(d, pw, st);
}

}  // namespace
