// Weight-only quantisation behind matmul_direct: bf16 activations x packed s4 | u4 weights with per-tensor, per-channel or
// per-group ({G,N}) scales and, for u4, zero points; no quantisation of the activations.
// Reference: contract lowoha_matmul_utils.cpp:213-226,314-331 (constant weights required, a zero point is mandatory for
// u4 and is s8 or bf16), backend pre-op setup backends/aocl/aocl_postop.cpp:489-549 (group size from the scale dims),
// scalar definition operators/matmul/matmul_ref_kernel.cpp:359-489: every weight is dequantised to bf16,
//   s4, or u4 with an integer zero point:  w = bf16((q - zp) * scale)      (zp = 0 for s4)
//   u4 with a bf16 zero point:             w = bf16((q - 8) * scale + zp)
// and the product is a bf16 x bf16 GEMM with f32 accumulation.  Here the dequantisation happens once, when the constant
// weight is packed into the tile layout of the tcgen05 kernel's bf16 form (cached by the addresses of weight, scales and
// zero points); the GEMM then is the bf16 path.  The cached pack holds 2 bytes per weight: this form buys the 4-bit
// checkpoint format, not HBM capacity.  Included by b200dnn.cu after bf16_api.cuh.
#pragma once

namespace {

inline bool is_woq_matmul(const b200dnn_matmul_t *d) {
  return d->src_dt == B200DNN_BF16 && (d->wei_dt == B200DNN_S4 || d->wei_dt == B200DNN_U4) && !d->dynamic_quant;
}

struct WoqPackArgs {
  const uint8_t *W4; int64_t ldb; int transB, is_u4;
  int64_t K, N, Kp;
  const void *scale; int32_t scale_dt; int64_t scale_n;
  const void *zp; int32_t zp_dt; int64_t zp_n;
  int64_t group;            // K elements per scale / zero-point group
};

// grid: (Kp/128, Np/32); block 256: a [64 k][32 n] tile, dequantised element by element, written as 128-byte row pieces
__global__ void __launch_bounds__(256) pack_weight_woq_kernel(const WoqPackArgs a, uint8_t *Wt) {
  __shared__ uint16_t tile[32][64 + 2];
  const int64_t k0 = (int64_t)blockIdx.x * 64, n0 = (int64_t)blockIdx.y * 32;
  const int tid = threadIdx.x;
  for (int i = tid; i < 64 * 32; i += 256) {
    const int kk = a.transB ? (i & 63) : (i >> 5), nn = a.transB ? (i >> 6) : (i & 31);
    const int64_t k = k0 + kk, n = n0 + nn;
    uint16_t out = 0;
    if (k < a.K && n < a.N) {
      const int64_t idx = a.transB ? n * a.ldb + k : k * a.ldb + n;
      const uint8_t byte = a.W4[idx >> 1];
      int q = (idx & 1) ? (byte >> 4) : (byte & 0xF);          // even element index: low nibble
      if (!a.is_u4 && (q & 8)) q -= 16;
      const int64_t g = k / a.group;
      const float s = load_as_f32(a.scale, a.scale_dt, a.scale_n == 1 ? 0 : (a.scale_n == a.N ? n : g * a.N + n));
      float w;
      if (a.is_u4) {
        const int64_t zi = a.zp_n == 1 ? 0 : (a.zp_n == a.N ? n : g * a.N + n);
        if (a.zp_dt == B200DNN_BF16) w = __fadd_rn(__fmul_rn((float)(q - 8), s), load_as_f32(a.zp, B200DNN_BF16, zi));
        else w = __fmul_rn(__fadd_rn((float)q, -(float)reinterpret_cast<const int8_t *>(a.zp)[zi]), s);
      } else w = __fmul_rn((float)q, s);
      out = (uint16_t)(pack_bf16x2(w, 0.0f) & 0xFFFFu);
    }
    tile[nn][kk] = out;
  }
  __syncthreads();
  for (int i = tid; i < 32 * 32; i += 256) {
    const int nn = i >> 5, k2 = i & 31;
    const uint32_t v = (uint32_t)tile[nn][2 * k2] | ((uint32_t)tile[nn][2 * k2 + 1] << 16);
    *reinterpret_cast<uint32_t *>(Wt + wt_offset(n0 + nn, (k0 + 2 * k2) * 2, a.Kp)) = v;
  }
}

int32_t validate_woq(const b200dnn_matmul_t *d, int64_t *group) {
  const int M = d->M, N = d->N, K = d->K;
  B2_CHECK(d->src && d->weight && d->dst, B200DNN_FAILURE, "null src, weight or dst");
  B2_CHECK(M > 0 && N > 0 && K > 0, B200DNN_FAILURE, "M, N, K must be positive (got %d, %d, %d)", M, N, K);
  B2_CHECK(d->lda >= K && d->ldc >= N && d->ldb >= (d->transB ? K : N), B200DNN_FAILURE, "leading dimension smaller than the row length");
  B2_CHECK(d->weights_const, B200DNN_FAILURE, "WOQ requires constant weights (is_weights_const=true)");
  B2_CHECK(d->wei_format == 'n' || d->wei_format == 0, B200DNN_UNIMPLEMENTED, "prepacked 4-bit weights are not implemented");
  B2_CHECK(d->dst_dt == B200DNN_BF16 || d->dst_dt == B200DNN_F32, B200DNN_UNIMPLEMENTED, "WOQ writes bf16 or f32 (dst dtype %d)", d->dst_dt);
  B2_CHECK(!d->src_scale.buff && !d->src_zp.buff && !d->dst_scale.buff && !d->dst_zp.buff, B200DNN_FAILURE,
           "Source/destination quantization params are only supported for INT8 (u8/s8 src + s8 weights) or W4A8 (bf16 src + s4 wei)");
  const auto &ws = d->wei_scale;
  B2_CHECK(ws.buff, B200DNN_FAILURE, "WOQ requires quantized weights with scale factors");
  B2_CHECK(ws.dt == B200DNN_F32 || ws.dt == B200DNN_BF16, B200DNN_UNIMPLEMENTED, "weight scale supports f32 or bf16");
  B2_CHECK(ws.count == 1 || (ws.count >= N && ws.count % N == 0), B200DNN_FAILURE, "weight scale dims must be {1}, {1,N} or {G,N} (count %lld, N %d)",
           (long long)ws.count, N);
  const int64_t G = ws.count <= N ? 1 : ws.count / N;
  B2_CHECK(K % G == 0, B200DNN_FAILURE, "WOQ: group_size must divide K (K=%d, G=%lld)", K, (long long)G);
  *group = K / G;
  if (d->wei_dt == B200DNN_U4) {
    B2_CHECK(d->wei_zp.buff, B200DNN_FAILURE, "Weights quant zero is mandatory for u4 weights");
    B2_CHECK(d->wei_zp.dt == B200DNN_BF16 || d->wei_zp.dt == B200DNN_S8, B200DNN_FAILURE,
             "Weights quant zero supports only bf16 or s8 data type (mandatory) for u4 weights");
    B2_CHECK(d->wei_zp.count == 1 || d->wei_zp.count == N || d->wei_zp.count == G * N, B200DNN_FAILURE,
             "weight zero point dims must be {1}, {1,N} or the scale's {G,N}");
  }
  B2_CHECK(!d->bias || d->bias_dt == B200DNN_F32 || d->bias_dt == B200DNN_BF16, B200DNN_UNIMPLEMENTED, "bias dtype %d", d->bias_dt);
  return B200DNN_SUCCESS;
}

int32_t resolve_woq_weight(const b200dnn_matmul_t *d, int64_t group, cudaStream_t st, PackedWeight *pw) {
  DeviceShared &D = *rt().shared;
  const int64_t K = d->K, N = d->N;
  const bool u4 = d->wei_dt == B200DNN_U4;
  auto key = std::make_tuple(d->weight, d->wei_scale.buff, u4 ? d->wei_zp.buff : (const void *)nullptr, K, N, (int64_t)d->ldb,
                             (int)d->transB, (int)d->wei_dt * 256 + (int)d->wei_scale.dt * 16 + (u4 ? (int)d->wei_zp.dt : 0));
  const bool cache = env_int("ZENDNNL_MATMUL_WEIGHT_CACHE", 1) != 0;
  std::unique_lock<std::mutex> lk(D.cache_mu, std::defer_lock);
  if (cache) {
    lk.lock();
    auto it = D.woq_cache.find(key);
    if (it != D.woq_cache.end()) { B2_TRY(wait_ready(it->second, st)); *pw = it->second; return B200DNN_SUCCESS; }
  }
  const int64_t wrows = d->transB ? N : K, wcols = d->transB ? K : N;
  WoqPackArgs a{};
  const void *p;
  B2_TRY(stage_in(d->weight, (size_t)(((wrows - 1) * d->ldb + wcols + 1) / 2), st, &p));
  a.W4 = (const uint8_t *)p; a.ldb = d->ldb; a.transB = d->transB; a.is_u4 = u4 ? 1 : 0;
  a.K = K; a.N = N; a.Kp = round_up(2 * K, 128); a.group = group;
  B2_TRY(stage_in(d->wei_scale.buff, (size_t)d->wei_scale.count * dt_size(d->wei_scale.dt), st, &p));
  a.scale = p; a.scale_dt = d->wei_scale.dt; a.scale_n = d->wei_scale.count;
  if (u4) {
    B2_TRY(stage_in(d->wei_zp.buff, (size_t)d->wei_zp.count * dt_size(d->wei_zp.dt), st, &p));
    a.zp = p; a.zp_dt = d->wei_zp.dt; a.zp_n = d->wei_zp.count;
  }
  const int64_t Np = round_up(N, 128);
  void *buf = nullptr;
  if (cache) B2_CUDA(cudaMalloc(&buf, pack_bytes_bf16(K, N)));
  else { buf = rt().ws.alloc(pack_bytes_bf16(K, N)); B2_CHECK(buf, B200DNN_FAILURE, "workspace allocation failed"); }
  dim3 grid((unsigned)(a.Kp / 128), (unsigned)(Np / 32));
  pack_weight_woq_kernel<<<grid, 256, 0, st>>>(a, (uint8_t *)buf);
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  *pw = PackedWeight{};
  pw->wt = (const int8_t *)buf; pw->K = K; pw->N = N; pw->Kp = a.Kp; pw->Np = Np;
  if (cache) { pw->owned = buf; B2_TRY(mark_ready(*pw, st)); D.woq_cache.emplace(key, *pw); }
  return B200DNN_SUCCESS;
}

int32_t matmul_woq(const b200dnn_matmul_t *d, cudaStream_t st) {
  int64_t group = 0;
  B2_TRY(validate_woq(d, &group));
  // everything else (post-ops, bias, destination) follows the bf16 path's rules
  b200dnn_matmul_t probe = *d;
  probe.wei_dt = B200DNN_BF16; probe.wei_scale = b200dnn_quant_t{}; probe.wei_zp = b200dnn_quant_t{};
  B2_TRY(validate_bf16_matmul(&probe));
  PackedWeight pw;
  B2_TRY(resolve_woq_weight(d, group, st, &pw));
  return matmul_bf16_packed(d, pw, st);
}

}  // namespace
