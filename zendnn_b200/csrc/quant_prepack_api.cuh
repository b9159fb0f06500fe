// Float weight -> per-channel s8 -> packed tile layout in one entry: the reference's weight preparation for the INT8
// path is a dynamic per-channel quantisation (reorder/lowoha_reorder.cpp:186, scale dims {1,N}) followed by the prepack
// reorder (reorder/prepack/lowoha_prepack.cpp:315).  Run as two calls that costs a write and a re-read of the s8 matrix;
// here the pack kernel quantises as it transposes, so the weight is read twice (column maxima, then pack) and only the
// packed form is written.  The bytes are those of b200dnn_quant_dynamic followed by b200dnn_prepack: same abs-max,
// same scale (scale_from_absmax), same division and rounding.  Included by b200dnn.cu after the C ABI's helpers.
#pragma once

namespace {

// abs-max of every row of a [rows, cols] matrix: one warp per row (the transB form, where a channel is a stored row)
template <typename T>
__global__ void __launch_bounds__(256) absmax_rows_kernel(const T *src, int64_t rows, int64_t cols, int64_t ld, uint32_t *out) {
  const int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  float amax = 0.f;
  for (int64_t c = lane; c < cols; c += 32) {
    const float f = elem_to_f32<T>(src[r * ld + c]);
    if (finite_f32(f)) amax = fmaxf(amax, fabsf(f));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (lane == 0) out[r] = __float_as_uint(amax);
}

// abs-max of every column of a [rows, cols] matrix with 16-byte loads: a thread owns 16/sizeof(T) neighbouring columns
// over the rows of its blockIdx.y slice, so a warp reads 512 contiguous bytes of each row.  The caller checks that the
// base is 16-byte aligned and that cols and ld are multiples of 16/sizeof(T).  out must be zero before the launch.
template <typename T>
__global__ void __launch_bounds__(256) absmax_cols_vec_kernel(const T *src, int64_t rows, int64_t cols, int64_t ld, uint32_t *out) {
  constexpr int E = 16 / (int)sizeof(T);
  const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (g * E >= cols) return;
  const int64_t rows_per = (rows + gridDim.y - 1) / gridDim.y;
  const int64_t m0 = (int64_t)blockIdx.y * rows_per, m1 = min(rows, m0 + rows_per);
  float amax[E];
#pragma unroll
  for (int i = 0; i < E; ++i) amax[i] = 0.f;
#pragma unroll 4
  for (int64_t m = m0; m < m1; ++m) {
    const uint4 v = *reinterpret_cast<const uint4 *>(src + m * ld + g * E);
    const T *e = reinterpret_cast<const T *>(&v);
#pragma unroll
    for (int i = 0; i < E; ++i) {
      const float f = elem_to_f32<T>(e[i]);
      if (finite_f32(f)) amax[i] = fmaxf(amax[i], fabsf(f));
    }
  }
#pragma unroll
  for (int i = 0; i < E; ++i) atomicMax(out + g * E + i, __float_as_uint(amax[i]));
}

__device__ __forceinline__ int8_t quant_channel(float v, float s) {
  const int q = __float2int_rn(__fdiv_rn(v, s));
  return (int8_t)max(-128, min(127, q));
}

// The same code without a division in the common case (the argument of quant_sym_r: the scale comes from the abs-max of
// the channel itself, so every finite |v/s| <= 127 up to rounding, and away from a near-tie v*rinv rounds to the integer
// the rounded quotient rounds to).  Near-ties and non-finite inputs take the division.
__device__ __forceinline__ int8_t quant_channel_r(float v, float s, float rinv) {
  const float magic = 12582912.0f;
  const float qa = v * rinv, m = qa + magic, t = m - magic;
  if (fabsf(qa - t) < 0.4999f) return (int8_t)(__float_as_int(m) & 0xFF);
  return quant_channel(v, s);
}

// pack_weight_kernel with the quantisation in its load: grid (Np/32, Kp/64), block 256, a [64 k][32 n] tile per CTA.
// Tiles that neighbour along n are neighbours in launch order: for the [K,N] form they read adjacent runs of the same
// rows of the weight.
template <typename T>
__global__ void __launch_bounds__(256) pack_quant_weight_kernel(const T *W, int64_t ldb, int transB, int64_t K, int64_t N, int64_t Kp,
                                                                int gated, int64_t I, const float *scale, int8_t *Wt) {
  __shared__ int8_t tile[32][64 + 4];
  const int64_t k0 = (int64_t)blockIdx.y * 64, pn0 = (int64_t)blockIdx.x * 32;
  const int64_t n0 = packed_to_logical(pn0, gated, I);
  const int64_t nstep = gated == 2 ? 2 : 1;
  const int tid = threadIdx.x;
  __shared__ float s_scale[32], s_rinv[32];
  if (tid < 32) {
    const float sc = pn0 + tid < N ? scale[n0 + tid * nstep] : 1.f;
    s_scale[tid] = sc; s_rinv[tid] = __frcp_rn(sc);
  }
  __syncthreads();
  if (!transB) {
    const int nn = tid & 31;                    // fixed per thread: 256 is a multiple of 32
    const int64_t n = n0 + nn * nstep;
    const bool n_ok = pn0 + nn < N;
    const float sc = s_scale[nn], rinv = s_rinv[nn];
#pragma unroll
    for (int kk = tid >> 5; kk < 64; kk += 8) {
      const int64_t k = k0 + kk;
      tile[nn][kk] = (k < K && n_ok) ? quant_channel_r(elem_to_f32<T>(W[k * ldb + n]), sc, rinv) : (int8_t)0;
    }
  } else {
    const int kk = tid & 63;
    const int64_t k = k0 + kk;
#pragma unroll
    for (int nn = tid >> 6; nn < 32; nn += 4) {
      const int64_t n = n0 + nn * nstep;
      tile[nn][kk] = (k < K && pn0 + nn < N) ? quant_channel_r(elem_to_f32<T>(W[n * ldb + k]), s_scale[nn], s_rinv[nn]) : (int8_t)0;
    }
  }
  __syncthreads();
  for (int i = tid; i < 32 * 16; i += 256) {
    const int nn = i >> 4, k4 = i & 15;
    const int8_t *t = &tile[nn][k4 * 4];
    const uint32_t v = (uint32_t)(uint8_t)t[0] | ((uint32_t)(uint8_t)t[1] << 8) | ((uint32_t)(uint8_t)t[2] << 16) |
                       ((uint32_t)(uint8_t)t[3] << 24);
    *reinterpret_cast<uint32_t *>(Wt + wt_offset(pn0 + nn, k0 + k4 * 4, Kp)) = v;
  }
}

template <typename T>
int32_t quant_pack_launch(const T *w, int64_t K, int64_t N, int64_t ldb, int transB, int gated, int64_t I, float *scale_dev,
                          uint8_t *base, cudaStream_t st, PackedWeight *pw) {
  const int64_t Kp = round_up(K, 128), Np = round_up(N, 128);
  uint32_t *amax = (uint32_t *)rt().ws.alloc((size_t)N * 4);
  B2_CHECK(amax, B200DNN_FAILURE, "workspace allocation failed");
  if (transB) {
    absmax_rows_kernel<T><<<(unsigned)((N + 7) / 8), 256, 0, st>>>(w, N, K, ldb, amax);
  } else {
    B2_CUDA(cudaMemsetAsync(amax, 0, (size_t)N * 4, st));
    constexpr int E = 16 / (int)sizeof(T);
    const unsigned slices = (unsigned)(K < 64 ? 1 : (K / 64 > 256 ? 256 : K / 64));
    if ((reinterpret_cast<uintptr_t>(w) & 15) == 0 && N % E == 0 && ldb % E == 0) {
      dim3 grid((unsigned)((N / E + 255) / 256), slices);
      absmax_cols_vec_kernel<T><<<grid, 256, 0, st>>>(w, K, N, ldb, amax);
    } else {
      dim3 grid((unsigned)((N + 255) / 256), slices);
      absmax_cols_kernel<T><<<grid, 256, 0, st>>>(w, K, N, ldb, 1, amax);
    }
  }
  B2_LAUNCHED();
  scales_from_absmax_kernel<<<(unsigned)((N + 255) / 256), 256, 0, st>>>(amax, N, scale_dev);
  B2_LAUNCHED();
  int32_t *colsum = reinterpret_cast<int32_t *>(base + kPackHeaderBytes);
  int8_t *wt = reinterpret_cast<int8_t *>(base + kPackHeaderBytes + Np * 4);
  pack_header_kernel<<<1, kPackHeaderBytes / 4, 0, st>>>(reinterpret_cast<PackHeader *>(base), K, N, Kp, Np, gated, I);
  B2_LAUNCHED();
  B2_CHECK(Kp / 64 <= 65535, B200DNN_UNIMPLEMENTED, "quant_prepack: K=%lld is too large", (long long)K);
  dim3 pgrid((unsigned)(Np / 32), (unsigned)(Kp / 64));
  pack_quant_weight_kernel<T><<<pgrid, 256, 0, st>>>(w, ldb, transB, K, N, Kp, gated, I, scale_dev, wt);
  B2_LAUNCHED();
  pack_colsum_kernel<<<(unsigned)((Np + 7) / 8), 256, 0, st>>>(wt, Np, Kp, colsum);
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  *pw = PackedWeight{};
  pw->colsum = colsum; pw->wt = wt; pw->K = K; pw->N = N; pw->Kp = Kp; pw->Np = Np; pw->gated = gated; pw->I = I;
  return B200DNN_SUCCESS;
}

}  // namespace

extern "C" int32_t b200dnn_quant_prepack(const void *weight, int32_t wei_dt, int64_t K, int64_t N, int64_t ldb, int32_t transB,
                                         int32_t gated, void *dst, float *scale, void *stream) {
  B2_ENTER(stream);
  B2_CHECK(weight && dst && scale && K > 0 && N > 0, B200DNN_FAILURE, "quant_prepack: null pointer or non-positive dimension");
  B2_CHECK(wei_dt == B200DNN_BF16 || wei_dt == B200DNN_F32, B200DNN_UNIMPLEMENTED, "quant_prepack: weight must be f32 or bf16");
  B2_CHECK(ldb >= (transB ? K : N), B200DNN_FAILURE, "quant_prepack: ldb=%lld too small", (long long)ldb);
  B2_CHECK(gated >= 0 && gated <= 2, B200DNN_FAILURE, "quant_prepack: gated must be 0, 1 or 2");
  const int64_t I = gated ? N / 2 : 0;
  if (gated) B2_CHECK(N % 2 == 0 && I % kGateGranule == 0, B200DNN_UNIMPLEMENTED,
                      "gated prepack needs N = 2*I with I a multiple of %d (N=%lld)", kGateGranule, (long long)N);
  const void *w_dev = nullptr;
  B2_TRY(stage_in(weight, span_bytes(transB ? N : K, transB ? K : N, ldb, wei_dt), st, &w_dev));
  Staged out, o_s;
  B2_TRY(stage_out(dst, pack_bytes(K, N), st, &out));
  B2_TRY(stage_out(scale, (size_t)N * 4, st, &o_s));
  B2_CHECK((reinterpret_cast<uintptr_t>(out.dev) & 255) == 0, B200DNN_FAILURE, "prepack destination must be 256-byte aligned");
  PackedWeight pw;
  if (wei_dt == B200DNN_BF16)
    B2_TRY(quant_pack_launch<uint16_t>((const uint16_t *)w_dev, K, N, ldb, transB, gated, I, (float *)o_s.dev, (uint8_t *)out.dev, st, &pw));
  else
    B2_TRY(quant_pack_launch<float>((const float *)w_dev, K, N, ldb, transB, gated, I, (float *)o_s.dev, (uint8_t *)out.dev, st, &pw));
  {
    DeviceShared &D = *rt().shared;
    std::lock_guard<std::mutex> lk(D.cache_mu);
    if (!out.copy_back && !out.sync) D.packed_registry[dst] = pw;
    else {
      auto it = D.host_packed.find(dst);
      if (it != D.host_packed.end()) { if (it->second.owned) cudaFree(it->second.owned); if (it->second.ready) cudaEventDestroy(it->second.ready); D.host_packed.erase(it); }
    }
  }
  return finish_out({&out, &o_s}, st);
}
