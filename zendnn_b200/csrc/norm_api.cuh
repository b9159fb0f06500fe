// normalization_direct: LayerNorm, RMSNorm, fused-add RMSNorm and inference BatchNorm, the operators on either side of the
// quantised GEMMs in a decoder layer (reference: lowoha_operators/normalization/lowoha_normalization.hpp:98-107, checks
// lowoha_normalization_utils.cpp:23-149, scalar definition kernel/reference_kernel.cpp:98-474).
//   LayerNorm        mean = sum(x)/n, var = sum((x-mean)^2)/n, y = (x-mean) * (1/sqrt(var+eps)) [* gamma] [+ beta]
//   RMSNorm          y = x * (1/sqrt(sum(x^2)/n + eps)) [* gamma]
//   fused-add RMS    residual <- round_to_src(residual + x) (in place); the sum of squares is taken over the unrounded sums,
//                    the output over the rounded residual (reference_kernel.cpp:437-462)
//   BatchNorm        y = (x - running_mean[c]) * (1/sqrt(running_var[c]+eps)) [* gamma[c]] [+ beta[c]], input [N, C, spatial]
// all in f32 with one rounding per operation; sums are block reductions here (the reference adds sequentially), so a result
// may differ from the reference's in the last f32 bit before the final rounding to the destination type.
// With no counterpart in the reference: the normalised row can leave, in the same pass, as per-token quantised s8 with its
// f32 scale (the arithmetic of reorder_direct's dynamic per-token quantisation applied to the row rounded to dst_dt), so that
// norm -> quantise -> W8A8 GEMM costs one read of the activations instead of a write and a second read.
// One CTA per row; the row is staged in shared memory as f32 (rows beyond the shared-memory budget are re-read from global
// memory).  HBM-bound: src + dst bytes per element.  Included at the end of b200dnn.cu.
#pragma once

namespace {

enum : int { NORM_LAYER = 0, NORM_BATCH = 1, NORM_RMS = 2, NORM_FUSED_ADD_RMS = 3 };
constexpr int kNormThreads = 256;
constexpr int kNormSmemElems = 48 * 1024;     // 192 KiB of staged f32

struct NormArgs {
  int type;
  int64_t batch, n;
  float eps;
  int use_scale, use_shift;
  int32_t src_dt, dst_dt, gamma_dt, beta_dt;
  const void *x; void *y; const void *gamma, *beta; void *residual;
  int8_t *q; int64_t q_ld; float *q_scale;     // optional fused per-token quantisation
  int staged;                                  // the row fits the shared-memory stage
};

__device__ __forceinline__ float norm_block_sum(float v, float *sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) r += sh[i];
  __syncthreads();
  return r;
}
__device__ __forceinline__ float norm_block_max(float v, float *sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) r = fmaxf(r, sh[i]);
  __syncthreads();
  return r;
}
__device__ __forceinline__ float norm_block_max_signed(float v, float *sh) {      // values may be negative (scores)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = sh[0];
  for (int i = 1; i < (int)(blockDim.x >> 5); ++i) r = fmaxf(r, sh[i]);
  __syncthreads();
  return r;
}
__device__ __forceinline__ float norm_round_to(float v, int32_t dt) {
  return dt == B200DNN_BF16 ? __uint_as_float(pack_bf16x2(v, 0.0f) << 16) : v;
}
__device__ __forceinline__ void norm_store(void *p, int32_t dt, int64_t i, float v) {
  if (dt == B200DNN_BF16) reinterpret_cast<uint16_t *>(p)[i] = (uint16_t)(pack_bf16x2(v, 0.0f) & 0xFFFFu);
  else reinterpret_cast<float *>(p)[i] = v;
}

__global__ void __launch_bounds__(kNormThreads) norm_rows_kernel(const NormArgs a) {
  extern __shared__ float row[];
  __shared__ float sh[kNormThreads / 32];
  const int64_t n = a.n;
  for (int64_t b = blockIdx.x; b < a.batch; b += gridDim.x) {
    const int64_t off = b * n;
    // ---- pass 1: stage the row (fused add: update the residual) and take the first sum
    float s1 = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
      float v = load_as_f32(a.x, a.src_dt, off + i);
      if (a.type == NORM_FUSED_ADD_RMS) {
        const float sum = __fadd_rn(load_as_f32(a.residual, a.src_dt, off + i), v);
        s1 = __fmaf_rn(sum, sum, s1);
        norm_store(a.residual, a.src_dt, off + i, sum);
        v = norm_round_to(sum, a.src_dt);
      } else if (a.type == NORM_RMS) s1 = __fmaf_rn(v, v, s1);
      else s1 = __fadd_rn(s1, v);
      if (a.staged) row[i] = v;
    }
    s1 = norm_block_sum(s1, sh);
    float mean = 0.f, inv;
    if (a.type == NORM_LAYER) {
      mean = __fdiv_rn(s1, (float)n);
      float s2 = 0.f;
      for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
        const float d = __fadd_rn(a.staged ? row[i] : load_as_f32(a.x, a.src_dt, off + i), -mean);
        s2 = __fmaf_rn(d, d, s2);
      }
      s2 = norm_block_sum(s2, sh);
      inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(s2, (float)n), a.eps)));
    } else inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(s1, (float)n), a.eps)));
    // ---- pass 2: normalise, store; with the fused quantisation keep the rounded result staged and take its abs-max
    float amax = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
      float v;
      if (a.staged) v = row[i];
      else if (a.type == NORM_FUSED_ADD_RMS) v = load_as_f32(a.residual, a.src_dt, off + i);
      else v = load_as_f32(a.x, a.src_dt, off + i);
      float y = __fmul_rn(__fadd_rn(v, -mean), inv);
      if (a.use_scale) y = __fmul_rn(y, load_as_f32(a.gamma, a.gamma_dt, i));
      if (a.use_shift && a.type == NORM_LAYER) y = __fadd_rn(y, load_as_f32(a.beta, a.beta_dt, i));
      if (a.y) norm_store(a.y, a.dst_dt, off + i, y);
      if (a.q) {
        y = norm_round_to(y, a.dst_dt);
        if (finite_f32(y)) amax = fmaxf(amax, fabsf(y));
        row[i] = y;
      }
    }
    if (a.q) {
      const float scale = scale_from_absmax(norm_block_max(amax, sh));     // (the barrier inside also publishes row[])
      for (int64_t i = threadIdx.x; i < n; i += blockDim.x) a.q[b * a.q_ld + i] = quant_sym(row[i], scale);
      if (threadIdx.x == 0) a.q_scale[b] = scale;
    }
    __syncthreads();      // row[] is reused by the next row of this CTA
  }
}

// The decoder-layer case at full width: bf16 rows of at most NV * 8 * blockDim elements, 16-byte aligned, bf16 out.  One
// CTA per row; a thread keeps its NV vectors of eight elements in registers (as the bf16 pairs they are at every stage that
// is kept) between the passes, so the row is read once and every access is a 16-byte vector (8 bytes for the s8 codes).
// Same arithmetic as the generic kernel.
template <int NV>
__global__ void __launch_bounds__(kNormThreads, NV <= 2 ? 6 : (NV <= 4 ? 4 : 2)) norm_rows_vec_kernel(const NormArgs a) {
  __shared__ float sh[kNormThreads / 32];
  const int nvec = (int)(a.n >> 3);
  auto lo = [](uint32_t w) { return __uint_as_float(w << 16); };
  auto hi = [](uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); };
  for (int64_t b = blockIdx.x; b < a.batch; b += gridDim.x) {
    const int64_t off = b * a.n;
    const uint4 *xv = reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(a.x) + off);
    uint4 *rv = a.residual ? reinterpret_cast<uint4 *>(reinterpret_cast<uint16_t *>(a.residual) + off) : nullptr;
    uint32_t v[NV][4];
    float s1 = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      v[j][0] = v[j][1] = v[j][2] = v[j][3] = 0u;
      if (i < nvec) {
        const uint4 q = xv[i];
        v[j][0] = q.x; v[j][1] = q.y; v[j][2] = q.z; v[j][3] = q.w;
      }
    }
    if (a.type == NORM_FUSED_ADD_RMS) {
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nvec) {
          const uint4 r = rv[i];
          const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float s_lo = __fadd_rn(lo(rw[e]), lo(v[j][e])), s_hi = __fadd_rn(hi(rw[e]), hi(v[j][e]));
            s1 = __fmaf_rn(s_lo, s_lo, s1); s1 = __fmaf_rn(s_hi, s_hi, s1);
            v[j][e] = pack_bf16x2(s_lo, s_hi);
          }
          rv[i] = make_uint4(v[j][0], v[j][1], v[j][2], v[j][3]);
        }
      }
    } else if (a.type == NORM_RMS) {
#pragma unroll
      for (int j = 0; j < NV; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) { s1 = __fmaf_rn(lo(v[j][e]), lo(v[j][e]), s1); s1 = __fmaf_rn(hi(v[j][e]), hi(v[j][e]), s1); }
    } else {
#pragma unroll
      for (int j = 0; j < NV; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) { s1 = __fadd_rn(s1, lo(v[j][e])); s1 = __fadd_rn(s1, hi(v[j][e])); }
    }
    s1 = norm_block_sum(s1, sh);
    float mean = 0.f, inv;
    if (a.type == NORM_LAYER) {
      mean = __fdiv_rn(s1, (float)a.n);
      float s2 = 0.f;
#pragma unroll
      for (int j = 0; j < NV; ++j)
        if (threadIdx.x + j * blockDim.x < nvec) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float d0 = __fadd_rn(lo(v[j][e]), -mean), d1 = __fadd_rn(hi(v[j][e]), -mean);
            s2 = __fmaf_rn(d0, d0, s2); s2 = __fmaf_rn(d1, d1, s2);
          }
        }
      s2 = norm_block_sum(s2, sh);
      inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(s2, (float)a.n), a.eps)));
    } else inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(s1, (float)a.n), a.eps)));
    float amax = 0.f;
    const bool layer = a.type == NORM_LAYER, shift = a.use_shift && layer;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < nvec) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {          // two halves of four elements
          float g[4] = {1.f, 1.f, 1.f, 1.f};
          if (a.use_scale) {
            if (a.gamma_dt == B200DNN_F32) {
              const float4 g4 = reinterpret_cast<const float4 *>(a.gamma)[2 * i + h];
              g[0] = g4.x; g[1] = g4.y; g[2] = g4.z; g[3] = g4.w;
            } else {
              const uint2 gq = reinterpret_cast<const uint2 *>(a.gamma)[2 * i + h];
              g[0] = lo(gq.x); g[1] = hi(gq.x); g[2] = lo(gq.y); g[3] = hi(gq.y);
            }
          }
          float bt[4] = {0.f, 0.f, 0.f, 0.f};
          if (shift) {
            if (a.beta_dt == B200DNN_F32) {
              const float4 b4 = reinterpret_cast<const float4 *>(a.beta)[2 * i + h];
              bt[0] = b4.x; bt[1] = b4.y; bt[2] = b4.z; bt[3] = b4.w;
            } else {
              const uint2 bq = reinterpret_cast<const uint2 *>(a.beta)[2 * i + h];
              bt[0] = lo(bq.x); bt[1] = hi(bq.x); bt[2] = lo(bq.y); bt[3] = hi(bq.y);
            }
          }
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const uint32_t w = v[j][2 * h + e];
            float y0 = lo(w), y1 = hi(w);
            if (layer) { y0 = __fadd_rn(y0, -mean); y1 = __fadd_rn(y1, -mean); }
            y0 = __fmul_rn(y0, inv); y1 = __fmul_rn(y1, inv);
            if (a.use_scale) { y0 = __fmul_rn(y0, g[2 * e]); y1 = __fmul_rn(y1, g[2 * e + 1]); }
            if (shift) { y0 = __fadd_rn(y0, bt[2 * e]); y1 = __fadd_rn(y1, bt[2 * e + 1]); }
            const uint32_t o = pack_bf16x2(y0, y1);
            v[j][2 * h + e] = o;
            // rounding to bf16 is monotonic: the largest rounded magnitude is the rounded largest magnitude (a NaN does not
            // enter fmaxf; an infinity does and is dealt with after the loop)
            if (a.q) amax = fmaxf(amax, fmaxf(fabsf(y0), fabsf(y1)));
          }
        }
        if (a.y) reinterpret_cast<uint4 *>(reinterpret_cast<uint16_t *>(a.y) + off)[i] = make_uint4(v[j][0], v[j][1], v[j][2], v[j][3]);
      }
    }
    if (a.q) {
      amax = norm_block_max(amax, sh);
      amax = __uint_as_float(pack_bf16x2(amax, 0.0f) << 16);
      if (!finite_f32(amax)) {
        // an infinite element (it quantises to 0): take the maximum over the finite rounded values instead
        uint32_t mb = 0u;
#pragma unroll
        for (int j = 0; j < NV; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t m0 = (v[j][e] << 16) & 0x7FFFFFFFu, m1 = v[j][e] & 0x7FFF0000u;
            mb = max(mb, m0 < 0x7F800000u ? m0 : 0u);
            mb = max(mb, m1 < 0x7F800000u ? m1 : 0u);
          }
        amax = norm_block_max(__uint_as_float(mb), sh);
      }
      const float scale = scale_from_absmax(amax);
      const float rinv = __frcp_rn(scale);
      // q = rne(v / scale) without a division: m = v * rinv + 1.5 * 2^23 holds the integer nearest to the product in its low
      // byte; d = v * rinv - that integer is the product's distance from it, and whenever |d| < 0.4999 (d^2 < 0.2499, one
      // fused operation whose sign bit is and-ed over the vector) the product and the exact quotient round alike: rinv is
      // the correctly rounded reciprocal, so v * rinv is within 127.5 * 2^-24 < 1e-5 of v / scale.  An element that fails
      // the test, through a near-tie or because it is not finite, takes the exact division.
      const float magic = 12582912.0f;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nvec) {
          uint32_t mbits[8], ok = 0x80000000u;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float v0 = lo(v[j][e]), v1 = hi(v[j][e]);
            const float m0 = __fmaf_rn(v0, rinv, magic), m1 = __fmaf_rn(v1, rinv, magic);
            const float d0 = __fmaf_rn(v0, rinv, __fsub_rn(magic, m0)), d1 = __fmaf_rn(v1, rinv, __fsub_rn(magic, m1));
            const uint32_t c0 = __float_as_uint(__fmaf_rn(d0, d0, -0.2499f)), c1 = __float_as_uint(__fmaf_rn(d1, d1, -0.2499f));
            ok &= c0 & c1;
            mbits[2 * e] = __float_as_uint(m0); mbits[2 * e + 1] = __float_as_uint(m1);
          }
          if (!ok) {
            // only the elements that failed take the division (about two in ten thousand)
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const float ve = (e & 1) ? hi(v[j][e >> 1]) : lo(v[j][e >> 1]);
              const float de = __fmaf_rn(ve, rinv, __fsub_rn(magic, __uint_as_float(mbits[e])));
              if (!(__fmaf_rn(de, de, -0.2499f) < 0.0f)) mbits[e] = (uint32_t)(uint8_t)quant_sym(ve, scale);
            }
          }
          *reinterpret_cast<uint2 *>(a.q + b * a.q_ld + (int64_t)i * 8) =
              make_uint2(low_bytes4(mbits[0], mbits[1], mbits[2], mbits[3]), low_bytes4(mbits[4], mbits[5], mbits[6], mbits[7]));
        }
      }
      if (threadIdx.x == 0) a.q_scale[b] = scale;
    }
  }
}

// BatchNorm: element-wise with per-channel constants
__global__ void norm_batch_kernel(const NormArgs a, const float *mean, const float *var, int64_t C, int64_t spatial) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= a.batch * C * spatial) return;
  const int64_t c = (i / spatial) % C;
  const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var[c], a.eps)));
  float y = __fmul_rn(__fadd_rn(load_as_f32(a.x, a.src_dt, i), -mean[c]), inv);
  if (a.use_scale) y = __fmul_rn(y, load_as_f32(a.gamma, a.gamma_dt, c));
  if (a.use_shift) y = __fadd_rn(y, load_as_f32(a.beta, a.beta_dt, c));
  norm_store(a.y, a.dst_dt, i, y);
}

}  // namespace

extern "C" int32_t b200dnn_normalization(const b200dnn_norm_t *d, void *stream) {
  B2_CHECK(d, B200DNN_FAILURE, "null descriptor");
  B2_ENTER(stream);
  Runtime &R = rt();
  // ---- the reference's checks, in its order and words (lowoha_normalization_utils.cpp:23-149)
  const bool quant = d->quant_dst != nullptr || d->quant_scale != nullptr;
  B2_CHECK(d->input, B200DNN_FAILURE, "Normalization: Input pointer is null");
  B2_CHECK(d->output || quant, B200DNN_FAILURE, "Normalization: Output pointer is null");
  B2_CHECK(d->norm_type >= NORM_LAYER && d->norm_type <= NORM_FUSED_ADD_RMS, B200DNN_FAILURE, "Normalization: norm_type not specified");
  auto known = [](int32_t dt) { return dt == B200DNN_F32 || dt == B200DNN_BF16 || dt == 2 /* f16 */; };
  B2_CHECK(known(d->src_dt), B200DNN_FAILURE, "Normalization: Unsupported source data type");
  B2_CHECK(known(d->dst_dt), B200DNN_FAILURE, "Normalization: Unsupported destination data type");
  B2_CHECK(!((d->src_dt == 2 && d->dst_dt == B200DNN_BF16) || (d->src_dt == B200DNN_BF16 && d->dst_dt == 2)), B200DNN_FAILURE,
           "Normalization: f16/bf16 cross-mixing between src and dst is not supported");
  B2_CHECK(d->batch > 0, B200DNN_FAILURE, "Normalization: batch must be > 0");
  B2_CHECK(d->norm_size > 0, B200DNN_FAILURE, "Normalization: norm_size must be > 0");
  if (d->use_scale) {
    B2_CHECK(d->gamma, B200DNN_FAILURE, "Normalization: use_scale=true but gamma pointer is null");
    B2_CHECK(known(d->gamma_dt), B200DNN_FAILURE, "Normalization: Unsupported gamma data type (%d). Supported: f32, bf16, f16", d->gamma_dt);
  }
  const bool rms = d->norm_type == NORM_RMS || d->norm_type == NORM_FUSED_ADD_RMS;
  if (d->use_shift && !rms) {
    B2_CHECK(d->beta, B200DNN_FAILURE, "Normalization: use_shift=true but beta pointer is null");
    B2_CHECK(known(d->beta_dt), B200DNN_FAILURE, "Normalization: Unsupported beta data type (%d). Supported: f32, bf16, f16", d->beta_dt);
  }
  if (d->norm_type == NORM_FUSED_ADD_RMS)
    B2_CHECK(d->residual, B200DNN_FAILURE, "Normalization: FUSED_ADD_RMS_NORM requires a non-null writable residual buffer");
  if (d->norm_type == NORM_BATCH) {
    B2_CHECK(d->running_mean, B200DNN_FAILURE, "Normalization: BatchNorm inference requires running_mean (pre-computed from training)");
    B2_CHECK(d->running_var, B200DNN_FAILURE, "Normalization: BatchNorm inference requires running_var (pre-computed from training)");
    B2_CHECK(d->num_channels > 0, B200DNN_FAILURE, "Normalization: BatchNorm needs num_channels > 0");
  }
  B2_CHECK(d->epsilon > 0.0f, B200DNN_FAILURE, "Normalization: epsilon must be > 0, got %g", (double)d->epsilon);
  // ---- what this library leaves out
  auto f16 = [](int32_t dt) { return dt == 2; };
  B2_CHECK(!f16(d->src_dt) && !f16(d->dst_dt) && !(d->use_scale && f16(d->gamma_dt)) && !(d->use_shift && !rms && f16(d->beta_dt)),
           B200DNN_UNIMPLEMENTED, "Normalization: f16 buffers are not implemented");
  if (quant) {
    B2_CHECK(d->quant_dst && d->quant_scale, B200DNN_FAILURE, "Normalization: the fused quantisation needs both quant_dst and quant_scale");
    B2_CHECK(d->norm_type != NORM_BATCH, B200DNN_UNIMPLEMENTED, "Normalization: no fused quantisation for BatchNorm");
    B2_CHECK(d->quant_ld >= d->norm_size, B200DNN_FAILURE, "Normalization: quant_ld smaller than norm_size");
    B2_CHECK(d->norm_size <= kNormSmemElems, B200DNN_UNIMPLEMENTED, "Normalization: the fused quantisation stages the row (norm_size <= %d)", kNormSmemElems);
  }

  const int64_t batch = d->batch, n = d->norm_size;
  const int64_t elems = d->norm_type == NORM_BATCH ? batch * d->num_channels * n : batch * n;
  NormArgs a{};
  a.type = d->norm_type; a.batch = batch; a.n = n; a.eps = d->epsilon;
  a.use_scale = d->use_scale ? 1 : 0; a.use_shift = d->use_shift ? 1 : 0;
  a.src_dt = d->src_dt; a.dst_dt = d->dst_dt; a.gamma_dt = d->gamma_dt; a.beta_dt = d->beta_dt;
  const void *p;
  B2_TRY(stage_in(d->input, (size_t)elems * dt_size(d->src_dt), st, &p));
  a.x = p;
  const int64_t n_par = d->norm_type == NORM_BATCH ? d->num_channels : n;
  if (a.use_scale) { B2_TRY(stage_in(d->gamma, (size_t)n_par * dt_size(d->gamma_dt), st, &p)); a.gamma = p; }
  if (a.use_shift && !rms) { B2_TRY(stage_in(d->beta, (size_t)n_par * dt_size(d->beta_dt), st, &p)); a.beta = p; }
  Staged o_y, o_res, o_q, o_s;
  o_y.copy_back = o_res.copy_back = o_q.copy_back = o_s.copy_back = false;
  if (d->output) { B2_TRY(stage_out(d->output, (size_t)elems * dt_size(d->dst_dt), st, &o_y)); a.y = o_y.dev; }
  if (d->norm_type == NORM_FUSED_ADD_RMS) {
    // the residual is read and written: bring a host buffer over first
    B2_TRY(stage_out(d->residual, (size_t)elems * dt_size(d->src_dt), st, &o_res, true));
    a.residual = o_res.dev;
  }
  if (quant) {
    B2_TRY(stage_out(d->quant_dst, (size_t)((batch - 1) * d->quant_ld + n), st, &o_q, d->quant_ld != n));
    B2_TRY(stage_out(d->quant_scale, (size_t)batch * 4, st, &o_s));
    a.q = (int8_t *)o_q.dev; a.q_ld = d->quant_ld; a.q_scale = (float *)o_s.dev;
  }
  if (d->norm_type == NORM_BATCH) {
    const void *m, *v;
    B2_TRY(stage_in(d->running_mean, (size_t)d->num_channels * 4, st, &m));
    B2_TRY(stage_in(d->running_var, (size_t)d->num_channels * 4, st, &v));
    norm_batch_kernel<<<(unsigned)((elems + 255) / 256), 256, 0, st>>>(a, (const float *)m, (const float *)v, d->num_channels, n);
  } else {
    // full-width form: bf16 in and out, whole 16-byte vectors everywhere, at most 8 vectors per thread
    auto al16 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    const bool vec = d->src_dt == B200DNN_BF16 && d->dst_dt == B200DNN_BF16 && n % 8 == 0 && n <= (int64_t)kNormThreads * 64 &&
                     al16(a.x) && al16(a.y) && al16(a.residual) && (!a.use_scale || al16(a.gamma)) && (!(a.use_shift && !rms) || al16(a.beta)) &&
                     (!a.q || (a.q_ld % 8 == 0 && (reinterpret_cast<uintptr_t>(a.q) & 7) == 0)) && env_int("B200DNN_NORM_VEC", 1) != 0;
    if (vec) {
      const int nvec = (int)(n / 8);
      // two vectors per thread before the CTA grows (measured: 58 us for 16384 rows of 4096 against 122 us with four and
      // 195 us with eight: registers, and so resident CTAs, matter more than bytes in flight per thread)
      const int per = env_int("B200DNN_NORM_NV", 2);
      int threads = 32;
      while (threads < kNormThreads && threads * per < nvec) threads <<= 1;
      const int nv = (nvec + threads - 1) / threads;
      const long long cap = (long long)R.sm_count * 64;
      const unsigned grid = (unsigned)(batch < cap ? batch : cap);
      if (nv <= 1) norm_rows_vec_kernel<1><<<grid, threads, 0, st>>>(a);
      else if (nv <= 2) norm_rows_vec_kernel<2><<<grid, threads, 0, st>>>(a);
      else if (nv <= 4) norm_rows_vec_kernel<4><<<grid, threads, 0, st>>>(a);
      else norm_rows_vec_kernel<8><<<grid, threads, 0, st>>>(a);
      B2_LAUNCHED();
      B2_CUDA(cudaGetLastError());
      return finish_out({&o_y, &o_res, &o_q, &o_s}, st);
    }
    a.staged = n <= kNormSmemElems ? 1 : 0;
    const size_t smem = a.staged ? (size_t)n * 4 : 0;
    B2_TRY(ensure_max_smem((const void *)norm_rows_kernel, (size_t)kNormSmemElems * 4));
    // short rows: fewer threads per row, more rows in flight per SM
    int threads = kNormThreads;
    while (threads > 32 && n < threads * 4) threads >>= 1;
    const long long cap = (long long)R.sm_count * 32;
    const unsigned grid = (unsigned)(batch < cap ? batch : cap);
    norm_rows_kernel<<<grid, threads, smem, st>>>(a);
  }
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  return finish_out({&o_y, &o_res, &o_q, &o_s}, st);
}
