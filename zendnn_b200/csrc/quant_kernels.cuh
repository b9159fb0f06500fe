// Memory-bound quantisation kernels behind reorder_direct / group_dynamic_quant.
//
//  - per-token symmetric dynamic quantisation (one pass over the row: the row is held in
//    registers between the abs-max reduction and the quantise step);
//    reference: reorder/reorder_data_type/scalar_impl/dynamic_per_token_ref_kernel.cpp:31-36,70-124
//    and the AVX-512 form dynamic_quant_impl/per_token_avx512_f32_fma_kernel.cpp:207-300.
//  - per-channel / per-tensor dynamic scales: reorder/lowoha_reorder_utils.cpp:708-766,908-935.
//  - static quantise / dequantise: reorder/lowoha_reorder_utils.hpp:148-153,
//    reorder_data_type/scalar_impl/scalar_ref_kernels.cpp:28-56.
//
// Arithmetic contract: abs-max over finite values, clamp to 1e-10, scale = absmax / 127 (IEEE
// division), clamp to 1e-10, q = rne(v / scale) with IEEE division; non-finite inputs give 0.
#pragma once
#include "common.cuh"

namespace b200 {

__device__ __forceinline__ float scale_from_absmax(float absmax) {
  if (absmax < 1e-10f) absmax = 1e-10f;
  float s = __fdiv_rn(absmax, 127.0f);
  if (s < 1e-10f) s = 1e-10f;
  return s;
}
__device__ __forceinline__ int8_t quant_sym(float v, float scale) {
  if (!finite_f32(v)) return 0;
  return (int8_t)__float2int_rn(__fdiv_rn(v, scale));
}
// Same result as quant_sym without a division or a conversion instruction in the common case, for a scale that
// comes from the abs-max of the row itself (so |v/scale| <= 127 up to rounding).  rinv = __frcp_rn(scale).
// rinv is the correctly rounded reciprocal, so v*rinv, its rounding and the rounded quotient v/scale all lie within
// 3 * 127.5 * 2^-24 < 2.3e-5 of the true quotient: whenever v*rinv is at least 1e-4 away from a half integer they round to the
// same integer; adding 1.5*2^23 rounds to that integer (nearest-even) and leaves its two's complement in the low mantissa
// byte.  The rare near-tie (two elements in ten thousand) and every non-finite input take the exact division.
__device__ __forceinline__ int8_t quant_sym_r(float v, float scale, float rinv) {
  const float magic = 12582912.0f;
  const float qa = v * rinv, m = qa + magic, t = m - magic;
  if (fabsf(qa - t) < 0.4999f) return (int8_t)(__float_as_int(m) & 0xFF);
  return quant_sym(v, scale);
}

// The same fast path for a whole 16-byte vector, on packed f32x2 arithmetic: per pair of elements
//   m = v*rinv + 1.5*2^23 (one fused rounding: the integer nearest to the product), t' = 1.5*2^23 - m = -round,
//   d = v*rinv + t' (the product's distance from that integer),
// three packed instructions instead of eight scalar ones, and ONE near-tie test per vector: the largest |d| (a
// NaN-propagating maximum, so non-finite inputs fail the test as well) must stay below 0.4999 (a wider band, 0.499, sent
// two vectors in a hundred, and with them four warps in ten, through the divisions).  Returns false when the
// vector needs the exact division; o[] then holds nothing useful.
__device__ __forceinline__ uint64_t f32x2_pack(float lo, float hi) { uint64_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
__device__ __forceinline__ void f32x2_unpack(uint64_t r, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(r)); }
__device__ __forceinline__ uint64_t f32x2_fma(uint64_t a, uint64_t b, uint64_t c) { uint64_t d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__device__ __forceinline__ float max_nan_abs(float e, float d) { float r; asm("{ .reg .f32 t; abs.f32 t, %2; max.NaN.f32 %0, %1, t; }" : "=f"(r) : "f"(e), "f"(d)); return r; }

template <int PAIRS>
__device__ __forceinline__ bool quant_pairs_fast(const float (&v)[2 * PAIRS], float rinv, uint32_t (&m_bits)[2 * PAIRS]) {
  const uint64_t rinv2 = f32x2_pack(rinv, rinv), magic2 = f32x2_pack(12582912.0f, 12582912.0f), neg1 = f32x2_pack(-1.0f, -1.0f);
  float e = 0.f;
#pragma unroll
  for (int p = 0; p < PAIRS; ++p) {
    const uint64_t v2 = f32x2_pack(v[2 * p], v[2 * p + 1]);
    const uint64_t m2 = f32x2_fma(v2, rinv2, magic2);
    const uint64_t tn = f32x2_fma(m2, neg1, magic2);
    const uint64_t d2 = f32x2_fma(v2, rinv2, tn);
    float m0, m1, d0, d1;
    f32x2_unpack(m2, m0, m1); f32x2_unpack(d2, d0, d1);
    m_bits[2 * p] = __float_as_uint(m0); m_bits[2 * p + 1] = __float_as_uint(m1);
    e = max_nan_abs(max_nan_abs(e, d0), d1);
  }
  return e < 0.4999f;
}
// low bytes of four words -> one word
__device__ __forceinline__ uint32_t low_bytes4(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}
// 8 bf16 (one uint4) -> 8 s8 (uint2); 4 f32 (one uint4) -> 4 s8 (one word)
__device__ __forceinline__ bool quant_vec_fast(const uint4 &q, float rinv, uint2 *out, uint16_t /*tag: bf16*/) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  float v[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
  uint32_t m[8];
  const bool ok = quant_pairs_fast<4>(v, rinv, m);
  out->x = low_bytes4(m[0], m[1], m[2], m[3]); out->y = low_bytes4(m[4], m[5], m[6], m[7]);
  return ok;
}
__device__ __forceinline__ bool quant_vec_fast(const uint4 &q, float rinv, uint32_t *out, float /*tag: f32*/) {
  const float v[4] = {__uint_as_float(q.x), __uint_as_float(q.y), __uint_as_float(q.z), __uint_as_float(q.w)};
  uint32_t m[4];
  const bool ok = quant_pairs_fast<2>(v, rinv, m);
  *out = low_bytes4(m[0], m[1], m[2], m[3]);
  return ok;
}

// Where the rows of one per-token quantisation come from and go to.  Rows can be a plain
// strided matrix, a gather of rows of a matrix (MoE dispatch), or the concatenation of several
// matrices (group_dynamic_quant / the per-expert src[] of group_matmul_direct).
struct RowQuantArgs {
  const void *src; int64_t src_ld;      // plain / gather source
  const int32_t *gather;                // optional: source row of output row r (entries < 0: row skipped)
  int32_t gather_div;                   // source row = gather_src[r] / gather_div (slot -> token)
  int8_t *dst; int64_t dst_ld;          // may be null (scales only)
  void *scale; int32_t scale_dt;        // f32 or bf16, one per row
  const uint32_t *absmax_bits;          // optional: per-row abs-max already known (float bits)
  // scatter form: source row r is quantised once and written to the rows scatter[r*scatter_n + j] of dst / scale
  // (entries < 0 skipped): a token routed to several experts is quantised once, not once per expert
  const int32_t *scatter; int32_t scatter_n; int32_t scatter_rows;
  // scatter across GPUs (expert-parallel dispatch): destination j of source row r lives on peer scatter_peer[r*scatter_n+j],
  // whose row buffers are peer_dst / peer_scale (addresses of peer memory mapped into this process; plain stores cross
  // NVLink).  Rows at or beyond scatter_cap are not written (the receiver's buffer ends there); *overflow is set instead.
  const int32_t *scatter_peer; int8_t *peer_dst[8]; float *peer_scale[8]; int32_t scatter_cap; int32_t *overflow;
  // number of rows when only the device knows it (rows received from other GPUs): the grid then strides over the rows
  const int32_t *n_rows_dev;
  int32_t K;
  // grouped form (used when n_groups > 0): row r belongs to the group with row_off[g] <= r < row_off[g+1]
  int32_t n_groups;
  const void *const *g_src; const int64_t *g_src_ld;
  void *const *g_dst; const int64_t *g_dst_ld;
  void *const *g_scale;
  const int32_t *row_off;
};

constexpr int kQuantThreads = 256;
constexpr int kQuantRegVec = 8;   // 16-byte vectors cached per thread

template <typename T> struct VecTraits;
template <> struct VecTraits<uint16_t> { static constexpr int kPer16B = 8; };
template <> struct VecTraits<float> { static constexpr int kPer16B = 4; };

template <typename T> __device__ __forceinline__ float elem_to_f32(T v);
template <> __device__ __forceinline__ float elem_to_f32<uint16_t>(uint16_t v) { return bf16_bits_to_f32(v); }
template <> __device__ __forceinline__ float elem_to_f32<float>(float v) { return v; }

// One 16-byte vector of the row: the packed fast path, or the exact division for a vector with a near-tie or a
// non-finite element.
template <typename T>
__device__ __forceinline__ void quant_vec(const uint4 &q, float scale, float rinv, int8_t (&o)[VecTraits<T>::kPer16B]) {
  if (sizeof(T) == 2) {
    uint2 pk;
    if (quant_vec_fast(q, rinv, &pk, uint16_t{})) { *reinterpret_cast<uint2 *>(o) = pk; return; }
  } else {
    uint32_t pk;
    if (quant_vec_fast(q, rinv, &pk, float{})) { *reinterpret_cast<uint32_t *>(o) = pk; return; }
  }
  const T *e = reinterpret_cast<const T *>(&q);
#pragma unroll
  for (int i = 0; i < VecTraits<T>::kPer16B; ++i) o[i] = quant_sym(elem_to_f32<T>(e[i]), scale);
}


__device__ __forceinline__ float block_max(float v, float *sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = sh[0];
  for (int i = 1; i < (int)(blockDim.x >> 5); ++i) r = fmaxf(r, sh[i]);
  __syncthreads();
  return r;
}

// One CTA per row.  T = uint16_t (bf16 bits) or float; NV = 16-byte vectors of the row that a thread keeps in registers
// between the two passes (2 for rows up to 512 vectors: few registers, six CTAs per SM; 8 for long rows, with the
// register budget of four or five CTAs per SM: left to its own choice the compiler took 32 registers and spilled the cache).
// EP: the expert-parallel forms (row count known only on the device: the CTAs stride over the rows; scatter into other
// GPUs' receive buffers).  They are a separate instantiation so that the plain form keeps its register budget.
template <typename T, int NV, bool EP>
__global__ void __launch_bounds__(kQuantThreads, NV > 2 ? (EP ? 4 : (sizeof(T) == 2 ? 5 : 4)) : 6) quant_per_token_kernel(RowQuantArgs a) {
  __shared__ float sh[kQuantThreads / 32];
  constexpr int E = VecTraits<T>::kPer16B;
  // a GEMM launched as a programmatic dependent may start its set-up while this grid drains (it waits for the whole
  // grid before it reads anything)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int row_limit = (EP && a.n_rows_dev) ? *a.n_rows_dev : (int)gridDim.x;
  for (int r = blockIdx.x; r < row_limit; r += EP ? (int)gridDim.x : row_limit) {
  const T *src; int8_t *dst; void *scale_out; int64_t scale_idx;
  if (a.n_groups > 0) {
    int g = 0;
    while (g + 1 < a.n_groups && r >= a.row_off[g + 1]) ++g;
    const int lr = r - a.row_off[g];
    src = reinterpret_cast<const T *>(a.g_src[g]) + (int64_t)lr * a.g_src_ld[g];
    dst = a.g_dst[g] ? reinterpret_cast<int8_t *>(a.g_dst[g]) + (int64_t)lr * a.g_dst_ld[g] : nullptr;
    scale_out = a.g_scale[g]; scale_idx = lr;
  } else {
    int64_t sr = r;
    if (a.gather) { int32_t s = a.gather[r]; if (s < 0) continue; sr = s / a.gather_div; }
    src = reinterpret_cast<const T *>(a.src) + sr * a.src_ld;
    dst = a.dst ? a.dst + (int64_t)r * a.dst_ld : nullptr;
    scale_out = a.scale; scale_idx = r;
  }
  const int32_t *sc = (a.scatter && a.n_groups == 0) ? a.scatter + (int64_t)r * a.scatter_n : nullptr;
  const int32_t *sp = (EP && sc && a.scatter_peer) ? a.scatter_peer + (int64_t)r * a.scatter_n : nullptr;
  if (sc) dst = sp ? a.peer_dst[0] : a.dst;     // row offsets (and the peer's base) are applied per destination
  const int K = a.K;
  const bool vec = ((reinterpret_cast<uintptr_t>(src) & 15) == 0) && (K % E == 0) &&
                   (!dst || (reinterpret_cast<uintptr_t>(dst) % E) == 0);
  const int nvec = vec ? K / E : 0;
  uint4 cache[NV];
  float amax = 0.f;
  const bool need_amax = a.absmax_bits == nullptr;   // the row maximum may be given
  if (vec) {
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      int v = threadIdx.x + j * kQuantThreads;
      if (v < nvec) {
        cache[j] = reinterpret_cast<const uint4 *>(src)[v];
        if (need_amax) {
          const T *e = reinterpret_cast<const T *>(&cache[j]);
#pragma unroll
          for (int i = 0; i < E; ++i) { float f = elem_to_f32<T>(e[i]); if (finite_f32(f)) amax = fmaxf(amax, fabsf(f)); }
        }
      }
    }
    for (int v = threadIdx.x + NV * kQuantThreads; need_amax && v < nvec; v += kQuantThreads) {
      uint4 q = reinterpret_cast<const uint4 *>(src)[v];
      const T *e = reinterpret_cast<const T *>(&q);
#pragma unroll
      for (int i = 0; i < E; ++i) { float f = elem_to_f32<T>(e[i]); if (finite_f32(f)) amax = fmaxf(amax, fabsf(f)); }
    }
  } else {
    for (int k = threadIdx.x; need_amax && k < K; k += kQuantThreads) {
      float f = elem_to_f32<T>(src[k]); if (finite_f32(f)) amax = fmaxf(amax, fabsf(f));
    }
  }
  float scale;
  if (a.absmax_bits) scale = scale_from_absmax(__uint_as_float(a.absmax_bits[r]));
  else scale = scale_from_absmax(block_max(amax, sh));
  if (threadIdx.x == 0 && (scale_out || sp)) {
    if (sc) {
      for (int j = 0; j < a.scatter_n; ++j) {
        const int d = sc[j];
        if (d < 0) continue;
        if (sp) { if (d < a.scatter_cap) a.peer_scale[sp[j]][d] = scale; else if (a.overflow) *a.overflow = 1; }
        else if (a.scale_dt == DT_BF16) reinterpret_cast<uint16_t *>(scale_out)[d] = f32_to_bf16_bits(scale);
        else reinterpret_cast<float *>(scale_out)[d] = scale;
      }
    } else if (a.scale_dt == DT_BF16) reinterpret_cast<uint16_t *>(scale_out)[scale_idx] = f32_to_bf16_bits(scale);
    else reinterpret_cast<float *>(scale_out)[scale_idx] = scale;
  }
  if (!dst) continue;
  const float rinv = __frcp_rn(scale);
  if (vec) {
    auto put = [&](int8_t *row, const int8_t (&o)[E], int v) {
      if (E == 8) reinterpret_cast<uint2 *>(row)[v] = *reinterpret_cast<const uint2 *>(o);
      else reinterpret_cast<uint32_t *>(row)[v] = *reinterpret_cast<const uint32_t *>(o);
    };
    auto emit = [&](const uint4 &q, int v) {
      __align__(8) int8_t o[E];
      quant_vec<T>(q, scale, rinv, o);
      if (sp) {
        for (int j = 0; j < a.scatter_n; ++j) { const int d = sc[j]; if (d >= 0 && d < a.scatter_cap) put(a.peer_dst[sp[j]] + (int64_t)d * a.dst_ld, o, v); }
      } else if (sc) {
        for (int j = 0; j < a.scatter_n; ++j) { const int d = sc[j]; if (d >= 0) put(dst + (int64_t)d * a.dst_ld, o, v); }
      } else put(dst, o, v);
    };
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      int v = threadIdx.x + j * kQuantThreads;
      if (v < nvec) emit(cache[j], v);
    }
    for (int v = threadIdx.x + NV * kQuantThreads; v < nvec; v += kQuantThreads)
      emit(reinterpret_cast<const uint4 *>(src)[v], v);
  } else {
    for (int k = threadIdx.x; k < K; k += kQuantThreads) {
      const int8_t qv = quant_sym_r(elem_to_f32<T>(src[k]), scale, rinv);
      if (sp) {
        for (int j = 0; j < a.scatter_n; ++j) { const int d = sc[j]; if (d >= 0 && d < a.scatter_cap) a.peer_dst[sp[j]][(int64_t)d * a.dst_ld + k] = qv; }
      } else if (sc) {
        for (int j = 0; j < a.scatter_n; ++j) { const int d = sc[j]; if (d >= 0) dst[(int64_t)d * a.dst_ld + k] = qv; }
      } else dst[k] = qv;
    }
  }
  }   // rows of this CTA
}

// Per-token ASYMMETRIC dynamic quantisation to u8 (one f32 scale and one s32 zero point per row):
// reorder/reorder_data_type/scalar_impl/dynamic_per_token_ref_kernel.cpp:38-56,128-183.  One CTA per row; min and max over
// the finite values, scale = (max - min) / 255, zp = round(-min / scale) in double, q = clamp(rne(v / scale) + zp, 0, 255).
// Not a hot path (the INT8 GEMMs take symmetric per-token rows), so the row is read twice and divided exactly.
template <typename T>
__global__ void __launch_bounds__(kQuantThreads) quant_per_token_asym_kernel(const T *src, int64_t src_ld, int K, uint8_t *dst, int64_t dst_ld,
                                                                            float *scales, int32_t *zps) {
  __shared__ float sh[kQuantThreads / 32];
  const int r = blockIdx.x;
  const T *row = src + (int64_t)r * src_ld;
  float lo = 3.402823466e+38f, hi = -3.402823466e+38f;
  for (int k = threadIdx.x; k < K; k += kQuantThreads) {
    const float v = elem_to_f32<T>(row[k]);
    if (finite_f32(v)) { lo = fminf(lo, v); hi = fmaxf(hi, v); }
  }
  hi = block_max(hi, sh);
  lo = -block_max(-lo, sh);
  if (lo == 3.402823466e+38f && hi == -3.402823466e+38f) { lo = 0.f; hi = 0.f; }
  if (hi <= lo) hi = __fadd_rn(lo, 1.0f);
  float scale = __fdiv_rn(__fsub_rn(hi, lo), 255.0f);
  if (scale < 1e-10f) scale = 1e-10f;
  const double zd = round((double)(-lo) / (double)scale);
  const int32_t zp = zd < -2147483648.0 ? (int32_t)0x80000000 : (zd > 2147483647.0 ? 0x7fffffff : (int32_t)zd);
  if (threadIdx.x == 0) { scales[r] = scale; zps[r] = zp; }
  if (!dst) return;
  uint8_t *out = dst + (int64_t)r * dst_ld;
  for (int k = threadIdx.x; k < K; k += kQuantThreads) {
    const float v = elem_to_f32<T>(row[k]);
    int q = 0;
    if (finite_f32(v)) {
      // nearbyint(v / scale) + zp without leaving the int range: the quotient is clamped first (any value beyond
      // +-2^30 saturates the result anyway)
      const float t = fminf(fmaxf(rintf(__fdiv_rn(v, scale)), -1073741824.f), 1073741824.f);
      const long long qq = (long long)t + (long long)zp;
      q = qq < 0 ? 0 : (qq > 255 ? 255 : (int)qq);
    }
    out[k] = (uint8_t)q;
  }
}

// Rows whose abs-max is already known (the re-quantisation between the two MoE GEMMs: the first GEMM's epilogue left the
// row maxima): a pure stream.  One warp per row at a time, U 16-byte loads in flight per lane, no shared memory and no
// barrier, so the warps of an SM drift apart and loads, arithmetic and stores of different rows overlap (a CTA per row
// that loads, then converts, then stores ran its phases in step with its neighbours: 110 us for 352 MB).
// Requires 16-byte aligned rows, K a multiple of the vector width, plain rows (no gather, scatter or groups).
template <typename T, int U>
__global__ void __launch_bounds__(256) quant_known_absmax_kernel(RowQuantArgs a, int rows, int segs, int seg_len) {
  constexpr int E = VecTraits<T>::kPer16B;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int lane = threadIdx.x & 31;
  const int row_limit = a.n_rows_dev ? min(rows, *a.n_rows_dev) : rows;
  const int nvec = a.K / E;
  // a work item is one segment of one row (seg_len vectors, a multiple of 32); the warps take the items in turn
  const long long items = (long long)row_limit * segs;
  for (long long it = blockIdx.x * 8 + (threadIdx.x >> 5); it < items; it += (long long)gridDim.x * 8) {
    const int r = (int)(it / segs), sg = (int)(it - (long long)r * segs);
    const float scale = scale_from_absmax(__uint_as_float(a.absmax_bits[r]));
    if (lane == 0 && sg == 0 && a.scale) {
      if (a.scale_dt == DT_BF16) reinterpret_cast<uint16_t *>(a.scale)[r] = f32_to_bf16_bits(scale);
      else reinterpret_cast<float *>(a.scale)[r] = scale;
    }
    if (!a.dst) continue;
    const float rinv = __frcp_rn(scale);
    const uint4 *src = reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(a.src) + (int64_t)r * a.src_ld);
    int8_t *dst = a.dst + (int64_t)r * a.dst_ld;
    const int v_end = min(nvec, (sg + 1) * seg_len);
    for (int v0 = sg * seg_len + lane; v0 < v_end; v0 += 32 * U) {
      uint4 q[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int v = v0 + u * 32;
        if (v < v_end) asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(q[u].x), "=r"(q[u].y), "=r"(q[u].z), "=r"(q[u].w) : "l"(src + v));
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int v = v0 + u * 32;
        if (v < v_end) {
          __align__(8) int8_t o[E];
          quant_vec<T>(q[u], scale, rinv, o);
          if (E == 8) reinterpret_cast<uint2 *>(dst)[v] = *reinterpret_cast<uint2 *>(o);
          else reinterpret_cast<uint32_t *>(dst)[v] = *reinterpret_cast<uint32_t *>(o);
        }
      }
    }
  }
}

// One warp per row, for short rows (K <= 32 * NV * elements-per-16-bytes): the row lives in the
// lanes' registers, the abs-max is a shuffle reduction, no shared memory and no CTA barrier.
// Requires 16-byte aligned rows and K a multiple of the vector width (the launcher checks).
template <typename T, int NV, bool EP>
__global__ void __launch_bounds__(256) quant_per_token_warp_kernel(RowQuantArgs a, int rows) {
  constexpr int E = VecTraits<T>::kPer16B;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int lane = threadIdx.x & 31;
  const int row_limit = (EP && a.n_rows_dev) ? min(rows, *a.n_rows_dev) : rows;
  for (int r = blockIdx.x * 8 + (threadIdx.x >> 5); r < row_limit; r += EP ? (int)gridDim.x * 8 : row_limit) {
  int64_t sr = r;
  if (a.gather) { int32_t s = a.gather[r]; if (s < 0) continue; sr = s / a.gather_div; }
  const T *src = reinterpret_cast<const T *>(a.src) + sr * a.src_ld;
  const int32_t *sc = a.scatter ? a.scatter + (int64_t)r * a.scatter_n : nullptr;
  const int32_t *sp = (EP && sc && a.scatter_peer) ? a.scatter_peer + (int64_t)r * a.scatter_n : nullptr;
  int8_t *dst = sp ? a.peer_dst[0] : (a.dst ? (sc ? a.dst : a.dst + (int64_t)r * a.dst_ld) : nullptr);
  const int nvec = a.K / E;
  uint4 cache[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int v = lane + j * 32;
    cache[j] = v < nvec ? reinterpret_cast<const uint4 *>(src)[v] : make_uint4(0, 0, 0, 0);
  }
  float scale;
  if (a.absmax_bits) scale = scale_from_absmax(__uint_as_float(a.absmax_bits[r]));
  else {
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const T *e = reinterpret_cast<const T *>(&cache[j]);
#pragma unroll
      for (int i = 0; i < E; ++i) { float f = elem_to_f32<T>(e[i]); if (finite_f32(f)) amax = fmaxf(amax, fabsf(f)); }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    scale = scale_from_absmax(amax);
  }
  if (a.scale || sp) {
    if (sp) {
      if (lane < a.scatter_n && sc[lane] >= 0) {
        if (sc[lane] < a.scatter_cap) a.peer_scale[sp[lane]][sc[lane]] = scale;
        else if (a.overflow) *a.overflow = 1;
      }
    } else if (sc) {
      if (lane < a.scatter_n && sc[lane] >= 0) {
        if (a.scale_dt == DT_BF16) reinterpret_cast<uint16_t *>(a.scale)[sc[lane]] = f32_to_bf16_bits(scale);
        else reinterpret_cast<float *>(a.scale)[sc[lane]] = scale;
      }
    } else if (lane == 0) {
      if (a.scale_dt == DT_BF16) reinterpret_cast<uint16_t *>(a.scale)[r] = f32_to_bf16_bits(scale);
      else reinterpret_cast<float *>(a.scale)[r] = scale;
    }
  }
  if (!dst) continue;
  const float rinv = __frcp_rn(scale);
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int v = lane + j * 32;
    if (v < nvec) {
      __align__(8) int8_t o[E];
      quant_vec<T>(cache[j], scale, rinv, o);
      if (sc) {
        for (int jj = 0; jj < a.scatter_n; ++jj) {
          const int d = sc[jj];
          if (d < 0 || (sp && d >= a.scatter_cap)) continue;
          int8_t *row = (sp ? a.peer_dst[sp[jj]] : dst) + (int64_t)d * a.dst_ld;
          if (E == 8) reinterpret_cast<uint2 *>(row)[v] = *reinterpret_cast<uint2 *>(o);
          else reinterpret_cast<uint32_t *>(row)[v] = *reinterpret_cast<uint32_t *>(o);
        }
      } else if (E == 8) reinterpret_cast<uint2 *>(dst)[v] = *reinterpret_cast<uint2 *>(o);
      else reinterpret_cast<uint32_t *>(dst)[v] = *reinterpret_cast<uint32_t *>(o);
    }
  }
  }   // rows of this warp
}

// ---- per-channel / per-tensor dynamic scales over a [M,N] matrix -----------------------------
// pass 1: abs-max per column (or one for the tensor) with atomicMax on the float bit pattern
// (non-negative floats order like unsigned integers); out must be zeroed first.
template <typename T>
__global__ void absmax_cols_kernel(const T *src, int64_t M, int64_t N, int64_t ld, int per_channel, uint32_t *out) {
  const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t rows_per = (M + gridDim.y - 1) / gridDim.y;
  const int64_t m0 = (int64_t)blockIdx.y * rows_per, m1 = min(M, m0 + rows_per);
  float amax = 0.f;
  if (n < N)
    for (int64_t m = m0; m < m1; ++m) {
      float f = elem_to_f32<T>(src[m * ld + n]);
      if (finite_f32(f)) amax = fmaxf(amax, fabsf(f));
    }
  if (per_channel) {
    if (n < N) atomicMax(out + n, __float_as_uint(amax));
  } else {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) atomicMax(out, __float_as_uint(amax));
  }
}
__global__ void scales_from_absmax_kernel(const uint32_t *amax, int64_t n, float *scale) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) scale[i] = scale_from_absmax(__uint_as_float(amax[i]));
}

// ---- static quantise / dequantise, element-wise over [M,N] --------------------------------------
template <typename T>
__global__ void quant_static_kernel(const T *src, int64_t M, int64_t N, int64_t ld, const float *scale, int64_t n_scale,
                                    const int32_t *zp, int64_t n_zp, void *dst, int32_t dst_dt, int64_t dst_ld) {
  const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  const float s = scale[n_scale > 1 ? n : 0];
  const int32_t z = zp ? zp[n_zp > 1 ? n : 0] : 0;
  const int lo = dst_dt == DT_U8 ? 0 : -128, hi = dst_dt == DT_U8 ? 255 : 127;
  for (int64_t m = blockIdx.y; m < M; m += gridDim.y) {
    float v = elem_to_f32<T>(src[m * ld + n]);
    int q = __float2int_rn(__fdiv_rn(v, s)) + z;
    q = max(lo, min(hi, q));
    if (dst_dt == DT_U8) reinterpret_cast<uint8_t *>(dst)[m * dst_ld + n] = (uint8_t)q;
    else reinterpret_cast<int8_t *>(dst)[m * dst_ld + n] = (int8_t)q;
  }
}
// Requantised matmul destination: q = rne(clamp(x * dst_scale + dst_zp)) over an f32 [M,N] result
// (operators/matmul/matmul_ref_kernel.cpp:770-797 scale and zero point, :155-192 clamp, then nearbyint).
__global__ void requant_dst_kernel(const float *src, int64_t M, int64_t N, const float *scale, const int32_t *zp, void *dst,
                                   int32_t dst_dt, int64_t ldc) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * N) return;
  const int64_t m = i / N, n = i - m * N;
  float x = src[i];
  if (scale) x = __fmul_rn(x, *scale);
  if (zp) x = __fadd_rn(x, (float)*zp);
  const float lo = dst_dt == DT_U8 ? 0.f : -128.f, hi = dst_dt == DT_U8 ? 255.f : 127.f;
  x = x < lo ? lo : (x > hi ? hi : x);      // (a NaN passes both comparisons and converts to 0)
  const int q = __float2int_rn(x);
  if (dst_dt == DT_U8) reinterpret_cast<uint8_t *>(dst)[m * ldc + n] = (uint8_t)q;
  else reinterpret_cast<int8_t *>(dst)[m * ldc + n] = (int8_t)q;
}

__global__ void dequant_static_kernel(const void *src, int32_t src_dt, int64_t M, int64_t N, int64_t ld,
                                      const float *scale, int64_t n_scale, const int32_t *zp, int64_t n_zp,
                                      void *dst, int32_t dst_dt, int64_t dst_ld) {
  const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  const float s = scale[n_scale > 1 ? n : 0];
  const int32_t z = zp ? zp[n_zp > 1 ? n : 0] : 0;
  for (int64_t m = blockIdx.y; m < M; m += gridDim.y) {
    int q = src_dt == DT_U8 ? (int)reinterpret_cast<const uint8_t *>(src)[m * ld + n]
                            : (int)reinterpret_cast<const int8_t *>(src)[m * ld + n];
    float x = __fmul_rn((float)(q - z), s);
    if (dst_dt == DT_BF16) reinterpret_cast<uint16_t *>(dst)[m * dst_ld + n] = f32_to_bf16_bits(x);
    else reinterpret_cast<float *>(dst)[m * dst_ld + n] = x;
  }
}

}  // namespace b200
