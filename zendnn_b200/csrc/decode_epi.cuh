// Epilogue of the decode-shape GEMM kernels: the per-column operands (weight scale, bias, column sum)
// and the per-row source scales of a CTA's outputs are copied into shared memory while the weights
// stream, so that the epilogue itself touches global memory only for its stores.  Arithmetic and
// operation order are those of epi_dequant / epi_finish (common.cuh).
#pragma once
#include "common.cuh"

namespace b200 {

struct DecodeEpiSmem {
  float *ws;        // [cols] weight scale (1 when absent)
  float *bias;      // [cols] bias as f32 (0 when absent)
  int32_t *cs;      // [cols] column sums (0 when no zero point)
  float *ss;        // [16] source scale per row (1 when absent)
};
__host__ __device__ inline size_t decode_epi_bytes(int max_local_groups) { return (size_t)max_local_groups * 8 * 12 + 64; }
__device__ __forceinline__ DecodeEpiSmem decode_epi_carve(uint8_t *base, int max_local_groups) {
  DecodeEpiSmem s;
  const int cols = max_local_groups * 8;
  s.ws = reinterpret_cast<float *>(base);
  s.bias = s.ws + cols;
  s.cs = reinterpret_cast<int32_t *>(s.bias + cols);
  s.ss = reinterpret_cast<float *>(s.cs + cols);
  return s;
}

// Called by `nthreads` threads (tid 0..nthreads-1) after griddepcontrol.wait; a barrier must follow before
// decode_epilogue.  Columns [n0, n0 + cols) of the GEMM, rows [0, M).
__device__ __forceinline__ void decode_epi_stage(const EpiParams &epi, const DecodeEpiSmem &s, int n0, int cols, int N, int M,
                                                 int tid, int nthreads) {
  if (epi.dst_dt == DT_S32) {
    if (epi.has_zp) for (int j = tid; j < cols; j += nthreads) s.cs[j] = (n0 + j < N) ? epi.colsum[n0 + j] : 0;
    return;
  }
  for (int j = tid; j < cols; j += nthreads) {
    const int n = n0 + j;
    const bool in = n < N;
    s.ws[j] = (in && epi.wei_scale_n) ? load_as_f32(epi.wei_scale, epi.wei_scale_dt, epi.wei_scale_n > 1 ? n : 0) : 1.0f;
    s.bias[j] = (in && epi.bias) ? load_as_f32(epi.bias, epi.bias_dt, n) : 0.0f;
    s.cs[j] = (in && epi.has_zp) ? epi.colsum[n] : 0;
  }
  for (int m = tid; m < 16; m += nthreads)
    s.ss[m] = (m < M && epi.src_scale_n) ? load_as_f32(epi.src_scale, epi.src_scale_dt, epi.src_scale_n > 1 ? m : 0) : 1.0f;
}

// red: [local group][16 rows][8 columns] s32 sums of the CTA's outputs; g0: first group of the CTA.
__device__ __forceinline__ void decode_epilogue(const EpiParams &epi, const DecodeEpiSmem &s, const int32_t *red, int g0, int n_local,
                                                int M, int N, int tid, int nthreads) {
  const int32_t zp = load_zp(epi);
  for (int i = tid; i < n_local * 128; i += nthreads) {
    const int gl = i >> 7, m = (i >> 3) & 15, j = gl * 8 + (i & 7), n = g0 * 8 + j;
    if (m >= M || n >= N) continue;
    int32_t v = red[i];
    if (zp != 0) v -= zp * s.cs[j];
    if (epi.dst_dt == DT_S32) { reinterpret_cast<int32_t *>(epi.dst)[(size_t)m * epi.ldc + n] = v; continue; }
    float x = (float)v;
    if (epi.src_scale_n) x = __fmul_rn(x, s.ss[m]);
    if (epi.wei_scale_n) x = __fmul_rn(x, s.ws[j]);
    if (epi.bias) x = __fadd_rn(x, s.bias[j]);
    for (int p = 0; p < epi.n_po; ++p) x = apply_postop(epi.po[p], x, m, n);
    if (epi.dst_dt == DT_BF16) reinterpret_cast<uint16_t *>(epi.dst)[(size_t)m * epi.ldc + n] = f32_to_bf16_bits(x);
    else reinterpret_cast<float *>(epi.dst)[(size_t)m * epi.ldc + n] = x;
  }
}

}  // namespace b200
