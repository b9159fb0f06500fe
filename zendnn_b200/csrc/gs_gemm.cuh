// Group-scaled symmetric INT8 GEMM: per-group source scales {M,G} x per-group weight scales {G,N}, with s8 or packed s4
// weights (W4A8).  Stands in for the reference's sym_quant path (matmul/backends/aocl/aocl_kernel.cpp:704-793,1060-1110:
// s4 weights are widened to s8 once, then aocl_gemm_s8s8s32o*_sym_quant with a group size) and follows the scalar
// definition operators/matmul/matmul_ref_kernel.cpp:961-1003:
//     out[m,n] = postops( sum_g ((float)(sum_{k in g} a[m,k] w[k,n]) * sa[m,g]) * sw[g,n]  + bias[n] )
// Integer sums per group are exact; the f32 sum over the groups runs in group order inside a warp.
//
// Layout: the weight is kept K-contiguous per output column, [N][Kp] s8 or [N][Kp/2] s4 (two codes per byte, even k in
// the low nibble) -- 4-bit weights stay 4-bit in HBM, which halves the bytes a decode-shaped call streams.  A is s8
// [M][Kp] (rows zero-padded to Kp, a multiple of 64).
//
// One CTA = 8 warps = MT row tiles of 16 rows x KS shares of the groups (MT * KS = 8) over NT * 8 output columns.
// mma.sync.m16n8k32 s8: a lane (g = lane / 4, t = lane % 4) reads ONE contiguous piece of a row per chunk -- 16 bytes at
// k0 + 16 t of a 64-byte chunk (8 bytes at k0 + 8 t of a 32-byte chunk when the group size is not a multiple of 64) --
// for the activation rows g and g + 8 and for weight column g of every column tile; both operands use the same
// assignment of k to fragment positions, so each MMA adds products of matching k and a chunk is covered exactly once.
// s4 codes are not sign-extended: the even and odd nibbles of a word are masked into the HIGH nibbles of two registers
// (16 * w, exact), the activation bytes are permuted to the same even / odd order with two byte permutes per row, and
// the group sum is shifted right by four (exact: it is a multiple of 16).
// Group sizes 4, 8 and 16 run the MMA of a 32-byte chunk once per group with the activation registers of the other
// groups zeroed.
// The warps that share a row tile add their f32 partial sums through shared memory in a fixed order.
#pragma once
#include "common.cuh"
#include "stream_gemm.cuh"

namespace b200 {

struct GsGemmArgs {
  const int8_t *A; int64_t lda;     // s8 [M, lda], 16-byte aligned rows, zero-padded to Kp
  const float *sa; int sa_cols;     // f32 [M, sa_cols]; sa_cols = G, or 1 (per-token scale used for every group)
  const uint8_t *W; int64_t w_row;  // bytes per output column: Kp (s8) or Kp / 2 (s4)
  int w4;                           // weights are packed s4
  const void *sw; int sw_dt;        // [G, N] f32 or bf16
  int M, N, K, Kp, gs, G;
  int MT;                           // row tiles of 16 per CTA: 1, 2, 4 or 8
};

constexpr int kGsWarps = 8;

__device__ __forceinline__ uint2 ldg_nc8(const void *p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_nc4(const void *p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

// One column tile's weight piece of a chunk, as MMA B registers {b0, b1} per 32 k: s8 pieces are used as they are,
// an s4 word becomes (even nibbles << 4, odd nibbles in place).
template <int CH, bool W4>
__device__ __forceinline__ void gs_load_b(const uint8_t *wcol, int k_piece, uint32_t (&b)[CH / 16]) {
  if (W4) {
    if (CH == 64) {
      const uint2 v = ldg_nc8(wcol + (k_piece >> 1));
      b[0] = (v.x << 4) & 0xF0F0F0F0u; b[1] = v.x & 0xF0F0F0F0u; b[2] = (v.y << 4) & 0xF0F0F0F0u; b[3] = v.y & 0xF0F0F0F0u;
    } else {
      const uint32_t v = ldg_nc4(wcol + (k_piece >> 1));
      b[0] = (v << 4) & 0xF0F0F0F0u; b[1] = v & 0xF0F0F0F0u;
    }
  } else {
    if (CH == 64) {
      const uint4 v = ldg_stream(wcol + k_piece);
      b[0] = v.x; b[1] = v.y; b[2] = v.z; b[3] = v.w;
    } else {
      const uint2 v = ldg_nc8(wcol + k_piece);
      b[0] = v.x; b[1] = v.y;
    }
  }
}
// The activation piece of one row in the same order: s8 weights take it as it is; for s4 weights the bytes of each
// 8-byte half are split into (even k, odd k).
template <int CH, bool W4>
__device__ __forceinline__ void gs_load_a(const int8_t *arow, int k_piece, uint32_t (&a)[CH / 16]) {
  uint32_t r[CH / 16];
  if (CH == 64) {
    const uint4 v = *reinterpret_cast<const uint4 *>(arow + k_piece);
    r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w;
  } else {
    const uint2 v = *reinterpret_cast<const uint2 *>(arow + k_piece);
    r[0] = v.x; r[1] = v.y;
  }
#pragma unroll
  for (int i = 0; i < CH / 16; i += 2) {
    if (W4) { a[i] = __byte_perm(r[i], r[i + 1], 0x6420); a[i + 1] = __byte_perm(r[i], r[i + 1], 0x7531); }
    else { a[i] = r[i]; a[i + 1] = r[i + 1]; }
  }
}

template <int NT, int CH, bool W4>
__global__ void __launch_bounds__(kGsWarps * 32) gs_gemm_kernel(GsGemmArgs g, EpiParams epi) {
  __shared__ float red[kGsWarps][16][NT * 8 + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, lg = lane >> 2, lt = lane & 3;
  const int MT = g.MT, KS = kGsWarps / MT;
  const int wm = warp % MT, wk = warp / MT;
  const int m0 = (blockIdx.y * MT + wm) * 16, n0 = blockIdx.x * NT * 8;
  const int r_lo = m0 + lg, r_hi = r_lo + 8;
  // rows and columns past the edge read the last real one; their results are not stored
  const int8_t *a_lo = g.A + (int64_t)min(r_lo, g.M - 1) * g.lda;
  const int8_t *a_hi = g.A + (int64_t)min(r_hi, g.M - 1) * g.lda;
  const float *sa_lo = g.sa + (int64_t)min(r_lo, g.M - 1) * g.sa_cols;
  const float *sa_hi = g.sa + (int64_t)min(r_hi, g.M - 1) * g.sa_cols;
  const uint8_t *wcol[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) wcol[j] = g.W + (int64_t)min(n0 + j * 8 + lg, g.N - 1) * g.w_row;
  constexpr int NR = CH / 16;          // registers per piece
  constexpr int PIECE = CH / 4;        // bytes of k per lane and chunk
  const int shift = W4 ? 4 : 0;

  float f[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) f[j][0] = f[j][1] = f[j][2] = f[j][3] = 0.f;
  int acc[NT][4];

  // group sum -> f32 -> x sa[m,g] -> x sw[g,n] -> added to the running sum, one rounding per operation
  auto apply = [&](int grp) {
    const float s_lo = sa_lo[g.sa_cols > 1 ? grp : 0], s_hi = sa_hi[g.sa_cols > 1 ? grp : 0];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const int n = n0 + j * 8 + lt * 2;
      const float w0 = n < g.N ? load_as_f32(g.sw, g.sw_dt, (int64_t)grp * g.N + n) : 0.f;
      const float w1 = n + 1 < g.N ? load_as_f32(g.sw, g.sw_dt, (int64_t)grp * g.N + n + 1) : 0.f;
      f[j][0] = __fadd_rn(f[j][0], __fmul_rn(__fmul_rn((float)(acc[j][0] >> shift), s_lo), w0));
      f[j][1] = __fadd_rn(f[j][1], __fmul_rn(__fmul_rn((float)(acc[j][1] >> shift), s_lo), w1));
      f[j][2] = __fadd_rn(f[j][2], __fmul_rn(__fmul_rn((float)(acc[j][2] >> shift), s_hi), w0));
      f[j][3] = __fadd_rn(f[j][3], __fmul_rn(__fmul_rn((float)(acc[j][3] >> shift), s_hi), w1));
    }
  };
  auto zero_acc = [&]() {
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0;
  };

  if (g.gs >= CH) {
    // whole chunks per group; the warps of a row tile take the groups in turn
    const int chunks = g.gs / CH;
    for (int grp = wk; grp < g.G; grp += KS) {
      zero_acc();
      for (int c = 0; c < chunks; ++c) {
        const int kp = grp * g.gs + c * CH + lt * PIECE;
        uint32_t al[NR], ah[NR];
        gs_load_a<CH, W4>(a_lo, kp, al);
        gs_load_a<CH, W4>(a_hi, kp, ah);
        uint32_t b[NT][NR];
#pragma unroll
        for (int j = 0; j < NT; ++j) gs_load_b<CH, W4>(wcol[j], kp, b[j]);
#pragma unroll
        for (int j = 0; j < NT; ++j) {
#pragma unroll
          for (int i = 0; i < NR; i += 2) mma_m16n8k32<false>(acc[j], al[i], ah[i], al[i + 1], ah[i + 1], b[j][i], b[j][i + 1]);
        }
      }
      apply(grp);
    }
  } else {
    // several groups per 32-byte chunk (CH == 32 here): one masked MMA per group
    const int nsub = CH / g.gs;
    const int n_chunks = (g.K + CH - 1) / CH;
    for (int ch = wk; ch < n_chunks; ch += KS) {
      const int kp = ch * CH + lt * PIECE;
      uint32_t al[NR], ah[NR];
      gs_load_a<CH, W4>(a_lo, kp, al);
      gs_load_a<CH, W4>(a_hi, kp, ah);
      uint32_t b[NT][NR];
#pragma unroll
      for (int j = 0; j < NT; ++j) gs_load_b<CH, W4>(wcol[j], kp, b[j]);
      for (int sub = 0; sub < nsub; ++sub) {
        const int grp = ch * nsub + sub;
        if (grp >= g.G) break;
        // which of this lane's activation bytes belong to the group: s8 registers hold k = 8t + 4i .. + 3; s4 registers hold
        // the even (odd) k of 8t .. 8t + 7, two per 4-element group
        uint32_t m0k, m1k;
        if (W4) {
          if (g.gs == 4) m0k = m1k = (sub == 2 * lt) ? 0x0000FFFFu : (sub == 2 * lt + 1 ? 0xFFFF0000u : 0u);
          else m0k = m1k = ((lt * 8) / g.gs == sub) ? 0xFFFFFFFFu : 0u;
        } else {
          m0k = ((lt * 8) / g.gs == sub) ? 0xFFFFFFFFu : 0u;
          m1k = ((lt * 8 + 4) / g.gs == sub) ? 0xFFFFFFFFu : 0u;
        }
        zero_acc();
#pragma unroll
        for (int j = 0; j < NT; ++j) mma_m16n8k32<false>(acc[j], al[0] & m0k, ah[0] & m0k, al[1] & m1k, ah[1] & m1k, b[j][0], b[j][1]);
        apply(grp);
      }
    }
  }

  // the shares of a row tile are added in the order of the shares
  if (KS > 1) {
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const int c = j * 8 + lt * 2;
      red[warp][lg][c] = f[j][0]; red[warp][lg][c + 1] = f[j][1];
      red[warp][lg + 8][c] = f[j][2]; red[warp][lg + 8][c + 1] = f[j][3];
    }
    __syncthreads();
    if (wk != 0) return;
    for (int s = 1; s < KS; ++s) {
      const int w = s * MT + wm;
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const int c = j * 8 + lt * 2;
        f[j][0] = __fadd_rn(f[j][0], red[w][lg][c]); f[j][1] = __fadd_rn(f[j][1], red[w][lg][c + 1]);
        f[j][2] = __fadd_rn(f[j][2], red[w][lg + 8][c]); f[j][3] = __fadd_rn(f[j][3], red[w][lg + 8][c + 1]);
      }
    }
  }

  // bias, post-ops, store
  const EpiCtx cx = epi_ctx(epi, 0);
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int row = (e < 2) ? r_lo : r_hi, col = n0 + j * 8 + lt * 2 + (e & 1);
      if (row >= g.M || col >= g.N) continue;
      const float x = epi_finish(epi, cx, f[j][e], row, col);
      if (epi.dst_dt == DT_BF16) reinterpret_cast<uint16_t *>(epi.dst)[(int64_t)row * epi.ldc + col] = f32_to_bf16_bits(x);
      else reinterpret_cast<float *>(epi.dst)[(int64_t)row * epi.ldc + col] = x;
    }
  }
}

// Weight preparation: any of the caller's layouts ([K,N] or transB [N,K], s8 or packed s4 at element index r*ldb + c,
// even index in the low nibble: matmul/backends/aocl/aocl_kernel.cpp:145-160) -> [N][Kp] s8 or [N][Kp/2] s4, zero padded.
__global__ void gs_pack_weight_kernel(const uint8_t *src, int64_t ldb, int transB, int src_s4, int K, int N, int Kp, uint8_t *dst) {
  // one thread per (n, pair of k)
  const int64_t pairs = Kp / 2;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= pairs * N) return;
  const int n = (int)(i / pairs), k = (int)(i - (int64_t)n * pairs) * 2;
  auto elem = [&](int kk) -> int {
    if (kk >= K) return 0;
    const int64_t idx = transB ? (int64_t)n * ldb + kk : (int64_t)kk * ldb + n;
    if (src_s4) { const uint8_t b = src[idx >> 1]; return (idx & 1) ? (b >> 4) : (b & 0xF); }   // raw code
    return (int)reinterpret_cast<const int8_t *>(src)[idx];
  };
  if (src_s4) dst[(int64_t)n * (Kp / 2) + (k >> 1)] = (uint8_t)(elem(k) | (elem(k + 1) << 4));
  else { dst[(int64_t)n * Kp + k] = (uint8_t)elem(k); dst[(int64_t)n * Kp + k + 1] = (uint8_t)elem(k + 1); }
}

}  // namespace b200
