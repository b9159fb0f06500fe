// Group-scaled symmetric INT8 GEMM: per-group source scales {M,G} x per-group weight scales {G,N}, with s8 or packed s4
// weights (W4A8).  Stands in for the reference's sym_quant path (matmul/backends/aocl/aocl_kernel.cpp:704-793,1060-1110:
// s4 weights are widened to s8 once, then aocl_gemm_s8s8s32o*_sym_quant with a group size) and follows the scalar
// definition operators/matmul/matmul_ref_kernel.cpp:961-1003:
//     out[m,n] = postops( sum_g ((float)(sum_{k in g} a[m,k] w[k,n]) * sa[m,g]) * sw[g,n]  + bias[n] )
// Integer sums per group are exact; the f32 sum over the groups runs in group order inside a warp.
//
// Layout: the weight is blocked as [N/8][Kp/64][8 columns][64 k], s8 (64 bytes per column and block) or s4 (32 bytes: two
// codes per byte, even k in the low nibble), zero padded -- 4-bit weights stay 4-bit in HBM, which halves the bytes a
// decode-shaped call streams, and the eight columns x 64 k that one warp-level load instruction fetches are one
// contiguous 512-byte (256-byte) block, with the next k block of the same columns right behind it.  A is s8 [M][Kp]
// (rows zero-padded to Kp, a multiple of 64).
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
#include "mbar.cuh"

namespace b200 {

struct GsGemmArgs {
  const int8_t *A; int64_t lda;     // s8 [M, lda], 16-byte aligned rows, zero-padded to Kp
  const float *sa; int sa_cols;     // f32 [M, sa_cols]; sa_cols = G, or 1 (per-token scale used for every group)
  const uint8_t *W;                 // blocked weight: [ceil(N/8)][Kp/64][8][64 B (s8) | 32 B (s4)]
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

// Raw pieces as they come from memory: one lane's share of a chunk for one weight column (RW words) or one activation
// row (CH / 16 words).  `cached`: several warps of the CTA read the same weight bytes (more than one row tile per CTA), so the
// loads may allocate in L1; a CTA with one row tile reads every weight byte once and streams past L1.
template <int CH, bool W4> struct GsRaw { static constexpr int RW = W4 ? CH / 32 : CH / 16; static constexpr int RA = CH / 16; };

template <int CH, bool W4>
__device__ __forceinline__ void gs_ld_b(const uint8_t *wbase, int k_piece, bool cached, uint32_t (&r)[GsRaw<CH, W4>::RW]) {
  // wbase: the lane's column inside its column tile's first k block; a k block of eight columns is 8 * CHB bytes
  constexpr int RW = GsRaw<CH, W4>::RW;
  constexpr int CHB = W4 ? 32 : 64;
  const uint8_t *p = wbase + (size_t)(k_piece >> 6) * (8 * CHB) + ((k_piece & 63) >> (W4 ? 1 : 0));
  if (cached) {
    if (RW == 4) { const uint4 v = __ldg(reinterpret_cast<const uint4 *>(p)); r[0] = v.x; r[1] = v.y; r[RW > 2 ? 2 : 0] = v.z; r[RW > 3 ? 3 : 0] = v.w; }
    else if (RW == 2) { const uint2 v = __ldg(reinterpret_cast<const uint2 *>(p)); r[0] = v.x; r[RW > 1 ? 1 : 0] = v.y; }
    else r[0] = __ldg(reinterpret_cast<const uint32_t *>(p));
  } else {
    if (RW == 4) { const uint4 v = ldg_stream(p); r[0] = v.x; r[1] = v.y; r[RW > 2 ? 2 : 0] = v.z; r[RW > 3 ? 3 : 0] = v.w; }
    else if (RW == 2) { const uint2 v = ldg_nc8(p); r[0] = v.x; r[RW > 1 ? 1 : 0] = v.y; }
    else r[0] = ldg_nc4(p);
  }
}
template <int CH>
__device__ __forceinline__ void gs_ld_a(const int8_t *arow, int k_piece, uint32_t (&r)[CH / 16]) {
  if (CH == 64) { const uint4 v = *reinterpret_cast<const uint4 *>(arow + k_piece); r[0] = v.x; r[1] = v.y; r[CH > 32 ? 2 : 0] = v.z; r[CH > 32 ? 3 : 0] = v.w; }
  else { const uint2 v = *reinterpret_cast<const uint2 *>(arow + k_piece); r[0] = v.x; r[1] = v.y; }
}
// MMA B registers {b0, b1} per 32 k: s8 pieces are used as they are, an s4 word becomes (even nibbles << 4, odd nibbles
// in place)
template <int CH, bool W4>
__device__ __forceinline__ void gs_expand_b(const uint32_t (&r)[GsRaw<CH, W4>::RW], uint32_t (&b)[CH / 16]) {
#pragma unroll
  for (int i = 0; i < CH / 32; ++i) {
    if (W4) { b[2 * i] = (r[i] << 4) & 0xF0F0F0F0u; b[2 * i + 1] = r[i] & 0xF0F0F0F0u; }
    else { b[2 * i] = r[(2 * i) % GsRaw<CH, W4>::RW]; b[2 * i + 1] = r[(2 * i + 1) % GsRaw<CH, W4>::RW]; }
  }
}
// The activation piece in the same order: unchanged for s8 weights; for s4 weights the bytes of each 8-byte half are split
// into (even k, odd k)
template <int CH, bool W4>
__device__ __forceinline__ void gs_expand_a(const uint32_t (&r)[CH / 16], uint32_t (&a)[CH / 16]) {
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
  {
    const int chb = W4 ? 32 : 64, nblk = g.Kp >> 6, last_ct = (g.N + 7) / 8 - 1;
#pragma unroll
    for (int j = 0; j < NT; ++j) wcol[j] = g.W + ((int64_t)min(n0 / 8 + j, last_ct) * nblk * 8 + lg) * chb;
  }
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

  const bool cached = MT > 1;
  if (g.gs >= CH) {
    // whole chunks per group; the warps of a row tile take the groups in turn.  The (group, chunk) items of a warp are
    // taken D at a time: all their loads are issued before the first MMA, so D chunks of every column tile are in flight
    constexpr int D = GsRaw<CH, W4>::RW >= 4 ? 2 : 4;
    const int chunks = g.gs / CH;
    const int my_groups = g.G > wk ? (g.G - wk + KS - 1) / KS : 0;
    const int n_items = my_groups * chunks;
    int lgrp = wk, lc = 0;      // load cursor
    int cgrp = wk, cc = 0;      // compute cursor
    for (int i0 = 0; i0 < n_items; i0 += D) {
      uint32_t rb[D][NT][GsRaw<CH, W4>::RW], ral[D][NR], rah[D][NR];
#pragma unroll
      for (int d = 0; d < D; ++d) {
        if (i0 + d < n_items) {
          const int kp = lgrp * g.gs + lc * CH + lt * PIECE;
          gs_ld_a<CH>(a_lo, kp, ral[d]);
          gs_ld_a<CH>(a_hi, kp, rah[d]);
#pragma unroll
          for (int j = 0; j < NT; ++j) gs_ld_b<CH, W4>(wcol[j], kp, cached, rb[d][j]);
          if (++lc == chunks) { lc = 0; lgrp += KS; }
        }
      }
#pragma unroll
      for (int d = 0; d < D; ++d) {
        if (i0 + d < n_items) {
          if (cc == 0) zero_acc();
          uint32_t al[NR], ah[NR];
          gs_expand_a<CH, W4>(ral[d], al);
          gs_expand_a<CH, W4>(rah[d], ah);
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            uint32_t b[NR];
            gs_expand_b<CH, W4>(rb[d][j], b);
#pragma unroll
            for (int i = 0; i < NR; i += 2) mma_m16n8k32<false>(acc[j], al[i], ah[i], al[i + 1], ah[i + 1], b[i], b[i + 1]);
          }
          if (++cc == chunks) { apply(cgrp); cc = 0; cgrp += KS; }
        }
      }
    }
  } else {
    // several groups per 32-byte chunk (CH == 32 here): one masked MMA per group
    const int nsub = CH / g.gs;
    const int n_chunks = (g.K + CH - 1) / CH;
    for (int ch = wk; ch < n_chunks; ch += KS) {
      const int kp = ch * CH + lt * PIECE;
      uint32_t ral[NR], rah[NR], al[NR], ah[NR];
      gs_ld_a<CH>(a_lo, kp, ral);
      gs_ld_a<CH>(a_hi, kp, rah);
      gs_expand_a<CH, W4>(ral, al);
      gs_expand_a<CH, W4>(rah, ah);
      uint32_t b[NT][NR];
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        uint32_t rb[GsRaw<CH, W4>::RW];
        gs_ld_b<CH, W4>(wcol[j], kp, cached, rb);
        gs_expand_b<CH, W4>(rb, b[j]);
      }
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

// Decode form (M <= 16, at least eight groups of a multiple of 32 elements, f32 weight scales, even N): persistent CTAs over
// tiles of 16 output columns.
//   - The activations (s8 [M][Kp]) and their scales are staged once per CTA in shared memory; the eight warps split the
//     groups (warp w: groups w, w + 8, ...), so a warp reads only its own k ranges, for every tile.  (Quantising a bf16
//     source inside this staging phase, to save the separate quantisation launch, measured slower: every CTA then walks
//     the source twice before its first MMA -- 12.3 against 9.0 us at M = 1 and 27.7 against 15.5 us at M = 16, K = N = 4096.)
//   - The weight stream never waits on registers: every lane owns a private ring of R slots in shared memory and fills it
//     with asynchronous copies (cp.async: its piece of a chunk for the two column tiles, plus the two weight scales of a
//     group's last chunk), R - 1 items ahead of the MMAs.  A lane reads back only what it copied itself, so the ring needs
//     no barrier, and a warp's (tile, group, chunk) items form one sequence that does not stop at a tile boundary.
//   - At the end of a tile the warps leave their f32 partial sums in shared memory (two buffers, one barrier per tile) and
//     all 256 threads finish one output each: sum over the warps in warp order, bias, post-ops, store.
struct GsDecodeArgs {
  GsGemmArgs g;
  int rows_staged;   // = M
  int a_stride;      // bytes per staged activation row
  int scale_slots;   // depth of the ring of weight-scale pairs: one slot per group that can be in flight, plus one
};

template <int BYTES>
__device__ __forceinline__ void gs_cp_async(uint32_t dst, const void *src, uint32_t plane = 0) {
  if (BYTES == 32) {      // two 16-byte halves, `plane` bytes apart in shared memory (each half next to the other lanes' halves)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + plane), "l"(reinterpret_cast<const uint8_t *>(src) + 16) : "memory");
  } else if (BYTES == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
  else if (BYTES == 8) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
  else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}

__device__ __forceinline__ uint4 lds16(uint32_t a) { uint4 v; asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a)); return v; }
__device__ __forceinline__ uint2 lds8(uint32_t a) { uint2 v; asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a)); return v; }
__device__ __forceinline__ uint32_t lds4(uint32_t a) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
// NW consecutive words from shared memory; the second 16 bytes of an eight-word piece sit `plane` bytes further on
template <int NW>
__device__ __forceinline__ void lds_words(uint32_t a, uint32_t plane, uint32_t (&r)[NW]) {
  if (NW == 1) r[0] = lds4(a);
  else if (NW == 2) { const uint2 v = lds8(a); r[0] = v.x; r[NW > 1 ? 1 : 0] = v.y; }
  else {
    const uint4 v = lds16(a); r[0] = v.x; r[NW > 1 ? 1 : 0] = v.y; r[NW > 2 ? 2 : 0] = v.z; r[NW > 3 ? 3 : 0] = v.w;
    if (NW == 8) { const uint4 w = lds16(a + plane); r[NW > 4 ? 4 : 0] = w.x; r[NW > 5 ? 5 : 0] = w.y; r[NW > 6 ? 6 : 0] = w.z; r[NW > 7 ? 7 : 0] = w.w; }
  }
}

template <int CH, bool W4, int R>
__global__ void __launch_bounds__(kGsWarps * 32, 2) gs_decode_kernel(GsDecodeArgs da, EpiParams epi) {
  extern __shared__ __align__(16) uint8_t gs_smem[];
  const GsGemmArgs &g = da.g;
  constexpr int NT = 2, NR = CH / 16, PIECE = CH / 4, RW = GsRaw<CH, W4>::RW;
  constexpr int PB = RW * 4;                       // bytes of one lane's weight piece
  // two rings per warp: R slots of [column tile j][lane] weight pieces, and scale_slots slots of [j][lane] (n, n+1) scale
  // pairs (filled only by the chunk that ends a group); a lane's piece sits next to its neighbours', so copies and reads
  // are conflict-free
  constexpr int SLOTW = 32 * NT * PB, SLOTS = 32 * NT * 8;
  constexpr int CHB = W4 ? 32 : 64, SH = W4 ? 1 : 0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, lg = lane >> 2, lt = lane & 3;
  const int RS = da.scale_slots;
  uint8_t *sA = gs_smem;
  float *s_sa = reinterpret_cast<float *>(gs_smem + (size_t)da.rows_staged * da.a_stride);
  float *red = s_sa + ((da.rows_staged * g.sa_cols + 3) & ~3);   // [2][8 warps][16][17]
  uint8_t *ring = reinterpret_cast<uint8_t *>(red + 2 * kGsWarps * 16 * 17);
  constexpr int PU = PB > 16 ? 16 : PB;            // a lane's piece is stored as PB / PU planes of PU bytes, lanes side by side
  const uint32_t ring_w = smem_u32(ring) + (uint32_t)(warp * R * SLOTW) + (uint32_t)lane * PU;      // this lane's first weight piece
  const uint32_t ring_s = smem_u32(ring) + (uint32_t)(kGsWarps * R * SLOTW) + (uint32_t)(warp * RS * SLOTS) + (uint32_t)lane * 8;
  const bool hi_rows = da.rows_staged > 8;
  const int shift = W4 ? 4 : 0;

  const int tiles = (g.N + 15) / 16;
  const int chunks = g.gs / CH;
  const uint32_t nblk = (uint32_t)(g.Kp >> 6);
  const int last_ct = (g.N + 7) / 8 - 1;
  // this lane's piece of a chunk: k = lt * PIECE onwards, which may lie in the chunk's second 64-k block
  const uint32_t lane_w = (uint32_t)((lt * PIECE) >> 6) * (8u * CHB) + (uint32_t)lg * CHB + (uint32_t)(((lt * PIECE) & 63) >> SH);
  const float *swp = reinterpret_cast<const float *>(g.sw);

  // ---- load side: cursor, and the parts of the addresses that change only with the tile
  int l_tile = blockIdx.x, l_grp = warp, l_c = 0, l_slot = 0, l_sslot = 0;
  uint32_t l_wbase[NT], l_n0[NT];
  auto l_set_tile = [&]() {
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      l_wbase[j] = (uint32_t)min(l_tile * 2 + j, last_ct) * nblk * (8u * CHB) + lane_w;
      l_n0[j] = (uint32_t)min(l_tile * 16 + j * 8 + lt * 2, g.N - 2);        // N is even: the pair stays inside the row
    }
  };
  l_set_tile();
  auto issue = [&]() {
    if (l_tile < tiles) {
      const uint32_t kbase = (uint32_t)(l_grp * g.gs + l_c * CH);
      const uint32_t koff = (kbase >> 6) * (8u * CHB) + ((kbase & 63u) >> SH);
      const uint32_t dw = ring_w + (uint32_t)l_slot * SLOTW, ds = ring_s + (uint32_t)l_sslot * SLOTS;
      const bool last = l_c == chunks - 1;
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        gs_cp_async<PB>(dw + j * 32 * PB, g.W + l_wbase[j] + koff, 32u * PU);
        if (last) gs_cp_async<8>(ds + j * 32 * 8, swp + (uint32_t)l_grp * (uint32_t)g.N + l_n0[j]);
      }
      if (last) {
        l_sslot = l_sslot + 1 == RS ? 0 : l_sslot + 1;
        l_c = 0; l_grp += kGsWarps;
        if (l_grp >= g.G) { l_grp = warp; l_tile += (int)gridDim.x; l_set_tile(); }
      }
      else ++l_c;
      l_slot = l_slot + 1 == R ? 0 : l_slot + 1;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  // ---- the ring first (weights do not depend on the activations), then the activations and their scales
#pragma unroll
  for (int i = 0; i < R - 1; ++i) issue();
  {
    const int segs = g.Kp >> 4;
    for (int i = threadIdx.x; i < da.rows_staged * segs; i += kGsWarps * 32) {
      const int r = i / segs, sg = i - r * segs;
      uint8_t *d = sA + (size_t)r * da.a_stride + sg * 16;
      if (r < g.M) *reinterpret_cast<uint4 *>(d) = *reinterpret_cast<const uint4 *>(g.A + (int64_t)r * g.lda + sg * 16);
      else *reinterpret_cast<uint4 *>(d) = make_uint4(0, 0, 0, 0);
    }
    for (int i = threadIdx.x; i < da.rows_staged * g.sa_cols; i += kGsWarps * 32) s_sa[i] = (i / g.sa_cols) < g.M ? g.sa[i] : 0.f;
  }
  __syncthreads();

  float f[NT][4];
  int acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) { f[j][0] = f[j][1] = f[j][2] = f[j][3] = 0.f; acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0; }
  int parity = 0, c_slot = 0, c_sslot = 0;
  // only the M real rows are staged: lanes of rows that do not exist read the last real row (their outputs are not stored)
  const int row_lo = min(lg, da.rows_staged - 1), row_hi = min(lg + 8, da.rows_staged - 1);
  const uint32_t a_lo = smem_u32(sA) + (uint32_t)row_lo * da.a_stride + (uint32_t)lt * PIECE;
  const uint32_t a_hi = smem_u32(sA) + (uint32_t)row_hi * da.a_stride + (uint32_t)lt * PIECE;
  const EpiCtx cx = epi_ctx(epi, 0);

  for (int tile = blockIdx.x; tile < tiles; tile += (int)gridDim.x) {
    for (int grp = warp; grp < g.G; grp += kGsWarps) {
      for (int c = 0; c < chunks; ++c) {
        issue();                                                   // the item R - 1 ahead (or an empty group past the end)
        asm volatile("cp.async.wait_group %0;" ::"n"(R - 1) : "memory");
        const uint32_t sw_ = ring_w + (uint32_t)c_slot * SLOTW;
        c_slot = c_slot + 1 == R ? 0 : c_slot + 1;
        const uint32_t kb = (uint32_t)(grp * g.gs + c * CH);
        uint32_t ral[NR], rah[NR], al[NR], ah[NR];
        lds_words<NR>(a_lo + kb, 16u, ral);
        if (hi_rows) lds_words<NR>(a_hi + kb, 16u, rah);
        else {
#pragma unroll
          for (int i = 0; i < NR; ++i) rah[i] = 0;
        }
        gs_expand_a<CH, W4>(ral, al);
        gs_expand_a<CH, W4>(rah, ah);
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          uint32_t rb[RW], b[NR];
          lds_words<RW>(sw_ + j * 32 * PB, 32u * PU, rb);
          gs_expand_b<CH, W4>(rb, b);
#pragma unroll
          for (int i = 0; i < NR; i += 2) mma_m16n8k32<false>(acc[j], al[i], ah[i], al[i + 1], ah[i + 1], b[i], b[i + 1]);
        }
      }
      // ---- the group is complete: scale and add, one rounding per operation
      const uint32_t slot_s = ring_s + (uint32_t)c_sslot * SLOTS;
      c_sslot = c_sslot + 1 == RS ? 0 : c_sslot + 1;
      const float s_lo = s_sa[row_lo * g.sa_cols + (g.sa_cols > 1 ? grp : 0)];
      const float s_hi = hi_rows ? s_sa[row_hi * g.sa_cols + (g.sa_cols > 1 ? grp : 0)] : 0.f;
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const uint2 wv = lds8(slot_s + j * 32 * 8);
        const float w0 = __uint_as_float(wv.x), w1 = __uint_as_float(wv.y);
        f[j][0] = __fadd_rn(f[j][0], __fmul_rn(__fmul_rn((float)(acc[j][0] >> shift), s_lo), w0));
        f[j][1] = __fadd_rn(f[j][1], __fmul_rn(__fmul_rn((float)(acc[j][1] >> shift), s_lo), w1));
        if (hi_rows) {
          f[j][2] = __fadd_rn(f[j][2], __fmul_rn(__fmul_rn((float)(acc[j][2] >> shift), s_hi), w0));
          f[j][3] = __fadd_rn(f[j][3], __fmul_rn(__fmul_rn((float)(acc[j][3] >> shift), s_hi), w1));
        }
        acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0;
      }
    }
    // ---- the tile is complete for this warp: partial sums to shared memory, one barrier, one output per thread
    float *r = red + ((size_t)parity * kGsWarps + warp) * 16 * 17;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const int c = j * 8 + lt * 2;
      r[lg * 17 + c] = f[j][0]; r[lg * 17 + c + 1] = f[j][1];
      r[(lg + 8) * 17 + c] = f[j][2]; r[(lg + 8) * 17 + c + 1] = f[j][3];
      f[j][0] = f[j][1] = f[j][2] = f[j][3] = 0.f;
    }
    __syncthreads();
    const int row = threadIdx.x >> 4, cl = threadIdx.x & 15, col = tile * 16 + cl;
    if (row < g.M && col < g.N) {
      const float *p = red + (size_t)parity * kGsWarps * 16 * 17 + row * 17 + cl;
      float x = p[0];
#pragma unroll
      for (int w = 1; w < kGsWarps; ++w) x = __fadd_rn(x, p[w * 16 * 17]);
      x = epi_finish(epi, cx, x, row, col);
      if (epi.dst_dt == DT_BF16) reinterpret_cast<uint16_t *>(epi.dst)[(int64_t)row * epi.ldc + col] = f32_to_bf16_bits(x);
      else reinterpret_cast<float *>(epi.dst)[(int64_t)row * epi.ldc + col] = x;
    }
    parity ^= 1;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// Weight preparation: any of the caller's layouts ([K,N] or transB [N,K], s8 or packed s4 at element index r*ldb + c,
// even index in the low nibble: matmul/backends/aocl/aocl_kernel.cpp:145-160) -> the blocked layout above, zero padded.
__global__ void gs_pack_weight_kernel(const uint8_t *src, int64_t ldb, int transB, int src_s4, int K, int N, int Kp, uint8_t *dst) {
  // one thread per (n, pair of k), n up to the next multiple of 8
  const int64_t pairs = Kp / 2, np8 = (N + 7) / 8 * 8;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= pairs * np8) return;
  const int n = (int)(i / pairs), k = (int)(i - (int64_t)n * pairs) * 2;
  auto elem = [&](int kk) -> int {
    if (kk >= K || n >= N) return 0;
    const int64_t idx = transB ? (int64_t)n * ldb + kk : (int64_t)kk * ldb + n;
    if (src_s4) { const uint8_t b = src[idx >> 1]; return (idx & 1) ? (b >> 4) : (b & 0xF); }   // raw code
    return (int)reinterpret_cast<const int8_t *>(src)[idx];
  };
  const int64_t nblk = Kp >> 6;
  const int64_t blk = ((int64_t)(n >> 3) * nblk + (k >> 6)) * 8 + (n & 7);     // (column tile, k block, column)
  if (src_s4) dst[blk * 32 + ((k & 63) >> 1)] = (uint8_t)(elem(k) | (elem(k + 1) << 4));
  else { dst[blk * 64 + (k & 63)] = (uint8_t)elem(k); dst[blk * 64 + (k & 63) + 1] = (uint8_t)elem(k + 1); }
}

}  // namespace b200
