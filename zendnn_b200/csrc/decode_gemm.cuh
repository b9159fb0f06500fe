// Decode-shape W8A8 GEMM (M <= 16): one persistent CTA per SM, work split evenly over every warp
// of the grid ("stream-K").  Stands in for the reference's small-M INT8 paths (AOCL-DLP call sites
// matmul/backends/aocl/aocl_kernel.cpp:1190-1301; native GEMV
// matmul/matmul_native/brgemm/kernel/int8/int8_gemv_bkc.cpp), which split N over CPU threads.
//
// The packed weight is W^T [Np][Kp], K contiguous.  The unit of work is a "chunk item": 8 weight
// rows (output columns) x 64 bytes of K.  All G*C items (G = ceil(N/8) row groups, C = Kp/64) are
// laid out group-major and cut into gridDim.x * warps equal contiguous ranges, so every SM streams
// the same number of bytes whatever N and K are.  A lane loads 16 bytes (row g, segment t of the
// chunk); mma.sync.m16n8k32 multiplies them with the 16 activation rows staged once per CTA in
// shared memory (same K permutation on both operands, see stream_gemm.cuh).
//
// A range may start or end in the middle of a row group.  Partial sums of such groups are added
// into a zero-initialised s32 scratch [G][16][8] with red.global.add (integer: order-free and
// exact); a per-group counter of finished chunks tells the warp that completes a group to run the
// epilogue.  That warp also puts the scratch words and the counter back to zero, so the scratch
// is all-zero again when the kernel ends.  Groups covered by a single warp never touch the scratch.
#pragma once
#include "common.cuh"
#include "stream_gemm.cuh"

namespace b200 {

struct DecodeGemmArgs {
  const uint8_t *A; int64_t lda;   // [M,lda] u8 or s8, M <= 16
  int M, N, K;
  const int8_t *Wt; int Kp;
  int groups;                      // ceil(N / 8)
  int chunks;                      // Kp / 64
  int a_stride;                    // smem row stride of A: Kp + 64
  int rows_staged;                 // 8 or 16
  int32_t *sums;                   // [groups][16][8] zero on entry, zero on exit
  uint32_t *counters;              // [groups]        zero on entry, zero on exit
};

constexpr int kDecodeWarps = 16;
constexpr int kDecodeBatch = 8;    // 16-byte loads in flight per lane

template <bool A_UNSIGNED>
__global__ void __launch_bounds__(kDecodeWarps * 32, 1) decode_gemm_kernel(DecodeGemmArgs g, EpiParams epi) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int lg = lane >> 2, lt = lane & 3;
  const long long total = (long long)g.groups * g.chunks;
  const long long nwarps = (long long)gridDim.x * kDecodeWarps;
  const long long wid = (long long)blockIdx.x * kDecodeWarps + warp;
  long long item = wid * total / nwarps;
  const long long item_end = (wid + 1) * total / nwarps;

  // the first batch of weight loads is issued before the activations are staged
  int grp = (int)(item / g.chunks);
  int c = (int)(item - (long long)grp * g.chunks);
  int run = (int)min((long long)(g.chunks - c), item_end - item);   // chunks of this group in this warp's range
  const int8_t *wbase = g.Wt + lt * 16;
  uint4 w[kDecodeBatch];
  {
    const int8_t *wrow = wbase + (size_t)(grp * 8 + lg) * g.Kp + (size_t)c * 64;
#pragma unroll
    for (int u = 0; u < kDecodeBatch; ++u) w[u] = (item < item_end && u < run) ? ldg_stream(wrow + u * 64) : make_uint4(0, 0, 0, 0);
  }

  // stage A[0..rows_staged) x [0, Kp) (zero beyond M and K)
  {
    const bool vec = ((reinterpret_cast<uintptr_t>(g.A) | (uintptr_t)g.lda) & 15) == 0;
    const int segs = g.Kp >> 4;
    for (int i = tid; i < g.rows_staged * segs; i += kDecodeWarps * 32) {
      const int r = i / segs, s = i - r * segs, k = s * 16;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < g.M && k < g.K) {
        const uint8_t *src = g.A + (size_t)r * g.lda + k;
        if (vec && k + 16 <= g.K) v = *reinterpret_cast<const uint4 *>(src);
        else {
          uint8_t tmp[16];
#pragma unroll
          for (int b = 0; b < 16; ++b) tmp[b] = (k + b < g.K) ? src[b] : (uint8_t)0;
          v = *reinterpret_cast<uint4 *>(tmp);
        }
      }
      *reinterpret_cast<uint4 *>(smem + (size_t)r * g.a_stride + k) = v;
    }
  }
  __syncthreads();

  const bool hi_rows = g.rows_staged > 8;
  const uint8_t *a_lo_base = smem + (size_t)lg * g.a_stride + lt * 16;
  const int32_t zp = load_zp(epi);

  while (item < item_end) {
    int acc[4] = {0, 0, 0, 0};
    const int8_t *wrow = wbase + (size_t)(grp * 8 + lg) * g.Kp;
    int done = 0;
    while (done < run) {
      const int nb = min(kDecodeBatch, run - done);
      if (done > 0) {
        const int8_t *p = wrow + (size_t)(c + done) * 64;
#pragma unroll
        for (int u = 0; u < kDecodeBatch; ++u) w[u] = u < nb ? ldg_stream(p + u * 64) : make_uint4(0, 0, 0, 0);
      }
      const uint8_t *ap = a_lo_base + (size_t)(c + done) * 64;
#pragma unroll
      for (int u = 0; u < kDecodeBatch; ++u) {
        if (u < nb) {
          const uint4 lo = *reinterpret_cast<const uint4 *>(ap + u * 64);
          const uint4 hi = hi_rows ? *reinterpret_cast<const uint4 *>(ap + u * 64 + (size_t)8 * g.a_stride) : make_uint4(0, 0, 0, 0);
          mma_m16n8k32<A_UNSIGNED>(acc, lo.x, hi.x, lo.y, hi.y, w[u].x, w[u].y);
          mma_m16n8k32<A_UNSIGNED>(acc, lo.z, hi.z, lo.w, hi.w, w[u].z, w[u].w);
        }
      }
      done += nb;
    }

    // ---- this warp's share of group `grp` is in acc: combine and, if it completes the group, finish it
    bool finish = true;
    if (run != g.chunks) {
      int32_t *s = g.sums + (size_t)grp * 128;
      const int col = lt * 2;
      atomicAdd(s + lg * 8 + col, acc[0]);
      atomicAdd(s + lg * 8 + col + 1, acc[1]);
      if (hi_rows) {
        atomicAdd(s + (lg + 8) * 8 + col, acc[2]);
        atomicAdd(s + (lg + 8) * 8 + col + 1, acc[3]);
      }
      __threadfence();
      __syncwarp();
      unsigned prev = 0;
      if (lane == 0) prev = atomicAdd(g.counters + grp, (unsigned)run);
      prev = __shfl_sync(0xffffffffu, prev, 0);
      finish = (prev + (unsigned)run == (unsigned)g.chunks);
      if (finish) {
        __threadfence();
        acc[0] = __ldcg(s + lg * 8 + col); acc[1] = __ldcg(s + lg * 8 + col + 1);
        __stcg(s + lg * 8 + col, 0); __stcg(s + lg * 8 + col + 1, 0);
        if (hi_rows) {
          acc[2] = __ldcg(s + (lg + 8) * 8 + col); acc[3] = __ldcg(s + (lg + 8) * 8 + col + 1);
          __stcg(s + (lg + 8) * 8 + col, 0); __stcg(s + (lg + 8) * 8 + col + 1, 0);
        }
        if (lane == 0) g.counters[grp] = 0;
      }
    }
    if (finish) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int m = lg + (j >> 1) * 8, n = grp * 8 + lt * 2 + (j & 1);
        if (m >= g.M || n >= g.N) continue;
        int32_t v = acc[j];
        if (epi.dst_dt == DT_S32) {
          if (zp != 0) v -= zp * epi.colsum[n];
          reinterpret_cast<int32_t *>(epi.dst)[(size_t)m * epi.ldc + n] = v;
          continue;
        }
        const EpiCtx cx = epi_ctx(epi, m);
        const float x = epi_finish(epi, cx, epi_dequant(epi, cx, v, zp, n, n), m, n);
        if (epi.dst_dt == DT_BF16) reinterpret_cast<uint16_t *>(epi.dst)[(size_t)m * epi.ldc + n] = f32_to_bf16_bits(x);
        else reinterpret_cast<float *>(epi.dst)[(size_t)m * epi.ldc + n] = x;
      }
    }

    // ---- next run
    item += run;
    if (item >= item_end) break;
    grp += 1; c = 0;
    run = (int)min((long long)g.chunks, item_end - item);
    {
      const int8_t *p = wbase + (size_t)(grp * 8 + lg) * g.Kp;
#pragma unroll
      for (int u = 0; u < kDecodeBatch; ++u) w[u] = u < run ? ldg_stream(p + u * 64) : make_uint4(0, 0, 0, 0);
    }
  }
}

}  // namespace b200
