// HBM-streaming W8A8 GEMM for decode-sized M (and the catch-all for shapes the tcgen05 kernel
// does not take).  Stands in for the reference's small-M INT8 paths: the AOCL-DLP GEMM call
// sites (matmul/backends/aocl/aocl_kernel.cpp:1190-1301) and the native GEMV
// (matmul/matmul_native/brgemm/kernel/int8/int8_gemv_bkc.cpp).
//
// Work decomposition.  The packed weight is W^T in 1 KiB blocks [Np/8][Kp/128][8 rows][128 B of K] (pack_kernels.cuh).  A warp owns 8
// weight rows (output columns) and a strided set of 64-byte K chunks; every lane issues 16-byte
// loads (lane = (g,t): row g, bytes t*16.. of the chunk), so the warp reads 8 rows x 64 B per
// load instruction and `kw` warps side by side cover 8 rows x 64*kw B.  The 16 x K activation
// block is staged once per CTA in shared memory.  mma.sync.m16n8k32 (s32 accumulate) does the
// arithmetic: with 16 activation rows per pass it is far below the tensor-pipe limit and the
// kernel is bound by the weight stream.  K is permuted consistently between the two operands
// (both take the same 8 bytes of a lane's 16-byte segment per MMA), which leaves the sums unchanged.
//
// Split-K.  K chunks are split across `kw` warps of a CTA (reduced through shared memory) and
// across gridDim.y CTAs (partials to global scratch; the last CTA to arrive, found with one
// atomic counter per tile, adds them in a fixed order and runs the epilogue, then resets the
// counter).  Integer addition makes the result independent of the split.
#pragma once
#include "common.cuh"

namespace b200 {

struct StreamGemmArgs {
  const uint8_t *A; int64_t lda;   // [M,lda] u8 or s8
  int M, N, K;
  const int8_t *Wt; int Kp;        // packed, block-interleaved (pack_kernels.cuh)
  int nb, kw;                      // n-groups (of 8 columns) and K-split warps per CTA; nb*kw == 8
  int chunks_total;                // Kp / 64
  int chunks_per_cta;              // ceil(chunks_total / gridDim.y)
  int a_stride;                    // shared-memory row stride of the staged activations (bytes)
  int32_t *partial;                // [tiles][gridDim.y][16 * nb*8] s32, only when gridDim.y > 1
  uint32_t *counters;              // [tiles], zero on entry, zero on exit
};

template <bool A_UNSIGNED>
__device__ __forceinline__ void mma_m16n8k32(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
  if (A_UNSIGNED)
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

constexpr int kStreamUnroll = 4;

template <bool A_UNSIGNED>
__global__ void __launch_bounds__(256) stream_gemm_kernel(StreamGemmArgs g, EpiParams epi) {
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ int s_last;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int lg = lane >> 2, lt = lane & 3;
  const int nbw = warp / g.kw, ks = warp % g.kw;   // which n-group / which K-split this warp is
  const int tile_cols = g.nb * 8;
  const int n_base = blockIdx.x * tile_cols;
  const int m0 = blockIdx.z * 16;
  const int cbeg = blockIdx.y * g.chunks_per_cta;
  const int cend = min(cbeg + g.chunks_per_cta, g.chunks_total);
  const int rows = min(16, g.M - m0);

  // first batch of weight loads goes out before the activation block is staged
  // block-interleaved weight (pack_kernels.cuh: wt_offset): 64-byte chunk cc of the eight rows of a group
  // sits at (cc/2)*1024 + row*128 + (cc%2)*64 inside the group's contiguous 8*Kp bytes
  const int8_t *wrow = g.Wt + (size_t)(n_base / 8 + nbw) * g.Kp * 8 + lg * 128 + lt * 16;
  uint4 w[kStreamUnroll];
  int c = cbeg + ks;
#pragma unroll
  for (int u = 0; u < kStreamUnroll; ++u) {
    int cc = c + u * g.kw;
    w[u] = cc < cend ? ldg_stream(wrow + (size_t)(cc >> 1) * 1024 + (cc & 1) * 64) : make_uint4(0, 0, 0, 0);
  }

  // stage A[m0 .. m0+rows) x [cbeg*64, cend*64) into shared memory, zero beyond M and K
  {
    const int kbytes = (cend - cbeg) * 64;
    const int kofs = cbeg * 64;
    const bool vec = ((reinterpret_cast<uintptr_t>(g.A) | (uintptr_t)g.lda) & 15) == 0;
    const int segs = kbytes >> 4;
    for (int i = tid; i < 16 * segs; i += 256) {
      int r = i / segs, s = i - r * segs;
      int k = kofs + s * 16;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < rows && k < g.K) {
        const uint8_t *src = g.A + (size_t)(m0 + r) * g.lda + k;
        if (vec && k + 16 <= g.K) {
          v = *reinterpret_cast<const uint4 *>(src);
        } else {
          uint8_t tmp[16];
#pragma unroll
          for (int b = 0; b < 16; ++b) tmp[b] = (k + b < g.K) ? src[b] : (uint8_t)0;
          v = *reinterpret_cast<uint4 *>(tmp);
        }
      }
      *reinterpret_cast<uint4 *>(smem + (size_t)r * g.a_stride + s * 16) = v;
    }
  }
  __syncthreads();

  int acc[4] = {0, 0, 0, 0};
  const uint8_t *a_lo_p = smem + (size_t)lg * g.a_stride + lt * 16;
  const uint8_t *a_hi_p = a_lo_p + (size_t)8 * g.a_stride;
  const bool hi_rows = rows > 8;
  while (c < cend) {
    uint4 wn[kStreamUnroll];
    const int cnext = c + kStreamUnroll * g.kw;
#pragma unroll
    for (int u = 0; u < kStreamUnroll; ++u) {   // prefetch the next batch
      int cc = cnext + u * g.kw;
      wn[u] = cc < cend ? ldg_stream(wrow + (size_t)(cc >> 1) * 1024 + (cc & 1) * 64) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kStreamUnroll; ++u) {
      int cc = c + u * g.kw;
      if (cc < cend) {
        const int off = (cc - cbeg) * 64;
        uint4 lo = *reinterpret_cast<const uint4 *>(a_lo_p + off);
        uint4 hi = hi_rows ? *reinterpret_cast<const uint4 *>(a_hi_p + off) : make_uint4(0, 0, 0, 0);
        mma_m16n8k32<A_UNSIGNED>(acc, lo.x, hi.x, lo.y, hi.y, w[u].x, w[u].y);
        mma_m16n8k32<A_UNSIGNED>(acc, lo.z, hi.z, lo.w, hi.w, w[u].z, w[u].w);
      }
    }
#pragma unroll
    for (int u = 0; u < kStreamUnroll; ++u) w[u] = wn[u];
    c = cnext;
  }
  __syncthreads();   // activations no longer needed: shared memory becomes the reduction buffer

  // red[ks][16][tile_cols]
  int32_t *red = reinterpret_cast<int32_t *>(smem);
  {
    int32_t *r = red + (size_t)ks * 16 * tile_cols;
    const int col = nbw * 8 + lt * 2;
    r[lg * tile_cols + col] = acc[0];
    r[lg * tile_cols + col + 1] = acc[1];
    r[(lg + 8) * tile_cols + col] = acc[2];
    r[(lg + 8) * tile_cols + col + 1] = acc[3];
  }
  __syncthreads();

  const int tile_elems = 16 * tile_cols;
  const int tile_id = blockIdx.z * gridDim.x + blockIdx.x;
  const int zp = load_zp(epi);
  const bool split = gridDim.y > 1;
  if (split) {
    int32_t *mine = g.partial + ((size_t)tile_id * gridDim.y + blockIdx.y) * tile_elems;
    for (int i = tid; i < rows * tile_cols; i += 256) {
      int32_t v = 0;
      for (int s = 0; s < g.kw; ++s) v += red[(size_t)s * tile_elems + i];
      __stcg(mine + i, v);
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(&g.counters[tile_id], 1u) == gridDim.y - 1) ? 1 : 0;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
  }
  for (int i = tid; i < rows * tile_cols; i += 256) {
    int32_t v = 0;
    if (split) {
      const int32_t *p = g.partial + (size_t)tile_id * gridDim.y * tile_elems + i;
      for (int y = 0; y < (int)gridDim.y; ++y) v += __ldcg(p + (size_t)y * tile_elems);
    } else {
      for (int s = 0; s < g.kw; ++s) v += red[(size_t)s * tile_elems + i];
    }
    const int r = i / tile_cols, cidx = i - r * tile_cols;
    const int m = m0 + r, n = n_base + cidx;
    if (n >= g.N) continue;
    if (epi.dst_dt == DT_S32) {
      if (zp != 0) v -= zp * epi.colsum[n];
      reinterpret_cast<int32_t *>(epi.dst)[(size_t)m * epi.ldc + n] = v;
      continue;
    }
    const EpiCtx cx = epi_ctx(epi, m);
    float x = epi_finish(epi, cx, epi_dequant(epi, cx, v, zp, n, n), m, n);
    if (epi.dst_dt == DT_BF16) reinterpret_cast<uint16_t *>(epi.dst)[(size_t)m * epi.ldc + n] = f32_to_bf16_bits(x);
    else reinterpret_cast<float *>(epi.dst)[(size_t)m * epi.ldc + n] = x;
  }
  if (split && tid == 0) g.counters[tile_id] = 0;
}

}  // namespace b200
