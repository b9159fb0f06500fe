// Decode-shape W8A8 GEMM (M <= 16): one persistent CTA of 32 warps per SM, HBM-bound weight stream.
// Stands in for the reference's small-M INT8 paths (AOCL-DLP call sites
// matmul/backends/aocl/aocl_kernel.cpp:1190-1301; native GEMV
// matmul/matmul_native/brgemm/kernel/int8/int8_gemv_bkc.cpp), which split N over CPU threads.
//
// The packed weight is block-interleaved (pack_kernels.cuh): a group of eight weight rows (output
// columns) is one contiguous span of 8*Kp bytes made of 1 KiB blocks [8 rows][128 B of K].
//   - CTA b owns the contiguous groups [b*G/grid, (b+1)*G/grid): its share of the weight is one
//     contiguous range of memory and no other CTA contributes to its outputs, so there is no
//     cross-CTA reduction and no global scratch.
//   - Inside the CTA the blocks of those groups are cut into 32 equal contiguous ranges, one per
//     warp.  Per block a lane issues one 32-byte load (row g, bytes t*32..), so one warp instruction
//     reads the whole block as eight full 128-byte lines; four blocks are loaded back to back and
//     then consumed.  mma.sync.m16n8k32 multiplies the fragments with the 16 activation rows
//     staged once per CTA in shared memory (same K permutation on both operands, see
//     stream_gemm.cuh).
//   - A warp's range may cover parts of several groups; partial sums go to a shared-memory s32
//     accumulator [groups of this CTA][16][8] with red.shared.add (integer: exact, order-free).
//     After one barrier all threads run the epilogue for the CTA's outputs.
// Programmatic dependent launch: the weight loads are issued before griddepcontrol.wait, so when
// the launch carries the programmatic-serialisation attribute they overlap the tail of the
// previous kernel on the stream; activations are read and outputs written only after the wait.
#pragma once
#include "common.cuh"
#include "decode_epi.cuh"
#include "mbar.cuh"
#include "stream_gemm.cuh"

namespace b200 {

struct DecodeGemmArgs {
  const uint8_t *A; int64_t lda;   // [M,lda] u8 or s8, M <= 16
  int M, N, K;
  const int8_t *Wt; int Kp;
  int groups;                      // ceil(N / 8)
  int blocks;                      // Kp / 128: 1 KiB blocks per group
  int a_stride;                    // smem row stride of A: Kp + 16 (conflict-free 16-byte reads at row*stride + t*32)
  int rows_staged;                 // 8 or 16
  int max_local_groups;            // ceil(groups / gridDim.x)
  int tune;                        // 1 = also prefetch the rest of the warp's range into L2 up front (measured slower; off)
};

constexpr int kDecodeWarps = 32;
constexpr int kDecodeBatch = 4;    // blocks per register batch: 8 x 16-byte loads per lane

__device__ __forceinline__ void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// 32 bytes per lane in one instruction: with lanes (g,t) at row g, bytes t*32.., a warp reads one whole
// 1 KiB block (eight full 128-byte lines) per load instruction.
struct W32 { uint4 a, b; };
__device__ __forceinline__ W32 ldg_stream32(const void *p) {
  W32 v;
  asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v.a.x), "=r"(v.a.y), "=r"(v.a.z), "=r"(v.a.w), "=r"(v.b.x), "=r"(v.b.y), "=r"(v.b.z), "=r"(v.b.w) : "l"(p));
  return v;
}
__device__ __forceinline__ W32 w32_zero() { W32 v; v.a = make_uint4(0, 0, 0, 0); v.b = v.a; return v; }

template <bool A_UNSIGNED>
__global__ void __launch_bounds__(kDecodeWarps * 32, 1) decode_gemm_kernel(DecodeGemmArgs g, EpiParams epi) {
  extern __shared__ __align__(16) uint8_t smem[];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int lg = lane >> 2, lt = lane & 3;
  const int g0 = (int)((long long)blockIdx.x * g.groups / gridDim.x);
  const int g1 = (int)((long long)(blockIdx.x + 1) * g.groups / gridDim.x);
  const int total = (g1 - g0) * g.blocks;               // blocks owned by this CTA
  int item = (int)((long long)warp * total / kDecodeWarps);
  const int item_end = (int)((long long)(warp + 1) * total / kDecodeWarps);
  int32_t *red = reinterpret_cast<int32_t *>(smem + (size_t)g.rows_staged * g.a_stride);   // [local groups][16][8]
  const DecodeEpiSmem es = decode_epi_carve(smem + (size_t)g.rows_staged * g.a_stride + (size_t)g.max_local_groups * 512, g.max_local_groups);

  // ---- weights first: the first register batch is in flight while the activations are staged
  const int8_t *wlane = g.Wt + (size_t)g0 * g.Kp * 8 + lg * 128 + lt * 32;   // CTA's span is contiguous: item i at i*1024
  W32 w[kDecodeBatch];
#pragma unroll
  for (int u = 0; u < kDecodeBatch; ++u) w[u] = (item + u < item_end) ? ldg_stream32(wlane + (size_t)(item + u) * 1024) : w32_zero();
  for (int i = item + kDecodeBatch; i < item_end; ++i) {
    // one 128-byte line per (row, block): lanes with lt == 0 cover the eight rows
    if (lt == 0 && (g.tune & 1)) prefetch_l2(wlane + (size_t)i * 1024);
  }
  for (int i = tid; i < (g1 - g0) * 128; i += kDecodeWarps * 32) red[i] = 0;

  // ---- everything below may depend on the previous kernel of the stream
  asm volatile("griddepcontrol.wait;" ::: "memory");
  {
    const bool vec = ((reinterpret_cast<uintptr_t>(g.A) | (uintptr_t)g.lda) & 15) == 0;
    const int segs = g.Kp >> 4;
    for (int i = tid; i < g.rows_staged * segs; i += kDecodeWarps * 32) {
      const int r = i / segs, s = i - r * segs, k = s * 16;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < g.M && k < g.K) {
        const uint8_t *src = g.A + (size_t)r * g.lda + k;
        // whole aligned segments: asynchronous 16-byte copies, all of a thread's copies in flight at once (a load and a
        // store per segment left one segment per thread in flight: 16 KB per SM per round trip, 3 us for 176 KB)
        if (vec && k + 16 <= g.K) {
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem + (size_t)r * g.a_stride + k)), "l"(src) : "memory");
          continue;
        } else {
          uint8_t tmp[16];
#pragma unroll
          for (int b = 0; b < 16; ++b) tmp[b] = (k + b < g.K) ? src[b] : (uint8_t)0;
          v = *reinterpret_cast<uint4 *>(tmp);
        }
      }
      *reinterpret_cast<uint4 *>(smem + (size_t)r * g.a_stride + k) = v;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    decode_epi_stage(epi, es, g0 * 8, (g1 - g0) * 8, g.N, g.M, tid, kDecodeWarps * 32);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  }
  __syncthreads();

  const bool hi_rows = g.rows_staged > 8;
  const uint8_t *a_lo_base = smem + (size_t)lg * g.a_stride + lt * 32;
  const size_t a_hi_off = (size_t)8 * g.a_stride;

  int lgrp = item / g.blocks;                 // local group of the current block
  int c = item - lgrp * g.blocks;             // K block inside the group
  int acc[4] = {0, 0, 0, 0};
  auto flush = [&](int grp_local) {
    int32_t *s = red + grp_local * 128;
    const int col = lt * 2;
    atomicAdd(s + lg * 8 + col, acc[0]);
    atomicAdd(s + lg * 8 + col + 1, acc[1]);
    if (hi_rows) {
      atomicAdd(s + (lg + 8) * 8 + col, acc[2]);
      atomicAdd(s + (lg + 8) * 8 + col + 1, acc[3]);
    }
    acc[0] = acc[1] = acc[2] = acc[3] = 0;
  };
  // Batches: all loads of a batch are issued back to back and then consumed together.  (A rolling
  // refill of single registers measured half the bandwidth: the loads of one warp then complete
  // one after the other instead of overlapping.)
  for (int base = item; base < item_end; base += kDecodeBatch) {
    if (base != item) {
#pragma unroll
      for (int u = 0; u < kDecodeBatch; ++u) w[u] = (base + u < item_end) ? ldg_stream32(wlane + (size_t)(base + u) * 1024) : w32_zero();
    }
#pragma unroll
    for (int u = 0; u < kDecodeBatch; ++u) {
      if (base + u < item_end) {
        const uint4 w0 = w[u].a, w1 = w[u].b;
        const uint8_t *ap = a_lo_base + (size_t)c * 128;
        {
          const uint4 lo = *reinterpret_cast<const uint4 *>(ap);
          const uint4 hi = hi_rows ? *reinterpret_cast<const uint4 *>(ap + a_hi_off) : make_uint4(0, 0, 0, 0);
          mma_m16n8k32<A_UNSIGNED>(acc, lo.x, hi.x, lo.y, hi.y, w0.x, w0.y);
          mma_m16n8k32<A_UNSIGNED>(acc, lo.z, hi.z, lo.w, hi.w, w0.z, w0.w);
        }
        {
          const uint4 lo = *reinterpret_cast<const uint4 *>(ap + 16);
          const uint4 hi = hi_rows ? *reinterpret_cast<const uint4 *>(ap + 16 + a_hi_off) : make_uint4(0, 0, 0, 0);
          mma_m16n8k32<A_UNSIGNED>(acc, lo.x, hi.x, lo.y, hi.y, w1.x, w1.y);
          mma_m16n8k32<A_UNSIGNED>(acc, lo.z, hi.z, lo.w, hi.w, w1.z, w1.w);
        }
        if (++c == g.blocks) { flush(lgrp); c = 0; ++lgrp; }
      }
    }
  }
  if (c != 0 && item < item_end) flush(lgrp);
  __syncthreads();

  decode_epilogue(epi, es, red, g0, g1 - g0, g.M, g.N, tid, kDecodeWarps * 32);
}

}  // namespace b200
