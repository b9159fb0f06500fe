// Decode-shape W8A8 GEMM (M <= 16), bulk-copy ring form: the weight stream does not pass through registers.
// Stands in for the same reference paths as decode_gemm.cuh (AOCL-DLP call sites
// matmul/backends/aocl/aocl_kernel.cpp:1190-1301; native GEMV
// matmul/matmul_native/brgemm/kernel/int8/int8_gemv_bkc.cpp).
//
// Work split as in decode_gemm.cuh: CTA b owns the groups of eight output columns
// [b*G/grid, (b+1)*G/grid) of the block-interleaved packed weight (a group is Kp/128 contiguous 1 KiB
// blocks [8 rows][128 B of K]); no other CTA contributes to its outputs.  Inside the CTA:
//   - The groups are taken R at a time.  A stage of the shared-memory ring holds, for each of the R
//     groups, the same eight K blocks [c0, c0+8): R bulk copies of 8 KiB, issued by R lanes of the
//     producer warp (parallel issue hides the per-copy cost), completion on the stage's "full"
//     mbarrier.  A slot is refilled when the eight consumer warps have arrived on its "empty" mbarrier.
//     The bytes in flight per SM are the ring size, not a register budget.
//   - Consumer warp w owns K block c0+w of the stage: it reads its activation fragment once per stage
//     and uses it against the R weight blocks (one per group), so shared-memory traffic per weight byte
//     is 1 write + 1 read + 1/R activation reads.  The two 16-byte weight reads of a lane are ordered by
//     row parity so that a quarter-warp covers eight distinct 16-byte slots (no bank conflict).
//     mma.sync.m16n8k32 with the same K permutation on both operands as stream_gemm.cuh.
//   - Partial sums stay in registers for the whole K range of the R groups and are added into the
//     shared s32 accumulator [local group][16][8] once per group set (eight warps, integer adds).
//   - After one barrier all threads run the epilogue for the CTA's outputs.
// Programmatic dependent launch: the whole ring is requested before griddepcontrol.wait; the
// activations are read after it with cp.async (bulk copies of one SM complete in issue order, so a
// bulk copy of the activations would queue behind the ring).
// Every mbarrier wait is bounded; on expiry the CTA records a code in *status, the producer waits
// (bounded) for the copies it has in flight, and the CTA leaves without writing outputs.
#pragma once
#include "common.cuh"
#include "decode_epi.cuh"
#include "mbar.cuh"
#include "stream_gemm.cuh"

namespace b200 {

struct DecodeRingArgs {
  const uint8_t *A; int64_t lda;   // [M,lda] u8 or s8, M <= 16
  int M, N, K;
  const int8_t *Wt; int Kp;
  int groups;                      // ceil(N / 8)
  int blocks;                      // Kp / 128: 1 KiB blocks per group
  int a_stride;                    // smem row stride of A: Kp + 16
  int rows_staged;                 // M for M <= 8, else 16
  int max_local_groups;            // ceil(groups / gridDim.x)
  int stages;                      // ring depth
  int32_t *status;                 // device word: 0 ok
  int test_no_loads;               // test hook: the producer issues no copies, so the consumers' bounded waits run out
};

constexpr int kRingMaxStages = 16;
constexpr int kRingWarps = 8;      // consumer warps = K blocks per stage

// shared memory: [A rows][red][epilogue operands][barriers + error word][ring]
__host__ __device__ inline size_t ring_off_red(int rows_staged, int a_stride) { return (size_t)rows_staged * a_stride; }
__host__ __device__ inline size_t ring_off_bars(int rows_staged, int a_stride, int max_local_groups) {
  return ring_off_red(rows_staged, a_stride) + (size_t)max_local_groups * 512 + decode_epi_bytes(max_local_groups);
}
__host__ __device__ inline size_t ring_off_ring(int rows_staged, int a_stride, int max_local_groups) {
  return (ring_off_bars(rows_staged, a_stride, max_local_groups) + (2 * kRingMaxStages + 2) * 8 + 127) & ~(size_t)127;
}

template <bool A_UNSIGNED, int R>
__global__ void __launch_bounds__((kRingWarps + 1) * 32, 1) decode_ring_kernel(DecodeRingArgs g, EpiParams epi) {
  extern __shared__ __align__(128) uint8_t ring_smem[];
  uint8_t *const smem = ring_smem;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  constexpr int NCW = kRingWarps;
  constexpr int kCopyBytes = NCW * 1024;                // one group's share of a stage
  constexpr int kStageBytes = R * kCopyBytes;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int lg = lane >> 2, lt = lane & 3;
  const int g0 = (int)((long long)blockIdx.x * g.groups / gridDim.x);
  const int g1 = (int)((long long)(blockIdx.x + 1) * g.groups / gridDim.x);
  const int n_local = g1 - g0;
  const int per_set = (g.blocks + NCW - 1) / NCW;       // stages per set of R groups
  const int n_stages = ((n_local + R - 1) / R) * per_set;
  const int S = g.stages;
  int32_t *red = reinterpret_cast<int32_t *>(smem + ring_off_red(g.rows_staged, g.a_stride));
  const DecodeEpiSmem es = decode_epi_carve(smem + ring_off_red(g.rows_staged, g.a_stride) + (size_t)g.max_local_groups * 512, g.max_local_groups);
  const size_t bars_off = ring_off_bars(g.rows_staged, g.a_stride, g.max_local_groups);
  const uint32_t bars = smem_u32(smem + bars_off);
  uint8_t *ring = smem + ring_off_ring(g.rows_staged, g.a_stride, g.max_local_groups);
  auto full_bar = [&](int s) { return bars + 8u * (uint32_t)s; };
  auto empty_bar = [&](int s) { return bars + 8u * (uint32_t)(kRingMaxStages + s); };
  volatile int &s_err = *reinterpret_cast<volatile int *>(smem + bars_off + 8 * (2 * kRingMaxStages + 1));

  if (tid == 0) {
    s_err = 0;
    for (int s = 0; s < S; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), NCW); }
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == NCW) {
    // ------------------------------------------------------------------ producer warp
    const int8_t *span = g.Wt + (size_t)g0 * g.Kp * 8;
    const uint32_t ring_s = smem_u32(ring);
    auto issue = [&](int st) {
      const int slot = st % S;
      const int set = st / per_set, c0 = (st - set * per_set) * NCW;
      const int nblk = (g.blocks - c0) < NCW ? (g.blocks - c0) : NCW;
      const int ngrp = (n_local - set * R) < R ? (n_local - set * R) : R;
      if (lane == 0) mbar_expect_tx(full_bar(slot), (uint32_t)(ngrp * nblk) * 1024u);
      __syncwarp();
      if (lane < ngrp)
        bulk_load(ring_s + (uint32_t)slot * kStageBytes + (uint32_t)lane * kCopyBytes,
                  span + ((size_t)(set * R + lane) * g.blocks + c0) * 1024, (uint32_t)nblk * 1024u, full_bar(slot));
    };
    int st = 0;
    bool ok = true;
    const int pre = g.test_no_loads ? 0 : (n_stages < S ? n_stages : S);
    for (; st < pre; ++st) issue(st);
    for (; st < n_stages && !g.test_no_loads; ++st) {
      if (st >= S && !mbar_wait(empty_bar(st % S), (uint32_t)((st / S) - 1) & 1u)) { ok = false; break; }
      issue(st);
    }
    if (!ok) {
      if (lane == 0) { s_err = 1; report_status(g.status, 11); }
      // copies in flight must land before the CTA leaves
      const int first = st > S ? st - S : 0;
      for (int q = first; q < st; ++q) mbar_wait(full_bar(q % S), (uint32_t)(q / S) & 1u);
    }
  } else {
    // ------------------------------------------------------------------ consumers
    asm volatile("griddepcontrol.wait;" ::: "memory");
    constexpr int kConsumers = NCW * 32;
    for (int i = tid; i < n_local * 128; i += kConsumers) red[i] = 0;
    {
      // activations: 16-byte asynchronous copies (cp.async), all in flight at once.  Not bulk copies: those
      // complete in issue order per SM and would queue behind the ring.
      const bool vec = ((reinterpret_cast<uintptr_t>(g.A) | (uintptr_t)g.lda) & 15) == 0;
      const int kv = vec ? (g.K & ~15) : 0;                // bytes per row that can go as aligned 16-byte pieces
      for (int r = 0; r < g.M; ++r) {
        const uint8_t *src = g.A + (size_t)r * g.lda;
        const uint32_t dst = smem_u32(smem + (size_t)r * g.a_stride);
        for (int k = tid * 16; k < kv; k += kConsumers * 16)
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (uint32_t)k), "l"(src + k) : "memory");
        for (int k = kv + tid; k < g.K; k += kConsumers) smem[(size_t)r * g.a_stride + k] = src[k];
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      decode_epi_stage(epi, es, g0 * 8, n_local * 8, g.N, g.M, tid, kConsumers);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory");
    bool ok = true;

    // Rows >= M of a 16-row staging area are never written: an output row depends only on its own
    // activation row, and rows >= M are not stored.  Columns k >= K hold zero weights.
    const bool hi_rows = g.rows_staged > 8;
    // M <= 8: only M rows are staged; lanes of the rows that do not exist read the last real row (their outputs are not stored)
    const int lo_row = hi_rows ? lg : (lg < g.rows_staged ? lg : g.rows_staged - 1);
    const uint8_t *a_lo_base = smem + (size_t)lo_row * g.a_stride + lt * 32;
    const size_t a_hi_off = (size_t)8 * g.a_stride;
    const int odd = lg & 1;
    const uint32_t w_lane = (uint32_t)warp * 1024u + (uint32_t)lg * 128u + (uint32_t)lt * 32u + (odd ? 16u : 0u);
    int acc[R][4];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0;

    int set = 0, sc = 0;                                   // group set and stage inside the set
    for (int st = 0; ok && st < n_stages; ++st) {
      const int slot = st % S;
      const int c = sc * NCW + warp;
      uint4 lo0 = make_uint4(0, 0, 0, 0), lo1 = lo0, hi0 = lo0, hi1 = lo0;
      if (c < g.blocks) {
        const uint8_t *ap = a_lo_base + (size_t)c * 128;
        lo0 = *reinterpret_cast<const uint4 *>(ap);
        lo1 = *reinterpret_cast<const uint4 *>(ap + 16);
        if (hi_rows) { hi0 = *reinterpret_cast<const uint4 *>(ap + a_hi_off); hi1 = *reinterpret_cast<const uint4 *>(ap + 16 + a_hi_off); }
      }
      if (!mbar_wait(full_bar(slot), (uint32_t)(st / S) & 1u)) { ok = false; if (lane == 0) { s_err = 1; report_status(g.status, 13); } break; }
      if (c < g.blocks) {
        const uint8_t *wp = ring + (size_t)slot * kStageBytes + w_lane;
        const int ngrp = n_local - set * R;
        uint4 wa[R], wb[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          if (r < ngrp) {
            wa[r] = *reinterpret_cast<const uint4 *>(wp + r * kCopyBytes);
            wb[r] = *reinterpret_cast<const uint4 *>(wp + r * kCopyBytes + (odd ? -16 : 16));
          }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
          if (r < ngrp) {
            const uint4 w0 = odd ? wb[r] : wa[r], w1 = odd ? wa[r] : wb[r];
            mma_m16n8k32<A_UNSIGNED>(acc[r], lo0.x, hi0.x, lo0.y, hi0.y, w0.x, w0.y);
            mma_m16n8k32<A_UNSIGNED>(acc[r], lo0.z, hi0.z, lo0.w, hi0.w, w0.z, w0.w);
            mma_m16n8k32<A_UNSIGNED>(acc[r], lo1.x, hi1.x, lo1.y, hi1.y, w1.x, w1.y);
            mma_m16n8k32<A_UNSIGNED>(acc[r], lo1.z, hi1.z, lo1.w, hi1.w, w1.z, w1.w);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(slot));
      if (++sc == per_set) {
        // the K range of this group set is complete: add the partial sums into the CTA accumulator
        const int ngrp = n_local - set * R;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          if (r < ngrp) {
            int32_t *s = red + (set * R + r) * 128;
            const int col = lt * 2;
            atomicAdd(s + lg * 8 + col, acc[r][0]);
            atomicAdd(s + lg * 8 + col + 1, acc[r][1]);
            if (hi_rows) {
              atomicAdd(s + (lg + 8) * 8 + col, acc[r][2]);
              atomicAdd(s + (lg + 8) * 8 + col + 1, acc[r][3]);
            }
          }
          acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0;
        }
        sc = 0; ++set;
      }
    }
  }
  __syncthreads();
  if (s_err) return;

  decode_epilogue(epi, es, red, g0, n_local, g.M, g.N, tid, (NCW + 1) * 32);
}

}  // namespace b200
