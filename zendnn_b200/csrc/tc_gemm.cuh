// tcgen05 W8A8 GEMM for sm_100a: the prefill-sized and grouped (MoE) form of the INT8 GEMM that
// the reference delegates to its backend (matmul/backends/aocl/aocl_kernel.cpp:1190-1301) and, for
// group_matmul_direct, to its tile micro-kernel (matmul/group_matmul/custom_kernel/ukernel/
// int8_microkernel.hpp:39-56) under a CPU scheduler (matmul/group_matmul/group_matmul_dispatch.cpp).
//
// One persistent CTA per SM, 608 threads, four roles:
//   warp 0     TMA producer: per K block of 128 bytes, one [128 x 128 B] box of A and one
//              [BN x 128 B] box of the packed weight into a ring of shared-memory stages
//              (SWIZZLE_128B, no multicast), completion on an mbarrier.
//   warp 1     MMA issuer: one lane issues tcgen05.mma.cta_group::1.kind::i8 (M=128, N=BN, K=32),
//              four per stage, accumulating s32 in tensor memory; tcgen05.commit releases the
//              stage and, after the last K block, publishes the accumulator.
//   warps 2-17 epilogue: tcgen05.ld the accumulator (one TMEM lane = one output row per thread, four
//              warps per lane quadrant, each taking a share of the tile's 32-column chunks), dequantise / bias /
//              post-ops (or gated activation) and store; results leave through a small per-warp
//              shared-memory block so that every store instruction writes whole 32-byte sectors of
//              16 rows.  Two accumulator buffers (2 x BN <= 512 TMEM columns) let the epilogue of tile i
//              overlap the MMAs of tile i+1.
//   warp 18    operand warp: runs one tile ahead of the epilogue and puts everything the epilogue needs
//              from global memory into double-buffered shared memory: the tile's coordinates and output
//              pointer, the per-column operands of its BN columns and the source scales of its 128 rows.
//              The epilogue warps then read only tensor memory and shared memory.
// Tile order: column-tile-major (CTAs running together share a weight tile through L2), or, when the
// activations are the large operand and a group's weight stays in L2, row-tile-major (n_fastest).
// Shared memory is the busiest resource (TMA writes the operands, the tensor core reads them back), so
// the epilogue keeps its own shared-memory traffic small.
// Grouped form: A is one [rows x K] matrix holding every expert's rows back to back; row offsets
// and the cumulative tile counts live in device memory, so no host round trip is needed after routing.
// Pair form (tc_gemm_kernel<false, true>, large plain and grouped GEMMs): clusters of two CTAs on neighbouring SMs
// work on one [256 x BN] tile with tcgen05.mma.cta_group::2.  Each CTA loads its own 128 rows of A and its own half
// (BN/2 rows) of the weight tile with plain, non-multicast TMA copies that complete on the leader CTA's barrier; the
// leader's MMA warp issues M256 MMAs for both, the tensor cores exchange the weight halves between the two shared
// memories themselves, and each CTA's epilogue warps finish the 128 rows whose accumulators sit in its own tensor
// memory.  Per MMA a CTA's shared memory takes half the weight bytes it takes in the single-CTA form, and shared-memory
// bandwidth (copy engine writing, tensor core reading) is what bounds the single-CTA form.
// Every wait is bounded: on expiry the kernel records a code in *status and leaves.
#pragma once
#include <cuda.h>
#include "common.cuh"
#include "mbar.cuh"
#include "pack_kernels.cuh"

namespace b200 {

constexpr int kTcBM = 128;
constexpr int kTcBK = 128;               // bytes of K per stage row (one 128-byte swizzle span)
#ifndef B200_TC_EPI_WARPS
#define B200_TC_EPI_WARPS 16
#endif
constexpr int kTcEpiWarps = B200_TC_EPI_WARPS;      // a multiple of 4: each warp may only read its own quadrant of TMEM lanes
constexpr int kTcEpiParts = kTcEpiWarps / 4;          // warps per lane quadrant, each taking a share of the tile's columns
constexpr int kTcThreads = 96 + 32 * kTcEpiWarps;   // producer warp + MMA warp + epilogue warps + operand warp
constexpr int kTcSmemBudget = 200 * 1024; // stage ring

struct TcGroupDesc {   // per expert, device memory (grouped form with caller-owned outputs)
  const void *wei_scale;
  const int32_t *colsum;
  const void *bias;
  void *dst;
  int64_t ldc;
};

struct TcGemmArgs {
  int n_groups;               // 1: plain GEMM
  int M_total;                // rows of A
  int N;                      // packed columns to produce (N, or 2*I in gated form)
  int k_blocks;               // Kp / 128
  int BN, stages;
  int n_tiles;                // ceil(N / BN)
  int m_tiles_plain;          // plain form: ceil(M / 128), or ceil(M / 256) in the pair form
  const int32_t *row_off;     // grouped: [n_groups+1] first row of each group (device)
  const int32_t *tile_prefix; // grouped: [n_groups+1] cumulative row tiles (128 rows each; 256 in the pair form) (device)
  const CUtensorMap *maps_b;  // grouped: one map per group (device memory); plain: null
  const TcGroupDesc *groups;  // grouped, optional: per-group epilogue pointers (local row index)
  int a_unsigned;
  int gated;                  // packed gate/up interleave: 0, 1 or 2 (see pack_kernels.cuh)
  int fast_act;               // FA_* code: which specialised epilogue loop to run
  int dbg;                    // timing experiments, only in builds with B200DNN_TIMING_EXPERIMENTS (results invalid):
                              // 1 no epilogue work, 2 tensor-memory loads only, 3 no stores; otherwise 0
  int shared_dst;             // every group writes epi.dst at its global row (set by the caller); plain GEMM: 1
  int tma_store;              // bf16 results of full 32-row blocks leave through TMA stores (map_c covers the shared destination)
  int test_no_loads;          // test hook: the producer issues no copies, so every wait on data runs out (bounded) and the
                              // kernel must leave with a status code and a usable context
  int k_splits;               // split form (tc_gemm_kernel<true>): the CTAs of a cluster each take a share of the K blocks of one
                              // tile and add their int32 partial sums through distributed shared memory (exact in any order)
  int n_fastest;              // tile order: 0 = all row tiles of a column tile first, 1 = all column tiles of a row tile first
  int pair;                   // pair form (tc_gemm_kernel<false, true>): row tiles are 256 rows, m_tiles_plain / tile_prefix count those
  int f16;                    // bf16 x bf16 form (tc_gemm_kernel<.., .., true>): kind::f16 MMAs, f32 accumulators, no scales
  int32_t *status;            // device word: 0 ok
  unsigned long long *stamps; // timing experiments only (builds with B200DNN_TIMING_EXPERIMENTS): 8 timer values per CTA; else null
};

#ifdef B200DNN_TIMING_EXPERIMENTS
#define TC_STAMP(i) do { if (a.stamps) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); \
                                          a.stamps[(size_t)blockIdx.x * 8 + (i)] = t_; } } while (0)
#else
#define TC_STAMP(i) do { } while (0)
#endif

// ---------------------------------------------------------------------------------------- PTX
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// weight box from the block-interleaved layout: coordinates {byte 0, row-in-group 0, K block, row group}
__device__ __forceinline__ void tma_load_wt(uint32_t dst, const CUtensorMap *map, int kblock, int group, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
               ::"r"(dst), "l"(map), "r"(0), "r"(0), "r"(kblock), "r"(group), "r"(bar) : "memory");
}
// pair form: the copy lands in this CTA's shared memory, its bytes are counted on the barrier `bar` of the leader CTA
// (a shared::cluster address); no multicast
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_wt_pair(uint32_t dst, const CUtensorMap *map, int kblock, int group, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
               ::"r"(dst), "l"(map), "r"(0), "r"(0), "r"(kblock), "r"(group), "r"(bar) : "memory");
}
// completion of the pair's MMAs, signalled on the barrier at the same offset in both CTAs
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tc_mma_i8_pair(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}"
               ::"r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// arrive on a barrier of another CTA of the cluster (shared::cluster address from cluster_map)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}"
               ::"r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
// 32 contiguous bytes of one row in one instruction: every lane writes a whole sector of its own row, so the stores of a
// warp are full sectors without any exchange between the lanes.  The address must be 32-byte aligned.
__device__ __forceinline__ void st_global_v8(void *p, const uint32_t (&v)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
// every thread of every CTA of the cluster; the cluster's CTAs are scheduled together, so the wait ends once each thread
// has left its own (bounded) waits
__device__ __forceinline__ void cluster_sync_all() {
  __syncwarp();
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_arrive_all() {
  __syncwarp();
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_all() {
  __syncwarp();
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_map(uint32_t saddr, uint32_t rank) {
  uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank)); return r;
}
__device__ __forceinline__ uint4 ld_cluster_v4(uint32_t caddr) {
  uint4 v; asm volatile("ld.shared::cluster.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(caddr) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t saddr) {
  uint4 v; asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(saddr) : "memory");
  return v;
}
__device__ __forceinline__ void st_shared_v4(uint32_t saddr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// bf16 x bf16 -> f32, M x N x 16 (32 bytes of K per instruction, as kind::i8)
__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}"
               ::"r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
               ::"r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}

// K-major, SWIZZLE_128B shared-memory operand descriptor: 8-row groups 1024 B apart
// (stride byte offset), leading byte offset unused for swizzled K-major, descriptor version 1.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// instruction descriptor, kind::i8: D = s32, A = u8|s8, B = s8, both K-major, M = 128, N = BN
__host__ __device__ inline uint32_t make_idesc_i8(int a_unsigned, int BN, int M = kTcBM) {
  return (2u << 4) | ((a_unsigned ? 0u : 1u) << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// instruction descriptor, kind::f16: D = f32, A = B = bf16, both K-major
__host__ __device__ inline uint32_t make_idesc_bf16(int BN, int M = kTcBM) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

struct TileCoord { int g, row0, rows, m_local0, nt; };

// Same mapping computed by a whole warp: the group of a row tile is the number of prefix entries
// tile_prefix[1..n_groups) that are <= the tile index (empty groups repeat a prefix value and are skipped).
// tile_m: rows of a tile (128, or 256 in the pair form); sub: this CTA's first row inside the tile (pair form: 128 for
// the second CTA).  rows may be 0 for the second CTA of a pair at the end of a group.
__device__ __forceinline__ TileCoord tc_tile_warp(const TcGemmArgs &a, int tile, int m_tiles, int lane, int tile_m = kTcBM, int sub = 0) {
  TileCoord t;
  int mt;
  if (a.n_fastest) { mt = tile / a.n_tiles; t.nt = tile - mt * a.n_tiles; }
  else { t.nt = tile / m_tiles; mt = tile - t.nt * m_tiles; }
  if (!a.tile_prefix) {
    t.g = 0; t.m_local0 = mt * tile_m + sub; t.row0 = t.m_local0; t.rows = max(0, min(kTcBM, a.M_total - t.row0));
    return t;
  }
  int g = 0;
  for (int base = 1; base < a.n_groups; base += 32) {
    const int i = base + lane;
    const bool le = i < a.n_groups && a.tile_prefix[i] <= mt;
    g += __popc(__ballot_sync(0xffffffffu, le));
  }
  t.g = g;
  t.m_local0 = (mt - a.tile_prefix[g]) * tile_m + sub;
  t.row0 = a.row_off[g] + t.m_local0;
  t.rows = max(0, min(kTcBM, a.row_off[g + 1] - t.row0));
  return t;
}

struct TileMeta {          // what the epilogue needs to know about a tile, written by the operand warp
  int row0, rows, m_dst0, nt;
  void *dst; int64_t ldc;
  int has_bias;
};

// ---- epilogue arithmetic ---------------------------------------------------------------------------
// Post-op structure resolved on the host so that the per-element loop carries no dispatch.
enum : int { FA_GENERIC = -1, FA_NONE = 0, FA_RELU, FA_GELU_TANH, FA_GELU_ERF, FA_SIGMOID, FA_SWISH, FA_TANH };

// sigmoid-family activations through one exp and one reciprocal.  gelu_tanh uses the identity
// 0.5*x*(1+tanh(u)) = x / (1 + exp(-2u)), which has no cancellation for very negative u.
__device__ __forceinline__ float fast_sigmoid_mul(float x, float arg) { return __fdividef(x, 1.0f + __expf(-arg)); }

template <int ACT>
__device__ __forceinline__ float tc_act(const EpiParams &epi, float x, int m, int n) {
  if (ACT == FA_NONE) return x;
  if (ACT == FA_RELU) return fmaxf(x, 0.0f);
  if (ACT == FA_GELU_TANH) {
    const float c = 0.79788458347320556640625f, f = 0.044715f;
    const float inner = (c * x) * (1.0f + (f * x) * x);
    return fast_sigmoid_mul(x, 2.0f * inner);
  }
  if (ACT == FA_GELU_ERF) return po_gelu_erf(x);
  if (ACT == FA_SIGMOID) return fast_sigmoid_mul(1.0f, x);
  if (ACT == FA_SWISH) return fast_sigmoid_mul(x, x);
  if (ACT == FA_TANH) return tanhf(x);
  for (int i = 0; i < epi.n_po; ++i) x = apply_postop(epi.po[i], x, m, n);
  return x;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  // one instruction; same round-to-nearest-even as the reference's bit trick for every finite value
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}

struct TileCols {          // per-tile column operands staged in shared memory
  float ws[256];
  float bias[256];
  int32_t comp[256];
};

// Coalesced store of a [32 rows x 32 bytes] block that a warp holds one row per lane (v[0], v[1] = the row's
// two 16-byte pieces).  The block goes through the warp's 1 KiB of shared memory (pieces swapped on every
// second group of four rows so that both the writes and the reads are free of bank conflicts) and leaves
// as two instructions that each write 16 rows x 32 contiguous bytes (whole sectors), instead of 32
// scattered 16-byte pieces per instruction.
// g_row0: address of the block's first row; rows_valid: how many of the 32 rows exist.
__device__ __forceinline__ void warp_store_rows32(uint8_t *sbuf, const uint4 &v0, const uint4 &v1, uint8_t *g_row0, int64_t pitch_bytes,
                                                  int rows_valid, int lane) {
  const int sw = (lane >> 2) & 1;
  *reinterpret_cast<uint4 *>(sbuf + lane * 32 + ((0 ^ sw) << 4)) = v0;
  *reinterpret_cast<uint4 *>(sbuf + lane * 32 + ((1 ^ sw) << 4)) = v1;
  __syncwarp();
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int R = 16 * j + (lane >> 1), p = lane & 1;
    const uint4 val = *reinterpret_cast<const uint4 *>(sbuf + R * 32 + ((p ^ ((R >> 2) & 1)) << 4));
    if (R < rows_valid) *reinterpret_cast<uint4 *>(g_row0 + (int64_t)R * pitch_bytes + p * 16) = val;
  }
  __syncwarp();
}
// [32 rows x 64 bytes] as two such blocks
__device__ __forceinline__ void warp_store_rows64(uint8_t *sbuf, const uint4 (&v)[4], uint8_t *g_row0, int64_t pitch_bytes,
                                                  int rows_valid, int lane) {
  warp_store_rows32(sbuf, v[0], v[1], g_row0, pitch_bytes, rows_valid, lane);
  warp_store_rows32(sbuf, v[2], v[3], g_row0 + 32, pitch_bytes, rows_valid, lane);
}

// The same [32 rows x 32 bytes] block as one TMA store: the lanes write their rows to the staging block (plain row-major),
// one lane hands it to the copy engine and waits until the engine has read it.  Keeps the result off the load/store path.
__device__ __forceinline__ void warp_tma_store_rows32(uint8_t *sbuf, const uint4 &v0, const uint4 &v1, const CUtensorMap *map,
                                                      int x_bytes, int row, int lane) {
  *reinterpret_cast<uint4 *>(sbuf + lane * 32) = v0;
  *reinterpret_cast<uint4 *>(sbuf + lane * 32 + 16) = v1;
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();
  if (lane == 0) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(x_bytes), "r"(row), "r"(smem_u32(sbuf)) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
  }
  __syncwarp();
}

struct EpiStore {          // where this warp's rows of the current tile go
  uint8_t *sbuf;           // the warp's staging block
  uint8_t *g_row0;         // address of (first row of the warp, column 0) in the destination
  int64_t pitch_bytes;
  int rows_valid;          // rows of the warp's 32 that exist in this tile
  bool coalesce;           // destination 16-byte aligned: use the staged path
  bool v8;                 // destination and pitch 32-byte aligned: every lane stores 32-byte pieces of its own row directly
  bool row_ok;             // this lane's row exists
  const CUtensorMap *map_c;  // non-null: full blocks go out as TMA stores, coordinates (byte column, row)
  int row_c;               // row coordinate of the warp's first row in map_c
};

// One 32-column chunk of one output row.  Results leave, in this order of preference, as 32-byte stores of the lane's own
// row (destination 32-byte aligned), through the warp's staging block (16-byte aligned), or element by element.
// accumulator -> f32 before bias: the dequantising chain of the INT8 forms, or the f32 sum of the bf16 form as it is
template <bool F16>
__device__ __forceinline__ float tc_acc_f32(uint32_t r, int comp, float s_src, float w) {
  if constexpr (F16) return __uint_as_float(r);
  else return __fmul_rn(__fmul_rn((float)((int32_t)r - comp), s_src), w);
}

template <int ACT, bool F16>
__device__ __forceinline__ void tc_epi_chunk(const EpiParams &epi, const EpiCtx &cx, const uint32_t (&r)[32], const TileCols &tc,
                                             int c0, int pc0, int N, int m_dst, bool has_bias, const EpiStore &es, int lane) {
  const bool has_zp = !F16 && epi.has_zp != 0;
  if (!F16 && epi.dst_dt == DT_S32) {
    int32_t y[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) y[i] = has_zp ? (int32_t)r[i] - tc.comp[c0 + i] : (int32_t)r[i];
    if (es.v8 && pc0 + 32 <= N) {
      if (es.row_ok) {
        uint8_t *o = reinterpret_cast<uint8_t *>(cx.dst) + ((int64_t)m_dst * cx.ldc + pc0) * 4;
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          uint32_t v[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = (uint32_t)y[8 * p + i];
          st_global_v8(o + 32 * p, v);
        }
      }
    } else if (es.coalesce && pc0 + 32 <= N) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint4 v[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) v[p] = make_uint4(y[16 * h + 4 * p], y[16 * h + 4 * p + 1], y[16 * h + 4 * p + 2], y[16 * h + 4 * p + 3]);
        warp_store_rows64(es.sbuf, v, es.g_row0 + (size_t)(pc0 + 16 * h) * 4, es.pitch_bytes, es.rows_valid, lane);
      }
    } else if (es.row_ok) {
      int32_t *o = reinterpret_cast<int32_t *>(cx.dst) + (int64_t)m_dst * cx.ldc + pc0;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (pc0 + i < N) o[i] = y[i];
    }
    return;
  }
  // two halves of 16 columns: fewer values live at once
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float x[16];
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
      // shared memory is the busiest resource of this kernel (the tensor core reads its operands from it):
      // bias and compensation are fetched only when they exist
      const int ci = c0 + 16 * h + i;
      float4 w4 = make_float4(1.f, 1.f, 1.f, 1.f);
      if constexpr (!F16) w4 = *reinterpret_cast<const float4 *>(&tc.ws[ci]);
      float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
      int4 k4 = make_int4(0, 0, 0, 0);
      if (has_bias) b4 = *reinterpret_cast<const float4 *>(&tc.bias[ci]);
      if (has_zp) k4 = *reinterpret_cast<const int4 *>(&tc.comp[ci]);
      const float wv[4] = {w4.x, w4.y, w4.z, w4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
      const int kv[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v = tc_acc_f32<F16>(r[16 * h + i + j], kv[j], cx.s_src, wv[j]);
        if (has_bias) v = __fadd_rn(v, bv[j]);
        x[i + j] = tc_act<ACT>(epi, v, m_dst, pc0 + 16 * h + i + j);
      }
    }
    const int pc = pc0 + 16 * h;          // first column of this half
    const bool full = pc + 16 <= N;
    if (epi.dst_dt == DT_BF16) {
      uint32_t pk[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) pk[i] = pack_bf16x2(x[2 * i], x[2 * i + 1]);
      if (es.map_c && es.rows_valid == 32 && full) {
        warp_tma_store_rows32(es.sbuf, make_uint4(pk[0], pk[1], pk[2], pk[3]), make_uint4(pk[4], pk[5], pk[6], pk[7]), es.map_c, pc * 2, es.row_c, lane);
      } else if (es.v8 && full) {
        if (es.row_ok) st_global_v8(reinterpret_cast<uint8_t *>(cx.dst) + ((int64_t)m_dst * cx.ldc + pc) * 2, pk);
      } else if (es.coalesce && full) {
        warp_store_rows32(es.sbuf, make_uint4(pk[0], pk[1], pk[2], pk[3]), make_uint4(pk[4], pk[5], pk[6], pk[7]),
                          es.g_row0 + (size_t)pc * 2, es.pitch_bytes, es.rows_valid, lane);
      } else if (es.row_ok) {
        uint16_t *o = reinterpret_cast<uint16_t *>(cx.dst) + (int64_t)m_dst * cx.ldc + pc;
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (pc + i < N) o[i] = (uint16_t)(pk[i >> 1] >> ((i & 1) * 16));
      }
    } else {
      if (es.v8 && full) {
        if (es.row_ok) {
          uint8_t *o = reinterpret_cast<uint8_t *>(cx.dst) + ((int64_t)m_dst * cx.ldc + pc) * 4;
#pragma unroll
          for (int p = 0; p < 2; ++p) {
            uint32_t v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __float_as_uint(x[8 * p + i]);
            st_global_v8(o + 32 * p, v);
          }
        }
      } else if (es.coalesce && full) {
        uint4 v[4];
#pragma unroll
        for (int p = 0; p < 4; ++p)
          v[p] = make_uint4(__float_as_uint(x[4 * p]), __float_as_uint(x[4 * p + 1]), __float_as_uint(x[4 * p + 2]), __float_as_uint(x[4 * p + 3]));
        warp_store_rows64(es.sbuf, v, es.g_row0 + (size_t)pc * 4, es.pitch_bytes, es.rows_valid, lane);
      } else if (es.row_ok) {
        float *o = reinterpret_cast<float *>(cx.dst) + (int64_t)m_dst * cx.ldc + pc;
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (pc + i < N) o[i] = x[i];
      }
    }
  }
}

template <bool F16>
__device__ __forceinline__ void tc_epi_dispatch(int fast_act, const EpiParams &epi, const EpiCtx &cx, const uint32_t (&r)[32],
                                                const TileCols &tcols, int c0, int pc0, int N, int m_dst, bool has_bias,
                                                const EpiStore &es, int lane) {
  switch (fast_act) {
  case FA_NONE: tc_epi_chunk<FA_NONE, F16>(epi, cx, r, tcols, c0, pc0, N, m_dst, has_bias, es, lane); break;
  case FA_RELU: tc_epi_chunk<FA_RELU, F16>(epi, cx, r, tcols, c0, pc0, N, m_dst, has_bias, es, lane); break;
  case FA_GELU_TANH: tc_epi_chunk<FA_GELU_TANH, F16>(epi, cx, r, tcols, c0, pc0, N, m_dst, has_bias, es, lane); break;
  case FA_GELU_ERF: tc_epi_chunk<FA_GELU_ERF, F16>(epi, cx, r, tcols, c0, pc0, N, m_dst, has_bias, es, lane); break;
  case FA_SIGMOID: tc_epi_chunk<FA_SIGMOID, F16>(epi, cx, r, tcols, c0, pc0, N, m_dst, has_bias, es, lane); break;
  case FA_SWISH: tc_epi_chunk<FA_SWISH, F16>(epi, cx, r, tcols, c0, pc0, N, m_dst, has_bias, es, lane); break;
  case FA_TANH: tc_epi_chunk<FA_TANH, F16>(epi, cx, r, tcols, c0, pc0, N, m_dst, has_bias, es, lane); break;
  default: tc_epi_chunk<FA_GENERIC, F16>(epi, cx, r, tcols, c0, pc0, N, m_dst, has_bias, es, lane); break;
  }
}

// SPLIT: launched in clusters of a.k_splits CTAs, one tile per cluster (see TcGemmArgs::k_splits); plain, non-gated form only.
// PAIR: launched in clusters of two CTAs that share [256 x BN] tiles through cta_group::2 MMAs (see the head of this file).
// F16: the bf16 x bf16 form (kind::f16 MMAs over the same byte tiles, f32 accumulators); with SPLIT its f32 partial sums are
// added in a fixed order.
template <bool SPLIT, bool PAIR = false, bool F16 = false>
__global__ void __launch_bounds__(kTcThreads, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b0,
               const __grid_constant__ CUtensorMap map_c, const TcGemmArgs a, const EpiParams epi) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * 8 + 8];
  __shared__ __align__(16) TileCols cols[2];
  __shared__ __align__(16) float row_scale[2][kTcBM];
  __shared__ TileMeta meta[2];
  __shared__ __align__(128) uint8_t epi_stage[kTcEpiWarps][1024];
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile int s_err;

  // programmatic dependent launch: the next kernel of the stream may take this CTA's SM as soon as it is free; this
  // kernel touches global memory only after griddepcontrol.wait below (the set-up before it uses none)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) TC_STAMP(0);
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  static_assert(!(SPLIT && PAIR), "the split form and the pair form are separate kernels");

  // pair form: this CTA holds its 128 rows of A and its half of the tile's weight rows
  const uint32_t a_bytes = kTcBM * kTcBK, b_bytes = (uint32_t)(PAIR ? a.BN / 2 : a.BN) * kTcBK, stage_bytes = a_bytes + b_bytes;
  const int S = a.stages;
  uint32_t crank = 0;
  if constexpr (SPLIT || PAIR) crank = cluster_ctarank();
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (8 + s); };
  auto tfull_bar = [&](int i) { return bar0 + 8u * (16 + i); };
  auto tempty_bar = [&](int i) { return bar0 + 8u * (18 + i); };
  auto cfull_bar = [&](int i) { return bar0 + 8u * (20 + i); };
  auto cempty_bar = [&](int i) { return bar0 + 8u * (22 + i); };

  if (threadIdx.x == 0) {
    // the copy engine reads the tensor maps from memory on first use: ask for them now
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    if (!a.maps_b) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b0) : "memory");
    if (a.tma_store) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_c) : "memory");
    for (int s = 0; s < S; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    // pair form: the epilogue warps of both CTAs release the accumulator on the leader's barrier
    for (int i = 0; i < 2; ++i) { mbar_init(tfull_bar(i), 1); mbar_init(tempty_bar(i), PAIR ? 2 * kTcEpiWarps : kTcEpiWarps); }
    for (int i = 0; i < 2; ++i) { mbar_init(cfull_bar(i), 1); mbar_init(cempty_bar(i), kTcEpiWarps); }
    s_err = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      // the same warp of both CTAs allocates for the pair
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(512u) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(512u) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();   // the partner's barriers exist before anything of this CTA signals them
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  asm volatile("griddepcontrol.wait;" ::: "memory");   // everything before this launch in the stream is complete and visible
  if (threadIdx.x == 0) TC_STAMP(1);

  const int m_tiles = a.tile_prefix ? a.tile_prefix[a.n_groups] : a.m_tiles_plain;
  const int total_tiles = m_tiles * a.n_tiles;
  // persistent form: tiles blockIdx.x, blockIdx.x + gridDim.x, ... over all K blocks; split form: the cluster's one tile,
  // this CTA's share of the K blocks
  int tile0 = blockIdx.x, tile_step = gridDim.x, kb_begin = 0, kb_end = a.k_blocks;
  constexpr int tile_m = PAIR ? 2 * kTcBM : kTcBM;
  const int sub = PAIR ? (int)crank * kTcBM : 0;
  if constexpr (PAIR) { tile0 = blockIdx.x >> 1; tile_step = gridDim.x >> 1; }
  if constexpr (SPLIT) {
    tile0 = blockIdx.x / a.k_splits; tile_step = total_tiles;
    const int per = (a.k_blocks + a.k_splits - 1) / a.k_splits;
    kb_begin = (int)crank * per; kb_end = min(a.k_blocks, kb_begin + per);
  }

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // (the whole warp walks the tiles so that the group lookup is a warp operation; lane 0 issues the copies)
    int stage = 0; uint32_t phase = 0;
    bool ok = true;
    for (int tile = tile0; tile < total_tiles && !a.test_no_loads; tile += tile_step) {
      // one decision for the whole warp (the lookup below uses warp-wide operations)
      if (!__shfl_sync(0xffffffffu, (ok && !s_err) ? 1 : 0, 0)) break;
      const TileCoord t = tc_tile_warp(a, tile, m_tiles, lane, tile_m, sub);
      if (lane == 0) {
        const CUtensorMap *mb = a.maps_b ? a.maps_b + t.g : &map_b0;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u)) { s_err = 1; report_status(a.status, 1); ok = false; break; }
          const uint32_t sa = smem0 + (uint32_t)stage * stage_bytes;
          if constexpr (PAIR) {
            // both CTAs' copies are counted on the leader's barrier; the leader expects the bytes of both
            const uint32_t lead_bar = cluster_map(full_bar(stage), 0);
            if (crank == 0) mbar_expect_tx(full_bar(stage), 2 * stage_bytes);
            tma_load_2d_pair(sa, &map_a, kb * kTcBK, t.row0, lead_bar);
            tma_load_wt_pair(sa + a_bytes, mb, kb, (t.nt * a.BN + (int)crank * (a.BN / 2)) >> 3, lead_bar);
          } else {
            mbar_expect_tx(full_bar(stage), stage_bytes);
            tma_load_2d(sa, &map_a, kb * kTcBK, t.row0, full_bar(stage));
            tma_load_wt(sa + a_bytes, mb, kb, (t.nt * a.BN) >> 3, full_bar(stage));
          }
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && (!PAIR || crank == 0)) {      // pair form: the leader issues for both CTAs
      const uint32_t idesc = F16 ? make_idesc_bf16(a.BN, tile_m) : make_idesc_i8(a.a_unsigned, a.BN, tile_m);
      int stage = 0; uint32_t phase = 0; int acc = 0; uint32_t acc_phase = 0;
      for (int tile = tile0; tile < total_tiles && !s_err; tile += tile_step) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u)) { s_err = 2; report_status(a.status, 2); break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * a.BN);
        bool ok = true;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(full_bar(stage), phase)) { ok = false; break; }
          if (kb == kb_begin && tile == tile0) TC_STAMP(2);
          tc_fence_after();
          const uint32_t sa = smem0 + (uint32_t)stage * stage_bytes;
          const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + a_bytes);
#pragma unroll
          for (int k = 0; k < kTcBK / 32; ++k) {
            const uint32_t accum = ((kb - kb_begin) | k) ? 1u : 0u;
            if constexpr (PAIR && F16) tc_mma_bf16_pair(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, accum);
            else if constexpr (PAIR) tc_mma_i8_pair(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, accum);
            else if constexpr (F16) tc_mma_bf16(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, accum);
            else tc_mma_i8(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, accum);
          }
          if constexpr (PAIR) tc_commit_pair(empty_bar(stage)); else tc_commit(empty_bar(stage));
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
        if (!ok) { s_err = 3; report_status(a.status, 3); break; }
        if constexpr (PAIR) tc_commit_pair(tfull_bar(acc)); else tc_commit(tfull_bar(acc));
        if (tile == tile0) TC_STAMP(3);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else if (warp == 2 + kTcEpiWarps) {
    // ------------------------------------------------------------------ operand warp
    const int32_t zp = load_zp(epi);
    int cb = 0; uint32_t cphase = 0;
    for (int tile = tile0; tile < total_tiles; tile += tile_step) {
      if (!__shfl_sync(0xffffffffu, s_err ? 0 : 1, 0)) break;
      const TileCoord t = tc_tile_warp(a, tile, m_tiles, lane, tile_m, sub);
      const void *wsp = epi.wei_scale; const int32_t *csp = epi.colsum; const void *bp = epi.bias;
      void *dst = epi.dst; int64_t ldc = epi.ldc; int m_dst0 = t.row0;
      if (a.groups) {
        const TcGroupDesc gd = a.groups[t.g];
        wsp = gd.wei_scale; csp = gd.colsum; bp = gd.bias;
        if (gd.dst) { dst = gd.dst; ldc = gd.ldc; m_dst0 = t.m_local0; }   // else: shared dst, global row index
      }
      const int pc_tile = t.nt * a.BN;
      float cw[8], cbv[8]; int32_t ck[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        cw[j] = 1.0f; cbv[j] = 0.0f; ck[j] = 0;
        const int pc = pc_tile + lane + 32 * j;
        if (lane + 32 * j < a.BN && pc < a.N) {
          const int n = (int)packed_to_logical(pc, a.gated, epi.gated_I);
          if (epi.wei_scale_n) cw[j] = load_as_f32(wsp, epi.wei_scale_dt, epi.wei_scale_n > 1 ? n : 0);
          if (bp) cbv[j] = load_as_f32(bp, epi.bias_dt, n);
          if (zp) ck[j] = zp * csp[pc];
        }
      }
      float rs[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = lane + 32 * j;
        rs[j] = (epi.src_scale_n && r < t.rows) ? load_as_f32(epi.src_scale, epi.src_scale_dt, epi.src_scale_n > 1 ? t.row0 + r : 0) : 1.0f;
      }
      // the buffer is free when the epilogue warps have left the tile that used it two tiles ago
      if (!__all_sync(0xffffffffu, mbar_wait(cempty_bar(cb), cphase ^ 1u))) { if (lane == 0) { s_err = 6; report_status(a.status, 6); } break; }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (lane + 32 * j < a.BN) { cols[cb].ws[lane + 32 * j] = cw[j]; cols[cb].bias[lane + 32 * j] = cbv[j]; cols[cb].comp[lane + 32 * j] = ck[j]; }
#pragma unroll
      for (int j = 0; j < 4; ++j) row_scale[cb][lane + 32 * j] = rs[j];
      if (lane == 0) {
        TileMeta m; m.row0 = t.row0; m.rows = t.rows; m.m_dst0 = m_dst0; m.nt = t.nt; m.dst = dst; m.ldc = ldc; m.has_bias = bp != nullptr;
        meta[cb] = m;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(cfull_bar(cb));
      if (++cb == 2) { cb = 0; cphase ^= 1u; }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    const int ew = warp - 2;                // 0..7
    const int q = warp & 3;                 // TMEM lane quadrant this warp may access
    const int part = ew >> 2;               // which share of the tile's columns this warp takes
    const int row_in_tile = q * 32 + lane;
    int acc = 0; uint32_t acc_phase = 0;
    int ob = 0; uint32_t ophase = 0;            // operand buffer of the current tile
    for (int tile = tile0; tile < total_tiles; tile += tile_step) {
      // everything from global memory was put into shared memory by the operand warp
      if (!mbar_wait(cfull_bar(ob), ophase)) { if (lane == 0) { s_err = 5; report_status(a.status, 5); } break; }
      const TileMeta tm = meta[ob];
      const TileCols &tcols = cols[ob];
      const bool row_ok = row_in_tile < tm.rows;
      const int m_global = tm.row0 + row_in_tile;
      const int m_dst = tm.m_dst0 + row_in_tile;
      EpiCtx cx;
      cx.wei_scale = nullptr; cx.colsum = nullptr; cx.bias = nullptr; cx.dst = tm.dst; cx.ldc = tm.ldc;
      cx.s_src = row_scale[ob][row_in_tile];
      const int pc_tile = tm.nt * a.BN;
      if (!mbar_wait(tfull_bar(acc), acc_phase)) { if (lane == 0) { s_err = 4; report_status(a.status, 4); } break; }
      if (warp == 2 && lane == 0 && tile == tile0) TC_STAMP(4);
      tc_fence_after();
      const bool has_bias = tm.has_bias != 0;
      EpiStore es;
      {
        const int esz = epi.dst_dt == DT_BF16 ? 2 : 4;
        es.sbuf = epi_stage[ew];
        es.pitch_bytes = tm.ldc * esz;
        es.g_row0 = reinterpret_cast<uint8_t *>(tm.dst) + (int64_t)(tm.m_dst0 + q * 32) * es.pitch_bytes;
        es.rows_valid = min(32, max(0, tm.rows - q * 32));
        es.coalesce = ((reinterpret_cast<uintptr_t>(tm.dst) | (uintptr_t)es.pitch_bytes) & 15) == 0;
        es.v8 = ((reinterpret_cast<uintptr_t>(tm.dst) | (uintptr_t)es.pitch_bytes) & 31) == 0;
        es.row_ok = row_ok;
        es.map_c = (a.tma_store && es.coalesce) ? &map_c : nullptr;
        es.row_c = tm.m_dst0 + q * 32;
      }
      const uint32_t taddr0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * a.BN);
      if constexpr (SPLIT) {
        // partial sums of this CTA's K blocks go to shared memory (the stage ring is free: every MMA that read it has
        // completed); [chunk][row][32 x int32], the eight 16-byte units of a row XOR-swizzled by the row
        const int nc = min(a.BN / 32, (a.N - pc_tile + 31) / 32);
        const int per = (a.BN / 32 + kTcEpiParts - 1) / kTcEpiParts;
        const int c_begin = part * per, c_end = min(nc, c_begin + per);
        for (int c = c_begin; c < c_end; ++c) {
          uint32_t r[32];
          if (kb_end > kb_begin) { tc_ld32(taddr0 + (uint32_t)(c * 32), r); tc_wait_ld(); }
          else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
          }
          const uint32_t base = smem0 + (uint32_t)((c * kTcBM + row_in_tile) * 128);
#pragma unroll
          for (int u = 0; u < 8; ++u)
            st_shared_v4(base + (uint32_t)((u ^ (row_in_tile & 7)) << 4), r[4 * u], r[4 * u + 1], r[4 * u + 2], r[4 * u + 3]);
        }
#ifdef B200DNN_TIMING_EXPERIMENTS
      } else if (a.dbg == 1) {
        // timing experiment: no epilogue work
#endif
      } else if (!a.gated) {
#ifdef B200DNN_TIMING_EXPERIMENTS
        if (a.dbg == 3) { es.coalesce = false; es.v8 = false; es.row_ok = false; es.map_c = nullptr; }
#endif
        // this warp's chunks: a contiguous share of the tile's 32-column chunks that lie inside N
        const int nc = min(a.BN / 32, (a.N - pc_tile + 31) / 32);
        const int per = (a.BN / 32 + kTcEpiParts - 1) / kTcEpiParts;
        const int c_begin = part * per, c_end = min(nc, c_begin + per);
        for (int c = c_begin; c < c_end; ++c) {
          uint32_t r[32];
          tc_ld32(taddr0 + (uint32_t)(c * 32), r);
          tc_wait_ld();
          const int pc0 = pc_tile + c * 32;
#ifdef B200DNN_TIMING_EXPERIMENTS
          if (a.dbg == 2) { uint32_t x = 0;
#pragma unroll
            for (int i = 0; i < 32; ++i) x ^= r[i];
            if (x == 0x12345678u) report_status(a.status, 99); continue; }
#endif
          tc_epi_dispatch<F16>(a.fast_act, epi, cx, r, tcols, c * 32, pc0, a.N, m_dst, has_bias, es, lane);
        }
      } else {
        // gated: packed columns [g(32) u(32)] -> 32 outputs; dst is [rows, I] bf16.  Sixteen outputs at a time: their
        // 32 bytes leave as one store of the lane's own row; the row maximum is taken on the bf16 bit patterns (two per
        // instruction; magnitudes order like integers, non-finite values do not count)
        uint32_t amax2 = 0u;
        for (int c = part; c < a.BN / 64; c += kTcEpiParts) {
          const int pc0 = pc_tile + c * 64;
          if (pc0 >= a.N) break;
          const int j0 = pc0 / 2;   // first output column of this pair of chunks
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t rg[16], ru[16];
            tc_ld16(taddr0 + (uint32_t)(c * 64 + 16 * h), rg);
            tc_ld16(taddr0 + (uint32_t)(c * 64 + 32 + 16 * h), ru);
            tc_wait_ld();
            const int cg = c * 64 + 16 * h, cu = cg + 32;
            uint32_t pk[8];
#pragma unroll
            for (int i = 0; i < 16; i += 4) {
              const float4 wg4 = *reinterpret_cast<const float4 *>(&tcols.ws[cg + i]);
              const float4 wu4 = *reinterpret_cast<const float4 *>(&tcols.ws[cu + i]);
              const float wg[4] = {wg4.x, wg4.y, wg4.z, wg4.w}, wu[4] = {wu4.x, wu4.y, wu4.z, wu4.w};
              float bg[4] = {0.f, 0.f, 0.f, 0.f}, bu[4] = {0.f, 0.f, 0.f, 0.f};
              if (has_bias) {
                const float4 bg4 = *reinterpret_cast<const float4 *>(&tcols.bias[cg + i]);
                const float4 bu4 = *reinterpret_cast<const float4 *>(&tcols.bias[cu + i]);
                bg[0] = bg4.x; bg[1] = bg4.y; bg[2] = bg4.z; bg[3] = bg4.w;
                bu[0] = bu4.x; bu[1] = bu4.y; bu[2] = bu4.z; bu[3] = bu4.w;
              }
              float z[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float gv = tc_acc_f32<F16>(rg[i + j], 0, cx.s_src, wg[j]);
                float uv = tc_acc_f32<F16>(ru[i + j], 0, cx.s_src, wu[j]);
                if (has_bias) { gv = __fadd_rn(gv, bg[j]); uv = __fadd_rn(uv, bu[j]); }
                if (epi.gated_act == ACT_SILU_MUL) z[j] = __fmul_rn(fast_sigmoid_mul(gv, gv), uv);
                else z[j] = gated_f32(epi.gated_act, gv, uv);
              }
              pk[i >> 1] = pack_bf16x2(z[0], z[1]);
              pk[(i >> 1) + 1] = pack_bf16x2(z[2], z[3]);
#pragma unroll
              for (int q2 = 0; q2 < 2; ++q2) {
                uint32_t mag = pk[(i >> 1) + q2] & 0x7FFF7FFFu;
                mag &= ~__vcmpgeu2(mag, 0x7F807F80u);          // infinities and NaNs do not enter the maximum
                amax2 = __vmaxu2(amax2, mag);
              }
            }
            const int jc = j0 + 16 * h;
            if (es.map_c && es.rows_valid == 32) {
              warp_tma_store_rows32(es.sbuf, make_uint4(pk[0], pk[1], pk[2], pk[3]), make_uint4(pk[4], pk[5], pk[6], pk[7]), es.map_c,
                                    jc * 2, es.row_c, lane);
            } else if (es.v8) {
              if (row_ok) st_global_v8(reinterpret_cast<uint8_t *>(cx.dst) + ((int64_t)m_dst * cx.ldc + jc) * 2, pk);
            } else if (es.coalesce) {
              warp_store_rows32(es.sbuf, make_uint4(pk[0], pk[1], pk[2], pk[3]), make_uint4(pk[4], pk[5], pk[6], pk[7]),
                                es.g_row0 + (size_t)jc * 2, es.pitch_bytes, es.rows_valid, lane);
            } else if (row_ok) {
              uint16_t *o = reinterpret_cast<uint16_t *>(cx.dst) + (int64_t)m_dst * cx.ldc + jc;
#pragma unroll
              for (int i = 0; i < 16; ++i) o[i] = (uint16_t)(pk[i >> 1] >> ((i & 1) * 16));
            }
          }
        }
        if (row_ok && epi.row_absmax) {
          const uint32_t m16 = max(amax2 & 0xFFFFu, amax2 >> 16);
          atomicMax(epi.row_absmax + m_global, m16 << 16);     // the bf16 magnitude as float bits
        }
      }
      if (warp == 2 && lane == 0 && tile == tile0) TC_STAMP(5);
      tc_fence_before();
      __syncwarp();
      // this warp is done with the accumulator and with the tile's operand buffer
      if (lane == 0) {
        if constexpr (PAIR) mbar_arrive_cluster(cluster_map(tempty_bar(acc), 0)); else mbar_arrive(tempty_bar(acc));
        mbar_arrive(cempty_bar(ob));
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      if (++ob == 2) { ob = 0; ophase ^= 1u; }
    }
  }

  if constexpr (SPLIT) {
    // ------------------------------------------------------------------ sum over the cluster, then the epilogue
    cluster_sync_all();   // every CTA's partial sums are in its shared memory
    bool arrived = false;
    if (threadIdx.x == 0) TC_STAMP(6);
    const bool healthy = __shfl_sync(0xffffffffu, s_err ? 0 : 1, 0) != 0;   // one decision per warp: the barriers below are warp-wide
    if (warp >= 2 && warp < 2 + kTcEpiWarps && healthy && tile0 < total_tiles) {
      const int ew = warp - 2, q = warp & 3, part = ew >> 2, row_in_tile = q * 32 + lane;
      const TileMeta tm = meta[0];
      const TileCols &tcols = cols[0];
      const int m_dst = tm.m_dst0 + row_in_tile;
      EpiCtx cx;
      cx.wei_scale = nullptr; cx.colsum = nullptr; cx.bias = nullptr; cx.dst = tm.dst; cx.ldc = tm.ldc;
      cx.s_src = row_scale[0][row_in_tile];
      const int pc_tile = tm.nt * a.BN;
      const bool has_bias = tm.has_bias != 0;
      EpiStore es;
      const int esz = epi.dst_dt == DT_BF16 ? 2 : 4;
      es.sbuf = epi_stage[ew];
      es.pitch_bytes = tm.ldc * esz;
      es.g_row0 = reinterpret_cast<uint8_t *>(tm.dst) + (int64_t)(tm.m_dst0 + q * 32) * es.pitch_bytes;
      es.rows_valid = min(32, max(0, tm.rows - q * 32));
      es.coalesce = ((reinterpret_cast<uintptr_t>(tm.dst) | (uintptr_t)es.pitch_bytes) & 15) == 0;
      es.v8 = ((reinterpret_cast<uintptr_t>(tm.dst) | (uintptr_t)es.pitch_bytes) & 31) == 0;
      es.row_ok = row_in_tile < tm.rows;
      es.map_c = (a.tma_store && es.coalesce) ? &map_c : nullptr;
      es.row_c = tm.m_dst0 + q * 32;
      const int nc = min(a.BN / 32, (a.N - pc_tile + 31) / 32);
      // chunk c is finished by CTA c % k_splits; its warp parts share that CTA's chunks.  First all sums: the warp's 32
      // rows of a chunk are 4 KiB in a row, added over the CTAs with whole-warp contiguous reads (remote shared memory is
      // slow when every lane asks for a different line) and written back in place (only this CTA reads its own copy of a
      // chunk it finishes).
      for (int c = (int)crank + a.k_splits * part; c < nc; c += a.k_splits * kTcEpiParts) {
        const uint32_t blk = smem0 + (uint32_t)((c * kTcBM + q * 32) * 128) + (uint32_t)(lane * 16);
        uint4 sum[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) sum[i] = ld_shared_v4(blk + (uint32_t)(i * 512));
        for (int j = 0; j < a.k_splits; ++j) {
          if (j == (int)crank) continue;
          const uint32_t rb = cluster_map(blk, (uint32_t)j);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint4 v = ld_cluster_v4(rb + (uint32_t)(i * 512));
            if constexpr (F16) {
              // f32 partial sums: added in a fixed order (own share first, then the other CTAs by rank), so a result is
              // reproducible; it is not the unsplit kernel's sum bit for bit
              sum[i].x = __float_as_uint(__fadd_rn(__uint_as_float(sum[i].x), __uint_as_float(v.x)));
              sum[i].y = __float_as_uint(__fadd_rn(__uint_as_float(sum[i].y), __uint_as_float(v.y)));
              sum[i].z = __float_as_uint(__fadd_rn(__uint_as_float(sum[i].z), __uint_as_float(v.z)));
              sum[i].w = __float_as_uint(__fadd_rn(__uint_as_float(sum[i].w), __uint_as_float(v.w)));
            } else { sum[i].x += v.x; sum[i].y += v.y; sum[i].z += v.z; sum[i].w += v.w; }
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) st_shared_v4(blk + (uint32_t)(i * 512), sum[i].x, sum[i].y, sum[i].z, sum[i].w);
      }
      cluster_arrive_all();   // this warp reads no neighbour any more
      arrived = true;
      for (int c = (int)crank + a.k_splits * part; c < nc; c += a.k_splits * kTcEpiParts) {
        uint32_t r[32];
        const uint32_t base = smem0 + (uint32_t)((c * kTcBM + row_in_tile) * 128);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const uint4 v = ld_shared_v4(base + (uint32_t)((u ^ (row_in_tile & 7)) << 4));
          r[4 * u] = v.x; r[4 * u + 1] = v.y; r[4 * u + 2] = v.z; r[4 * u + 3] = v.w;
        }
        tc_epi_dispatch<F16>(a.fast_act, epi, cx, r, tcols, c * 32, pc_tile + c * 32, a.N, m_dst, has_bias, es, lane);
      }
    }
    // nobody leaves while a neighbour may still read its shared memory: arrive as soon as the own reads are done,
    // wait at the very end
    if (!arrived) cluster_arrive_all();
  }

  // ---------------------------------------------------------------------- teardown
  if (a.tma_store && warp >= 2 && warp < 2 + kTcEpiWarps && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  if constexpr (SPLIT) cluster_wait_all();
  tc_fence_before();
  __syncthreads();
  // pair form: neither CTA frees its tensor memory or leaves while the partner may still issue into it or signal its barriers
  if constexpr (PAIR) cluster_sync_all();
  if (s_err) {
    // give copies that may still be in flight time to land before shared memory is released
    for (int i = 0; i < 64; ++i) __nanosleep(20000);
    __syncthreads();
  }
  if (threadIdx.x == 0) TC_STAMP(7);
  if (warp == 1) {
    tc_fence_after();
    if constexpr (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

}  // namespace b200
