// Weight prepack: the B200 counterpart of the reference's weight reorder
// (reorder/prepack/lowoha_prepack.cpp:173-252, matmul/backends/aocl/aocl_kernel.cpp:310-494) and
// of its zero-point compensation pass (matmul/lru_cache/lowoha_cache.hpp:65-133).
//
// Packed form, all in one caller- or cache-owned buffer:
//   [0,256)                 PackHeader
//   [256, 256+4*Np)         int32 colsum[Np]: sum over K of each packed weight row
//   [256+4*Np, ...)         int8  Wt: the weight transposed (K contiguous inside a row), K zero-padded
//                           to Kp = roundup(K,128), rows zero-padded to Np = roundup(N,128), rows
//                           interleaved eight at a time in 128-byte pieces: Wt[Np/8][Kp/128][8][128]
//                           (see wt_offset).
// The tcgen05 kernel loads [BN rows x 128 B] boxes with a 4-D tensor map and SWIZZLE_128B (in
// shared memory they are ordinary K-major rows); the streaming kernels read the 1 KiB blocks with
// 16-byte loads, eight rows per warp instruction, contiguously.
//
// Gated form (first GEMM of the fused MoE, N = 2*I with caller columns [gate(0:I) | up(I:2I)]):
// packed row order is [g(0:32) u(0:32) g(32:64) u(32:64) ...] so that one accumulator tile holds
// the (gate, up) pair of every output column it produces.  The reference interleaves for the same
// reason (matmul/group_matmul/custom_kernel/pack.hpp:217-258).  For swiglu_oai_mul the caller
// layout is already interleaved by element ([g0,u0,g1,u1,...]); it is mapped to the same packed
// order (gated == 2).
#pragma once
#include "common.cuh"

namespace b200 {

constexpr uint32_t kPackMagic = 0x38573242u;  // "B2W8"
constexpr int kPackHeaderBytes = 256;
constexpr int kGateGranule = 32;

struct PackHeader {
  uint32_t magic, version;
  int64_t K, N, Kp, Np;
  int32_t gated;  // 0 plain, 1 split halves [gate|up], 2 element-interleaved pairs
  int32_t I;
};

__host__ __device__ inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }
inline size_t pack_bytes(int64_t K, int64_t N) {
  int64_t Kp = round_up(K, 128), Np = round_up(N, 128);
  return (size_t)kPackHeaderBytes + (size_t)Np * 4 + (size_t)Np * Kp;
}

// caller column of packed row pn
__host__ __device__ __forceinline__ int64_t packed_to_logical(int64_t pn, int gated, int64_t I) {
  if (!gated) return pn;
  int64_t blk = pn / (2 * kGateGranule), r = pn % (2 * kGateGranule);
  int64_t j = blk * kGateGranule + (r % kGateGranule);   // output column
  bool up = r >= kGateGranule;
  if (gated == 1) return up ? I + j : j;
  return 2 * j + (up ? 1 : 0);
}

// Byte offset of element (packed row pn, k) inside Wt.  Rows are interleaved in groups of eight
// at 128-byte granularity: Wt[pn/8][k/128][pn%8][k%128].  One group of eight rows is then one
// contiguous span of 8*Kp bytes, made of 1 KiB blocks that hold 128 bytes of K for each of the
// eight rows.  A warp of the streaming kernels (which needs eight rows at a time for its MMA
// fragments) walks memory contiguously, and a TMA box of BN rows x 128 B is BN/8 contiguous
// 1 KiB blocks that land in shared memory as plain [BN rows][128 B].
__host__ __device__ __forceinline__ size_t wt_offset(int64_t pn, int64_t k, int64_t Kp) {
  return (size_t)(pn >> 3) * (size_t)Kp * 8 + (size_t)(k >> 7) * 1024 + (size_t)(pn & 7) * 128 + (size_t)(k & 127);
}

// grid: (Kp/64, Np/32); block 256.  Each CTA moves a [64 k][32 n] tile through shared memory.
static __global__ void __launch_bounds__(256) pack_weight_kernel(const int8_t *W, int64_t ldb, int transB, int64_t K, int64_t N,
                                                          int64_t Kp, int gated, int64_t I, int8_t *Wt) {
  __shared__ int8_t tile[32][64 + 4];
  const int64_t k0 = (int64_t)blockIdx.x * 64, pn0 = (int64_t)blockIdx.y * 32;
  // 32 consecutive packed rows map to 32 consecutive caller columns (stride 1, or 2 when gated == 2)
  const int64_t n0 = packed_to_logical(pn0, gated, I);
  const int64_t nstep = gated == 2 ? 2 : 1;
  const int tid = threadIdx.x;
  if (!transB) {
    // W[k][n]: read 32 n per k (coalesced along n)
    for (int i = tid; i < 64 * 32; i += 256) {
      int kk = i >> 5, nn = i & 31;
      int64_t k = k0 + kk, n = n0 + nn * nstep;
      tile[nn][kk] = (k < K && pn0 + nn < N) ? W[k * ldb + n] : (int8_t)0;
    }
  } else {
    // W[n][k]: read 64 k per n (coalesced along k)
    for (int i = tid; i < 64 * 32; i += 256) {
      int nn = i >> 6, kk = i & 63;
      int64_t k = k0 + kk, n = n0 + nn * nstep;
      tile[nn][kk] = (k < K && pn0 + nn < N) ? W[n * ldb + k] : (int8_t)0;
    }
  }
  __syncthreads();
  for (int i = tid; i < 32 * 16; i += 256) {
    int nn = i >> 4, k4 = i & 15;
    const int8_t *t = &tile[nn][k4 * 4];
    uint32_t v = (uint32_t)(uint8_t)t[0] | ((uint32_t)(uint8_t)t[1] << 8) | ((uint32_t)(uint8_t)t[2] << 16) |
                 ((uint32_t)(uint8_t)t[3] << 24);
    *reinterpret_cast<uint32_t *>(Wt + wt_offset(pn0 + nn, k0 + k4 * 4, Kp)) = v;
  }
}

// bf16 weight into the same byte layout (a packed row holds 2*K bytes of K, zero-padded to Kp bytes): the tcgen05
// kernel's bf16 form reads the same [BN rows x 128 B] boxes, 64 elements of K each.
// grid: (Kp/128, Np/32); block 256.  Each CTA moves a [64 k][32 n] tile of 2-byte elements through shared memory.
static __device__ __forceinline__ void pack_weight_bf16_tile(const uint16_t *W, int64_t ldb, int transB, int64_t K, int64_t N,
                                                             int64_t Kp, int gated, int64_t I, uint8_t *Wt) {
  __shared__ uint16_t tile[32][64 + 2];
  const int64_t k0 = (int64_t)blockIdx.x * 64, pn0 = (int64_t)blockIdx.y * 32;
  const int64_t n0 = packed_to_logical(pn0, gated, I);
  const int64_t nstep = gated == 2 ? 2 : 1;
  const int tid = threadIdx.x;
  if (!transB) {
    for (int i = tid; i < 64 * 32; i += 256) {
      int kk = i >> 5, nn = i & 31;
      int64_t k = k0 + kk, n = n0 + nn * nstep;
      tile[nn][kk] = (k < K && pn0 + nn < N) ? W[k * ldb + n] : (uint16_t)0;
    }
  } else {
    for (int i = tid; i < 64 * 32; i += 256) {
      int nn = i >> 6, kk = i & 63;
      int64_t k = k0 + kk, n = n0 + nn * nstep;
      tile[nn][kk] = (k < K && pn0 + nn < N) ? W[n * ldb + k] : (uint16_t)0;
    }
  }
  __syncthreads();
  for (int i = tid; i < 32 * 32; i += 256) {
    int nn = i >> 5, k2 = i & 31;
    const uint32_t v = (uint32_t)tile[nn][2 * k2] | ((uint32_t)tile[nn][2 * k2 + 1] << 16);
    *reinterpret_cast<uint32_t *>(Wt + wt_offset(pn0 + nn, (k0 + 2 * k2) * 2, Kp)) = v;
  }
}

static __global__ void __launch_bounds__(256) pack_weight_bf16_kernel(const uint16_t *W, int64_t ldb, int transB, int64_t K, int64_t N,
                                                               int64_t Kp, int gated, int64_t I, uint8_t *Wt) {
  pack_weight_bf16_tile(W, ldb, transB, K, N, Kp, gated, I, Wt);
}
// many matrices of one shape in one launch (the K or V blocks of attention heads): matrix z = (b, h) starts at
// W + b * stride_b + h * stride_h and is packed to Wt + z * pack_stride.  grid: (Kp/128, Np/32, matrices)
static __global__ void __launch_bounds__(256) pack_weight_bf16_batched_kernel(const uint16_t *W, int64_t stride_b, int64_t stride_h, int heads,
                                                                       int first, int64_t ldb, int transB, int64_t K, int64_t N,
                                                                       int64_t Kp, uint8_t *Wt, size_t pack_stride) {
  const int z = first + (int)blockIdx.z;
  pack_weight_bf16_tile(W + (int64_t)(z / heads) * stride_b + (int64_t)(z % heads) * stride_h, ldb, transB, K, N, Kp, 0, 0,
                        Wt + (size_t)blockIdx.z * pack_stride);
}

// one warp per packed row
static __global__ void __launch_bounds__(256) pack_colsum_kernel(const int8_t *Wt, int64_t Np, int64_t Kp, int32_t *colsum) {
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= Np) return;
  const int lane = threadIdx.x & 31;
  int s = 0;
  for (int64_t i = lane; i < Kp / 16; i += 32) {
    const uint4 v = *reinterpret_cast<const uint4 *>(Wt + wt_offset(row, i * 16, Kp));
    s = __dp4a((int)v.x, 0x01010101, s); s = __dp4a((int)v.y, 0x01010101, s);
    s = __dp4a((int)v.z, 0x01010101, s); s = __dp4a((int)v.w, 0x01010101, s);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) colsum[row] = s;
}

// block of kPackHeaderBytes/4 threads: the bytes of the header block that carry no field are written as zero, so that a
// packed buffer is a function of the weight alone
static __global__ void pack_header_kernel(PackHeader *h, int64_t K, int64_t N, int64_t Kp, int64_t Np, int gated, int64_t I) {
  reinterpret_cast<uint32_t *>(h)[threadIdx.x] = 0u;
  __syncthreads();
  if (threadIdx.x != 0) return;
  h->magic = kPackMagic; h->version = 1; h->K = K; h->N = N; h->Kp = Kp; h->Np = Np; h->gated = gated; h->I = (int32_t)I;
}

}  // namespace b200
