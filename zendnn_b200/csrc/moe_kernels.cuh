// Memory-bound pieces of the fused MoE path around the grouped GEMMs:
//  - gated activation as a separate pass  (matmul/group_matmul/group_matmul_moe_act.cpp:88-196, 728)
//  - weighted top-k reduce over gathered rows (matmul/group_matmul/group_matmul_moe_postop.cpp:103-129, 216-283)
//  - router softmax / top-k / renormalise and the stable expert-sorted permutation.  The reference has no
//    such code (its callers prepare src[e] and row_ptrs themselves,
//    examples/lowoha_group_matmul_example.cpp:273-300); the specification is stated at route_topk_kernel.
#pragma once
#include "common.cuh"
#include "quant_kernels.cuh"

namespace b200 {

// ---- gated activation, in place on [M, N=2I] rows; one CTA per row --------------------------------
// Chunked so that the in-place element-interleaved form never overwrites a value before it is read:
// chunk c reads columns [2cB, 2(c+1)B) (or the two halves) and writes [cB, (c+1)B).
template <typename T>
__global__ void __launch_bounds__(256) gated_act_kernel(T *buf, int64_t N, int64_t ldc, int act) {
  T *row = buf + (int64_t)blockIdx.x * ldc;
  const int64_t I = N / 2;
  for (int64_t base = 0; base < I; base += blockDim.x) {
    const int64_t n = base + threadIdx.x;
    float g = 0.f, u = 0.f;
    if (n < I) {
      if (act == ACT_SWIGLU_OAI) { g = elem_to_f32<T>(row[2 * n]); u = elem_to_f32<T>(row[2 * n + 1]); }
      else { g = elem_to_f32<T>(row[n]); u = elem_to_f32<T>(row[I + n]); }
    }
    __syncthreads();
    if (n < I) {
      float r = gated_f32(act, g, u);
      if (sizeof(T) == 2) reinterpret_cast<uint16_t *>(row)[n] = f32_to_bf16_bits(r);
      else reinterpret_cast<float *>(row)[n] = r;
    }
    __syncthreads();
  }
}

// ---- weighted reduce ---------------------------------------------------------------------------------
// out[t,d] = sum_k w[t,k] * row(t,k)[d]; f32 accumulate in k order: multiply for k = 0, fused
// multiply-add afterwards (the association of the reference's vector form), RNE store.
// Rows come either from a device array of pointers (the reference's row_ptrs) or from
// base + slot_rows[t*nslots+k] * ld (the in-library un-permute).
struct ReduceArgs {
  const void *const *row_ptrs;
  const void *base; int64_t ld; const int32_t *slot_rows;
  // expert-parallel combine: slot (t,k)'s row lives in peer_base[slot_peer[slot]] (another GPU's output buffer mapped into
  // this process; the loads cross NVLink) instead of `base`
  const int32_t *slot_peer; const void *peer_base[8]; int32_t row_cap;   // rows at or beyond row_cap do not exist
  const float *w; int skip_weighted;
  int nslots, D, dt;
  void *out; int64_t ld_out;
};
__global__ void __launch_bounds__(256) moe_reduce_kernel(ReduceArgs a) {
  const int t = blockIdx.x;
  extern __shared__ uint8_t rsm[];
  const void **rows = reinterpret_cast<const void **>(rsm);
  float *ws = reinterpret_cast<float *>(rsm + sizeof(void *) * a.nslots);
  for (int k = threadIdx.x; k < a.nslots; k += blockDim.x) {
    const int64_t slot = (int64_t)t * a.nslots + k;
    const void *p;
    if (a.row_ptrs) p = a.row_ptrs[slot];
    else {
      const void *b = a.slot_peer ? a.peer_base[a.slot_peer[slot]] : a.base;
      int32_t row = a.slot_rows[slot];
      if (a.row_cap && (row < 0 || row >= a.row_cap)) row = 0;   // dropped by an overflowing receive buffer (reported separately)
      p = reinterpret_cast<const uint8_t *>(b) + (int64_t)row * a.ld * (a.dt == DT_BF16 ? 2 : 4);
    }
    rows[k] = p;
    ws[k] = a.skip_weighted ? 1.f : a.w[slot];
  }
  __syncthreads();
  if (a.dt == DT_BF16) {
    uint16_t *o = reinterpret_cast<uint16_t *>(a.out) + (int64_t)t * a.ld_out;
    bool vec = (a.D % 8 == 0) && ((reinterpret_cast<uintptr_t>(o) & 15) == 0);
    for (int k = 0; k < a.nslots; ++k) vec = vec && ((reinterpret_cast<uintptr_t>(rows[k]) & 15) == 0);
    if (vec) {
      for (int v = threadIdx.x; v < a.D / 8; v += blockDim.x) {
        float acc[8];
        for (int k = 0; k < a.nslots; ++k) {
          uint4 q = reinterpret_cast<const uint4 *>(rows[k])[v];
          const uint16_t *e = reinterpret_cast<const uint16_t *>(&q);
          const float wk = ws[k];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float x = bf16_bits_to_f32(e[i]);
            acc[i] = k == 0 ? __fmul_rn(wk, x) : __fmaf_rn(wk, x, acc[i]);
          }
        }
        uint16_t r[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) r[i] = f32_to_bf16_bits(a.nslots ? acc[i] : 0.f);
        reinterpret_cast<uint4 *>(o)[v] = *reinterpret_cast<uint4 *>(r);
      }
    } else {
      for (int d = threadIdx.x; d < a.D; d += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < a.nslots; ++k) {
          float x = bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(rows[k])[d]);
          acc = k == 0 ? __fmul_rn(ws[k], x) : __fmaf_rn(ws[k], x, acc);
        }
        o[d] = f32_to_bf16_bits(acc);
      }
    }
  } else {
    float *o = reinterpret_cast<float *>(a.out) + (int64_t)t * a.ld_out;
    for (int d = threadIdx.x; d < a.D; d += blockDim.x) {
      float acc = 0.f;
      for (int k = 0; k < a.nslots; ++k) {
        float x = reinterpret_cast<const float *>(rows[k])[d];
        acc = k == 0 ? __fmul_rn(ws[k], x) : __fmaf_rn(ws[k], x, acc);
      }
      o[d] = acc;
    }
  }
}

// ---- router ------------------------------------------------------------------------------------------
// Specification (no reference counterpart): p = softmax(logits[t,:]) in f32 (subtract the row max,
// expf, sum sequentially in expert order, divide); the k experts with the largest p, ties to the
// lower expert id, in descending order; weights renormalised by their sequential sum when renorm.
constexpr int kMaxTopk = 16;
__global__ void route_topk_kernel(const float *logits, int T, int E, int k, int renorm, int32_t *ids, float *w) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const float *l = logits + (int64_t)t * E;
  float mx = l[0];
  for (int e = 1; e < E; ++e) mx = fmaxf(mx, l[e]);
  float sum = 0.f;
  for (int e = 0; e < E; ++e) sum = __fadd_rn(sum, expf(__fadd_rn(l[e], -mx)));
  int chosen[kMaxTopk]; float pw[kMaxTopk];
  float tot = 0.f;
  for (int j = 0; j < k; ++j) {
    int best = -1; float bp = 0.f;
    for (int e = 0; e < E; ++e) {
      bool taken = false;
      for (int q = 0; q < j; ++q) taken |= chosen[q] == e;
      if (taken) continue;
      float p = __fdiv_rn(expf(__fadd_rn(l[e], -mx)), sum);
      if (best < 0 || p > bp) { best = e; bp = p; }
    }
    chosen[j] = best; pw[j] = bp; tot = __fadd_rn(tot, bp);
  }
  for (int j = 0; j < k; ++j) {
    ids[(int64_t)t * k + j] = chosen[j];
    if (w) w[(int64_t)t * k + j] = renorm ? __fdiv_rn(pw[j], tot) : pw[j];
  }
}

// Stable rank of every (token,k) slot inside its expert: one CTA per expert walks all slots in order.
__global__ void __launch_bounds__(1024) expert_rank_kernel(const int32_t *ids, int nslots, int32_t *rank, int32_t *counts) {
  __shared__ int warp_sums[32];
  __shared__ int running;
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if (threadIdx.x == 0) running = 0;
  __syncthreads();
  for (int base = 0; base < nslots; base += blockDim.x) {
    const int s = base + threadIdx.x;
    const bool mine = s < nslots && ids[s] == e;
    const unsigned bal = __ballot_sync(0xffffffffu, mine);
    if (lane == 0) warp_sums[warp] = __popc(bal);
    __syncthreads();
    int before = running;
    for (int i = 0; i < warp; ++i) before += warp_sums[i];
    if (mine) rank[s] = before + __popc(bal & ((1u << lane) - 1u));
    __syncthreads();
    if (threadIdx.x == 0) { int tot = 0; for (int i = 0; i < nwarps; ++i) tot += warp_sums[i]; running += tot; }
    __syncthreads();
  }
  if (threadIdx.x == 0) counts[e] = running;
}

// Warp-per-token form of route_topk_kernel for E <= 32*PER: every probability is computed once, the sum runs
// in expert order (lane e%32 holds expert e), the k selections are warp arg-max reductions with ties to the
// lower expert id.  Same results as route_topk_kernel bit for bit.
template <int PER>
__global__ void __launch_bounds__(256) route_topk_warp_kernel(const float *logits, int T, int E, int k, int renorm, int32_t *ids, float *w) {
  const int t = (int)((blockIdx.x * (unsigned)blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  const float *l = logits + (int64_t)t * E;
  const float ninf = __int_as_float(0xff800000);
  float v[PER], mx = ninf;
#pragma unroll
  for (int j = 0; j < PER; ++j) { const int e = j * 32 + lane; v[j] = e < E ? l[e] : ninf; mx = fmaxf(mx, v[j]); }
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
#pragma unroll
  for (int j = 0; j < PER; ++j) v[j] = (j * 32 + lane < E) ? expf(__fadd_rn(v[j], -mx)) : 0.f;
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    if (j * 32 < E) {
      const int n = min(32, E - j * 32);
      for (int src = 0; src < n; ++src) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, v[j], src));
    }
  }
#pragma unroll
  for (int j = 0; j < PER; ++j) v[j] = (j * 32 + lane < E) ? __fdiv_rn(v[j], sum) : -2.f;
  float my_p = 0.f, tot = 0.f; int my_id = 0;
  for (int jj = 0; jj < k; ++jj) {
    float bp = -3.f; int be = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < PER; ++j) if (v[j] > bp) { bp = v[j]; be = j * 32 + lane; }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float op = __shfl_xor_sync(0xffffffffu, bp, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (op > bp || (op == bp && oe < be)) { bp = op; be = oe; }
    }
#pragma unroll
    for (int j = 0; j < PER; ++j) if (be == j * 32 + lane) v[j] = -1.f;     // taken
    if (lane == jj) { my_p = bp; my_id = be; }
    tot = __fadd_rn(tot, bp);
  }
  if (lane < k) {
    ids[(int64_t)t * k + lane] = my_id;
    if (w) w[(int64_t)t * k + lane] = renorm ? __fdiv_rn(my_p, tot) : my_p;
  }
}

// Stable rank of every slot inside its key, in three passes over chunks of 1024 slots (keys <= kRankMaxKeys):
// per-chunk histograms, a scan over chunks per key, and the in-chunk stable rank.  Same output as expert_rank_kernel.
constexpr int kRankChunk = 1024;
constexpr int kRankMaxKeys = 256;
__global__ void __launch_bounds__(kRankChunk) rank_count_kernel(const int32_t *ids, int nslots, int nkeys, int32_t *chunk_counts) {
  __shared__ int hist[kRankMaxKeys];
  for (int i = threadIdx.x; i < nkeys; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  const int s = blockIdx.x * kRankChunk + threadIdx.x;
  if (s < nslots) { const int key = ids[s]; if ((unsigned)key < (unsigned)nkeys) atomicAdd(&hist[key], 1); }
  __syncthreads();
  for (int i = threadIdx.x; i < nkeys; i += blockDim.x) chunk_counts[(size_t)blockIdx.x * nkeys + i] = hist[i];
}
// one warp per key: exclusive scan of that key's counts over the chunks (in place), total to counts[key]
__global__ void __launch_bounds__(256) rank_scan_kernel(int32_t *chunk_counts, int nchunks, int nkeys, int32_t *counts) {
  const int key = (int)((blockIdx.x * (unsigned)blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
  if (key >= nkeys) return;
  int running = 0;
  for (int base = 0; base < nchunks; base += 32) {
    const int c = base + lane;
    const int v = c < nchunks ? chunk_counts[(size_t)c * nkeys + key] : 0;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int n = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += n; }
    if (c < nchunks) chunk_counts[(size_t)c * nkeys + key] = running + incl - v;
    running += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) counts[key] = running;
}
__global__ void __launch_bounds__(kRankChunk) rank_assign_kernel(const int32_t *ids, int nslots, int nkeys, const int32_t *chunk_base,
                                                                 int32_t *rank) {
  extern __shared__ int wcnt[];     // [32 warps][nkeys]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 32 * nkeys; i += blockDim.x) wcnt[i] = 0;
  __syncthreads();
  const int s = blockIdx.x * kRankChunk + threadIdx.x;
  int key = s < nslots ? ids[s] : -1;
  if ((unsigned)key >= (unsigned)nkeys) key = -1;
  const unsigned same = __match_any_sync(0xffffffffu, key);
  const int in_warp = __popc(same & ((1u << lane) - 1u));
  if (key >= 0 && in_warp == 0) wcnt[warp * nkeys + key] = __popc(same);
  __syncthreads();
  if (key >= 0) {
    int before = chunk_base[(size_t)blockIdx.x * nkeys + key];
    for (int i = 0; i < warp; ++i) before += wcnt[i * nkeys + key];
    rank[s] = before + in_warp;
  }
}

// Device-side expert offsets, one warp: counts[0..E) are the routed experts' rows; shared experts (if any) get T rows each.
// Writes row_off[E+S+1] and, when tile_prefix is given, the running number of row tiles (tile_rows rows each) per group,
// tile_prefix[E+S+1], which the grouped GEMM reads.
__global__ void expert_offsets_kernel(const int32_t *counts, int E, int S, int T, int32_t *row_off, int32_t *tile_prefix = nullptr,
                                      int tile_rows = 1) {
  if (blockIdx.x != 0 || threadIdx.x >= 32) return;
  const int lane = threadIdx.x, G = E + S;
  int row_carry = 0, tile_carry = 0;
  for (int base = 0; base < G; base += 32) {
    const int g = base + lane;
    const int rows = g < E ? counts[g] : (g < G ? T : 0);
    const int tiles = (rows + tile_rows - 1) / tile_rows;
    int rsum = rows, tsum = tiles;       // inclusive scans over the warp
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int r = __shfl_up_sync(0xffffffffu, rsum, o), t = __shfl_up_sync(0xffffffffu, tsum, o);
      if (lane >= o) { rsum += r; tsum += t; }
    }
    if (g < G) {
      row_off[g] = row_carry + rsum - rows;
      if (tile_prefix) tile_prefix[g] = tile_carry + tsum - tiles;
    }
    row_carry += __shfl_sync(0xffffffffu, rsum, 31);
    tile_carry += __shfl_sync(0xffffffffu, tsum, 31);
  }
  if (lane == 0) { row_off[G] = row_carry; if (tile_prefix) tile_prefix[G] = tile_carry; }
}

// slot -> row (expert-sorted order) and row -> source token; shared-expert rows follow the routed ones.
// slot_rows is [T][k+S]; slot_w is [T][k+S] (shared slots get weight 1).
__global__ void build_maps_kernel(const int32_t *ids, const int32_t *rank, const float *w, const int32_t *row_off,
                                  int T, int k, int E, int S, int32_t *slot_rows, float *slot_w, int32_t *row_token) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int ns = k + S;
  if (i >= T * ns) return;
  const int t = i / ns, j = i - t * ns;
  int row; float wt;
  if (j < k) { const int s = t * k + j; row = row_off[ids[s]] + rank[s]; wt = w[s]; }
  else { row = row_off[E + (j - k)] + t; wt = 1.0f; }
  slot_rows[i] = row; slot_w[i] = wt; row_token[row] = t;
}

}  // namespace b200
