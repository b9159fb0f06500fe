// libb200dnn: extern "C" entry points (include/b200dnn.h) over the sm_100a kernels.
// Validation mirrors the INT8 rules of the reference's validator
// (matmul/lowoha_matmul_utils.cpp:180-420) for the supported subset; everything else returns
// unimplemented, never a different computation.
#include <cudaTypedefs.h>
#include <algorithm>
#include <chrono>

#include "runtime.cuh"
#include "common.cuh"
#include "matmul_validate.cuh"
#include "quant_kernels.cuh"
#include "pack_kernels.cuh"
#include "stream_gemm.cuh"
#include "decode_gemm.cuh"
#include "decode_ring.cuh"
#include "tc_gemm.cuh"
#include "moe_kernels.cuh"

using namespace b200;

namespace {

cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

// Tuning and test knobs.  The environment is read once per knob (a lookup walks the whole environment, a microsecond
// per call on a box with a few hundred variables, and a call asks for several); with B200DNN_ENV_DYNAMIC=1, which the
// tests set, every call reads it afresh.  name must be a string literal (the cache is keyed by its address).
int env_int(const char *name, int dflt) {
  static const bool dynamic = [] { const char *e = getenv("B200DNN_ENV_DYNAMIC"); return e && atoi(e) != 0; }();
  if (dynamic) { const char *e = getenv(name); return e ? atoi(e) : dflt; }
  struct Slot { const char *name; bool set; int value; };
  static Slot slots[64];
  static int n_slots = 0;
  static std::mutex mu;
  std::lock_guard<std::mutex> lk(mu);
  for (int i = 0; i < n_slots; ++i)
    if (slots[i].name == name) return slots[i].set ? slots[i].value : dflt;
  const char *e = getenv(name);
  if (n_slots < 64) { slots[n_slots].name = name; slots[n_slots].set = e != nullptr; slots[n_slots].value = e ? atoi(e) : 0; ++n_slots; }
  return e ? atoi(e) : dflt;
}

// ------------------------------------------------------------------------------------ prepack
int32_t pack_into(const void *w_dev, int64_t K, int64_t N, int64_t ldb, int transB, int gated, void *dst_dev,
                  cudaStream_t st, PackedWeight *out) {
  const int64_t Kp = round_up(K, 128), Np = round_up(N, 128);
  const int64_t I = gated ? N / 2 : 0;
  if (gated) B2_CHECK(N % 2 == 0 && I % kGateGranule == 0, B200DNN_UNIMPLEMENTED,
                      "gated prepack needs N = 2*I with I a multiple of %d (N=%lld)", kGateGranule, (long long)N);
  uint8_t *base = reinterpret_cast<uint8_t *>(dst_dev);
  B2_CHECK((reinterpret_cast<uintptr_t>(base) & 255) == 0, B200DNN_FAILURE, "prepack destination must be 256-byte aligned");
  int32_t *colsum = reinterpret_cast<int32_t *>(base + kPackHeaderBytes);
  int8_t *wt = reinterpret_cast<int8_t *>(base + kPackHeaderBytes + Np * 4);
  pack_header_kernel<<<1, kPackHeaderBytes / 4, 0, st>>>(reinterpret_cast<PackHeader *>(base), K, N, Kp, Np, gated, I);
  B2_LAUNCHED();
  dim3 grid((unsigned)(Kp / 64), (unsigned)(Np / 32));
  pack_weight_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const int8_t *>(w_dev), ldb, transB, K, N, Kp, gated, I, wt);
  B2_LAUNCHED();
  pack_colsum_kernel<<<(unsigned)((Np + 7) / 8), 256, 0, st>>>(wt, Np, Kp, colsum);
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  if (out) { out->colsum = colsum; out->wt = wt; out->K = K; out->N = N; out->Kp = Kp; out->Np = Np; out->gated = gated; out->I = I; }
  return B200DNN_SUCCESS;
}

PackedWeight view_of(const void *dev_base, const PackHeader &h) {
  PackedWeight pw;
  const uint8_t *b = reinterpret_cast<const uint8_t *>(dev_base);
  pw.colsum = reinterpret_cast<const int32_t *>(b + kPackHeaderBytes);
  pw.wt = reinterpret_cast<const int8_t *>(b + kPackHeaderBytes + h.Np * 4);
  pw.K = h.K; pw.N = h.N; pw.Kp = h.Kp; pw.Np = h.Np; pw.gated = h.gated; pw.I = h.I;
  return pw;
}

// A cache-owned packed weight was written on the stream of the call that first saw it: a call on another stream waits
// for that work (until it has been seen complete once).  Callers hold the cache mutex.
int32_t wait_ready(PackedWeight &pw, cudaStream_t st) {
  if (pw.complete || !pw.ready || st == pw.ready_stream) return B200DNN_SUCCESS;
  {
    RelaxedCapture relaxed;      // an event query is not a capturable call: allowed while this thread captures a graph
    if (cudaEventQuery(pw.ready) == cudaSuccess) { pw.complete = true; return B200DNN_SUCCESS; }
  }
  cudaGetLastError();
  B2_CUDA(cudaStreamWaitEvent(st, pw.ready, 0));
  return B200DNN_SUCCESS;
}
int32_t mark_ready(PackedWeight &pw, cudaStream_t st) {
  B2_CUDA(cudaEventCreateWithFlags(&pw.ready, cudaEventDisableTiming));
  B2_CUDA(cudaEventRecord(pw.ready, st));
  pw.ready_stream = st; pw.complete = false;
  return B200DNN_SUCCESS;
}

// Resolves the weight argument of a GEMM to a packed device buffer.  The caches belong to the device and are shared
// by all streams; the mutex is held while a new weight is packed (once per weight).
int32_t resolve_weight(const void *weight, int wei_format, int64_t K, int64_t N, int64_t ldb, int transB, int gated,
                       int weights_const, cudaStream_t st, PackedWeight *pw) {
  DeviceShared &D = *rt().shared;
  if (wei_format == 'r') {
    std::lock_guard<std::mutex> lk(D.cache_mu);
    if (is_device_ptr(weight)) {
      auto it = D.packed_registry.find(weight);
      if (it == D.packed_registry.end()) {
        PackHeader h;
        B2_CUDA(cudaMemcpyAsync(&h, weight, sizeof h, cudaMemcpyDeviceToHost, st));
        B2_CUDA(cudaStreamSynchronize(st));
        B2_CHECK(h.magic == kPackMagic, B200DNN_FAILURE, "mem_format_b='r' but the weight buffer was not written by b200dnn_prepack");
        it = D.packed_registry.emplace(weight, view_of(weight, h)).first;
      }
      *pw = it->second;
    } else {
      auto it = D.host_packed.find(weight);
      if (it == D.host_packed.end()) {
        PackHeader h; memcpy(&h, weight, sizeof h);
        B2_CHECK(h.magic == kPackMagic, B200DNN_FAILURE, "mem_format_b='r' but the weight buffer was not written by b200dnn_prepack");
        size_t bytes = pack_bytes(h.K, h.N);
        void *d = nullptr;
        B2_CUDA(cudaMalloc(&d, bytes));
        B2_CUDA(cudaMemcpyAsync(d, weight, bytes, cudaMemcpyHostToDevice, st));
        PackedWeight v = view_of(d, h); v.owned = d;
        B2_TRY(mark_ready(v, st));
        it = D.host_packed.emplace(weight, v).first;
      }
      B2_TRY(wait_ready(it->second, st));
      *pw = it->second;
    }
    B2_CHECK(pw->K == K && pw->N == N && pw->gated == gated, B200DNN_FAILURE,
             "prepacked weight is K=%lld N=%lld gated=%d, call asks for K=%lld N=%lld gated=%d", (long long)pw->K,
             (long long)pw->N, pw->gated, (long long)K, (long long)N, gated);
    return B200DNN_SUCCESS;
  }
  B2_CHECK(wei_format == 'n' || wei_format == 0, B200DNN_FAILURE, "mem_format_b must be 'n' or 'r'");
  auto key = std::make_tuple(weight, K, N, ldb, transB, gated);
  const bool cache = weights_const && env_int("ZENDNNL_MATMUL_WEIGHT_CACHE", 1) != 0;
  std::unique_lock<std::mutex> lk(D.cache_mu, std::defer_lock);
  if (cache) {
    lk.lock();
    auto it = D.wcache.find(key);
    if (it != D.wcache.end()) { B2_TRY(wait_ready(it->second, st)); *pw = it->second; return B200DNN_SUCCESS; }
  }
  const int64_t wrows = transB ? N : K, wcols = transB ? K : N;
  const void *w_dev = nullptr;
  B2_TRY(stage_in(weight, span_bytes(wrows, wcols, ldb, B200DNN_S8), st, &w_dev));
  void *buf = nullptr;
  if (cache) B2_CUDA(cudaMalloc(&buf, pack_bytes(K, N)));
  else { buf = rt().ws.alloc(pack_bytes(K, N)); B2_CHECK(buf, B200DNN_FAILURE, "workspace allocation failed"); }
  B2_TRY(pack_into(w_dev, K, N, ldb, transB, gated, buf, st, pw));
  if (cache) { pw->owned = buf; B2_TRY(mark_ready(*pw, st)); D.wcache.emplace(key, *pw); }
  return B200DNN_SUCCESS;
}

// ------------------------------------------------------------------------------------ quant helpers
template <bool EP>
int32_t launch_quant_rows_t(const RowQuantArgs &a, int32_t src_dt, int64_t rows, cudaStream_t st) {
  if (rows <= 0) return B200DNN_SUCCESS;
  // short, aligned, non-grouped rows: one warp per row
  const int E = src_dt == B200DNN_BF16 ? 8 : 4;
  const bool aligned = a.n_groups == 0 && a.K % E == 0 && (reinterpret_cast<uintptr_t>(a.src) & 15) == 0 &&
                       (a.src_ld * (src_dt == B200DNN_BF16 ? 2 : 4)) % 16 == 0 &&
                       (!a.dst || ((reinterpret_cast<uintptr_t>(a.dst) % E) == 0 && a.dst_ld % E == 0));
  // rows whose abs-max is known: the streaming form (B200DNN_QUANT_STREAM=0 keeps the row-per-CTA kernel)
  if (aligned && a.absmax_bits && !a.gather && !a.scatter && rows >= 64 && a.K / E >= 64 &&
      (src_dt == B200DNN_BF16 || src_dt == B200DNN_F32) && env_int("B200DNN_QUANT_STREAM", 1) != 0) {
    // five CTAs of eight warps per SM are resident; rows are cut into segments (multiples of 128 vectors: four loads per
    // lane) until every warp has several items, so the last wave is short
    const int nvec = a.K / E;
    const long long warps = (long long)rt().sm_count * 5 * 8;
    int segs = 1;
    while (segs < 8 && rows * segs < 4 * warps && (nvec + segs) / (segs + 1) >= 128) ++segs;
    const int seg_len = (((nvec + segs - 1) / segs) + 31) & ~31;
    segs = (nvec + seg_len - 1) / seg_len;
    long long want = (rows * segs + 7) / 8;
    const unsigned grid = (unsigned)(want < rt().sm_count * 5 ? want : rt().sm_count * 5);
    // (eight loads in flight per lane measured slower: 110 against 92 us at configuration 4)
    if (src_dt == B200DNN_BF16) quant_known_absmax_kernel<uint16_t, 4><<<grid, 256, 0, st>>>(a, (int)rows, segs, seg_len);
    else quant_known_absmax_kernel<float, 4><<<grid, 256, 0, st>>>(a, (int)rows, segs, seg_len);
    B2_LAUNCHED();
    B2_CUDA(cudaGetLastError());
    return B200DNN_SUCCESS;
  }
  if (aligned && rows >= 64 && a.K / E <= 32 * 8 && (src_dt == B200DNN_BF16 || src_dt == B200DNN_F32)) {
    const int nv = (a.K / E + 31) / 32;
    unsigned grid = (unsigned)((rows + 7) / 8);
    if (EP && a.n_rows_dev && grid > (unsigned)(rt().sm_count * 16)) grid = (unsigned)(rt().sm_count * 16);   // the warps stride over the rows
#define B2_QW(T, NV) quant_per_token_warp_kernel<T, NV, EP><<<grid, 256, 0, st>>>(a, (int)rows)
    if (src_dt == B200DNN_BF16) { if (nv <= 2) B2_QW(uint16_t, 2); else if (nv <= 4) B2_QW(uint16_t, 4); else if (nv <= 8) B2_QW(uint16_t, 8); else B2_QW(uint16_t, 16); }
    else { if (nv <= 2) B2_QW(float, 2); else if (nv <= 4) B2_QW(float, 4); else if (nv <= 8) B2_QW(float, 8); else B2_QW(float, 16); }
#undef B2_QW
    B2_LAUNCHED();
    B2_CUDA(cudaGetLastError());
    return B200DNN_SUCCESS;
  }
  const bool short_row = a.K / E <= 2 * kQuantThreads;     // the whole row fits two cached vectors per thread
  unsigned grid_rows = (unsigned)rows;
  if (EP && a.n_rows_dev && grid_rows > (unsigned)(rt().sm_count * 32)) grid_rows = (unsigned)(rt().sm_count * 32);   // the CTAs stride over the rows
  if (src_dt == B200DNN_BF16) {
    if (short_row) quant_per_token_kernel<uint16_t, 2, EP><<<grid_rows, kQuantThreads, 0, st>>>(a);
    else quant_per_token_kernel<uint16_t, kQuantRegVec, EP><<<grid_rows, kQuantThreads, 0, st>>>(a);
  } else if (src_dt == B200DNN_F32) {
    if (short_row) quant_per_token_kernel<float, 2, EP><<<grid_rows, kQuantThreads, 0, st>>>(a);
    else quant_per_token_kernel<float, kQuantRegVec, EP><<<grid_rows, kQuantThreads, 0, st>>>(a);
  } else return fail(B200DNN_UNIMPLEMENTED, "per-token quantisation takes f32 or bf16 input");
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  return B200DNN_SUCCESS;
}
int32_t launch_quant_rows(const RowQuantArgs &a, int32_t src_dt, int64_t rows, cudaStream_t st) {
  if (a.n_rows_dev || a.scatter_peer) return launch_quant_rows_t<true>(a, src_dt, rows, st);
  return launch_quant_rows_t<false>(a, src_dt, rows, st);
}

// ------------------------------------------------------------------------------------ GEMM launchers
// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per kernel and device: raises the limit to the largest size
// the kernel is launched with and remembers that it did.
int32_t ensure_max_smem(const void *fn, int bytes = 227 * 1024) {
  DeviceShared &D = *rt().shared;
  std::lock_guard<std::mutex> lk(D.attr_mu);
  int &have = D.smem_limit[fn];
  if (have < bytes) {
    B2_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    have = bytes;
  }
  return B200DNN_SUCCESS;
}

int32_t launch_stream(const uint8_t *A, int64_t lda, bool a_unsigned, int M, int N, int K, const PackedWeight &pw,
                      const EpiParams &epi, cudaStream_t st) {
  Runtime &R = rt();
  StreamGemmArgs g{};
  g.A = A; g.lda = lda; g.M = M; g.N = N; g.K = K; g.Wt = pw.wt; g.Kp = (int)pw.Kp;
  g.chunks_total = (int)(pw.Kp / 64);
  // shape heuristic: enough CTAs to cover the SMs about twice, K range per CTA >= 1024 bytes
  int nb = env_int("B200DNN_STREAM_NB", 4);
  if (nb != 1 && nb != 2 && nb != 4 && nb != 8) nb = 4;
  g.nb = nb; g.kw = 8 / nb;
  const int tiles_n = (N + nb * 8 - 1) / (nb * 8);
  const int tiles_m = (M + 15) / 16;
  int ksplit = env_int("B200DNN_STREAM_KSPLIT", 0);
  if (ksplit <= 0) {
    ksplit = 1;
    while (tiles_n * tiles_m * ksplit < 2 * R.sm_count && g.chunks_total / (ksplit * 2) >= 16) ksplit *= 2;
  }
  if (ksplit > g.chunks_total) ksplit = g.chunks_total;
  g.chunks_per_cta = (g.chunks_total + ksplit - 1) / ksplit;
  ksplit = (g.chunks_total + g.chunks_per_cta - 1) / g.chunks_per_cta;
  const int kbytes = g.chunks_per_cta * 64;
  g.a_stride = (int)round_up(kbytes, 128) + 64;
  size_t smem = (size_t)16 * g.a_stride;
  if (smem < 4096) smem = 4096;
  B2_CHECK(smem <= 200 * 1024, B200DNN_FAILURE, "streaming kernel: K range per CTA too large (%d bytes)", kbytes);
  const size_t tiles = (size_t)tiles_n * tiles_m;
  if (ksplit > 1) {
    B2_CHECK(tiles <= R.n_counters, B200DNN_FAILURE, "streaming kernel: too many tiles for the split-K counters");
    g.partial = (int32_t *)R.ws.alloc(tiles * ksplit * 16 * nb * 8 * sizeof(int32_t));
    B2_CHECK(g.partial, B200DNN_FAILURE, "workspace allocation failed");
    g.counters = R.counters;
  }
  dim3 grid(tiles_n, ksplit, tiles_m);
  if (a_unsigned) {
    B2_TRY(ensure_max_smem((const void *)stream_gemm_kernel<true>, 200 * 1024));
    stream_gemm_kernel<true><<<grid, 256, smem, st>>>(g, epi);
  } else {
    B2_TRY(ensure_max_smem((const void *)stream_gemm_kernel<false>, 200 * 1024));
    stream_gemm_kernel<false><<<grid, 256, smem, st>>>(g, epi);
  }
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  return B200DNN_SUCCESS;
}

// Decode-shape kernel (M <= 16): persistent, evenly split over all warps of the device.
// Returns unimplemented when the shape does not fit it (the caller then uses the tiled streaming kernel).
int32_t launch_decode(const uint8_t *A, int64_t lda, bool a_unsigned, int M, int N, int K, const PackedWeight &pw,
                      const EpiParams &epi, bool early_weights, cudaStream_t st) {
  Runtime &R = rt();
  DecodeGemmArgs g{};
  g.A = A; g.lda = lda; g.M = M; g.N = N; g.K = K; g.Wt = pw.wt; g.Kp = (int)pw.Kp;
  g.groups = (N + 7) / 8; g.blocks = (int)(pw.Kp / 128);
  g.a_stride = (int)pw.Kp + 16;
  g.rows_staged = M > 8 ? 16 : 8;
  const int grid = g.groups < R.sm_count ? g.groups : R.sm_count;
  g.max_local_groups = (g.groups + grid - 1) / grid;
  g.tune = env_int("B200DNN_DECODE_TUNE", 0);
  const size_t smem = (size_t)g.rows_staged * g.a_stride + (size_t)g.max_local_groups * 512 + decode_epi_bytes(g.max_local_groups);
  if (M > 16 || smem > 220 * 1024) return B200DNN_UNIMPLEMENTED;
  void (*kern)(DecodeGemmArgs, EpiParams) = a_unsigned ? decode_gemm_kernel<true> : decode_gemm_kernel<false>;
  B2_TRY(ensure_max_smem((const void *)kern));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(kDecodeWarps * 32); cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = early_weights ? 1 : 0;
  B2_CUDA(cudaLaunchKernelEx(&cfg, kern, g, epi));
  B2_LAUNCHED();
  return B200DNN_SUCCESS;
}

// Ring form of the decode GEMM (decode_ring.cuh).  unimplemented when the ring would be too shallow.
template <int R>
int32_t launch_decode_ring(const uint8_t *A, int64_t lda, bool a_unsigned, int M, int N, int K, const PackedWeight &pw,
                           const EpiParams &epi, bool early_weights, cudaStream_t st) {
  Runtime &R_ = rt();
  DecodeRingArgs g{};
  g.A = A; g.lda = lda; g.M = M; g.N = N; g.K = K; g.Wt = pw.wt; g.Kp = (int)pw.Kp;
  g.groups = (N + 7) / 8; g.blocks = (int)(pw.Kp / 128);
  g.a_stride = (int)pw.Kp + 16;
  g.rows_staged = M > 8 ? 16 : M;
  const int grid = g.groups < R_.sm_count ? g.groups : R_.sm_count;
  g.max_local_groups = (g.groups + grid - 1) / grid;
  g.status = R_.status;
  g.test_no_loads = env_int("B200DNN_TEST_NO_LOADS", 0);   // see decode_ring.cuh; off unless a test sets it
  const size_t stage_bytes = (size_t)R * kRingWarps * 1024;
  const size_t fixed = ring_off_ring(g.rows_staged, g.a_stride, g.max_local_groups);
  const size_t budget = 227 * 1024;
  if (M > 16 || fixed + 3 * stage_bytes > budget) return B200DNN_UNIMPLEMENTED;
  int stages = (int)((budget - fixed) / stage_bytes);
  const int need = ((g.max_local_groups + R - 1) / R) * ((g.blocks + kRingWarps - 1) / kRingWarps);
  if (stages > kRingMaxStages) stages = kRingMaxStages;
  if (stages > need) stages = need;
  // three stages measured best: a deeper ring delays the activation loads behind its own requests
  const int cap = env_int("B200DNN_RING_STAGES", 3);
  if (cap > 1 && stages > cap) stages = cap;
  g.stages = stages;
  const size_t smem = fixed + (size_t)stages * stage_bytes;
  void (*kern)(DecodeRingArgs, EpiParams) = a_unsigned ? decode_ring_kernel<true, R> : decode_ring_kernel<false, R>;
  B2_TRY(ensure_max_smem((const void *)kern));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3((kRingWarps + 1) * 32); cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = early_weights ? 1 : 0;
  B2_CUDA(cudaLaunchKernelEx(&cfg, kern, g, epi));
  B2_LAUNCHED();
  return B200DNN_SUCCESS;
}

// Tile width.  With at least one tile per SM the candidates are the multiples of 32 from 256 down to 128 (multiples of
// 64 in the gated form) and the cost of a candidate is its number of waves over the SMs times (width + 16): the last,
// partly filled wave of a persistent grid can cost more than a narrower tile does (M=2048, N=14336: 896 tiles of 256
// columns are 7 waves on 148 SMs, 1024 tiles of 224 columns are 7 waves as well and each is an eighth shorter).
// Smaller problems take the widest tile that still gives every SM one.
int pick_bn(int m_tiles, int N, int sm_count, int gated, int pair = 0) {
  int forced = env_int("B200DNN_TC_BN", 0);
  if (forced > 0) return forced;
  if (pair) {
    // pair form: m_tiles counts 256-row tiles, one per CTA pair; each CTA's half of the tile must hold whole
    // 64-column gate/up blocks in the gated form (and whole 8-row weight groups always)
    const int pairs = sm_count / 2, pstep = gated ? 128 : 32;
    int best = 256; long long best_cost = -1;
    for (int bn = 256; bn >= 128; bn -= pstep) {
      const long long tiles = (long long)m_tiles * ((N + bn - 1) / bn);
      const long long cost = ((tiles + pairs - 1) / pairs) * (bn + 16);
      if (best_cost < 0 || cost < best_cost) { best = bn; best_cost = cost; }
    }
    return best;
  }
  const int step = gated ? 64 : 32;
  if ((long long)m_tiles * ((N + 127) / 128) >= sm_count) {
    int best = 256; long long best_cost = -1;
    for (int bn = 256; bn >= 128; bn -= step) {
      const long long tiles = (long long)m_tiles * ((N + bn - 1) / bn);
      const long long cost = ((tiles + sm_count - 1) / sm_count) * (bn + 16);
      if (best_cost < 0 || cost < best_cost) { best = bn; best_cost = cost; }
    }
    return best;
  }
  const int cands[3] = {128, 64, 32};
  for (int i = 0; i < 3; ++i) {
    int bn = cands[i];
    if (gated && bn < 64) break;
    if ((long long)m_tiles * ((N + bn - 1) / bn) >= sm_count || i == 2 || (gated && bn == 64)) return bn;
  }
  return gated ? 64 : 32;
}

// Split form for small plain GEMMs.  With fewer tiles than SMs the persistent kernel leaves SMs idle and, worse, too few
// weight bytes in flight (stages x BN x 128 B per CTA) to cover the HBM latency: M = 128, N = K = 4096 streamed its weight
// at 1.2 TB/s.  Clusters of 2 to 4 CTAs share one tile, each taking a share of the K blocks; the int32 partial sums are
// added through distributed shared memory, so the result is the same bit for bit.  Chooses the (tile width, splits)
// pair that puts the most CTAs on the device in one wave.
#ifdef B200DNN_TIMING_EXPERIMENTS
constexpr size_t kStampCtas = 4096;
unsigned long long *stamp_buffer() {
  static unsigned long long *p = nullptr;
  if (!p && cudaMalloc(&p, kStampCtas * 8 * sizeof(unsigned long long)) != cudaSuccess) p = nullptr;
  return p;
}
extern "C" __attribute__((visibility("default"))) int32_t b200dnn_debug_stamps(unsigned long long *host, int32_t ctas) {
  if (!stamp_buffer() || ctas < 0 || (size_t)ctas > kStampCtas) return B200DNN_FAILURE;
  return cudaMemcpy(host, stamp_buffer(), (size_t)ctas * 8 * sizeof(unsigned long long), cudaMemcpyDeviceToHost) == cudaSuccess ? B200DNN_SUCCESS : B200DNN_FAILURE;
}
#endif

// CTAs that are resident at once when the split form is launched in clusters of s (clusters do not tile the GPCs perfectly)
int split_room(int s) {
  int *cache = rt().shared->split_room;   // per device; two threads may both compute the same value
  if (cache[s] == 0) {
    cache[s] = -1;
    if (ensure_max_smem((const void *)tc_gemm_kernel<true>, kTcSmemBudget + 1024) == B200DNN_SUCCESS) {
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3((unsigned)(s * 64)); cfg.blockDim = dim3(kTcThreads); cfg.dynamicSmemBytes = kTcSmemBudget + 1024;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = (unsigned)s; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr; cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, tc_gemm_kernel<true>, &cfg) == cudaSuccess && n > 0) cache[s] = n * s;
      else cudaGetLastError();
      if (env_int("B200DNN_DEBUG", 0)) fprintf(stderr, "b200dnn: clusters of %d: %d resident CTAs\n", s, cache[s]);
    }
  }
  return cache[s];
}

void pick_split(int m_tiles, int N, int k_blocks, int *bn, int *splits) {
  const int forced = env_int("B200DNN_TC_KSPLIT", 0);   // 0 choose, 1 never, 2..4 that many
  if (forced == 1) return;
  const int sm = rt().sm_count;
  const int room[5] = {0, 0, split_room(2), split_room(3), split_room(4)};
  // Cost model fitted to measurements (microseconds, without the fixed cost of a launch): the stage ring is filled
  // from L2 at about 100 GB/s per SM and 9.5 TB/s over the device (every CTA re-reads its rows of A, so wide tiles
  // move fewer bytes); adding the partial sums costs about 1.6 us per extra CTA of the cluster and 128 columns of tile.
  auto stream_us = [&](long long ctas, int b, int kb_per_cta, int waves) {
    const double per_cta = (double)(kTcBM + b) * kTcBK * kb_per_cta;
    const double dev = per_cta * (double)ctas / 9.5e6, one = per_cta * waves / 1.0e5;
    return dev > one ? dev : one;
  };
  const long long tiles0 = (long long)m_tiles * ((N + *bn - 1) / *bn);
  const double unsplit = stream_us(tiles0, *bn, k_blocks, (int)((tiles0 + sm - 1) / sm));
  double best = forced >= 2 ? 1e30 : unsplit - 0.5;
  int best_bn = 0, best_s = 1;
  const int widths[3] = {256, 128, 64};
  const int forced_bn = env_int("B200DNN_TC_BN", 0);
  for (int w = 0; w < 3; ++w) {
    const int b = forced_bn > 0 ? forced_bn : widths[w];
    if (b % 32 != 0 || b < 32 || b > 256) continue;
    const long long tiles = (long long)m_tiles * ((N + b - 1) / b);
    for (int s = 2; s <= 4; ++s) {
      if (forced >= 2 && s != forced) continue;
      const int per = (k_blocks + s - 1) / s;
      if (per * (s - 1) >= k_blocks || per < 2) continue;          // every CTA needs K blocks of its own
      if ((b / 32) < s) continue;                                   // and at least one 32-column chunk to finish
      if (forced < 2 && (room[s] <= 0 || tiles * s > room[s])) continue;   // one wave of resident clusters
      const double cost = stream_us(tiles * s, b, per, 1) + 1.6 * (s - 1) * b / 128.0;
      if (cost < best) { best = cost; best_bn = b; best_s = s; }
    }
  }
  if (best_s > 1) { *bn = best_bn; *splits = best_s; }
}

// Rows of a row tile for a GEMM over about `rows` rows: 256 (pair form, two CTAs per tile) for large problems, else 128.
// B200DNN_TC_PAIR: -1 (default) by size, 0 never, 1 whenever the shape allows.
int tc_tile_rows(long long rows, int N) {
  const int mode = env_int("B200DNN_TC_PAIR", -1);
  if (mode == 0 || N < 128) return kTcBM;
  if (mode == 1) return 2 * kTcBM;
  // worth it once every CTA pair has several tiles: the pair form wastes up to 255 rows at the end of a group
  const long long tiles = ((rows + 255) / 256) * ((N + 255) / 256);
  return tiles >= 2LL * (rt().sm_count / 2) ? 2 * kTcBM : kTcBM;
}

// Plain or grouped tcgen05 GEMM.  A: [M_total, lda] device, 16-byte aligned rows.  bf16 form (args.f16): K and lda count
// bytes (two per element) and pw0 holds a bf16 pack.
int32_t launch_tc(const uint8_t *A, int64_t lda, bool a_unsigned, int M_total, int N, int K, const PackedWeight &pw0,
                  TcGemmArgs args, const EpiParams &epi, int m_tiles_hint, cudaStream_t st) {
  Runtime &R = rt();
  CUtensorMap map_a, map_b, map_c;
  B2_TRY(make_map_2d(&map_a, A, (uint64_t)K, (uint64_t)M_total, (uint64_t)lda, kTcBM));
  args.M_total = M_total; args.N = N; args.k_blocks = (int)(pw0.Kp / 128);
  args.a_unsigned = a_unsigned ? 1 : 0; args.gated = pw0.gated; args.status = R.status;
  args.fast_act = FA_GENERIC;
  if (epi.n_po == 0) args.fast_act = FA_NONE;
  else if (epi.n_po == 1) {
    switch (epi.po[0].type) {
    case PO_RELU: args.fast_act = FA_RELU; break;
    case PO_GELU_TANH: args.fast_act = FA_GELU_TANH; break;
    case PO_GELU_ERF: args.fast_act = FA_GELU_ERF; break;
    case PO_SIGMOID: args.fast_act = FA_SIGMOID; break;
    case PO_SWISH: args.fast_act = FA_SWISH; break;
    case PO_TANH: args.fast_act = FA_TANH; break;
    default: break;
    }
  }
  args.test_no_loads = env_int("B200DNN_TEST_NO_LOADS", 0);   // see tc_gemm.cuh; off unless a test sets it
  args.stamps = nullptr;
#ifdef B200DNN_TIMING_EXPERIMENTS
  args.dbg = env_int("B200DNN_TC_DBG", 0);    // parts of the epilogue switched off: results are invalid
  if (env_int("B200DNN_TC_STAMPS", 0)) args.stamps = stamp_buffer();
#else
  args.dbg = 0;
#endif
  args.BN = pick_bn(m_tiles_hint, N, R.sm_count, pw0.gated, args.pair);
  args.k_splits = 1;
  if (!args.pair && args.n_groups <= 1 && !args.maps_b && !args.groups && !args.tile_prefix && !pw0.gated) pick_split(m_tiles_hint, N, args.k_blocks, &args.BN, &args.k_splits);
  B2_CHECK(args.BN % 32 == 0 && args.BN >= 32 && args.BN <= 256 && (!pw0.gated || args.BN % 64 == 0), B200DNN_FAILURE,
           "bad tile width %d", args.BN);
  B2_CHECK(!args.pair || (args.BN % 32 == 0 && args.BN >= 64 && (!pw0.gated || args.BN % 128 == 0)), B200DNN_FAILURE,
           "bad tile width %d for the pair form", args.BN);
  args.n_tiles = (N + args.BN - 1) / args.BN;
  // Tile order.  Sweeping the row tiles under one column tile keeps that weight slice hot and re-reads the
  // activations once per column tile.  When the weight of a group is small enough to stay in L2 and the
  // activations are the larger operand (many rows, as in a fine-grained MoE), the column tiles of one row tile
  // run together instead: activations are read once, the weight is re-read from L2.
  // Which one moves fewer DRAM bytes is estimated from what the L2 can keep (ncu on the down projection of a
  // Mixtral-like layer, 14336 x 4096 per expert: column-tile-major read the 117 MB of activations once per wave of tiles,
  // 1.43 GB for 0.59 GB of operands; row-tile-major finishes an expert in about one wave).
  {
    const long long kL2 = 96ll << 20;                                   // what a sweep can count on, of 126 MB
    const long long w_group = (long long)pw0.Kp * pw0.Np, groups = args.n_groups > 0 ? args.n_groups : 1;
    const long long w_all = w_group * groups, a_bytes = (long long)M_total * K;
    const long long conc = R.sm_count / (args.pair ? 2 : 1);           // tiles in flight
    const long long tiles_all = (long long)m_tiles_hint * args.n_tiles;
    const long long waves = (tiles_all + conc - 1) / conc;
    // column-tile-major: the activations survive between the waves only if they fit beside the weight slices in flight
    const long long a_reads = (a_bytes + w_all / (args.n_tiles > 0 ? args.n_tiles : 1) <= kL2) ? 1 : (waves < args.n_tiles ? waves : args.n_tiles);
    const long long traffic_col = w_all + a_bytes * a_reads;
    // row-tile-major: a group's weight is read again for every wave of that group's row tiles unless it stays in L2
    const long long tiles_group = ((long long)m_tiles_hint + groups - 1) / groups * args.n_tiles;
    const long long w_reads = (w_group <= kL2 / 2) ? 1 : (tiles_group + conc - 1) / conc;
    const long long traffic_row = a_bytes + w_all * w_reads;
    args.n_fastest = env_int("B200DNN_TC_ORDER", traffic_row < traffic_col ? 1 : 0);
  }
  const int stage_bytes = kTcBM * kTcBK + (args.pair ? args.BN / 2 : args.BN) * kTcBK;   // per CTA
  int stages = kTcSmemBudget / stage_bytes;
  if (stages > 8) stages = 8;
  int forced_stages = env_int("B200DNN_TC_STAGES", 0);
  if (forced_stages > 0 && forced_stages <= stages) stages = forced_stages;
  args.stages = stages;
  B2_TRY(make_map_wt(&map_b, pw0.wt, (uint64_t)pw0.Kp, (uint64_t)pw0.Np, (uint32_t)(args.pair ? args.BN / 2 : args.BN)));
  const size_t smem = (size_t)stages * stage_bytes + 1024;
  B2_TRY(ensure_max_smem((const void *)tc_gemm_kernel<false>, kTcSmemBudget + 1024));   // the kernel also has static shared memory
  long long tiles = (long long)m_tiles_hint * args.n_tiles;
  int grid = (int)(tiles < R.sm_count ? (tiles > 0 ? tiles : 1) : R.sm_count);
  // bf16 results into one shared destination (plain GEMM, or a grouped GEMM whose groups all write epi.dst at their
  // global row): whole 32-row blocks leave as TMA stores.  Measured: 9 % faster for short-K plain GEMMs, no gain for
  // long K, slower for the gated epilogue (its tiles are bound by the epilogue and the wait for the copy engine to
  // read the staging block serialises it), so the gated form keeps the load/store path.
  // B200DNN_TC_TMA_STORE: 0 never, 1 always, 2 (default) all but the gated form.
  {
    const int64_t cols = pw0.gated ? epi.gated_I : N;
    const bool can = args.shared_dst && epi.dst_dt == B200DNN_BF16 && epi.dst && cols * 2 >= 32 &&
                     ((reinterpret_cast<uintptr_t>(epi.dst) | (uintptr_t)(epi.ldc * 2)) & 15) == 0 &&
                     (env_int("B200DNN_TC_TMA_STORE", 2) == 1 || (env_int("B200DNN_TC_TMA_STORE", 2) == 2 && !pw0.gated));
    args.tma_store = can ? 1 : 0;
    if (can) B2_TRY(make_map_store(&map_c, epi.dst, (uint64_t)cols * 2, (uint64_t)M_total, (uint64_t)epi.ldc * 2));
    else map_c = map_a;
  }
  // Both forms are launched with the programmatic-serialisation attribute: the kernel waits (griddepcontrol.wait) for
  // everything before it in the stream before it touches global memory, so the ordering is that of a plain launch; what
  // overlaps with the tail of the previous kernel is the launch itself.
  {
    cudaLaunchConfig_t cfg{};
    cfg.blockDim = dim3(kTcThreads); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (env_int("B200DNN_PDL", 1) != 0) {
      attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[na].val.programmaticStreamSerializationAllowed = 1;
      ++na;
    }
    if (args.pair) {
      // clusters of two CTAs, one [256 x BN] tile at a time per cluster, persistent over the tiles
      B2_TRY(ensure_max_smem((const void *)tc_gemm_kernel<false, true>, kTcSmemBudget + 1024));
      attr[na].id = cudaLaunchAttributeClusterDimension;
      attr[na].val.clusterDim.x = 2; attr[na].val.clusterDim.y = 1; attr[na].val.clusterDim.z = 1;
      ++na;
      const long long pairs = tiles < R.sm_count / 2 ? (tiles > 0 ? tiles : 1) : R.sm_count / 2;
      cfg.gridDim = dim3((unsigned)(2 * pairs));
      cfg.attrs = attr; cfg.numAttrs = na;
      if (args.f16) {
        B2_TRY(ensure_max_smem((const void *)tc_gemm_kernel<false, true, true>, kTcSmemBudget + 1024));
        B2_CUDA(cudaLaunchKernelEx(&cfg, tc_gemm_kernel<false, true, true>, map_a, map_b, map_c, args, epi));
      } else B2_CUDA(cudaLaunchKernelEx(&cfg, tc_gemm_kernel<false, true>, map_a, map_b, map_c, args, epi));
    } else if (args.k_splits > 1) {
      // one cluster of k_splits CTAs per tile; the partial sums need BN * 512 bytes of the stage ring
      B2_CHECK((size_t)args.BN * 512 <= (size_t)stages * stage_bytes, B200DNN_FAILURE, "split form: stage ring smaller than the partial sums");
      B2_TRY(ensure_max_smem((const void *)tc_gemm_kernel<true>, kTcSmemBudget + 1024));
      attr[na].id = cudaLaunchAttributeClusterDimension;
      attr[na].val.clusterDim.x = (unsigned)args.k_splits; attr[na].val.clusterDim.y = 1; attr[na].val.clusterDim.z = 1;
      ++na;
      cfg.gridDim = dim3((unsigned)(tiles * args.k_splits));
      cfg.attrs = attr; cfg.numAttrs = na;
      if (args.f16) {
        B2_TRY(ensure_max_smem((const void *)tc_gemm_kernel<true, false, true>, kTcSmemBudget + 1024));
        B2_CUDA(cudaLaunchKernelEx(&cfg, tc_gemm_kernel<true, false, true>, map_a, map_b, map_c, args, epi));
      } else B2_CUDA(cudaLaunchKernelEx(&cfg, tc_gemm_kernel<true>, map_a, map_b, map_c, args, epi));
    } else {
      cfg.gridDim = dim3((unsigned)grid);
      cfg.attrs = attr; cfg.numAttrs = na;
      if (args.f16) {
        B2_TRY(ensure_max_smem((const void *)tc_gemm_kernel<false, false, true>, kTcSmemBudget + 1024));
        B2_CUDA(cudaLaunchKernelEx(&cfg, tc_gemm_kernel<false, false, true>, map_a, map_b, map_c, args, epi));
      } else B2_CUDA(cudaLaunchKernelEx(&cfg, tc_gemm_kernel<false>, map_a, map_b, map_c, args, epi));
    }
  }
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  return B200DNN_SUCCESS;
}

// the stream has been drained: report a kernel that gave up on one of its bounded waits
int32_t check_tc_status(cudaStream_t st) {
  B2_CUDA(cudaStreamSynchronize(st));
  return read_status();
}

int32_t fill_epi(const b200dnn_matmul_t *d, EpiParams *e) {
  memset(e, 0, sizeof *e);
  e->dst_dt = d->dst_dt; e->ldc = d->ldc;
  e->bias_dt = d->bias_dt;
  e->n_po = d->n_postops;
  return B200DNN_SUCCESS;
}

}  // namespace

namespace {
// matmul_direct's transA: the source arrives as [K, lda] (element (m, k) at k * lda + m) and is transposed into the
// workspace as [M, pitch]; 32 x 32 tiles through shared memory, elements of 1, 2 or 4 bytes.
template <typename T>
__global__ void transpose_src_kernel(const T *src, int64_t lda, int M, int K, T *dst, int64_t pitch) {
  __shared__ T tile[32][33];
  const int k0 = blockIdx.y * 32, m0 = blockIdx.x * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int k = k0 + r, m = m0 + threadIdx.x;
    if (k < K && m < M) tile[r][threadIdx.x] = src[(int64_t)k * lda + m];
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int m = m0 + r, k = k0 + threadIdx.x;
    if (m < M && k < K) dst[(int64_t)m * pitch + k] = tile[threadIdx.x][r];
  }
}

int32_t untranspose_source(const b200dnn_matmul_t *d, b200dnn_matmul_t *t, cudaStream_t st) {
  const int M = d->M, K = d->K;
  B2_CHECK(d->src && M > 0 && K > 0, B200DNN_FAILURE, "null src or non-positive dimension");
  B2_CHECK(d->lda >= M, B200DNN_FAILURE, "transA: lda smaller than M");
  const size_t esz = dt_size(d->src_dt);
  B2_CHECK(esz == 1 || esz == 2 || esz == 4, B200DNN_UNIMPLEMENTED, "transA: source dtype %d", d->src_dt);
  const void *src = nullptr;
  B2_TRY(stage_in(d->src, span_bytes(K, M, d->lda, d->src_dt), st, &src));
  const int64_t pitch = round_up(K, (int64_t)(16 / esz));
  void *buf = rt().ws.alloc((size_t)M * pitch * esz);
  B2_CHECK(buf, B200DNN_FAILURE, "workspace allocation failed");
  if (pitch != K) B2_CUDA(cudaMemsetAsync(buf, 0, (size_t)M * pitch * esz, st));
  dim3 grid((unsigned)((M + 31) / 32), (unsigned)((K + 31) / 32)), block(32, 8);
  if (esz == 1) transpose_src_kernel<uint8_t><<<grid, block, 0, st>>>((const uint8_t *)src, d->lda, M, K, (uint8_t *)buf, pitch);
  else if (esz == 2) transpose_src_kernel<uint16_t><<<grid, block, 0, st>>>((const uint16_t *)src, d->lda, M, K, (uint16_t *)buf, pitch);
  else transpose_src_kernel<uint32_t><<<grid, block, 0, st>>>((const uint32_t *)src, d->lda, M, K, (uint32_t *)buf, pitch);
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  *t = *d;
  t->transA = 0; t->src = buf; t->lda = pitch;
  return B200DNN_SUCCESS;
}
}  // namespace

#include "gs_api.cuh"
#include "bf16_api.cuh"
#include "woq_api.cuh"

// =========================================================================================== C ABI
extern "C" {

const char *b200dnn_last_error(void) { return err_text().c_str(); }
int32_t b200dnn_version(void) { return 100; }
int32_t b200dnn_device_count(void) { return device_count(); }
int64_t b200dnn_launch_count(void) { return launch_counter().load(); }

size_t b200dnn_prepack_size(int64_t K, int64_t N, int32_t gated) {
  (void)gated;
  if (K <= 0 || N <= 0) return 0;
  return (pack_bytes(K, N) + 63) & ~size_t(63);
}

int32_t b200dnn_prepack(const void *weight, int64_t K, int64_t N, int64_t ldb, int32_t transB, int32_t gated, void *dst,
                        void *stream) {
  B2_ENTER(stream);
  B2_CHECK(weight && dst && K > 0 && N > 0, B200DNN_FAILURE, "prepack: null pointer or non-positive dimension");
  B2_CHECK(ldb >= (transB ? K : N), B200DNN_FAILURE, "prepack: ldb=%lld too small", (long long)ldb);
  const void *w_dev = nullptr;
  B2_TRY(stage_in(weight, span_bytes(transB ? N : K, transB ? K : N, ldb, B200DNN_S8), st, &w_dev));
  Staged out;
  B2_TRY(stage_out(dst, pack_bytes(K, N), st, &out));
  PackedWeight pw;
  B2_TRY(pack_into(w_dev, K, N, ldb, transB, gated, out.dev, st, &pw));
  {
    DeviceShared &D = *rt().shared;
    std::lock_guard<std::mutex> lk(D.cache_mu);
    if (!out.copy_back && !out.sync) D.packed_registry[dst] = pw;
    else {
      auto it = D.host_packed.find(dst);
      if (it != D.host_packed.end()) { if (it->second.owned) cudaFree(it->second.owned); if (it->second.ready) cudaEventDestroy(it->second.ready); D.host_packed.erase(it); }
    }
  }
  return finish_out({&out}, st);
}

int32_t b200dnn_quant_per_token(const void *src, int32_t src_dt, int64_t M, int64_t K, int64_t src_ld, void *dst,
                                int64_t dst_ld, void *scale, int32_t scale_dt, void *stream) {
  B2_ENTER(stream);
  B2_CHECK(src && scale, B200DNN_FAILURE, "dynamic quantisation needs src and a scale buffer");
  B2_CHECK(M > 0 && K > 0 && src_ld >= K && (!dst || dst_ld >= K), B200DNN_FAILURE, "bad shape or stride");
  B2_CHECK(scale_dt == B200DNN_F32 || scale_dt == B200DNN_BF16, B200DNN_UNIMPLEMENTED, "scale dtype must be f32 or bf16");
  const void *s_dev = nullptr;
  B2_TRY(stage_in(src, span_bytes(M, K, src_ld, src_dt), st, &s_dev));
  Staged o_q, o_s;
  B2_TRY(stage_out(dst, span_bytes(M, K, dst_ld, B200DNN_S8), st, &o_q, dst && dst_ld != K));
  B2_TRY(stage_out(scale, (size_t)M * dt_size(scale_dt), st, &o_s));
  RowQuantArgs a{};
  a.src = s_dev; a.src_ld = src_ld; a.dst = (int8_t *)o_q.dev; a.dst_ld = dst_ld; a.scale = o_s.dev; a.scale_dt = scale_dt;
  a.K = (int32_t)K; a.gather_div = 1;
  B2_TRY(launch_quant_rows(a, src_dt, M, st));
  return finish_out({&o_q, &o_s}, st);
}

int32_t b200dnn_quant_per_token_asym(const void *src, int32_t src_dt, int64_t M, int64_t K, int64_t src_ld, void *dst,
                                     int64_t dst_ld, float *scale, int32_t *zero_point, void *stream) {
  B2_ENTER(stream);
  B2_CHECK(src && scale && zero_point, B200DNN_FAILURE, "asymmetric dynamic quantisation needs src, a scale buffer and a zero-point buffer");
  B2_CHECK(M > 0 && K > 0 && src_ld >= K && (!dst || dst_ld >= K), B200DNN_FAILURE, "bad shape or stride");
  B2_CHECK(src_dt == B200DNN_BF16 || src_dt == B200DNN_F32, B200DNN_UNIMPLEMENTED, "source must be f32 or bf16");
  const void *s_dev = nullptr;
  B2_TRY(stage_in(src, span_bytes(M, K, src_ld, src_dt), st, &s_dev));
  Staged o_q, o_s, o_z;
  B2_TRY(stage_out(dst, span_bytes(M, K, dst_ld, B200DNN_U8), st, &o_q, dst && dst_ld != K));
  B2_TRY(stage_out(scale, (size_t)M * 4, st, &o_s));
  B2_TRY(stage_out(zero_point, (size_t)M * 4, st, &o_z));
  if (src_dt == B200DNN_BF16)
    quant_per_token_asym_kernel<uint16_t><<<(unsigned)M, kQuantThreads, 0, st>>>((const uint16_t *)s_dev, src_ld, (int)K, (uint8_t *)o_q.dev, dst_ld, (float *)o_s.dev, (int32_t *)o_z.dev);
  else
    quant_per_token_asym_kernel<float><<<(unsigned)M, kQuantThreads, 0, st>>>((const float *)s_dev, src_ld, (int)K, (uint8_t *)o_q.dev, dst_ld, (float *)o_s.dev, (int32_t *)o_z.dev);
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  return finish_out({&o_q, &o_s, &o_z}, st);
}

int32_t b200dnn_group_quant_per_token(int32_t num_groups, const void *const *src, int32_t src_dt, const int32_t *M,
                                      const int32_t *K, const int64_t *src_ld, void *const *dst, const int64_t *dst_ld,
                                      void *const *scale, int32_t scale_dt, void *stream) {
  B2_ENTER(stream);
  B2_CHECK(num_groups > 0 && src && M && K && src_ld && dst && dst_ld && scale, B200DNN_FAILURE, "null argument");
  // groups of one row length share a launch; the reference lets K differ per group (reorder/lowoha_reorder.cpp:279-400):
  // one launch per distinct K
  std::vector<Staged> outs;
  outs.reserve(2 * num_groups);
  std::vector<const void *> s_dev(num_groups); std::vector<void *> d_dev(num_groups), sc_dev(num_groups);
  std::vector<int> distinct_k;
  for (int g = 0; g < num_groups; ++g) {
    if (M[g] <= 0) { s_dev[g] = nullptr; d_dev[g] = nullptr; sc_dev[g] = nullptr; continue; }
    B2_CHECK(K[g] > 0 && (!dst[g] || dst_ld[g] >= K[g]), B200DNN_FAILURE, "group %d: bad K or destination stride", g);
    B2_CHECK(src[g] && scale[g] && src_ld[g] >= K[g], B200DNN_FAILURE, "group %d: null pointer or bad stride", g);
    B2_TRY(stage_in(src[g], span_bytes(M[g], K[g], src_ld[g], src_dt), st, &s_dev[g]));
    Staged a, b;
    B2_TRY(stage_out(dst[g], span_bytes(M[g], K[g], dst_ld[g], B200DNN_S8), st, &a, dst[g] && dst_ld[g] != K[g]));
    B2_TRY(stage_out(scale[g], (size_t)M[g] * dt_size(scale_dt), st, &b));
    d_dev[g] = a.dev; sc_dev[g] = b.dev; outs.push_back(a); outs.push_back(b);
    if (std::find(distinct_k.begin(), distinct_k.end(), K[g]) == distinct_k.end()) distinct_k.push_back(K[g]);
  }
  if (distinct_k.empty()) return B200DNN_SUCCESS;
  for (int Kc : distinct_k) {
    // groups of another row length have no rows in this launch
    std::vector<int32_t> row_off(num_groups + 1, 0);
    for (int g = 0; g < num_groups; ++g) row_off[g + 1] = row_off[g] + ((M[g] > 0 && K[g] == Kc) ? M[g] : 0);
    const size_t tb = sizeof(void *) * num_groups;
    std::vector<uint8_t> host(3 * tb + 2 * sizeof(int64_t) * num_groups + sizeof(int32_t) * (num_groups + 1));
    uint8_t *h = host.data();
    memcpy(h, s_dev.data(), tb); memcpy(h + tb, d_dev.data(), tb); memcpy(h + 2 * tb, sc_dev.data(), tb);
    memcpy(h + 3 * tb, src_ld, sizeof(int64_t) * num_groups);
    memcpy(h + 3 * tb + sizeof(int64_t) * num_groups, dst_ld, sizeof(int64_t) * num_groups);
    memcpy(h + 3 * tb + 2 * sizeof(int64_t) * num_groups, row_off.data(), sizeof(int32_t) * (num_groups + 1));
    void *tab_dev = nullptr;
    B2_TRY(upload_blob(h, host.size(), st, &tab_dev));
    uint8_t *tab = (uint8_t *)tab_dev;
    RowQuantArgs a{};
    a.n_groups = num_groups; a.K = Kc; a.scale_dt = scale_dt; a.gather_div = 1;
    a.g_src = (const void *const *)tab; a.g_dst = (void *const *)(tab + tb); a.g_scale = (void *const *)(tab + 2 * tb);
    a.g_src_ld = (const int64_t *)(tab + 3 * tb); a.g_dst_ld = (const int64_t *)(tab + 3 * tb + sizeof(int64_t) * num_groups);
    a.row_off = (const int32_t *)(tab + 3 * tb + 2 * sizeof(int64_t) * num_groups);
    B2_TRY(launch_quant_rows(a, src_dt, row_off[num_groups], st));
  }
  bool any = false;
  for (auto &s : outs) { if (s.copy_back) { B2_CUDA(cudaMemcpyAsync(s.host, s.dev, s.bytes, cudaMemcpyDeviceToHost, st)); any = true; } else if (s.sync) any = true; }
  if (any) B2_CUDA(cudaStreamSynchronize(st));
  return B200DNN_SUCCESS;
}

int32_t b200dnn_quant_dynamic(const void *src, int32_t src_dt, int64_t M, int64_t N, int64_t src_ld, int32_t per_channel,
                              void *dst, int64_t dst_ld, float *scale, void *stream) {
  B2_ENTER(stream);
  B2_CHECK(src && scale && M > 0 && N > 0 && src_ld >= N && (!dst || dst_ld >= N), B200DNN_FAILURE, "bad argument");
  B2_CHECK(src_dt == B200DNN_BF16 || src_dt == B200DNN_F32, B200DNN_UNIMPLEMENTED, "source must be f32 or bf16");
  const void *s_dev = nullptr;
  B2_TRY(stage_in(src, span_bytes(M, N, src_ld, src_dt), st, &s_dev));
  const int64_t ns = per_channel ? N : 1;
  Staged o_q, o_s;
  B2_TRY(stage_out(dst, span_bytes(M, N, dst_ld, B200DNN_S8), st, &o_q, dst && dst_ld != N));
  B2_TRY(stage_out(scale, (size_t)ns * 4, st, &o_s));
  uint32_t *amax = (uint32_t *)rt().ws.alloc((size_t)ns * 4);
  B2_CHECK(amax, B200DNN_FAILURE, "workspace allocation failed");
  B2_CUDA(cudaMemsetAsync(amax, 0, (size_t)ns * 4, st));
  dim3 grid((unsigned)((N + 255) / 256), (unsigned)(M < 64 ? 1 : (M / 64 > 256 ? 256 : M / 64)));
  if (src_dt == B200DNN_BF16) absmax_cols_kernel<uint16_t><<<grid, 256, 0, st>>>((const uint16_t *)s_dev, M, N, src_ld, per_channel, amax);
  else absmax_cols_kernel<float><<<grid, 256, 0, st>>>((const float *)s_dev, M, N, src_ld, per_channel, amax);
  B2_LAUNCHED();
  scales_from_absmax_kernel<<<(unsigned)((ns + 255) / 256), 256, 0, st>>>(amax, ns, (float *)o_s.dev);
  B2_LAUNCHED();
  if (dst) {
    dim3 g2((unsigned)((N + 255) / 256), (unsigned)(M > 1024 ? 1024 : M));
    if (src_dt == B200DNN_BF16)
      quant_static_kernel<uint16_t><<<g2, 256, 0, st>>>((const uint16_t *)s_dev, M, N, src_ld, (const float *)o_s.dev, ns, nullptr, 0, o_q.dev, B200DNN_S8, dst_ld);
    else
      quant_static_kernel<float><<<g2, 256, 0, st>>>((const float *)s_dev, M, N, src_ld, (const float *)o_s.dev, ns, nullptr, 0, o_q.dev, B200DNN_S8, dst_ld);
    B2_LAUNCHED();
  }
  B2_CUDA(cudaGetLastError());
  return finish_out({&o_q, &o_s}, st);
}

int32_t b200dnn_quant_static(const void *src, int32_t src_dt, int64_t M, int64_t N, int64_t src_ld, const float *scale,
                             int64_t n_scale, const int32_t *zp, int64_t n_zp, void *dst, int32_t dst_dt, int64_t dst_ld,
                             void *stream) {
  B2_ENTER(stream);
  B2_CHECK(src && dst && scale && M > 0 && N > 0 && src_ld >= N && dst_ld >= N, B200DNN_FAILURE, "bad argument");
  B2_CHECK((n_scale == 1 || n_scale == N) && (!zp || n_zp == 1 || n_zp == N), B200DNN_UNIMPLEMENTED, "scale / zero-point granularity");
  B2_CHECK((src_dt == B200DNN_BF16 || src_dt == B200DNN_F32) && (dst_dt == B200DNN_S8 || dst_dt == B200DNN_U8), B200DNN_UNIMPLEMENTED, "dtype combination");
  const void *s_dev, *sc_dev, *zp_dev = nullptr;
  B2_TRY(stage_in(src, span_bytes(M, N, src_ld, src_dt), st, &s_dev));
  B2_TRY(stage_in(scale, (size_t)n_scale * 4, st, &sc_dev));
  if (zp) B2_TRY(stage_in(zp, (size_t)n_zp * 4, st, &zp_dev));
  Staged o;
  B2_TRY(stage_out(dst, span_bytes(M, N, dst_ld, dst_dt), st, &o, dst_ld != N));
  dim3 g2((unsigned)((N + 255) / 256), (unsigned)(M > 1024 ? 1024 : M));
  if (src_dt == B200DNN_BF16)
    quant_static_kernel<uint16_t><<<g2, 256, 0, st>>>((const uint16_t *)s_dev, M, N, src_ld, (const float *)sc_dev, n_scale, (const int32_t *)zp_dev, n_zp, o.dev, dst_dt, dst_ld);
  else
    quant_static_kernel<float><<<g2, 256, 0, st>>>((const float *)s_dev, M, N, src_ld, (const float *)sc_dev, n_scale, (const int32_t *)zp_dev, n_zp, o.dev, dst_dt, dst_ld);
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  return finish_out({&o}, st);
}

int32_t b200dnn_dequant_static(const void *src, int32_t src_dt, int64_t M, int64_t N, int64_t src_ld, const float *scale,
                               int64_t n_scale, const int32_t *zp, int64_t n_zp, void *dst, int32_t dst_dt, int64_t dst_ld,
                               void *stream) {
  B2_ENTER(stream);
  B2_CHECK(src && dst && scale && M > 0 && N > 0 && src_ld >= N && dst_ld >= N, B200DNN_FAILURE, "bad argument");
  B2_CHECK((n_scale == 1 || n_scale == N) && (!zp || n_zp == 1 || n_zp == N), B200DNN_UNIMPLEMENTED, "scale / zero-point granularity");
  B2_CHECK((src_dt == B200DNN_S8 || src_dt == B200DNN_U8) && (dst_dt == B200DNN_F32 || dst_dt == B200DNN_BF16), B200DNN_UNIMPLEMENTED, "dtype combination");
  const void *s_dev, *sc_dev, *zp_dev = nullptr;
  B2_TRY(stage_in(src, span_bytes(M, N, src_ld, src_dt), st, &s_dev));
  B2_TRY(stage_in(scale, (size_t)n_scale * 4, st, &sc_dev));
  if (zp) B2_TRY(stage_in(zp, (size_t)n_zp * 4, st, &zp_dev));
  Staged o;
  B2_TRY(stage_out(dst, span_bytes(M, N, dst_ld, dst_dt), st, &o, dst_ld != N));
  dim3 g2((unsigned)((N + 255) / 256), (unsigned)(M > 1024 ? 1024 : M));
  dequant_static_kernel<<<g2, 256, 0, st>>>(s_dev, src_dt, M, N, src_ld, (const float *)sc_dev, n_scale, (const int32_t *)zp_dev, n_zp, o.dev, dst_dt, dst_ld);
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  return finish_out({&o}, st);
}

int32_t b200dnn_gated_act(void *buf, int32_t dt, int64_t M, int64_t N, int64_t ldc, int32_t act, void *stream) {
  B2_ENTER(stream);
  B2_CHECK(buf && M > 0 && N > 0 && N % 2 == 0 && ldc >= N, B200DNN_FAILURE, "bad argument");
  B2_CHECK(act >= 1 && act <= 3, B200DNN_FAILURE, "unknown gated activation %d", act);
  B2_CHECK(dt == B200DNN_BF16 || dt == B200DNN_F32, B200DNN_UNIMPLEMENTED, "gated activation on f32 or bf16 only");
  Staged o;
  B2_TRY(stage_out(buf, span_bytes(M, N, ldc, dt), st, &o, true));
  if (dt == B200DNN_BF16) gated_act_kernel<uint16_t><<<(unsigned)M, 256, 0, st>>>((uint16_t *)o.dev, N, ldc, act);
  else gated_act_kernel<float><<<(unsigned)M, 256, 0, st>>>((float *)o.dev, N, ldc, act);
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  return finish_out({&o}, st);
}

int32_t b200dnn_moe_weighted_reduce(const void *const *row_ptrs, const float *topk_weights, int32_t T, int32_t topk,
                                    int32_t D, int32_t skip_weighted, int32_t dt, void *out, int64_t ld_out, void *stream) {
  B2_ENTER(stream);
  B2_CHECK(row_ptrs && out && T > 0 && topk > 0 && D > 0 && ld_out >= D, B200DNN_FAILURE, "bad argument");
  B2_CHECK(skip_weighted || topk_weights, B200DNN_FAILURE, "topk_weights is null");
  B2_CHECK(dt == B200DNN_BF16 || dt == B200DNN_F32, B200DNN_UNIMPLEMENTED, "weighted reduce on f32 or bf16 only");
  const size_t nslot = (size_t)T * topk;
  // row_ptrs is a host array (the reference's contract).  Rows in host memory are gathered into one pinned slab and
  // sent with one copy (a copy per row costs microseconds each: 8192 of them at 4096 tokens x top-2).
  std::vector<const void *> dev_rows(nslot);
  const bool rows_on_device = is_device_ptr(row_ptrs[0]);
  if (rows_on_device) {
    for (size_t i = 0; i < nslot; ++i) { B2_CHECK(row_ptrs[i], B200DNN_FAILURE, "row_ptrs[%zu] is null", i); dev_rows[i] = row_ptrs[i]; }
  } else {
    const size_t rb = (size_t)D * dt_size(dt), pitch = (rb + 15) & ~size_t(15);
    uint8_t *slab = (uint8_t *)rt().ws.alloc(nslot * pitch);
    uint8_t *pin = rt().pinned_slab(nslot * pitch);
    B2_CHECK(slab && pin, B200DNN_FAILURE, "staging allocation failed");
    for (size_t i = 0; i < nslot; ++i) {
      B2_CHECK(row_ptrs[i], B200DNN_FAILURE, "row_ptrs[%zu] is null", i);
      memcpy(pin + i * pitch, row_ptrs[i], rb);
      dev_rows[i] = slab + i * pitch;
    }
    B2_CUDA(cudaMemcpyAsync(slab, pin, nslot * pitch, cudaMemcpyHostToDevice, st));
    B2_CUDA(cudaStreamSynchronize(st));   // the pinned slab is reused by the next call
  }
  void *tab = nullptr;
  B2_TRY(upload_blob(dev_rows.data(), nslot * sizeof(void *), st, &tab));
  const void *w_dev = nullptr;
  if (!skip_weighted) B2_TRY(stage_in(topk_weights, nslot * 4, st, &w_dev));
  Staged o;
  B2_TRY(stage_out(out, span_bytes(T, D, ld_out, dt), st, &o, ld_out != D));
  ReduceArgs a{};
  a.row_ptrs = (const void *const *)tab; a.w = (const float *)w_dev; a.skip_weighted = skip_weighted;
  a.nslots = topk; a.D = D; a.dt = dt; a.out = o.dev; a.ld_out = ld_out;
  moe_reduce_kernel<<<(unsigned)T, 256, (sizeof(void *) + 4) * topk, st>>>(a);
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  return finish_out({&o}, st);
}

}  // extern "C"

// Router and stable-rank launches: the fast forms when the sizes allow, the general kernels otherwise.
int32_t launch_route_topk(const float *logits, int T, int E, int topk, int renorm, int32_t *ids, float *w, cudaStream_t st) {
  const unsigned blocks = (unsigned)(((size_t)T * 32 + 255) / 256);
  if (E <= 32) route_topk_warp_kernel<1><<<blocks, 256, 0, st>>>(logits, T, E, topk, renorm, ids, w);
  else if (E <= 64) route_topk_warp_kernel<2><<<blocks, 256, 0, st>>>(logits, T, E, topk, renorm, ids, w);
  else if (E <= 128) route_topk_warp_kernel<4><<<blocks, 256, 0, st>>>(logits, T, E, topk, renorm, ids, w);
  else if (E <= 256) route_topk_warp_kernel<8><<<blocks, 256, 0, st>>>(logits, T, E, topk, renorm, ids, w);
  else route_topk_kernel<<<(unsigned)((T + 127) / 128), 128, 0, st>>>(logits, T, E, topk, renorm, ids, w);
  B2_LAUNCHED();
  return B200DNN_SUCCESS;
}
int32_t launch_expert_rank(const int32_t *ids, int nslots, int nkeys, int32_t *rank, int32_t *counts, cudaStream_t st) {
  const int nchunks = (nslots + kRankChunk - 1) / kRankChunk;
  if (nkeys > kRankMaxKeys || nchunks < 4) {
    expert_rank_kernel<<<(unsigned)nkeys, 1024, 0, st>>>(ids, nslots, rank, counts);
    B2_LAUNCHED();
    return B200DNN_SUCCESS;
  }
  int32_t *cc = (int32_t *)rt().ws.alloc((size_t)nchunks * nkeys * 4);
  B2_CHECK(cc, B200DNN_FAILURE, "workspace allocation failed");
  rank_count_kernel<<<(unsigned)nchunks, kRankChunk, 0, st>>>(ids, nslots, nkeys, cc);
  B2_LAUNCHED();
  rank_scan_kernel<<<(unsigned)((nkeys * 32 + 255) / 256), 256, 0, st>>>(cc, nchunks, nkeys, counts);
  B2_LAUNCHED();
  rank_assign_kernel<<<(unsigned)nchunks, kRankChunk, (size_t)32 * nkeys * 4, st>>>(ids, nslots, nkeys, cc, rank);
  B2_LAUNCHED();
  return B200DNN_SUCCESS;
}

extern "C" {

int32_t b200dnn_moe_route(const float *logits, int32_t T, int32_t E, int32_t topk, int32_t renorm, int32_t *ids,
                          float *weights, int32_t *expert_counts, int32_t *slot_to_row, void *stream) {
  B2_ENTER(stream);
  B2_CHECK(logits && ids && T > 0 && E > 0 && topk > 0 && topk <= E && topk <= kMaxTopk, B200DNN_FAILURE, "bad argument");
  const void *l_dev;
  B2_TRY(stage_in(logits, (size_t)T * E * 4, st, &l_dev));
  const size_t ns = (size_t)T * topk;
  Staged o_ids, o_w, o_cnt, o_s2r;
  B2_TRY(stage_out(ids, ns * 4, st, &o_ids));
  B2_TRY(stage_out(weights, ns * 4, st, &o_w));
  B2_TRY(stage_out(expert_counts, (size_t)E * 4, st, &o_cnt));
  B2_TRY(stage_out(slot_to_row, ns * 4, st, &o_s2r));
  float *w_dev = (float *)o_w.dev;
  if (!w_dev) { w_dev = (float *)rt().ws.alloc(ns * 4); B2_CHECK(w_dev, B200DNN_FAILURE, "workspace allocation failed"); }
  B2_TRY(launch_route_topk((const float *)l_dev, T, E, topk, renorm, (int32_t *)o_ids.dev, w_dev, st));
  if (expert_counts || slot_to_row) {
    int32_t *cnt = (int32_t *)o_cnt.dev;
    if (!cnt) { cnt = (int32_t *)rt().ws.alloc((size_t)E * 4); B2_CHECK(cnt, B200DNN_FAILURE, "workspace allocation failed"); }
    int32_t *rank = (int32_t *)rt().ws.alloc(ns * 4);
    int32_t *off = (int32_t *)rt().ws.alloc((size_t)(E + 1) * 4);
    B2_CHECK(rank && off, B200DNN_FAILURE, "workspace allocation failed");
    B2_TRY(launch_expert_rank((const int32_t *)o_ids.dev, (int)ns, E, rank, cnt, st));
    if (slot_to_row) {
      expert_offsets_kernel<<<1, 32, 0, st>>>(cnt, E, 0, T, off);
      B2_LAUNCHED();
      int32_t *row_tok = (int32_t *)rt().ws.alloc(ns * 4);
      float *sw = (float *)rt().ws.alloc(ns * 4);
      B2_CHECK(row_tok && sw, B200DNN_FAILURE, "workspace allocation failed");
      build_maps_kernel<<<(unsigned)((ns + 255) / 256), 256, 0, st>>>((const int32_t *)o_ids.dev, rank, w_dev, off, T, topk, E, 0,
                                                                     (int32_t *)o_s2r.dev, sw, row_tok);
      B2_LAUNCHED();
    }
  }
  B2_CUDA(cudaGetLastError());
  return finish_out({&o_ids, &o_w, &o_cnt, &o_s2r}, st);
}

// -------------------------------------------------------------------------------------------- matmul
int32_t b200dnn_matmul(const b200dnn_matmul_t *d, void *stream) {
  B2_CHECK(d, B200DNN_FAILURE, "null descriptor");
  B2_ENTER(stream);
  b200dnn_matmul_t untransposed;
  if (d->transA) { B2_TRY(untranspose_source(d, &untransposed, st)); d = &untransposed; }
  if (is_woq_matmul(d)) return matmul_woq(d, st);               // bf16 source x s4|u4 weights, no dynamic quantisation
  if (is_group_scaled(d)) return matmul_group_scaled(d, st);   // per-group scales and W4A8: own validation and kernel
  if (is_bf16_matmul(d)) return matmul_bf16(d, st);             // bf16 x bf16: own validation, the kernel's bf16 form
  Runtime &R = rt();
  const int M = d->M, N = d->N, K = d->K;
  B2_TRY(validate_matmul_desc(d));
  const bool dyn = d->dynamic_quant != 0;

  // ---- operands on the device
  PackedWeight pw;
  B2_TRY(resolve_weight(d->weight, d->wei_format, K, N, d->ldb, d->transB, 0, d->weights_const, st, &pw));
  EpiParams epi;
  fill_epi(d, &epi);
  const void *src_dev = nullptr;
  B2_TRY(stage_in(d->src, span_bytes(M, K, d->lda, d->src_dt), st, &src_dev, &R.small));
  const uint8_t *A = (const uint8_t *)src_dev; int64_t lda = d->lda; bool a_unsigned = d->src_dt == B200DNN_U8;
  Staged o_scale;
  if (dyn) {
    const int64_t Kq = round_up(K, 16);
    int8_t *q = (int8_t *)R.ws.alloc((size_t)M * Kq);
    B2_CHECK(q, B200DNN_FAILURE, "workspace allocation failed");
    const int32_t sdt = d->src_scale.buff ? d->src_scale.dt : B200DNN_F32;
    B2_TRY(stage_out(const_cast<void *>(d->src_scale.buff), (size_t)M * dt_size(sdt), st, &o_scale));
    void *sc = o_scale.dev;
    if (!sc) { sc = R.ws.alloc((size_t)M * 4); B2_CHECK(sc, B200DNN_FAILURE, "workspace allocation failed"); }
    RowQuantArgs qa{};
    qa.src = src_dev; qa.src_ld = d->lda; qa.dst = q; qa.dst_ld = Kq; qa.scale = sc; qa.scale_dt = sdt; qa.K = K; qa.gather_div = 1;
    B2_TRY(R.small.flush(st, false));
    B2_TRY(launch_quant_rows(qa, d->src_dt, M, st));
    A = (const uint8_t *)q; lda = Kq; a_unsigned = false;
    epi.src_scale = sc; epi.src_scale_dt = sdt; epi.src_scale_n = M > 1 ? M : 1;
  } else if (d->src_scale.count > 0) {
    const void *p;
    B2_TRY(stage_in(d->src_scale.buff, (size_t)d->src_scale.count * dt_size(d->src_scale.dt), st, &p, &R.small));
    epi.src_scale = p; epi.src_scale_dt = d->src_scale.dt; epi.src_scale_n = (int32_t)d->src_scale.count;
  }
  if (d->wei_scale.count > 0) {
    const void *p;
    B2_TRY(stage_in(d->wei_scale.buff, (size_t)d->wei_scale.count * dt_size(d->wei_scale.dt), st, &p, &R.small));
    epi.wei_scale = p; epi.wei_scale_dt = d->wei_scale.dt; epi.wei_scale_n = (int32_t)d->wei_scale.count;
  }
  if (d->src_zp.buff) {
    B2_CHECK(d->src_zp.dt == B200DNN_S32 || d->src_zp.dt == B200DNN_S8 || d->src_zp.dt == B200DNN_U8, B200DNN_UNIMPLEMENTED, "src zero-point dtype");
    const void *p;
    B2_TRY(stage_in(d->src_zp.buff, dt_size(d->src_zp.dt), st, &p, &R.small));
    epi.src_zp = p; epi.src_zp_dt = d->src_zp.dt; epi.has_zp = 1;
  }
  epi.colsum = pw.colsum;
  if (d->bias) {
    const void *p;
    B2_TRY(stage_in(d->bias, (size_t)N * dt_size(d->bias_dt), st, &p, &R.small));
    epi.bias = p;
  }
  for (int i = 0; i < d->n_postops; ++i) {
    const b200dnn_postop_t &p = d->postops[i];
    epi.po[i].type = p.type; epi.po[i].dt = p.dt; epi.po[i].ld = p.ld; epi.po[i].alpha = p.alpha; epi.po[i].beta = p.beta;
    epi.po[i].buff = nullptr;
    if (p.type == PO_BINARY_ADD || p.type == PO_BINARY_MUL) {
      const void *b;
      B2_TRY(stage_in(p.buff, p.ld ? span_bytes(M, N, p.ld, p.dt) : (size_t)N * dt_size(p.dt), st, &b, &R.small));
      epi.po[i].buff = b;
    }
  }
  Staged o_dst;
  B2_TRY(stage_out(d->dst, span_bytes(M, N, d->ldc, d->dst_dt), st, &o_dst, d->ldc != N));
  epi.dst = o_dst.dev;
  // requantised integer destination: the GEMM writes f32 into the workspace, one more pass scales, shifts, clamps and rounds
  const bool requant = d->dst_dt == B200DNN_S8 || d->dst_dt == B200DNN_U8;
  const void *dst_scale_dev = nullptr, *dst_zp_dev = nullptr;
  if (requant) {
    float *tmp = (float *)R.ws.alloc((size_t)M * N * 4);
    B2_CHECK(tmp, B200DNN_FAILURE, "workspace allocation failed");
    epi.dst = tmp; epi.ldc = N; epi.dst_dt = B200DNN_F32;
    if (d->dst_scale.buff) B2_TRY(stage_in(d->dst_scale.buff, 4, st, &dst_scale_dev, &R.small));
    if (d->dst_zp.buff) B2_TRY(stage_in(d->dst_zp.buff, 4, st, &dst_zp_dev, &R.small));
  }
  B2_TRY(R.small.flush(st, o_dst.copy_back || o_dst.sync));

  // ---- kernel choice: weight-streaming kernel for decode-sized M, tcgen05 otherwise
  const bool tc_ok = (lda % 16 == 0) && ((reinterpret_cast<uintptr_t>(A) & 15) == 0);
  int which = d->force_kernel;
  if (which == 0) which = (M <= 16 || !tc_ok) ? 1 : 2;
  B2_CHECK(which == 1 || which == 3 || tc_ok, B200DNN_FAILURE, "tcgen05 kernel needs a 16-byte aligned source with lda %% 16 == 0");
  if (which == 1 || which == 3) {
    int32_t rc = B200DNN_UNIMPLEMENTED;
    // decode kernel: 0 tiled only, 1 register-batch form, 2 ring form, 3..5 ring with that many groups per stage;
    // default: ring for M <= 2 and weights of 24 MB or more (measured faster there: 10.9 against 11.5 us at 45 MB, but
    // 5.9 against 5.7 us at 16.8 MB), register-batch form otherwise
    const int dk = env_int("B200DNN_DECODE_KERNEL", (M <= 2 && (long long)K * N >= (24ll << 20)) ? 2 : 1);
    const bool pdl = (d->flags & B200DNN_FLAG_STABLE_WEIGHTS) != 0 && env_int("B200DNN_PDL", 1) != 0;
    if (which == 1 && M <= 16 && dk >= 2) {
      // groups per stage: split the CTA's groups into equal sets of at most five
      const int groups = (N + 7) / 8, grid = groups < rt().sm_count ? groups : rt().sm_count;
      const int local = (groups + grid - 1) / grid, sets = (local + 4) / 5;
      int r = dk > 2 ? dk : (local + sets - 1) / sets;
      if (r <= 2) rc = launch_decode_ring<2>(A, lda, a_unsigned, M, N, K, pw, epi, pdl, st);
      else if (r == 3) rc = launch_decode_ring<3>(A, lda, a_unsigned, M, N, K, pw, epi, pdl, st);
      else if (r == 4) rc = launch_decode_ring<4>(A, lda, a_unsigned, M, N, K, pw, epi, pdl, st);
      else rc = launch_decode_ring<5>(A, lda, a_unsigned, M, N, K, pw, epi, pdl, st);
    }
    if (which == 1 && M <= 16 && dk != 0 && rc == B200DNN_UNIMPLEMENTED) rc = launch_decode(A, lda, a_unsigned, M, N, K, pw, epi, pdl, st);
    if (rc == B200DNN_UNIMPLEMENTED) rc = launch_stream(A, lda, a_unsigned, M, N, K, pw, epi, st);
    B2_TRY(rc);
  } else {
    TcGemmArgs ta{};
    const int tile_rows = tc_tile_rows(M, N);
    ta.pair = tile_rows > kTcBM ? 1 : 0;
    ta.n_groups = 1; ta.m_tiles_plain = (M + tile_rows - 1) / tile_rows; ta.shared_dst = 1;
    B2_TRY(launch_tc(A, lda, a_unsigned, M, N, K, pw, ta, epi, ta.m_tiles_plain, st));
  }
  if (requant) {
    const int64_t n = (int64_t)M * N;
    requant_dst_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>((const float *)epi.dst, M, N, (const float *)dst_scale_dev,
                                                                    (const int32_t *)dst_zp_dev, o_dst.dev, d->dst_dt, d->ldc);
    B2_LAUNCHED();
    B2_CUDA(cudaGetLastError());
  }
  return finish_out({&o_dst, &o_scale}, st);   // calls that synchronise read the status word there
}

int32_t b200dnn_stream_status(void *stream) {
  B2_ENTER(stream);
  B2_CUDA(cudaStreamSynchronize(st));
  return read_status();
}

int32_t b200dnn_phase_timing(void *stream, int32_t enable) {
  B2_ENTER(stream);
  rt().timing = enable != 0;
  rt().n_tev = 0;
  return B200DNN_SUCCESS;
}

int32_t b200dnn_phase_times(void *stream, float *ms, int32_t n, int32_t *calls) {
  B2_ENTER(stream);
  B2_CHECK(ms && n > 0, B200DNN_FAILURE, "bad argument");
  B2_CUDA(cudaStreamSynchronize(st));
  Runtime &R = rt();
  for (int i = 0; i < n; ++i) ms[i] = 0.f;
  int n_calls = 0;
  for (size_t i = 0; i < R.n_tev; ++i) {
    if (R.tphase[i] < 0) { ++n_calls; continue; }      // a call starts here
    if (i == 0) continue;
    float t = 0.f;
    B2_CUDA(cudaEventElapsedTime(&t, R.tev[i - 1], R.tev[i]));
    if (R.tphase[i] < n) ms[R.tphase[i]] += t;
  }
  if (n_calls > 0) for (int i = 0; i < n; ++i) ms[i] /= (float)n_calls;
  if (calls) *calls = n_calls;
  R.n_tev = 0;
  return B200DNN_SUCCESS;
}

int32_t b200dnn_clear_caches(void) {
  if (device_count() <= 0) return B200DNN_SUCCESS;
  int cur = 0;
  cudaGetDevice(&cur);
  for (int dev = 0; dev < 64; ++dev) {
    DeviceShared *D;
    { std::lock_guard<std::mutex> lk(devices_mu()); D = device_slot(dev); }
    if (!D) continue;
    cudaSetDevice(dev);
    cudaDeviceSynchronize();
    {
      std::lock_guard<std::mutex> lk(D->cache_mu);
      for (auto &kv : D->wcache) { if (kv.second.owned) cudaFree(kv.second.owned); if (kv.second.ready) cudaEventDestroy(kv.second.ready); }
      D->wcache.clear();
      for (auto &kv : D->woq_cache) { if (kv.second.owned) cudaFree(kv.second.owned); if (kv.second.ready) cudaEventDestroy(kv.second.ready); }
      D->woq_cache.clear();
      for (auto &kv : D->host_packed) { if (kv.second.owned) cudaFree(kv.second.owned); if (kv.second.ready) cudaEventDestroy(kv.second.ready); }
      D->host_packed.clear();
      D->packed_registry.clear();
    }
    std::lock_guard<std::mutex> lk(D->ctx_mu);
    for (auto &kv : D->ctxs) { std::lock_guard<std::mutex> lk2(kv.second->mu); kv.second->release_buffers(); }
  }
  cudaSetDevice(cur);
  return B200DNN_SUCCESS;
}

}  // extern "C"

#include "moe_api.cuh"
#include "moe_ep.cuh"
#include "group_api.cuh"
#include "nshard_api.cuh"
#include "norm_api.cuh"
#include "sdpa_api.cuh"
#include "quant_prepack_api.cuh"
