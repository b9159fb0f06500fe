// b200dnn_matmul_static_scratch: the streaming W8A8 GEMM with its split-K scratch in a fixed
// device array instead of library-allocated workspace.
//
// Who needs this: callers that must not trigger a device allocation at call time -- an inference
// server that has handed all remaining device memory to its own pool, a real-time loop where a
// cudaMalloc (which can block behind other work on the device) would break the latency budget, or
// code that runs where allocation is simply not allowed.  b200dnn_matmul grows a workspace with
// cudaMalloc on demand; this entry point never does.  It calls no cudaMalloc / cudaFree / allocating
// library routine, takes only device pointers (nothing is staged) and a weight already written by
// b200dnn_prepack.
//
// The scratch (split-K partial sums + one arrival counter per output tile) lives in the file-scope
// array below: kScratchBytes of device memory held by every GPU that loads this library, from load
// until exit.  Shapes whose split-K scratch would not fit are rejected with an error; nothing is
// truncated.  In host code the array's name is only a handle, not a device address, so the address
// is resolved with cudaGetSymbolAddress once per device (with that device current) on the first
// call made on that device, and that pointer is what the kernel receives.  Because that first call
// does this set-up, make it before starting any stream capture.
//
// All calls share the one array and it keeps whatever the previous call left there.  The partial
// sums need no initial value (every word is written before it is read); the arrival counters must
// start at zero, so each call clears them on the stream before the kernel (the kernel also returns
// them to zero when it finishes).  Two calls that overlap on the GPU (different streams, or
// different host threads using different streams) would race on the array: serialise them.
#include <mutex>

#include "runtime.cuh"
#include "common.cuh"
#include "stream_gemm.cuh"

using namespace b200;

namespace {

constexpr size_t kPartialBytes = size_t(8) << 20;   // split-K partial sums
constexpr int kMaxTiles = 4096;                     // arrival counters
constexpr size_t kScratchBytes = kPartialBytes + kMaxTiles * sizeof(uint32_t);

static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mu;
void *g_scratch_addr[kMaxDevices] = {nullptr};

// Resolves the device address of the scratch array for the current device (once per device).
int32_t scratch_for_current_device(void **out) {
  int dev = -1;
  B2_CUDA(cudaGetDevice(&dev));
  B2_CHECK(dev >= 0 && dev < kMaxDevices, B200DNN_FAILURE, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_setup_mu);
  if (!g_scratch_addr[dev]) {
    void *p = nullptr;
    B2_CUDA(cudaGetSymbolAddress((void **)&p, g_static_scratch));
    B2_CHECK(p != nullptr, B200DNN_FAILURE, "cudaGetSymbolAddress returned a null address");
    // the kernel's dynamic shared memory limit is raised once here as well (not an allocation)
    B2_CUDA(cudaFuncSetAttribute(stream_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    B2_CUDA(cudaFuncSetAttribute(stream_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return B200DNN_SUCCESS;
}

}  // namespace

extern "C" int32_t b200dnn_matmul_static_scratch(const b200dnn_matmul_t *d, void *stream) {
  B2_CHECK(d, B200DNN_FAILURE, "null descriptor");
  B2_CHECK(device_count() > 0, B200DNN_FAILURE, "no CUDA device: libb200dnn has no CPU fallback");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int M = d->M, N = d->N, K = d->K;
  B2_CHECK(d->src && d->weight && d->dst, B200DNN_FAILURE, "null src, weight or dst");
  B2_CHECK(M > 0 && N > 0 && K > 0 && d->lda >= K && d->ldc >= N, B200DNN_FAILURE, "bad shape or leading dimension");
  B2_CHECK(d->wei_format == 'r', B200DNN_UNIMPLEMENTED, "static-scratch matmul takes a prepacked weight (mem_format_b='r') only");
  B2_CHECK(!d->dynamic_quant, B200DNN_UNIMPLEMENTED, "static-scratch matmul does not quantise the source (it would need workspace)");
  B2_CHECK(d->src_dt == B200DNN_S8 || d->src_dt == B200DNN_U8, B200DNN_UNIMPLEMENTED, "source must be s8 or u8");
  B2_CHECK(d->wei_dt == B200DNN_S8, B200DNN_UNIMPLEMENTED, "weights must be s8");
  B2_CHECK(d->dst_dt == B200DNN_BF16 || d->dst_dt == B200DNN_F32 || d->dst_dt == B200DNN_S32, B200DNN_UNIMPLEMENTED, "dst dtype");
  B2_CHECK(d->n_postops >= 0 && d->n_postops <= B200DNN_MAX_POSTOPS, B200DNN_FAILURE, "too many post-ops");
  B2_CHECK(d->src_scale.count == 0 || d->src_scale.count == 1 || d->src_scale.count == M, B200DNN_UNIMPLEMENTED, "src scale granularity");
  B2_CHECK(d->wei_scale.count == 0 || d->wei_scale.count == 1 || d->wei_scale.count == N, B200DNN_UNIMPLEMENTED, "weight scale granularity");
  B2_CHECK((d->src_scale.count == 0 || d->src_scale.buff) && (d->wei_scale.count == 0 || d->wei_scale.buff), B200DNN_FAILURE, "null scale buffer");
  if (d->dst_dt == B200DNN_S32)
    B2_CHECK(d->src_scale.count == 0 && d->wei_scale.count == 0 && !d->bias && d->n_postops == 0, B200DNN_UNIMPLEMENTED,
             "s32 destination returns raw compensated accumulators");
  for (int i = 0; i < d->n_postops; ++i) {
    const int t = d->postops[i].type;
    B2_CHECK(t == PO_RELU || t == PO_LEAKY_RELU || t == PO_GELU_TANH || t == PO_GELU_ERF || t == PO_SIGMOID || t == PO_SWISH ||
             t == PO_TANH || t == PO_ELU || t == PO_CLIP || ((t == PO_BINARY_ADD || t == PO_BINARY_MUL) && d->postops[i].buff),
             B200DNN_UNIMPLEMENTED, "post-op %d", t);
  }

  void *scratch = nullptr;
  B2_TRY(scratch_for_current_device(&scratch));

  // geometry: the same decomposition the allocating path uses, bounded by the fixed scratch
  int sm_count = 148;
  {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  const int64_t Kp = round_up(K, 128), Np = round_up(N, 128);
  StreamGemmArgs g{};
  g.A = reinterpret_cast<const uint8_t *>(d->src); g.lda = d->lda; g.M = M; g.N = N; g.K = K;
  const uint8_t *base = reinterpret_cast<const uint8_t *>(d->weight);
  g.Wt = reinterpret_cast<const int8_t *>(base + kPackHeaderBytes + Np * 4); g.Kp = (int)Kp;
  g.nb = 4; g.kw = 2;
  g.chunks_total = (int)(Kp / 64);
  const int tiles_n = (N + 31) / 32, tiles_m = (M + 15) / 16;
  int ksplit = 1;
  while (tiles_n * tiles_m * ksplit < 2 * sm_count && g.chunks_total / (ksplit * 2) >= 16) ksplit *= 2;
  g.chunks_per_cta = (g.chunks_total + ksplit - 1) / ksplit;
  ksplit = (g.chunks_total + g.chunks_per_cta - 1) / g.chunks_per_cta;
  const int kbytes = g.chunks_per_cta * 64;
  g.a_stride = (int)round_up(kbytes, 128) + 64;
  size_t smem = (size_t)16 * g.a_stride;
  if (smem < 4096) smem = 4096;
  B2_CHECK(smem <= 200 * 1024, B200DNN_FAILURE, "K = %d is too large for the static-scratch kernel", K);
  const size_t tiles = (size_t)tiles_n * tiles_m;
  const size_t need = ksplit > 1 ? tiles * ksplit * 16 * 32 * sizeof(int32_t) : 0;
  B2_CHECK(tiles <= (size_t)kMaxTiles && need <= kPartialBytes, B200DNN_FAILURE,
           "shape M=%d N=%d K=%d needs %zu bytes of split-K scratch in %zu tiles; the static scratch holds %zu bytes and %d tiles",
           M, N, K, need, tiles, kPartialBytes, kMaxTiles);
  g.partial = reinterpret_cast<int32_t *>(scratch);
  g.counters = reinterpret_cast<uint32_t *>(reinterpret_cast<unsigned char *>(scratch) + kPartialBytes);
  // the counters must be zero when the kernel starts, whatever an earlier call left behind
  if (ksplit > 1) B2_CUDA(cudaMemsetAsync(g.counters, 0, tiles * sizeof(uint32_t), st));

  EpiParams e;
  memset(&e, 0, sizeof e);
  e.dst = d->dst; e.ldc = d->ldc; e.dst_dt = d->dst_dt;
  e.src_scale = d->src_scale.count ? d->src_scale.buff : nullptr; e.src_scale_dt = d->src_scale.dt; e.src_scale_n = (int32_t)d->src_scale.count;
  e.wei_scale = d->wei_scale.count ? d->wei_scale.buff : nullptr; e.wei_scale_dt = d->wei_scale.dt; e.wei_scale_n = (int32_t)d->wei_scale.count;
  if (d->src_zp.buff) { e.src_zp = d->src_zp.buff; e.src_zp_dt = d->src_zp.dt; e.has_zp = 1; }
  e.colsum = reinterpret_cast<const int32_t *>(base + kPackHeaderBytes);
  e.bias = d->bias; e.bias_dt = d->bias_dt; e.n_po = d->n_postops;
  for (int i = 0; i < d->n_postops; ++i) {
    e.po[i].type = d->postops[i].type; e.po[i].dt = d->postops[i].dt; e.po[i].buff = d->postops[i].buff;
    e.po[i].ld = d->postops[i].ld; e.po[i].alpha = d->postops[i].alpha; e.po[i].beta = d->postops[i].beta;
  }
  dim3 grid(tiles_n, ksplit, tiles_m);
  if (d->src_dt == B200DNN_U8) stream_gemm_kernel<true><<<grid, 256, smem, st>>>(g, e);
  else stream_gemm_kernel<false><<<grid, 256, smem, st>>>(g, e);
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  return B200DNN_SUCCESS;
}
