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
// array below: kScratchBytes of device memory on every GPU that uses this library, held until the
// process exits.  With CUDA's lazy module loading the array is committed when this file's module is
// first loaded on a device, which can be as late as the first call made there: treat the first call
// on each device as a warm-up and make it BEFORE the application's pool takes the remaining memory
// (and before any stream capture).  Shapes whose split-K scratch would not fit are rejected with an
// error; nothing is truncated.  Shapes that are not split use no scratch at all and are never
// rejected for it.  In host code the array's name is only a handle, not a device address, so the address
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
#include "matmul_validate.cuh"
#include "pack_kernels.cuh"
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

// Split of the streaming kernel for one shape on a device with sm_count SMs, and the bytes of the fixed array a launch
// of it would use (0 when the shape is not split: the kernel then touches neither partial sums nor counters).
struct StaticPlan { int tiles_n, tiles_m, ksplit, chunks_total, chunks_per_cta; size_t tiles, need; };
StaticPlan plan_for(int M, int N, int K, int sm_count) {
  StaticPlan p{};
  const int64_t Kp = round_up(K, 128);
  p.chunks_total = (int)(Kp / 64);
  p.tiles_n = (N + 31) / 32; p.tiles_m = (M + 15) / 16;
  int ksplit = 1;
  while ((long long)p.tiles_n * p.tiles_m * ksplit < 2ll * sm_count && p.chunks_total / (ksplit * 2) >= 16) ksplit *= 2;
  p.chunks_per_cta = (p.chunks_total + ksplit - 1) / ksplit;
  p.ksplit = (p.chunks_total + p.chunks_per_cta - 1) / p.chunks_per_cta;
  p.tiles = (size_t)p.tiles_n * p.tiles_m;
  p.need = p.ksplit > 1 ? p.tiles * p.ksplit * 16 * 32 * sizeof(int32_t) : 0;
  return p;
}
bool plan_fits(const StaticPlan &p) { return p.ksplit <= 1 || (p.tiles <= (size_t)kMaxTiles && p.need <= kPartialBytes); }

}  // namespace

// Bytes of the fixed scratch a call of b200dnn_matmul_static_scratch with this shape uses on a device with sm_count
// SMs (0 = the current device), in *bytes (0 for shapes that are not split); failure when the shape does not fit.
// Pure arithmetic with an explicit sm_count, so a caller can size-check its shapes ahead of time.
extern "C" int32_t b200dnn_static_scratch_query(int32_t M, int32_t N, int32_t K, int32_t sm_count, size_t *bytes) {
  B2_CHECK(M > 0 && N > 0 && K > 0 && bytes, B200DNN_FAILURE, "bad argument");
  if (sm_count <= 0) {
    int dev = 0;
    B2_CHECK(device_count() > 0, B200DNN_FAILURE, "no CUDA device and no sm_count given");
    B2_CUDA(cudaGetDevice(&dev));
    B2_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  const StaticPlan p = plan_for(M, N, K, sm_count);
  *bytes = p.need + (p.ksplit > 1 ? p.tiles * sizeof(uint32_t) : 0);
  B2_CHECK(plan_fits(p), B200DNN_FAILURE,
           "shape M=%d N=%d K=%d needs %zu bytes of split-K scratch in %zu tiles; the static scratch holds %zu bytes and %d tiles",
           M, N, K, p.need, p.tiles, kPartialBytes, kMaxTiles);
  return B200DNN_SUCCESS;
}

extern "C" int32_t b200dnn_matmul_static_scratch(const b200dnn_matmul_t *d, void *stream) {
  B2_CHECK(d, B200DNN_FAILURE, "null descriptor");
  B2_CHECK(device_count() > 0, B200DNN_FAILURE, "no CUDA device: libb200dnn has no CPU fallback");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int M = d->M, N = d->N, K = d->K;
  // the contract of b200dnn_matmul, then what this entry point leaves out
  B2_TRY(validate_matmul_desc(d));
  B2_CHECK(!d->transA, B200DNN_UNIMPLEMENTED, "a transposed source needs a workspace pass: use b200dnn_matmul");
  B2_CHECK(d->dst_dt != B200DNN_S8 && d->dst_dt != B200DNN_U8, B200DNN_UNIMPLEMENTED,
           "requantised s8/u8 destinations need a workspace pass: use b200dnn_matmul");
  B2_CHECK(d->wei_format == 'r', B200DNN_UNIMPLEMENTED, "static-scratch matmul takes a prepacked weight (mem_format_b='r') only");
  B2_CHECK(!d->dynamic_quant, B200DNN_UNIMPLEMENTED, "static-scratch matmul does not quantise the source (it would need workspace)");
  // nothing is staged: a host pointer would go straight into the kernel and fault the GPU (classifying a pointer allocates nothing)
  B2_CHECK(is_device_ptr(d->src) && is_device_ptr(d->weight) && is_device_ptr(d->dst), B200DNN_FAILURE,
           "static-scratch matmul takes device pointers only (src, weight, dst)");
  B2_CHECK((d->src_scale.count == 0 || is_device_ptr(d->src_scale.buff)) && (d->wei_scale.count == 0 || is_device_ptr(d->wei_scale.buff)) &&
           (!d->src_zp.buff || is_device_ptr(d->src_zp.buff)) && (!d->bias || is_device_ptr(d->bias)), B200DNN_FAILURE,
           "static-scratch matmul takes device pointers only (scales, zero-point, bias)");
  for (int i = 0; i < d->n_postops; ++i)
    if (d->postops[i].type == PO_BINARY_ADD || d->postops[i].type == PO_BINARY_MUL)
      B2_CHECK(is_device_ptr(d->postops[i].buff), B200DNN_FAILURE, "static-scratch matmul takes device pointers only (post-op %d operand)", i);

  // the weight must be a buffer that b200dnn_prepack wrote for this K and N, plain (not the gate/up interleaved) form:
  // looked up in the host-side registry of packed buffers, else its header is read once (a 256-byte copy; no allocation)
  DeviceShared *D = nullptr;
  B2_TRY(device_shared(&D));
  PackedWeight pw;
  {
    std::lock_guard<std::mutex> lk(D->cache_mu);
    auto it = D->packed_registry.find(d->weight);
    if (it == D->packed_registry.end()) {
      PackHeader h;
      B2_CUDA(cudaMemcpyAsync(&h, d->weight, sizeof h, cudaMemcpyDeviceToHost, st));
      B2_CUDA(cudaStreamSynchronize(st));
      B2_CHECK(h.magic == kPackMagic, B200DNN_FAILURE, "the weight buffer was not written by b200dnn_prepack");
      PackedWeight v;
      const uint8_t *b = reinterpret_cast<const uint8_t *>(d->weight);
      v.colsum = reinterpret_cast<const int32_t *>(b + kPackHeaderBytes);
      v.wt = reinterpret_cast<const int8_t *>(b + kPackHeaderBytes + h.Np * 4);
      v.K = h.K; v.N = h.N; v.Kp = h.Kp; v.Np = h.Np; v.gated = h.gated; v.I = h.I;
      it = D->packed_registry.emplace(d->weight, v).first;
    }
    pw = it->second;
  }
  B2_CHECK(pw.K == K && pw.N == N && pw.gated == 0, B200DNN_FAILURE,
           "prepacked weight is K=%lld N=%lld gated=%d, call asks for K=%d N=%d plain", (long long)pw.K, (long long)pw.N, pw.gated, K, N);

  void *scratch = nullptr;
  B2_TRY(scratch_for_current_device(&scratch));

  // geometry: the same decomposition the allocating path uses, bounded by the fixed scratch when the shape is split
  const StaticPlan pl = plan_for(M, N, K, D->sm_count);
  StreamGemmArgs g{};
  g.A = reinterpret_cast<const uint8_t *>(d->src); g.lda = d->lda; g.M = M; g.N = N; g.K = K;
  g.Wt = pw.wt; g.Kp = (int)pw.Kp;
  g.nb = 4; g.kw = 2;
  g.chunks_total = pl.chunks_total; g.chunks_per_cta = pl.chunks_per_cta;
  const int ksplit = pl.ksplit;
  const int kbytes = g.chunks_per_cta * 64;
  g.a_stride = (int)round_up(kbytes, 128) + 64;
  size_t smem = (size_t)16 * g.a_stride;
  if (smem < 4096) smem = 4096;
  B2_CHECK(smem <= 200 * 1024, B200DNN_FAILURE, "K = %d is too large for the static-scratch kernel", K);
  B2_CHECK(plan_fits(pl), B200DNN_FAILURE,
           "shape M=%d N=%d K=%d needs %zu bytes of split-K scratch in %zu tiles; the static scratch holds %zu bytes and %d tiles",
           M, N, K, pl.need, pl.tiles, kPartialBytes, kMaxTiles);
  if (ksplit > 1) {
    g.partial = reinterpret_cast<int32_t *>(scratch);
    g.counters = reinterpret_cast<uint32_t *>(reinterpret_cast<unsigned char *>(scratch) + kPartialBytes);
    // the counters must be zero when the kernel starts, whatever an earlier call left behind
    B2_CUDA(cudaMemsetAsync(g.counters, 0, pl.tiles * sizeof(uint32_t), st));
  }

  EpiParams e;
  memset(&e, 0, sizeof e);
  e.dst = d->dst; e.ldc = d->ldc; e.dst_dt = d->dst_dt;
  e.src_scale = d->src_scale.count ? d->src_scale.buff : nullptr; e.src_scale_dt = d->src_scale.dt; e.src_scale_n = (int32_t)d->src_scale.count;
  e.wei_scale = d->wei_scale.count ? d->wei_scale.buff : nullptr; e.wei_scale_dt = d->wei_scale.dt; e.wei_scale_n = (int32_t)d->wei_scale.count;
  if (d->src_zp.buff) { e.src_zp = d->src_zp.buff; e.src_zp_dt = d->src_zp.dt; e.has_zp = 1; }
  e.colsum = pw.colsum;
  e.bias = d->bias; e.bias_dt = d->bias_dt; e.n_po = d->n_postops;
  for (int i = 0; i < d->n_postops; ++i) {
    e.po[i].type = d->postops[i].type; e.po[i].dt = d->postops[i].dt; e.po[i].buff = d->postops[i].buff;
    e.po[i].ld = d->postops[i].ld; e.po[i].alpha = d->postops[i].alpha; e.po[i].beta = d->postops[i].beta;
  }
  dim3 grid(pl.tiles_n, ksplit, pl.tiles_m);
  if (d->src_dt == B200DNN_U8) stream_gemm_kernel<true><<<grid, 256, smem, st>>>(g, e);
  else stream_gemm_kernel<false><<<grid, 256, smem, st>>>(g, e);
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  return B200DNN_SUCCESS;
}
