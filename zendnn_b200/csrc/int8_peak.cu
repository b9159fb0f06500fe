// b200dnn_measure_int8_peak: the issue-bound rate of tcgen05.mma.kind::i8 on this GPU, the denominator of the
// tensor-pipe roofline of the W8A8 GEMMs.  No reference counterpart (a measurement aid).
//
// One CTA per SM.  The operands (a [128 x 128 B] A block and a [256 x 128 B] B block of pseudo-random bytes: operand
// values decide how much power the multipliers draw, and with it the clock the GPU holds under its power cap) sit in
// shared memory and are never reloaded; one thread issues M128 x N256 x K32 MMAs back to back, alternating between two accumulators in
// tensor memory exactly as the GEMM kernel does, and waits (bounded) for the last one.  Nothing is read from global
// memory, so the time is that of the tensor pipe (and of its shared-memory operand reads) alone.
#include "runtime.cuh"
#include "common.cuh"
#include "tc_gemm.cuh"

using namespace b200;

namespace {

constexpr int kPeakBN = 256;
constexpr int kPeakSmem = kTcBM * kTcBK + kPeakBN * kTcBK + 1024;

__global__ void __launch_bounds__(128, 1) int8_peak_kernel(int iters, int32_t *status, uint32_t *sink) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5;
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *base = smem_raw + (smem0 - smem_u32(smem_raw));
  for (int i = threadIdx.x * 16; i < kTcBM * kTcBK + kPeakBN * kTcBK; i += blockDim.x * 16) {
    uint32_t h = (uint32_t)i * 2654435761u + 0x9E3779B9u * (blockIdx.x + 1);
    uint32_t v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) { h ^= h >> 15; h *= 0x2C1B3C6Du; h ^= h >> 12; h *= 0x297A2D39u; h ^= h >> 15; v[j] = h; }
    *reinterpret_cast<uint4 *>(base + i) = make_uint4(v[0], v[1], v[2], v[3]);
  }
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  bool ok = true;
  if (threadIdx.x == 0) {
    const uint32_t idesc = make_idesc_i8(0, kPeakBN);
    const uint64_t da = make_smem_desc(smem0), db = make_smem_desc(smem0 + kTcBM * kTcBK);
    for (int it = 0; it < iters; ++it) {
      const uint32_t d = tmem_base + (uint32_t)((it & 1) * kPeakBN);
#pragma unroll
      for (int k = 0; k < kTcBK / 32; ++k) tc_mma_i8(d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (it > 1 || k) ? 1u : 0u);
    }
    tc_commit(smem_u32(&bar));
    ok = mbar_wait(smem_u32(&bar), 0);
    if (!ok) report_status(status, 31);
  }
  __syncthreads();
  tc_fence_after();
  if (warp == 0) {
    uint32_t r[32];
    tc_ld32(tmem_base, r);
    tc_wait_ld();
    if (sink) sink[threadIdx.x] = r[0];                  // (no caller passes a sink; the load stays in the program)
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

}  // namespace

// Runs `launches` launches of `iters` K-blocks (4 MMAs of M128 x N256 x K32 each) on every SM, back to back on `stream`,
// and returns the device time of all of them in *ms and the operations they performed in *ops.
extern "C" int32_t b200dnn_measure_int8_peak(int32_t iters, int32_t launches, float *ms, double *ops, void *stream) {
  B2_CHECK(iters > 0 && launches > 0 && ms && ops, B200DNN_FAILURE, "bad argument");
  B2_ENTER(stream);
  Runtime &R = rt();
  B2_CUDA(cudaFuncSetAttribute(int8_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPeakSmem));
  cudaEvent_t e0, e1;
  B2_CUDA(cudaEventCreate(&e0));
  B2_CUDA(cudaEventCreate(&e1));
  int8_peak_kernel<<<R.sm_count, 128, kPeakSmem, st>>>(iters, R.status, nullptr);   // warm-up
  B2_CUDA(cudaEventRecord(e0, st));
  for (int i = 0; i < launches; ++i) int8_peak_kernel<<<R.sm_count, 128, kPeakSmem, st>>>(iters, R.status, nullptr);
  B2_CUDA(cudaEventRecord(e1, st));
  B2_LAUNCHED();
  cudaError_t e = cudaStreamSynchronize(st);
  float t = 0.f;
  if (e == cudaSuccess) e = cudaEventElapsedTime(&t, e0, e1);
  cudaEventDestroy(e0); cudaEventDestroy(e1);
  B2_CUDA(e);
  *ms = t;
  *ops = (double)R.sm_count * launches * iters * (kTcBK / 32) * 2.0 * kTcBM * kPeakBN * 32;
  return read_status();
}
