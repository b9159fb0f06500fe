// Host-side runtime of libb200dnn: error text, pointer classification, device workspace,
// the packed-weight cache (the counterpart of the reference's weight-reorder LRU keyed by the
// weight address, matmul/backends/aocl/aocl_kernel.cpp:237-307 and matmul/lru_cache/zendnnl_key.hpp:28-75)
// and the TMA descriptor encoder.
#pragma once
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include <atomic>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <tuple>
#include <vector>

#include "../../include/b200dnn.h"
#include "pack_kernels.cuh"

namespace b200 {

inline std::string &err_text() { static thread_local std::string s; return s; }
inline int32_t fail(int32_t code, const char *fmt, ...) {
  char buf[512];
  va_list ap; va_start(ap, fmt); vsnprintf(buf, sizeof buf, fmt, ap); va_end(ap);
  err_text() = buf;
  if (const char *e = getenv("ZENDNNL_API_LOG_LEVEL")) if (atoi(e) > 0) fprintf(stderr, "[b200dnn] %s\n", buf);
  return code;
}
#define B2_CUDA(expr)                                                                              \
  do { cudaError_t e__ = (expr);                                                                   \
    if (e__ != cudaSuccess) return fail(B200DNN_FAILURE, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, __LINE__); \
  } while (0)
#define B2_CHECK(cond, code, ...) do { if (!(cond)) return fail(code, __VA_ARGS__); } while (0)
#define B2_TRY(expr) do { int32_t rc__ = (expr); if (rc__ != B200DNN_SUCCESS) return rc__; } while (0)

inline std::atomic<int64_t> &launch_counter() { static std::atomic<int64_t> c{0}; return c; }
#define B2_LAUNCHED() (++b200::launch_counter())

inline int device_count() {
  static int n = [] { int c = 0; if (cudaGetDeviceCount(&c) != cudaSuccess) { cudaGetLastError(); c = 0; } return c; }();
  return n;
}

inline bool is_device_ptr(const void *p) {
  if (!p) return false;
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) { cudaGetLastError(); return false; }
  return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
}

// Allocations made while the calling thread captures a stream into a CUDA graph (a first call on a new stream, a
// workspace that has to grow): the capture mode is relaxed for the duration of the allocation, which is not part of
// the captured work.
struct RelaxedCapture {
  cudaStreamCaptureMode mode = cudaStreamCaptureModeRelaxed;
  RelaxedCapture() { if (cudaThreadExchangeStreamCaptureMode(&mode) != cudaSuccess) cudaGetLastError(); }
  ~RelaxedCapture() { if (cudaThreadExchangeStreamCaptureMode(&mode) != cudaSuccess) cudaGetLastError(); }
};

// ---- workspace: bump allocator over device blocks, rewound at the start of every API call -------
struct Workspace {
  struct Block { uint8_t *p; size_t cap, used; };
  std::vector<Block> blocks;
  void rewind() { for (auto &b : blocks) b.used = 0; }
  void *alloc(size_t bytes) {
    bytes = (bytes + 255) & ~size_t(255);
    if (bytes == 0) bytes = 256;
    for (auto &b : blocks)
      if (b.cap - b.used >= bytes) { void *r = b.p + b.used; b.used += bytes; return r; }
    size_t cap = bytes > (size_t(64) << 20) ? bytes : (size_t(64) << 20);
    void *p = nullptr;
    RelaxedCapture relaxed;
    if (cudaMalloc(&p, cap) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    blocks.push_back({(uint8_t *)p, cap, bytes});
    return p;
  }
  void release() { for (auto &b : blocks) cudaFree(b.p); blocks.clear(); }
  // a call that repeats a sub-step (one attention head after the other) gives the sub-step's allocations back: work on one
  // stream is ordered, so the next sub-step may write where the previous one has read
  std::vector<size_t> mark() const { std::vector<size_t> m; for (auto &b : blocks) m.push_back(b.used); return m; }
  void restore(const std::vector<size_t> &m) { for (size_t i = 0; i < blocks.size(); ++i) blocks[i].used = i < m.size() ? m[i] : 0; }
};

struct PackedWeight {
  const int32_t *colsum = nullptr;
  const int8_t *wt = nullptr;
  int64_t K = 0, N = 0, Kp = 0, Np = 0;
  int gated = 0; int64_t I = 0;
  void *owned = nullptr;   // cache-owned device buffer
  // cache-owned buffers are packed on the stream of the call that first saw the weight; calls on other streams wait
  // for this event until it has been seen complete once
  cudaEvent_t ready = nullptr; cudaStream_t ready_stream = nullptr; bool complete = true;
};

// Small host inputs of one call (activations of a decode step, scales, zero point, bias, descriptor tables) are
// gathered into one pinned block and sent with as few copies as possible: every separate copy costs a few
// microseconds of enqueue time, and a pinned source lets the call return without waiting for the copy.
struct SmallBatch {
  static constexpr size_t kCap = 1 << 20, kMaxItem = 256 << 10, kBatchItem = 16 << 10;
  uint8_t *pinned = nullptr, *dev = nullptr;
  size_t used = 0, sent = 0;
  cudaEvent_t ev = nullptr; bool in_flight = false;   // the last copy may still be reading `pinned`
  void begin() {
    if (in_flight) { cudaEventSynchronize(ev); in_flight = false; }
    used = sent = 0;
  }
  // returns the device address the bytes will have after flush(), or nullptr when they do not fit
  void *add(const void *p, size_t bytes, size_t max_item = kBatchItem) {
    const size_t room = (bytes + 255) & ~size_t(255);
    if (!pinned || bytes > max_item || used + room > kCap) return nullptr;
    memcpy(pinned + used, p, bytes);
    void *d = dev + used; used += room;
    return d;
  }
  // will_sync: the caller drains the stream before it returns, so no event is needed to protect `pinned`
  int32_t flush(cudaStream_t st, bool will_sync) {
    if (used == sent) return B200DNN_SUCCESS;
    B2_CUDA(cudaMemcpyAsync(dev + sent, pinned + sent, used - sent, cudaMemcpyHostToDevice, st));
    sent = used;
    if (!will_sync) { B2_CUDA(cudaEventRecord(ev, st)); in_flight = true; }
    return B200DNN_SUCCESS;
  }
  void release() {
    if (ev) { cudaEventSynchronize(ev); cudaEventDestroy(ev); ev = nullptr; }
    if (pinned) { cudaFreeHost(pinned); pinned = nullptr; }
    if (dev) { cudaFree(dev); dev = nullptr; }
    in_flight = false; used = sent = 0;
  }
};

struct Runtime;

// State shared by every stream of one device: the weight caches (mutex-protected, as the reference's are:
// matmul/backends/aocl/aocl_kernel.cpp:349,394) and per-device facts.
struct DeviceShared {
  int dev = -1, sm_count = 0;
  PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
  std::mutex cache_mu;
  std::map<std::tuple<const void *, int64_t, int64_t, int64_t, int, int>, PackedWeight> wcache;
  // 4-bit weights dequantised to bf16 at pack time: the scale and zero-point buffers are part of the identity
  std::map<std::tuple<const void *, const void *, const void *, int64_t, int64_t, int64_t, int, int>, PackedWeight> woq_cache;
  std::map<const void *, PackedWeight> packed_registry;   // buffers written by b200dnn_prepack (device address)
  std::map<const void *, PackedWeight> host_packed;       // host-resident prepacked buffers uploaded once
  std::mutex ctx_mu;
  std::map<cudaStream_t, Runtime *> ctxs;
  std::mutex attr_mu;
  std::map<const void *, int> smem_limit;                 // kernels whose dynamic shared-memory limit was raised
  int split_room[5] = {0, 0, 0, 0, 0};
};

// Descriptor tables that depend only on the caller's weight pointers (per-expert epilogue pointers, tensor maps) are
// kept on the device and found again by their bytes, so that a steady-state MoE call uploads nothing.
struct BlobCache {
  struct Entry { std::vector<uint8_t> bytes; void *dev; };
  std::vector<Entry> entries;
  void *find(const void *host, size_t n) const {
    for (const Entry &e : entries)
      if (e.bytes.size() == n && memcmp(e.bytes.data(), host, n) == 0) return e.dev;
    return nullptr;
  }
  void release() { for (Entry &e : entries) cudaFree(e.dev); entries.clear(); }
};

// Everything a call touches besides the weight caches: one per (device, stream).  Calls on different streams (from
// different host threads) share nothing here; calls on one stream are serialised by `mu` and by the stream itself.
struct Runtime {
  std::mutex mu;
  DeviceShared *shared = nullptr;
  cudaStream_t stream = nullptr;
  Workspace ws;
  SmallBatch small;
  BlobCache blobs;
  uint8_t *slab = nullptr; size_t slab_cap = 0;           // pinned staging for large gathered host inputs
  uint32_t *counters = nullptr; size_t n_counters = 0;   // split-K tile counters, kept zero between launches
  int32_t *status = nullptr;                              // status word the kernels write: device view of mapped pinned memory
  volatile int32_t *status_host = nullptr;                // host view of the same word
  PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
  int sm_count = 0;
  // optional per-phase device times of the MoE entry points (b200dnn_phase_timing): events on this stream
  bool timing = false;
  std::vector<cudaEvent_t> tev; std::vector<int> tphase; size_t n_tev = 0;
  // mark(p): phase p ends here; mark(-1): a timed call starts
  void mark(int phase) {
    if (!timing || n_tev >= 65536) return;     // every call since timing was switched on keeps its own events
    if (n_tev == tev.size()) {
      cudaEvent_t e = nullptr;
      if (cudaEventCreate(&e) != cudaSuccess) { cudaGetLastError(); return; }
      tev.push_back(e); tphase.push_back(0);
    }
    tphase[n_tev] = phase;
    cudaEventRecord(tev[n_tev], stream);
    ++n_tev;
  }

  int32_t init(DeviceShared *sh, cudaStream_t st) {
    shared = sh; stream = st; encode = sh->encode; sm_count = sh->sm_count;
    n_counters = 1 << 16;
    RelaxedCapture relaxed;     // the first call on a stream may come while that stream is being captured
    B2_CUDA(cudaMalloc(&counters, n_counters * sizeof(uint32_t)));
    {
      // zeroed on a stream of its own: the legacy default stream must not be touched during a capture
      cudaStream_t tmp = nullptr;
      B2_CUDA(cudaStreamCreateWithFlags(&tmp, cudaStreamNonBlocking));
      cudaError_t e = cudaMemsetAsync(counters, 0, n_counters * sizeof(uint32_t), tmp);
      if (e == cudaSuccess) e = cudaStreamSynchronize(tmp);
      cudaStreamDestroy(tmp);
      B2_CUDA(e);
    }
    void *h = nullptr, *d = nullptr;
    B2_CUDA(cudaHostAlloc(&h, 256, cudaHostAllocMapped));
    memset(h, 0, 256);
    B2_CUDA(cudaHostGetDevicePointer(&d, h, 0));
    status_host = (volatile int32_t *)h; status = (int32_t *)d;
    B2_CUDA(cudaMallocHost(&small.pinned, SmallBatch::kCap));
    B2_CUDA(cudaMalloc(&small.dev, SmallBatch::kCap));
    B2_CUDA(cudaEventCreateWithFlags(&small.ev, cudaEventDisableTiming));
    return B200DNN_SUCCESS;
  }
  uint8_t *pinned_slab(size_t bytes) {
    if (bytes > slab_cap) {
      if (slab) cudaFreeHost(slab);
      slab = nullptr; slab_cap = 0;
      if (cudaMallocHost(&slab, bytes) != cudaSuccess) { cudaGetLastError(); return nullptr; }
      slab_cap = bytes;
    }
    return slab;
  }
  void release_buffers() { ws.release(); blobs.release(); if (slab) { cudaFreeHost(slab); slab = nullptr; slab_cap = 0; } }
};

inline std::mutex &devices_mu() { static std::mutex m; return m; }
inline DeviceShared *&device_slot(int dev) { static DeviceShared *slots[64] = {nullptr}; return slots[dev]; }

// State of the CURRENT device (created at the first call made with that device current).  A call never touches
// another device's buffers: which state it gets is decided by cudaGetDevice at its start.
inline int32_t device_shared(DeviceShared **out) {
  B2_CHECK(device_count() > 0, B200DNN_FAILURE, "no CUDA device: libb200dnn has no CPU fallback");
  int dev = 0;
  B2_CUDA(cudaGetDevice(&dev));
  B2_CHECK(dev >= 0 && dev < 64, B200DNN_FAILURE, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(devices_mu());
  DeviceShared *&slot = device_slot(dev);
  if (!slot) {
    cudaDeviceProp prop;
    B2_CUDA(cudaGetDeviceProperties(&prop, dev));
    B2_CHECK(prop.major == 10, B200DNN_FAILURE, "device is sm_%d%d; this library is built for sm_100a only", prop.major, prop.minor);
    void *fn = nullptr; cudaDriverEntryPointQueryResult qres;
    B2_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    B2_CHECK(fn && qres == cudaDriverEntryPointSuccess, B200DNN_FAILURE, "cuTensorMapEncodeTiled not available from the driver");
    DeviceShared *sh = new DeviceShared();
    sh->dev = dev; sh->sm_count = prop.multiProcessorCount; sh->encode = (PFN_cuTensorMapEncodeTiled_v12000)fn;
    slot = sh;
  }
  *out = slot;
  return B200DNN_SUCCESS;
}

inline Runtime *&current_rt() { static thread_local Runtime *r = nullptr; return r; }
// The context of the call in progress on this thread (set by CallGuard).
inline Runtime &rt() { return *current_rt(); }

// Entered at the top of every C-ABI entry point: finds (or creates) the context of (current device, stream), takes its
// lock for the duration of the call and rewinds its workspace.
struct CallGuard {
  Runtime *r = nullptr, *prev = nullptr;
  int32_t enter(cudaStream_t st) {
    DeviceShared *sh = nullptr;
    B2_TRY(device_shared(&sh));
    {
      std::lock_guard<std::mutex> lk(sh->ctx_mu);
      auto it = sh->ctxs.find(st);
      if (it == sh->ctxs.end()) {
        Runtime *n = new Runtime();
        int32_t rc = n->init(sh, st);
        if (rc != B200DNN_SUCCESS) { delete n; return rc; }
        it = sh->ctxs.emplace(st, n).first;
      }
      r = it->second;
    }
    r->mu.lock();
    prev = current_rt(); current_rt() = r;
    r->ws.rewind();
    r->small.begin();
    return B200DNN_SUCCESS;
  }
  ~CallGuard() { if (r) { current_rt() = prev; r->mu.unlock(); } }
};
#define B2_ENTER(stream_ptr)                                       \
  b200::CallGuard guard__;                                         \
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_ptr);    \
  B2_TRY(guard__.enter(st))

// After the stream has been drained: did a kernel of this context give up on one of its bounded waits since the last
// check?  The kernels write the code into mapped pinned memory, so the check is one host load.
inline int32_t read_status() {
  Runtime &R = rt();
  const int32_t code = *R.status_host;
  if (code != 0) {
    *R.status_host = 0;
    return fail(B200DNN_FAILURE, "a GEMM kernel gave up waiting on a barrier (code %d)", code);
  }
  return B200DNN_SUCCESS;
}

// Sends a host table to workspace memory without waiting for the copy: it travels through the call's pinned block.
// Tables too large for the block are copied synchronously.
inline int32_t upload_blob(const void *host, size_t bytes, cudaStream_t st, void **dev) {
  Runtime &R = rt();
  if (void *d = R.small.add(host, bytes, SmallBatch::kMaxItem)) {
    B2_TRY(R.small.flush(st, false));
    *dev = d;
    return B200DNN_SUCCESS;
  }
  void *d = R.ws.alloc(bytes);
  B2_CHECK(d, B200DNN_FAILURE, "workspace allocation failed");
  B2_CUDA(cudaMemcpyAsync(d, host, bytes, cudaMemcpyHostToDevice, st));
  B2_CUDA(cudaStreamSynchronize(st));
  *dev = d;
  return B200DNN_SUCCESS;
}
// The same for tables that depend only on the caller's weight pointers: kept on the device and found again by their
// bytes, so a repeated call uploads nothing.
inline int32_t cached_blob(const void *host, size_t bytes, cudaStream_t st, void **dev) {
  Runtime &R = rt();
  if (void *d = R.blobs.find(host, bytes)) { *dev = d; return B200DNN_SUCCESS; }
  if (R.blobs.entries.size() >= 256) {      // bounded: start again (nothing in flight may still read the old tables)
    B2_CUDA(cudaStreamSynchronize(st));
    R.blobs.release();
  }
  void *d = nullptr;
  {
    RelaxedCapture relaxed;
    B2_CUDA(cudaMalloc(&d, bytes ? bytes : 16));
  }
  B2_CUDA(cudaMemcpyAsync(d, host, bytes, cudaMemcpyHostToDevice, st));
  B2_CUDA(cudaStreamSynchronize(st));
  BlobCache::Entry e; e.bytes.assign((const uint8_t *)host, (const uint8_t *)host + bytes); e.dev = d;
  R.blobs.entries.push_back(std::move(e));
  *dev = d;
  return B200DNN_SUCCESS;
}

// 2-D uint8 tensor map [rows][row_bytes used of pitch] with a [box_rows x 128 B] box, SWIZZLE_128B.
inline int32_t make_map_2d(CUtensorMap *m, const void *base, uint64_t inner_bytes, uint64_t rows, uint64_t pitch_bytes, uint32_t box_rows) {
  B2_CHECK((reinterpret_cast<uintptr_t>(base) & 15) == 0 && pitch_bytes % 16 == 0, B200DNN_FAILURE,
           "TMA operand must be 16-byte aligned with a 16-byte multiple pitch");
  cuuint64_t dims[2] = {inner_bytes, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = rt().encode(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B2_CHECK(r == CUDA_SUCCESS, B200DNN_FAILURE, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return B200DNN_SUCCESS;
}

// 2-D byte map over a row-major destination for TMA stores of [32 rows x 32 bytes] blocks (no swizzle).
inline int32_t make_map_store(CUtensorMap *m, void *base, uint64_t row_bytes, uint64_t rows, uint64_t pitch_bytes) {
  B2_CHECK((reinterpret_cast<uintptr_t>(base) & 15) == 0 && pitch_bytes % 16 == 0 && row_bytes >= 32, B200DNN_FAILURE,
           "TMA store destination must be 16-byte aligned with a 16-byte multiple pitch");
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = rt().encode(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B2_CHECK(r == CUDA_SUCCESS, B200DNN_FAILURE, "cuTensorMapEncodeTiled (store) failed with %d", (int)r);
  return B200DNN_SUCCESS;
}

// 4-D uint8 tensor map over a block-interleaved packed weight Wt[Np/8][Kp/128][8][128] (pack_kernels.cuh).
// Dimensions, innermost first: 128 bytes of K, 8 rows of a group, Kp/128 K-blocks, Np/8 groups.  The box
// {128, 8, 1, box_rows/8} lands in shared memory as box_rows consecutive 128-byte rows (SWIZZLE_128B).
inline int32_t make_map_wt(CUtensorMap *m, const void *wt, uint64_t Kp, uint64_t Np, uint32_t box_rows) {
  B2_CHECK((reinterpret_cast<uintptr_t>(wt) & 15) == 0 && Kp % 128 == 0 && Np % 8 == 0 && box_rows % 8 == 0, B200DNN_FAILURE,
           "packed weight is not laid out for TMA");
  cuuint64_t dims[4] = {128, 8, Kp / 128, Np / 8};
  cuuint64_t strides[3] = {128, 1024, Kp * 8};
  cuuint32_t box[4] = {128, 8, 1, box_rows / 8};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = rt().encode(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(wt), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B2_CHECK(r == CUDA_SUCCESS, B200DNN_FAILURE, "cuTensorMapEncodeTiled (weight) failed with %d", (int)r);
  return B200DNN_SUCCESS;
}

// One host-or-device buffer made visible on the device for the duration of a call.
struct Staged {
  void *dev = nullptr; void *host = nullptr; size_t bytes = 0; bool copy_back = false;
  bool sync = false;   // written in place in pinned host memory: the stream must be drained before returning
};
// batch: small host inputs join the call's SmallBatch (the caller flushes it before its first launch).
inline int32_t stage_in(const void *p, size_t bytes, cudaStream_t st, const void **out, SmallBatch *batch = nullptr) {
  if (!p || bytes == 0) { *out = p; return B200DNN_SUCCESS; }
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) { cudaGetLastError(); at.type = cudaMemoryTypeUnregistered; }
  if (at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged) { *out = p; return B200DNN_SUCCESS; }
  if (batch)
    if (void *d = batch->add(p, bytes)) { *out = d; return B200DNN_SUCCESS; }
  // (Reading small pinned inputs in place over the bus was measured slower: every CTA of the GEMM re-reads them.)
  void *d = rt().ws.alloc(bytes);
  B2_CHECK(d, B200DNN_FAILURE, "workspace allocation of %zu bytes failed", bytes);
  B2_CUDA(cudaMemcpyAsync(d, p, bytes, cudaMemcpyHostToDevice, st));
  *out = d;
  return B200DNN_SUCCESS;
}
// Output buffer: device pointer is used as is; a host pointer gets a workspace twin that finish() copies back.
// preload: the kernel updates the buffer (in-place ops) so its current contents are needed too.
inline int32_t stage_out(void *p, size_t bytes, cudaStream_t st, Staged *s, bool preload = false) {
  s->host = nullptr; s->dev = p; s->bytes = bytes; s->copy_back = false; s->sync = false;
  if (!p || bytes == 0) return B200DNN_SUCCESS;
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) { cudaGetLastError(); at.type = cudaMemoryTypeUnregistered; }
  if (at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged) return B200DNN_SUCCESS;
  // Small results go straight into pinned host memory from the kernel's own stores (each element crosses the
  // bus once, no separate copy is enqueued); larger ones, and pageable memory, use a device twin and one copy.
  if (at.type == cudaMemoryTypeHost && at.devicePointer && bytes <= (size_t(1) << 20) && !preload) {
    s->host = p; s->dev = at.devicePointer; s->sync = true;
    return B200DNN_SUCCESS;
  }
  void *d = rt().ws.alloc(bytes);
  B2_CHECK(d, B200DNN_FAILURE, "workspace allocation of %zu bytes failed", bytes);
  if (preload) B2_CUDA(cudaMemcpyAsync(d, p, bytes, cudaMemcpyHostToDevice, st));
  s->host = p; s->dev = d; s->copy_back = true;
  return B200DNN_SUCCESS;
}
inline int32_t finish_out(std::initializer_list<Staged *> outs, cudaStream_t st) {
  bool any = false;
  for (Staged *s : outs)
    if (s->copy_back) { B2_CUDA(cudaMemcpyAsync(s->host, s->dev, s->bytes, cudaMemcpyDeviceToHost, st)); any = true; }
    else if (s->sync) any = true;
  if (any) {
    B2_CUDA(cudaStreamSynchronize(st));   // (polling cudaStreamQuery instead was measured 4 us slower per call; spinning on a pinned flag written by a stream-ordered cuStreamWriteValue32 was no faster)
    return read_status();
  }
  return B200DNN_SUCCESS;
}

inline size_t dt_size(int32_t dt) {
  switch (dt) { case B200DNN_F32: case B200DNN_S32: return 4; case B200DNN_BF16: return 2; case B200DNN_S8: case B200DNN_U8: return 1; default: return 0; }
}
inline size_t span_bytes(int64_t rows, int64_t cols, int64_t ld, int32_t dt) {
  if (rows <= 0 || cols <= 0) return 0;
  return (size_t)((rows - 1) * ld + cols) * dt_size(dt);
}

}  // namespace b200
