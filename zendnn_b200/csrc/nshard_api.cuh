// N-column sharding of one large matmul_direct over the GPUs of a node (one process per GPU).  No counterpart in the
// reference (one process on one CPU; the closest is its N-tiling of grouped GEMMs,
// lowoha_operators/matmul/group_matmul/n_tile/group_matmul_n_tile.cpp).  Rank r computes the column block
// [n0, n1) of C from its column block of the weight, the matching slices of the weight scales, the bias and the binary
// post-op operands, and the whole (replicated) A: no reduction, so the s32 sums stay exact and every output element is the
// one a single GPU computes.  A GEMM is only split when it is wide enough (N >= 8 tiles of 256 columns); narrower ones
// run whole on every rank.  Optionally the column blocks are gathered so that every rank holds the full C
// (ncclAllGather of packed blocks, then strided copies into C).  Included at the end of b200dnn.cu.
#pragma once

namespace {

constexpr int kNshardTile = 256;

struct NshardCtx {
  int world = 1, rank = 0, device = 0;
  ncclComm_t comm = nullptr;
  bool own_comm = false;
  void *stage = nullptr; size_t stage_bytes = 0;     // gather staging: [world][M][widest block]
};

// columns of rank r: whole 128-column tiles dealt as evenly as possible; `sharded` = 0 when the GEMM is too narrow to split
inline void nshard_range(int64_t N, int world, int rank, int64_t *n0, int64_t *n1, int *sharded) {
  if (world <= 1 || N < (int64_t)8 * kNshardTile) { *n0 = 0; *n1 = N; if (sharded) *sharded = 0; return; }
  const int64_t tiles = (N + 127) / 128, base = tiles / world, extra = tiles % world;
  const int64_t t0 = rank * base + (rank < extra ? rank : extra), t1 = t0 + base + (rank < extra ? 1 : 0);
  *n0 = t0 * 128 < N ? t0 * 128 : N;
  *n1 = t1 * 128 < N ? t1 * 128 : N;
  if (sharded) *sharded = 1;
}

}  // namespace

extern "C" {

int32_t b200dnn_nshard_range(int64_t N, int32_t world, int32_t rank, int64_t *n0, int64_t *n1, int32_t *sharded) {
  B2_CHECK(N > 0 && world >= 1 && rank >= 0 && rank < world && n0 && n1, B200DNN_FAILURE, "nshard_range: bad argument");
  int s = 0;
  nshard_range(N, world, rank, n0, n1, &s);
  if (sharded) *sharded = s;
  return B200DNN_SUCCESS;
}

int32_t b200dnn_nshard_create(int32_t world, int32_t rank, const void *id128, void *nccl_comm, void **handle) {
  B2_CHECK(handle && world >= 1 && world <= 8 && rank >= 0 && rank < world, B200DNN_FAILURE, "nshard_create: bad argument");
  NshardCtx *c = new NshardCtx();
  c->world = world; c->rank = rank;
  if (cudaGetDevice(&c->device) != cudaSuccess) { delete c; return fail(B200DNN_FAILURE, "no CUDA device"); }
  if (world > 1 && (id128 || nccl_comm)) {
    NcclApi *api = nullptr;
    int32_t rc = nccl_api(&api);
    if (rc != B200DNN_SUCCESS) { delete c; return rc; }
    if (nccl_comm) c->comm = (ncclComm_t)nccl_comm;
    else {
      ncclUniqueId id; memcpy(&id, id128, sizeof id);
      ncclResult_t r = api->CommInitRank(&c->comm, world, id, rank);
      if (r != ncclSuccess) { delete c; return fail(B200DNN_FAILURE, "ncclCommInitRank failed: %s", api->GetErrorString(r)); }
      c->own_comm = true;
    }
  }
  *handle = c;
  return B200DNN_SUCCESS;
}

int32_t b200dnn_nshard_destroy(void *handle) {
  NshardCtx *c = (NshardCtx *)handle;
  if (!c) return B200DNN_SUCCESS;
  if (c->stage) cudaFree(c->stage);
  if (c->own_comm && c->comm) { NcclApi *api = nullptr; if (nccl_api(&api) == B200DNN_SUCCESS) api->CommDestroy(c->comm); }
  delete c;
  return B200DNN_SUCCESS;
}

// desc describes the WHOLE problem (as for b200dnn_matmul, weights in the caller's layout); this rank computes its column
// block of dst.  gather != 0: afterwards every rank holds the whole dst (device memory; needs the communicator).
int32_t b200dnn_matmul_nshard(void *handle, const b200dnn_matmul_t *desc, int32_t gather, void *stream) {
  NshardCtx *c = (NshardCtx *)handle;
  B2_CHECK(c && desc, B200DNN_FAILURE, "matmul_nshard: null argument");
  int64_t n0, n1; int sharded;
  nshard_range(desc->N, c->world, c->rank, &n0, &n1, &sharded);
  if (!sharded) return b200dnn_matmul(desc, stream);          // too narrow to split: every rank computes all of it
  B2_CHECK(desc->wei_format == 'n' || desc->wei_format == 0, B200DNN_UNIMPLEMENTED,
           "matmul_nshard slices weights in the caller's layout; prepack this rank's column block (b200dnn_nshard_range) and call b200dnn_matmul");
  B2_CHECK(desc->wei_dt == B200DNN_S8 && desc->wei_scale.count <= desc->N && desc->src_scale.count <= desc->M, B200DNN_UNIMPLEMENTED,
           "matmul_nshard: s8 weights with per-tensor or per-channel scales");
  b200dnn_matmul_t d = *desc;
  const int64_t w = n1 - n0;
  if (w == 0) return B200DNN_SUCCESS;
  auto esz = [](int32_t dt) -> int64_t { return (int64_t)dt_size(dt); };
  d.N = (int32_t)w;
  d.weight = (const uint8_t *)desc->weight + (desc->transB ? n0 * desc->ldb : n0);
  if (desc->wei_scale.count == desc->N && desc->N > 1) {
    d.wei_scale.buff = (const uint8_t *)desc->wei_scale.buff + n0 * esz(desc->wei_scale.dt);
    d.wei_scale.count = w;
  }
  if (desc->bias) d.bias = (const uint8_t *)desc->bias + n0 * esz(desc->bias_dt);
  d.dst = (uint8_t *)desc->dst + n0 * esz(desc->dst_dt);
  for (int i = 0; i < desc->n_postops; ++i)
    if ((desc->postops[i].type == PO_BINARY_ADD || desc->postops[i].type == PO_BINARY_MUL) && desc->postops[i].buff)
      d.postops[i].buff = (const uint8_t *)desc->postops[i].buff + n0 * esz(desc->postops[i].dt);
  B2_TRY(b200dnn_matmul(&d, stream));
  if (!gather) return B200DNN_SUCCESS;

  // ---- every rank gets the whole C: pack the own block, all-gather equal-sized blocks, unpack the others' blocks
  B2_CHECK(c->comm, B200DNN_FAILURE, "matmul_nshard: gathering needs the communicator (b200dnn_nshard_create with an id or a communicator)");
  B2_CHECK(is_device_ptr(desc->dst), B200DNN_UNIMPLEMENTED, "matmul_nshard: gathering needs a destination in device memory");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  NcclApi *api = nullptr;
  B2_TRY(nccl_api(&api));
  const int64_t es = esz(desc->dst_dt), M = desc->M;
  int64_t widest = 0;
  for (int r = 0; r < c->world; ++r) { int64_t a, b; nshard_range(desc->N, c->world, r, &a, &b, nullptr); widest = b - a > widest ? b - a : widest; }
  const size_t blk = (size_t)(M * widest * es);
  if (c->stage_bytes < blk * c->world) {
    if (c->stage) { B2_CUDA(cudaStreamSynchronize(st)); cudaFree(c->stage); c->stage = nullptr; }
    B2_CUDA(cudaMalloc(&c->stage, blk * c->world));
    c->stage_bytes = blk * c->world;
  }
  uint8_t *stg = (uint8_t *)c->stage;
  B2_CUDA(cudaMemcpy2DAsync(stg + blk * c->rank, (size_t)(w * es), d.dst, (size_t)(desc->ldc * es), (size_t)(w * es), (size_t)M, cudaMemcpyDeviceToDevice, st));
  B2_NCCL(api, api->AllGather(stg + blk * c->rank, stg, blk, ncclInt8, c->comm, st));
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    int64_t a, b; nshard_range(desc->N, c->world, r, &a, &b, nullptr);
    if (b == a) continue;
    B2_CUDA(cudaMemcpy2DAsync((uint8_t *)desc->dst + a * es, (size_t)(desc->ldc * es), stg + blk * r, (size_t)((b - a) * es), (size_t)((b - a) * es),
                              (size_t)M, cudaMemcpyDeviceToDevice, st));
  }
  return B200DNN_SUCCESS;
}

}  // extern "C"
