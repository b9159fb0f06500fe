// Expert-parallel fused MoE over several GPUs (included at the end of b200dnn.cu).
//
// The reference is a single-process CPU library and has no multi-device path; what it fixes is the per-expert
// contract of group_matmul_direct (matmul/group_matmul_direct.cpp:747: independent experts, M_e = 0 allowed,
// group_matmul/group_matmul_parallel_common.hpp:1240-1248) and the fused data flow
// (group_matmul/group_matmul_fused_moe.cpp:906-1078).  Here the experts are sharded over the GPUs of one node
// (expert e lives on rank expert_rank[e]; shared experts are replicated), tokens are data-parallel.
//
// One layer on every rank, all on the caller's stream, with no host round trip:
//   route the rank's tokens, stable rank of every (token,k) slot inside its expert        (local kernels)
//   all-gather of the per-expert row counts (E+1 integers per rank)                        (NCCL, tiny)
//   offsets: where this rank's rows start inside every expert's block on the owning GPU    (one small kernel)
//   quantise every token once (s8 + f32 scale) and STORE it into the rows of all its slots in the owners' receive
//     buffers: the dispatch all-to-all is the quantisation kernel's own stores over NVLink (peer memory)
//   barrier                                                                                (NCCL, 4 bytes)
//   grouped GEMM (gate|up) + gated activation -> requantise -> grouped GEMM (down), one group per local expert,
//     rows of all source ranks back to back, row count known only on the device
//   barrier
//   weighted reduce on the owning rank, LOADING every slot's output row from the expert's GPU: the combine
//     all-to-all is the reduce kernel's own loads over NVLink
// Buffers that peers touch (received rows, their scales, expert outputs) are one allocation per rank, opened on the
// other ranks through CUDA IPC (or used directly when all ranks live in one process).  Every row is computed by the
// same kernels with the same operands wherever it lands, so the result equals the single-GPU result bit for bit.
// No TMA load or library kernel ever reads peer memory here: the GEMMs read only local HBM.
#pragma once
#include <dlfcn.h>
#include <nccl.h>

namespace {

constexpr int kEpMaxPeers = 8;

// ---- NCCL, loaded at run time (libb200dnn itself does not link against it)
struct NcclApi {
  void *lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
};
int32_t nccl_api(NcclApi **out) {
  static NcclApi api;
  static std::mutex mu;
  std::lock_guard<std::mutex> lk(mu);
  if (!api.lib) {
    // a process that already carries NCCL (PyTorch brings its own copy) keeps using that copy
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    B2_CHECK(h, B200DNN_FAILURE, "the expert-parallel layer needs NCCL (libnccl.so.2 not found: %s)", dlerror());
#define B2_SYM(field, name) *(void **)(&api.field) = dlsym(h, name); B2_CHECK(api.field, B200DNN_FAILURE, "NCCL symbol %s missing", name)
    B2_SYM(GetUniqueId, "ncclGetUniqueId"); B2_SYM(CommInitRank, "ncclCommInitRank"); B2_SYM(CommDestroy, "ncclCommDestroy");
    B2_SYM(AllGather, "ncclAllGather"); B2_SYM(AllReduce, "ncclAllReduce"); B2_SYM(CommGetAsyncError, "ncclCommGetAsyncError");
    B2_SYM(GetErrorString, "ncclGetErrorString");
#undef B2_SYM
    api.lib = h;
  }
  *out = &api;
  return B200DNN_SUCCESS;
}
#define B2_NCCL(api, expr)                                                                                              \
  do { ncclResult_t r__ = (expr);                                                                                      \
    if (r__ != ncclSuccess) return fail(B200DNN_FAILURE, "%s failed: %s", #expr, (api)->GetErrorString(r__)); } while (0)

struct EpCtx {
  b200dnn_ep_config_t cfg{};
  int device = 0;
  std::vector<int32_t> expert_rank;      // [E]
  std::vector<int> local_experts;        // global ids owned by this rank, ascending
  int n_local = 0, G = 0;                // groups: shared experts first, then the local routed experts
  int64_t Kq = 0, Iq = 0, cap_total = 0;
  // memory that peers read or write: [received s8 rows | their scales | expert outputs]
  uint8_t *xbuf = nullptr; size_t x_bytes = 0, off_q = 0, off_scale = 0, off_o = 0;
  uint8_t *peer_x[kEpMaxPeers] = {nullptr};
  bool peer_opened[kEpMaxPeers] = {false};
  // local
  uint8_t *lbuf = nullptr;
  int32_t *all_counts = nullptr, *dst_base = nullptr, *row_off = nullptr, *tile_prefix = nullptr, *n_rows = nullptr,
          *rank_rows = nullptr, *expert_rank_dev = nullptr, *ids = nullptr, *rank = nullptr, *slot_rows = nullptr,
          *slot_peer = nullptr, *barrier_word = nullptr, *overflow = nullptr;
  float *w = nullptr, *slot_w = nullptr, *s2 = nullptr;
  uint16_t *Z = nullptr; uint32_t *zmax = nullptr; int8_t *A2 = nullptr;
  std::vector<ExpertWeightsIn> ew;       // group order
  bool have_experts = false, connected = false;
  ncclComm_t comm = nullptr; bool own_comm = false;
};

__global__ void ep_set_int_kernel(int32_t *p, int32_t v) { if (threadIdx.x == 0 && blockIdx.x == 0) *p = v; }

// all_counts[s][0..E) = rows rank s sends to each expert, all_counts[s][E] = tokens of rank s.  One CTA.
// dst_base[e]: row, inside the receive buffer of expert e's owner, of this rank's first row for e.
// This rank's groups (shared experts, then its routed experts in ascending id): row_off, tile_prefix, n_rows.
__global__ void __launch_bounds__(256) ep_offsets_kernel(const int32_t *all_counts, const int32_t *expert_rank, int world, int me, int E, int S,
                                                         int cap_total, int tile_rows, int32_t *dst_base, int32_t *row_off, int32_t *tile_prefix,
                                                         int32_t *n_rows, int32_t *rank_rows, int32_t *status) {
  __shared__ int tot[256], before_me[256];
  const int stride = E + 1;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int t = 0, b = 0;
    for (int s = 0; s < world; ++s) { const int c = all_counts[s * stride + e]; t += c; if (s < me) b += c; }
    tot[e] = t; before_me[e] = b;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run[kEpMaxPeers];
    for (int d = 0; d < world; ++d) run[d] = S * all_counts[d * stride + E];
    const int t_me = all_counts[me * stride + E];
    int g = 0, acc = 0, tiles = 0;
    for (int s = 0; s < S; ++s) { row_off[g] = acc; tile_prefix[g] = tiles; acc += t_me; tiles += (t_me + tile_rows - 1) / tile_rows; ++g; }
    for (int e = 0; e < E; ++e) {
      const int d = expert_rank[e];
      dst_base[e] = run[d] + before_me[e];
      if (d == me) { row_off[g] = acc; tile_prefix[g] = tiles; acc += tot[e]; tiles += (tot[e] + tile_rows - 1) / tile_rows; ++g; }
      run[d] += tot[e];
    }
    row_off[g] = acc; tile_prefix[g] = tiles;
    *n_rows = acc;
    bool over = false;
    for (int d = 0; d < world; ++d) { rank_rows[d] = run[d]; over |= run[d] > cap_total; }
    if (over) report_status(status, 21);   // a receive buffer is too small for this routing (capacity_rows was set too low)
    if (acc > cap_total) {                 // this rank's own buffer: compute nothing rather than run past its end
      for (int i = 0; i <= g; ++i) { row_off[i] = 0; tile_prefix[i] = 0; }
      *n_rows = 0;
    }
  }
}

// slot (t, j): j < topk routed -> (owner of its expert, dst_base + stable rank); j >= topk shared -> (this rank, (j-topk)*T + t)
__global__ void ep_slot_maps_kernel(const int32_t *ids, const int32_t *rank, const float *w, const int32_t *dst_base,
                                    const int32_t *expert_rank, int T, int topk, int S, int me, int32_t *slot_rows,
                                    int32_t *slot_peer, float *slot_w) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int ns = topk + S;
  if (i >= T * ns) return;
  const int t = i / ns, j = i - t * ns;
  if (j < topk) {
    const int s = t * topk + j, e = ids[s];
    slot_rows[i] = dst_base[e] + rank[s]; slot_peer[i] = expert_rank[e]; slot_w[i] = w[s];
  } else { slot_rows[i] = (j - topk) * T + t; slot_peer[i] = me; slot_w[i] = 1.0f; }
}

// Row tile of this rank's grouped GEMMs, from what a balanced routing would give it (the real row count is known only
// on the device); the offsets kernel and the GEMM launches must agree on it.
int ep_tile_rows(const EpCtx &c, int T) {
  const b200dnn_ep_config_t &f = c.cfg;
  return tc_tile_rows((long long)T * (f.num_shared + f.topk), f.H < 2 * f.I ? f.H : 2 * f.I);
}

// ---- the phases of one layer on one rank (see the head of this file)
int32_t ep_phase_route(EpCtx &c, const void *x_dev, const float *logits_dev, int T, cudaStream_t st) {
  const b200dnn_ep_config_t &f = c.cfg;
  const int E = f.num_experts;
  int32_t *mine = c.all_counts + (size_t)f.rank * (E + 1);
  if (T > 0) {
    B2_TRY(launch_route_topk(logits_dev, T, E, f.topk, 1, c.ids, c.w, st));
    B2_TRY(launch_expert_rank(c.ids, T * f.topk, E, c.rank, mine, st));
  } else B2_CUDA(cudaMemsetAsync(mine, 0, (size_t)E * 4, st));
  ep_set_int_kernel<<<1, 32, 0, st>>>(mine + E, T);
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  (void)x_dev;
  return B200DNN_SUCCESS;
}

int32_t ep_phase_dispatch(EpCtx &c, const void *x_dev, int64_t ldx, int T, cudaStream_t st) {
  const b200dnn_ep_config_t &f = c.cfg;
  const int E = f.num_experts, S = f.num_shared, ns = f.topk + S;
  ep_offsets_kernel<<<1, 256, 0, st>>>(c.all_counts, c.expert_rank_dev, f.world, f.rank, E, S, (int)c.cap_total, ep_tile_rows(c, T), c.dst_base, c.row_off,
                                       c.tile_prefix, c.n_rows, c.rank_rows, rt().status);
  B2_LAUNCHED();
  if (T > 0) {
    ep_slot_maps_kernel<<<(unsigned)((T * ns + 255) / 256), 256, 0, st>>>(c.ids, c.rank, c.w, c.dst_base, c.expert_rank_dev, T, f.topk, S,
                                                                         f.rank, c.slot_rows, c.slot_peer, c.slot_w);
    B2_LAUNCHED();
    RowQuantArgs qa{};
    qa.src = x_dev; qa.src_ld = ldx; qa.gather_div = 1; qa.K = f.K; qa.dst_ld = c.Kq; qa.scale_dt = B200DNN_F32;
    qa.scatter = c.slot_rows; qa.scatter_peer = c.slot_peer; qa.scatter_n = ns; qa.scatter_rows = T;
    qa.scatter_cap = (int32_t)c.cap_total; qa.overflow = c.overflow;
    for (int s = 0; s < f.world; ++s) {
      qa.peer_dst[s] = reinterpret_cast<int8_t *>(c.peer_x[s] + c.off_q);
      qa.peer_scale[s] = reinterpret_cast<float *>(c.peer_x[s] + c.off_scale);
    }
    qa.dst = qa.peer_dst[f.rank]; qa.scale = qa.peer_scale[f.rank];
    B2_TRY(launch_quant_rows(qa, B200DNN_BF16, T, st));
  }
  B2_CUDA(cudaGetLastError());
  return B200DNN_SUCCESS;
}

int32_t ep_phase_experts(EpCtx &c, int T, cudaStream_t st) {
  const b200dnn_ep_config_t &f = c.cfg;
  const int G = c.G, K = f.K, I = f.I, H = f.H;
  const int gated = f.act == ACT_SWIGLU_OAI ? 2 : 1;
  std::vector<PackedWeight> p13(G), p2(G);
  std::vector<TcGroupDesc> g13(G), g2(G);
  int32_t b13_dt = 0, b2_dt = 0;
  for (int g = 0; g < G; ++g) {
    const ExpertWeightsIn &e = c.ew[g];
    B2_TRY(resolve_weight(e.w13, 'n', K, 2 * (int64_t)I, e.ldb13, f.transB, gated, 1, st, &p13[g]));
    B2_TRY(resolve_weight(e.w2, 'n', I, H, e.ldb2, f.transB, 0, 1, st, &p2[g]));
    if (e.b13) { B2_CHECK(b13_dt == 0 || b13_dt == e.b13_dt, B200DNN_UNIMPLEMENTED, "the experts' first-GEMM biases must share one dtype"); b13_dt = e.b13_dt; }
    if (e.b2) { B2_CHECK(b2_dt == 0 || b2_dt == e.b2_dt, B200DNN_UNIMPLEMENTED, "the experts' second-GEMM biases must share one dtype"); b2_dt = e.b2_dt; }
    g13[g] = TcGroupDesc{e.s13, p13[g].colsum, e.b13, nullptr, 0};
    g2[g] = TcGroupDesc{e.s2, p2[g].colsum, e.b2, nullptr, 0};
  }
  B2_CHECK((b13_dt == 0 || b13_dt == B200DNN_F32 || b13_dt == B200DNN_BF16) && (b2_dt == 0 || b2_dt == B200DNN_F32 || b2_dt == B200DNN_BF16),
           B200DNN_UNIMPLEMENTED, "bias dtype must be f32 or bf16");
  void *g13_dev, *g2_dev;
  B2_TRY(cached_blob(g13.data(), sizeof(TcGroupDesc) * G, st, &g13_dev));
  B2_TRY(cached_blob(g2.data(), sizeof(TcGroupDesc) * G, st, &g2_dev));
  const int R = (int)c.cap_total;
  // what a balanced routing would give this rank; only shapes the tile width and the grid, the tiles come from the device tables
  const int64_t expect = (int64_t)T * (f.num_shared + f.topk);
  const int tile_rows = ep_tile_rows(c, T);
  const int m_tiles_hint = (int)((expect + tile_rows - 1) / tile_rows) + G;
  B2_CUDA(cudaMemsetAsync(c.zmax, 0, (size_t)R * 4, st));
  const uint8_t *A1 = c.xbuf + c.off_q;
  const float *s1 = reinterpret_cast<const float *>(c.xbuf + c.off_scale);
  EpiParams e1{};
  e1.src_scale = s1; e1.src_scale_dt = B200DNN_F32; e1.src_scale_n = R > 1 ? R : 2;
  e1.wei_scale_dt = B200DNN_F32; e1.wei_scale_n = 2 * I;
  e1.dst = c.Z; e1.ldc = I; e1.dst_dt = B200DNN_BF16; e1.gated_act = f.act; e1.gated_I = I; e1.row_absmax = c.zmax;
  e1.bias_dt = b13_dt;
  B2_TRY(grouped_gemm(A1, c.Kq, R, 2 * I, K, p13, c.row_off, c.tile_prefix, (const TcGroupDesc *)g13_dev, m_tiles_hint, e1, true, st, tile_rows));
  rt().mark(4);
  RowQuantArgs q2{};
  q2.src = c.Z; q2.src_ld = I; q2.dst = c.A2; q2.dst_ld = c.Iq; q2.scale = c.s2; q2.scale_dt = B200DNN_F32; q2.K = I;
  q2.absmax_bits = c.zmax; q2.gather_div = 1; q2.n_rows_dev = c.n_rows;
  B2_TRY(launch_quant_rows(q2, B200DNN_BF16, R, st));
  rt().mark(5);
  EpiParams e2{};
  e2.src_scale = c.s2; e2.src_scale_dt = B200DNN_F32; e2.src_scale_n = R > 1 ? R : 2;
  e2.wei_scale_dt = B200DNN_F32; e2.wei_scale_n = H;
  e2.dst = c.xbuf + c.off_o; e2.ldc = H; e2.dst_dt = B200DNN_BF16; e2.bias_dt = b2_dt;
  B2_TRY(grouped_gemm((const uint8_t *)c.A2, c.Iq, R, H, I, p2, c.row_off, c.tile_prefix, (const TcGroupDesc *)g2_dev,
                      m_tiles_hint, e2, true, st, tile_rows));
  rt().mark(6);
  return B200DNN_SUCCESS;
}

int32_t ep_phase_combine(EpCtx &c, int T, void *out_dev, int64_t ld_out, cudaStream_t st) {
  const b200dnn_ep_config_t &f = c.cfg;
  if (T <= 0) return B200DNN_SUCCESS;
  const int ns = f.topk + f.num_shared;
  ReduceArgs ra{};
  ra.base = c.xbuf + c.off_o; ra.ld = f.H; ra.slot_rows = c.slot_rows; ra.slot_peer = c.slot_peer;
  for (int s = 0; s < f.world; ++s) ra.peer_base[s] = c.peer_x[s] + c.off_o;
  ra.row_cap = (int32_t)c.cap_total; ra.w = c.slot_w; ra.nslots = ns; ra.D = f.H; ra.dt = B200DNN_BF16; ra.out = out_dev; ra.ld_out = ld_out;
  moe_reduce_kernel<<<(unsigned)T, 256, (sizeof(void *) + 4) * ns, st>>>(ra);
  B2_LAUNCHED();
  B2_CUDA(cudaGetLastError());
  return B200DNN_SUCCESS;
}

int32_t ep_check_call(EpCtx *c, const void *x, const float *logits, int T, const void *out, int64_t ldx, int64_t ld_out) {
  B2_CHECK(c, B200DNN_FAILURE, "null expert-parallel handle");
  B2_CHECK(c->have_experts && c->connected, B200DNN_FAILURE, "expert-parallel handle needs b200dnn_ep_set_experts and a connect call first");
  B2_CHECK(T >= 0 && T <= c->cfg.max_tokens, B200DNN_FAILURE, "T = %d outside [0, max_tokens = %d]", T, c->cfg.max_tokens);
  B2_CHECK(T == 0 || (x && logits && out && ldx >= c->cfg.K && ld_out >= c->cfg.H), B200DNN_FAILURE, "null buffer or leading dimension too small");
  int dev = -1;
  B2_CUDA(cudaGetDevice(&dev));
  B2_CHECK(dev == c->device, B200DNN_FAILURE, "the handle belongs to device %d, the current device is %d", c->device, dev);
  return B200DNN_SUCCESS;
}

}  // namespace

extern "C" {

int32_t b200dnn_ep_create(const b200dnn_ep_config_t *cfg, void **handle) {
  B2_CHECK(cfg && handle, B200DNN_FAILURE, "null argument");
  B2_CHECK(cfg->world >= 1 && cfg->world <= kEpMaxPeers && cfg->rank >= 0 && cfg->rank < cfg->world, B200DNN_FAILURE,
           "world must be 1..%d and rank inside it", kEpMaxPeers);
  B2_CHECK(cfg->num_experts > 0 && cfg->num_experts <= kRankMaxKeys && cfg->num_shared >= 0 && cfg->topk > 0 &&
           cfg->topk <= cfg->num_experts && cfg->topk <= kMaxTopk && cfg->topk + cfg->num_shared <= 32, B200DNN_FAILURE,
           "expert counts out of range (experts <= %d, topk <= %d, topk + shared <= 32)", kRankMaxKeys, kMaxTopk);
  B2_CHECK(cfg->max_tokens > 0 && cfg->K > 0 && cfg->I > 0 && cfg->H > 0, B200DNN_FAILURE, "non-positive size");
  B2_CHECK(cfg->act >= 1 && cfg->act <= 3, B200DNN_UNIMPLEMENTED, "fused MoE needs a gated activation (got %d)", cfg->act);
  B2_CHECK(cfg->I % kGateGranule == 0, B200DNN_UNIMPLEMENTED, "expert FFN width must be a multiple of %d", kGateGranule);
  B2_CHECK(device_count() > 0, B200DNN_FAILURE, "no CUDA device: libb200dnn has no CPU fallback");
  EpCtx *c = new EpCtx();
  c->cfg = *cfg; c->cfg.expert_rank = nullptr;
  if (cudaGetDevice(&c->device) != cudaSuccess) { delete c; return fail(B200DNN_FAILURE, "cudaGetDevice failed"); }
  const int E = cfg->num_experts, S = cfg->num_shared, W = cfg->world;
  c->expert_rank.resize(E);
  for (int e = 0; e < E; ++e) {
    const int r = cfg->expert_rank ? cfg->expert_rank[e] : e % W;
    if (r < 0 || r >= W) { delete c; return fail(B200DNN_FAILURE, "expert_rank[%d] = %d is outside the world", e, r); }
    c->expert_rank[e] = r;
    if (r == cfg->rank) c->local_experts.push_back(e);
  }
  c->n_local = (int)c->local_experts.size(); c->G = S + c->n_local;
  c->Kq = round_up(cfg->K, 16); c->Iq = round_up(cfg->I, 16);
  const int64_t Tm = cfg->max_tokens;
  const int64_t per_src = cfg->capacity_rows > 0 ? cfg->capacity_rows : Tm * cfg->topk;
  c->cap_total = S * Tm + (int64_t)W * per_src;
  if (c->cap_total >= (int64_t)1 << 30) { delete c; return fail(B200DNN_FAILURE, "receive buffer of %lld rows is too large", (long long)c->cap_total); }
  auto al = [](size_t v) { return (v + 255) & ~size_t(255); };
  const size_t R = (size_t)c->cap_total;
  c->off_q = 0; c->off_scale = al(R * c->Kq); c->off_o = c->off_scale + al(R * 4); c->x_bytes = c->off_o + al(R * cfg->H * 2);
  // local buffers, one allocation
  size_t o = 0;
  auto take = [&](size_t bytes) { size_t at = o; o += al(bytes); return at; };
  const size_t slots = (size_t)Tm * cfg->topk, nsl = (size_t)Tm * (cfg->topk + S);
  const size_t o_cnt = take((size_t)W * (E + 1) * 4), o_db = take((size_t)E * 4), o_ro = take((size_t)(c->G + 1) * 4),
               o_tp = take((size_t)(c->G + 1) * 4), o_nr = take(4), o_rr = take((size_t)W * 4), o_er = take((size_t)E * 4),
               o_ids = take(slots * 4), o_rank = take(slots * 4), o_w = take(slots * 4), o_sr = take(nsl * 4), o_sp = take(nsl * 4),
               o_sw = take(nsl * 4), o_bw = take(256), o_ov = take(4), o_s2 = take(R * 4), o_zm = take(R * 4),
               o_z = take(R * (size_t)cfg->I * 2), o_a2 = take(R * (size_t)c->Iq);
  cudaError_t e1 = cudaMalloc(&c->xbuf, c->x_bytes), e2 = cudaMalloc(&c->lbuf, o);
  if (e1 != cudaSuccess || e2 != cudaSuccess) {
    cudaGetLastError();
    if (c->xbuf) cudaFree(c->xbuf);
    if (c->lbuf) cudaFree(c->lbuf);
    const size_t want = c->x_bytes + o;
    delete c;
    return fail(B200DNN_FAILURE, "expert-parallel buffers of %zu bytes could not be allocated (lower max_tokens or capacity_rows)", want);
  }
  uint8_t *b = c->lbuf;
  c->all_counts = (int32_t *)(b + o_cnt); c->dst_base = (int32_t *)(b + o_db); c->row_off = (int32_t *)(b + o_ro);
  c->tile_prefix = (int32_t *)(b + o_tp); c->n_rows = (int32_t *)(b + o_nr); c->rank_rows = (int32_t *)(b + o_rr);
  c->expert_rank_dev = (int32_t *)(b + o_er); c->ids = (int32_t *)(b + o_ids); c->rank = (int32_t *)(b + o_rank); c->w = (float *)(b + o_w);
  c->slot_rows = (int32_t *)(b + o_sr); c->slot_peer = (int32_t *)(b + o_sp); c->slot_w = (float *)(b + o_sw);
  c->barrier_word = (int32_t *)(b + o_bw); c->overflow = (int32_t *)(b + o_ov); c->s2 = (float *)(b + o_s2); c->zmax = (uint32_t *)(b + o_zm);
  c->Z = (uint16_t *)(b + o_z); c->A2 = (int8_t *)(b + o_a2);
  bool ok = cudaMemset(c->lbuf, 0, o_s2) == cudaSuccess &&
            cudaMemcpy(c->expert_rank_dev, c->expert_rank.data(), (size_t)E * 4, cudaMemcpyHostToDevice) == cudaSuccess;
  if (!ok) { cudaGetLastError(); cudaFree(c->xbuf); cudaFree(c->lbuf); delete c; return fail(B200DNN_FAILURE, "initialising the expert-parallel buffers failed"); }
  c->peer_x[cfg->rank] = c->xbuf;
  if (cfg->world == 1) c->connected = true;
  *handle = c;
  return B200DNN_SUCCESS;
}

int32_t b200dnn_ep_destroy(void *handle) {
  EpCtx *c = (EpCtx *)handle;
  if (!c) return B200DNN_SUCCESS;
  int cur = 0;
  cudaGetDevice(&cur);
  cudaSetDevice(c->device);
  cudaDeviceSynchronize();
  for (int s = 0; s < c->cfg.world; ++s)
    if (c->peer_opened[s]) cudaIpcCloseMemHandle(c->peer_x[s]);
  if (c->comm && c->own_comm) { NcclApi *api = nullptr; if (nccl_api(&api) == B200DNN_SUCCESS) api->CommDestroy(c->comm); }
  if (c->xbuf) cudaFree(c->xbuf);
  if (c->lbuf) cudaFree(c->lbuf);
  cudaSetDevice(cur);
  delete c;
  return B200DNN_SUCCESS;
}

int32_t b200dnn_ep_local_expert_count(void *handle, int32_t *n_local) {
  EpCtx *c = (EpCtx *)handle;
  B2_CHECK(c && n_local, B200DNN_FAILURE, "null argument");
  *n_local = c->n_local;
  return B200DNN_SUCCESS;
}

int32_t b200dnn_ep_set_experts(void *handle, const b200dnn_moe_expert_t *ex, int32_t n) {
  EpCtx *c = (EpCtx *)handle;
  B2_CHECK(c && (ex || n == 0), B200DNN_FAILURE, "null argument");
  B2_CHECK(n == c->G, B200DNN_FAILURE, "this rank owns %d routed experts and %d shared ones: %d weight sets expected, %d given",
           c->n_local, c->cfg.num_shared, c->G, n);
  c->ew.assign(c->G, ExpertWeightsIn{});
  const int S = c->cfg.num_shared;
  for (int i = 0; i < n; ++i) {
    B2_CHECK(ex[i].w13 && ex[i].w2 && ex[i].w13_scale && ex[i].w2_scale, B200DNN_FAILURE, "expert %d: null weight or scale", i);
    B2_CHECK(is_device_ptr(ex[i].w13_scale) && is_device_ptr(ex[i].w2_scale), B200DNN_UNIMPLEMENTED, "expert %d: scales must be device memory", i);
    // the caller lists its routed experts first, then the shared ones; the groups run shared first
    const int g = i < c->n_local ? S + i : i - c->n_local;
    B2_CHECK((!ex[i].bias13 || is_device_ptr(ex[i].bias13)) && (!ex[i].bias2 || is_device_ptr(ex[i].bias2)), B200DNN_UNIMPLEMENTED,
             "expert %d: biases must be device memory", i);
    c->ew[g] = expert_in(ex[i]);
  }
  c->have_experts = true;
  return B200DNN_SUCCESS;
}

int32_t b200dnn_ep_connect_local(void *const *handles, int32_t world) {
  B2_CHECK(handles && world >= 1 && world <= kEpMaxPeers, B200DNN_FAILURE, "bad argument");
  for (int r = 0; r < world; ++r) {
    EpCtx *c = (EpCtx *)handles[r];
    B2_CHECK(c && c->cfg.world == world && c->cfg.rank == r, B200DNN_FAILURE, "handle %d is not rank %d of a world of %d", r, r, world);
    B2_CHECK(c->x_bytes == ((EpCtx *)handles[0])->x_bytes, B200DNN_FAILURE, "the ranks were created with different sizes");
  }
  int cur = 0;
  B2_CUDA(cudaGetDevice(&cur));
  for (int r = 0; r < world; ++r) {
    EpCtx *c = (EpCtx *)handles[r];
    for (int s = 0; s < world; ++s) {
      EpCtx *p = (EpCtx *)handles[s];
      if (p->device != c->device) {
        B2_CUDA(cudaSetDevice(c->device));
        cudaError_t e = cudaDeviceEnablePeerAccess(p->device, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) { cudaSetDevice(cur); return fail(B200DNN_FAILURE, "no peer access from device %d to %d", c->device, p->device); }
        cudaGetLastError();
      }
      c->peer_x[s] = p->xbuf;
    }
    c->connected = true;
  }
  B2_CUDA(cudaSetDevice(cur));
  return B200DNN_SUCCESS;
}

int32_t b200dnn_ep_nccl_unique_id(void *id128) {
  B2_CHECK(id128, B200DNN_FAILURE, "null argument");
  NcclApi *api = nullptr;
  B2_TRY(nccl_api(&api));
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
  B2_NCCL(api, api->GetUniqueId((ncclUniqueId *)id128));
  return B200DNN_SUCCESS;
}

int32_t b200dnn_ep_connect_nccl(void *handle, const void *id128, void *nccl_comm) {
  EpCtx *c = (EpCtx *)handle;
  B2_CHECK(c && (id128 || nccl_comm), B200DNN_FAILURE, "null argument");
  B2_CHECK(!c->connected || c->cfg.world == 1, B200DNN_FAILURE, "already connected");
  int dev = -1;
  B2_CUDA(cudaGetDevice(&dev));
  B2_CHECK(dev == c->device, B200DNN_FAILURE, "the handle belongs to device %d, the current device is %d", c->device, dev);
  NcclApi *api = nullptr;
  B2_TRY(nccl_api(&api));
  if (nccl_comm) { c->comm = (ncclComm_t)nccl_comm; c->own_comm = false; }
  else {
    ncclUniqueId id; memcpy(&id, id128, sizeof id);
    B2_NCCL(api, api->CommInitRank(&c->comm, c->cfg.world, id, c->cfg.rank));
    c->own_comm = true;
  }
  if (c->cfg.world == 1) return B200DNN_SUCCESS;
  // exchange the IPC handles of the peer-visible allocation (one all-gather of 64 bytes per rank, once)
  const int W = c->cfg.world;
  cudaIpcMemHandle_t mine;
  B2_CUDA(cudaIpcGetMemHandle(&mine, c->xbuf));
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  uint8_t *stage = nullptr;
  B2_CUDA(cudaMalloc(&stage, (size_t)W * 64));
  std::vector<cudaIpcMemHandle_t> all(W);
  cudaError_t ce = cudaMemcpy(stage + (size_t)c->cfg.rank * 64, &mine, 64, cudaMemcpyHostToDevice);
  ncclResult_t nr = ncclSuccess;
  if (ce == cudaSuccess) nr = api->AllGather(stage + (size_t)c->cfg.rank * 64, stage, 64, ncclInt8, c->comm, nullptr);
  if (ce == cudaSuccess && nr == ncclSuccess) ce = cudaStreamSynchronize(nullptr);
  if (ce == cudaSuccess && nr == ncclSuccess) ce = cudaMemcpy(all.data(), stage, (size_t)W * 64, cudaMemcpyDeviceToHost);
  cudaFree(stage);
  B2_CHECK(nr == ncclSuccess, B200DNN_FAILURE, "ncclAllGather of the IPC handles failed: %s", api->GetErrorString(nr));
  B2_CUDA(ce);
  for (int s = 0; s < W; ++s) {
    if (s == c->cfg.rank) continue;
    void *p = nullptr;
    B2_CUDA(cudaIpcOpenMemHandle(&p, all[s], cudaIpcMemLazyEnablePeerAccess));
    c->peer_x[s] = (uint8_t *)p; c->peer_opened[s] = true;
  }
  c->connected = true;
  return B200DNN_SUCCESS;
}

int32_t b200dnn_moe_layer_ep(void *handle, const void *x, int64_t ldx, const float *logits, int32_t T, void *out, int64_t ld_out,
                             void *stream) {
  EpCtx *c = (EpCtx *)handle;
  B2_TRY(ep_check_call(c, x, logits, T, out, ldx, ld_out));
  B2_ENTER(stream);
  const b200dnn_ep_config_t &f = c->cfg;
  B2_CHECK(f.world == 1 || c->comm, B200DNN_FAILURE, "a world of %d ranks needs b200dnn_ep_connect_nccl", f.world);
  NcclApi *api = nullptr;
  if (f.world > 1) B2_TRY(nccl_api(&api));
  const void *x_dev = x, *l_dev = logits;
  Staged o_out{};
  if (T > 0) {
    B2_TRY(stage_in(x, span_bytes(T, f.K, ldx, B200DNN_BF16), st, &x_dev));
    B2_TRY(stage_in(logits, (size_t)T * f.num_experts * 4, st, &l_dev));
    B2_TRY(stage_out(out, span_bytes(T, f.H, ld_out, B200DNN_BF16), st, &o_out, ld_out != f.H));
  }
  rt().mark(-1);
  B2_TRY(ep_phase_route(*c, x_dev, (const float *)l_dev, T, st));
  rt().mark(0);
  if (f.world > 1) {
    int32_t *mine = c->all_counts + (size_t)f.rank * (f.num_experts + 1);
    B2_NCCL(api, api->AllGather(mine, c->all_counts, (size_t)f.num_experts + 1, ncclInt32, c->comm, st));
  }
  rt().mark(1);
  B2_TRY(ep_phase_dispatch(*c, x_dev, ldx, T, st));
  rt().mark(2);
  if (f.world > 1) B2_NCCL(api, api->AllReduce(c->barrier_word, c->barrier_word, 1, ncclInt32, ncclSum, c->comm, st));
  rt().mark(3);
  B2_TRY(ep_phase_experts(*c, T, st));
  if (f.world > 1) B2_NCCL(api, api->AllReduce(c->barrier_word, c->barrier_word, 1, ncclInt32, ncclSum, c->comm, st));
  rt().mark(7);
  B2_TRY(ep_phase_combine(*c, T, o_out.dev, ld_out, st));
  rt().mark(8);
  if (T > 0) return finish_out({&o_out}, st);
  return B200DNN_SUCCESS;
}

int32_t b200dnn_moe_layer_ep_local(void *const *handles, int32_t world, const void *const *x, int64_t ldx, const float *const *logits,
                                   const int32_t *T, void *const *out, int64_t ld_out, void *stream) {
  B2_CHECK(handles && x && logits && T && out && world >= 1 && world <= kEpMaxPeers, B200DNN_FAILURE, "bad argument");
  for (int r = 0; r < world; ++r) {
    EpCtx *c = (EpCtx *)handles[r];
    B2_TRY(ep_check_call(c, x[r], logits[r], T[r], out[r], ldx, ld_out));
    B2_CHECK(c->cfg.world == world && c->cfg.rank == r, B200DNN_FAILURE, "handle %d is not rank %d of %d", r, r, world);
    B2_CHECK(T[r] == 0 || (is_device_ptr(x[r]) && is_device_ptr(logits[r]) && is_device_ptr(out[r])), B200DNN_UNIMPLEMENTED,
             "the in-process form takes device buffers only");
  }
  B2_ENTER(stream);
  // every rank's phase in turn on one stream: stream order stands in for the barriers, copies for the all-gather
  for (int r = 0; r < world; ++r) B2_TRY(ep_phase_route(*(EpCtx *)handles[r], x[r], logits[r], T[r], st));
  const size_t row = ((size_t)((EpCtx *)handles[0])->cfg.num_experts + 1) * 4;
  for (int r = 0; r < world; ++r)
    for (int s = 0; s < world; ++s)
      if (s != r)
        B2_CUDA(cudaMemcpyAsync((uint8_t *)((EpCtx *)handles[r])->all_counts + s * row, (uint8_t *)((EpCtx *)handles[s])->all_counts + s * row,
                                row, cudaMemcpyDeviceToDevice, st));
  for (int r = 0; r < world; ++r) B2_TRY(ep_phase_dispatch(*(EpCtx *)handles[r], x[r], ldx, T[r], st));
  for (int r = 0; r < world; ++r) B2_TRY(ep_phase_experts(*(EpCtx *)handles[r], T[r], st));
  for (int r = 0; r < world; ++r) B2_TRY(ep_phase_combine(*(EpCtx *)handles[r], T[r], out[r], ld_out, st));
  return B200DNN_SUCCESS;
}

int32_t b200dnn_ep_rows_per_rank(void *handle, int32_t *rows, void *stream) {
  EpCtx *c = (EpCtx *)handle;
  B2_CHECK(c && rows, B200DNN_FAILURE, "null argument");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  B2_CUDA(cudaMemcpyAsync(rows, c->rank_rows, (size_t)c->cfg.world * 4, cudaMemcpyDeviceToHost, st));
  B2_CUDA(cudaStreamSynchronize(st));
  return B200DNN_SUCCESS;
}

int32_t b200dnn_ep_status(void *handle, void *stream) {
  EpCtx *c = (EpCtx *)handle;
  B2_CHECK(c, B200DNN_FAILURE, "null argument");
  if (c->comm) {
    NcclApi *api = nullptr;
    B2_TRY(nccl_api(&api));
    ncclResult_t async = ncclSuccess;
    B2_NCCL(api, api->CommGetAsyncError(c->comm, &async));
    B2_CHECK(async == ncclSuccess, B200DNN_FAILURE, "the NCCL communicator reports an asynchronous error: %s", api->GetErrorString(async));
  }
  B2_ENTER(stream);
  B2_CUDA(cudaStreamSynchronize(st));
  int32_t over = 0;
  B2_CUDA(cudaMemcpy(&over, c->overflow, 4, cudaMemcpyDeviceToHost));
  const int32_t code = *rt().status_host;
  const int32_t rc = read_status();        // clears the word
  if (over || code == 21) {
    cudaMemset(c->overflow, 0, 4);
    return fail(B200DNN_FAILURE, "rows were dropped: a receive buffer was too small for this routing (capacity_rows)");
  }
  return rc;
}

}  // extern "C"
