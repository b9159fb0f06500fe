// sdpa_direct: softmax(Q K^T * scale + mask) V per (batch, head), the attention operator beside the MoE block of a decoder
// layer (reference: lowoha_operators/sdpa/lowoha_sdpa.hpp:48-55, sdpa_params lowoha_sdpa_common.hpp:57-103, checks
// flash_sdpa/lowoha_flash_sdpa_utils.cpp:23-178).  Built here in the form of the reference's BMM backend
// (bmm_sdpa/lowoha_sdpa_bmm.cpp: scores by matmul_direct, mask and causal mask on the f32 scores, softmax, matmul_direct
// with V), every product on the tcgen05 kernel's bf16 form:
//   S[seq, kv]  = Q_bh K_bh^T          bf16 x bf16 -> f32   (K_bh taken as a transposed weight, packed per head)
//   P           = softmax(S * scale + mask) over kv, f32, rounded to bf16; causal: key j > query i is masked
//   O_bh        = P V_bh               bf16 x bf16 -> out_dt
// scale == 0 means 1 / sqrt(head_dim) (bmm_sdpa/lowoha_sdpa_utils.cpp:25-27).  A row whose keys are all masked gives zeros.
// Not a flash kernel: the scores make a round trip through HBM (seq * kv * 6 bytes per head).  Tensors whose query rows
// follow each other at one pitch over all heads ([batch, head, seq, dim] storage) take five launches for all heads (K and V
// of every head into the tile layout, two grouped products, one softmax); other layouts go head by head.
// Included at the end of b200dnn.cu.
#pragma once

namespace {

struct SoftmaxArgs {
  const float *S; int64_t lds;          // scores of the heads of this launch back to back: row r = head * seq + i
  uint16_t *P; int64_t ldp;
  int seq, kv;
  float scale;
  int causal;
  // mask element (b, h, i, j) at mask + b * mb + h * mh + i * mi + j (a stride of 0 broadcasts); head0: first (b * H + h) of the launch
  const void *mask; int32_t mask_dt; int64_t mb, mh, mi; int heads, head0;
};

// one CTA per query row
__global__ void __launch_bounds__(256) sdpa_softmax_kernel(const SoftmaxArgs a) {
  __shared__ float sh[8];
  const int64_t r = blockIdx.x;
  const int i = (int)(r % a.seq);
  const int64_t bh = a.head0 + r / a.seq;
  const float *s = a.S + r * a.lds;
  uint16_t *p = a.P + r * a.ldp;
  const int n_keys = a.causal ? min(a.kv, i + 1) : a.kv;
  const float ninf = __int_as_float(0xff800000);
  const int64_t moff = a.mask ? (bh / a.heads) * a.mb + (bh % a.heads) * a.mh + (int64_t)i * a.mi : 0;
  auto score = [&](int j) {
    float x = __fmul_rn(s[j], a.scale);
    if (a.mask) x = __fadd_rn(x, load_as_f32(a.mask, a.mask_dt, moff + j));
    return x;
  };
  float m = ninf;
  for (int j = threadIdx.x; j < n_keys; j += blockDim.x) m = fmaxf(m, score(j));
  m = norm_block_max_signed(m, sh);
  float sum = 0.f;
  if (m > ninf)
    for (int j = threadIdx.x; j < n_keys; j += blockDim.x) sum += expf(score(j) - m);
  sum = norm_block_sum(sum, sh);
  const float inv = sum > 0.f ? __fdiv_rn(1.0f, sum) : 0.f;
  for (int j = threadIdx.x; j < a.ldp; j += blockDim.x) {
    float v = 0.f;
    if (j < n_keys && m > ninf) v = __fmul_rn(expf(score(j) - m), inv);
    p[j] = (uint16_t)(pack_bf16x2(v, 0.0f) & 0xFFFFu);
  }
}

}  // namespace

extern "C" int32_t b200dnn_sdpa(const b200dnn_sdpa_t *d, void *stream) {
  B2_CHECK(d, B200DNN_FAILURE, "null descriptor");
  B2_ENTER(stream);
  Runtime &R = rt();
  // ---- the reference's checks (flash_sdpa/lowoha_flash_sdpa_utils.cpp:23-178)
  B2_CHECK(d->query, B200DNN_FAILURE, "sdpa: query pointer is null");
  B2_CHECK(d->key, B200DNN_FAILURE, "sdpa: key pointer is null");
  B2_CHECK(d->value, B200DNN_FAILURE, "sdpa: value pointer is null");
  B2_CHECK(d->output, B200DNN_FAILURE, "sdpa: output pointer is null");
  B2_CHECK(d->batch > 0, B200DNN_FAILURE, "sdpa: batch must be > 0");
  B2_CHECK(d->num_heads > 0, B200DNN_FAILURE, "sdpa: num_heads must be > 0");
  B2_CHECK(d->seq_len > 0, B200DNN_FAILURE, "sdpa: seq_len must be > 0");
  B2_CHECK(d->kv_seq_len >= 0, B200DNN_FAILURE, "sdpa: kv_seq_len must be >= 0");
  B2_CHECK(d->head_dim > 0, B200DNN_FAILURE, "sdpa: head_dim must be > 0");
  B2_CHECK(d->q_stride[3] == 1 && d->k_stride[3] == 1 && d->v_stride[3] == 1, B200DNN_FAILURE, "sdpa: q/k/v stride of head_dim must be 1");
  B2_CHECK(d->q_stride[2] > 0 && d->k_stride[2] > 0 && d->v_stride[2] > 0 && d->o_stride[2] > 0 && d->o_stride[3] > 0, B200DNN_FAILURE,
           "sdpa: sequence strides must be > 0");
  B2_CHECK(d->batch == 1 || d->o_stride[0] > 0, B200DNN_FAILURE, "sdpa: o_stride_b must be > 0 when batch > 1");
  B2_CHECK(d->num_heads == 1 || d->o_stride[1] > 0, B200DNN_FAILURE, "sdpa: o_stride_h must be > 0 when num_heads > 1");
  B2_CHECK(d->qkv_dt == B200DNN_F32 || d->qkv_dt == B200DNN_BF16 || d->qkv_dt == 2, B200DNN_FAILURE, "sdpa: qkv_dt must be f32, bf16, or f16");
  B2_CHECK(d->dropout_p == 0.0, B200DNN_FAILURE, "sdpa: dropout_p must be 0");
  B2_CHECK(d->mask_ndims == 0 || d->mask_ndims == 2 || d->mask_ndims == 4, B200DNN_FAILURE, "sdpa: mask_ndims must be 0, 2, or 4");
  B2_CHECK(!(d->attn_mask && d->mask_ndims == 0), B200DNN_FAILURE, "sdpa: attn_mask is non-null but mask_ndims is 0");
  B2_CHECK(!(!d->attn_mask && d->mask_ndims != 0), B200DNN_FAILURE, "sdpa: attn_mask is null but mask_ndims is %d", d->mask_ndims);
  B2_CHECK(d->out_dt == d->qkv_dt, B200DNN_FAILURE, "sdpa: out_dt must be the same as qkv_dt");
  // ---- what this library leaves out
  B2_CHECK(d->qkv_dt == B200DNN_BF16, B200DNN_UNIMPLEMENTED, "sdpa: bf16 tensors are implemented (qkv_dt %d)", d->qkv_dt);
  B2_CHECK(!d->attn_mask || d->mask_dt == B200DNN_F32 || d->mask_dt == B200DNN_BF16, B200DNN_FAILURE, "sdpa: mask_dt must be f32 or bf16 when qkv_dt is bf16");
  B2_CHECK(d->o_stride[3] == 1, B200DNN_UNIMPLEMENTED, "sdpa: the output's head_dim stride must be 1");
  const int64_t B = d->batch, H = d->num_heads, S = d->seq_len, KV = d->kv_seq_len > 0 ? d->kv_seq_len : d->seq_len, D = d->head_dim;
  B2_CHECK(S < (1 << 30) && KV < (1 << 30) && D < (1 << 20), B200DNN_UNIMPLEMENTED, "sdpa: sizes beyond 2^30");
  // mask broadcast: sizes innermost = kv; each outer size is 1 or the tensor's extent
  int64_t msz[4] = {1, 1, 1, KV}, mst[4] = {0, 0, 0, 1};
  if (d->attn_mask) {
    const int off = 4 - d->mask_ndims;
    for (int i = 0; i < d->mask_ndims; ++i) { msz[off + i] = d->mask_sizes[i]; mst[off + i] = d->mask_strides[i]; }
    B2_CHECK(msz[3] == KV && mst[3] == 1, B200DNN_UNIMPLEMENTED, "sdpa: the mask's last dimension must be kv_seq_len with stride 1");
    B2_CHECK((msz[0] == 1 || msz[0] == B) && (msz[1] == 1 || msz[1] == H) && (msz[2] == 1 || msz[2] == S), B200DNN_FAILURE,
             "sdpa: the mask must be broadcastable to [batch, heads, seq, kv]");
  }
  auto span = [](const int64_t *n, const int64_t *st) { int64_t e = 1; for (int i = 0; i < 4; ++i) e += (n[i] - 1) * st[i]; return e; };
  const int64_t nq[4] = {B, H, S, D}, nk[4] = {B, H, KV, D};
  const void *q, *k, *v, *mk = nullptr;
  B2_TRY(stage_in(d->query, (size_t)span(nq, d->q_stride) * 2, st, &q));
  B2_TRY(stage_in(d->key, (size_t)span(nk, d->k_stride) * 2, st, &k));
  B2_TRY(stage_in(d->value, (size_t)span(nk, d->v_stride) * 2, st, &v));
  if (d->attn_mask) B2_TRY(stage_in(d->attn_mask, (size_t)span(msz, mst) * dt_size(d->mask_dt), st, &mk));
  Staged o_out;
  B2_TRY(stage_out(d->output, (size_t)span(nq, d->o_stride) * 2, st, &o_out, true));

  const int64_t kvp = round_up(KV, 8);
  const float scale = d->scale == 0.0 ? 1.0f / std::sqrt((float)D) : (float)d->scale;
  const int64_t mb = msz[0] > 1 ? mst[0] : 0, mh = msz[1] > 1 ? mst[1] : 0, mi = msz[2] > 1 ? mst[2] : 0;

  // ---- all heads at once: when the query rows of all heads follow each other at one pitch, the two products are grouped
  // launches (one group per head, the head's K or V as its weight) and the softmax is one launch; several rounds when the
  // scores of all heads would not fit 1.5 GB
  const bool rows_regular = d->q_stride[1] == S * d->q_stride[2] && (B == 1 || d->q_stride[0] == H * d->q_stride[1]) &&
                            d->q_stride[2] % 8 == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0 && B * H * S < (1ll << 30);
  if (rows_regular && env_int("B200DNN_SDPA_GROUPED", 1) != 0) {
    const int64_t G = B * H;
    int64_t per_round = (int64_t)((1536ll << 20) / (S * (KV * 4 + kvp * 2)));
    per_round = per_round < 1 ? 1 : (per_round > G ? G : per_round);
    float *Sbuf = (float *)R.ws.alloc((size_t)per_round * S * KV * 4);
    uint16_t *Pbuf = (uint16_t *)R.ws.alloc((size_t)per_round * S * kvp * 2);
    B2_CHECK(Sbuf && Pbuf, B200DNN_FAILURE, "workspace allocation failed");
    const std::vector<size_t> mark = R.ws.mark();
    for (int64_t g0 = 0; g0 < G; g0 += per_round) {
      R.ws.restore(mark);
      const int n = (int)(G - g0 < per_round ? G - g0 : per_round);
      const int tile_rows = tc_tile_rows((long long)n * S, (int)(KV < D ? KV : D));
      std::vector<int32_t> tabs(2 * (n + 1));
      std::vector<PackedWeight> pk(n), pv(n);
      std::vector<TcGroupDesc> g1(n), g2(n);
      // every head's K (as a transposed weight, [kv, d]) and V ([kv, d]) into the tile layout: one launch each
      const int64_t kKp = round_up(2 * D, 128), kNp = round_up(KV, 128), vKp = round_up(2 * KV, 128), vNp = round_up(D, 128);
      const size_t k_bytes = (size_t)kKp * kNp, v_bytes = (size_t)vKp * vNp;
      uint8_t *kpack = (uint8_t *)R.ws.alloc(k_bytes * n), *vpack = (uint8_t *)R.ws.alloc(v_bytes * n);
      B2_CHECK(kpack && vpack, B200DNN_FAILURE, "workspace allocation failed");
      for (int z0 = 0; z0 < n; z0 += 32768) {          // (the grid's third dimension ends at 65535)
        const int nz = n - z0 < 32768 ? n - z0 : 32768;
        pack_weight_bf16_batched_kernel<<<dim3((unsigned)(kKp / 128), (unsigned)(kNp / 32), (unsigned)nz), 256, 0, st>>>(
            (const uint16_t *)k, d->k_stride[0], d->k_stride[1], (int)H, (int)(g0 + z0), d->k_stride[2], 1, D, KV, kKp, kpack + k_bytes * z0, k_bytes);
        pack_weight_bf16_batched_kernel<<<dim3((unsigned)(vKp / 128), (unsigned)(vNp / 32), (unsigned)nz), 256, 0, st>>>(
            (const uint16_t *)v, d->v_stride[0], d->v_stride[1], (int)H, (int)(g0 + z0), d->v_stride[2], 0, KV, D, vKp, vpack + v_bytes * z0, v_bytes);
        B2_LAUNCHED(); B2_LAUNCHED();
      }
      B2_CUDA(cudaGetLastError());
      for (int g = 0; g < n; ++g) {
        const int64_t b = (g0 + g) / H, h = (g0 + g) % H;
        tabs[g + 1] = (int32_t)((g + 1) * S);
        tabs[n + 1 + g + 1] = tabs[n + 1 + g] + (int32_t)((S + tile_rows - 1) / tile_rows);
        pk[g].wt = (const int8_t *)(kpack + k_bytes * g); pk[g].K = D; pk[g].N = KV; pk[g].Kp = kKp; pk[g].Np = kNp;
        pv[g].wt = (const int8_t *)(vpack + v_bytes * g); pv[g].K = KV; pv[g].N = D; pv[g].Kp = vKp; pv[g].Np = vNp;
        g1[g] = TcGroupDesc{nullptr, nullptr, nullptr, Sbuf + (size_t)g * S * KV, KV};
        g2[g] = TcGroupDesc{nullptr, nullptr, nullptr, (uint16_t *)o_out.dev + b * d->o_stride[0] + h * d->o_stride[1], d->o_stride[2]};
      }
      void *tabs_dev, *g1_dev, *g2_dev;
      B2_TRY(upload_blob(tabs.data(), tabs.size() * 4, st, &tabs_dev));
      B2_TRY(upload_blob(g1.data(), sizeof(TcGroupDesc) * n, st, &g1_dev));
      B2_TRY(upload_blob(g2.data(), sizeof(TcGroupDesc) * n, st, &g2_dev));
      const int32_t *row_off = (const int32_t *)tabs_dev, *tile_prefix = row_off + n + 1;
      const uint16_t *q0 = (const uint16_t *)q + (g0 / H) * d->q_stride[0] + (g0 % H) * d->q_stride[1];
      EpiParams e1{};
      e1.ldc = KV; e1.dst_dt = B200DNN_F32;
      B2_TRY(grouped_gemm((const uint8_t *)q0, d->q_stride[2] * 2, (int)(n * S), (int)KV, (int)(2 * D), pk, row_off, tile_prefix, (const TcGroupDesc *)g1_dev,
                          tabs[2 * n + 1], e1, false, st, tile_rows, true));
      SoftmaxArgs sa{};
      sa.S = Sbuf; sa.lds = KV; sa.P = Pbuf; sa.ldp = kvp; sa.seq = (int)S; sa.kv = (int)KV; sa.scale = scale; sa.causal = d->is_causal ? 1 : 0;
      sa.mask = mk; sa.mask_dt = d->mask_dt; sa.mb = mb; sa.mh = mh; sa.mi = mi; sa.heads = (int)H; sa.head0 = (int)g0;
      sdpa_softmax_kernel<<<(unsigned)(n * S), 256, 0, st>>>(sa);
      B2_LAUNCHED();
      B2_CUDA(cudaGetLastError());
      EpiParams e2{};
      e2.ldc = D; e2.dst_dt = d->out_dt;
      B2_TRY(grouped_gemm((const uint8_t *)Pbuf, kvp * 2, (int)(n * S), (int)D, (int)(2 * KV), pv, row_off, tile_prefix, (const TcGroupDesc *)g2_dev,
                          tabs[2 * n + 1], e2, false, st, tile_rows, true));
    }
    return finish_out({&o_out}, st);
  }

  // ---- head by head (any strides)
  float *Sbuf = (float *)R.ws.alloc((size_t)S * KV * 4);
  uint16_t *Pbuf = (uint16_t *)R.ws.alloc((size_t)S * kvp * 2);
  B2_CHECK(Sbuf && Pbuf, B200DNN_FAILURE, "workspace allocation failed");
  const std::vector<size_t> mark = R.ws.mark();
  for (int64_t b = 0; b < B; ++b)
    for (int64_t h = 0; h < H; ++h) {
      R.ws.restore(mark);           // the per-head packs reuse the same workspace (everything is ordered on one stream)
      const uint16_t *qb = (const uint16_t *)q + b * d->q_stride[0] + h * d->q_stride[1];
      const uint16_t *kb = (const uint16_t *)k + b * d->k_stride[0] + h * d->k_stride[1];
      const uint16_t *vb = (const uint16_t *)v + b * d->v_stride[0] + h * d->v_stride[1];
      uint16_t *ob = (uint16_t *)o_out.dev + b * d->o_stride[0] + h * d->o_stride[1];
      b200dnn_matmul_t g{};
      g.M = (int32_t)S; g.N = (int32_t)KV; g.K = (int32_t)D; g.transB = 1;
      g.src_dt = g.wei_dt = B200DNN_BF16; g.dst_dt = B200DNN_F32;
      g.lda = d->q_stride[2]; g.ldb = d->k_stride[2]; g.ldc = KV;
      g.src = qb; g.weight = kb; g.dst = Sbuf; g.wei_format = 'n';
      B2_TRY(matmul_bf16(&g, st));
      SoftmaxArgs sa{};
      sa.S = Sbuf; sa.lds = KV; sa.P = Pbuf; sa.ldp = kvp; sa.seq = (int)S; sa.kv = (int)KV; sa.scale = scale; sa.causal = d->is_causal ? 1 : 0;
      sa.mask = mk; sa.mask_dt = d->mask_dt; sa.mb = mb; sa.mh = mh; sa.mi = mi; sa.heads = (int)H; sa.head0 = (int)(b * H + h);
      sdpa_softmax_kernel<<<(unsigned)S, 256, 0, st>>>(sa);
      B2_LAUNCHED();
      B2_CUDA(cudaGetLastError());
      b200dnn_matmul_t o{};
      o.M = (int32_t)S; o.N = (int32_t)D; o.K = (int32_t)KV; o.transB = 0;
      o.src_dt = o.wei_dt = B200DNN_BF16; o.dst_dt = d->out_dt;
      o.lda = kvp; o.ldb = d->v_stride[2]; o.ldc = d->o_stride[2];
      o.src = Pbuf; o.weight = vb; o.dst = ob; o.wei_format = 'n';
      B2_TRY(matmul_bf16(&o, st));
    }
  return finish_out({&o_out}, st);
}
