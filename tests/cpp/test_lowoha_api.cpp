// Drop-in test of the C++ LowOHA interface (include/zendnnl_b200/lowoha.hpp): written the way a
// caller of the reference writes it -- reference include paths, namespaces, parameter structs and
// host buffers -- and checked against scalar loops in this file.  Mirrors, at small sizes, the
// reference's TestMatmul.INT8 / INT8_SYM_QUANT_PER_TOKEN / INT8_DYNAMIC_GEMM cases
// (zendnnl/gtests/test_matmul.cpp:975,1318,1444), its reorder round trips
// (zendnnl/gtests/reorder/test_dynamic_quant.cpp) and TestFusedMoEQuantDynINT8.BothPasses compared
// with a two-call unfused run (zendnnl/gtests/group_matmul/test_fused_moe.cpp:2491,
// moe_test_utils.hpp:1387).  Needs a GPU.  Exit code 0 = all checks passed.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include "lowoha_operators/matmul/lowoha_matmul.hpp"
#include "lowoha_operators/reorder/lowoha_reorder.hpp"

using namespace zendnnl::lowoha::matmul;
using namespace zendnnl::lowoha::reorder;
using zendnnl::memory::data_type_t;
using zendnnl::memory::status_t;
using zendnnl::ops::post_op_type_t;
using zendnnl::ops::matmul_algo_t;

static int g_fail = 0, g_checks = 0;
#define CHECK(cond, ...) do { ++g_checks; if (!(cond)) { ++g_fail; std::printf("FAIL %s:%d: ", __FILE__, __LINE__); std::printf(__VA_ARGS__); std::printf("\n"); } } while (0)

static uint16_t f2bf(float f) { uint32_t u; std::memcpy(&u, &f, 4); u += 0x7FFFu + ((u >> 16) & 1u); return (uint16_t)(u >> 16); }
static float bf2f(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; std::memcpy(&f, &u, 4); return f; }
static int ulp_diff(uint16_t a, uint16_t b) {
  auto key = [](uint16_t x) { int v = x & 0x7FFF; return (x & 0x8000) ? -v : v; };
  return std::abs(key(a) - key(b));
}

struct Rng {
  std::mt19937_64 g;
  explicit Rng(uint64_t s) : g(s) {}
  int ri(int lo, int hi) { return std::uniform_int_distribution<int>(lo, hi)(g); }
  float rf(float lo, float hi) { return std::uniform_real_distribution<float>(lo, hi)(g); }
  float rn() { return std::normal_distribution<float>(0.f, 1.f)(g); }
};

// exact int32 accumulators
template <class TA>
static std::vector<int32_t> gemm_s32(const std::vector<TA> &A, int lda, const std::vector<int8_t> &B, int ldb, bool transB, int M, int N, int K) {
  std::vector<int32_t> C((size_t)M * N);
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      int32_t s = 0;
      for (int k = 0; k < K; ++k) s += (int32_t)A[(size_t)m * lda + k] * (int32_t)(transB ? B[(size_t)n * ldb + k] : B[(size_t)k * ldb + n]);
      C[(size_t)m * N + n] = s;
    }
  return C;
}

static void per_token_quant(const std::vector<uint16_t> &x, int M, int K, std::vector<int8_t> &q, std::vector<float> &s) {
  q.assign((size_t)M * K, 0); s.assign(M, 0.f);
  for (int m = 0; m < M; ++m) {
    float amax = 0.f;
    for (int k = 0; k < K; ++k) amax = std::fmax(amax, std::fabs(bf2f(x[(size_t)m * K + k])));
    if (amax < 1e-10f) amax = 1e-10f;
    float sc = amax / 127.0f; if (sc < 1e-10f) sc = 1e-10f;
    s[m] = sc;
    for (int k = 0; k < K; ++k) q[(size_t)m * K + k] = (int8_t)std::nearbyint(bf2f(x[(size_t)m * K + k]) / sc);
  }
}

static void test_int8_u8_zp_bias_relu() {
  // u8 source with per-tensor scale and zero-point, per-channel weight scales, f32 bias, ReLU, bf16 out
  Rng r(0);
  const int M = 37, K = 200, N = 72, lda = 208, ldc = 80;
  std::vector<uint8_t> A((size_t)M * lda);
  std::vector<int8_t> W((size_t)K * N);
  std::vector<float> ws(N), bias(N);
  for (auto &v : A) v = (uint8_t)r.ri(0, 255);
  for (auto &v : W) v = (int8_t)r.ri(-127, 127);
  for (auto &v : ws) v = r.rf(0.001f, 0.01f);
  for (auto &v : bias) v = r.rn();
  float src_scale = 0.02f; int32_t src_zp = 128;
  std::vector<uint16_t> C((size_t)M * ldc, 0x1234);
  matmul_params p;
  p.dtypes.src = data_type_t::u8; p.dtypes.wei = data_type_t::s8; p.dtypes.dst = data_type_t::bf16; p.dtypes.bias = data_type_t::f32;
  p.quant_params.src_scale.buff = &src_scale; p.quant_params.src_scale.dt = data_type_t::f32; p.quant_params.src_scale.dims = {1};
  p.quant_params.src_zp.buff = &src_zp; p.quant_params.src_zp.dt = data_type_t::s32; p.quant_params.src_zp.dims = {1};
  p.quant_params.wei_scale.buff = ws.data(); p.quant_params.wei_scale.dt = data_type_t::f32; p.quant_params.wei_scale.dims = {1, N};
  matmul_post_op relu; relu.po_type = post_op_type_t::relu; p.postop_.push_back(relu);
  matmul_batch_params_t bp;
  status_t st = matmul_direct('r', false, false, M, N, K, 1.0f, A.data(), lda, W.data(), N, bias.data(), 0.0f, C.data(), ldc, true, bp, p);
  CHECK(st == status_t::success, "matmul_direct u8: %s", last_error());
  std::vector<int32_t> acc = gemm_s32(A, lda, W, N, false, M, N, K);
  int bad = 0;
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      int32_t cs = 0; for (int k = 0; k < K; ++k) cs += W[(size_t)k * N + n];
      float x = (float)(acc[(size_t)m * N + n] - src_zp * cs);
      x = x * src_scale; x = x * ws[n]; x = x + bias[n]; x = x > 0 ? x : 0;
      if (C[(size_t)m * ldc + n] != f2bf(x)) ++bad;
    }
  CHECK(bad == 0, "u8 zp/bias/relu: %d mismatching elements", bad);
  bool pad_ok = true;
  for (int m = 0; m < M; ++m) for (int n = N; n < ldc; ++n) pad_ok &= C[(size_t)m * ldc + n] == 0x1234;
  CHECK(pad_ok, "columns beyond N were written");
  // second call hits the packed-weight cache; transposed weights give the same result
  std::vector<int8_t> Wt((size_t)N * K);
  for (int k = 0; k < K; ++k) for (int n = 0; n < N; ++n) Wt[(size_t)n * K + k] = W[(size_t)k * N + n];
  std::vector<uint16_t> C2((size_t)M * ldc, 0);
  st = matmul_direct('r', false, true, M, N, K, 1.0f, A.data(), lda, Wt.data(), K, bias.data(), 0.0f, C2.data(), ldc, true, bp, p);
  CHECK(st == status_t::success, "matmul_direct transB: %s", last_error());
  bad = 0;
  for (int m = 0; m < M; ++m) for (int n = 0; n < N; ++n) bad += C2[(size_t)m * ldc + n] != C[(size_t)m * ldc + n];
  CHECK(bad == 0, "transB result differs in %d elements", bad);
}

static void test_int8_sym_quant_per_token() {
  Rng r(1);
  for (int M : {1, 4, 16, 150}) {
    const int K = 256, N = 96;
    std::vector<int8_t> A((size_t)M * K), W((size_t)K * N);
    std::vector<float> sa(M), ws(N);
    for (auto &v : A) v = (int8_t)r.ri(-127, 127);
    for (auto &v : W) v = (int8_t)r.ri(-127, 127);
    for (auto &v : sa) v = r.rf(0.005f, 0.05f);
    for (auto &v : ws) v = r.rf(0.001f, 0.01f);
    std::vector<float> C((size_t)M * N, 0.f);
    matmul_params p;
    p.dtypes.src = data_type_t::s8; p.dtypes.wei = data_type_t::s8; p.dtypes.dst = data_type_t::f32;
    p.quant_params.src_scale.buff = sa.data(); p.quant_params.src_scale.dt = data_type_t::f32; p.quant_params.src_scale.dims = {M, 1};
    p.quant_params.wei_scale.buff = ws.data(); p.quant_params.wei_scale.dt = data_type_t::f32; p.quant_params.wei_scale.dims = {1, N};
    matmul_batch_params_t bp;
    status_t st = matmul_direct('r', false, false, M, N, K, 1.0f, A.data(), K, W.data(), N, nullptr, 0.0f, C.data(), N, false, bp, p);
    CHECK(st == status_t::success, "per-token M=%d: %s", M, last_error());
    std::vector<int32_t> acc = gemm_s32(A, K, W, N, false, M, N, K);
    int bad = 0;
    for (int m = 0; m < M; ++m) for (int n = 0; n < N; ++n) { float x = (float)acc[(size_t)m * N + n]; x = x * sa[m]; x = x * ws[n]; bad += C[(size_t)m * N + n] != x; }
    CHECK(bad == 0, "per-token M=%d: %d mismatching f32 elements", M, bad);
  }
}

// TestMatmul.INT8_SYM_QUANT_PER_GROUP_* (zendnnl/gtests/test_matmul.cpp:1049): s8 source with {M,G} scales, s8 weights with
// {G,N} scales; reference definition operators/matmul/matmul_ref_kernel.cpp:961-1003 (groups in order, f32)
static void test_int8_sym_quant_per_group() {
  Rng r(11);
  for (int M : {3, 150}) {
    for (int gs : {8, 64}) {
      const int K = 256, N = 72, G = K / gs;
      std::vector<int8_t> A((size_t)M * K), W((size_t)K * N);
      std::vector<float> sa((size_t)M * G), ws((size_t)G * N), bias(N);
      for (auto &v : A) v = (int8_t)r.ri(-127, 127);
      for (auto &v : W) v = (int8_t)r.ri(-127, 127);
      for (auto &v : sa) v = r.rf(0.005f, 0.05f);
      for (auto &v : ws) v = r.rf(0.001f, 0.01f);
      for (auto &v : bias) v = r.rn();
      std::vector<uint16_t> C((size_t)M * N, 0);
      matmul_params p;
      p.dtypes.src = data_type_t::s8; p.dtypes.wei = data_type_t::s8; p.dtypes.dst = data_type_t::bf16; p.dtypes.bias = data_type_t::f32;
      p.quant_params.src_scale.buff = sa.data(); p.quant_params.src_scale.dt = data_type_t::f32; p.quant_params.src_scale.dims = {M, G};
      p.quant_params.wei_scale.buff = ws.data(); p.quant_params.wei_scale.dt = data_type_t::f32; p.quant_params.wei_scale.dims = {G, N};
      matmul_batch_params_t bp;
      status_t st = matmul_direct('r', false, false, M, N, K, 1.0f, A.data(), K, W.data(), N, bias.data(), 0.0f, C.data(), N, false, bp, p);
      CHECK(st == status_t::success, "per-group M=%d gs=%d: %s", M, gs, last_error());
      int worst = 0;
      for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
          float sum = 0.f;
          for (int g = 0; g < G; ++g) {
            int32_t acc = 0;
            for (int k = g * gs; k < (g + 1) * gs; ++k) acc += (int32_t)A[(size_t)m * K + k] * (int32_t)W[(size_t)k * N + n];
            float v = (float)acc * sa[(size_t)m * G + g]; v = v * ws[(size_t)g * N + n]; sum = sum + v;
          }
          worst = std::max(worst, ulp_diff(C[(size_t)m * N + n], f2bf(sum + bias[n])));
        }
      CHECK(worst <= 1, "per-group M=%d gs=%d: %d bf16 ulp", M, gs, worst);
    }
  }
}

// bf16:bf16:bf16 matmul_direct with bias and GELU (the reference's non-quantised path): f32 accumulation, 1 bf16 ulp against a
// double-precision sum (plus the f32 accumulation slack of a 320-term sum)
static void test_bf16_matmul_direct() {
  Rng r(14);
  const int M = 90, K = 320, N = 104;
  std::vector<uint16_t> A((size_t)M * K), W((size_t)K * N), C((size_t)M * N, 0);
  std::vector<float> bias(N);
  for (auto &v : A) v = f2bf(r.rn());
  for (auto &v : W) v = f2bf(r.rn() * 0.06f);
  for (auto &v : bias) v = r.rn();
  matmul_params p;
  p.dtypes.src = data_type_t::bf16; p.dtypes.wei = data_type_t::bf16; p.dtypes.dst = data_type_t::bf16; p.dtypes.bias = data_type_t::f32;
  matmul_post_op po; po.po_type = post_op_type_t::gelu_tanh;
  p.postop_.push_back(po);
  matmul_batch_params_t bp;
  status_t st = matmul_direct('r', false, false, M, N, K, 1.0f, A.data(), K, W.data(), N, bias.data(), 0.0f, C.data(), N, true, bp, p);
  CHECK(st == status_t::success, "bf16 matmul_direct: %s", last_error());
  int worst = 0;
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      double acc = 0.0;
      for (int k = 0; k < K; ++k) acc += (double)bf2f(A[(size_t)m * K + k]) * (double)bf2f(W[(size_t)k * N + n]);
      const float x = (float)acc + bias[n];
      const float c = 0.79788458347320556640625f;
      const float y = 0.5f * x * (1.0f + std::tanh(c * x * (1.0f + 0.044715f * x * x)));
      const uint16_t want = f2bf(y);
      if (std::fabs(bf2f(C[(size_t)m * N + n]) - y) > 1e-4f) worst = std::max(worst, ulp_diff(C[(size_t)m * N + n], want));
    }
  CHECK(worst <= 1, "bf16 matmul_direct: %d bf16 ulp", worst);
  // quantisation parameters are refused outside INT8 / W4A8 (lowoha_matmul_utils.cpp:227-233)
  float one = 1.0f;
  p.quant_params.src_scale.buff = &one; p.quant_params.src_scale.dt = data_type_t::f32; p.quant_params.src_scale.dims = {1};
  st = matmul_direct('r', false, false, M, N, K, 1.0f, A.data(), K, W.data(), N, bias.data(), 0.0f, C.data(), N, true, bp, p);
  CHECK(st == status_t::failure, "bf16 matmul_direct with a source scale must fail (got %d)", (int)st);
}

// normalization_direct: RMSNorm and fused-add RMSNorm on bf16 rows against the scalar definition
// (lowoha_operators/normalization/kernel/reference_kernel.cpp:383-421, 449-492)
static void test_normalization_direct() {
  using namespace zendnnl::lowoha::normalization;
  Rng r(15);
  const int B = 37, D = 520;
  std::vector<uint16_t> X((size_t)B * D), R0((size_t)B * D), Y((size_t)B * D, 0);
  std::vector<float> gamma(D);
  for (auto &v : X) v = f2bf(r.rn() * 2.0f);
  for (auto &v : R0) v = f2bf(r.rn());
  for (auto &v : gamma) v = r.rn();
  for (int fused = 0; fused < 2; ++fused) {
    std::vector<uint16_t> Rs = R0;
    norm_params p;
    p.norm_type = fused ? norm_type_t::FUSED_ADD_RMS_NORM : norm_type_t::RMS_NORM;
    p.batch = B; p.norm_size = D; p.epsilon = 1e-6f; p.use_scale = true;
    p.src_dt = data_type_t::bf16; p.dst_dt = data_type_t::bf16; p.gamma_dt = data_type_t::f32;
    status_t st = normalization_direct(X.data(), Y.data(), gamma.data(), nullptr, nullptr, nullptr, fused ? Rs.data() : nullptr, p);
    CHECK(st == status_t::success, "normalization_direct (fused=%d): %s", fused, last_error());
    int worst = 0, res_bad = 0;
    for (int b = 0; b < B; ++b) {
      float ss = 0.f;
      std::vector<float> row(D);
      for (int i = 0; i < D; ++i) {
        float v = bf2f(X[(size_t)b * D + i]);
        if (fused) { v = bf2f(R0[(size_t)b * D + i]) + v; res_bad += f2bf(v) != Rs[(size_t)b * D + i]; row[i] = bf2f(f2bf(v)); }
        else row[i] = v;
        ss += v * v;
      }
      const float inv = 1.0f / std::sqrt(ss / (float)D + 1e-6f);
      for (int i = 0; i < D; ++i) worst = std::max(worst, ulp_diff(Y[(size_t)b * D + i], f2bf(row[i] * inv * gamma[i])));
    }
    CHECK(worst <= 1 && res_bad == 0, "normalization_direct (fused=%d): %d bf16 ulp, %d residual elements differ", fused, worst, res_bad);
  }
  norm_params bad;
  bad.norm_type = norm_type_t::RMS_NORM; bad.batch = 1; bad.norm_size = 8; bad.epsilon = 0.f;
  bad.src_dt = data_type_t::bf16; bad.dst_dt = data_type_t::bf16;
  CHECK(normalization_direct(X.data(), Y.data(), nullptr, nullptr, nullptr, nullptr, nullptr, bad) == status_t::failure, "epsilon 0 must fail");
}

// group_matmul_direct, sequential mode (one src, several layers: layer i + 1 reads layer i's destination;
// matmul/group_matmul_direct.cpp:1138-1163): two dynamically quantised W8A8 layers against the same two calls of matmul_direct
static void test_group_matmul_sequential_chain() {
  Rng r(16);
  const int M = 45, K0 = 256, N0 = 192, N1 = 136;
  std::vector<uint16_t> X((size_t)M * K0);
  for (auto &v : X) v = f2bf(r.rn());
  std::vector<int8_t> W0((size_t)K0 * N0), W1((size_t)N0 * N1);
  for (auto &v : W0) v = (int8_t)r.ri(-127, 127);
  for (auto &v : W1) v = (int8_t)r.ri(-127, 127);
  std::vector<float> s0(N0), s1(N1), b0(N0);
  for (auto &v : s0) v = r.rf(1e-4f, 5e-4f);
  for (auto &v : s1) v = r.rf(1e-3f, 5e-3f);
  for (auto &v : b0) v = r.rn();
  auto params_for = [&](std::vector<float> &ws, int n) {
    matmul_params p;
    p.dtypes.src = data_type_t::bf16; p.dtypes.wei = data_type_t::s8; p.dtypes.dst = data_type_t::bf16; p.dtypes.bias = data_type_t::f32;
    p.dtypes.compute = data_type_t::s8; p.dynamic_quant = true;
    p.quant_params.src_scale.dt = data_type_t::f32; p.quant_params.src_scale.dims = {M, 1};
    p.quant_params.wei_scale.buff = ws.data(); p.quant_params.wei_scale.dt = data_type_t::f32; p.quant_params.wei_scale.dims = {1, n};
    return p;
  };
  matmul_params p0 = params_for(s0, N0), p1 = params_for(s1, N1);
  matmul_post_op relu; relu.po_type = post_op_type_t::relu; p0.postop_.push_back(relu);
  std::vector<uint16_t> Y0((size_t)M * N0, 0), Y1((size_t)M * N1, 0), R0((size_t)M * N0, 0), R1((size_t)M * N1, 0);
  status_t st = group_matmul_direct({'r', 'r'}, {false, false}, {false, false}, {M, M}, {N0, N1}, {K0, N0}, {1.f, 1.f}, {X.data()}, {K0, N0},
                                    {W0.data(), W1.data()}, {N0, N1}, {b0.data(), nullptr}, {0.f, 0.f}, {Y0.data(), Y1.data()}, {N0, N1},
                                    {true, true}, {p0, p1}, nullptr, nullptr, nullptr);
  CHECK(st == status_t::success, "sequential chain: %s", last_error());
  matmul_batch_params_t bp;
  st = matmul_direct('r', false, false, M, N0, K0, 1.f, X.data(), K0, W0.data(), N0, b0.data(), 0.f, R0.data(), N0, true, bp, p0);
  CHECK(st == status_t::success, "layer 0 alone: %s", last_error());
  st = matmul_direct('r', false, false, M, N1, N0, 1.f, R0.data(), N0, W1.data(), N1, nullptr, 0.f, R1.data(), N1, true, bp, p1);
  CHECK(st == status_t::success, "layer 1 alone: %s", last_error());
  CHECK(Y0 == R0 && Y1 == R1, "sequential chain differs from the same two calls of matmul_direct");
  double sum = 0; for (auto v : Y1) sum += std::fabs(bf2f(v));
  CHECK(sum > 1.0, "sequential chain produced an all-zero result");
  // contract: K of a layer must be N of the one before; the MoE extras belong to the parallel mode
  st = group_matmul_direct({'r', 'r'}, {false, false}, {false, false}, {M, M}, {N0, N1}, {K0, N0 + 8}, {1.f, 1.f}, {X.data()}, {K0, N0},
                           {W0.data(), W1.data()}, {N0, N1}, {nullptr, nullptr}, {0.f, 0.f}, {Y0.data(), Y1.data()}, {N0, N1}, {true, true},
                           {p0, p1}, nullptr, nullptr, nullptr);
  CHECK(st == status_t::failure, "sequential chain with K[1] != N[0] must fail");
}

// matmul_direct with transA: the source stored [K, lda] gives the same bytes as the untransposed call
static void test_int8_transposed_source() {
  Rng r(17);
  const int M = 70, K = 200, N = 96, lda_t = 72;
  std::vector<int8_t> A((size_t)M * K), At((size_t)K * lda_t, 0), W((size_t)K * N);
  for (auto &v : A) v = (int8_t)r.ri(-127, 127);
  for (auto &v : W) v = (int8_t)r.ri(-127, 127);
  for (int m = 0; m < M; ++m) for (int k = 0; k < K; ++k) At[(size_t)k * lda_t + m] = A[(size_t)m * K + k];
  std::vector<float> sa(M), ws(N);
  for (auto &v : sa) v = r.rf(0.01f, 0.05f);
  for (auto &v : ws) v = r.rf(1e-4f, 5e-4f);
  matmul_params p;
  p.dtypes.src = data_type_t::s8; p.dtypes.wei = data_type_t::s8; p.dtypes.dst = data_type_t::bf16;
  p.quant_params.src_scale.buff = sa.data(); p.quant_params.src_scale.dt = data_type_t::f32; p.quant_params.src_scale.dims = {M, 1};
  p.quant_params.wei_scale.buff = ws.data(); p.quant_params.wei_scale.dt = data_type_t::f32; p.quant_params.wei_scale.dims = {1, N};
  matmul_batch_params_t bp;
  std::vector<uint16_t> C0((size_t)M * N, 0), C1((size_t)M * N, 1);
  status_t st = matmul_direct('r', false, false, M, N, K, 1.0f, A.data(), K, W.data(), N, nullptr, 0.0f, C0.data(), N, false, bp, p);
  CHECK(st == status_t::success, "untransposed: %s", last_error());
  st = matmul_direct('r', true, false, M, N, K, 1.0f, At.data(), lda_t, W.data(), N, nullptr, 0.0f, C1.data(), N, false, bp, p);
  CHECK(st == status_t::success, "transA: %s", last_error());
  CHECK(C0 == C1, "transA result differs from the untransposed call");
  st = matmul_direct('r', true, false, M, N, K, 1.0f, At.data(), M - 1, W.data(), N, nullptr, 0.0f, C1.data(), N, false, bp, p);
  CHECK(st == status_t::failure, "transA with lda < M must fail");
}

// sdpa_direct: causal self-attention on contiguous [batch, heads, seq, dim] bf16 tensors against a scalar softmax attention
static void test_sdpa_direct() {
  using namespace zendnnl::lowoha::sdpa;
  Rng r(18);
  const int B = 2, H = 2, S = 40, D = 32;
  const size_t n = (size_t)B * H * S * D;
  std::vector<uint16_t> Q(n), K(n), V(n), O(n, 0);
  for (auto &v : Q) v = f2bf(r.rn());
  for (auto &v : K) v = f2bf(r.rn());
  for (auto &v : V) v = f2bf(r.rn());
  sdpa_params p;
  p.batch = B; p.num_heads = H; p.seq_len = S; p.kv_seq_len = S; p.head_dim = D;
  p.q_stride_b = p.k_stride_b = p.v_stride_b = p.o_stride_b = (int64_t)H * S * D;
  p.q_stride_h = p.k_stride_h = p.v_stride_h = p.o_stride_h = (int64_t)S * D;
  p.q_stride_s = p.k_stride_s = p.v_stride_s = p.o_stride_s = D;
  p.qkv_dt = data_type_t::bf16; p.out_dt = data_type_t::bf16; p.is_causal = true;
  status_t st = sdpa_direct(Q.data(), K.data(), V.data(), nullptr, O.data(), p);
  CHECK(st == status_t::success, "sdpa_direct: %s", last_error());
  double worst = 0.0;
  const float scale = 1.0f / std::sqrt((float)D);
  for (int bh = 0; bh < B * H; ++bh)
    for (int i = 0; i < S; ++i) {
      std::vector<double> pr(i + 1);
      double mx = -1e30, sum = 0.0;
      for (int j = 0; j <= i; ++j) {
        double s = 0.0;
        for (int c = 0; c < D; ++c) s += (double)bf2f(Q[((size_t)bh * S + i) * D + c]) * (double)bf2f(K[((size_t)bh * S + j) * D + c]);
        pr[j] = s * scale; mx = std::max(mx, pr[j]);
      }
      for (int j = 0; j <= i; ++j) { pr[j] = std::exp(pr[j] - mx); sum += pr[j]; }
      for (int c = 0; c < D; ++c) {
        double o = 0.0;
        for (int j = 0; j <= i; ++j) o += pr[j] / sum * (double)bf2f(V[((size_t)bh * S + j) * D + c]);
        worst = std::max(worst, std::fabs(o - (double)bf2f(O[((size_t)bh * S + i) * D + c])));
      }
    }
  CHECK(worst < 0.03, "sdpa_direct: largest absolute difference %.4f", worst);
  p.dropout_p = 0.5;
  CHECK(sdpa_direct(Q.data(), K.data(), V.data(), nullptr, O.data(), p) == status_t::failure, "dropout must fail");
}

// INT8 with a quantised u8 / s8 output tensor: dst_scale and dst_zp close the epilogue chain
// (backends/aocl/aocl_postop.cpp:1421-1448), clamp and nearbyint as operators/matmul/matmul_ref_kernel.cpp:155-192
static void test_int8_requantised_dst() {
  Rng r(13);
  const int M = 70, K = 192, N = 88;
  std::vector<uint8_t> A((size_t)M * K);
  std::vector<int8_t> W((size_t)K * N);
  std::vector<float> ws(N), bias(N);
  for (auto &v : A) v = (uint8_t)r.ri(0, 255);
  for (auto &v : W) v = (int8_t)r.ri(-127, 127);
  for (auto &v : ws) v = r.rf(0.002f, 0.01f);
  for (auto &v : bias) v = r.rn();
  float ss = 0.02f, ds = 2.0f;
  int32_t zp = 128, dzp = 11;
  std::vector<int32_t> acc = gemm_s32(A, K, W, N, false, M, N, K);
  std::vector<int32_t> colsum(N, 0);
  for (int k = 0; k < K; ++k) for (int n = 0; n < N; ++n) colsum[n] += W[(size_t)k * N + n];
  for (int is_u8 = 0; is_u8 < 2; ++is_u8) {
    std::vector<uint8_t> C((size_t)M * N, 0);
    matmul_params p;
    p.dtypes.src = data_type_t::u8; p.dtypes.wei = data_type_t::s8; p.dtypes.dst = is_u8 ? data_type_t::u8 : data_type_t::s8;
    p.dtypes.bias = data_type_t::f32;
    p.quant_params.src_scale.buff = &ss; p.quant_params.src_scale.dt = data_type_t::f32; p.quant_params.src_scale.dims = {1};
    p.quant_params.src_zp.buff = &zp; p.quant_params.src_zp.dt = data_type_t::s32; p.quant_params.src_zp.dims = {1};
    p.quant_params.wei_scale.buff = ws.data(); p.quant_params.wei_scale.dt = data_type_t::f32; p.quant_params.wei_scale.dims = {1, N};
    p.quant_params.dst_scale.buff = &ds; p.quant_params.dst_scale.dt = data_type_t::f32; p.quant_params.dst_scale.dims = {1};
    p.quant_params.dst_zp.buff = &dzp; p.quant_params.dst_zp.dt = data_type_t::s32; p.quant_params.dst_zp.dims = {1};
    matmul_batch_params_t bp;
    status_t st = matmul_direct('r', false, false, M, N, K, 1.0f, A.data(), K, W.data(), N, bias.data(), 0.0f, C.data(), N, false, bp, p);
    CHECK(st == status_t::success, "requantised dst (u8=%d): %s", is_u8, last_error());
    int worst = 0, off = 0;
    for (int m = 0; m < M; ++m)
      for (int n = 0; n < N; ++n) {
        float x = (float)(acc[(size_t)m * N + n] - zp * colsum[n]);
        x = x * ss; x = x * ws[n]; x = x + bias[n];
        x = x * ds; x = x + (float)dzp;
        const float lo = is_u8 ? 0.f : -128.f, hi = is_u8 ? 255.f : 127.f;
        x = x < lo ? lo : (x > hi ? hi : x);
        const int want = (int)std::nearbyint(x);
        const int got = is_u8 ? (int)C[(size_t)m * N + n] : (int)(int8_t)C[(size_t)m * N + n];
        worst = std::max(worst, std::abs(want - got));
        off += want != got;
      }
    CHECK(worst <= 1 && off * 500 <= M * N, "requantised dst (u8=%d): worst step %d, %d of %d differ", is_u8, worst, off, M * N);
  }
}

// TestMatmul.W4A8_BF16 (zendnnl/gtests/test_matmul.cpp:266): bf16 source quantised by the library, packed s4 weights
// (two per byte, even index low; backends/aocl/aocl_kernel.cpp:145-160), {G,N} weight scales, bf16 out
static void test_w4a8_bf16() {
  Rng r(12);
  const int M = 20, K = 256, N = 48, gs = 32, G = K / gs;
  std::vector<uint16_t> X((size_t)M * K);
  for (auto &v : X) v = f2bf(r.rn());
  std::vector<int8_t> W((size_t)K * N);
  for (auto &v : W) v = (int8_t)r.ri(-8, 7);
  std::vector<uint8_t> W4((size_t)K * N / 2);
  for (size_t i = 0; i < W4.size(); ++i) W4[i] = (uint8_t)((W[2 * i] & 0xF) | ((W[2 * i + 1] & 0xF) << 4));
  std::vector<float> ws((size_t)G * N);
  for (auto &v : ws) v = r.rf(0.001f, 0.01f);
  std::vector<int8_t> q; std::vector<float> sa;
  per_token_quant(X, M, K, q, sa);
  for (int per_group = 0; per_group < 2; ++per_group) {
    std::vector<float> sg((size_t)M * G);
    std::vector<int8_t> qg((size_t)M * K);
    if (per_group) {
      for (int m = 0; m < M; ++m)
        for (int g = 0; g < G; ++g) {
          std::vector<uint16_t> seg(X.begin() + (size_t)m * K + g * gs, X.begin() + (size_t)m * K + (g + 1) * gs);
          std::vector<int8_t> qs; std::vector<float> ss;
          per_token_quant(seg, 1, gs, qs, ss);
          sg[(size_t)m * G + g] = ss[0];
          std::copy(qs.begin(), qs.end(), qg.begin() + (size_t)m * K + g * gs);
        }
    } else {
      qg = q;
      for (int m = 0; m < M; ++m) for (int g = 0; g < G; ++g) sg[(size_t)m * G + g] = sa[m];
    }
    std::vector<uint16_t> C((size_t)M * N, 0);
    std::vector<float> scale_out((size_t)M * (per_group ? G : 1), 0.f);
    matmul_params p;
    p.dtypes.src = data_type_t::bf16; p.dtypes.wei = data_type_t::s4; p.dtypes.dst = data_type_t::bf16; p.dtypes.compute = data_type_t::s8;
    p.dynamic_quant = true;
    p.quant_params.src_scale.buff = scale_out.data(); p.quant_params.src_scale.dt = data_type_t::f32;
    p.quant_params.src_scale.dims = {M, per_group ? G : 1};
    p.quant_params.wei_scale.buff = ws.data(); p.quant_params.wei_scale.dt = data_type_t::f32; p.quant_params.wei_scale.dims = {G, N};
    matmul_batch_params_t bp;
    status_t st = matmul_direct('r', false, false, M, N, K, 1.0f, X.data(), K, W4.data(), N, nullptr, 0.0f, C.data(), N, true, bp, p);
    CHECK(st == status_t::success, "W4A8 per_group=%d: %s", per_group, last_error());
    int worst = 0, bad_scale = 0;
    for (int m = 0; m < M; ++m) {
      for (int g = 0; g < (per_group ? G : 1); ++g) bad_scale += scale_out[(size_t)m * (per_group ? G : 1) + g] != sg[(size_t)m * G + g];
      for (int n = 0; n < N; ++n) {
        float sum = 0.f;
        for (int g = 0; g < G; ++g) {
          int32_t acc = 0;
          for (int k = g * gs; k < (g + 1) * gs; ++k) acc += (int32_t)qg[(size_t)m * K + k] * (int32_t)W[(size_t)k * N + n];
          float v = (float)acc * sg[(size_t)m * G + g]; v = v * ws[(size_t)g * N + n]; sum = sum + v;
        }
        worst = std::max(worst, ulp_diff(C[(size_t)m * N + n], f2bf(sum)));
      }
    }
    CHECK(bad_scale == 0, "W4A8 per_group=%d: %d source scales differ", per_group, bad_scale);
    CHECK(worst <= 1, "W4A8 per_group=%d: %d bf16 ulp", per_group, worst);
    // the reference's refusals: s8 compute is required; an f32 destination is refused
    matmul_params bad = p; bad.dtypes.compute = data_type_t::none;
    CHECK(matmul_direct('r', false, false, M, N, K, 1.0f, X.data(), K, W4.data(), N, nullptr, 0.0f, C.data(), N, true, bp, bad) == status_t::failure,
          "W4A8 without s8 compute accepted");
  }
}

static void test_int8_dynamic_gemm() {
  Rng r(2);
  const int M = 70, K = 320, N = 128;
  std::vector<uint16_t> X((size_t)M * K);
  std::vector<int8_t> W((size_t)K * N);
  std::vector<float> ws(N), bias(N);
  for (auto &v : X) v = f2bf(r.rn());
  for (auto &v : W) v = (int8_t)r.ri(-127, 127);
  for (auto &v : ws) v = r.rf(0.001f, 0.01f);
  for (auto &v : bias) v = r.rn();
  std::vector<int8_t> q; std::vector<float> sa;
  per_token_quant(X, M, K, q, sa);
  std::vector<int32_t> acc = gemm_s32(q, K, W, N, false, M, N, K);
  for (int with_buf = 0; with_buf < 2; ++with_buf) {
    std::vector<float> scales(M, 0.f);
    std::vector<uint16_t> C((size_t)M * N, 0);
    matmul_params p;
    p.dtypes.src = data_type_t::bf16; p.dtypes.wei = data_type_t::s8; p.dtypes.dst = data_type_t::bf16; p.dtypes.bias = data_type_t::f32;
    p.dtypes.compute = data_type_t::s8; p.dynamic_quant = true;
    p.quant_params.src_scale.buff = with_buf ? scales.data() : nullptr; p.quant_params.src_scale.dt = data_type_t::f32; p.quant_params.src_scale.dims = {M, 1};
    p.quant_params.wei_scale.buff = ws.data(); p.quant_params.wei_scale.dt = data_type_t::f32; p.quant_params.wei_scale.dims = {1, N};
    matmul_batch_params_t bp;
    status_t st = matmul_direct('r', false, false, M, N, K, 1.0f, X.data(), K, W.data(), N, bias.data(), 0.0f, C.data(), N, true, bp, p);
    CHECK(st == status_t::success, "dynamic gemm: %s", last_error());
    int bad = 0;
    for (int m = 0; m < M; ++m) for (int n = 0; n < N; ++n) { float x = (float)acc[(size_t)m * N + n]; x = x * sa[m]; x = x * ws[n]; x = x + bias[n]; bad += C[(size_t)m * N + n] != f2bf(x); }
    CHECK(bad == 0, "dynamic gemm (scale buffer %d): %d mismatching elements", with_buf, bad);
    if (with_buf) { int sb = 0; for (int m = 0; m < M; ++m) sb += scales[m] != sa[m]; CHECK(sb == 0, "scales written back differ in %d rows", sb); }
  }
}

static void test_reorder_and_prepack() {
  Rng r(3);
  const int K = 300, N = 136, M = 9;
  // weights: bf16 -> per-channel s8 through reorder_direct(dynamic_quant, scale dims {1,N})
  std::vector<uint16_t> Wf((size_t)K * N);
  for (auto &v : Wf) v = f2bf(0.02f * r.rn());
  std::vector<int8_t> Wq((size_t)K * N);
  std::vector<float> ws(N, 0.f);
  reorder_params_t rp;
  rp.src_dtype = data_type_t::bf16; rp.dst_dtype = data_type_t::s8; rp.src_shape = {K, N}; rp.dst_shape = {K, N};
  rp.dynamic_quant = true;
  rp.quant_params.scale.buff = ws.data(); rp.quant_params.scale.dt = data_type_t::f32; rp.quant_params.scale.dims = {1, N};
  status_t st = reorder_direct(Wf.data(), Wq.data(), rp);
  CHECK(st == status_t::success, "per-channel quant: %s", last_error());
  int bad = 0;
  for (int n = 0; n < N; ++n) {
    float amax = 0.f; for (int k = 0; k < K; ++k) amax = std::fmax(amax, std::fabs(bf2f(Wf[(size_t)k * N + n])));
    float sc = std::fmax(amax, 1e-10f) / 127.0f;
    bad += ws[n] != sc;
    for (int k = 0; k < K; ++k) { int q = (int)std::nearbyint(bf2f(Wf[(size_t)k * N + n]) / sc); q = std::max(-128, std::min(127, q)); bad += Wq[(size_t)k * N + n] != (int8_t)q; }
  }
  CHECK(bad == 0, "per-channel weight quantisation: %d mismatches", bad);
  // activations: per-token through reorder_direct(dynamic_quant, scale dims {M,1})
  std::vector<uint16_t> X((size_t)M * K);
  for (auto &v : X) v = f2bf(r.rn());
  std::vector<int8_t> Aq((size_t)M * K); std::vector<float> sa(M, 0.f);
  reorder_params_t ra;
  ra.src_dtype = data_type_t::bf16; ra.dst_dtype = data_type_t::s8; ra.src_shape = {M, K}; ra.dst_shape = {M, K}; ra.dynamic_quant = true;
  ra.quant_params.scale.buff = sa.data(); ra.quant_params.scale.dt = data_type_t::f32; ra.quant_params.scale.dims = {M, 1};
  st = reorder_direct(X.data(), Aq.data(), ra);
  CHECK(st == status_t::success, "per-token quant: %s", last_error());
  std::vector<int8_t> q_ref; std::vector<float> s_ref;
  per_token_quant(X, M, K, q_ref, s_ref);
  CHECK(q_ref == Aq && s_ref == sa, "per-token quantisation differs from the scalar statement");
  // two-step prepack, then matmul with mem_format_b = 'r'
  reorder_params_t pk;
  pk.is_prepack = true;
  pk.prepack.algo = matmul_algo_t::aocl_dlp_blocked; pk.prepack.wei_dtype = data_type_t::s8; pk.prepack.src_dtype = data_type_t::s8;
  pk.prepack.K = K; pk.prepack.N = N; pk.prepack.ldb = N; pk.prepack.transposed = false;
  const size_t sz = weight_prepack_size(pk);
  CHECK(sz >= (size_t)K * N && sz % 64 == 0, "weight_prepack_size = %zu", sz);
  std::vector<uint8_t> packed(sz + 256);
  uint8_t *pbuf = packed.data() + (256 - (reinterpret_cast<uintptr_t>(packed.data()) & 255)) % 256;
  st = reorder_direct(Wq.data(), pbuf, pk);
  CHECK(st == status_t::success, "prepack: %s", last_error());
  matmul_params p;
  p.dtypes.src = data_type_t::s8; p.dtypes.wei = data_type_t::s8; p.dtypes.dst = data_type_t::bf16;
  p.mem_format_b = 'r'; p.lowoha_algo = matmul_algo_t::aocl_dlp_blocked;
  p.quant_params.src_scale.buff = sa.data(); p.quant_params.src_scale.dt = data_type_t::f32; p.quant_params.src_scale.dims = {M, 1};
  p.quant_params.wei_scale.buff = ws.data(); p.quant_params.wei_scale.dt = data_type_t::f32; p.quant_params.wei_scale.dims = {1, N};
  std::vector<uint16_t> C((size_t)M * N, 0);
  matmul_batch_params_t bp;
  st = matmul_direct('r', false, false, M, N, K, 1.0f, Aq.data(), K, pbuf, N, nullptr, 0.0f, C.data(), N, true, bp, p);
  CHECK(st == status_t::success, "matmul with prepacked weight: %s", last_error());
  std::vector<int32_t> acc = gemm_s32(Aq, K, Wq, N, false, M, N, K);
  bad = 0;
  for (int m = 0; m < M; ++m) for (int n = 0; n < N; ++n) { float x = (float)acc[(size_t)m * N + n]; x = x * sa[m]; x = x * ws[n]; bad += C[(size_t)m * N + n] != f2bf(x); }
  CHECK(bad == 0, "prepacked matmul: %d mismatching elements", bad);
  // static quantise / dequantise round trip (per-tensor)
  std::vector<float> xs((size_t)M * K), back((size_t)M * K);
  for (auto &v : xs) v = r.rf(-2.f, 2.f);
  float s1 = 0.02f; std::vector<int8_t> qs((size_t)M * K);
  reorder_params_t rs;
  rs.src_dtype = data_type_t::f32; rs.dst_dtype = data_type_t::s8; rs.src_shape = {M, K}; rs.dst_shape = {M, K};
  rs.quant_params.scale.buff = &s1; rs.quant_params.scale.dt = data_type_t::f32; rs.quant_params.scale.dims = {1};
  CHECK(reorder_direct(xs.data(), qs.data(), rs) == status_t::success, "static quant: %s", last_error());
  reorder_params_t rd = rs; rd.src_dtype = data_type_t::s8; rd.dst_dtype = data_type_t::f32;
  CHECK(reorder_direct(qs.data(), back.data(), rd) == status_t::success, "static dequant: %s", last_error());
  float maxerr = 0.f;
  for (size_t i = 0; i < xs.size(); ++i) maxerr = std::fmax(maxerr, std::fabs(back[i] - xs[i]));
  CHECK(maxerr <= 0.5f * s1 + 1e-6f, "quant/dequant round trip error %g", maxerr);
}

// with_bias: f32 biases on both GEMMs (grp_matmul_fused_moe_params::bias_down); want_op1: the activated output of the first
// GEMM must appear in the caller's dst[]; reuse_src: dst_down left empty, the result comes back in src[] (the reference's
// mode 2).  Mirrors zendnnl/gtests/group_matmul/test_fused_moe.cpp:1791-2045 (bias), :2491-2721 (dynamic INT8, both passes).
static void test_fused_moe_vs_two_call(bool with_bias, bool want_op1, bool reuse_src) {
  // 4 experts (one without tokens), top-2, hidden 128, FFN 64: fused group_matmul_direct against the same
  // data flow made of single calls (quantise, matmul f32, SiLU*up in this file, quantise, matmul).
  Rng r(4);
  const int T = 40, H = 128, I = 64, E = 4, topk = 2;
  std::vector<uint16_t> X((size_t)T * H);
  for (auto &v : X) v = f2bf(r.rn());
  std::vector<std::vector<int8_t>> W13(E, std::vector<int8_t>((size_t)H * 2 * I)), W2(E, std::vector<int8_t>((size_t)I * H));
  std::vector<std::vector<float>> S13(E, std::vector<float>(2 * I)), S2(E, std::vector<float>(H));
  for (int e = 0; e < E; ++e) {
    for (auto &v : W13[e]) v = (int8_t)r.ri(-127, 127);
    for (auto &v : W2[e]) v = (int8_t)r.ri(-127, 127);
    for (auto &v : S13[e]) v = r.rf(0.0005f, 0.002f);
    for (auto &v : S2[e]) v = r.rf(0.0005f, 0.002f);
  }
  // routing: expert 2 never chosen (M_e = 0); uniform weights as the reference's benchmark driver does
  std::vector<int> ids((size_t)T * topk);
  std::vector<float> tw((size_t)T * topk);
  const int choices[3] = {0, 1, 3};
  for (int t = 0; t < T; ++t) { int a = r.ri(0, 2), b = (a + 1 + r.ri(0, 1)) % 3; ids[t * 2] = choices[a]; ids[t * 2 + 1] = choices[b]; tw[t * 2] = r.rf(0.2f, 0.8f); tw[t * 2 + 1] = 1.0f - tw[t * 2]; }
  std::vector<std::vector<uint16_t>> src(E), down(E), op1(E);
  std::vector<std::vector<float>> B13(E), B2(E);
  std::vector<std::vector<int>> slot_of(E);
  for (int e = 0; e < E; ++e)
    for (int s = 0; s < T * topk; ++s)
      if (ids[s] == e) { slot_of[e].push_back(s); src[e].insert(src[e].end(), X.begin() + (size_t)(s / topk) * H, X.begin() + (size_t)(s / topk + 1) * H); }
  std::vector<const void *> row_ptrs((size_t)T * topk);
  std::vector<int> Mv(E), Nv(E, 2 * I), Kv(E, H), ldav(E, H), ldbv(E, 2 * I), ldcv(E, 2 * I);
  std::vector<char> layout(E, 'r'); std::vector<bool> tA(E, false), tB(E, false), wc(E, true);
  std::vector<float> alpha(E, 1.0f), beta(E, 0.0f);
  std::vector<const void *> srcv(E), wv(E), biasv(E, nullptr);
  std::vector<void *> dstv(E, nullptr);
  std::vector<matmul_params> params(E);
  grp_matmul_fused_moe_params fused;
  for (int e = 0; e < E; ++e) {
    Mv[e] = (int)slot_of[e].size();
    if (src[e].empty()) src[e].resize(H);
    down[e].assign((size_t)std::max(Mv[e], 1) * H, 0);
    srcv[e] = src[e].data(); wv[e] = W13[e].data();
    B13[e].resize(2 * I); B2[e].resize(H);
    for (auto &v : B13[e]) v = with_bias ? r.rf(-0.5f, 0.5f) : 0.f;
    for (auto &v : B2[e]) v = with_bias ? r.rf(-0.5f, 0.5f) : 0.f;
    if (with_bias) biasv[e] = B13[e].data();
    op1[e].assign((size_t)std::max(Mv[e], 1) * 2 * I, 0);      // dst[e] is [M, ldc = 2I]: the activated values fill its first I columns
    if (want_op1) dstv[e] = op1[e].data();
    matmul_params &p = params[e];
    p.dtypes.src = data_type_t::bf16; p.dtypes.wei = data_type_t::s8; p.dtypes.dst = data_type_t::bf16; p.dtypes.compute = data_type_t::s8;
    p.dtypes.bias = data_type_t::f32;
    p.dynamic_quant = true;
    p.quant_params.src_scale.dt = data_type_t::f32; p.quant_params.src_scale.dims = {std::max(Mv[e], 1), 1};
    p.quant_params.wei_scale.buff = S13[e].data(); p.quant_params.wei_scale.dt = data_type_t::f32; p.quant_params.wei_scale.dims = {1, 2 * I};
    fused.down_weight.push_back(W2[e].data()); fused.N_down.push_back(H); fused.ldb_down.push_back(H);
    fused.bias_down.push_back(with_bias ? B2[e].data() : nullptr);
    grp_matmul_fused_moe_params::down_weight_quant_t ds; ds.buff = S2[e].data(); ds.dt = data_type_t::f32; ds.dims = {1, H};
    fused.down_scale.push_back(ds);
    if (!reuse_src) { fused.dst_down.push_back(down[e].data()); fused.ldc_down.push_back(H); }
    // the rows the weighted reduce reads: the expert's dst_down, or its src buffer in the src-reuse mode (H == K here)
    uint16_t *res = reuse_src ? src[e].data() : down[e].data();
    for (int i = 0; i < Mv[e]; ++i) row_ptrs[slot_of[e][i]] = res + (size_t)i * H;
  }
  if (with_bias) fused.bias_dt_down = data_type_t::f32;
  const std::vector<std::vector<uint16_t>> src_in = src;     // the src-reuse mode overwrites src
  std::vector<uint16_t> out((size_t)T * H, 0);
  group_matmul_moe_postop_params post; post.num_tokens = T; post.topk = topk; post.output = out.data(); post.ldc_output = H;
  post.topk_weights = tw.data(); post.row_ptrs = row_ptrs.data();
  grp_matmul_gated_act_params act; act.act = grp_matmul_gated_act_t::silu_and_mul;
  status_t st = group_matmul_direct(layout, tA, tB, Mv, Nv, Kv, alpha, srcv, ldav, wv, ldbv, biasv, beta, dstv, ldcv, wc, params, &post, &act, &fused);
  CHECK(st == status_t::success, "fused group_matmul_direct: %s", last_error());
  // two-call statement of the same flow
  std::vector<std::vector<uint16_t>> down_ref(E);
  double sum_abs = 0;
  int bad = 0, worst = 0;
  for (int e = 0; e < E; ++e) {
    const int M = Mv[e]; if (M == 0) continue;
    std::vector<int8_t> q1; std::vector<float> s1; per_token_quant(src_in[e], M, H, q1, s1);
    const std::vector<uint16_t> &got_down = reuse_src ? src[e] : down[e];
    std::vector<int32_t> a1 = gemm_s32(q1, H, W13[e], 2 * I, false, M, 2 * I, H);
    std::vector<uint16_t> Z((size_t)M * I);
    for (int m = 0; m < M; ++m) for (int n = 0; n < I; ++n) {
      float g = (float)a1[(size_t)m * 2 * I + n]; g = g * s1[m]; g = g * S13[e][n]; g = g + B13[e][n];
      float u = (float)a1[(size_t)m * 2 * I + I + n]; u = u * s1[m]; u = u * S13[e][I + n]; u = u + B13[e][I + n];
      float sg = 1.0f / (1.0f + std::exp(-g));
      Z[(size_t)m * I + n] = f2bf((g * sg) * u);
    }
    if (want_op1) {
      int bad1 = 0;
      for (int m = 0; m < M; ++m) for (int n = 0; n < I; ++n) {
        const uint16_t got = op1[e][(size_t)m * 2 * I + n], want = Z[(size_t)m * I + n];
        bad1 += ulp_diff(got, want) > 1 && std::fabs(bf2f(got) - bf2f(want)) > 1e-5f;
      }
      CHECK(bad1 == 0, "expert %d: activated first-GEMM output in dst[]: %d elements beyond 1 ulp", e, bad1);
    }
    std::vector<int8_t> q2; std::vector<float> s2; per_token_quant(Z, M, I, q2, s2);
    std::vector<int32_t> a2 = gemm_s32(q2, I, W2[e], H, false, M, H, I);
    down_ref[e].resize((size_t)M * H);
    for (int m = 0; m < M; ++m) for (int n = 0; n < H; ++n) {
      float x = (float)a2[(size_t)m * H + n]; x = x * s2[m]; x = x * S2[e][n]; x = x + B2[e][n];
      down_ref[e][(size_t)m * H + n] = f2bf(x);
      // a one-ulp change of one activated value can move a few outputs: accept 2 bf16 ulp or 1 % of the row scale
      int d = ulp_diff(got_down[(size_t)m * H + n], f2bf(x));
      worst = std::max(worst, d);
      if (d > 2 && std::fabs(bf2f(got_down[(size_t)m * H + n]) - x) > 8e-3f * std::fabs(x) + 2e-3f) ++bad;
    }
  }
  CHECK(bad == 0, "fused MoE down outputs: %d elements out of tolerance (worst %d ulp)", bad, worst);
  bad = 0;
  for (int t = 0; t < T; ++t) for (int n = 0; n < H; ++n) {
    float acc = 0.f;
    for (int k = 0; k < topk; ++k) { const uint16_t *row = static_cast<const uint16_t *>(row_ptrs[t * topk + k]); float x = bf2f(row[n]); acc = k == 0 ? tw[t * topk] * x : std::fmaf(tw[t * topk + k], x, acc); }
    sum_abs += std::fabs(bf2f(out[(size_t)t * H + n]));
    bad += out[(size_t)t * H + n] != f2bf(acc);      // the reduce itself is exact given the library's own down outputs
  }
  CHECK(bad == 0, "weighted reduce: %d mismatching elements", bad);
  CHECK(sum_abs > 1e-3, "output is all zero");
  clear_fused_moe_scratch();
}

static void test_contract_violations() {
  std::vector<int8_t> A(4 * 64), W(64 * 16); std::vector<float> C(4 * 16);
  matmul_params p; p.dtypes.src = data_type_t::s8; p.dtypes.wei = data_type_t::s8; p.dtypes.dst = data_type_t::f32;
  matmul_batch_params_t bp;
  CHECK(matmul_direct('r', false, false, 4, 16, 64, 1.0f, nullptr, 64, W.data(), 16, nullptr, 0.0f, C.data(), 16, false, bp, p) == status_t::failure, "null src accepted");
  CHECK(matmul_direct('r', false, false, 0, 16, 64, 1.0f, A.data(), 64, W.data(), 16, nullptr, 0.0f, C.data(), 16, false, bp, p) == status_t::failure, "M = 0 accepted");
  CHECK(matmul_direct('c', false, false, 4, 16, 64, 1.0f, A.data(), 64, W.data(), 16, nullptr, 0.0f, C.data(), 16, false, bp, p) == status_t::unimplemented, "column-major not reported");
  CHECK(matmul_direct('r', true, false, 4, 16, 64, 1.0f, A.data(), 3, W.data(), 16, nullptr, 0.0f, C.data(), 16, false, bp, p) == status_t::failure, "transA with lda < M not reported");
  CHECK(matmul_direct('r', false, false, 4, 16, 64, 2.0f, A.data(), 64, W.data(), 16, nullptr, 0.0f, C.data(), 16, false, bp, p) == status_t::unimplemented, "alpha != 1 not reported");
  matmul_params p4 = p; p4.dtypes.wei = data_type_t::s4;
  CHECK(matmul_direct('r', false, false, 4, 16, 64, 1.0f, A.data(), 64, W.data(), 16, nullptr, 0.0f, C.data(), 16, false, bp, p4) == status_t::failure, "s4 weights with a pre-quantised s8 source accepted");
  p4.dtypes.wei = data_type_t::u4;
  CHECK(matmul_direct('r', false, false, 4, 16, 64, 1.0f, A.data(), 64, W.data(), 16, nullptr, 0.0f, C.data(), 16, false, bp, p4) == status_t::unimplemented, "u4 weights not reported");
  matmul_params pm = p; matmul_post_op mish; mish.po_type = post_op_type_t::mish; pm.postop_.push_back(mish);
  CHECK(matmul_direct('r', false, false, 4, 16, 64, 1.0f, A.data(), 64, W.data(), 16, nullptr, 0.0f, C.data(), 16, false, bp, pm) == status_t::failure, "mish accepted on INT8");
  // group: active_matmul > total_matmul, short vectors
  std::vector<matmul_params> ps(2, p); ps[0].active_matmul = 3; ps[0].total_matmul = 2;
  std::vector<char> lay(2, 'r'); std::vector<bool> f2(2, false); std::vector<int> M2(2, 4), N2(2, 16), K2(2, 64), ld(2, 64), ldn(2, 16);
  std::vector<float> one(2, 1.f), zero(2, 0.f); std::vector<const void *> s2{A.data(), A.data()}, w2{W.data(), W.data()}, b2(2, nullptr);
  std::vector<void *> d2{C.data(), C.data()};
  CHECK(group_matmul_direct(lay, f2, f2, M2, N2, K2, one, s2, ld, w2, ldn, b2, zero, d2, ldn, f2, ps) == status_t::failure, "active > total accepted");
  ps[0].active_matmul = 0; ps[0].total_matmul = 0;
  std::vector<int> Kshort(1, 64);
  CHECK(group_matmul_direct(lay, f2, f2, M2, N2, Kshort, one, s2, ld, w2, ldn, b2, zero, d2, ldn, f2, ps) == status_t::failure, "short K vector accepted");
  // plain grouped mode computes every expert and skips M == 0
  M2[1] = 0;
  CHECK(group_matmul_direct(lay, f2, f2, M2, N2, K2, one, s2, ld, w2, ldn, b2, zero, d2, ldn, f2, ps) == status_t::success, "plain grouped call: %s", last_error());
}

#define RUN(call) do { std::fprintf(stderr, "running %s\n", #call); call; } while (0)

// one refused call (alpha = 2 is refused in the shim, before any device work): with the reference's log knobs set the
// caller sees one line for it on stderr, without them none
static int log_line_only() {
  matmul_params p;
  p.dtypes.src = data_type_t::s8; p.dtypes.wei = data_type_t::s8; p.dtypes.dst = data_type_t::bf16;
  matmul_batch_params_t bp;
  int8_t a[8] = {0}, w[8] = {0};
  uint16_t d[4] = {0};
  status_t st = matmul_direct('r', true, false, 2, 2, 4, 2.0f, a, 4, w, 2, nullptr, 0.0f, d, 2, true, bp, p);   // alpha = 2: refused in the shim
  return st == status_t::success ? 1 : 0;
}

int main(int argc, char **argv) {
  if (argc > 1 && std::string(argv[1]) == "--log-line") return log_line_only();
  RUN(test_int8_u8_zp_bias_relu());
  RUN(test_int8_sym_quant_per_token());
  RUN(test_int8_dynamic_gemm());
  RUN(test_int8_sym_quant_per_group());
  RUN(test_w4a8_bf16());
  RUN(test_int8_requantised_dst());
  RUN(test_bf16_matmul_direct());
  RUN(test_normalization_direct());
  RUN(test_group_matmul_sequential_chain());
  RUN(test_int8_transposed_source());
  RUN(test_sdpa_direct());
  RUN(test_reorder_and_prepack());
  RUN(test_fused_moe_vs_two_call(false, false, false));
  RUN(test_fused_moe_vs_two_call(true, true, false));
  RUN(test_fused_moe_vs_two_call(true, false, true));
  RUN(test_contract_violations());
  std::printf("%d checks, %d failures\n", g_checks, g_fail);
  return g_fail ? 1 : 0;
}
