// Test-only driver around the REFERENCE's own INT8 tile kernel.
//
// The reference file zendnnl/src/lowoha_operators/matmul/matmul_native/brgemm/kernel/int8/
// int8_brgemm_ukernel.cpp (u8 x s8 -> s32 with vpdpbusd, then zero-point / scale / bias /
// activation / bf16 epilogue) compiles on its own.  oracle/Makefile compiles it where it lies
// in the reference checkout and links it with this driver into oracle/_ref/libzendnn_ref.so;
// no reference source is copied.  The driver only does what the kernel's contract asks of its
// caller (int8_brgemm_ukernel.hpp:25-37): pack B into 64-column VNNI panels
// (4 consecutive K per column, 256 bytes per K-quad), compute the per-column sums, and walk
// the M x N tile grid.  All arithmetic on the data is the reference's.
//
// Needs AVX-512 VNNI + BF16 on the host; ref_available() reports that.
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "lowoha_operators/matmul/matmul_native/brgemm/kernel/int8/int8_brgemm_ukernel.hpp"

using namespace zendnnl::lowoha::matmul::native;

extern "C" __attribute__((visibility("default"))) int ref_available() {
  __builtin_cpu_init();
  return __builtin_cpu_supports("avx512vnni") && __builtin_cpu_supports("avx512bf16") &&
         __builtin_cpu_supports("avx512bw") && __builtin_cpu_supports("avx512vl");
}

// A: u8 [M,lda]; B: s8 [K,ldb] row-major.  N must be a multiple of 16.  fused_op follows the
// reference's fused_postop_t (0 none, 1 relu, 2 gelu_tanh, 3 gelu_erf, 4 sigmoid, 5 swish, 6 tanh).
// Exactly one of out_bf16 / out_f32 is non-null.  Returns 0 on success.
extern "C" __attribute__((visibility("default")))
int ref_int8_matmul(const uint8_t *A, int lda, const int8_t *B, int ldb, int M, int N, int K,
                    int32_t src_zp, float src_scale, const float *wei_scale, int wei_scale_count,
                    const float *bias, int fused_op, uint16_t *out_bf16, float *out_f32, int ldc) {
  if (!ref_available() || N % 16 != 0 || M <= 0 || K <= 0) return -1;
  const int kq = (K + 3) / 4;
  const int panels = (N + 63) / 64;
  const int b_stride = 64 * 4;
  std::vector<int8_t> packed((size_t)panels * kq * b_stride, 0);
  std::vector<int32_t> col_sum((size_t)panels * 64, 0);
  for (int k = 0; k < K; ++k)
    for (int n = 0; n < N; ++n) {
      int8_t v = B[(size_t)k * ldb + n];
      packed[((size_t)(n / 64) * kq + k / 4) * b_stride + (n % 64) * 4 + (k % 4)] = v;
      col_sum[n] += v;
    }
  #pragma omp parallel for schedule(static)
  for (int p = 0; p < panels; ++p) {
    const int n0 = p * 64;
    const int nr = (N - n0 >= 64) ? 64 : (N - n0);      // 16, 32, 48 or 64
    const int8_t *bp = packed.data() + (size_t)p * kq * b_stride;
    for (int c0 = 0; c0 < nr;) {
      // widest kernel that fits and keeps the panel-relative column offset legal
      int NR = (nr - c0 >= 64) ? 64 : (nr - c0 >= 32 ? 32 : 16);
      for (int m = 0; m < M;) {
        int MR = (M - m >= 6) ? 6 : (M - m >= 4 ? 4 : (M - m >= 3 ? 3 : (M - m >= 2 ? 2 : 1)));
        int8_brgemm_fn_t fn = select_int8_brgemm_kernel(MR, NR);
        if (!fn) { m += MR; continue; }
        const int n = n0 + c0;
        fn(A + (size_t)m * lda, lda, bp + c0 * 4, b_stride,
           out_f32 ? out_f32 + (size_t)m * ldc + n : nullptr, ldc, K, K,
           col_sum.data() + n, src_zp, src_scale,
           wei_scale_count > 1 ? wei_scale + n : wei_scale, wei_scale_count,
           bias ? bias + n : nullptr, static_cast<fused_postop_t>(fused_op),
           out_bf16 ? out_bf16 + (size_t)m * ldc + n : nullptr, ldc);
        m += MR;
      }
      c0 += NR;
    }
  }
  return 0;
}
