// w8a8_block_fp8_matmul: dense block-FP8 GEMM entry point (tcgen05 / TMEM / TMA kernel in
// gemm_kernel.cuh).
#include <stdlib.h>

#include "gemm_host.cuh"

extern "C" size_t b200_w8a8_block_fp8_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  (void)M; (void)N; (void)K;
  return 0;  // accumulators live in registers / TMEM; no global scratch
}

extern "C" int b200_w8a8_block_fp8_gemm(const void* A, const float* As, int64_t as_stride_m, int64_t as_stride_k,
                                        const void* B, const float* Bs, void* C, int c_dtype, int64_t M, int64_t N,
                                        int64_t K, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace b200;
  (void)workspace; (void)workspace_bytes;
  B200_CHECK_ARG(M >= 0 && N >= 0 && K >= 0, "gemm: negative shape");
  if (M == 0 || N == 0) return B200_OK;
  B200_CHECK_ARG(K > 0, "gemm: K must be positive");
  B200_CHECK_ARG(A && As && B && Bs && C, "gemm: null pointer");
  B200_CHECK_ARG(((uintptr_t)A & 15) == 0 && ((uintptr_t)B & 15) == 0 && ((uintptr_t)C & 15) == 0,
                 "gemm: A, B and C must be 16-byte aligned");
  B200_UNSUPPORTED(K % 16 != 0, "gemm: K=%lld must be a multiple of 16 (TMA row pitch)", (long long)K);
  B200_UNSUPPORTED(M > 0x7fffff00LL || N > 0x7fffff00LL || K > 0x7fffff00LL, "gemm: dimension too large");
  B200_UNSUPPORTED(N % 8 != 0, "gemm: N=%lld must be a multiple of 8 (vector stores)", (long long)N);
  GemmParams p = {};
  p.As = As; p.as_sm = as_stride_m; p.as_sk = as_stride_k;
  p.Bs = Bs; p.C = C; p.ldc = N;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  int force_bn = 0;
  if (const char* e = getenv("B200_GEMM_BN")) force_bn = atoi(e);  // test hook: 128 or 256
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (c_dtype) {
    case B200_BF16: return launch_gemm<GEMM_DENSE, __nv_bfloat16>(A, B, N, p, force_bn, st);
    case B200_F16: return launch_gemm<GEMM_DENSE, __half>(A, B, N, p, force_bn, st);
    case B200_F32: return launch_gemm<GEMM_DENSE, float>(A, B, N, p, force_bn, st);
    default:
      set_error_detail("gemm: unknown output dtype code %d", c_dtype);
      return B200_E_BAD_ARG;
  }
}
