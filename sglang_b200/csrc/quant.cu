// per_token_group_quant_fp8: [M,K] bf16/f16/f32 -> FP8 E4M3 bytes + one fp32 scale per
// (row, group). HBM-bound streaming kernel: every thread owns 16 consecutive elements
// (two 16-byte loads for 16-bit inputs, four for fp32, one 16-byte store), the G/16 lanes
// that share a group reduce |x| with shuffles. Algorithmic bytes per element:
// sizeof(in) + 1 + 4/G.
#include "common.cuh"

namespace b200 {

template <typename T, int LPG>
__global__ void __launch_bounds__(256) quant_group_kernel(const T* __restrict__ x, uint8_t* __restrict__ q,
                                                          float* __restrict__ s, int64_t total_chunks,
                                                          int chunks_per_row, int64_t s_stride_m,
                                                          int64_t s_stride_g, float eps, int formula) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool active = c < total_chunks;  // whole lane-groups are active or not (total % LPG == 0)
  float f[16];
  if (active) {
    Vec16<T>::load(x + c * 16, f);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) f[i] = 0.f;
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
  amax = fmaxf(group_max<LPG>(amax), eps);
  uint4 out;
  const float scale = quant16(f, amax, formula, out);
  if (active) {
    *reinterpret_cast<uint4*>(q + c * 16) = out;
    if ((threadIdx.x & (LPG - 1)) == 0) {
      const int64_t row = c / chunks_per_row;
      const int g = (int)(c - row * chunks_per_row) / LPG;
      s[row * s_stride_m + g * s_stride_g] = scale;
    }
  }
}

template <typename T>
static int launch_quant(const void* x, void* q, float* s, int64_t M, int64_t K, int group, int64_t ssm,
                        int64_t ssg, float eps, int formula, cudaStream_t st) {
  const int64_t total = M * (K / 16);
  if (total == 0) return B200_OK;
  const int threads = 256;
  const int64_t blocks = cdiv(total, threads);
  if (blocks > 0x7fffffffLL) {
    set_error_detail("quant: too many blocks");
    return B200_E_UNSUPPORTED;
  }
  const int cpr = (int)(K / 16);
#define B200_Q_LAUNCH(LPG)                                                                              \
  quant_group_kernel<T, LPG><<<(unsigned)blocks, threads, 0, st>>>(static_cast<const T*>(x),            \
                                                                   static_cast<uint8_t*>(q), s, total, \
                                                                   cpr, ssm, ssg, eps, formula)
  switch (group) {
    case 16: B200_Q_LAUNCH(1); break;
    case 32: B200_Q_LAUNCH(2); break;
    case 64: B200_Q_LAUNCH(4); break;
    case 128: B200_Q_LAUNCH(8); break;
    case 256: B200_Q_LAUNCH(16); break;
    case 512: B200_Q_LAUNCH(32); break;
    default:
      set_error_detail("quant: group size %d not in {16,32,64,128,256,512}", group);
      return B200_E_UNSUPPORTED;
  }
#undef B200_Q_LAUNCH
  return check_launch("per_token_group_quant_fp8");
}

}  // namespace b200

extern "C" int b200_per_token_group_quant_fp8(const void* x, int x_dtype, void* q, float* s, int64_t M,
                                              int64_t K, int group, int64_t s_stride_m, int64_t s_stride_g,
                                              float eps, int formula, void* stream) {
  using namespace b200;
  B200_CHECK_ARG(M >= 0 && K >= 0, "quant: negative shape");
  if (M == 0 || K == 0) return B200_OK;
  B200_CHECK_ARG(x && q && s, "quant: null pointer");
  B200_CHECK_ARG(group > 0 && K % group == 0, "quant: K=%lld is not a multiple of group=%d", (long long)K, group);
  B200_CHECK_ARG(formula >= 0 && formula <= 2, "quant: unknown formula %d", formula);
  B200_CHECK_ARG(((uintptr_t)x & 15) == 0 && ((uintptr_t)q & 15) == 0, "quant: x and q must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (x_dtype) {
    case B200_BF16:
      return launch_quant<__nv_bfloat16>(x, q, s, M, K, group, s_stride_m, s_stride_g, eps, formula, st);
    case B200_F16:
      return launch_quant<__half>(x, q, s, M, K, group, s_stride_m, s_stride_g, eps, formula, st);
    case B200_F32:
      return launch_quant<float>(x, q, s, M, K, group, s_stride_m, s_stride_g, eps, formula, st);
    default:
      set_error_detail("quant: unknown input dtype code %d", x_dtype);
      return B200_E_BAD_ARG;
  }
}
