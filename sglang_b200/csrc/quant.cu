// per_token_group_quant_fp8: [M,K] bf16/f16/f32 -> FP8 E4M3 bytes + one fp32 scale per
// (row, group). HBM-bound streaming kernel: every thread owns 16 consecutive elements
// (two 16-byte loads for 16-bit inputs, four for fp32, one 16-byte store), the G/16 lanes
// that share a group reduce |x| with shuffles. Algorithmic bytes per element:
// sizeof(in) + 1 + 4/G.
#include "common.cuh"

namespace b200 {

template <typename T, int LPG, int FORMULA>
__global__ void __launch_bounds__(256) quant_group_kernel(const T* __restrict__ x, uint8_t* __restrict__ q,
                                                          float* __restrict__ s, int64_t total_chunks,
                                                          int chunks_per_row, int64_t s_stride_m,
                                                          int64_t s_stride_g, float eps) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool active = c < total_chunks;  // whole lane-groups are active or not (total % LPG == 0)
  // a GEMM launched as programmatic dependent may set itself up now; it waits for this grid's
  // completion before it reads the bytes and scales written here
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
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
  const float scale = quant16(f, amax, FORMULA, out);
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
#define B200_Q_LAUNCH_F(LPG, F)                                                                            \
  quant_group_kernel<T, LPG, F><<<(unsigned)blocks, threads, 0, st>>>(static_cast<const T*>(x),            \
                                                                      static_cast<uint8_t*>(q), s, total, \
                                                                      cpr, ssm, ssg, eps)
#define B200_Q_LAUNCH(LPG)                                        \
  switch (formula) {                                              \
    case B200_QUANT_RECIP: B200_Q_LAUNCH_F(LPG, B200_QUANT_RECIP); break; \
    case B200_QUANT_V2: B200_Q_LAUNCH_F(LPG, B200_QUANT_V2); break;       \
    case B200_QUANT_DIV_CORRECTED: B200_Q_LAUNCH_F(LPG, B200_QUANT_DIV_CORRECTED); break; \
    default: B200_Q_LAUNCH_F(LPG, B200_QUANT_DIV); break;         \
  }
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
#undef B200_Q_LAUNCH_F
  return check_launch("per_token_group_quant_fp8");
}

// Power-of-two ("UE8M0") scales, packed for MN-major consumers: the scale of (row t, group g) is
// the biased exponent byte at byte (g % 4) of the int32 word [g / 4][t] of a [ceil(G/4)][aligned_mn]
// array (per expert for a 3-D input). Arithmetic of the reference's kernel
// (sgl-kernel/csrc/gemm/per_token_group_quant_8bit_v2.cu:56-80, 343-395): amax floored at 1e-10,
// e = ceil(log2(amax * (1/448))) read off the bits, q = x * 2^-e. SILU: the input row is
// gate | up (2K wide) and the quantised value is T(silu(gate)) * up in the input type T.
// masked_m: rows t >= masked_m[expert] of a [E][rows_per_expert] input are skipped.
template <typename T, int LPG, bool SILU>
__global__ void __launch_bounds__(256) quant_group_ue8m0_kernel(const T* __restrict__ x, uint8_t* __restrict__ q,
                                                                uint8_t* __restrict__ s, int64_t total_chunks,
                                                                int chunks_per_row, int64_t aligned_mn,
                                                                const int32_t* __restrict__ masked_m,
                                                                int64_t rows_per_expert) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  bool active = c < total_chunks;
  const int64_t row = active ? c / chunks_per_row : 0;
  const int col_chunk = (int)(c - row * chunks_per_row);
  const int64_t e = row / rows_per_expert, t = row - e * rows_per_expert;
  if (active && masked_m != nullptr && t >= masked_m[e]) active = false;  // uniform per lane group (one row)
  float f[16];
  if (active) {
    const int64_t in_row = (int64_t)chunks_per_row * 16 * (SILU ? 2 : 1);
    Vec16<T>::load(x + row * in_row + col_chunk * 16, f);
    if (SILU) {
      float u[16];
      Vec16<T>::load(x + row * in_row + (int64_t)chunks_per_row * 16 + col_chunk * 16, u);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float act = to_f32<T>(from_f32<T>(f[i] / (1.0f + expf(-f[i]))));
        f[i] = to_f32<T>(from_f32<T>(act * u[i]));
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) f[i] = 0.f;
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
  amax = fmaxf(group_max<LPG>(amax), 1e-10f);
  const uint32_t bits = __float_as_uint(amax * (1.0f / 448.0f));
  const uint32_t ebyte = ((bits >> 23) & 0xffu) + ((bits & 0x7fffffu) != 0 ? 1u : 0u);
  const float scale = __uint_as_float((254u - ebyte) << 23);  // 2^-(ebyte - 127)
  uint4 out;
  out.x = pack4_e4m3(f[0] * scale, f[1] * scale, f[2] * scale, f[3] * scale);
  out.y = pack4_e4m3(f[4] * scale, f[5] * scale, f[6] * scale, f[7] * scale);
  out.z = pack4_e4m3(f[8] * scale, f[9] * scale, f[10] * scale, f[11] * scale);
  out.w = pack4_e4m3(f[12] * scale, f[13] * scale, f[14] * scale, f[15] * scale);
  if (active) {
    *reinterpret_cast<uint4*>(q + c * 16) = out;
    if ((threadIdx.x & (LPG - 1)) == 0) {
      const int groups = chunks_per_row / LPG;
      const int g = col_chunk / LPG;
      const int64_t words_per_expert = (int64_t)((groups + 3) / 4) * aligned_mn;
      uint8_t* dst = s + (e * words_per_expert + (int64_t)(g / 4) * aligned_mn + t) * 4 + (g & 3);
      *dst = (uint8_t)ebyte;
      if (g == groups - 1)  // bytes of the last word that belong to no group read as zero
        for (int k = (g & 3) + 1; k < 4; ++k) dst[k - (g & 3)] = 0;
    }
  }
}

template <typename T>
static int launch_quant_ue8m0(const void* x, void* q, void* s, int64_t M, int64_t K, int group, int64_t aligned_mn,
                              int silu, const int32_t* masked_m, int64_t rows_per_expert, cudaStream_t st) {
  const int64_t total = M * (K / 16);
  if (total == 0) return B200_OK;
  const int64_t blocks = cdiv(total, 256);
  if (blocks > 0x7fffffffLL) {
    set_error_detail("quant: too many blocks");
    return B200_E_UNSUPPORTED;
  }
  const int cpr = (int)(K / 16);
#define B200_QU_LAUNCH(LPG)                                                                                          \
  do {                                                                                                               \
    if (silu)                                                                                                        \
      quant_group_ue8m0_kernel<T, LPG, true><<<(unsigned)blocks, 256, 0, st>>>(                                      \
          static_cast<const T*>(x), static_cast<uint8_t*>(q), static_cast<uint8_t*>(s), total, cpr, aligned_mn,     \
          masked_m, rows_per_expert);                                                                                \
    else                                                                                                             \
      quant_group_ue8m0_kernel<T, LPG, false><<<(unsigned)blocks, 256, 0, st>>>(                                     \
          static_cast<const T*>(x), static_cast<uint8_t*>(q), static_cast<uint8_t*>(s), total, cpr, aligned_mn,     \
          masked_m, rows_per_expert);                                                                                \
  } while (0)
  switch (group) {
    case 16: B200_QU_LAUNCH(1); break;
    case 32: B200_QU_LAUNCH(2); break;
    case 64: B200_QU_LAUNCH(4); break;
    case 128: B200_QU_LAUNCH(8); break;
    default:
      set_error_detail("quant (UE8M0): group size %d not in {16,32,64,128}", group);
      return B200_E_UNSUPPORTED;
  }
#undef B200_QU_LAUNCH
  return check_launch("per_token_group_quant_fp8_ue8m0");
}

}  // namespace b200

extern "C" int b200_per_token_group_quant_fp8_ue8m0(const void* x, int x_dtype, void* q, void* s_packed, int64_t M,
                                                    int64_t K, int group, int64_t aligned_mn, int fuse_silu_and_mul,
                                                    const int32_t* masked_m, int num_experts, void* stream) {
  using namespace b200;
  B200_CHECK_ARG(M >= 0 && K >= 0 && num_experts >= 1, "quant: negative shape");
  if (M == 0 || K == 0) return B200_OK;
  B200_CHECK_ARG(x && q && s_packed, "quant: null pointer");
  B200_CHECK_ARG(group > 0 && K % group == 0, "quant: K=%lld is not a multiple of group=%d", (long long)K, group);
  B200_CHECK_ARG(M % num_experts == 0, "quant: M=%lld rows do not split over %d experts", (long long)M, num_experts);
  B200_CHECK_ARG(masked_m != nullptr || num_experts == 1, "quant: several experts need masked_m");
  const int64_t rows_per_expert = M / num_experts;
  B200_CHECK_ARG(aligned_mn >= rows_per_expert && aligned_mn % 4 == 0, "quant: aligned_mn=%lld for %lld rows",
                 (long long)aligned_mn, (long long)rows_per_expert);
  B200_CHECK_ARG(((uintptr_t)x & 15) == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)s_packed & 3) == 0,
                 "quant: x and q must be 16-byte aligned, the scales 4-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (x_dtype) {
    case B200_BF16:
      return launch_quant_ue8m0<__nv_bfloat16>(x, q, s_packed, M, K, group, aligned_mn, fuse_silu_and_mul, masked_m,
                                               rows_per_expert, st);
    case B200_F16:
      return launch_quant_ue8m0<__half>(x, q, s_packed, M, K, group, aligned_mn, fuse_silu_and_mul, masked_m,
                                        rows_per_expert, st);
    case B200_F32:
      return launch_quant_ue8m0<float>(x, q, s_packed, M, K, group, aligned_mn, fuse_silu_and_mul, masked_m,
                                       rows_per_expert, st);
    default:
      set_error_detail("quant: unknown input dtype code %d", x_dtype);
      return B200_E_BAD_ARG;
  }
}

extern "C" int b200_per_token_group_quant_fp8(const void* x, int x_dtype, void* q, float* s, int64_t M,
                                              int64_t K, int group, int64_t s_stride_m, int64_t s_stride_g,
                                              float eps, int formula, void* stream) {
  using namespace b200;
  B200_CHECK_ARG(M >= 0 && K >= 0, "quant: negative shape");
  if (M == 0 || K == 0) return B200_OK;
  B200_CHECK_ARG(x && q && s, "quant: null pointer");
  B200_CHECK_ARG(group > 0 && K % group == 0, "quant: K=%lld is not a multiple of group=%d", (long long)K, group);
  B200_CHECK_ARG(formula >= 0 && formula <= 3, "quant: unknown formula %d", formula);
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
