// w8a8_block_fp8_matmul: dense block-FP8 GEMM entry point (tcgen05 / TMEM / TMA kernel in
// gemm_kernel.cuh).
#include "gemm_host.cuh"
#include "gemm_2cta.cuh"
#include "gemm_skinny.cuh"
#include "linear_decode.cuh"
#include "gemm_ue8m0.cuh"

namespace b200 {

// Destinations of a fan-out GEMM (see GemmParams::n_dest): n == 0 means "C only".
struct FanOut {
  int n, by_tile;
  void* dest[kMaxFan];
};

// C[m, n] = sum over splits of the fp32 partials; 8 elements per thread. With a fan-out the sum
// goes to every destination buffer (or to the owner of the 128-row block) instead of C.
template <typename OutT>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partial, OutT* __restrict__ C,
                                                            int64_t mn, int splits, const FanOut fan, int64_t N) {
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  // launched with programmatic stream serialisation: this grid may start while the GEMM that
  // writes the partials is still draining; everything above is index arithmetic only
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (i >= mn) return;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < splits; ++s) {
    const float4 a = *reinterpret_cast<const float4*>(partial + (int64_t)s * mn + i);
    const float4 b = *reinterpret_cast<const float4*>(partial + (int64_t)s * mn + i + 4);
    acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
    acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
  }
  if (fan.n == 0) {
    store8<OutT>(C + i, acc);
    return;
  }
  const int d0 = fan.by_tile ? (int)((i / N / kBM) % fan.n) : 0;
  const int d1 = fan.by_tile ? d0 + 1 : fan.n;
  for (int d = d0; d < d1; ++d) store8<OutT>(static_cast<OutT*>(fan.dest[d]) + i, acc);
}

template <typename OutT>
static int launch_reduce(const float* partial, void* C, int64_t mn, int splits, cudaStream_t st,
                         const FanOut& fan = FanOut{}, int64_t N = 1) {
  // Programmatic dependent launch: the grid is set up while the producing GEMM finishes (the decode
  // kernel signals launch_dependents once all its CTAs run); griddepcontrol.wait in the kernel holds
  // it until the partials are complete and visible.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)cdiv(mn, 8 * 256));
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, splitk_reduce_kernel<OutT>, partial, static_cast<OutT*>(C), mn, splits, fan, N);
  if (e != cudaSuccess) {
    set_error_detail("splitk_reduce_kernel: %s", cudaGetErrorString(e));
    return B200_E_LAUNCH;
  }
  return check_launch("splitk_reduce_kernel");
}

}  // namespace b200

namespace b200 {
constexpr int64_t kSkinnyMaxM = 64;  // rows up to which the swapped-operand decode kernel is used
constexpr bool kPairedByDefault = false;  // CTA-pair kernel for large dense problems
}

extern "C" size_t b200_w8a8_block_fp8_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  // sized for the largest split any SM count <= 148 picks (or the tuning knobs force)
  const b200::Tuning& tune = b200::tuning();
  int s = M <= b200::kSkinnyMaxM ? b200::skinny_k_splits(M, N, K, b200::skinny_token_tile(M), 148)
                                 : b200::choose_k_splits(M, N, K, 148);
  if (tune.gemm_splitk > s) s = (int)tune.gemm_splitk;
  if (tune.gemm_skinny_max_m >= 0 && s < 16) s = 16;
  return s > 1 ? (size_t)s * (size_t)M * (size_t)N * sizeof(float) : 0;
}

namespace b200 {
static int gemm_impl(const void* A, const float* As, int64_t as_stride_m, int64_t as_stride_k, const void* B,
                     const float* Bs, void* C, int c_dtype, int64_t M, int64_t N, int64_t K, void* workspace,
                     size_t workspace_bytes, void* stream, const FanOut& fan) {
  B200_CHECK_ARG(M >= 0 && N >= 0 && K >= 0, "gemm: negative shape");
  if (M == 0 || N == 0) return B200_OK;
  B200_CHECK_ARG(K > 0, "gemm: K must be positive");
  B200_CHECK_ARG(A && As && B && Bs && (C || fan.n > 0), "gemm: null pointer");
  B200_CHECK_ARG(((uintptr_t)A & 15) == 0 && ((uintptr_t)B & 15) == 0 && ((uintptr_t)C & 15) == 0,
                 "gemm: A, B and C must be 16-byte aligned");
  for (int d = 0; d < fan.n; ++d)
    B200_CHECK_ARG(fan.dest[d] && ((uintptr_t)fan.dest[d] & 15) == 0, "gemm: fan-out destination %d null or unaligned", d);
  B200_UNSUPPORTED(K % 16 != 0, "gemm: K=%lld must be a multiple of 16 (TMA row pitch)", (long long)K);
  B200_UNSUPPORTED(M > 0x7fffff00LL || N > 0x7fffff00LL || K > 0x7fffff00LL, "gemm: dimension too large");
  B200_UNSUPPORTED(N % 8 != 0, "gemm: N=%lld must be a multiple of 8 (vector stores)", (long long)N);
  GemmParams p = {};
  p.As = As; p.as_sm = as_stride_m; p.as_sk = as_stride_k;
  p.Bs = Bs; p.C = C; p.ldc = N;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.n_dest = fan.n; p.dest_by_tile = fan.by_tile;
  for (int d = 0; d < fan.n; ++d) p.dest[d] = fan.dest[d];
  const Tuning& tune = tuning();
  const int force_bn = tune.gemm_bn == 128 || tune.gemm_bn == 256 ? (int)tune.gemm_bn : 0;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200_CHECK_ARG(c_dtype == B200_BF16 || c_dtype == B200_F16 || c_dtype == B200_F32, "gemm: unknown output dtype code %d",
                 c_dtype);
  const int sms = sm_count() < 148 ? sm_count() : 148;
  const int64_t skinny_max_m = tune.gemm_skinny_max_m >= 0 ? tune.gemm_skinny_max_m : kSkinnyMaxM;
  const bool skinny = M <= skinny_max_m && force_bn == 0 && tune.gemm_skinny != 0;
  int splits = skinny ? skinny_k_splits(M, N, K, skinny_token_tile(M), sms) : choose_k_splits(M, N, K, sms);
  if (tune.gemm_splitk > 0) splits = (int)tune.gemm_splitk;
  if (splits > (int)cdiv(K, 128)) splits = (int)cdiv(K, 128);
  if (skinny) {
    while (cdiv(cdiv(K, 128), splits) > SkinnyCfg<16>::kMaxKb) ++splits;  // scales of one item fit its smem table
    SkinnyParams sp = {};
    sp.As = As; sp.as_sm = as_stride_m; sp.as_sk = as_stride_k; sp.Bs = Bs;
    sp.M = (int)M; sp.N = (int)N; sp.K = (int)K;
    if (splits == 1 && fan.n == 0) {
      sp.C = C;
      if (c_dtype == B200_BF16) return launch_skinny<__nv_bfloat16>(A, B, sp, 1, st);
      if (c_dtype == B200_F16) return launch_skinny<__half>(A, B, sp, 1, st);
      return launch_skinny<float>(A, B, sp, 1, st);
    }
    const size_t need = (size_t)splits * (size_t)M * (size_t)N * sizeof(float);
    if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 15) != 0) {
      set_error_detail("gemm: split-K needs a 16-byte aligned workspace of %zu bytes (got %zu)", need, workspace_bytes);
      return B200_E_WORKSPACE;
    }
    sp.C = workspace;
    int rc = launch_skinny<float>(A, B, sp, splits, st);
    if (rc) return rc;
    const float* part = static_cast<const float*>(workspace);
    if (c_dtype == B200_BF16) return launch_reduce<__nv_bfloat16>(part, C, M * N, splits, st, fan, N);
    if (c_dtype == B200_F16) return launch_reduce<__half>(part, C, M * N, splits, st, fan, N);
    return launch_reduce<float>(part, C, M * N, splits, st, fan, N);
  }
  if (splits > 1) {
    // decode-sized problem: fp32 partials per K split in the workspace, then one reduction pass
    const size_t need = (size_t)splits * (size_t)M * (size_t)N * sizeof(float);
    if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 15) != 0) {
      set_error_detail("gemm: split-K needs a 16-byte aligned workspace of %zu bytes (got %zu)", need, workspace_bytes);
      return B200_E_WORKSPACE;
    }
    p.C = workspace;
    p.split_stride = M * N;
    p.n_dest = 0;  // the partials stay local; the reduction pass fans the sum out
    int rc = launch_gemm<GEMM_DENSE, float>(A, B, N, p, force_bn, st, 0, splits);
    if (rc) return rc;
    const float* part = static_cast<const float*>(workspace);
    if (c_dtype == B200_BF16) return launch_reduce<__nv_bfloat16>(part, C, M * N, splits, st, fan, N);
    if (c_dtype == B200_F16) return launch_reduce<__half>(part, C, M * N, splits, st, fan, N);
    return launch_reduce<float>(part, C, M * N, splits, st, fan, N);
  }
  // Large dense problems with 16-bit output: CTA pairs (each CTA loads half of the B tile)
  {
    const int mode2 = (int)tune.gemm_2cta;  // 0 = never, 1 = whenever legal
    const bool legal = c_dtype != B200_F32 && force_bn == 0 && N >= 256 && fan.n == 0;
    const bool want = mode2 == 1 || (mode2 != 0 && kPairedByDefault && M >= 1024 && cdiv(M, 256) * cdiv(N, 256) >= 64);
    if (legal && want) {
      if (c_dtype == B200_BF16) return launch_gemm_2cta<__nv_bfloat16>(A, B, p, st);
      return launch_gemm_2cta<__half>(A, B, p, st);
    }
  }
  switch (c_dtype) {
    case B200_BF16: return launch_gemm<GEMM_DENSE, __nv_bfloat16>(A, B, N, p, force_bn, st);
    case B200_F16: return launch_gemm<GEMM_DENSE, __half>(A, B, N, p, force_bn, st);
    case B200_F32: return launch_gemm<GEMM_DENSE, float>(A, B, N, p, force_bn, st);
    default:
      set_error_detail("gemm: unknown output dtype code %d", c_dtype);
      return B200_E_BAD_ARG;
  }
}
}  // namespace b200

extern "C" int b200_w8a8_block_fp8_gemm(const void* A, const float* As, int64_t as_stride_m, int64_t as_stride_k,
                                        const void* B, const float* Bs, void* C, int c_dtype, int64_t M, int64_t N,
                                        int64_t K, void* workspace, size_t workspace_bytes, void* stream) {
  return b200::gemm_impl(A, As, as_stride_m, as_stride_k, B, Bs, C, c_dtype, M, N, K, workspace, workspace_bytes, stream,
                         b200::FanOut{});
}

extern "C" size_t b200_w8a8_block_fp8_gemm_fanout_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const size_t plain = b200_w8a8_block_fp8_gemm_workspace_bytes(M, N, K);
  // the decode kernel always goes through an fp32 partial when its result is fanned out
  const size_t one = M <= b200::kSkinnyMaxM ? (size_t)M * (size_t)N * sizeof(float) : 0;
  return plain > one ? plain : one;
}

extern "C" int b200_w8a8_block_fp8_gemm_fanout(const void* A, const float* As, int64_t as_stride_m, int64_t as_stride_k,
                                               const void* B, const float* Bs, void* const* dest, int n_dest,
                                               int dest_by_tile, int c_dtype, int64_t M, int64_t N, int64_t K,
                                               void* workspace, size_t workspace_bytes, void* stream) {
  using namespace b200;
  B200_CHECK_ARG(dest != nullptr && n_dest >= 1 && n_dest <= kMaxFan, "gemm fan-out: %d destinations (1..%d)", n_dest,
                 kMaxFan);
  FanOut fan = {};
  fan.n = n_dest;
  fan.by_tile = dest_by_tile != 0;
  for (int d = 0; d < n_dest; ++d) fan.dest[d] = dest[d];
  return gemm_impl(A, As, as_stride_m, as_stride_k, B, Bs, nullptr, c_dtype, M, N, K, workspace, workspace_bytes, stream,
                   fan);
}

extern "C" size_t b200_w8a8_block_fp8_linear_decode_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int s = b200::decode_linear_k_splits(N, K, 148);
  return s > 1 ? (size_t)s * (size_t)M * (size_t)N * sizeof(float) : 0;
}

extern "C" int b200_w8a8_block_fp8_linear_decode(const void* x, int x_dtype, const void* B, const float* Bs, void* out,
                                                 int64_t M, int64_t N, int64_t K, float eps, void* workspace,
                                                 size_t workspace_bytes, void* tickets, void* stream) {
  using namespace b200;
  B200_CHECK_ARG(M >= 0 && N >= 0 && K > 0, "linear_decode: bad shape");
  if (M == 0 || N == 0) return B200_OK;
  B200_UNSUPPORTED(M > DecodeLinearCfg::NT, "linear_decode: M=%lld rows (at most %d)", (long long)M, DecodeLinearCfg::NT);
  B200_UNSUPPORTED(x_dtype != B200_BF16 && x_dtype != B200_F16, "linear_decode: 16-bit activations only (dtype code %d)", x_dtype);
  B200_UNSUPPORTED(K % 16 != 0 || N % 8 != 0, "linear_decode: K=%lld must be a multiple of 16, N=%lld of 8", (long long)K,
                   (long long)N);
  B200_UNSUPPORTED(N > 4096 * 128, "linear_decode: N=%lld exceeds the ticket array (4096 weight tiles)", (long long)N);
  B200_CHECK_ARG(x && B && Bs && out && tickets, "linear_decode: null pointer");
  B200_CHECK_ARG(((uintptr_t)x & 15) == 0 && ((uintptr_t)B & 15) == 0, "linear_decode: x and B must be 16-byte aligned");
  const int sms = sm_count() < 148 ? sm_count() : 148;
  DecodeLinearParams p = {};
  p.x = x; p.Bs = Bs; p.out = out; p.M = (int)M; p.N = (int)N; p.K = (int)K; p.eps = eps;
  p.num_kb = (int)cdiv(K, kBK);
  p.n_tiles = (int)cdiv(N, 128);
  p.k_splits = decode_linear_k_splits(N, K, sms);
  p.kb_per_split = (int)cdiv(p.num_kb, p.k_splits);
  p.k_splits = (int)cdiv(p.num_kb, p.kb_per_split);  // no empty split: every ticket is drawn
  p.tickets = static_cast<unsigned*>(tickets);
  if (p.k_splits > 1) {
    const size_t need = (size_t)p.k_splits * (size_t)M * (size_t)N * sizeof(float);
    if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 15) != 0) {
      set_error_detail("linear_decode: split-K needs a 16-byte aligned workspace of %zu bytes (got %zu)", need, workspace_bytes);
      return B200_E_WORKSPACE;
    }
    p.partial = static_cast<float*>(workspace);
  }
  p.status = device_status_word();
  if (!p.status) {
    set_error_detail("cannot resolve the device status word");
    return B200_E_LAUNCH;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (x_dtype == B200_BF16) return launch_decode_linear<__nv_bfloat16, __nv_bfloat16>(B, p, st);
  return launch_decode_linear<__half, __half>(B, p, st);
}

extern "C" int b200_w8a8_block_fp8_gemm_ue8m0(const void* A, const int32_t* sfa, int64_t sfa_ld, const void* B,
                                              const int32_t* sfb, int64_t sfb_ld, int sfb_rows_per_word, void* C,
                                              int c_dtype, int64_t M, int64_t N, int64_t K, void* stream) {
  using namespace b200;
  B200_CHECK_ARG(M >= 0 && N >= 0 && K > 0, "gemm_ue8m0: bad shape");
  if (M == 0 || N == 0) return B200_OK;
  B200_CHECK_ARG(A && B && C && sfa && sfb, "gemm_ue8m0: null pointer");
  B200_CHECK_ARG(((uintptr_t)A & 15) == 0 && ((uintptr_t)B & 15) == 0 && ((uintptr_t)C & 15) == 0,
                 "gemm_ue8m0: A, B and C must be 16-byte aligned");
  B200_CHECK_ARG(sfb_rows_per_word == 1 || sfb_rows_per_word == 128, "gemm_ue8m0: one scale word per row or per 128 rows of B");
  B200_CHECK_ARG(sfa_ld >= M && sfb_ld >= cdiv(N, sfb_rows_per_word), "gemm_ue8m0: scale row pitch shorter than the rows");
  B200_UNSUPPORTED(K % 16 != 0 || N % 8 != 0, "gemm_ue8m0: K=%lld must be a multiple of 16, N=%lld of 8", (long long)K,
                   (long long)N);
  B200_UNSUPPORTED(M > 0x7fffff00LL || N > 0x7fffff00LL || K > 0x7fffff00LL, "gemm_ue8m0: dimension too large");
  Ue8m0Params p = {};
  p.sfa = sfa; p.sfb = sfb; p.sfa_ld = sfa_ld; p.sfb_ld = sfb_ld; p.sfb_rows_per_word = sfb_rows_per_word;
  p.C = C; p.M = (int)M; p.N = (int)N; p.K = (int)K;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (c_dtype) {
    case B200_BF16: return launch_gemm_ue8m0<__nv_bfloat16>(A, B, p, st);
    case B200_F16: return launch_gemm_ue8m0<__half>(A, B, p, st);
    case B200_F32: return launch_gemm_ue8m0<float>(A, B, p, st);
    default:
      set_error_detail("gemm_ue8m0: unknown output dtype code %d", c_dtype);
      return B200_E_BAD_ARG;
  }
}
