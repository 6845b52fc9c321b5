// Decode-sized block-FP8 GEMM (M <= 64 rows of activations): the roles of the operands are
// swapped so that the 128 weight rows of a tile fill the 128 lanes of the tensor-core tile
// and the few tokens are its N dimension:
//     D[n, m] = sum_k W[n, k] * X[m, k]        (UMMA M = 128 weight rows, N = NT tokens)
// A thread of the promotion warps then owns ONE weight row and NT (16 or 32) token
// accumulators instead of 128, so the per-K-block TMEM -> register promotion that bounds the
// large-tile kernel at small M shrinks 4-8x and the kernel streams the weights at HBM rate.
// Work item = (128-row weight tile, token tile, K split); one CTA per item, two CTAs per SM.
// K splits write fp32 partials that splitk_reduce_kernel sums.
#pragma once

#include "gemm_host.cuh"

namespace b200 {

struct SkinnyParams {
  const float* As;  // As[m*as_sm + kb*as_sk]
  int64_t as_sm, as_sk;
  const float* Bs;  // [ceil(N/128)][num_kb]
  void* C;          // OutT [M, N], or fp32 partials [splits][M, N]
  int M, N, K, num_kb;
  int n_tiles, t_tiles, k_splits, kb_per_split;
  int* status;
};

template <int NT>
struct SkinnyCfg {
  static constexpr int kStages = 5;
  static constexpr int kStageW = 128 * kBK;  // 16 KB of weights
  static constexpr int kStageX = NT * kBK;   // 2 or 4 KB of activations
  static constexpr int kThreads = 6 * 32;    // 4 promotion warps, producer, MMA issuer
  // TMEM accumulator buffers: the tensor core runs this many K blocks ahead of the promotion warps, so the
  // commit -> tcgen05.ld -> arrive round trip (about a microsecond) is off the per-K-block path
  static constexpr int kAccBufs = 4;
  static constexpr int kTmemCols = kAccBufs * NT;
  static constexpr int kMaxKb = 64;          // K blocks one CTA may own (scales staged in smem)
  static constexpr size_t kSmemBytes =
      (size_t)kStages * (kStageW + kStageX) + (size_t)kMaxKb * NT * 4 + 1024 + 256;
};

template <int NT, typename OutT>
__global__ void __launch_bounds__(SkinnyCfg<NT>::kThreads, 2)
block_fp8_gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                             const SkinnyParams p) {
  using Cfg = SkinnyCfg<NT>;
  constexpr int S = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t sW = smem_base;
  const uint32_t sX = smem_base + S * Cfg::kStageW;
  float* scales = reinterpret_cast<float*>(smem_al + (size_t)S * (Cfg::kStageW + Cfg::kStageX));  // [kb][NT]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(scales) + (size_t)Cfg::kMaxKb * NT * 4);
  const uint32_t bar0 = ptx::smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (S + s); };
  constexpr int NB = Cfg::kAccBufs;
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * S + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * S + NB + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * S + 2 * NB);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * S + 2 * NB + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kProducerWarp = 4, kMmaWarp = 5;

  // work item
  const int item = blockIdx.x;
  const int ks = item % p.k_splits;
  const int tt = (item / p.k_splits) % p.t_tiles;
  const int nt = item / (p.k_splits * p.t_tiles);
  const int kb0 = ks * p.kb_per_split, kb1 = min(p.num_kb, kb0 + p.kb_per_split);
  const int n0 = nt * 128, m0 = tt * NT;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < NB; ++b) {
      ptx::mbar_init(tfull_bar(b), 1);
      ptx::mbar_init(tempty_bar(b), 4);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), Cfg::kTmemCols);
    ptx::tmem_relinquish();
  }
  if (warp == kProducerWarp && lane == 0) {
    ptx::prefetch_tensormap(&tmap_w);
    ptx::prefetch_tensormap(&tmap_x);
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // every CTA of this grid is running: a dependent grid (the split-K reduction) may be set up now;
  // it waits for this grid's completion before it reads anything
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // The producer and the MMA issuer start at once; meanwhile the promotion warps stage
  // As[m, kb] * Bs[n0/128, kb] for this item's tokens and K blocks in shared memory (their own
  // 128-thread barrier: only they read the table), so the first weight tiles are already in
  // flight while the scales are fetched.
  if (warp < 4) {
    // the activation scales (and, at the end, the output buffer) belong to the kernels before this
    // one in the stream: this grid is launched as their programmatic dependent, so wait for them here
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const float* bs_row = p.Bs + (int64_t)nt * p.num_kb;
    for (int i = threadIdx.x; i < (kb1 - kb0) * NT; i += 128) {
      const int kb = kb0 + i / NT, t = i % NT;
      const int m = m0 + t;
      scales[i] = m < p.M ? __ldg(p.As + (int64_t)m * p.as_sm + (int64_t)kb * p.as_sk) * __ldg(bs_row + kb) : 0.f;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
  }

  if (warp == kProducerWarp) {
    bool ok = true;
    // Prologue: the weights do not depend on the previous kernel, the quantised activations do.
    // The weight tiles of the first stages are requested before waiting for that kernel, so the
    // weight stream starts while it is still finishing.
    const int npro = min(S, kb1 - kb0);
    if (lane == 0) {
      for (int i = 0; i < npro; ++i) {
        ptx::mbar_expect_tx(full_bar(i), Cfg::kStageW + Cfg::kStageX);
        ptx::tma_load_2d(sW + i * Cfg::kStageW, &tmap_w, (kb0 + i) * kBK, n0, full_bar(i));
      }
      asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int i = 0; i < npro; ++i) ptx::tma_load_2d(sX + i * Cfg::kStageX, &tmap_x, (kb0 + i) * kBK, m0, full_bar(i));
    }
    __syncwarp();
    uint32_t it = npro;
    for (int kb = kb0 + npro; kb < kb1 && ok; ++kb, ++it) {
      const int s = it % S;
      ok = ptx::mbar_wait(empty_bar(s), ((it / S) & 1) ^ 1, abort_flag);
      if (!ok) break;
      if (lane == 0) {
        ptx::mbar_expect_tx(full_bar(s), Cfg::kStageW + Cfg::kStageX);
        ptx::tma_load_2d(sW + s * Cfg::kStageW, &tmap_w, kb * kBK, n0, full_bar(s));
        ptx::tma_load_2d(sX + s * Cfg::kStageX, &tmap_x, kb * kBK, m0, full_bar(s));
      }
      __syncwarp();
    }
  } else if (warp == kMmaWarp) {
    constexpr uint32_t idesc = ptx::idesc_e4m3_f32(128, NT);
    bool ok = true;
    uint32_t it = 0;
    for (int kb = kb0; kb < kb1 && ok; ++kb, ++it) {
      const int s = it % S, b = it % NB;
      ok = ptx::mbar_wait(tempty_bar(b), ((it / NB) & 1) ^ 1, abort_flag) &&
           ptx::mbar_wait(full_bar(s), (it / S) & 1, abort_flag);
      if (!ok) break;
      ptx::tc_fence_after();
      if (lane == 0) {
        const uint64_t dw = ptx::smem_desc_sw128(sW + s * Cfg::kStageW);
        const uint64_t dx = ptx::smem_desc_sw128(sX + s * Cfg::kStageX);
        const uint32_t d = tmem_base + b * NT;
#pragma unroll
        for (int k = 0; k < kBK / 32; ++k) ptx::mma_f8(d, dw + 2 * k, dx + 2 * k, idesc, k > 0);
        ptx::mma_commit(empty_bar(s));
        ptx::mma_commit(tfull_bar(b));
      }
      __syncwarp();
    }
  } else {
    // promotion warps: lane = weight row, columns = tokens
    const int n = n0 + warp * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
    float acc[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t] = 0.f;
    bool ok = true;
    uint32_t it = 0;
    for (int kb = kb0; kb < kb1; ++kb, ++it) {
      const int b = it % NB;
      ok = ptx::mbar_wait(tfull_bar(b), (it / NB) & 1, abort_flag);
      if (!ok) break;
      ptx::tc_fence_after();
      uint32_t v[32];
      if (NT == 32) {
        ptx::tmem_ld32(lane_base + b * NT, v);
        ptx::tmem_ld_wait(v);
      } else {
        ptx::tmem_ld16(lane_base + b * NT, v);
        ptx::tmem_ld_wait16(v);
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(tempty_bar(b));
      const float4* sc = reinterpret_cast<const float4*>(scales + (size_t)(kb - kb0) * NT);
#pragma unroll
      for (int j = 0; j < NT / 4; ++j) {
        const float4 s4 = sc[j];  // same address for every lane: broadcast
        acc[4 * j + 0] = fmaf(__uint_as_float(v[4 * j + 0]), s4.x, acc[4 * j + 0]);
        acc[4 * j + 1] = fmaf(__uint_as_float(v[4 * j + 1]), s4.y, acc[4 * j + 1]);
        acc[4 * j + 2] = fmaf(__uint_as_float(v[4 * j + 2]), s4.z, acc[4 * j + 2]);
        acc[4 * j + 3] = fmaf(__uint_as_float(v[4 * j + 3]), s4.w, acc[4 * j + 3]);
      }
    }
    if (ok && n < p.N) {
      OutT* out = static_cast<OutT*>(p.C) + (int64_t)ks * p.M * p.N + n;
#pragma unroll
      for (int t = 0; t < NT; ++t)
        if (m0 + t < p.M) out[(int64_t)(m0 + t) * p.N] = from_f32<OutT>(acc[t]);  // 32 lanes -> 32 consecutive n
    }
  }

  if (*abort_flag) {
    const unsigned long long t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicCAS(p.status, 0, 1);
  if (warp == kMmaWarp) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// Number of K splits for the skinny kernel: about two work items per SM, each with at least
// two K blocks and at most kMaxKb.
inline int skinny_k_splits(int64_t M, int64_t N, int64_t K, int nt, int sms) {
  const int64_t items = cdiv(N, 128) * cdiv(M, nt);
  const int64_t num_kb = cdiv(K, 128);
  int64_t s = (2 * (int64_t)sms) / items;
  if (s > num_kb / 2) s = num_kb / 2;
  if (s < 1) s = 1;
  const int64_t need = cdiv(num_kb, 64);  // a CTA stages the scales of at most 64 K blocks
  if (s < need) s = need;
  if (s > 16) s = 16 > need ? 16 : need;
  return (int)s;
}

inline int skinny_token_tile(int64_t M) { return M <= 16 ? 16 : 32; }

template <int NT, typename OutT>
inline int launch_skinny_inst(const CUtensorMap& tw, const CUtensorMap& tx, const SkinnyParams& p, cudaStream_t st) {
  auto k = block_fp8_gemm_skinny_kernel<NT, OutT>;
  const size_t smem = SkinnyCfg<NT>::kSmemBytes;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error_detail("cudaFuncSetAttribute(smem=%zu): %s", smem, cudaGetErrorString(e));
    return B200_E_LAUNCH;
  }
  const int grid = p.n_tiles * p.t_tiles * p.k_splits;
  // programmatic dependent of the kernel before it (normally the activation quantiser, which
  // signals launch_dependents at once): set-up and the first weight loads overlap its tail
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(SkinnyCfg<NT>::kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, k, tw, tx, p);
  if (e != cudaSuccess) {
    set_error_detail("block_fp8_gemm_skinny_kernel: %s", cudaGetErrorString(e));
    return B200_E_LAUNCH;
  }
  return check_launch("block_fp8_gemm_skinny_kernel");
}

// out: OutT [M, N] when splits == 1, else fp32 partials [splits][M, N].
template <typename OutT>
inline int launch_skinny(const void* X, const void* W, SkinnyParams p, int splits, cudaStream_t st) {
  const int nt = skinny_token_tile(p.M);
  p.num_kb = (int)cdiv(p.K, kBK);
  p.n_tiles = (int)cdiv(p.N, 128);
  p.t_tiles = (int)cdiv(p.M, nt);
  p.k_splits = splits;
  p.kb_per_split = (int)cdiv(p.num_kb, splits);
  p.status = device_status_word();
  if (!p.status) {
    set_error_detail("cannot resolve the device status word");
    return B200_E_LAUNCH;
  }
  CUtensorMap tw, tx;
  int rc = make_tmap_u8(&tw, W, (uint64_t)p.N, (uint64_t)p.K, 128, "W");
  if (rc) return rc;
  rc = make_tmap_u8(&tx, X, (uint64_t)p.M, (uint64_t)p.K, (uint32_t)nt, "X");
  if (rc) return rc;
  if (nt == 16) return launch_skinny_inst<16, OutT>(tw, tx, p, st);
  return launch_skinny_inst<32, OutT>(tw, tx, p, st);
}

}  // namespace b200
