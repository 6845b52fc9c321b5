// Decode-sized quantised linear in ONE launch (M <= 16 rows of 16-bit activations):
//     out[m, n] = sum_kb (q(x)[m, kb] . W[n, kb]) * xs[m, kb] * Bs[n/128, kb]
// where q / xs are the 1x128 group quantisation of x. The separate sequence
// quantiser -> decode GEMM -> split-K sum costs three launches before a weight byte moves; here
//  * every CTA quantises the <= 16 x (its K range) slice of x it needs itself (a few KB, read from
//    L2), writing the FP8 bytes straight into shared memory in the 128-byte-swizzled K-major layout
//    the tensor core reads (what a TMA load of the quantised activations would have produced), with
//    the arithmetic of the stand-alone quantiser (bit-identical bytes and scales);
//  * the weight tiles stream by TMA exactly as in the decode GEMM (operands swapped: 128 weight rows
//    are the UMMA M dimension, the 16 tokens its N);
//  * K splits write fp32 partials and take a ticket per weight tile; the CTA that draws the last
//    ticket sums the partials in split order (deterministic) and writes the 16-bit result, then
//    resets the ticket, so the ticket array only has to be zero before the first call.
// Work item = (128-row weight tile, K split); two CTAs per SM.
#pragma once

#include "gemm_skinny.cuh"

namespace b200 {

struct DecodeLinearParams {
  const void* x;     // [M, K] bf16 / f16, row-major
  const float* Bs;   // [ceil(N/128)][num_kb]
  void* out;         // OutT [M, N]
  float* partial;    // fp32 [k_splits][M][N] (k_splits > 1)
  unsigned* tickets; // [n_tiles], zero before the first call; left zero by every call
  int M, N, K, num_kb;
  int n_tiles, k_splits, kb_per_split;
  float eps;
  int* status;
};

struct DecodeLinearCfg {
  static constexpr int NT = 16;
  static constexpr int kStages = 5;
  static constexpr int kStageW = 128 * kBK;  // 16 KB of weights
  static constexpr int kStageX = NT * kBK;   // 2 KB of quantised activations
  static constexpr int kThreads = 10 * 32;   // 4 promotion warps, TMA producer, MMA issuer, 4 quantiser warps
  // TMEM accumulator buffers: the tensor core runs this many K blocks ahead of the promotion warps, so the
  // commit -> tcgen05.ld -> arrive round trip (about a microsecond) is off the per-K-block path
  static constexpr int kAccBufs = 4;
  static constexpr int kTmemCols = kAccBufs * NT;
  static constexpr int kMaxKb = 64;          // K blocks one CTA may own (scales staged in smem)
  static constexpr size_t kSmemBytes = (size_t)kStages * (kStageW + kStageX) + (size_t)kMaxKb * NT * 4 + 1024 + 256;
};

template <typename InT, typename OutT>
__global__ void __launch_bounds__(DecodeLinearCfg::kThreads, 2)
block_fp8_linear_decode_kernel(const __grid_constant__ CUtensorMap tmap_w, const DecodeLinearParams p) {
  using Cfg = DecodeLinearCfg;
  constexpr int S = Cfg::kStages, NT = Cfg::NT;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t sW = smem_base;
  const uint32_t sX = smem_base + S * Cfg::kStageW;
  uint8_t* sX_ptr = smem_al + (size_t)S * Cfg::kStageW;
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
  volatile int* last_flag = reinterpret_cast<volatile int*>(bars + 2 * S + 2 * NB + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kProducerWarp = 4, kMmaWarp = 5, kFirstQuantWarp = 6;

  const int item = blockIdx.x;
  const int ks = item % p.k_splits;
  const int nt = item / p.k_splits;
  const int kb0 = ks * p.kb_per_split, kb1 = min(p.num_kb, kb0 + p.kb_per_split);
  const int nkb = kb1 - kb0;
  const int n0 = nt * 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      ptx::mbar_init(full_bar(s), 1 + 4);  // the producer's expect_tx + one arrival per quantising warp
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < NB; ++b) {
      ptx::mbar_init(tfull_bar(b), 1);
      ptx::mbar_init(tempty_bar(b), 4);
    }
    *abort_flag = 0;
    *last_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), Cfg::kTmemCols);
    ptx::tmem_relinquish();
  }
  if (warp == kProducerWarp && lane == 0) ptx::prefetch_tensormap(&tmap_w);
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // every CTA of this grid is running: the next kernel of the stream may set itself up
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------- weight stream (TMA)
    // the weights do not depend on the kernel before this one: no griddepcontrol.wait here
    bool ok = true;
    uint32_t it = 0;
    for (int kb = kb0; kb < kb1 && ok; ++kb, ++it) {
      const int s = it % S;
      if (it >= (uint32_t)S) {
        ok = ptx::mbar_wait(empty_bar(s), ((it / S) & 1) ^ 1, abort_flag);
        if (!ok) break;
      }
      if (lane == 0) {
        ptx::mbar_expect_tx(full_bar(s), Cfg::kStageW);
        ptx::tma_load_2d(sW + s * Cfg::kStageW, &tmap_w, kb * kBK, n0, full_bar(s));
      }
      __syncwarp();
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------- MMA issuer
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
  } else if (warp >= kFirstQuantWarp) {
    // --------------------------------------------------- quantiser warps: x -> FP8 stages
    // They run ahead of the tensor core by up to S stages and fetch the rows of two K blocks at a time, so the
    // L2 round trip of x is never on the path of the weight stream.
    // x (and the output / partial buffers) may belong to the kernel before this one in the stream
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int tid = threadIdx.x - kFirstQuantWarp * 32;  // 0..127
    const int q_row = tid >> 3;                            // token row this thread quantises (8 threads per row)
    const int q_chunk = tid & 7;                           // 16-element chunk of the 128-wide group
    const bool q_live = q_row < p.M;
    const InT* x_row = static_cast<const InT*>(p.x) + (int64_t)(q_live ? q_row : 0) * p.K + q_chunk * 16;
    const float* bs_row = p.Bs + (int64_t)nt * p.num_kb;
    // byte offset of (row, chunk) inside a stage: 8-row groups of 1024 bytes, 16-byte chunk index
    // XORed with the row index inside the group (the 128-byte swizzle of the UMMA descriptor)
    const uint32_t q_off = (uint32_t)(q_row >> 3) * 1024u + (uint32_t)(q_row & 7) * 128u +
                           (uint32_t)((q_chunk ^ (q_row & 7)) << 4);
    // raw 16-bit elements of one (row, chunk): two 16-byte registers
    auto fetch = [&](int j, uint4 (&raw)[2], float& bs) {
      const int kb = kb0 + j;
      const bool in = q_live && j < nkb && kb * 128 + q_chunk * 16 < p.K;
      const InT* src = x_row + (int64_t)kb * 128;
      raw[0] = in ? ld_nc_16(src) : make_uint4(0, 0, 0, 0);
      raw[1] = in ? ld_nc_16(src + 8) : make_uint4(0, 0, 0, 0);
      bs = q_live && j < nkb && q_chunk == 0 ? __ldg(bs_row + kb) : 0.f;
    };
    auto emit = [&](int j, const uint4 (&raw)[2], float bs) {  // K block kb0 + j -> stage j % S, scales[j][*]
      float f[16];
      const InT* e = reinterpret_cast<const InT*>(raw);
#pragma unroll
      for (int i = 0; i < 16; ++i) f[i] = to_f32<InT>(e[i]);
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
      amax = fmaxf(group_max<8>(amax), p.eps);
      uint4 qv;
      const float sc = quant16(f, amax, B200_QUANT_DIV_CORRECTED, qv);
      if (!q_live) qv = make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(sX_ptr + (size_t)(j % S) * Cfg::kStageX + q_off) = qv;
      if (q_chunk == 0) scales[j * NT + q_row] = q_live ? sc * bs : 0.f;
      // generic-proxy writes -> visible to the tensor core's (async proxy) reads of this stage, and the
      // scale table to the promotion warps that read it after the MMA of this stage has completed
      __threadfence_block();
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(full_bar(j % S));
    };
    // Rows of kDepth K blocks are requested before any is used: under a saturated weight stream an L2 round
    // trip takes microseconds, and the quantiser must deliver a K block every ~0.5 us to keep the stream going.
    constexpr int kDepth = 4;
    bool ok = true;
    for (int j = 0; j < nkb && ok; j += kDepth) {
      uint4 raw[kDepth][2];
      float bs[kDepth];
#pragma unroll
      for (int u = 0; u < kDepth; ++u) fetch(j + u, raw[u], bs[u]);
#pragma unroll
      for (int u = 0; u < kDepth; ++u) {
        const int jj = j + u;
        if (jj >= nkb) break;
        if (jj >= S) {  // the stage is free once the MMAs that read it have completed
          ok = ptx::mbar_wait(empty_bar(jj % S), ((jj / S) & 1) ^ 1, abort_flag);
          if (!ok) break;
        }
        emit(jj, raw[u], bs[u]);
      }
    }
  } else {
    // ------------------------------------------------------------ promotion warps (lane = weight row)
    asm volatile("griddepcontrol.wait;" ::: "memory");  // they write the output / partials at the end
    const int tid = threadIdx.x;  // 0..127
    const int n = n0 + warp * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
    float acc[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t] = 0.f;
    bool ok = true;
    for (int j = 0; j < nkb; ++j) {
      const int b = j % NB;
      ok = ptx::mbar_wait(tfull_bar(b), (j / NB) & 1, abort_flag);
      if (!ok) break;
      ptx::tc_fence_after();
      uint32_t v[32];
      ptx::tmem_ld16(lane_base + b * NT, v);
      ptx::tmem_ld_wait16(v);
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(tempty_bar(b));
      // written by the quantiser warps before they released this stage to the tensor core
      const float* sc = scales + (size_t)j * NT;
#pragma unroll
      for (int q = 0; q < NT / 4; ++q) {
        const float4 s4 = ld_shared_f4(sc + 4 * q);  // same address for every lane: broadcast
        acc[4 * q + 0] = fmaf(__uint_as_float(v[4 * q + 0]), s4.x, acc[4 * q + 0]);
        acc[4 * q + 1] = fmaf(__uint_as_float(v[4 * q + 1]), s4.y, acc[4 * q + 1]);
        acc[4 * q + 2] = fmaf(__uint_as_float(v[4 * q + 2]), s4.z, acc[4 * q + 2]);
        acc[4 * q + 3] = fmaf(__uint_as_float(v[4 * q + 3]), s4.w, acc[4 * q + 3]);
      }
    }
    // A wait that gave up must not leave the other warps alone at the named barriers below: all four warps
    // meet here and take the same branch on the CTA-wide abort flag.
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (!*abort_flag) {
      if (p.k_splits == 1) {
        if (n < p.N) {
          OutT* out = static_cast<OutT*>(p.out) + n;
#pragma unroll
          for (int t = 0; t < NT; ++t)
            if (t < p.M) out[(int64_t)t * p.N] = from_f32<OutT>(acc[t]);  // 32 lanes -> 32 consecutive n
        }
      } else {
        const int64_t mn = (int64_t)p.M * p.N;
        if (n < p.N) {
          float* part = p.partial + (int64_t)ks * mn + n;
#pragma unroll
          for (int t = 0; t < NT; ++t)
            if (t < p.M) part[(int64_t)t * p.N] = acc[t];
        }
        // ticket: the CTA that arrives last at this weight tile sums the partials
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (tid == 0) {
          const unsigned old = atomicAdd(p.tickets + nt, 1u);
          *last_flag = old == (unsigned)p.k_splits - 1;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*last_flag) {
          __threadfence();
          if (n < p.N) {
#pragma unroll
            for (int t = 0; t < NT; ++t) {
              if (t >= p.M) break;
              float sum = 0.f;
              for (int s = 0; s < p.k_splits; ++s) sum += __ldcg(p.partial + (int64_t)s * mn + (int64_t)t * p.N + n);
              static_cast<OutT*>(p.out)[(int64_t)t * p.N + n] = from_f32<OutT>(sum);
            }
          }
          if (tid == 0) p.tickets[nt] = 0;  // ready for the next call
        }
      }
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

// K splits for the fused decode linear: about two work items per SM, each with at least two K
// blocks and at most kMaxKb.
inline int decode_linear_k_splits(int64_t N, int64_t K, int sms) {
  const int64_t items = cdiv(N, 128);
  const int64_t num_kb = cdiv(K, 128);
  int64_t s = (2 * (int64_t)sms) / items;
  if (s > num_kb / 2) s = num_kb / 2;
  if (s < 1) s = 1;
  const int64_t need = cdiv(num_kb, DecodeLinearCfg::kMaxKb);
  if (s < need) s = need;
  if (s > 16) s = 16 > need ? 16 : need;
  return (int)s;
}

template <typename InT, typename OutT>
inline int launch_decode_linear(const void* W, DecodeLinearParams p, cudaStream_t st) {
  CUtensorMap tw;
  int rc = make_tmap_u8(&tw, W, (uint64_t)p.N, (uint64_t)p.K, 128, "W");
  if (rc) return rc;
  auto k = block_fp8_linear_decode_kernel<InT, OutT>;
  const size_t smem = DecodeLinearCfg::kSmemBytes;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error_detail("cudaFuncSetAttribute(smem=%zu): %s", smem, cudaGetErrorString(e));
    return B200_E_LAUNCH;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(p.n_tiles * p.k_splits));
  cfg.blockDim = dim3(DecodeLinearCfg::kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  // programmatic dependent of the kernel before it: the weight stream starts while that kernel drains
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, k, tw, p);
  if (e != cudaSuccess) {
    set_error_detail("block_fp8_linear_decode_kernel: %s", cudaGetErrorString(e));
    return B200_E_LAUNCH;
  }
  return check_launch("block_fp8_linear_decode_kernel");
}

}  // namespace b200
