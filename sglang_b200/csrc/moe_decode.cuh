// fused_experts for a handful of tokens (T <= 64): both grouped GEMMs with the operands swapped, as in the
// decode linear. A few tokens per expert make the layer a weight stream; the 128 x 256 tile kernel then
// promotes a whole tile per K block for a few real rows and needs whole waves of tiles to reach the HBM
// rate. Here
//   * a work item is (routed expert, 128-row weight tile[, K split]); 128 weight rows fill the UMMA M
//     dimension and the expert's <= NT tokens are its N, so a promotion thread owns one weight row and NT
//     accumulators; two CTAs per SM (one for NT = 64) keep every item streaming at once;
//   * there is no align / gather pass: every CTA finds its expert and that expert's (token, slot) pairs in
//     topk_ids itself (a few hundred ids from L2) and quantises / gathers the token rows it needs straight
//     into shared memory in the tensor core's 128-byte-swizzled layout;
//   * gate_up (STAGE 1): a weight tile is 64 gate rows + the matching 64 up rows, so silu(gate) * up is
//     formed in the epilogue (one exchange through shared memory) and written as fp32 rows [pair][I];
//   * down (STAGE 2): quantises those fp32 rows per 1x128 group itself (the oracle's arithmetic), applies
//     the router weight and writes fp32 partials [split][pair][H]; the slot / split sum is the existing
//     reduction kernel.
// Three launches (gate_up, down, sum) instead of five or six.
#pragma once

#include "gemm_host.cuh"

namespace b200 {

constexpr int kDecodeMaxIds = 1024;     // (token, slot) pairs a CTA scans
constexpr int kDecodeMaxExperts = 1024;

struct MoeDecodeParams {
  // routing
  const int32_t* topk_ids;     // [numel]
  const float* topk_weights;   // [numel]
  int numel, topk, E;
  // STAGE 1 input: 16-bit rows [T, K] (x_q == nullptr) or FP8 rows + row-major scales [T, K/128]
  const void* x;
  const uint8_t* x_q;
  const float* x_s;
  // STAGE 2 input / STAGE 1 output: fp32 activation rows [numel, I]
  float* act;
  // weights: scales [E][rows/128][num_kb]
  const float* Bs;
  // STAGE 2 output: fp32 partials [k_splits][numel][H]
  float* partial;
  int K, num_kb;        // reduction size of this stage (H for gate_up, I for down)
  int n_out;            // output columns of this stage (I for gate_up, H for down)
  int n_tiles;          // weight tiles per expert: I/64 (gate_up), H/128 (down)
  int k_splits, kb_per_split;
  int weight_on_input;  // gate_up: multiply the product by the router weight before the activation
  int apply_weight;     // down: multiply the output by the router weight
  int* status;
};

template <int NT>
struct MoeDecodeCfg {
  static constexpr int kStages = NT == 64 ? 7 : (NT == 32 ? 4 : 5);  // two CTAs of NT <= 32 fit one SM's shared memory
  static constexpr int kCtasPerSm = NT == 64 ? 1 : 2;
  static constexpr int kStageW = 128 * kBK;
  static constexpr int kStageX = NT * kBK;
  static constexpr int kQuantWarps = NT == 64 ? 8 : 4;  // each thread quantises one or two (row, 16-element chunk) pairs per K block
  static constexpr int kThreads = (6 + kQuantWarps) * 32;  // 4 promotion warps, TMA producer, MMA issuer, quantiser warps
  // TMEM accumulator buffers: the tensor core runs this many K blocks ahead of the promotion warps, so the
  // commit -> tcgen05.ld -> arrive round trip (about a microsecond) is off the per-K-block path
  static constexpr int kAccBufs = 4;
  static constexpr int kTmemCols = kAccBufs * NT < 32 ? 32 : kAccBufs * NT;
  static constexpr int kMaxKb = 64;
  static constexpr int kScaleBytes = kMaxKb * NT * 4;
  static constexpr int kExchangeBytes = 64 * NT * 4;  // up rows handed to the gate rows' threads
  static constexpr int kMetaBytes = 2048;             // pair list, weights, expert bitmap
  static constexpr size_t kSmemBytes =
      (size_t)kStages * (kStageW + kStageX) + kScaleBytes + kExchangeBytes + kMetaBytes + 1024 + 256;
};

// 16 consecutive fp32 values -> registers
__device__ __forceinline__ void load16_f32(const float* p, float (&f)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 v = __ldcg(reinterpret_cast<const float4*>(p) + i);  // written by the kernel before this one
    f[4 * i] = v.x; f[4 * i + 1] = v.y; f[4 * i + 2] = v.z; f[4 * i + 3] = v.w;
  }
}

template <int NT, int STAGE, typename InT>
__global__ void __launch_bounds__(MoeDecodeCfg<NT>::kThreads, MoeDecodeCfg<NT>::kCtasPerSm)
moe_decode_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const MoeDecodeParams p) {
  using Cfg = MoeDecodeCfg<NT>;
  constexpr int S = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t sW = smem_base;
  const uint32_t sX = smem_base + S * Cfg::kStageW;
  uint8_t* sX_ptr = smem_al + (size_t)S * Cfg::kStageW;
  uint8_t* after = smem_al + (size_t)S * (Cfg::kStageW + Cfg::kStageX);
  float* scales = reinterpret_cast<float*>(after);                                  // [kb][NT]
  float* exchange = reinterpret_cast<float*>(after + Cfg::kScaleBytes);             // [64][NT]
  int* pairs = reinterpret_cast<int*>(after + Cfg::kScaleBytes + Cfg::kExchangeBytes);  // [NT] flat (token*topk+slot)
  float* pair_w = reinterpret_cast<float*>(pairs + 64);                             // [NT] router weights
  uint32_t* bitmap = reinterpret_cast<uint32_t*>(pairs + 128);                      // [32] experts present
  int* meta = pairs + 160;                                                          // [0] expert, [1] count
  uint64_t* bars = reinterpret_cast<uint64_t*>(after + Cfg::kScaleBytes + Cfg::kExchangeBytes + Cfg::kMetaBytes);
  const uint32_t bar0 = ptx::smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (S + s); };
  constexpr int NB = Cfg::kAccBufs;
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * S + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * S + NB + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * S + 2 * NB);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * S + 2 * NB + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kProducerWarp = 4, kMmaWarp = 5, kFirstQuantWarp = 6;

  // ---------------------------------------------------------------- which expert, which pairs
  // The routing (and, for the down stage, the activation rows) come from the kernels before this one.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x < 32) bitmap[threadIdx.x] = 0;
  if (threadIdx.x == 0) { meta[0] = -1; meta[1] = 0; *abort_flag = 0; }
  __syncthreads();
  for (int i = threadIdx.x; i < p.numel; i += blockDim.x) {
    const int e = __ldg(p.topk_ids + i);
    if (e >= 0 && e < p.E) atomicOr(bitmap + (e >> 5), 1u << (e & 31));
  }
  __syncthreads();
  if (warp == 0) {
    // the blockIdx.y-th expert present, in ascending id order
    const uint32_t word = bitmap[lane];
    const int cnt = __popc(word);
    int incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    const int want = blockIdx.y;
    const int before = incl - cnt;
    if (want >= before && want < incl) {
      uint32_t w = word;
      for (int k = 0; k < want - before; ++k) w &= w - 1;  // drop the lower set bits
      meta[0] = lane * 32 + (__ffs(w) - 1);
    }
    __syncwarp();
    const int expert = meta[0];
    // its pairs in ascending flat order (ballot compaction: deterministic)
    int n = 0;
    if (expert >= 0) {
      for (int base = 0; base < p.numel; base += 32) {
        const int i = base + lane;
        const bool hit = i < p.numel && __ldg(p.topk_ids + i) == expert;
        const uint32_t m = __ballot_sync(0xffffffffu, hit);
        const int pos = n + __popc(m & ((1u << lane) - 1));
        if (hit && pos < NT) {
          pairs[pos] = i;
          pair_w[pos] = __ldg(p.topk_weights + i);
        }
        n += __popc(m);
      }
      if (lane == 0) {
        if (n > NT) atomicCAS(p.status, 0, 3);  // more tokens for one expert than this kernel's token tile
        meta[1] = n < NT ? n : NT;
      }
    }
  }
  __syncthreads();
  const int expert = meta[0];
  const int cnt = meta[1];
  // every CTA of this grid has read what it needs from the kernels before: dependents may set up
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (expert < 0 || cnt == 0) return;  // fewer distinct experts than grid rows: nothing to do (before any allocation)

  const int tile = blockIdx.x % p.n_tiles;
  const int ks = blockIdx.x / p.n_tiles;
  const int kb0 = ks * p.kb_per_split, kb1 = min(p.num_kb, kb0 + p.kb_per_split);
  const int nkb = kb1 - kb0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      ptx::mbar_init(full_bar(s), 1 + Cfg::kQuantWarps);  // the producer's expect_tx + one arrival per quantiser warp
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < NB; ++b) {
      ptx::mbar_init(tfull_bar(b), 1);
      ptx::mbar_init(tempty_bar(b), 4);
    }
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

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------- weight stream (TMA)
    // gate_up: rows [tile*64, +64) of the expert's gate half and of its up half (w1 is [E][2*n_out][K]);
    // down: rows [tile*128, +128) of w2 [E][n_out][K]
    const int row_a = STAGE == 1 ? expert * 2 * p.n_out + tile * 64 : expert * p.n_out + tile * 128;
    const int row_b = row_a + p.n_out;
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
        const uint32_t d = sW + s * Cfg::kStageW;
        if (STAGE == 1) {
          ptx::tma_load_2d(d, &tmap_w, kb * kBK, row_a, full_bar(s));
          ptx::tma_load_2d(d + 64 * kBK, &tmap_w, kb * kBK, row_b, full_bar(s));
        } else {
          ptx::tma_load_2d(d, &tmap_w, kb * kBK, row_a, full_bar(s));
        }
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
    // ------------------------------------ quantiser warps: token rows -> FP8 stages in shared memory
    // They run ahead of the tensor core by up to S stages and fetch the rows of two K blocks at a time, so the
    // L2 round trip of the rows is never on the path of the weight stream.
    constexpr int kRowsPerThread = NT * 8 / (Cfg::kQuantWarps * 32);
    constexpr int kRowStep = Cfg::kQuantWarps * 4;  // rows covered by one pass of the quantiser threads
    const int tid = threadIdx.x - kFirstQuantWarp * 32;
    const int q_chunk = tid & 7;
    // raw bytes of one (row, 16-element chunk): 16 B of FP8, 32 B of 16-bit or 64 B of fp32 values
    constexpr bool kFp32Rows = STAGE == 2;
    constexpr int kRawRegs = kFp32Rows ? 4 : 2;
    struct Fetched {
      uint4 raw[kRawRegs];
      float sc;
    };
    const bool prequantised = STAGE == 1 && p.x_q != nullptr;
    auto fetch = [&](int j, int rr, Fetched& d) {
      const int kb = kb0 + j;
      const int row = (tid >> 3) + kRowStep * rr;
      const bool live = row < cnt && j < nkb;
#pragma unroll
      for (int i = 0; i < kRawRegs; ++i) d.raw[i] = make_uint4(0, 0, 0, 0);
      d.sc = 0.f;
      if (!live) return;
      if (prequantised) {
        // rows already quantised (expert-parallel receive area): bytes and scale as they are
        const int64_t tok = pairs[row] / p.topk;
        d.raw[0] = ld_nc_16(p.x_q + tok * p.K + kb * 128 + q_chunk * 16);
        if (q_chunk == 0) d.sc = __ldg(p.x_s + tok * p.num_kb + kb);
      } else if (STAGE == 1) {
        const InT* src = static_cast<const InT*>(p.x) + (int64_t)(pairs[row] / p.topk) * p.K + kb * 128 + q_chunk * 16;
        d.raw[0] = ld_nc_16(src);
        d.raw[1] = ld_nc_16(src + 8);
      } else {
        // written by the kernel before this one: L2 loads
        const uint4* src = reinterpret_cast<const uint4*>(p.act + (int64_t)pairs[row] * p.K + kb * 128 + q_chunk * 16);
#pragma unroll
        for (int i = 0; i < kRawRegs; ++i) d.raw[i] = __ldcg(src + i);
      }
    };
    auto emit = [&](int j, int rr, const Fetched& d) {
      const int row = (tid >> 3) + kRowStep * rr;
      const bool live = row < cnt;
      uint4 qv = d.raw[0];
      float sc = d.sc;
      if (!prequantised) {
        float f[16];
        if (kFp32Rows) {
          const float* e = reinterpret_cast<const float*>(d.raw);
#pragma unroll
          for (int i = 0; i < 16; ++i) f[i] = e[i];
        } else {
          const InT* e = reinterpret_cast<const InT*>(d.raw);
#pragma unroll
          for (int i = 0; i < 16; ++i) f[i] = to_f32<InT>(e[i]);
        }
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
        amax = fmaxf(group_max<8>(amax), 1e-10f);
        // 16-bit rows: the division-free evaluation that equals x / (amax / 448) on every 16-bit input;
        // fp32 rows (the activation between the two GEMMs): the division itself, as the oracle computes it
        sc = quant16(f, amax, STAGE == 1 ? B200_QUANT_DIV_CORRECTED : B200_QUANT_DIV, qv);
        if (!live) qv = make_uint4(0, 0, 0, 0);
      }
      const uint32_t off = (uint32_t)(row >> 3) * 1024u + (uint32_t)(row & 7) * 128u + (uint32_t)((q_chunk ^ (row & 7)) << 4);
      *reinterpret_cast<uint4*>(sX_ptr + (size_t)(j % S) * Cfg::kStageX + off) = qv;
      if (q_chunk == 0) scales[j * NT + row] = live ? sc : 0.f;
    };
    // Rows of kDepth K blocks are requested before any is used: under a saturated weight stream an L2 round
    // trip takes microseconds, and the quantisers must deliver a K block every ~0.5 us to keep the stream going.
    constexpr int kRegsPerBlock = kRawRegs * 4 * kRowsPerThread;  // registers one K block's rows occupy
    constexpr int kDepth = 64 / kRegsPerBlock > 4 ? 4 : 64 / kRegsPerBlock;
    static_assert(kDepth >= 2, "quantiser prefetch depth");
    bool ok = true;
    for (int j = 0; j < nkb && ok; j += kDepth) {
      Fetched d[kDepth][kRowsPerThread];
#pragma unroll
      for (int u = 0; u < kDepth; ++u)
#pragma unroll
        for (int rr = 0; rr < kRowsPerThread; ++rr) fetch(j + u, rr, d[u][rr]);
#pragma unroll
      for (int u = 0; u < kDepth; ++u) {
        const int jj = j + u;
        if (jj >= nkb) break;
        if (jj >= S) {  // the stage is free once the MMAs that read it have completed
          ok = ptx::mbar_wait(empty_bar(jj % S), ((jj / S) & 1) ^ 1, abort_flag);
          if (!ok) break;
        }
#pragma unroll
        for (int rr = 0; rr < kRowsPerThread; ++rr) emit(jj, rr, d[u][rr]);
        // generic-proxy writes -> visible to the tensor core's (async proxy) reads of this stage, and the
        // scale table to the promotion warps that read it after the MMA of this stage has completed
        __threadfence_block();
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(full_bar(jj % S));
      }
    }
  } else {
    // ------------------------------------------------------------ promotion warps (lane = weight row)
    // weight-scale rows: gate_up rows [tile*64..) live in block tile/2 of the gate half, the up rows in the
    // same block of the up half (n_out/128 blocks further); down: block `tile`
    const int blocks_per_expert = (STAGE == 1 ? 2 * p.n_out : p.n_out) / 128;
    const float* bs_a = p.Bs + ((int64_t)expert * blocks_per_expert + (STAGE == 1 ? tile / 2 : tile)) * p.num_kb;
    const float* bs_b = bs_a + (int64_t)(p.n_out / 128) * p.num_kb;  // STAGE 1: scales of the up rows
    const int r = warp * 32 + lane;  // weight row of the tile
    // the block scale of this thread's weight row for every K block of the item
    const float* bs_mine = STAGE == 1 && r >= 64 ? bs_b : bs_a;
    const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
    float acc[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t] = 0.f;
    bool ok = true;
    float bsc = __ldg(bs_mine + kb0);
    for (int j = 0; j < nkb; ++j) {
      const int b = j % NB;
      const float bsc_next = j + 1 < nkb ? __ldg(bs_mine + kb0 + j + 1) : 0.f;
      ok = ptx::mbar_wait(tfull_bar(b), (j / NB) & 1, abort_flag);
      if (!ok) break;
      ptx::tc_fence_after();
      uint32_t v[NT < 32 ? 32 : NT];
      if constexpr (NT == 16) {
        ptx::tmem_ld16(lane_base + b * NT, v);
        ptx::tmem_ld_wait16(v);
      } else if constexpr (NT == 32) {
        ptx::tmem_ld32(lane_base + b * NT, v);
        ptx::tmem_ld_wait(v);
      } else {
        ptx::tmem_ld64(lane_base + b * NT, v);
        ptx::tmem_ld_wait64(v);
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(tempty_bar(b));
      // written by the quantiser warps before they released this stage to the tensor core
      const float* sc = scales + (size_t)j * NT;
#pragma unroll
      for (int q = 0; q < NT / 4; ++q) {
        const float4 s4 = ld_shared_f4(sc + 4 * q);  // same address for every lane: broadcast
        acc[4 * q + 0] = fmaf(__uint_as_float(v[4 * q + 0]), s4.x * bsc, acc[4 * q + 0]);
        acc[4 * q + 1] = fmaf(__uint_as_float(v[4 * q + 1]), s4.y * bsc, acc[4 * q + 1]);
        acc[4 * q + 2] = fmaf(__uint_as_float(v[4 * q + 2]), s4.z * bsc, acc[4 * q + 2]);
        acc[4 * q + 3] = fmaf(__uint_as_float(v[4 * q + 3]), s4.w * bsc, acc[4 * q + 3]);
      }
      bsc = bsc_next;
    }
    // A wait that gave up must not leave the other warps alone at the named barrier below: all four warps
    // meet here and take the same branch on the CTA-wide abort flag.
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (!*abort_flag) {
      if (STAGE == 1) {
        if (p.weight_on_input) {
#pragma unroll
          for (int t = 0; t < NT; ++t) acc[t] *= pair_w[t < cnt ? t : 0];
        }
        // rows 64..127 (up) hand their sums to the threads of rows 0..63 (gate)
        if (r >= 64) {
#pragma unroll
          for (int t = 0; t < NT; ++t) exchange[(r - 64) * NT + t] = acc[t];
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (r < 64) {
          const int col = tile * 64 + r;
#pragma unroll
          for (int t = 0; t < NT; ++t)
            if (t < cnt) p.act[(int64_t)pairs[t] * p.n_out + col] = silu_mul_fast(acc[t], exchange[r * NT + t]);
        }
      } else {
        const int col = tile * 128 + r;
        float* out = p.partial + (int64_t)ks * p.numel * p.n_out + col;
#pragma unroll
        for (int t = 0; t < NT; ++t)
          if (t < cnt) out[(int64_t)pairs[t] * p.n_out] = p.apply_weight ? acc[t] * pair_w[t] : acc[t];
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

template <int NT, int STAGE, typename InT>
inline int launch_moe_decode(const void* W, int64_t w_rows, const MoeDecodeParams& p, int max_active, cudaStream_t st) {
  CUtensorMap tw;
  int rc = make_tmap_u8(&tw, W, (uint64_t)w_rows, (uint64_t)p.K, STAGE == 1 ? 64u : 128u, STAGE == 1 ? "w1 (64-row boxes)" : "w2");
  if (rc) return rc;
  auto k = moe_decode_gemm_kernel<NT, STAGE, InT>;
  const size_t smem = MoeDecodeCfg<NT>::kSmemBytes;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error_detail("cudaFuncSetAttribute(smem=%zu): %s", smem, cudaGetErrorString(e));
    return B200_E_LAUNCH;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(p.n_tiles * p.k_splits), (unsigned)max_active);
  cfg.blockDim = dim3(MoeDecodeCfg<NT>::kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, k, tw, p);
  if (e != cudaSuccess) {
    set_error_detail("moe_decode_gemm_kernel: %s", cudaGetErrorString(e));
    return B200_E_LAUNCH;
  }
  return check_launch("moe_decode_gemm_kernel");
}

}  // namespace b200
