// Block-FP8 GEMM for sm_100a: C[m,n] = sum_kb (A_kb . B_kb^T)[m,n] * As[m,kb] * Bs[n/128,kb].
//
// One persistent CTA per SM walks output tiles of 128 x BN (BN = 128 or 256). Roles:
//   warps [0, BN/32)  "promotion" warps: per K block they pull the fp32 partial product out
//                     of TMEM (tcgen05.ld), multiply by the two block scales and accumulate
//                     in registers (128 accumulators per thread); at the end of a tile they
//                     convert and store the row they own.
//   warp  BN/32       TMA producer: cp.async.bulk.tensor (128-byte swizzle, no multicast)
//                     of the A [128 x 128 B] and B [BN x 128 B] tiles into an S-stage ring.
//   warp  BN/32 + 1   MMA issuer: 4 x tcgen05.mma (K = 32 each) per K block into one of two
//                     TMEM accumulator buffers, tcgen05.commit to free the smem stage and to
//                     hand the buffer to the promotion warps.
// Because fp32 block scales change every 128 of K, the tensor core never accumulates
// across K blocks: TMEM is a double-buffered staging area and the running sum lives in
// registers, so the MMA of block k+1 overlaps the promotion of block k.
//
// The same kernel serves the dense linear (MODE 0) and the two grouped MoE GEMMs, whose
// A rows are laid out in expert-sorted, 128-row-padded order:
//   MODE 1 (gate_up): the B tile interleaves 64-row chunks of the expert's gate and up rows
//           (gate[0,64) | up[0,64) | gate[64,128) | up[64,128) of one 128-wide output group), so
//           every promotion thread holds gate AND up of the same 64 columns; the tile epilogue
//           computes silu(gate)*up in fp32 and re-quantises it to FP8 with its 1x128 scale
//           straight from the accumulators (no 16-bit round trip, no exchange of operands);
//   MODE 2 (down): rows are scattered to their (token, slot) position, times the router weight.
#pragma once

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace b200 {

enum { GEMM_DENSE = 0, GEMM_GROUPED_SILU_QUANT = 1, GEMM_GROUPED_SCATTER = 2 };

// Division by a divisor fixed at launch as a multiply-high and a shift (exact for 0 <= n < 2^31): the 32-bit
// integer division of the hardware is a ~25-instruction dependent chain, and three of them in a row sat on the
// critical path between two tiles of the promotion warps.
struct FastDiv {
  uint32_t mul, shr;
};
inline FastDiv make_fastdiv(int d) {
  FastDiv f = {0u, 0u};
  if (d <= 1) return f;  // mul == 0 marks "divide by one"
  int l = 0;
  while ((1ll << l) < d) ++l;  // ceil(log2 d)
  const int p = 31 + l;
  f.mul = (uint32_t)(((1ull << p) + (uint64_t)d - 1) / (uint64_t)d);
  f.shr = (uint32_t)(p - 32);
  return f;
}
__device__ __forceinline__ int fast_div(int n, FastDiv f) {
  return f.mul == 0u ? n : (int)(__umulhi((uint32_t)n, f.mul) >> f.shr);
}

struct GemmParams {
  const float* As;  // A scales: As[m*as_sm + kb*as_sk]
  int64_t as_sm, as_sk;
  const float* Bs;  // [experts][n_blocks][num_kb]
  void* C;
  int64_t ldc;     // elements
  int M, N, K;     // M = rows of A (grouped: capacity of the sorted layout)
  int num_kb;      // ceil(K/128)
  int n_blocks;    // ceil(N/128): rows of Bs per expert
  int n_tiles;     // ceil(N/BN)
  int m_tiles;     // ceil(M/128) (grouped: upper bound; the live count is read on device)
  int group_m;     // tiles of M swept together for L2 reuse (a power of two)
  FastDiv per_group_div, k_splits_div;  // division by group_m * n_tiles and by k_splits
  // split-K (dense, small problems): work item = (tile, split); split s covers K blocks
  // [s*kb_per_split, ...) and writes an fp32 partial at C + s*split_stride
  int k_splits, kb_per_split;
  int64_t split_stride;
  // grouped modes
  const int32_t* expert_ids;    // [m_tiles] expert of every 128-row block, -1 = skip
  const int32_t* num_post_pad;  // [1] live rows (multiple of 128)
  const int32_t* sorted_ids;    // [M] flat (token*topk+slot) index of every row, >= numel = pad
  const float* topk_weights;    // [numel] router weight per (token, slot); null = no weighting in this GEMM
  int numel;
  // MODE 1 outputs: FP8 activation [M, N] (N = intermediate size I; B holds 2I rows per
  // expert) and its scales, column-major: q_scales[(n/128)*q_scale_ld + row]
  uint8_t* q_out;
  float* q_scales;
  int64_t q_scale_ld;
  int* status;  // device status word
  // Fan-out (dense mode, tensor-parallel row-parallel linear): n_dest > 0 sends every finished
  // tile to the [M, N] buffers dest[0..n_dest) instead of C; they may be peer GPUs' memory (the
  // bulk tensor stores and 16-byte stores below cross NVLink like any store). dest_by_tile != 0
  // sends the tile of row block mt only to dest[mt % n_dest] (its owner in a reduce-scatter).
  int n_dest, dest_by_tile;
  void* dest[8];
  // Scatter mode over several buffers (expert-parallel combine by push): the row of pair `flat` goes to
  // dest[flat / scatter_rows_per_dest], row flat % scatter_rows_per_dest -- the source rank's own
  // [tokens x slots, N] area, possibly over NVLink. 0 = one buffer, C.
  int scatter_rows_per_dest;
  FastDiv scatter_div;
};

constexpr int kMaxFan = 8;
// Output tensor maps of one launch: one, or one per fan-out destination.
template <int FAN>
struct alignas(64) TmapOut {
  CUtensorMap m[FAN];
};

constexpr int kBM = 128;
constexpr int kBK = 128;  // bytes == elements (fp8) == one scale block == one swizzle row

template <int BN>
struct GemmCfg {
  static constexpr int kEpiWarps = BN / 32;  // 4 or 8: warp e -> TMEM lanes 32*(e%4), columns 128*(e/4)
  // BN = 256 runs three full warpgroups (8 promotion warps; producer, MMA issuer and two idle
  // warps) so that registers can be moved between warpgroups with setmaxnreg.
  static constexpr int kThreads = BN == 256 ? 384 : (kEpiWarps + 2) * 32;
  static constexpr bool kRebalanceRegs = BN == 256;
  static constexpr int kRegsPromotion = 224, kRegsOther = 56;  // 256*224 + 128*56 = 64512 <= 65536
  static constexpr int kStageA = kBM * kBK;
  static constexpr int kStageB = BN * kBK;
  static constexpr int kTmemCols = 2 * BN;  // two accumulator buffers
  // Register budget: the register file is split over the four SM sub-partitions (16 K each).
  // 12 warps start with 168 registers each (3 warps per sub-partition); the promotion warps,
  // which hold 128 accumulators + 64 staged TMEM values, then grow to 224 with setmaxnreg
  // while the producer / MMA warpgroup shrinks to 56 (2*224 + 56 = 504 <= 512 per sub-partition).
  static constexpr int kExchangeBytes = 2 * kBM * 4;  // MODE 1: partial row amax of the two column halves
};

// Shared-memory plan of one instantiation. The promotion warps stage their part of the output
// tile (32 rows x 128 columns per warp) in shared memory and write it out asynchronously: in the
// TMA 128-byte-swizzled box layout with bulk tensor stores (dense, gate_up), or (scatter) row-major
// with a 16-byte pad per row -- conflict-free for one 16-byte chunk per lane -- and one untiled bulk
// copy per row, issued by the lane that owns the row. A thread owns a whole row, so direct stores
// would touch 32 different rows per instruction, and plain stores out of the staging area stall the
// promotion warps while 64 KB per tile drain through the store queue. Staging is used by the 256-wide tile with 16-bit / FP8 output (the shapes
// where the epilogue is on the critical path); fp32 output and the 128-wide tile (small
// problems, split-K partials) keep direct row stores.
template <int BN, int MODE, typename OutT>
struct GemmLayout {
  using Cfg = GemmCfg<BN>;
  static constexpr int kRowBytes = MODE == GEMM_GROUPED_SILU_QUANT ? 128 : 128 * (int)sizeof(OutT);  // per thread
  static constexpr bool kStaged = BN == 256 && kRowBytes <= 256;
  static constexpr int kBoxesPerWarp = kRowBytes / 128;     // boxes of 32 rows x 128 bytes
  static constexpr int kRowStride = MODE == GEMM_GROUPED_SCATTER ? kRowBytes + 16 : kRowBytes;  // scatter: padded rows
  static constexpr int kWarpStageBytes = 32 * kRowStride;   // 4, 8 or 16 KB (+ 512 B of padding)
  static constexpr int kStoreWarps = MODE == GEMM_GROUPED_SILU_QUANT ? 4 : Cfg::kEpiWarps;
  static constexpr int kStagingBytes =
      (MODE == GEMM_GROUPED_SILU_QUANT ? Cfg::kExchangeBytes : 0) + (kStaged ? kStoreWarps * kWarpStageBytes : 0);
  static_assert(Cfg::kExchangeBytes == 1024, "row-amax exchange: two halves x 128 rows of fp32");
  static constexpr int kSmemLimit = 232448;  // 227 KB per CTA
  static constexpr int kFit = (kSmemLimit - 1024 - 256 - kStagingBytes) / (Cfg::kStageA + Cfg::kStageB);
  static constexpr int kStages = kFit > (BN == 256 ? 4 : 6) ? (BN == 256 ? 4 : 6) : kFit;
  static constexpr size_t kSmemBytes = (size_t)kStages * (Cfg::kStageA + Cfg::kStageB) + kStagingBytes + 1024 + 256;
  static_assert(kStages >= 3, "pipeline too shallow");
};

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// silu(g) * u = g * u * (0.5 + 0.5 * tanh(g / 2)) with the hardware tanh: one special-function
// instruction per element instead of an exponential and a reciprocal (the special-function unit issues
// a warp instruction every 8 cycles and was half of this epilogue). Relative error of tanh.approx.f32
// about 2^-11: far below the FP8 quantisation step (2^-4) that follows.
__device__ __forceinline__ float silu_mul_fast(float g, float u) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * g));
  return (g * u) * fmaf(0.5f, t, 0.5f);
}

// eight floats -> eight 16-bit values in one 16-byte register quad
template <typename OutT>
__device__ __forceinline__ uint4 pack8(const float* a);
template <>
__device__ __forceinline__ uint4 pack8<__nv_bfloat16>(const float* a) {
  uint4 v;
  __nv_bfloat162 t;
  t = __floats2bfloat162_rn(a[0], a[1]); v.x = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(a[2], a[3]); v.y = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(a[4], a[5]); v.z = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(a[6], a[7]); v.w = *reinterpret_cast<uint32_t*>(&t);
  return v;
}
template <>
__device__ __forceinline__ uint4 pack8<__half>(const float* a) {
  uint4 v;
  __half2 t;
  t = __floats2half2_rn(a[0], a[1]); v.x = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2half2_rn(a[2], a[3]); v.y = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2half2_rn(a[4], a[5]); v.z = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2half2_rn(a[6], a[7]); v.w = *reinterpret_cast<uint32_t*>(&t);
  return v;
}
template <>
__device__ __forceinline__ uint4 pack8<float>(const float* a) {  // never staged; keeps the template total
  return make_uint4(__float_as_uint(a[0]), __float_as_uint(a[1]), __float_as_uint(a[2]), __float_as_uint(a[3]));
}

template <typename OutT>
__device__ __forceinline__ void store8(OutT* dst, const float* a);
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* dst, const float* a) {
  uint4 v;
  __nv_bfloat162 t;
  t = __floats2bfloat162_rn(a[0], a[1]); v.x = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(a[2], a[3]); v.y = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(a[4], a[5]); v.z = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(a[6], a[7]); v.w = *reinterpret_cast<uint32_t*>(&t);
  *reinterpret_cast<uint4*>(dst) = v;
}
template <>
__device__ __forceinline__ void store8<__half>(__half* dst, const float* a) {
  uint4 v;
  __half2 t;
  t = __floats2half2_rn(a[0], a[1]); v.x = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2half2_rn(a[2], a[3]); v.y = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2half2_rn(a[4], a[5]); v.z = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2half2_rn(a[6], a[7]); v.w = *reinterpret_cast<uint32_t*>(&t);
  *reinterpret_cast<uint4*>(dst) = v;
}
template <>
__device__ __forceinline__ void store8<float>(float* dst, const float* a) {
  *reinterpret_cast<float4*>(dst) = make_float4(a[0], a[1], a[2], a[3]);
  *reinterpret_cast<float4*>(dst + 4) = make_float4(a[4], a[5], a[6], a[7]);
}

// acc[0..32) += v[0..32) * scale. Packed fp32 FMAs (__ffma2_rn on register pairs) were measured 25 % slower
// here, with and without float2 accumulators: the pairing constraints on 128 accumulators plus 64 staged
// values cost more in spills and moves than the halved issue count saves.
__device__ __forceinline__ void promote32(float* acc, const uint32_t (&v)[32], float sc) {
#pragma unroll
  for (int j = 0; j < 32; ++j) acc[j] = fmaf(__uint_as_float(v[j]), sc, acc[j]);
}

// tile index -> (m_tile, n_tile): sweep group_m row-tiles for every column tile before moving
// on, so the CTAs running together share A rows and B columns in L2. group_m is a power of two;
// only the last, shorter group of row tiles pays for a real division.
__device__ __forceinline__ void tile_coords(int t, int m_tiles, int n_tiles, int group_m, FastDiv per_group_div,
                                            int& mt, int& nt) {
  const int per_group = group_m * n_tiles;
  const int g = fast_div(t, per_group_div);
  const int first_m = g * group_m;
  const int rows = min(group_m, m_tiles - first_m);
  const int r = t - g * per_group;
  nt = rows == group_m ? r >> (31 - __clz(group_m)) : r / rows;
  mt = first_m + r - nt * rows;
}

template <int BN, int MODE, typename OutT, int FAN = 1>
__global__ void __launch_bounds__(GemmCfg<BN>::kThreads, 1)
block_fp8_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ TmapOut<FAN> tmap_out, const GemmParams p) {
  const CUtensorMap& tmap_c = tmap_out.m[0];
  using Cfg = GemmCfg<BN>;
  using L = GemmLayout<BN, MODE, OutT>;
  constexpr int S = L::kStages;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte-swizzled tiles need 1024-byte alignment
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t sA = smem_base;
  const uint32_t sB = smem_base + S * Cfg::kStageA;
  // after the stage ring (a multiple of 1024 bytes): [exchange (mode 1)] [output staging] [barriers]
  float* exchange = reinterpret_cast<float*>(smem_al + (size_t)S * (Cfg::kStageA + Cfg::kStageB));
  const uint32_t staging = smem_base + S * (Cfg::kStageA + Cfg::kStageB) +
                           (MODE == GEMM_GROUPED_SILU_QUANT ? Cfg::kExchangeBytes : 0);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_al + (size_t)S * (Cfg::kStageA + Cfg::kStageB) + L::kStagingBytes);
  const uint32_t bar0 = ptx::smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (S + s); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * S + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * S + 2 + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * S + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * S + 5);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kProducerWarp = Cfg::kEpiWarps, kMmaWarp = Cfg::kEpiWarps + 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(tfull_bar(b), 1);
      ptx::mbar_init(tempty_bar(b), Cfg::kEpiWarps);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), Cfg::kTmemCols);
    ptx::tmem_relinquish();
  }
  if (warp == kProducerWarp && lane == 0) {
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
    if (L::kStaged && MODE != GEMM_GROUPED_SCATTER) ptx::prefetch_tensormap(&tmap_c);
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // live problem size (grouped: decided on the device by the align kernel)
  int m_tiles = p.m_tiles;
  if (MODE != GEMM_DENSE) m_tiles = min(m_tiles, *p.num_post_pad / kBM);
  const int S_k = p.k_splits;
  const int total_items = m_tiles * p.n_tiles * S_k;
  const int num_kb = p.num_kb;

  if (warp >= Cfg::kEpiWarps) {
  // the producer / MMA warpgroup hands registers to the promotion warpgroups
  if constexpr (Cfg::kRebalanceRegs) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Cfg::kRegsOther));
  if (warp == kProducerWarp) {
    // ------------------------------------------------------------------ TMA producer
    uint32_t it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
      const int t = fast_div(item, p.k_splits_div), ks = item - t * S_k;
      const int kb0 = ks * p.kb_per_split, kb1 = min(num_kb, kb0 + p.kb_per_split);
      int mt, nt;
      tile_coords(t, m_tiles, p.n_tiles, p.group_m, p.per_group_div, mt, nt);
      int b_row = nt * BN, b_row2 = 0;
      if (MODE != GEMM_DENSE) {
        const int e = p.expert_ids[mt];
        if (e < 0) continue;
        if (MODE == GEMM_GROUPED_SILU_QUANT) {
          b_row = e * 2 * p.N + nt * 128;  // gate rows of this 128-wide output group
          b_row2 = b_row + p.N;            // matching up rows
        } else {
          b_row += e * p.N;
        }
      }
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % S;
        ok = ptx::mbar_wait(empty_bar(s), ((it / S) & 1) ^ 1, abort_flag);
        if (!ok) break;
        if (lane == 0) {
          ptx::mbar_expect_tx(full_bar(s), Cfg::kStageA + Cfg::kStageB);
          ptx::tma_load_2d(sA + s * Cfg::kStageA, &tmap_a, kb * kBK, mt * kBM, full_bar(s));
          if (MODE == GEMM_GROUPED_SILU_QUANT) {
            // B box is 64 rows in this mode: gate lo | up lo | gate hi | up hi
            const uint32_t d = sB + s * Cfg::kStageB;
            ptx::tma_load_2d(d, &tmap_b, kb * kBK, b_row, full_bar(s));
            ptx::tma_load_2d(d + 64 * kBK, &tmap_b, kb * kBK, b_row2, full_bar(s));
            ptx::tma_load_2d(d + 128 * kBK, &tmap_b, kb * kBK, b_row + 64, full_bar(s));
            ptx::tma_load_2d(d + 192 * kBK, &tmap_b, kb * kBK, b_row2 + 64, full_bar(s));
          } else {
            ptx::tma_load_2d(sB + s * Cfg::kStageB, &tmap_b, kb * kBK, b_row, full_bar(s));
          }
        }
        __syncwarp();
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc = ptx::idesc_e4m3_f32(kBM, BN);
    uint32_t it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
      const int t = fast_div(item, p.k_splits_div), ks = item - t * S_k;
      const int kb0 = ks * p.kb_per_split, kb1 = min(num_kb, kb0 + p.kb_per_split);
      int mt, nt;
      tile_coords(t, m_tiles, p.n_tiles, p.group_m, p.per_group_div, mt, nt);
      if (MODE != GEMM_DENSE && p.expert_ids[mt] < 0) continue;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % S, b = it & 1;
        ok = ptx::mbar_wait(tempty_bar(b), ((it >> 1) & 1) ^ 1, abort_flag) &&
             ptx::mbar_wait(full_bar(s), (it / S) & 1, abort_flag);
        if (!ok) break;
        ptx::tc_fence_after();
        if (lane == 0) {
          const uint64_t da = ptx::smem_desc_sw128(sA + s * Cfg::kStageA);
          const uint64_t db = ptx::smem_desc_sw128(sB + s * Cfg::kStageB);
          const uint32_t d = tmem_base + b * BN;
#pragma unroll
          for (int k = 0; k < kBK / 32; ++k)  // +32 bytes along K inside the swizzle row = +2 in the address field
            ptx::mma_f8(d, da + 2 * k, db + 2 * k, idesc, k > 0);  // k == 0 overwrites the buffer
          // One commit per K block: partial product ready for the promotion warps. (The smem
          // stage is released by promotion warp 0 once it sees this barrier: a second commit
          // here costs the issuing thread more than a hundred cycles per K block.)
          ptx::mma_commit(tfull_bar(b));
        }
        __syncwarp();
      }
    }
  }
  } else {
    // ------------------------------------------------------------- promotion warps
    if constexpr (Cfg::kRebalanceRegs) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Cfg::kRegsPromotion));
    const int quarter = warp & 3, half = warp >> 2;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16) + half * 128;

    // Everything a work item needs, including its first four scale pairs already in flight.
    // The context of item i+1 is set up BEFORE the epilogue of item i, so the L2 round trips
    // of its scales (and of its expert id) overlap the stores instead of stalling the MMA.
    struct Item {
      int item, mt, nt, ks, kb0, kb1, expert, row, col0;
      int flat;  // scatter mode: (token, slot) index of this thread's row, >= numel for a pad row
      bool row_ok;
      const float* as_ptr;
      const float* bs_ptr;
      float a_pf[4], b_pf[4];
      const float* bs2_ptr;  // MODE 1: scales of the up rows (b_pf/bs_ptr are the gate rows')
      float b2_pf[4];
    };
    // hint: the expert of work item `hint_item`, requested at the start of the previous tile so that the
    // dependent chain "expert id -> scale rows" does not start with an L2 round trip between two tiles
    auto setup = [&](int item, Item& c, int hint_item, int hint_expert) -> bool {
      for (; item < total_items; item += gridDim.x) {
        const int t = fast_div(item, p.k_splits_div);
        c.ks = item - t * S_k;
        c.kb0 = c.ks * p.kb_per_split;
        c.kb1 = min(num_kb, c.kb0 + p.kb_per_split);
        tile_coords(t, m_tiles, p.n_tiles, p.group_m, p.per_group_div, c.mt, c.nt);
        c.expert = 0;
        if (MODE != GEMM_DENSE) {
          c.expert = item == hint_item ? hint_expert : p.expert_ids[c.mt];
          if (c.expert < 0) continue;  // rows of experts that live on another rank
        }
        c.item = item;
        c.row = c.mt * kBM + row_in_tile;
        c.col0 = MODE == GEMM_GROUPED_SILU_QUANT ? c.nt * 128 + half * 64 : c.nt * BN + half * 128;
        c.row_ok = c.row < p.M;
        c.as_ptr = p.As + (int64_t)(c.row_ok ? c.row : 0) * p.as_sm;
        // row of Bs: the 128-row block of B this thread's columns come from (MODE 1: gate block
        // nt for its first 64 TMEM columns, up block I/128 + nt for the other 64)
        const int nb = MODE == GEMM_GROUPED_SILU_QUANT ? c.nt : min(c.col0 / 128, p.n_blocks - 1);
        const int bs_rows = MODE == GEMM_GROUPED_SILU_QUANT ? 2 * p.n_blocks : p.n_blocks;
        c.bs_ptr = p.Bs + ((int64_t)c.expert * bs_rows + nb) * num_kb;
        c.bs2_ptr = c.bs_ptr + (int64_t)p.n_blocks * num_kb;
        c.flat = 0;
        if (MODE == GEMM_GROUPED_SCATTER) c.flat = c.row_ok ? __ldg(p.sorted_ids + c.row) : p.numel;
#pragma unroll
        for (int d = 0; d < 4; ++d) {
          const bool in = c.row_ok && c.kb0 + d < c.kb1;
          c.a_pf[d] = in ? __ldg(c.as_ptr + (int64_t)(c.kb0 + d) * p.as_sk) : 0.f;
          c.b_pf[d] = in ? __ldg(c.bs_ptr + c.kb0 + d) : 0.f;
          if (MODE == GEMM_GROUPED_SILU_QUANT) c.b2_pf[d] = in ? __ldg(c.bs2_ptr + c.kb0 + d) : 0.f;
        }
        return true;
      }
      return false;
    };

    uint32_t it = 0;
    bool ok = true;
    Item cur;
    bool have = setup(blockIdx.x, cur, -1, 0);
    while (have) {
      // expert of the next work item of this CTA: in flight during the whole K loop
      int hint_expert = 0;
      const int hint_item = cur.item + gridDim.x;
      if (MODE != GEMM_DENSE && hint_item < total_items) {
        int hmt, hnt;
        tile_coords(fast_div(hint_item, p.k_splits_div), m_tiles, p.n_tiles, p.group_m, p.per_group_div, hmt, hnt);
        hint_expert = __ldg(p.expert_ids + hmt);
      }
      float acc[128];
#pragma unroll
      for (int j = 0; j < 128; ++j) acc[j] = 0.f;
      // scatter mode: the router weight of this row, requested now (its index was fetched one tile
      // ahead) and used only in the epilogue
      float row_weight = 1.f;
      if (MODE == GEMM_GROUPED_SCATTER && p.topk_weights != nullptr && cur.flat < p.numel)
        row_weight = __ldg(p.topk_weights + cur.flat);

      // The scale registers form a ring of four: K block kb uses slot (kb - kb0) % 4 and refills it
      // for kb + 4. The loop is unrolled by four so the slots are fixed registers (a rotating
      // copy would read the value loaded one iteration ago and wait a full L2 round trip).
      for (int kbase = cur.kb0; kbase < cur.kb1 && ok; kbase += 4) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int kb = kbase + j;
          if (kb >= cur.kb1 || !ok) break;
          const int b = it & 1;
          const float sc = cur.a_pf[j] * cur.b_pf[j];
          // columns 64..127 of this thread: same block scale, except the up rows of MODE 1
          const float sc2 = MODE == GEMM_GROUPED_SILU_QUANT ? cur.a_pf[j] * cur.b2_pf[j] : sc;
          {
            const bool in = cur.row_ok && kb + 4 < cur.kb1;
            cur.a_pf[j] = in ? __ldg(cur.as_ptr + (int64_t)(kb + 4) * p.as_sk) : 0.f;
            cur.b_pf[j] = in ? __ldg(cur.bs_ptr + kb + 4) : 0.f;
            if (MODE == GEMM_GROUPED_SILU_QUANT) cur.b2_pf[j] = in ? __ldg(cur.bs2_ptr + kb + 4) : 0.f;
          }
          ok = ptx::mbar_wait(tfull_bar(b), (it >> 1) & 1, abort_flag);
          if (!ok) break;
          ptx::tc_fence_after();
          const uint32_t ta = lane_base + b * BN;
          uint32_t va[32], vb[32];
          // one TMEM load in flight behind the FMAs of the previous 32 columns
          ptx::tmem_ld32(ta, va);
          // The MMAs of this K block have completed, so they have also finished reading their
          // shared-memory stage: hand it back to the TMA producer. Done behind the first TMEM load: the
          // accumulator buffer goes back to the MMA warp only when the slowest of the eight warps has read
          // it, and this arrival in front of the load made warp 0 that warp by about 120 cycles per K block.
          if (warp == 0 && lane == 0) ptx::mbar_arrive(empty_bar(it % S));
          ptx::tmem_ld_wait(va);
          ptx::tmem_ld32(ta + 32, vb);
          promote32(acc, va, sc);
          ptx::tmem_ld_wait(vb);
          ptx::tmem_ld32(ta + 64, va);
          promote32(acc + 32, vb, sc);
          ptx::tmem_ld_wait(va);
          ptx::tmem_ld32(ta + 96, vb);
          promote32(acc + 64, va, sc2);
          ptx::tmem_ld_wait(vb);
          // every TMEM read of this buffer has landed: give it back to the MMA warp
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(tempty_bar(b));
          promote32(acc + 96, vb, sc2);
          ++it;
        }
      }
      if (!ok) break;

      Item nxt;
      const bool have_next = setup(cur.item + gridDim.x, nxt, hint_item, hint_expert);

      // ------------------------------------------------------------ tile epilogue
      const int row = cur.row, col0 = cur.col0, nt = cur.nt, ks = cur.ks;
      const bool row_ok = cur.row_ok;
      // this warp's staging area: kBoxesPerWarp boxes of [32 rows x 128 bytes], 128-byte swizzled
      const int store_warp = MODE == GEMM_GROUPED_SILU_QUANT ? quarter : warp;
      const uint32_t wstage = staging + store_warp * L::kWarpStageBytes;
      // 16-byte chunk c of this thread's row (= lane) goes to box c/8, slot (c%8) ^ (lane%8)
      auto stage_chunk = [&](int c, uint4 v) {
        const uint32_t addr = MODE == GEMM_GROUPED_SCATTER
                                  ? wstage + lane * L::kRowStride + (c << 4)
                                  : wstage + (c >> 3) * 4096 + lane * 128 + (((c & 7) ^ (lane & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                     : "memory");
      };
      if (L::kStaged) {
        // the bulk stores of the previous tile must have read the staging area before it is rewritten
        if (MODE == GEMM_GROUPED_SCATTER || lane < L::kBoxesPerWarp) ptx::tma_store_wait_read();
        __syncwarp();
        if (MODE == GEMM_GROUPED_SILU_QUANT) named_bar_sync(2 + quarter, 64);  // the box is shared with warp ^ 4
      }
      if (MODE == GEMM_GROUPED_SILU_QUANT) {
        if (p.topk_weights != nullptr) {
          // router weight applied to the gate_up product in fp32, before the activation (where
          // the reference's first grouped GEMM applies it when apply_router_weight_on_input is set)
          const int flat = row_ok ? p.sorted_ids[row] : p.numel;
          const float w = flat < p.numel ? __ldg(p.topk_weights + flat) : 0.f;
#pragma unroll
          for (int j = 0; j < 128; ++j) acc[j] *= w;
        }
        // acc[0..64) = gate, acc[64..128) = up of output columns col0 .. col0+63; the other half of
        // the 128-wide quantisation group lives in the warp with the same lane quarter (warp ^ 4):
        // only the partial row amax is exchanged (pair barrier 2 + quarter, 64 threads).
#pragma unroll
        for (int j = 0; j < 64; ++j) acc[j] = silu_mul_fast(acc[j], acc[64 + j]);
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 64; ++j) amax = fmaxf(amax, fabsf(acc[j]));
        exchange[half * kBM + row_in_tile] = amax;
        named_bar_sync(2 + quarter, 64);
        amax = fmaxf(fmaxf(amax, exchange[(half ^ 1) * kBM + row_in_tile]), 1e-10f);
        const float inv = __fdividef(448.0f, amax);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float q[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) q[i] = acc[16 * j + i] * inv;  // the conversion saturates to +-448
          uint4 v;
          v.x = pack4_e4m3(q[0], q[1], q[2], q[3]);
          v.y = pack4_e4m3(q[4], q[5], q[6], q[7]);
          v.z = pack4_e4m3(q[8], q[9], q[10], q[11]);
          v.w = pack4_e4m3(q[12], q[13], q[14], q[15]);
          stage_chunk(half * 4 + j, v);
        }
        if (half == 0 && row_ok) p.q_scales[(int64_t)nt * p.q_scale_ld + row] = __fdiv_rn(amax, 448.0f);
        ptx::fence_proxy_async_smem();
        named_bar_sync(2 + quarter, 64);  // both halves of the box are staged (and the amax slots are free again)
        if (half == 0 && lane == 0) {  // FP8 rows [32 x 128 B] of the expert-sorted activation
          ptx::tma_store_3d(&tmap_c, wstage, nt * 128, cur.mt * kBM + quarter * 32, 0);
          ptx::tma_store_commit();
        }
      } else {
        const float w = row_weight;
        const int flat = cur.flat;  // (token, slot) this row belongs to; >= numel: pad
        if (L::kStaged) {
#pragma unroll
          for (int c = 0; c < 16; ++c) {  // 16 chunks of 8 sixteen-bit elements
            float t[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) t[i] = acc[c * 8 + i] * w;
            stage_chunk(c, pack8<OutT>(t));
          }
          if (MODE == GEMM_DENSE) {
            ptx::fence_proxy_async_smem();
            __syncwarp();
            // one lane per box: the issue cost of a bulk tensor store (several hundred cycles on the thread
            // that issues it) is paid once per warp instead of once per box
            if (lane < L::kBoxesPerWarp) {
              constexpr int kColsPerBox = 128 / (int)sizeof(OutT);
              {
                const int bx = lane;
                if (col0 + bx * kColsPerBox < p.N) {
                  if (FAN == 1) {
                    ptx::tma_store_3d(&tmap_c, wstage + bx * 4096, col0 + bx * kColsPerBox, cur.mt * kBM + quarter * 32, ks);
                  } else {
                    // the staged box goes to every destination (or to the owner of this row block)
                    const int d0 = p.dest_by_tile ? cur.mt % p.n_dest : 0;
                    const int d1 = p.dest_by_tile ? d0 + 1 : p.n_dest;
                    for (int d = d0; d < d1; ++d)
                      ptx::tma_store_3d(&tmap_out.m[d], wstage + bx * 4096, col0 + bx * kColsPerBox,
                                        cur.mt * kBM + quarter * 32, 0);
                  }
                }
              }
              ptx::tma_store_commit();
            }
          } else {
            // scatter: rows go to arbitrary (token, slot) positions; every lane sends its own staged row as
            // one contiguous bulk copy (it reads only what this thread wrote: no warp barrier)
            ptx::fence_proxy_async_smem();
            const int cols = min(128, p.N - col0);  // N is a multiple of 8: whole 16-byte chunks
            if (flat < p.numel && cols > 0) {
              OutT* base = static_cast<OutT*>(p.C);
              int local = flat;
              if (p.scatter_rows_per_dest > 0) {
                const int r = fast_div(flat, p.scatter_div);
                base = static_cast<OutT*>(p.dest[r]);
                local = flat - r * p.scatter_rows_per_dest;
              }
              ptx::bulk_store_1d(base + (int64_t)local * p.ldc + col0, wstage + lane * L::kRowStride,
                                 (uint32_t)cols * (uint32_t)sizeof(OutT));
              ptx::tma_store_commit();
            }
          }
        } else {
          // fp32 output with 256-wide tiles: direct row stores
          const bool store = row_ok && (MODE != GEMM_GROUPED_SCATTER || flat < p.numel);
          if (store) {
            const int64_t out_row = MODE == GEMM_GROUPED_SCATTER ? flat : row;
            const int d0 = FAN > 1 && p.dest_by_tile ? cur.mt % p.n_dest : 0;
            const int d1 = FAN == 1 ? 1 : (p.dest_by_tile ? d0 + 1 : p.n_dest);
            for (int d = d0; d < d1; ++d) {
              OutT* base = static_cast<OutT*>(FAN == 1 ? p.C : p.dest[d]);
              OutT* dst = base + ks * p.split_stride + out_row * p.ldc + col0;
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                float t[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) t[i] = acc[j * 8 + i] * w;
                if (col0 + j * 8 < p.N) store8<OutT>(dst + j * 8, t);
              }
            }
          }
        }
      }
      cur = nxt;
      have = have_next;
    }
  }

  // every bulk store of this CTA must have completed before its shared memory is released
  if (L::kStaged && warp < Cfg::kEpiWarps && (MODE == GEMM_GROUPED_SCATTER || lane < L::kBoxesPerWarp)) ptx::tma_store_wait_all();

  // ---------------------------------------------------------------------- teardown
  if (*abort_flag) {
    // A wait ran out: give copies / MMAs still in flight time to land before TMEM is freed.
    const unsigned long long t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicCAS(p.status, 0, 1);  // the host reads this word
  if (warp == kMmaWarp) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

}  // namespace b200
