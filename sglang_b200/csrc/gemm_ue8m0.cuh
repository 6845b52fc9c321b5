// Block-FP8 GEMM for power-of-two (UE8M0) scales: the scales are applied INSIDE the tensor core.
//     C[m, n] = sum_k A[m, k] * B[n, k] * 2^ea[m, k/128] * 2^eb[n, k/128]
// With fp32 scales the tensor core can never accumulate across 128-K blocks and every partial product has
// to be pulled out of TMEM and scaled in registers (gemm_kernel.cuh). When every scale is a power of two,
// tcgen05.mma.kind::mxf8f6f4.block_scale multiplies each 32-K slice of A and B by an 8-bit exponent it reads
// from TMEM, so the accumulator stays in TMEM for the whole K loop and the only register work left is the
// tile epilogue.
//
// Scale format: the packed words the quantisers of this library already produce for DeepGEMM-style consumers
// (python/sglang/srt/layers/quantization/fp8_utils.py:1306-1334): int32 [ceil(K/512)][rows_padded], word
// (g, r) = the exponent bytes of row r for the four 128-K blocks 4g .. 4g+3. That is exactly one 32-bit TMEM
// scale column per 32 rows: the instruction reads the scale of row r from lane r % 32, column r / 32, byte
// `sf_id`, so the four K = 32 MMAs of K block kb all select byte kb % 4 and the scales are refreshed once
// per four K blocks. A helper warp reads the words of a tile (coalesced), writes them transposed 32 x 4
// into shared memory and tcgen05.cp (32x128b.warpx4) copies each 512-byte atom into four TMEM columns of all
// four lane quarters.
//
// One persistent CTA per SM, tiles of 128 x 224: two accumulator stages of 224 columns + the scale columns
// fit the 512 TMEM columns, so the epilogue of a tile overlaps the K loop of the next one.
//   warps 0-7  epilogue: tcgen05.ld of the finished accumulator, convert, 16-byte row stores
//   warp  8    TMA producer (A 128 x 128 B, B 224 x 128 B per stage, 128-byte swizzle, no multicast)
//   warp  9    MMA issuer (and the scale copies smem -> TMEM)
//   warp  10   scale loader: packed words -> transposed atoms in a 4-slot shared-memory ring
#pragma once

#include "gemm_host.cuh"

namespace b200 {

struct Ue8m0Params {
  const int32_t* sfa;   // [ceil(K/512)][sfa_ld] packed exponents of the rows of A
  const int32_t* sfb;   // [ceil(K/512)][sfb_ld] packed exponents of the rows of B (or of its 128-row blocks)
  int64_t sfa_ld, sfb_ld;
  int sfb_rows_per_word;  // 1: one word per row of B; 128: one word per 128-row block
  void* C;
  int M, N, K, num_kb, m_tiles, n_tiles, group_m;
  FastDiv per_group_div;  // division by group_m * n_tiles
  int* status;
};

struct Ue8m0Cfg {
  static constexpr int BN = 224;
  static constexpr int kStages = 4;
  static constexpr int kStageA = kBM * kBK;       // 16 KB
  static constexpr int kStageB = BN * kBK;        // 28 KB
  static constexpr int kSfSlots = 4;              // scale ring: groups of four K blocks
  static constexpr int kSfSlotBytes = 512 + 1024; // one atom for A (128 rows), two for B (224 rows)
  static constexpr int kThreads = 384;
  static constexpr int kEpiWarps = 8, kProducerWarp = 8, kMmaWarp = 9, kSfWarp = 10;
  static constexpr int kAccCols = BN;             // per accumulator stage
  static constexpr int kSfaCol = 2 * BN;          // 448: two buffers of 4 columns
  static constexpr int kSfbCol = 2 * BN + 8;      // 456: two buffers of 8 columns
  static constexpr int kTmemCols = 512;
  static constexpr size_t kSmemBytes = (size_t)kStages * (kStageA + kStageB) + kSfSlots * kSfSlotBytes + 1024 + 256;
};

namespace ptx {
// Instruction descriptor of kind::mxf8f6f4.block_scale, E4M3 x E4M3, both operands K-major, E8M0 scales.
//   bits 4-5 B scale id   7-9 A format (0 = e4m3)   10-12 B format   15/16 A/B major (0 = K)
//   bits 17-22 N >> 3     23 scale format (1 = E8M0)   24-28 M >> 4   29-30 A scale id   31 K size (0 = 32)
__host__ __device__ constexpr uint32_t idesc_e4m3_block_scaled(int M, int N) {
  return ((uint32_t)(N >> 3) << 17) | (1u << 23) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void mma_f8_block_scaled(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                    uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
      "}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}
// 32 rows x 16 bytes of shared memory -> four TMEM columns of lanes 0-31, replicated into all four lane quarters
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
}
// Shared-memory descriptor of a scale atom: 32 rows of 16 bytes, no swizzle; 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sf_atom(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)(128 >> 4) << 32) | ((uint64_t)1 << 46);
}
}  // namespace ptx

template <typename OutT>
__global__ void __launch_bounds__(Ue8m0Cfg::kThreads, 1)
block_fp8_gemm_ue8m0_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                            const Ue8m0Params p) {
  using Cfg = Ue8m0Cfg;
  constexpr int S = Cfg::kStages, BN = Cfg::BN, SFS = Cfg::kSfSlots;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t sA = smem_base;
  const uint32_t sB = smem_base + S * Cfg::kStageA;
  const uint32_t sSF = smem_base + S * (Cfg::kStageA + Cfg::kStageB);
  uint8_t* sSF_ptr = smem_al + (size_t)S * (Cfg::kStageA + Cfg::kStageB);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sSF_ptr + SFS * Cfg::kSfSlotBytes);
  const uint32_t bar0 = ptx::smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (S + s); };
  auto sf_full_bar = [&](int s) { return bar0 + 8u * (2 * S + s); };
  auto sf_empty_bar = [&](int s) { return bar0 + 8u * (2 * S + SFS + s); };
  auto acc_full_bar = [&](int a) { return bar0 + 8u * (2 * S + 2 * SFS + a); };
  auto acc_empty_bar = [&](int a) { return bar0 + 8u * (2 * S + 2 * SFS + 2 + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * S + 2 * SFS + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * S + 2 * SFS + 5);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < SFS; ++s) {
      ptx::mbar_init(sf_full_bar(s), 1);
      ptx::mbar_init(sf_empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(acc_full_bar(a), 1);
      ptx::mbar_init(acc_empty_bar(a), Cfg::kEpiWarps);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == Cfg::kMmaWarp) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), Cfg::kTmemCols);
    ptx::tmem_relinquish();
  }
  if (warp == Cfg::kProducerWarp && lane == 0) {
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = p.m_tiles * p.n_tiles;
  const int num_kb = p.num_kb;
  const int groups = (num_kb + 3) / 4;  // scale groups (four K blocks each) per tile

  if (warp == Cfg::kProducerWarp) {
    // ------------------------------------------------------------------ TMA producer
    uint32_t it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int mt, nt;
      tile_coords(t, p.m_tiles, p.n_tiles, p.group_m, p.per_group_div, mt, nt);
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % S;
        ok = ptx::mbar_wait(empty_bar(s), ((it / S) & 1) ^ 1, abort_flag);
        if (!ok) break;
        if (lane == 0) {
          ptx::mbar_expect_tx(full_bar(s), Cfg::kStageA + Cfg::kStageB);
          ptx::tma_load_2d(sA + s * Cfg::kStageA, &tmap_a, kb * kBK, mt * kBM, full_bar(s));
          ptx::tma_load_2d(sB + s * Cfg::kStageB, &tmap_b, kb * kBK, nt * BN, full_bar(s));
        }
        __syncwarp();
      }
    }
  } else if (warp == Cfg::kSfWarp) {
    // ------------------------------------------------------------------ scale loader
    // Atom layout expected by the 32x128b.warpx4 copy: row r of a 128-row atom at byte (r % 32) * 16 + (r / 32) * 4.
    // Lane l therefore holds rows l, 32 + l, 64 + l, 96 + l and writes one 16-byte vector.
    constexpr int32_t kOne = 0x7F7F7F7F;  // exponent 127 = 2^0 for rows past the edge (their data is zero-filled)
    uint32_t gi = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int mt, nt;
      tile_coords(t, p.m_tiles, p.n_tiles, p.group_m, p.per_group_div, mt, nt);
      const int m0 = mt * kBM, n0 = nt * BN;
      for (int g = 0; g < groups; ++g, ++gi) {
        const int slot = gi % SFS;
        int32_t wa[4], wb[8];
        const int32_t* ga = p.sfa + (int64_t)g * p.sfa_ld;
        const int32_t* gb = p.sfb + (int64_t)g * p.sfb_ld;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = m0 + 32 * j + lane;
          wa[j] = r < p.M ? __ldg(ga + r) : kOne;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int r = n0 + 32 * j + lane;
          wb[j] = (j < BN / 32 && r < p.N) ? __ldg(gb + r / p.sfb_rows_per_word) : kOne;
        }
        ok = ptx::mbar_wait(sf_empty_bar(slot), ((gi / SFS) & 1) ^ 1, abort_flag);
        if (!ok) break;
        uint8_t* dst = sSF_ptr + (size_t)slot * Cfg::kSfSlotBytes + lane * 16;
        *reinterpret_cast<int4*>(dst) = make_int4(wa[0], wa[1], wa[2], wa[3]);
        *reinterpret_cast<int4*>(dst + 512) = make_int4(wb[0], wb[1], wb[2], wb[3]);
        *reinterpret_cast<int4*>(dst + 1024) = make_int4(wb[4], wb[5], wb[6], wb[7]);
        ptx::fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core's copy
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(sf_full_bar(slot));
      }
    }
  } else if (warp == Cfg::kMmaWarp) {
    // ------------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc0 = ptx::idesc_e4m3_block_scaled(kBM, BN);
    uint32_t it = 0, gi = 0, tile_no = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_no) {
      const int as = tile_no & 1;
      ok = ptx::mbar_wait(acc_empty_bar(as), ((tile_no >> 1) & 1) ^ 1, abort_flag);
      if (!ok) break;
      const uint32_t d = tmem_base + as * Cfg::kAccCols;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % S;
        if ((kb & 3) == 0) {
          // scales of the next four K blocks: three 512-byte atoms into the scale columns of buffer gi & 1
          const int slot = gi % SFS;
          ok = ptx::mbar_wait(sf_full_bar(slot), (gi / SFS) & 1, abort_flag);
          if (!ok) break;
          ptx::tc_fence_after();
          if (lane == 0) {
            const uint32_t src = sSF + slot * Cfg::kSfSlotBytes;
            const uint32_t buf = gi & 1;
            ptx::tmem_cp_32x128b_warpx4(tmem_base + Cfg::kSfaCol + buf * 4, ptx::smem_desc_sf_atom(src));
            ptx::tmem_cp_32x128b_warpx4(tmem_base + Cfg::kSfbCol + buf * 8, ptx::smem_desc_sf_atom(src + 512));
            ptx::tmem_cp_32x128b_warpx4(tmem_base + Cfg::kSfbCol + buf * 8 + 4, ptx::smem_desc_sf_atom(src + 1024));
            ptx::mma_commit(sf_empty_bar(slot));  // the slot is free once the copies have read it
          }
          __syncwarp();
          ++gi;
        }
        ok = ptx::mbar_wait(full_bar(s), (it / S) & 1, abort_flag);
        if (!ok) break;
        ptx::tc_fence_after();
        if (lane == 0) {
          const uint64_t da = ptx::smem_desc_sw128(sA + s * Cfg::kStageA);
          const uint64_t db = ptx::smem_desc_sw128(sB + s * Cfg::kStageB);
          const uint32_t buf = (gi - 1) & 1, byte = kb & 3;
          const uint32_t idesc = idesc0 | (byte << 4) | (byte << 29);  // scale byte of this K block, for A and B
          const uint32_t tsfa = tmem_base + Cfg::kSfaCol + buf * 4;
          const uint32_t tsfb = tmem_base + Cfg::kSfbCol + buf * 8;
#pragma unroll
          for (int k = 0; k < kBK / 32; ++k)
            ptx::mma_f8_block_scaled(d, da + 2 * k, db + 2 * k, idesc, tsfa, tsfb, (kb > 0 || k > 0) ? 1u : 0u);
          ptx::mma_commit(empty_bar(s));  // stage free once these MMAs have read it
          if (kb == num_kb - 1) ptx::mma_commit(acc_full_bar(as));  // the tile's accumulator is complete
        }
        __syncwarp();
      }
    }
  } else if (warp < Cfg::kEpiWarps) {
    // ------------------------------------------------------------------- epilogue warps
    const int quarter = warp & 3, half = warp >> 2;  // TMEM lanes 32*quarter.., columns 112*half..
    uint32_t tile_no = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_no) {
      int mt, nt;
      tile_coords(t, p.m_tiles, p.n_tiles, p.group_m, p.per_group_div, mt, nt);
      const int as = tile_no & 1;
      ok = ptx::mbar_wait(acc_full_bar(as), (tile_no >> 1) & 1, abort_flag);
      if (!ok) break;
      ptx::tc_fence_after();
      const int row = mt * kBM + quarter * 32 + lane;
      const int col0 = nt * BN + half * (BN / 2);
      const uint32_t ta = tmem_base + ((uint32_t)(quarter * 32) << 16) + as * Cfg::kAccCols + half * (BN / 2);
      OutT* out = static_cast<OutT*>(p.C) + (int64_t)row * p.N + col0;
#pragma unroll 1
      for (int c = 0; c < BN / 2; c += 16) {
        uint32_t v[32];
        ptx::tmem_ld16(ta + c, v);
        ptx::tmem_ld_wait16(v);
        if (row < p.M) {
          float f[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) f[i] = __uint_as_float(v[i]);
          if (col0 + c < p.N) store8<OutT>(out + c, f);
          if (col0 + c + 8 < p.N) store8<OutT>(out + c + 8, f + 8);
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(acc_empty_bar(as));
    }
  }

  if (*abort_flag) {
    const unsigned long long t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicCAS(p.status, 0, 1);
  if (warp == Cfg::kMmaWarp) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <typename OutT>
inline int launch_gemm_ue8m0(const void* A, const void* B, Ue8m0Params p, cudaStream_t st) {
  p.num_kb = (int)cdiv(p.K, kBK);
  p.m_tiles = (int)cdiv(p.M, kBM);
  p.n_tiles = (int)cdiv(p.N, Ue8m0Cfg::BN);
  p.group_m = 16;
  p.per_group_div = make_fastdiv(p.group_m * p.n_tiles);
  p.status = device_status_word();
  if (!p.status) {
    set_error_detail("cannot resolve the device status word");
    return B200_E_LAUNCH;
  }
  const int64_t tiles = (int64_t)p.m_tiles * p.n_tiles;
  if (tiles == 0) return B200_OK;
  const int sms = sm_count();
  const int grid = (int)(tiles < sms ? tiles : sms);
  CUtensorMap ta, tb;
  int rc = make_tmap_u8(&ta, A, (uint64_t)p.M, (uint64_t)p.K, kBM, "A");
  if (rc) return rc;
  rc = make_tmap_u8(&tb, B, (uint64_t)p.N, (uint64_t)p.K, (uint32_t)Ue8m0Cfg::BN, "B (224-row tiles)");
  if (rc) return rc;
  auto k = block_fp8_gemm_ue8m0_kernel<OutT>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Ue8m0Cfg::kSmemBytes);
  if (e != cudaSuccess) {
    set_error_detail("cudaFuncSetAttribute(smem=%zu): %s", Ue8m0Cfg::kSmemBytes, cudaGetErrorString(e));
    return B200_E_LAUNCH;
  }
  k<<<grid, Ue8m0Cfg::kThreads, Ue8m0Cfg::kSmemBytes, st>>>(ta, tb, p);
  return check_launch("block_fp8_gemm_ue8m0_kernel");
}

}  // namespace b200
