// Dense block-FP8 GEMM on CTA pairs (tcgen05 cta_group::2): two CTAs of a cluster compute one
// 256 x 256 output tile. Each CTA loads its own 128 rows of A and only HALF of the B tile
// (128 of its 256 rows); the pair's tensor cores read both halves, so the L2 -> SM traffic per
// flop is 2/3 of the single-CTA kernel's, which is what bounds that kernel's MMA rate.
// No TMA multicast is involved: every load has one destination CTA.
//
// Roles per CTA are those of the single-CTA kernel (8 promotion warps, TMA producer, MMA
// issuer, 2 idle warps for setmaxnreg). Cross-CTA protocol (rank 0 = leader):
//   full[s]   (leader's)  2 arrivals (one expect_tx per CTA's producer) + the bytes of both
//                         CTAs' TMA loads (cta_group::2 loads signal the leader's barrier)
//   empty[s]  (each CTA)  arrival from the leader's tcgen05.commit (one commit per CTA)
//   tfull[b]  (each CTA)  arrival from the leader's tcgen05.commit (one commit per CTA)
//   tempty[b] (leader's)  16 arrivals: the 8 promotion warps of both CTAs
// Only the leader's MMA warp issues tcgen05.mma; TMEM is allocated with cta_group::2 in both.
#pragma once

#include "gemm_host.cuh"

namespace b200 {

namespace ptx {
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.relaxed.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr), "r"(bytes)
               : "memory");
}
// tiled load whose completion bytes are counted on a barrier of the CTA pair's leader
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, int c0, int c1, uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(m), "r"(c0), "r"(c1), "r"(leader_bar)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void mma_f8_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive (count 1) on the barrier at shared::cluster address `bar` once the pair's MMAs issued so far completed
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// one commit that arrives on the barrier at the same shared-memory offset in every CTA of `mask`
// (tcgen05.commit is the one multicast form used anywhere in this library; no data is moved)
__device__ __forceinline__ void mma_commit_pair_multicast(uint32_t bar, uint16_t mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(mask)
               : "memory");
}
}  // namespace ptx

struct Pair {
  static constexpr int kBN = 256;            // columns of the pair's tile
  static constexpr int kStageA = kBM * kBK;  // this CTA's 128 rows of A
  static constexpr int kStageB = 128 * kBK;  // this CTA's half of the B tile
  static constexpr int kStages = 5;
  static constexpr int kEpiWarps = 8;
  static constexpr int kThreads = 384;
  static constexpr int kStagingBytes = 8 * 32 * 256;  // 8 warps x 32 rows x 256 bytes of 16-bit output
  static constexpr int kTmemCols = 512;
  static constexpr size_t kSmemBytes = (size_t)kStages * (kStageA + kStageB) + kStagingBytes + 1024 + 256;
  static constexpr int kRegsPromotion = 224, kRegsOther = 56;
};

template <typename OutT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Pair::kThreads, 1)
block_fp8_gemm_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                           const __grid_constant__ CUtensorMap tmap_c, const GemmParams p) {
  static_assert(sizeof(OutT) == 2, "the paired kernel stages 16-bit output");
  constexpr int S = Pair::kStages;
  constexpr int BN = Pair::kBN;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t sA = smem_base;
  const uint32_t sB = smem_base + S * Pair::kStageA;
  const uint32_t staging = smem_base + S * (Pair::kStageA + Pair::kStageB);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_al + (size_t)S * (Pair::kStageA + Pair::kStageB) + Pair::kStagingBytes);
  const uint32_t bar0 = ptx::smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (S + s); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * S + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * S + 2 + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * S + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * S + 5);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kProducerWarp = 8, kMmaWarp = 9;
  const uint32_t rank = ptx::cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      ptx::mbar_init(full_bar(s), 2);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(tfull_bar(b), 1);
      ptx::mbar_init(tempty_bar(b), 2 * Pair::kEpiWarps);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    ptx::tmem_alloc_pair(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), Pair::kTmemCols);
    ptx::tmem_relinquish_pair();
  }
  if (warp == kProducerWarp && lane == 0) {
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
    ptx::prefetch_tensormap(&tmap_c);
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();  // the peer's barriers are initialised before anything signals them
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int m_tiles2 = (p.M + 2 * kBM - 1) / (2 * kBM);
  const int total_tiles = m_tiles2 * p.n_tiles;
  const int num_kb = p.num_kb;
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

  if (warp >= Pair::kEpiWarps) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Pair::kRegsOther));
    if (warp == kProducerWarp) {
      // ---------------------------------------------------------------- TMA producer (both CTAs)
      uint32_t it = 0;
      bool ok = true;
      for (int t = pair; t < total_tiles && ok; t += npairs) {
        int mt2, nt;
        tile_coords(t, m_tiles2, p.n_tiles, p.group_m, p.per_group_div, mt2, nt);
        const int a_row = mt2 * 2 * kBM + (int)rank * kBM;
        const int b_row = nt * BN + (int)rank * 128;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % S;
          ok = ptx::mbar_wait(empty_bar(s), ((it / S) & 1) ^ 1, abort_flag);
          if (!ok) break;
          if (lane == 0) {
            const uint32_t lf = ptx::mapa(full_bar(s), 0);
            ptx::mbar_expect_tx_cluster(lf, Pair::kStageA + Pair::kStageB);
            ptx::tma_load_2d_pair(sA + s * Pair::kStageA, &tmap_a, kb * kBK, a_row, lf);
            ptx::tma_load_2d_pair(sB + s * Pair::kStageB, &tmap_b, kb * kBK, b_row, lf);
          }
          __syncwarp();
        }
      }
    } else if (warp == kMmaWarp && leader) {
      // ---------------------------------------------------------------- MMA issuer (leader only)
      constexpr uint32_t idesc = ptx::idesc_e4m3_f32(2 * kBM, BN);
      uint32_t it = 0;
      bool ok = true;
      for (int t = pair; t < total_tiles && ok; t += npairs) {
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % S, b = it & 1;
          ok = ptx::mbar_wait(tempty_bar(b), ((it >> 1) & 1) ^ 1, abort_flag) &&
               ptx::mbar_wait(full_bar(s), (it / S) & 1, abort_flag);
          if (!ok) break;
          ptx::tc_fence_after();
          if (lane == 0) {
            const uint64_t da = ptx::smem_desc_sw128(sA + s * Pair::kStageA);
            const uint64_t db = ptx::smem_desc_sw128(sB + s * Pair::kStageB);
            const uint32_t d = tmem_base + b * BN;
#pragma unroll
            for (int k = 0; k < kBK / 32; ++k) ptx::mma_f8_pair(d, da + 2 * k, db + 2 * k, idesc, k > 0);
            // partial product ready: one commit, delivered to the tfull barrier of both CTAs. Each
            // CTA's promotion warp 0 releases its own shared-memory stage when it sees the barrier.
            ptx::mma_commit_pair_multicast(tfull_bar(b), (uint16_t)3);
          }
          __syncwarp();
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ promotion warps (both CTAs)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Pair::kRegsPromotion));
    const int quarter = warp & 3, half = warp >> 2;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16) + half * 128;
    const uint32_t wstage = staging + warp * 8192;
    struct Item {
      int t, mt2, nt, row, col0;
      bool row_ok;
      const float* as_ptr;
      const float* bs_ptr;
      float a_pf[4], b_pf[4];
    };
    auto setup = [&](int t, Item& c) -> bool {
      if (t >= total_tiles) return false;
      c.t = t;
      tile_coords(t, m_tiles2, p.n_tiles, p.group_m, p.per_group_div, c.mt2, c.nt);
      c.row = c.mt2 * 2 * kBM + (int)rank * kBM + row_in_tile;
      c.col0 = c.nt * BN + half * 128;
      c.row_ok = c.row < p.M;
      c.as_ptr = p.As + (int64_t)(c.row_ok ? c.row : 0) * p.as_sm;
      c.bs_ptr = p.Bs + (int64_t)min(c.col0 / 128, p.n_blocks - 1) * num_kb;
#pragma unroll
      for (int d = 0; d < 4; ++d) {
        const bool in = c.row_ok && d < num_kb;
        c.a_pf[d] = in ? __ldg(c.as_ptr + (int64_t)d * p.as_sk) : 0.f;
        c.b_pf[d] = in ? __ldg(c.bs_ptr + d) : 0.f;
      }
      return true;
    };
    const uint32_t leader_tempty0 = ptx::mapa(tempty_bar(0), 0), leader_tempty1 = ptx::mapa(tempty_bar(1), 0);
    uint32_t it = 0;
    bool ok = true;
    Item cur;
    bool have = setup(pair, cur);
    while (have) {
      float acc[128];
#pragma unroll
      for (int j = 0; j < 128; ++j) acc[j] = 0.f;
      for (int kbase = 0; kbase < num_kb && ok; kbase += 4) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int kb = kbase + j;
          if (kb >= num_kb || !ok) break;
          const int b = it & 1;
          const float sc = cur.a_pf[j] * cur.b_pf[j];
          {
            const bool in = cur.row_ok && kb + 4 < num_kb;
            cur.a_pf[j] = in ? __ldg(cur.as_ptr + (int64_t)(kb + 4) * p.as_sk) : 0.f;
            cur.b_pf[j] = in ? __ldg(cur.bs_ptr + kb + 4) : 0.f;
          }
          ok = ptx::mbar_wait(tfull_bar(b), (it >> 1) & 1, abort_flag);
          if (!ok) break;
          if (warp == 0 && lane == 0) ptx::mbar_arrive(empty_bar(it % S));  // MMAs done reading this stage
          ptx::tc_fence_after();
          const uint32_t ta = lane_base + b * BN;
          uint32_t va[32], vb[32];
          ptx::tmem_ld32(ta, va);
          ptx::tmem_ld_wait(va);
          ptx::tmem_ld32(ta + 32, vb);
          promote32(acc, va, sc);
          ptx::tmem_ld_wait(vb);
          ptx::tmem_ld32(ta + 64, va);
          promote32(acc + 32, vb, sc);
          ptx::tmem_ld_wait(va);
          ptx::tmem_ld32(ta + 96, vb);
          promote32(acc + 64, va, sc);
          ptx::tmem_ld_wait(vb);
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive_cluster(b ? leader_tempty1 : leader_tempty0);
          promote32(acc + 96, vb, sc);
          ++it;
        }
      }
      if (!ok) break;
      Item nxt;
      const bool have_next = setup(cur.t + npairs, nxt);

      // ------------------------------------------------------------ tile epilogue (staged bulk store)
      if (lane == 0) ptx::tma_store_wait_read();
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const uint32_t addr = wstage + (c >> 3) * 4096 + lane * 128 + (((c & 7) ^ (lane & 7)) << 4);
        const uint4 v = pack8<OutT>(acc + c * 8);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
      }
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const int row0 = cur.mt2 * 2 * kBM + (int)rank * kBM + quarter * 32;
#pragma unroll
        for (int bx = 0; bx < 2; ++bx)
          if (cur.col0 + bx * 64 < p.N && row0 < p.M) ptx::tma_store_3d(&tmap_c, wstage + bx * 4096, cur.col0 + bx * 64, row0, 0);
        ptx::tma_store_commit();
      }
      cur = nxt;
      have = have_next;
    }
    if (lane == 0) ptx::tma_store_wait_all();
  }

  // ---------------------------------------------------------------------- teardown
  if (*abort_flag) {
    const unsigned long long t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();  // neither CTA leaves while the other may still signal its barriers or use its smem
  if (threadIdx.x == 0 && *abort_flag) atomicCAS(p.status, 0, 1);
  if (warp == kMmaWarp) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, Pair::kTmemCols);
  }
}

// Dense, 16-bit output, no split-K. p.M/N/K/As/Bs/C filled by the caller.
template <typename OutT>
inline int launch_gemm_2cta(const void* A, const void* B, GemmParams p, cudaStream_t st) {
  p.num_kb = (int)cdiv(p.K, kBK);
  p.n_blocks = (int)cdiv(p.N, 128);
  p.n_tiles = (int)cdiv(p.N, Pair::kBN);
  p.m_tiles = (int)cdiv(p.M, 2 * kBM);
  p.group_m = 8;  // 8 pair-tiles = 2048 rows swept per column tile
  p.k_splits = 1;
  p.kb_per_split = p.num_kb;
  p.per_group_div = make_fastdiv(p.group_m * p.n_tiles);
  p.k_splits_div = make_fastdiv(1);
  p.status = device_status_word();
  if (!p.status) {
    set_error_detail("cannot resolve the device status word");
    return B200_E_LAUNCH;
  }
  const int64_t tiles = (int64_t)p.m_tiles * p.n_tiles;
  if (tiles == 0) return B200_OK;
  const int max_pairs = sm_count() / 2;
  const int pairs = (int)(tiles < max_pairs ? tiles : max_pairs);
  CUtensorMap ta, tb, tc;
  int rc = make_tmap_u8(&ta, A, (uint64_t)p.M, (uint64_t)p.K, kBM, "A");
  if (rc) return rc;
  rc = make_tmap_u8(&tb, B, (uint64_t)p.N, (uint64_t)p.K, 128, "B (half tile)");
  if (rc) return rc;
  rc = make_tmap_out(&tc, p.C, 1, (uint64_t)p.M, (uint64_t)p.N, (int)sizeof(OutT), std::is_same<OutT, __nv_bfloat16>::value, "C");
  if (rc) return rc;
  auto k = block_fp8_gemm_2cta_kernel<OutT>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Pair::kSmemBytes);
  if (e != cudaSuccess) {
    set_error_detail("cudaFuncSetAttribute(smem=%zu): %s", Pair::kSmemBytes, cudaGetErrorString(e));
    return B200_E_LAUNCH;
  }
  k<<<2 * pairs, Pair::kThreads, Pair::kSmemBytes, st>>>(ta, tb, tc, p);
  return check_launch("block_fp8_gemm_2cta_kernel");
}

}  // namespace b200
