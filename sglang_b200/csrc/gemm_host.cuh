// Host side of the block-FP8 GEMM: TMA descriptor encoding and the launch helper shared by
// the dense linear entry point and the fused-MoE entry point.
#pragma once

#include <type_traits>
#include <unordered_map>

#include "gemm_kernel.cuh"

namespace b200 {

// Split-K factor for the dense GEMM: when the 128 x 256 tiles alone would leave most SMs idle
// (a few hundred rows), split K so that about one work item per SM streams the weights.
inline int choose_k_splits(int64_t M, int64_t N, int64_t K, int sms) {
  const int64_t tiles = cdiv(M, 128) * cdiv(N, N > 128 ? 256 : 128);
  const int64_t num_kb = cdiv(K, 128);
  if (tiles * 4 >= (int64_t)sms * 3 || num_kb < 8) return 1;
  int64_t s = sms / tiles;
  if (s > num_kb / 4) s = num_kb / 4;
  if (s > 8) s = 8;
  return s < 1 ? 1 : (int)s;
}

// cuTensorMapEncodeTiled, resolved through the runtime so the library needs no -lcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Row-major [rows, k_bytes] byte matrix, box = [box_rows x 128 bytes], 128-byte swizzle,
// out-of-range elements read as zero.
inline int make_tmap_u8(CUtensorMap* m, const void* base, uint64_t rows, uint64_t k_bytes, uint32_t box_rows,
                        const char* what) {
  // Encoding a descriptor costs a driver call of a microsecond or two, as much as a decode kernel's whole
  // launch: the descriptors of operands seen before (weights, reused activation buffers) are kept per
  // thread, keyed by everything they are built from.
  struct Key {
    const void* base;
    uint64_t rows, k_bytes;
    uint32_t box_rows;
    bool operator==(const Key& o) const {
      return base == o.base && rows == o.rows && k_bytes == o.k_bytes && box_rows == o.box_rows;
    }
  };
  struct Hash {
    size_t operator()(const Key& k) const {
      return (size_t)((uintptr_t)k.base * 0x9E3779B97F4A7C15ull) ^ (size_t)(k.rows * 31 + k.k_bytes * 131 + k.box_rows);
    }
  };
  static thread_local std::unordered_map<Key, CUtensorMap, Hash> cache;
  const Key key{base, rows, k_bytes, box_rows};
  auto hit = cache.find(key);
  if (hit != cache.end()) {
    *m = hit->second;
    return B200_OK;
  }
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) {
    set_error_detail("cuTensorMapEncodeTiled is not available from the driver");
    return B200_E_LAUNCH;
  }
  cuuint64_t dims[2] = {k_bytes, rows};
  cuuint64_t strides[1] = {k_bytes};
  cuuint32_t box[2] = {(cuuint32_t)kBK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error_detail("cuTensorMapEncodeTiled(%s: rows=%llu k=%llu box_rows=%u) failed with CUresult %d", what,
                     (unsigned long long)rows, (unsigned long long)k_bytes, box_rows, (int)r);
    return B200_E_LAUNCH;
  }
  if (cache.size() >= 4096) cache.clear();
  cache.emplace(key, *m);
  return B200_OK;
}

// Output tensor [S, rows, cols] (S = K splits, 1 otherwise) of `elem_bytes`-wide elements, stored
// through boxes of [32 rows x 128 bytes] with the 128-byte swizzle.
inline int make_tmap_out(CUtensorMap* m, const void* base, uint64_t splits, uint64_t rows, uint64_t cols,
                         int elem_bytes, bool is_bf16, const char* what) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) {
    set_error_detail("cuTensorMapEncodeTiled is not available from the driver");
    return B200_E_LAUNCH;
  }
  const CUtensorMapDataType dt = elem_bytes == 1   ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : is_bf16         ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                   : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  cuuint64_t dims[3] = {cols, rows, splits};
  cuuint64_t strides[2] = {cols * (uint64_t)elem_bytes, rows * cols * (uint64_t)elem_bytes};
  cuuint32_t box[3] = {(cuuint32_t)(128 / elem_bytes), 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error_detail("cuTensorMapEncodeTiled(%s: splits=%llu rows=%llu cols=%llu elem=%d) failed with CUresult %d", what,
                     (unsigned long long)splits, (unsigned long long)rows, (unsigned long long)cols, elem_bytes, (int)r);
    return B200_E_LAUNCH;
  }
  return B200_OK;
}

inline int sm_count() {
  static thread_local int dev_cached = -1, sms = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != dev_cached) {
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    dev_cached = dev;
  }
  return sms > 0 ? sms : 148;
}

template <int BN, int MODE, typename OutT, int FAN = 1>
inline int launch_gemm_inst(const CUtensorMap& ta, const CUtensorMap& tb, const TmapOut<FAN>& tc, const GemmParams& p,
                            int grid, cudaStream_t st) {
  auto k = block_fp8_gemm_kernel<BN, MODE, OutT, FAN>;
  // per device and cheap: set on every launch rather than caching per device
  const size_t smem = GemmLayout<BN, MODE, OutT>::kSmemBytes;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error_detail("cudaFuncSetAttribute(smem=%zu): %s", smem, cudaGetErrorString(e));
    return B200_E_LAUNCH;
  }
  k<<<grid, GemmCfg<BN>::kThreads, smem, st>>>(ta, tb, tc, p);
  return check_launch("block_fp8_gemm_kernel");
}

// a_rows x K (fp8) times b_rows_total x K (fp8; grouped: experts stacked) -> C.
// p must be filled except num_kb / n_blocks / n_tiles / m_tiles / group_m / status.
// m_tiles_hint: expected number of live 128-row tiles when that is decided on the device.
template <int MODE, typename OutT>
inline int launch_gemm(const void* A, const void* B, int64_t b_rows_total, GemmParams p, int force_bn,
                       cudaStream_t st, int64_t m_tiles_hint = 0, int k_splits = 1) {
  p.num_kb = (int)cdiv(p.K, kBK);
  p.n_blocks = (int)cdiv(p.N, 128);
  p.m_tiles = (int)cdiv(p.M, kBM);
  p.status = device_status_word();
  if (!p.status) {
    set_error_detail("cannot resolve the device status word");
    return B200_E_LAUNCH;
  }
  const int sms = sm_count();
  // 128 x 256 tiles: eight promotion warps hide the TMEM round trips of each other and the
  // shared-memory traffic per flop is halved. The 128-wide tile (four promotion warps) is
  // slower per flop even when it fills more SMs; it is kept for N <= 128 (small problems are
  // spread over the SMs by split-K instead).
  int bn = 256;
  if (MODE == GEMM_GROUPED_SILU_QUANT) force_bn = 256;  // gate + up halves of one tile
  (void)m_tiles_hint;
  if (p.N <= 128) bn = 128;
  if (force_bn == 128 || force_bn == 256) bn = force_bn;
  p.n_tiles = MODE == GEMM_GROUPED_SILU_QUANT ? p.N / 128 : (int)cdiv(p.N, bn);
  p.group_m = 16;
  p.k_splits = k_splits < 1 ? 1 : k_splits;
  p.kb_per_split = (int)cdiv(p.num_kb, p.k_splits);
  p.per_group_div = make_fastdiv(p.group_m * p.n_tiles);
  p.k_splits_div = make_fastdiv(p.k_splits);
  const int64_t tiles = (int64_t)p.m_tiles * p.n_tiles * p.k_splits;
  if (tiles == 0) return B200_OK;
  const int grid = (int)(tiles < sms ? tiles : sms);
  CUtensorMap ta, tb;
  int rc = make_tmap_u8(&ta, A, (uint64_t)p.M, (uint64_t)p.K, kBM, "A");
  if (rc) return rc;
  rc = make_tmap_u8(&tb, B, (uint64_t)b_rows_total, (uint64_t)p.K,
                    MODE == GEMM_GROUPED_SILU_QUANT ? 64u : (uint32_t)bn, "B");
  if (rc) return rc;
  if constexpr (MODE == GEMM_DENSE) {
    if (p.n_dest > 0) {
      // fan-out: one output map per destination buffer (unsplit only; the caller reduces split-K
      // partials itself and fans the sum out)
      if (p.n_dest > kMaxFan || p.k_splits != 1) {
        set_error_detail("gemm fan-out: %d destinations, %d K splits", p.n_dest, p.k_splits);
        return B200_E_BAD_ARG;
      }
      TmapOut<kMaxFan> tf;
      for (int d = 0; d < kMaxFan; ++d) {
        rc = make_tmap_out(&tf.m[d], p.dest[d < p.n_dest ? d : 0], 1, (uint64_t)p.M, (uint64_t)p.N, (int)sizeof(OutT),
                           std::is_same<OutT, __nv_bfloat16>::value, "fan-out C");
        if (rc) return rc;
      }
      if (bn == 256) return launch_gemm_inst<256, MODE, OutT, kMaxFan>(ta, tb, tf, p, grid, st);
      return launch_gemm_inst<128, MODE, OutT, kMaxFan>(ta, tb, tf, p, grid, st);
    }
  }
  // output map: dense -> C [splits, M, N]; gate_up -> FP8 activation [cap, I]; scatter -> unused
  TmapOut<1> tc;
  tc.m[0] = ta;
  if (MODE == GEMM_DENSE)
    rc = make_tmap_out(&tc.m[0], p.C, (uint64_t)p.k_splits, (uint64_t)p.M, (uint64_t)p.N, (int)sizeof(OutT),
                       std::is_same<OutT, __nv_bfloat16>::value, "C");
  else if (MODE == GEMM_GROUPED_SILU_QUANT)
    rc = make_tmap_out(&tc.m[0], p.q_out, 1, (uint64_t)p.M, (uint64_t)p.N, 1, false, "q_out");
  if (rc) return rc;
  if (bn == 256) return launch_gemm_inst<256, MODE, OutT>(ta, tb, tc, p, grid, st);
  if constexpr (MODE == GEMM_GROUPED_SILU_QUANT) {
    set_error_detail("gate_up GEMM needs 256-wide tiles");
    return B200_E_BAD_ARG;
  } else {
    return launch_gemm_inst<128, MODE, OutT>(ta, tb, tc, p, grid, st);
  }
}

}  // namespace b200
