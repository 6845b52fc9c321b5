// moe_align_block_size: bucket flat top-k expert ids, pad every bucket to a multiple of
// block_size, and emit the flat indices bucket by bucket in ASCENDING order (deterministic,
// no global atomics), the expert id of every block and the padded total.
//
// Integer / HBM-latency bound. Two shapes of launch:
//   numel <= 1024 : one 1024-thread block does everything (decode sizes, one launch);
//   otherwise     : histogram per 1024-id chunk -> one-block scan -> stable scatter,
//                   with the per-chunk histograms (int32 [chunks][buckets]) in the workspace.
// Algorithmic bytes: numel*sizeof(id) + 4*(max_pad + max_blocks + buckets + 2).
#include "common.cuh"

namespace b200 {

constexpr int kAlignThreads = 1024;
constexpr int kAlignWarps = kAlignThreads / 32;
constexpr int kMaxBuckets = 1025;  // 1024 experts + the "-1" bucket

template <typename IdT>
__device__ __forceinline__ int load_bucket(const IdT* ids, int64_t i, int64_t numel, int B) {
  if (i >= numel) return -1;
  const long long v = (long long)ids[i] + 1;
  return (v >= 0 && v < B) ? (int)v : -1;  // ids outside [-1, E) are ignored
}

// Stable rank of every thread's id among the ids of its bucket in this block.
// On return (after the trailing __syncthreads) warp_cnt[w*B+b] holds the number of ids of
// bucket b in warps < w, and the return value is this thread's rank inside its warp.
// block_tot[b] (shared, B ints) receives the block's count per bucket.
__device__ __forceinline__ int block_stable_rank(int bucket, int B, int* warp_cnt, int* block_tot) {
  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31;
  for (int i = tid; i < kAlignWarps * B; i += kAlignThreads) warp_cnt[i] = 0;
  __syncthreads();
  const unsigned same = __match_any_sync(0xffffffffu, bucket);
  const int rank = __popc(same & ((1u << lane) - 1u));
  if (bucket >= 0 && rank == 0) warp_cnt[w * B + bucket] = __popc(same);
  __syncthreads();
  for (int b = tid; b < B; b += kAlignThreads) {
    int run = 0;
#pragma unroll 8
    for (int ww = 0; ww < kAlignWarps; ++ww) {
      const int t = warp_cnt[ww * B + b];
      warp_cnt[ww * B + b] = run;
      run += t;
    }
    block_tot[b] = run;
  }
  __syncthreads();
  return rank;
}

// Exclusive scan over the B bucket sizes padded to block_size. In: cnt[b]. Out: start[b]
// (padded start of bucket b), start[B] = padded total. All 1024 threads must call.
__device__ __forceinline__ void bucket_scan(const int* cnt, int* start, int B, int block_size, int* warp_sums) {
  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31;
  const int b0 = 2 * tid, b1 = 2 * tid + 1;
  const int p0 = b0 < B ? (cnt[b0] + block_size - 1) / block_size * block_size : 0;
  const int p1 = b1 < B ? (cnt[b1] + block_size - 1) / block_size * block_size : 0;
  int v = p0 + p1, incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  if (lane == 31) warp_sums[w] = incl;
  __syncthreads();
  if (w == 0) {
    int t = warp_sums[lane], ti = t;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, ti, o);
      if (lane >= o) ti += n;
    }
    warp_sums[lane] = ti - t;  // exclusive
  }
  __syncthreads();
  const int excl = warp_sums[w] + incl - v;
  if (b0 < B) start[b0] = excl;
  if (b1 < B) start[b1] = excl + p0;
  if (b1 == B || b0 == B) start[B] = (b0 == B) ? excl : excl + p0;
  __syncthreads();
}

// expert id per block, padded total, cumsum: shared tail of both launch shapes.
__device__ __forceinline__ void write_block_outputs(const int* cnt, const int* start, int B, int block_size,
                                                    int32_t* expert_ids, int64_t max_blocks,
                                                    int32_t* num_post_pad, int32_t* cumsum) {
  const int tid = threadIdx.x;
  const int total = start[B];
  for (int b = tid; b < B; b += kAlignThreads) cumsum[b] = start[b] + cnt[b];
  // One thread per block (not per bucket: with expert parallelism the "not mine" bucket alone owns hundreds of
  // blocks, which one thread used to write in a row): the bucket of block i is the last b with
  // start[b] <= i * block_size; empty buckets share their start with the next one and are skipped by the search.
  const int nblocks = (int)min((int64_t)(total / block_size), max_blocks);
  for (int i = tid; i < nblocks; i += kAlignThreads) {
    const int pos = i * block_size;
    int lo = 0, hi = B;  // invariant: start[lo] <= pos < start[hi]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (start[mid] <= pos) lo = mid; else hi = mid;
    }
    expert_ids[i] = lo - 1;
  }
  for (int64_t i = total / block_size + tid; i < max_blocks; i += kAlignThreads) expert_ids[i] = -1;
  if (tid == 0) {
    cumsum[B] = total;
    *num_post_pad = total;
  }
}

// ------------------------------------------------------------------ numel <= 1024
template <typename IdT>
__global__ void __launch_bounds__(kAlignThreads) align_single_kernel(
    const IdT* __restrict__ ids, int64_t numel, int B, int block_size, int32_t* __restrict__ sorted,
    int64_t max_pad, int32_t* __restrict__ expert_ids, int64_t max_blocks, int32_t* __restrict__ num_post_pad,
    int32_t* __restrict__ cumsum) {
  extern __shared__ int smem[];
  int* warp_cnt = smem;                   // [32][B]
  int* cnt = warp_cnt + kAlignWarps * B;  // [B]
  int* start = cnt + B;                   // [B+1]
  __shared__ int warp_sums[32];
  const int tid = threadIdx.x;
  for (int64_t i = tid; i < max_pad; i += kAlignThreads) sorted[i] = (int32_t)numel;
  const int bucket = load_bucket(ids, tid, numel, B);
  const int rank = block_stable_rank(bucket, B, warp_cnt, cnt);
  bucket_scan(cnt, start, B, block_size, warp_sums);
  write_block_outputs(cnt, start, B, block_size, expert_ids, max_blocks, num_post_pad, cumsum);
  // the fill above and this scatter touch disjoint or identical slots only after a barrier
  __syncthreads();
  if (bucket >= 0) {
    const int64_t pos = (int64_t)start[bucket] + warp_cnt[(tid >> 5) * B + bucket] + rank;
    if (pos < max_pad) sorted[pos] = tid;  // always true when max_pad follows the reference's sizing
  }
}

// ------------------------------------------------------------------ numel > 1024
template <typename IdT>
__global__ void __launch_bounds__(kAlignThreads) align_hist_kernel(const IdT* __restrict__ ids, int64_t numel, int B,
                                                                   int32_t* __restrict__ sorted, int64_t max_pad,
                                                                   int32_t* __restrict__ chunk_hist) {
  extern __shared__ int smem[];
  int* hist = smem;  // [B]
  const int tid = threadIdx.x;
  for (int b = tid; b < B; b += kAlignThreads) hist[b] = 0;
  __syncthreads();
  const int64_t i = (int64_t)blockIdx.x * kAlignThreads + tid;
  const int bucket = load_bucket(ids, i, numel, B);
  if (bucket >= 0) atomicAdd(&hist[bucket], 1);
  for (int64_t j = i; j < max_pad; j += (int64_t)gridDim.x * kAlignThreads) sorted[j] = (int32_t)numel;
  __syncthreads();
  for (int b = tid; b < B; b += kAlignThreads) chunk_hist[(int64_t)blockIdx.x * B + b] = hist[b];
}

// One block: turns chunk_hist[c][b] into the global position of chunk c's first id of bucket b.
// Threads are laid out as (segment, bucket): kAlignThreads / B' segments (B' = buckets rounded up
// to a power of two <= 1024) each own a contiguous range of chunks, so the strided loads of one
// bucket are spread over several threads instead of being one long dependent chain.
__global__ void __launch_bounds__(kAlignThreads) align_scan_kernel(int32_t* __restrict__ chunk_hist, int chunks, int B,
                                                                   int block_size, int32_t* __restrict__ expert_ids,
                                                                   int64_t max_blocks, int32_t* __restrict__ num_post_pad,
                                                                   int32_t* __restrict__ cumsum) {
  extern __shared__ int smem[];
  int* cnt = smem;            // [B]
  int* start = cnt + B;       // [B+1]
  int* seg_sum = start + B + 1;  // [segs][B]: ids of bucket b in the chunks of segment s
  __shared__ int warp_sums[32];
  const int tid = threadIdx.x;
  int bp = 32;
  while (bp < B && bp < kAlignThreads) bp <<= 1;
  const int segs = B > kAlignThreads ? 1 : kAlignThreads / bp;
  const int per_seg = (chunks + segs - 1) / segs;
  for (int b = tid % bp, sgm = tid / bp; b < B && sgm < segs; b += bp) {  // b += bp only loops when B > 1024
    const int c0 = sgm * per_seg, c1 = min(chunks, c0 + per_seg);
    int run = 0;
#pragma unroll 8
    for (int c = c0; c < c1; ++c) run += chunk_hist[(int64_t)c * B + b];
    seg_sum[sgm * B + b] = run;
  }
  __syncthreads();
  for (int b = tid; b < B; b += kAlignThreads) {
    int run = 0;
    for (int sgm = 0; sgm < segs; ++sgm) {
      const int t = seg_sum[sgm * B + b];
      seg_sum[sgm * B + b] = run;  // ids of bucket b in earlier segments
      run += t;
    }
    cnt[b] = run;
  }
  __syncthreads();
  bucket_scan(cnt, start, B, block_size, warp_sums);
  write_block_outputs(cnt, start, B, block_size, expert_ids, max_blocks, num_post_pad, cumsum);
  for (int b = tid % bp, sgm = tid / bp; b < B && sgm < segs; b += bp) {
    const int c0 = sgm * per_seg, c1 = min(chunks, c0 + per_seg);
    int run = start[b] + seg_sum[sgm * B + b];
#pragma unroll 8
    for (int c = c0; c < c1; ++c) {
      const int t = chunk_hist[(int64_t)c * B + b];
      chunk_hist[(int64_t)c * B + b] = run;
      run += t;
    }
  }
}

template <typename IdT>
__global__ void __launch_bounds__(kAlignThreads) align_scatter_kernel(const IdT* __restrict__ ids, int64_t numel, int B,
                                                                      const int32_t* __restrict__ chunk_base,
                                                                      int32_t* __restrict__ sorted, int64_t max_pad) {
  extern __shared__ int smem[];
  int* warp_cnt = smem;                   // [32][B]
  int* cnt = warp_cnt + kAlignWarps * B;  // [B] (unused result)
  const int tid = threadIdx.x;
  const int64_t i = (int64_t)blockIdx.x * kAlignThreads + tid;
  const int bucket = load_bucket(ids, i, numel, B);
  const int rank = block_stable_rank(bucket, B, warp_cnt, cnt);
  if (bucket >= 0) {
    const int64_t pos = (int64_t)chunk_base[(int64_t)blockIdx.x * B + bucket] + warp_cnt[(tid >> 5) * B + bucket] + rank;
    if (pos < max_pad) sorted[pos] = (int32_t)i;
  }
}

template <typename IdT>
static int launch_align(const void* ids_, int64_t numel, int B, int block_size, int32_t* sorted, int64_t max_pad,
                        int32_t* expert_ids, int64_t max_blocks, int32_t* num_post_pad, int32_t* cumsum, void* ws,
                        cudaStream_t st) {
  const IdT* ids = static_cast<const IdT*>(ids_);
  const size_t rank_smem = (size_t)(kAlignWarps * B + 2 * B + 1) * sizeof(int);
  if (numel <= kAlignThreads) {
    auto k = align_single_kernel<IdT>;
    if (rank_smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)rank_smem);
    k<<<1, kAlignThreads, rank_smem, st>>>(ids, numel, B, block_size, sorted, max_pad, expert_ids, max_blocks,
                                           num_post_pad, cumsum);
    return check_launch("moe_align_block_size (single block)");
  }
  const int chunks = (int)cdiv(numel, kAlignThreads);
  int32_t* chunk_hist = static_cast<int32_t*>(ws);
  align_hist_kernel<IdT><<<chunks, kAlignThreads, (size_t)B * sizeof(int), st>>>(ids, numel, B, sorted, max_pad, chunk_hist);
  int bp = 32;
  while (bp < B && bp < kAlignThreads) bp <<= 1;
  const int segs = B > kAlignThreads ? 1 : kAlignThreads / bp;
  align_scan_kernel<<<1, kAlignThreads, (size_t)(2 * B + 1 + segs * B) * sizeof(int), st>>>(chunk_hist, chunks, B, block_size,
                                                                               expert_ids, max_blocks, num_post_pad, cumsum);
  auto k = align_scatter_kernel<IdT>;
  if (rank_smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)rank_smem);
  k<<<chunks, kAlignThreads, rank_smem, st>>>(ids, numel, B, chunk_hist, sorted, max_pad);
  return check_launch("moe_align_block_size");
}

// ---------------------------------------------------------------- allocation-free variant
// Scratch for callers that must not allocate device memory: the per-chunk histograms of the
// multi-block path live in this fixed array instead of a caller-provided workspace. Every
// device that loads the library carries the array (about 129 KB) until the process exits.
constexpr int64_t kStaticAlignMaxNumel = 131072;  // e.g. 16384 tokens x top-8
constexpr int kStaticAlignMaxBuckets = 257;       // 256 experts + the "-1" bucket
static __device__ __align__(256) int32_t g_align_static_scratch[(kStaticAlignMaxNumel / kAlignThreads) *
                                                                kStaticAlignMaxBuckets];

// Device address of the array on the CURRENT device. The symbol name is only a host-side
// handle; a kernel must be given the address cudaGetSymbolAddress reports for that device.
static int32_t* align_static_scratch_ptr() {
  constexpr int kMaxDevices = 64;
  static int32_t* cache[kMaxDevices] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_error_detail("align (static scratch): cannot identify the current device");
    return nullptr;
  }
  if (cache[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_align_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_error_detail("align (static scratch): cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    cache[dev] = static_cast<int32_t*>(p);  // same value from any thread: a benign race
  }
  return cache[dev];
}

}  // namespace b200

extern "C" size_t b200_moe_align_workspace_bytes(int64_t numel, int num_buckets) {
  if (numel <= b200::kAlignThreads || num_buckets <= 0) return 0;
  return (size_t)b200::cdiv(numel, b200::kAlignThreads) * (size_t)num_buckets * sizeof(int32_t);
}

extern "C" int b200_moe_align_block_size(const void* topk_ids, int ids_dtype, int64_t numel, int num_buckets,
                                         int block_size, int32_t* sorted_token_ids, int64_t max_pad,
                                         int32_t* expert_ids, int64_t max_blocks, int32_t* num_post_pad,
                                         int32_t* cumsum, int pad_sorted, void* workspace, size_t workspace_bytes,
                                         void* stream) {
  using namespace b200;
  (void)pad_sorted;  // pad slots are always written (a superset of both reference behaviours)
  B200_CHECK_ARG(numel >= 0 && max_pad >= 0 && max_blocks >= 0, "align: negative size");
  B200_CHECK_ARG(num_buckets >= 1 && block_size >= 1, "align: num_buckets=%d block_size=%d", num_buckets, block_size);
  B200_UNSUPPORTED(num_buckets > kMaxBuckets, "align: more than %d buckets", kMaxBuckets);
  B200_UNSUPPORTED(numel >= (1LL << 30), "align: numel too large for int32 positions");
  B200_CHECK_ARG(num_post_pad && cumsum, "align: null output");
  B200_CHECK_ARG((sorted_token_ids || max_pad == 0) && (expert_ids || max_blocks == 0), "align: null output");
  B200_CHECK_ARG(numel == 0 || topk_ids, "align: null topk_ids");
  // worst case every bucket needs block_size-1 pads
  B200_CHECK_ARG(max_pad >= 0 && max_blocks * block_size >= 0, "align: bad output sizes");
  const size_t need = b200_moe_align_workspace_bytes(numel, num_buckets);
  if (need && (!workspace || workspace_bytes < need)) {
    set_error_detail("align: workspace %zu < %zu bytes", workspace_bytes, need);
    return B200_E_WORKSPACE;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (ids_dtype == B200_I32)
    return launch_align<int32_t>(topk_ids, numel, num_buckets, block_size, sorted_token_ids, max_pad, expert_ids,
                                 max_blocks, num_post_pad, cumsum, workspace, st);
  if (ids_dtype == B200_I64)
    return launch_align<int64_t>(topk_ids, numel, num_buckets, block_size, sorted_token_ids, max_pad, expert_ids,
                                 max_blocks, num_post_pad, cumsum, workspace, st);
  set_error_detail("align: ids dtype code %d is not int32/int64", ids_dtype);
  return B200_E_BAD_ARG;
}

extern "C" int b200_moe_align_block_size_static(const void* topk_ids, int ids_dtype, int64_t numel, int num_buckets,
                                                int block_size, int32_t* sorted_token_ids, int64_t max_pad,
                                                int32_t* expert_ids, int64_t max_blocks, int32_t* num_post_pad,
                                                int32_t* cumsum, void* stream) {
  using namespace b200;
  if (numel > kStaticAlignMaxNumel || num_buckets > kStaticAlignMaxBuckets) {
    set_error_detail("align (static scratch): numel=%lld / num_buckets=%d exceed the built-in limits of %lld ids and "
                     "%d buckets; use b200_moe_align_block_size with a workspace",
                     (long long)numel, num_buckets, (long long)kStaticAlignMaxNumel, kStaticAlignMaxBuckets);
    return B200_E_UNSUPPORTED;
  }
  int32_t* scratch = align_static_scratch_ptr();
  if (scratch == nullptr) return B200_E_LAUNCH;
  return b200_moe_align_block_size(topk_ids, ids_dtype, numel, num_buckets, block_size, sorted_token_ids, max_pad,
                                   expert_ids, max_blocks, num_post_pad, cumsum, 1, scratch,
                                   sizeof(int32_t) * (size_t)(kStaticAlignMaxNumel / kAlignThreads) * kStaticAlignMaxBuckets,
                                   stream);
}
