// Tensor-parallel all-reduce of the row-parallel linear, built around peer memory instead of a
// library collective. The GEMM's epilogue has already written this rank's partial [M, N] into
// slot `rank` of the destination ranks' slot buffers (fan-out stores over NVLink, tile by tile
// while the GEMM runs); what is left is
//   1. a cross-rank "partials have landed" handshake,
//   2. out = sum over ranks of slot[r] (fp32, rank order: every rank gets the same bits),
//      optionally + residual and RMSNorm (the reference fuses the same three steps,
//      python/sglang/srt/layers/flashinfer_comm_fusion.py, layernorm.py forward_native),
//   3. two-shot only: the owner of a 128-row block writes its result into every rank's output.
// Handshakes are epoch counters in a small flag array per rank: rank r writes epoch into
// peer[d].flags[r] with a system-scope release after a system fence, and polls its own
// flags[0..n) with system-scope acquires. Every poll is bounded (2 s by default): on expiry the kernel
// records status 2 in the device status word and returns without touching peer memory again.
// epoch == 0 selects device-side epochs: the call's epoch is 1 + a counter kept next to the flags
// (flags[16 + phase]), bumped by the last block of the kernel, so the identical launch can be
// replayed from a CUDA graph; all ranks then advance in lockstep because they replay the same
// sequence of calls. A flag array is used with host epochs or with device epochs, never both.
// Slots written by peers are read with L2-only loads (ld.global.cg): the L1 of this SM may
// still hold lines of the previous call that used the same buffer.
#include "common.cuh"

namespace b200 {

constexpr int kMaxRanks = 8;

struct AllReduceParams {
  const void* slots;  // local [n_ranks][slot_stride], slot r = rank r's partial [M][N]
  int64_t slot_stride;  // elements between slots (>= M*N)
  void* out[kMaxRanks];       // one-shot: out[0] (local). two-shot: out[d] = rank d's output buffer
  const void* residual;       // [M, N] or null
  void* residual_out[kMaxRanks];  // like out: [M, N] buffers for sum + residual, or null (may alias residual)
  // two-shot with NVSwitch multicast: one address that maps every rank's output buffer; a
  // multimem.st to it is replicated by the switch, so the owner sends each result once instead
  // of once per rank. Null: plain peer stores to out[d] / residual_out[d].
  void* out_mc;
  void* residual_out_mc;
  const void* rms_weight;     // [N] or null
  uint32_t* my_flags;         // local [2][kMaxRanks]
  uint32_t* peer_flags[kMaxRanks];
  int* status;
  int64_t M, N;
  int n_ranks, rank;
  int by_tile;  // two-shot: reduce only row blocks mt % n_ranks == rank, write them to every rank
  uint32_t epoch;
  float eps;
  unsigned long long wait_ns;  // limit of every poll
};

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// 16 bytes to every replica of a multicast address (no data conversion: the type only sizes it)
__device__ __forceinline__ void multimem_st_16(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Thread d < n signals rank d; returns after it has seen every rank's signal or the time limit.
// `phase` selects the flag row. Epochs only grow, so `>=` tolerates a rank that is already a
// call ahead.
__device__ bool handshake(uint32_t* my_flags, uint32_t* const* peer_flags, int n, int rank, int phase, uint32_t epoch,
                          bool signal, unsigned long long wait_ns) {
  const int d = threadIdx.x;
  bool ok = true;
  if (d < n) {
    if (signal) {
      __threadfence_system();
      st_release_sys(peer_flags[d] + phase * kMaxRanks + rank, epoch);
    }
    const unsigned long long t0 = now_ns();
    while ((int32_t)(ld_acquire_sys(my_flags + phase * kMaxRanks + d) - epoch) < 0) {
      if (now_ns() - t0 > wait_ns) {
        ok = false;
        break;
      }
      __nanosleep(100);
    }
  }
  return ok;
}

constexpr int kCounterBase = 2 * kMaxRanks;  // flags[16 + phase]: device-side epoch counters
constexpr int kTicket = kCounterBase + 2;     // flags[18]: blocks of the running kernel that are done

// Last block out bumps the device-side epoch counter of `phase` (device epochs only).
__device__ void finish_epoch(uint32_t* my_flags, int phase, bool device_epoch) {
  if (!device_epoch) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(my_flags + kTicket, 1u) == gridDim.x - 1) {
      my_flags[kTicket] = 0;
      __threadfence();
      atomicAdd(my_flags + kCounterBase + phase, 1u);
    }
  }
}

// NR = number of ranks (compile time: the slot loop unrolls and all its loads are in flight together)
template <typename T, int NR>
__global__ void __launch_bounds__(256) allreduce_finish_kernel(const AllReduceParams p) {
  __shared__ int s_ok;
  __shared__ float s_red[8];
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  const bool device_epoch = p.epoch == 0;
  // stable for the whole kernel: the counter moves only when every block has finished
  const uint32_t epoch = device_epoch ? *reinterpret_cast<volatile uint32_t*>(p.my_flags + kCounterBase) + 1u : p.epoch;
  // block 0 announces this rank's partials; every block waits for all ranks' announcements
  if (!handshake(p.my_flags, p.peer_flags, p.n_ranks, p.rank, 0, epoch, blockIdx.x == 0, p.wait_ns)) atomicExch(&s_ok, 0);
  __syncthreads();
  const int64_t N = p.N;
  if (!s_ok) {
    // A rank never announced its partials: report it, and poison this rank's own result with NaNs
    // so that a caller that does not poll the status word cannot mistake stale bytes for a sum.
    if (threadIdx.x == 0) atomicCAS(p.status, 0, 2);
    const uint4 nan16 = make_uint4(0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu);  // NaN in bf16 and fp16
    T* mine = static_cast<T*>(p.out[p.by_tile ? p.rank : 0]);
    T* mine_res = static_cast<T*>(p.residual_out[p.by_tile ? p.rank : 0]);
    for (int64_t row = blockIdx.x; row < p.M; row += gridDim.x)
      for (int64_t c = threadIdx.x * 8; c < N; c += (int64_t)blockDim.x * 8) {
        *reinterpret_cast<uint4*>(mine + row * N + c) = nan16;
        if (mine_res != nullptr && mine_res != p.residual) *reinterpret_cast<uint4*>(mine_res + row * N + c) = nan16;
      }
    finish_epoch(p.my_flags, 0, device_epoch);
    return;
  }
  const T* __restrict__ slots = static_cast<const T*>(p.slots);
  const T* residual = static_cast<const T*>(p.residual);  // may be the same buffer as residual_out (in place)
  const T* w = static_cast<const T*>(p.rms_weight);
  const int n_out = p.by_tile ? p.n_ranks : 1;
  // fp32 sums of one 8-element chunk of a row: the slots in rank order, then the residual
  auto sum_chunk = [&](int64_t row, int64_t c, float (&acc)[8]) {
    uint4 raw[NR + 1];
#pragma unroll
    for (int r = 0; r < NR; ++r)
      raw[r] = __ldcg(reinterpret_cast<const uint4*>(slots + (int64_t)r * p.slot_stride + row * N + c));
    raw[NR] = residual != nullptr ? *reinterpret_cast<const uint4*>(residual + row * N + c) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
    for (int r = 0; r <= NR; ++r) {  // rank order, then the residual (+0 when there is none)
      const T* h = reinterpret_cast<const T*>(&raw[r]);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += to_f32<T>(h[i]);
    }
  };
  auto store_out = [&](int64_t row, int64_t c, const uint4& o) {
    if (p.out_mc != nullptr) multimem_st_16(static_cast<T*>(p.out_mc) + row * N + c, o);
    else
      for (int d = 0; d < n_out; ++d) *reinterpret_cast<uint4*>(static_cast<T*>(p.out[d]) + row * N + c) = o;
  };
  // With a norm the row is needed twice (sum of squares, then the scaled values). The sums of the
  // first kKeep chunks per thread (rows up to 8192 columns) stay in registers between the two
  // passes; anything beyond is summed again from the slots.
  constexpr int kKeep = 4;
  const int64_t stride = (int64_t)blockDim.x * 8;
  for (int64_t row = blockIdx.x; row < p.M; row += gridDim.x) {
    if (p.by_tile && (row / 128) % p.n_ranks != p.rank) continue;
    float ss = 0.f;
    float keep[kKeep][8];
    // pass 1: sum (+ residual) -> residual_out, and -> out when there is no norm
    auto pass1 = [&](int64_t c, float (&acc)[8]) {
      sum_chunk(row, c, acc);
      uint4 o;
      T* oh = reinterpret_cast<T*>(&o);
#pragma unroll
      for (int i = 0; i < 8; ++i) oh[i] = from_f32<T>(acc[i]);
      if (p.residual_out[0] != nullptr) {
        if (p.residual_out_mc != nullptr) multimem_st_16(static_cast<T*>(p.residual_out_mc) + row * N + c, o);
        else
          for (int d = 0; d < n_out; ++d) *reinterpret_cast<uint4*>(static_cast<T*>(p.residual_out[d]) + row * N + c) = o;
      }
      if (w == nullptr) {
        store_out(row, c, o);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += acc[i] * acc[i];
      }
    };
#pragma unroll
    for (int it = 0; it < kKeep; ++it) {
      const int64_t c = threadIdx.x * 8 + it * stride;
      if (c < N) pass1(c, keep[it]);
    }
    for (int64_t c = threadIdx.x * 8 + kKeep * stride; c < N; c += stride) {
      float acc[8];
      pass1(c, acc);
    }
    if (w != nullptr) {
      // RMSNorm over the row from the unrounded fp32 sums
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = ss;
      __syncthreads();
      float tot = 0.f;
      for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += s_red[i];
      const float inv = rsqrtf(tot / (float)N + p.eps);
      __syncthreads();
      auto pass2 = [&](int64_t c, const float (&acc)[8]) {
        const uint4 wv = *reinterpret_cast<const uint4*>(w + c);
        const T* wh = reinterpret_cast<const T*>(&wv);
        uint4 o;
        T* oh = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int i = 0; i < 8; ++i) oh[i] = from_f32<T>(acc[i] * inv * to_f32<T>(wh[i]));
        store_out(row, c, o);
      };
#pragma unroll
      for (int it = 0; it < kKeep; ++it) {
        const int64_t c = threadIdx.x * 8 + it * stride;
        if (c < N) pass2(c, keep[it]);
      }
      for (int64_t c = threadIdx.x * 8 + kKeep * stride; c < N; c += stride) {
        float acc[8];
        sum_chunk(row, c, acc);  // residual_out never aliases residual when a norm is asked for
        pass2(c, acc);
      }
    }
  }
  finish_epoch(p.my_flags, 0, device_epoch);
}

// Two-shot tail: "my results are in your output" handshake (flag row 1). One block.
__global__ void __launch_bounds__(32) allreduce_results_landed_kernel(const AllReduceParams p) {
  const bool device_epoch = p.epoch == 0;
  const uint32_t epoch = device_epoch ? *reinterpret_cast<volatile uint32_t*>(p.my_flags + kCounterBase + 1) + 1u : p.epoch;
  const bool ok = handshake(p.my_flags, p.peer_flags, p.n_ranks, p.rank, 1, epoch, true, p.wait_ns);
  if (!__all_sync(0xffffffffu, ok)) {
    // an owner never delivered its row blocks: report it and poison this rank's result (slow, one warp:
    // this is the failure path)
    if (threadIdx.x == 0) atomicCAS(p.status, 0, 2);
    const uint4 nan16 = make_uint4(0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu);
    uint4* mine = static_cast<uint4*>(p.out[p.rank]);
    for (int64_t i = threadIdx.x; i < p.M * p.N / 8; i += 32) mine[i] = nan16;
  }
  finish_epoch(p.my_flags, 1, device_epoch);
}

}  // namespace b200

extern "C" int b200_allreduce_finish(const void* slots, int64_t slot_stride, void* const* out, int dtype, int64_t M, int64_t N, int n_ranks,
                                     int rank, int by_tile, const void* residual, void* const* residual_out,
                                     const void* rms_weight, float eps, void* my_flags, void* const* peer_flags,
                                     uint32_t epoch, void* out_multicast, void* residual_out_multicast, void* stream) {
  using namespace b200;
  B200_CHECK_ARG(M >= 0 && N > 0 && n_ranks >= 1 && n_ranks <= kMaxRanks && rank >= 0 && rank < n_ranks,
                 "allreduce_finish: bad shape M=%lld N=%lld ranks=%d rank=%d", (long long)M, (long long)N, n_ranks, rank);
  if (M == 0) return B200_OK;
  B200_CHECK_ARG(slots && out && my_flags && peer_flags, "allreduce_finish: null pointer");
  B200_CHECK_ARG(slot_stride >= M * N && slot_stride % 8 == 0 && ((uintptr_t)slots & 15) == 0,
                 "allreduce_finish: slot stride %lld for M*N=%lld, or unaligned slots", (long long)slot_stride,
                 (long long)(M * N));
  B200_UNSUPPORTED(N % 8 != 0, "allreduce_finish: N=%lld must be a multiple of 8", (long long)N);
  B200_CHECK_ARG(dtype == B200_BF16 || dtype == B200_F16, "allreduce_finish: dtype code %d is not bf16/f16", dtype);
  // In place (residual_out == residual) each element is read and written by the same thread in
  // pass 1, but the norm's second pass would then read the updated value: not supported together.
  B200_UNSUPPORTED(rms_weight != nullptr && residual != nullptr && residual_out != nullptr && residual_out[0] == residual,
                   "allreduce_finish: an RMSNorm needs residual_out separate from residual");
  AllReduceParams p = {};
  p.slots = slots; p.slot_stride = slot_stride; p.residual = residual; p.rms_weight = rms_weight;
  p.my_flags = static_cast<uint32_t*>(my_flags); p.M = M; p.N = N; p.n_ranks = n_ranks; p.rank = rank;
  p.by_tile = by_tile != 0; p.epoch = epoch; p.eps = eps; p.wait_ns = peer_wait_ns();
  if (p.by_tile) {  // multicast only replaces the fan-out of the two-shot mode
    B200_CHECK_ARG(((uintptr_t)out_multicast & 15) == 0 && ((uintptr_t)residual_out_multicast & 15) == 0,
                   "allreduce_finish: unaligned multicast address");
    p.out_mc = out_multicast;
    p.residual_out_mc = residual_out != nullptr ? residual_out_multicast : nullptr;
  }
  p.status = device_status_word();
  if (!p.status) {
    set_error_detail("cannot resolve the device status word");
    return B200_E_LAUNCH;
  }
  const int n_out = p.by_tile ? n_ranks : 1;
  for (int d = 0; d < n_out; ++d) {
    B200_CHECK_ARG(out[d] && ((uintptr_t)out[d] & 15) == 0, "allreduce_finish: output %d null or unaligned", d);
    p.out[d] = out[d];
    if (residual_out != nullptr) {
      B200_CHECK_ARG(residual_out[d] && ((uintptr_t)residual_out[d] & 15) == 0,
                     "allreduce_finish: residual output %d null or unaligned", d);
      p.residual_out[d] = residual_out[d];
    }
  }
  for (int d = 0; d < n_ranks; ++d) {
    B200_CHECK_ARG(peer_flags[d] != nullptr, "allreduce_finish: flag pointer %d is null", d);
    p.peer_flags[d] = static_cast<uint32_t*>(peer_flags[d]);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int sms = 148;
  {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int64_t want = M < (int64_t)sms * 8 ? M : (int64_t)sms * 8;
#define B200_FINISH(NR)                                                                           \
  case NR:                                                                                        \
    if (dtype == B200_BF16) allreduce_finish_kernel<__nv_bfloat16, NR><<<(unsigned)want, 256, 0, st>>>(p); \
    else allreduce_finish_kernel<__half, NR><<<(unsigned)want, 256, 0, st>>>(p);                  \
    break;
  switch (n_ranks) {
    B200_FINISH(1) B200_FINISH(2) B200_FINISH(3) B200_FINISH(4) B200_FINISH(5) B200_FINISH(6) B200_FINISH(7) B200_FINISH(8)
    default: break;
  }
#undef B200_FINISH
  int rc = check_launch("allreduce_finish_kernel");
  if (rc || !p.by_tile) return rc;
  allreduce_results_landed_kernel<<<1, 32, 0, st>>>(p);
  return check_launch("allreduce_results_landed_kernel");
}
