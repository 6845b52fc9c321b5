// Expert-parallel token exchange over NVLink peer memory (no library collective, no host sync).
//
// Rank r owns experts [r*E/p, (r+1)*E/p). Every rank holds a receive area laid out by SOURCE rank
// and SOURCE token index, recv[s][t] for s < p, t < T_max, made of four arrays:
//   q   [p][T_max][H]      FP8 bytes of the token row
//   s   [p][T_max][H/128]  its 1x128 scales (row-major)
//   w   [p][T_max][k]      router weights
//   ids [p][T_max][k]      expert ids rebased to the owner (-1: not for this rank / no such token)
// Fixed positions mean no counts to exchange, no prefix sums and no atomics: a source stores each
// of its tokens straight into the owners' areas (dispatch), the owners run the grouped GEMMs over
// all p*T_max positions (positions nobody filled carry ids -1 and are skipped by the alignment
// step), and the source sums the partial rows straight out of the owners' output areas
// out[s][t][H] with peer loads (combine). The cross-rank ordering -- "dispatch has landed",
// "expert outputs are ready" -- is the bounded epoch handshake below, as its own tiny kernel:
// kernels of one GPU never wait for one another, only for other GPUs' flags.
//
// Reference semantics: python/sglang/srt/layers/moe/token_dispatcher/deepep.py:507-602 (normal
// dispatch: FP8 rows + scales + topk ids / weights to the owning ranks; combine: partial rows
// back, summed at the source) and standard.py:172-210 (id rebasing).
#include "common.cuh"

namespace b200 {

constexpr int kEpMaxRanks = 8;
constexpr int kEpMaxTopk = 32;

struct EpDispatchParams {
  const uint8_t* x_q;        // [T, H]
  const float* x_s;          // [T, H/128]
  const float* topk_weights; // [T, k]
  const int32_t* topk_ids;   // [T, k] global expert ids (-1 allowed)
  uint8_t* recv_q[kEpMaxRanks];   // per destination rank: base of its q area
  float* recv_s[kEpMaxRanks];
  float* recv_w[kEpMaxRanks];
  int32_t* recv_ids[kEpMaxRanks];
  int64_t T, T_max, H;
  int k, E, p, rank;
};

// One block per source token position t < T_max (positions >= T only publish ids = -1).
__global__ void __launch_bounds__(128) ep_dispatch_kernel(const EpDispatchParams a) {
  const int64_t t = blockIdx.x;
  const int per = a.E / a.p;
  __shared__ int s_ids[kEpMaxTopk];
  __shared__ float s_w[kEpMaxTopk];
  if (threadIdx.x < a.k) {
    const bool real = t < a.T;
    s_ids[threadIdx.x] = real ? a.topk_ids[t * a.k + threadIdx.x] : -1;
    s_w[threadIdx.x] = real ? a.topk_weights[t * a.k + threadIdx.x] : 0.f;
  }
  __syncthreads();
  const int64_t slot = (int64_t)a.rank * a.T_max + t;  // my position in every destination's area
  const int64_t chunks = a.H / 16, groups = a.H / 128;
  for (int d = 0; d < a.p; ++d) {
    bool need = false;
    for (int j = 0; j < a.k; ++j) need |= s_ids[j] >= d * per && s_ids[j] < (d + 1) * per;
    if (threadIdx.x < a.k) {
      const int id = s_ids[threadIdx.x];
      const bool mine = id >= d * per && id < (d + 1) * per;
      a.recv_ids[d][slot * a.k + threadIdx.x] = mine ? id - d * per : -1;
      if (need) a.recv_w[d][slot * a.k + threadIdx.x] = s_w[threadIdx.x];
    }
    if (!need) continue;  // uniform over the block
    const uint4* src = reinterpret_cast<const uint4*>(a.x_q + t * a.H);
    uint4* dst = reinterpret_cast<uint4*>(a.recv_q[d] + slot * a.H);
    for (int64_t c = threadIdx.x; c < chunks; c += blockDim.x) dst[c] = ld_nc_16(src + c);
    for (int64_t g = threadIdx.x; g < groups; g += blockDim.x) a.recv_s[d][slot * groups + g] = a.x_s[t * groups + g];
  }
}

struct EpCombineParams {
  const void* peer_out[kEpMaxRanks];  // per owner rank: base of its out area [p][T_max][H]
  const int32_t* topk_ids;            // [T, k] global ids of the local tokens
  void* out;                          // [T, H]
  const int* status;                  // device status word: non-zero = a handshake of this call gave up
  int64_t T, T_max, H;
  int k, E, p, rank;
};

// out[t] = sum over the owner ranks d of token t (ascending d, fp32) of d.out[rank][t].
template <typename T>
__global__ void __launch_bounds__(128) ep_combine_kernel(const EpCombineParams a) {
  const int64_t t = blockIdx.x;
  const int per = a.E / a.p;
  __shared__ int s_need[kEpMaxRanks];
  if (threadIdx.x < a.p) {
    const int d = threadIdx.x;
    bool need = false;
    for (int j = 0; j < a.k; ++j) {
      const int id = a.topk_ids[t * a.k + j];
      need |= id >= d * per && id < (d + 1) * per;
    }
    s_need[d] = need;
  }
  __syncthreads();
  const int64_t slot = (int64_t)a.rank * a.T_max + t;
  T* out = static_cast<T*>(a.out) + t * a.H;
  if (*reinterpret_cast<const volatile int*>(a.status) != 0) {
    // an owner never said "outputs ready" (the handshake before this kernel ran out): its rows are stale.
    // Poison the result with NaNs so that a caller that does not poll the status word notices.
    const uint4 nan16 = make_uint4(0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu);  // NaN in bf16 and fp16
    for (int64_t c = threadIdx.x * 8; c < a.H; c += blockDim.x * 8) *reinterpret_cast<uint4*>(out + c) = nan16;
    return;
  }
  for (int64_t c = threadIdx.x * 8; c < a.H; c += blockDim.x * 8) {
    // all owners' rows are requested before any is used: the peer loads overlap instead of
    // paying one NVLink round trip after the other
    uint4 v[kEpMaxRanks];
#pragma unroll
    for (int d = 0; d < kEpMaxRanks; ++d) {
      v[d] = make_uint4(0, 0, 0, 0);
      // written by another GPU's kernels: L2-only load (no stale L1 line of an earlier call)
      if (d < a.p && s_need[d])
        v[d] = __ldcg(reinterpret_cast<const uint4*>(static_cast<const T*>(a.peer_out[d]) + slot * a.H + c));
    }
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int d = 0; d < kEpMaxRanks; ++d) {  // ascending rank; a rank that is not needed contributes +0
      const T* h = reinterpret_cast<const T*>(&v[d]);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += to_f32<T>(h[i]);
    }
    uint4 o;
    T* oh = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int i = 0; i < 8; ++i) oh[i] = from_f32<T>(acc[i]);
    *reinterpret_cast<uint4*>(out + c) = o;
  }
}

// Epoch handshake: thread d signals rank d (system fence, release store of `epoch` into
// peer[d].flags[phase][rank]) and waits until its own flags[phase][d] has reached `epoch`.
// Bounded: after the wait limit (2 s by default) the device status word becomes 2 and the kernel
// returns.
struct HandshakeParams {
  uint32_t* my_flags;
  uint32_t* peer_flags[kEpMaxRanks];
  int* status;
  int p, rank, phase;
  uint32_t epoch;
  unsigned long long wait_ns;
};

__global__ void __launch_bounds__(32) peer_handshake_kernel(const HandshakeParams a) {
  const int d = threadIdx.x;
  bool ok = true;
  // epoch 0 = device-side epochs: 1 + the counter kept at flags[16 + phase] (bumped below), so the
  // identical launch can be replayed from a CUDA graph
  uint32_t* counter = a.my_flags + 2 * kEpMaxRanks + a.phase;
  const uint32_t epoch = a.epoch != 0 ? a.epoch : *reinterpret_cast<volatile uint32_t*>(counter) + 1u;
  __syncwarp();
  if (d < a.p) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.peer_flags[d] + a.phase * kEpMaxRanks + a.rank), "r"(epoch)
                 : "memory");
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    for (;;) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(a.my_flags + a.phase * kEpMaxRanks + d) : "memory");
      if ((int32_t)(v - epoch) >= 0) break;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
      if (t1 - t0 > a.wait_ns) {
        ok = false;
        break;
      }
      __nanosleep(100);
    }
  }
  if (!__all_sync(0xffffffffu, ok) && threadIdx.x == 0) atomicCAS(a.status, 0, 2);
  if (a.epoch == 0 && threadIdx.x == 0) *counter = epoch;
}

}  // namespace b200

extern "C" int b200_ep_dispatch(const void* x_q, const float* x_s, const float* topk_weights, const int32_t* topk_ids,
                                int64_t T, int64_t T_max, int topk, int64_t H, int E, int n_ranks, int rank,
                                void* const* recv_q, void* const* recv_s, void* const* recv_w, void* const* recv_ids,
                                void* stream) {
  using namespace b200;
  B200_CHECK_ARG(T >= 0 && T_max >= T && T_max > 0 && topk > 0 && topk <= kEpMaxTopk && H > 0 && E > 0,
                 "ep_dispatch: bad shape T=%lld T_max=%lld topk=%d H=%lld E=%d", (long long)T, (long long)T_max, topk,
                 (long long)H, E);
  B200_CHECK_ARG(n_ranks >= 1 && n_ranks <= kEpMaxRanks && rank >= 0 && rank < n_ranks && E % n_ranks == 0,
                 "ep_dispatch: ranks=%d rank=%d E=%d", n_ranks, rank, E);
  B200_UNSUPPORTED(H % 128 != 0, "ep_dispatch: H=%lld must be a multiple of 128", (long long)H);
  B200_CHECK_ARG((T == 0 || (x_q && x_s && topk_weights && topk_ids)) && recv_q && recv_s && recv_w && recv_ids,
                 "ep_dispatch: null pointer");
  EpDispatchParams a = {};
  a.x_q = static_cast<const uint8_t*>(x_q); a.x_s = x_s; a.topk_weights = topk_weights; a.topk_ids = topk_ids;
  a.T = T; a.T_max = T_max; a.H = H; a.k = topk; a.E = E; a.p = n_ranks; a.rank = rank;
  for (int d = 0; d < n_ranks; ++d) {
    B200_CHECK_ARG(recv_q[d] && recv_s[d] && recv_w[d] && recv_ids[d] && ((uintptr_t)recv_q[d] & 15) == 0,
                   "ep_dispatch: receive area %d null or unaligned", d);
    a.recv_q[d] = static_cast<uint8_t*>(recv_q[d]); a.recv_s[d] = static_cast<float*>(recv_s[d]);
    a.recv_w[d] = static_cast<float*>(recv_w[d]); a.recv_ids[d] = static_cast<int32_t*>(recv_ids[d]);
  }
  ep_dispatch_kernel<<<(unsigned)T_max, 128, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return check_launch("ep_dispatch_kernel");
}

extern "C" int b200_ep_combine(void* const* peer_out, const int32_t* topk_ids, void* out, int dtype, int64_t T,
                               int64_t T_max, int topk, int64_t H, int E, int n_ranks, int rank, void* stream) {
  using namespace b200;
  B200_CHECK_ARG(T >= 0 && T_max >= T && topk > 0 && H > 0 && E > 0, "ep_combine: bad shape");
  B200_CHECK_ARG(n_ranks >= 1 && n_ranks <= kEpMaxRanks && rank >= 0 && rank < n_ranks && E % n_ranks == 0,
                 "ep_combine: ranks=%d rank=%d E=%d", n_ranks, rank, E);
  if (T == 0) return B200_OK;
  B200_UNSUPPORTED(H % 8 != 0, "ep_combine: H=%lld must be a multiple of 8", (long long)H);
  B200_CHECK_ARG(peer_out && topk_ids && out && ((uintptr_t)out & 15) == 0, "ep_combine: null or unaligned pointer");
  B200_CHECK_ARG(dtype == B200_BF16 || dtype == B200_F16, "ep_combine: dtype code %d is not bf16/f16", dtype);
  EpCombineParams a = {};
  a.topk_ids = topk_ids; a.out = out; a.T = T; a.T_max = T_max; a.H = H; a.k = topk; a.E = E; a.p = n_ranks; a.rank = rank;
  a.status = device_status_word();
  if (!a.status) {
    set_error_detail("cannot resolve the device status word");
    return B200_E_LAUNCH;
  }
  for (int d = 0; d < n_ranks; ++d) {
    B200_CHECK_ARG(peer_out[d] && ((uintptr_t)peer_out[d] & 15) == 0, "ep_combine: output area %d null or unaligned", d);
    a.peer_out[d] = peer_out[d];
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == B200_BF16) ep_combine_kernel<__nv_bfloat16><<<(unsigned)T, 128, 0, st>>>(a);
  else ep_combine_kernel<__half><<<(unsigned)T, 128, 0, st>>>(a);
  return check_launch("ep_combine_kernel");
}

extern "C" int b200_peer_handshake(void* my_flags, void* const* peer_flags, int n_ranks, int rank, int phase,
                                   uint32_t epoch, void* stream) {
  using namespace b200;
  B200_CHECK_ARG(my_flags && peer_flags && n_ranks >= 1 && n_ranks <= kEpMaxRanks && rank >= 0 && rank < n_ranks &&
                     (phase == 0 || phase == 1),
                 "peer_handshake: bad arguments (ranks=%d rank=%d phase=%d)", n_ranks, rank, phase);
  HandshakeParams a = {};
  a.my_flags = static_cast<uint32_t*>(my_flags); a.p = n_ranks; a.rank = rank; a.phase = phase; a.epoch = epoch;
  a.wait_ns = peer_wait_ns();
  a.status = device_status_word();
  if (!a.status) {
    set_error_detail("cannot resolve the device status word");
    return B200_E_LAUNCH;
  }
  for (int d = 0; d < n_ranks; ++d) {
    B200_CHECK_ARG(peer_flags[d] != nullptr, "peer_handshake: flag pointer %d is null", d);
    a.peer_flags[d] = static_cast<uint32_t*>(peer_flags[d]);
  }
  peer_handshake_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return check_launch("peer_handshake_kernel");
}
