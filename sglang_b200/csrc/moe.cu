// fused_experts(use_fp8_w8a8=True, block_shape=[128,128]) for sm_100a.
//
// Launch sequence (all on the caller's stream, no host sync):
//   1 align            token->expert buckets padded to 128 rows                 (align.cu)
//   2 gather_quant     hidden rows -> expert-sorted FP8 rows + 1x128 scales     (HBM bound;
//                      top-k >= 3: rows quantised once per token, then FP8 rows gathered)
//   3 grouped GEMM 1   sorted rows x w1[expert]^T; the epilogue applies silu(gate)*up in fp32
//                      and re-quantises to FP8 + 1x128 scales from the accumulators (tcgen05)
//   4 grouped GEMM 2   x w2[expert]^T, * router weight, scattered to (token, slot)
//   5 sum_reduce       fp32 sum over the top-k slots -> out                     (HBM bound)
// Scales of the two intermediate activations are stored column-major ([K/128][rows]) so a
// GEMM promotion warp reads 32 consecutive floats per K block.
#include <stdlib.h>

#include "gemm_host.cuh"
#include "moe_decode.cuh"

namespace b200 {

constexpr int kMoeBlockM = 128;

// One thread = 16 consecutive elements of kGatherRows consecutive sorted rows (8 lanes share a
// 128-group). blockIdx.x = group of rows, blockIdx.y = 256-chunk segment of the row. The row
// indices and then the row data of all kGatherRows rows are requested before any is used, so
// the dependent index -> data round trips overlap instead of adding up per row.
constexpr int kGatherRows = 4;  // divides the 128-row expert blocks

template <typename T>
__global__ void __launch_bounds__(256) moe_gather_quant_kernel(
    const T* __restrict__ hidden, const int32_t* __restrict__ sorted_ids, const int32_t* __restrict__ expert_ids,
    const int32_t* __restrict__ num_post_pad, uint8_t* __restrict__ q, float* __restrict__ s, int chunks_per_row,
    int64_t H, int numel, int topk, int64_t cap, int zero_pads) {
  const int64_t slot0 = (int64_t)blockIdx.x * kGatherRows;
  if (slot0 >= *num_post_pad || expert_ids[slot0 / kMoeBlockM] < 0) return;  // uniform per block
  const int chunk = blockIdx.y * blockDim.x + threadIdx.x;
  const bool active = chunk < chunks_per_row;  // whole 8-lane groups are in or out (H % 128 == 0)
  int flat[kGatherRows];
#pragma unroll
  for (int r = 0; r < kGatherRows; ++r) flat[r] = __ldg(sorted_ids + slot0 + r);
  constexpr int kRegs = 16 * (int)sizeof(T) / 16;  // 16-byte registers per 16 elements
  uint4 raw[kGatherRows][kRegs];
#pragma unroll
  for (int r = 0; r < kGatherRows; ++r) {
    const bool real = active && flat[r] < numel;
    const T* src = hidden + (int64_t)(real ? flat[r] / topk : 0) * H + chunk * 16;
#pragma unroll
    for (int i = 0; i < kRegs; ++i) raw[r][i] = real ? ld_nc_16(src + i * (16 / (int)sizeof(T))) : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int r = 0; r < kGatherRows; ++r) {
    float f[16];
    const T* e = reinterpret_cast<const T*>(raw[r]);
#pragma unroll
    for (int i = 0; i < 16; ++i) f[i] = to_f32<T>(e[i]);
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
    amax = fmaxf(group_max<8>(amax), 1e-10f);
    // scale = amax / 448 and q = x / scale as the reference's quantiser computes them. The quotient
    // is formed as x * (1 / scale) plus one residual correction (rem = x - q * scale, exact in an
    // FMA): two FMAs per element instead of an IEEE division sequence. For 16-bit inputs the
    // FP8 bytes equal those of the division on every (x, amax) pair (the quantiser's tests
    // enumerate them all). A plain
    // reciprocal multiply is not enough for 16-bit inputs: when amax has a short mantissa many
    // quotients sit exactly on an FP8 tie and would be broken the other way.
    const float scale = __fdiv_rn(amax, 448.0f);
    const float inv = __fdiv_rn(1.0f, scale);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float q0 = f[i] * inv;
      f[i] = copysignf(fmaf(fmaf(-q0, scale, f[i]), inv, q0), f[i]);  // -0 stays -0, as with x / scale
    }
    uint4 out;
    out.x = pack4_e4m3(f[0], f[1], f[2], f[3]);
    out.y = pack4_e4m3(f[4], f[5], f[6], f[7]);
    out.z = pack4_e4m3(f[8], f[9], f[10], f[11]);
    out.w = pack4_e4m3(f[12], f[13], f[14], f[15]);
    // Pad rows: a GEMM output row depends on its own A row only and rows computed from pad slots
    // are never scattered, so their content is free. Zeros keep the tensor cores' power draw
    // down when tiles are mostly real rows; with a few tokens per expert (tiles that are mostly
    // padding, weight streaming bound) writing them would dominate this kernel, so they are skipped.
    if (active && (zero_pads || flat[r] < numel)) {
      *reinterpret_cast<uint4*>(q + (slot0 + r) * H + chunk * 16) = out;
      if ((threadIdx.x & 7) == 0) s[(int64_t)(chunk / 8) * cap + slot0 + r] = scale;
    }
  }
}

// Pre-quantised input (rows quantised once per token by the step before, or FP8 rows + 1x128
// scales delivered by the expert-parallel dispatch): plain gather of bytes and scales into the
// expert-sorted layout. One thread = 16 bytes of kGatherRows consecutive sorted rows; indices,
// then data, of all rows are requested before any is stored.
__global__ void __launch_bounds__(256) moe_gather_fp8_kernel(
    const uint8_t* __restrict__ hidden_q, const float* __restrict__ hidden_s, const int32_t* __restrict__ sorted_ids,
    const int32_t* __restrict__ expert_ids, const int32_t* __restrict__ num_post_pad, uint8_t* __restrict__ q,
    float* __restrict__ s, int chunks_per_row, int64_t H, int numel, int topk, int64_t cap, int zero_pads) {
  const int64_t slot0 = (int64_t)blockIdx.x * kGatherRows;
  if (slot0 >= *num_post_pad || expert_ids[slot0 / kMoeBlockM] < 0) return;  // uniform per block
  const int chunk = blockIdx.y * blockDim.x + threadIdx.x;
  if (chunk >= chunks_per_row) return;
  int flat[kGatherRows];
#pragma unroll
  for (int r = 0; r < kGatherRows; ++r) flat[r] = __ldg(sorted_ids + slot0 + r);
  uint4 v[kGatherRows];
  float sc[kGatherRows];
#pragma unroll
  for (int r = 0; r < kGatherRows; ++r) {
    const bool real = flat[r] < numel;
    const int64_t tok = real ? flat[r] / topk : 0;
    v[r] = real ? ld_nc_16(hidden_q + tok * H + chunk * 16) : make_uint4(0, 0, 0, 0);
    sc[r] = real && (chunk & 7) == 0 ? __ldg(hidden_s + tok * (H / 128) + chunk / 8) : 0.f;
  }
#pragma unroll
  for (int r = 0; r < kGatherRows; ++r) {
    if (!zero_pads && flat[r] >= numel) continue;  // see moe_gather_quant_kernel
    *reinterpret_cast<uint4*>(q + (slot0 + r) * H + chunk * 16) = v[r];
    if ((chunk & 7) == 0) s[(int64_t)(chunk / 8) * cap + slot0 + r] = sc[r];
  }
}

// out[t, :] = scale * sum_j y[t*topk + j, :] over the slots whose expert id is valid. One block per token: the
// valid slots are listed once in shared memory, so a row none of whose slots is valid (most rows of an
// expert-parallel receive area) costs one read of its ids, and there is no per-thread division. Four row loads
// are in flight per thread and six blocks fit an SM; the sum stays in slot order.
constexpr int kSumReduceMaxSlots = 64;
template <typename T>
__global__ void __launch_bounds__(256, 6) moe_sum_reduce_kernel(const T* __restrict__ y, const int32_t* __restrict__ topk_ids,
                                                                T* __restrict__ out, int topk, int E, int64_t H, float scale,
                                                                int skip_unrouted, const int* __restrict__ poison_status) {
  __shared__ int s_slot[kSumReduceMaxSlots];
  __shared__ int s_n;
  const int64_t t = blockIdx.x;
  if (poison_status != nullptr && *reinterpret_cast<const volatile int*>(poison_status) != 0) {
    // the rows were to be written by other GPUs and the handshake before this kernel gave up: NaNs, not stale rows
    const uint4 nan16 = make_uint4(0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu);  // NaN in bf16 and fp16
    for (int64_t c = threadIdx.x * 8; c < H; c += blockDim.x * 8) *reinterpret_cast<uint4*>(out + t * H + c) = nan16;
    return;
  }
  if (threadIdx.x < 32) {  // warp 0 compacts the valid slots, ascending (topk <= 64: two rounds of 32)
    int n = 0;
    for (int j0 = 0; j0 < topk; j0 += 32) {
      const int j = j0 + (int)threadIdx.x;
      const int e = j < topk ? __ldg(topk_ids + t * topk + j) : -1;
      const bool ok = e >= 0 && e < E;
      const unsigned m = __ballot_sync(0xffffffffu, ok);
      if (ok) s_slot[n + __popc(m & ((1u << threadIdx.x) - 1u))] = j;
      n += __popc(m);
    }
    if (threadIdx.x == 0) s_n = n;
  }
  __syncthreads();
  const int n = s_n;
  if (n == 0 && skip_unrouted) return;  // a row no local expert serves: nobody reads it
  const int vec_per_row = (int)(H / 8);
  const T* base = y + t * topk * H;
  for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int k0 = 0; k0 < n; k0 += 4) {
      uint4 r[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (k0 + k < n) r[k] = ld_nc_16(base + (int64_t)s_slot[k0 + k] * H + v * 8);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (k0 + k < n) {
          const T* h = reinterpret_cast<const T*>(&r[k]);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += to_f32<T>(h[i]);
        }
      }
    }
    uint4 o;
    T* oh = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int i = 0; i < 8; ++i) oh[i] = from_f32<T>(acc[i] * scale);
    *reinterpret_cast<uint4*>(out + t * H + v * 8) = o;
  }
}

// Same reduction over fp32 split-K partials y[splits][rows * slots][H] of the down GEMM
// (few-token case): out[r, :] = scale * sum over valid slots j and splits s. Rows whose slots
// are all invalid come out as zeros.
template <typename T>
__global__ void __launch_bounds__(256) moe_sum_reduce_splits_kernel(const float* __restrict__ y,
                                                                    const int32_t* __restrict__ topk_ids,
                                                                    T* __restrict__ out, int64_t rows, int slots,
                                                                    int splits, int64_t split_stride, int E, int64_t H,
                                                                    float scale, int skip_unrouted) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int vec_per_row = (int)(H / 8);
  if (c >= rows * vec_per_row) return;
  const int64_t r = c / vec_per_row;
  const int v = (int)(c - r * vec_per_row);
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  bool any = false;
  for (int j = 0; j < slots; ++j) {
    const int e = topk_ids[r * slots + j];
    if (e < 0 || e >= E) continue;
    any = true;
    for (int sp = 0; sp < splits; ++sp) {
      const float* src = y + sp * split_stride + (r * slots + j) * H + v * 8;
      const uint4 a = ld_nc_16(src), b = ld_nc_16(src + 4);
      acc[0] += __uint_as_float(a.x); acc[1] += __uint_as_float(a.y);
      acc[2] += __uint_as_float(a.z); acc[3] += __uint_as_float(a.w);
      acc[4] += __uint_as_float(b.x); acc[5] += __uint_as_float(b.y);
      acc[6] += __uint_as_float(b.z); acc[7] += __uint_as_float(b.w);
    }
  }
  if (!any && skip_unrouted) return;
  uint4 o;
  T* oh = reinterpret_cast<T*>(&o);
#pragma unroll
  for (int i = 0; i < 8; ++i) oh[i] = from_f32<T>(acc[i] * scale);
  *reinterpret_cast<uint4*>(out + r * H + v * 8) = o;
}

// Split-K factor of the down GEMM. With a handful of tokens the live tiles (about one 128-row
// tile per routed expert, H/256 column tiles each) leave most SMs without weights to stream;
// K = I is then split and the fp32 partials are summed by the slot reduction.
static int moe_down_k_splits(int64_t numel, int E, int64_t H, int64_t I, int sms) {
  const int64_t live = (numel < E ? numel : E) + numel / kMoeBlockM;
  const int64_t tiles = live * cdiv(H, 256);
  const int64_t num_kb = I / 128;
  if (tiles * 4 >= (int64_t)sms * 3 || num_kb < 8) return 1;
  int64_t s = sms / tiles;
  if (s > num_kb / 4) s = num_kb / 4;
  if (s > 8) s = 8;
  return s < 2 ? 1 : (int)s;
}

struct MoeWorkspace {
  int64_t cap;  // rows of the expert-sorted layout (multiple of 128)
  int64_t cap_blocks;
  int down_splits;  // > 1: the down GEMM writes fp32 split-K partials instead of 16-bit rows
  bool decode;      // few-token path: swapped-operand kernels, no align / gather pass
  int decode_nt;    // its token tile (16, 32 or 64)
  int decode_splits;  // K splits of its down stage
  size_t off_act;   // its fp32 activation rows [numel][I] between the two stages
  bool quant_first;  // quantise the T input rows once, then gather FP8 rows (instead of quantising every pair)
  size_t off_sorted, off_expert, off_npp, off_cumsum, off_align, off_aq1, off_as1, off_aq2, off_as2, off_c3, off_xq, off_xs, total;
};

// K splits of the few-token down stage: about two work items (routed expert x 128-row weight tile x split)
// per SM, at least as many as the scale table of one CTA requires.
static int moe_decode_down_splits(int64_t numel, int E, int64_t H, int64_t I, int sms) {
  const int64_t active = numel < E ? numel : E;
  const int64_t items = active * (H / 128);
  const int64_t num_kb = I / 128;
  int64_t s = (2 * (int64_t)sms) / (items > 0 ? items : 1);
  if (s > num_kb / 4) s = num_kb / 4;
  const int64_t need = cdiv(num_kb, 64);
  if (s < need) s = need;
  if (s < 1) s = 1;
  if (s > 16) s = 16 > need ? 16 : need;
  return (int)s;
}

static MoeWorkspace moe_workspace_layout(int64_t T, int topk, int E, int64_t H, int64_t I) {
  MoeWorkspace w = {};
  const int64_t numel = T * topk;
  int64_t max_pad = numel < E + 1 ? numel * kMoeBlockM : numel + (int64_t)(E + 1) * (kMoeBlockM - 1);
  w.cap = cdiv(max_pad, kMoeBlockM) * kMoeBlockM;
  w.cap_blocks = w.cap / kMoeBlockM;
  size_t o = 0;
  auto take = [&](size_t bytes) { size_t at = o; o = align_up(o + bytes, 256); return at; };
  w.off_sorted = take((size_t)w.cap * 4);
  w.off_expert = take((size_t)w.cap_blocks * 4);
  w.off_npp = take(4);
  w.off_cumsum = take((size_t)(E + 2) * 4);
  w.off_align = take(b200_moe_align_workspace_bytes(numel, E + 1));
  w.off_aq1 = take((size_t)w.cap * H);
  w.off_as1 = take((size_t)w.cap * (H / 128) * 4);
  w.off_aq2 = take((size_t)w.cap * I);
  w.off_as2 = take((size_t)w.cap * (I / 128) * 4);
  w.down_splits = moe_down_k_splits(numel, E, H, I, sm_count());
  w.off_c3 = take(w.down_splits > 1 ? (size_t)w.down_splits * numel * H * 4 : (size_t)numel * H * 2);
  // Each token's row is used by topk pairs: from three slots up, quantising it once and moving
  // FP8 bytes moves fewer bytes than re-reading the 16-bit row per pair.
  w.quant_first = topk >= 3;
  w.off_xq = take(w.quant_first ? (size_t)T * H : 0);
  w.off_xs = take(w.quant_first ? (size_t)T * (H / 128) * 4 : 0);
  // a handful of tokens: the swapped-operand path (its buffers are taken in addition, so that the
  // tuning knob can switch paths on the same workspace)
  w.decode = T <= 64 && numel <= kDecodeMaxIds && E <= kDecodeMaxExperts && H <= 64 * 128 && H % 128 == 0 && I % 128 == 0;
  w.decode_nt = T <= 16 ? 16 : (T <= 32 ? 32 : 64);
  w.decode_splits = w.decode ? moe_decode_down_splits(numel, E, H, I, 148) : 1;
  w.off_act = take(w.decode ? (size_t)numel * I * 4 : 0);
  if (w.decode) {
    const size_t need = (size_t)w.decode_splits * numel * H * 4;
    const size_t have = w.down_splits > 1 ? (size_t)w.down_splits * numel * H * 4 : (size_t)numel * H * 2;
    if (need > have) {  // the partials of the decode path share the c3 region: grow it
      w.off_c3 = take(need);
    }
  }
  w.total = o;
  return w;
}

// Few-token path (see moe_decode.cuh): gate_up -> fp32 activation rows -> down -> slot / split sum.
template <typename T>
static int run_fused_experts_decode(const void* hidden, const float* hidden_scale, const void* w1, const void* w2,
                                    const float* w1_scale, const float* w2_scale, const float* topk_weights,
                                    const int32_t* topk_ids, void* out, int64_t T_tokens, int topk, int E, int64_t H,
                                    int64_t I, int combine_mode, int weight_on_input, float routed_scale, uint8_t* ws,
                                    const MoeWorkspace& L, cudaStream_t st) {
  const int no_combine = combine_mode == B200_COMBINE_NONE;
  const int skip_unrouted = combine_mode == B200_COMBINE_SUM_SKIP_UNROUTED;
  const int64_t numel = T_tokens * topk;
  const int max_active = (int)(numel < E ? numel : E);
  MoeDecodeParams p = {};
  p.topk_ids = topk_ids; p.topk_weights = topk_weights; p.numel = (int)numel; p.topk = topk; p.E = E;
  p.act = reinterpret_cast<float*>(ws + L.off_act);
  p.partial = reinterpret_cast<float*>(ws + L.off_c3);
  p.status = device_status_word();
  if (!p.status) {
    set_error_detail("cannot resolve the device status word");
    return B200_E_LAUNCH;
  }
  // gate_up: K = H, 64 gate + 64 up rows per tile
  p.x = hidden_scale ? nullptr : hidden;
  p.x_q = hidden_scale ? static_cast<const uint8_t*>(hidden) : nullptr;
  p.x_s = hidden_scale;
  p.Bs = w1_scale; p.K = (int)H; p.num_kb = (int)(H / 128); p.n_out = (int)I; p.n_tiles = (int)(I / 64);
  p.k_splits = 1; p.kb_per_split = p.num_kb; p.weight_on_input = weight_on_input; p.apply_weight = 0;
  int rc;
#define B200_MOE_DECODE(STAGE, W, ROWS)                                                             \
  (L.decode_nt == 16   ? launch_moe_decode<16, STAGE, T>(W, ROWS, p, max_active, st)                \
   : L.decode_nt == 32 ? launch_moe_decode<32, STAGE, T>(W, ROWS, p, max_active, st)                \
                       : launch_moe_decode<64, STAGE, T>(W, ROWS, p, max_active, st))
  if ((rc = B200_MOE_DECODE(1, w1, (int64_t)E * 2 * I))) return rc;
  // down: K = I, 128 rows of w2 per tile, K split
  p.x = nullptr; p.x_q = nullptr; p.x_s = nullptr;
  p.Bs = w2_scale; p.K = (int)I; p.num_kb = (int)(I / 128); p.n_out = (int)H; p.n_tiles = (int)(H / 128);
  p.kb_per_split = (int)cdiv(p.num_kb, L.decode_splits);
  p.k_splits = (int)cdiv(p.num_kb, p.kb_per_split);
  p.weight_on_input = 0; p.apply_weight = weight_on_input ? 0 : 1;
  if ((rc = B200_MOE_DECODE(2, w2, (int64_t)E * H))) return rc;
#undef B200_MOE_DECODE
  const int64_t rows = no_combine ? numel : T_tokens;
  const int64_t total = rows * (H / 8);
  moe_sum_reduce_splits_kernel<T><<<(unsigned)cdiv(total, 256), 256, 0, st>>>(
      p.partial, topk_ids, static_cast<T*>(out), rows, no_combine ? 1 : topk, p.k_splits, numel * H, E, H,
      no_combine ? 1.0f : routed_scale, skip_unrouted);
  return check_launch("moe_sum_reduce_splits");
}

// Destinations of the (token, slot) rows when they leave for several buffers (expert-parallel combine by push).
struct ScatterDests {
  void* dest[8];
  int n;
  int64_t rows_per_dest;
};

template <typename T>
static int run_fused_experts(const void* hidden, const float* hidden_scale, const void* w1, const void* w2, const float* w1_scale,
                             const float* w2_scale, const float* topk_weights, const int32_t* topk_ids, void* out,
                             int64_t T_tokens, int topk, int E, int64_t H, int64_t I, int combine_mode,
                             int weight_on_input, float routed_scale, uint8_t* ws, cudaStream_t st,
                             const ScatterDests* scatter = nullptr) {
  if (scatter != nullptr) combine_mode = B200_COMBINE_NONE;  // rows leave per (token, slot); the receiver sums
  const int no_combine = combine_mode == B200_COMBINE_NONE;
  const int skip_unrouted = combine_mode == B200_COMBINE_SUM_SKIP_UNROUTED;
  const MoeWorkspace L = moe_workspace_layout(T_tokens, topk, E, H, I);
  const int64_t numel = T_tokens * topk;
  int32_t* sorted = reinterpret_cast<int32_t*>(ws + L.off_sorted);
  int32_t* expert_ids = reinterpret_cast<int32_t*>(ws + L.off_expert);
  int32_t* npp = reinterpret_cast<int32_t*>(ws + L.off_npp);
  int32_t* cumsum = reinterpret_cast<int32_t*>(ws + L.off_cumsum);
  uint8_t* aq1 = ws + L.off_aq1;
  float* as1 = reinterpret_cast<float*>(ws + L.off_as1);
  uint8_t* aq2 = ws + L.off_aq2;
  float* as2 = reinterpret_cast<float*>(ws + L.off_as2);
  // Opt-in (knob moe_decode = 1): measured slower than the tile path below at every token count tried (the
  // in-kernel row fetches sit behind the saturated weight stream in L2 and pace the pipeline, and more work
  // items than resident CTAs run in waves), so the tile path stays the default.
  if (L.decode && tuning().moe_decode == 1 && scatter == nullptr)
    return run_fused_experts_decode<T>(hidden, hidden_scale, w1, w2, w1_scale, w2_scale, topk_weights, topk_ids, out, T_tokens,
                                       topk, E, H, I, combine_mode, weight_on_input, routed_scale, ws, L, st);
  int down_splits = L.down_splits;
  if (tuning().moe_down_splitk == 0) down_splits = 1;  // knob: keep the 16-bit single-pass path
  if (scatter != nullptr) down_splits = 1;             // rows go straight to their receivers in 16 bits
  const bool split = down_splits > 1;
  T* c3 = no_combine && !split ? static_cast<T*>(out) : reinterpret_cast<T*>(ws + L.off_c3);

  int rc = b200_moe_align_block_size(topk_ids, B200_I32, numel, E + 1, kMoeBlockM, sorted, L.cap, expert_ids,
                                     L.cap_blocks, npp, cumsum, 1, ws + L.off_align,
                                     b200_moe_align_workspace_bytes(numel, E + 1), st);
  if (rc) return rc;
  if (no_combine && !split && scatter == nullptr) {
    // rows of slots whose expert is not on this rank are never written by GEMM 2
    cudaError_t e = cudaMemsetAsync(out, 0, (size_t)numel * H * sizeof(T), st);
    if (e != cudaSuccess) {
      set_error_detail("memset(out): %s", cudaGetErrorString(e));
      return B200_E_LAUNCH;
    }
  }
  {
    const uint8_t* hq = static_cast<const uint8_t*>(hidden);
    const float* hs = hidden_scale;
    if (hs == nullptr && L.quant_first) {
      uint8_t* xq = ws + L.off_xq;
      float* xs = reinterpret_cast<float*>(ws + L.off_xs);
      rc = b200_per_token_group_quant_fp8(hidden, std::is_same<T, __half>::value ? B200_F16 : B200_BF16, xq, xs, T_tokens,
                                          H, 128, H / 128, 1, 1e-10f, B200_QUANT_DIV_CORRECTED, st);  // 16-bit input: same bits as the division
      if (rc) return rc;
      hq = xq;
      hs = xs;
    }
    const int cpr = (int)(H / 16);
    const int threads = cpr < 256 ? (cpr + 31) / 32 * 32 : 256;  // whole warps; cpr is a multiple of 8
    dim3 grid((unsigned)(L.cap / kGatherRows), (unsigned)cdiv(cpr, threads));
    int zero_pads = numel >= (int64_t)E * 32;  // on average a quarter of a tile per expert or more
    if (tuning().moe_zero_pads >= 0) zero_pads = (int)tuning().moe_zero_pads;
    if (hs != nullptr)
      moe_gather_fp8_kernel<<<grid, threads, 0, st>>>(hq, hs, sorted, expert_ids, npp, aq1, as1, cpr, H, (int)numel, topk,
                                                     L.cap, zero_pads);
    else
      moe_gather_quant_kernel<T><<<grid, threads, 0, st>>>(static_cast<const T*>(hidden), sorted, expert_ids, npp, aq1,
                                                          as1, cpr, H, (int)numel, topk, L.cap, zero_pads);
    if ((rc = check_launch("moe_gather"))) return rc;
  }
  const int force_bn = tuning().gemm_bn == 128 || tuning().gemm_bn == 256 ? (int)tuning().gemm_bn : 0;
  // expected live row tiles: every pair once, plus up to one partial tile per expert
  const int64_t tiles_hint = cdiv(numel, kMoeBlockM) + (numel < E ? numel : E) / 2;
  GemmParams p = {};
  p.expert_ids = expert_ids; p.num_post_pad = npp; p.sorted_ids = sorted; p.numel = (int)numel;
  p.M = (int)L.cap;
  // GEMM 1: [cap, H] x w1[E, 2I, H]^T -> silu(gate)*up -> FP8 [cap, I] + column-major scales
  p.As = as1; p.as_sm = 1; p.as_sk = L.cap; p.Bs = w1_scale; p.C = nullptr; p.ldc = 0;
  p.N = (int)I; p.K = (int)H; p.topk_weights = weight_on_input ? topk_weights : nullptr;
  p.q_out = aq2; p.q_scales = as2; p.q_scale_ld = L.cap;
  if ((rc = launch_gemm<GEMM_GROUPED_SILU_QUANT, T>(aq1, w1, (int64_t)E * 2 * I, p, 256, st, tiles_hint))) return rc;
  // GEMM 2: [cap, I] x w2[E, H, I]^T -> rows scattered to (token, slot), times the router weight
  p.As = as2; p.as_sk = L.cap; p.Bs = w2_scale; p.C = c3; p.ldc = H; p.N = (int)H; p.K = (int)I;
  p.topk_weights = weight_on_input ? nullptr : topk_weights;
  if (scatter != nullptr) {
    p.C = nullptr;
    p.scatter_rows_per_dest = (int)scatter->rows_per_dest;
    p.scatter_div = make_fastdiv((int)scatter->rows_per_dest);
    for (int d = 0; d < scatter->n; ++d) p.dest[d] = scatter->dest[d];
  }
  if (split) {
    p.split_stride = numel * H;
    if ((rc = launch_gemm<GEMM_GROUPED_SCATTER, float>(aq2, w2, (int64_t)E * H, p, 256, st, tiles_hint, down_splits)))
      return rc;
    const int64_t rows = no_combine ? numel : T_tokens;
    const int64_t total = rows * (H / 8);
    moe_sum_reduce_splits_kernel<T><<<(unsigned)cdiv(total, 256), 256, 0, st>>>(
        reinterpret_cast<const float*>(c3), topk_ids, static_cast<T*>(out), rows, no_combine ? 1 : topk, down_splits,
        numel * H, E, H, no_combine ? 1.0f : routed_scale, skip_unrouted);
    return check_launch("moe_sum_reduce_splits");
  }
  if ((rc = launch_gemm<GEMM_GROUPED_SCATTER, T>(aq2, w2, (int64_t)E * H, p, force_bn, st, tiles_hint))) return rc;
  if (!no_combine) {
    moe_sum_reduce_kernel<T><<<(unsigned)T_tokens, 256, 0, st>>>(c3, topk_ids, static_cast<T*>(out), topk, E, H,
                                                                  routed_scale, skip_unrouted, nullptr);
    if ((rc = check_launch("moe_sum_reduce"))) return rc;
  }
  return B200_OK;
}

// ---------------------------------------------------------------- masked (low-latency) layout
// Tokens arrive already grouped by expert: hidden [E][T_pad][H] with the first masked_m[e] rows of
// expert e valid (what a low-latency expert-parallel dispatch delivers). The grouped GEMMs above
// run unchanged on that layout: row tile mt belongs to expert mt / (T_pad/128) and is skipped
// when it starts at or beyond masked_m[e]; rows past masked_m[e] inside a live tile are computed
// and dropped by the store predicate (their "destination" is the out-of-range index).
__global__ void __launch_bounds__(256) masked_meta_kernel(const int32_t* __restrict__ masked_m, int32_t* __restrict__ sorted,
                                                          int32_t* __restrict__ expert_ids, int32_t* __restrict__ npp,
                                                          int E, int64_t T_pad) {
  const int64_t cap = (int64_t)E * T_pad;
  const int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (row == 0) *npp = (int32_t)cap;
  if (row >= cap) return;
  const int e = (int)(row / T_pad);
  const int64_t r = row - (int64_t)e * T_pad;
  const int m = min(max(masked_m[e], 0), (int)T_pad);
  sorted[row] = r < m ? (int32_t)row : (int32_t)cap;
  if (r % kMoeBlockM == 0) expert_ids[row / kMoeBlockM] = r < m ? e : -1;
}

struct MaskedWorkspace {
  int64_t cap;
  size_t off_sorted, off_expert, off_npp, off_aq2, off_as2, total;
};

static MaskedWorkspace masked_workspace_layout(int E, int64_t T_pad, int64_t I) {
  MaskedWorkspace w = {};
  w.cap = (int64_t)E * T_pad;
  size_t o = 0;
  auto take = [&](size_t bytes) { size_t at = o; o = align_up(o + bytes, 256); return at; };
  w.off_sorted = take((size_t)w.cap * 4);
  w.off_expert = take((size_t)(w.cap / kMoeBlockM) * 4);
  w.off_npp = take(4);
  w.off_aq2 = take((size_t)w.cap * I);
  w.off_as2 = take((size_t)w.cap * (I / 128) * 4);
  w.total = o;
  return w;
}

template <typename T>
static int run_masked_experts(const void* hidden_q, const float* hidden_s, const void* w1, const void* w2,
                              const float* w1_scale, const float* w2_scale, const int32_t* masked_m, void* out, int E,
                              int64_t T_pad, int64_t H, int64_t I, uint8_t* ws, cudaStream_t st) {
  const MaskedWorkspace L = masked_workspace_layout(E, T_pad, I);
  int32_t* sorted = reinterpret_cast<int32_t*>(ws + L.off_sorted);
  int32_t* expert_ids = reinterpret_cast<int32_t*>(ws + L.off_expert);
  int32_t* npp = reinterpret_cast<int32_t*>(ws + L.off_npp);
  uint8_t* aq2 = ws + L.off_aq2;
  float* as2 = reinterpret_cast<float*>(ws + L.off_as2);
  masked_meta_kernel<<<(unsigned)cdiv(L.cap, 256), 256, 0, st>>>(masked_m, sorted, expert_ids, npp, E, T_pad);
  int rc = check_launch("masked_meta_kernel");
  if (rc) return rc;
  GemmParams p = {};
  p.expert_ids = expert_ids; p.num_post_pad = npp; p.sorted_ids = sorted; p.numel = (int)L.cap;
  p.M = (int)L.cap;
  // gate_up: row-major input scales [cap][H/128]
  p.As = hidden_s; p.as_sm = H / 128; p.as_sk = 1; p.Bs = w1_scale; p.N = (int)I; p.K = (int)H;
  p.q_out = aq2; p.q_scales = as2; p.q_scale_ld = L.cap;
  if ((rc = launch_gemm<GEMM_GROUPED_SILU_QUANT, T>(hidden_q, w1, (int64_t)E * 2 * I, p, 256, st, 0))) return rc;
  // down: rows stay where they are (identity "scatter"), no router weight
  p.As = as2; p.as_sm = 1; p.as_sk = L.cap; p.Bs = w2_scale; p.C = out; p.ldc = H; p.N = (int)H; p.K = (int)I;
  return launch_gemm<GEMM_GROUPED_SCATTER, T>(aq2, w2, (int64_t)E * H, p, 0, st, 0);
}

}  // namespace b200

extern "C" size_t b200_masked_experts_fp8_workspace_bytes(int E, int64_t T_pad, int64_t H, int64_t I) {
  if (E <= 0 || T_pad <= 0 || H <= 0 || I <= 0) return 0;
  return b200::masked_workspace_layout(E, T_pad, I).total;
}

extern "C" int b200_masked_experts_fp8(const void* hidden_q, const float* hidden_s, const void* w1, const void* w2,
                                       const float* w1_scale, const float* w2_scale, const int32_t* masked_m, void* out,
                                       int out_dtype, int E, int64_t T_pad, int64_t H, int64_t I, void* workspace,
                                       size_t workspace_bytes, void* stream) {
  using namespace b200;
  B200_CHECK_ARG(E > 0 && T_pad > 0 && H > 0 && I > 0, "masked_experts: bad shape");
  B200_CHECK_ARG(hidden_q && hidden_s && w1 && w2 && w1_scale && w2_scale && masked_m && out, "masked_experts: null pointer");
  B200_UNSUPPORTED(T_pad % 128 != 0, "masked_experts: T_pad=%lld must be a multiple of 128", (long long)T_pad);
  B200_UNSUPPORTED(H % 128 != 0 || I % 128 != 0, "masked_experts: H=%lld and I=%lld must be multiples of 128",
                   (long long)H, (long long)I);
  B200_UNSUPPORTED((int64_t)E * T_pad >= (1LL << 30), "masked_experts: too many rows");
  B200_CHECK_ARG(((uintptr_t)hidden_q & 15) == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)w1 & 15) == 0 &&
                     ((uintptr_t)w2 & 15) == 0, "masked_experts: tensors must be 16-byte aligned");
  const size_t need = b200_masked_experts_fp8_workspace_bytes(E, T_pad, H, I);
  if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255) != 0) {
    set_error_detail("masked_experts: workspace %zu < %zu bytes or not 256-byte aligned", workspace_bytes, need);
    return B200_E_WORKSPACE;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  if (out_dtype == B200_BF16)
    return run_masked_experts<__nv_bfloat16>(hidden_q, hidden_s, w1, w2, w1_scale, w2_scale, masked_m, out, E, T_pad, H, I, ws, st);
  if (out_dtype == B200_F16)
    return run_masked_experts<__half>(hidden_q, hidden_s, w1, w2, w1_scale, w2_scale, masked_m, out, E, T_pad, H, I, ws, st);
  set_error_detail("masked_experts: output dtype code %d is not bf16/f16", out_dtype);
  return B200_E_UNSUPPORTED;
}

extern "C" size_t b200_fused_experts_fp8_workspace_bytes(int64_t T, int topk, int E, int64_t H, int64_t I) {
  if (T <= 0 || topk <= 0 || E <= 0 || H <= 0 || I <= 0) return 0;
  return b200::moe_workspace_layout(T, topk, E, H, I).total;
}

extern "C" int b200_fused_experts_fp8(const void* hidden, const float* hidden_scale, int h_dtype, const void* w1,
                                      const void* w2,
                                      const float* w1_scale, const float* w2_scale, const float* topk_weights,
                                      const int32_t* topk_ids, void* out, int64_t T, int topk, int E, int64_t H,
                                      int64_t I, int no_combine, int apply_router_weight_on_input,
                                      float routed_scaling_factor, void* workspace, size_t workspace_bytes,
                                      void* stream) {
  using namespace b200;
  B200_CHECK_ARG(T >= 0 && topk > 0 && E > 0 && H > 0 && I > 0, "fused_experts: bad shape");
  if (T == 0) return B200_OK;
  B200_CHECK_ARG(hidden && w1 && w2 && w1_scale && w2_scale && topk_weights && topk_ids && out,
                 "fused_experts: null pointer");
  B200_UNSUPPORTED(H % 128 != 0 || I % 128 != 0, "fused_experts: H=%lld and I=%lld must be multiples of 128",
                   (long long)H, (long long)I);
  B200_UNSUPPORTED(E + 1 > 1025, "fused_experts: more than 1024 experts");
  B200_UNSUPPORTED(T * topk >= (1LL << 30), "fused_experts: too many (token, slot) pairs");
  B200_UNSUPPORTED(topk > kSumReduceMaxSlots, "fused_experts: more than %d experts per token", kSumReduceMaxSlots);
  B200_CHECK_ARG(!apply_router_weight_on_input || topk == 1, "apply_router_weight_on_input needs topk == 1");
  B200_CHECK_ARG(no_combine >= 0 && no_combine <= 2, "fused_experts: unknown combine mode %d", no_combine);
  B200_CHECK_ARG(((uintptr_t)hidden & 15) == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)w1 & 15) == 0 &&
                     ((uintptr_t)w2 & 15) == 0, "fused_experts: tensors must be 16-byte aligned");
  const size_t need = b200_fused_experts_fp8_workspace_bytes(T, topk, E, H, I);
  if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255) != 0) {
    set_error_detail("fused_experts: workspace %zu < %zu bytes or not 256-byte aligned", workspace_bytes, need);
    return B200_E_WORKSPACE;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  if (h_dtype == B200_BF16)
    return run_fused_experts<__nv_bfloat16>(hidden, hidden_scale, w1, w2, w1_scale, w2_scale, topk_weights, topk_ids, out, T, topk, E,
                                            H, I, no_combine, apply_router_weight_on_input, routed_scaling_factor, ws, st);
  if (h_dtype == B200_F16)
    return run_fused_experts<__half>(hidden, hidden_scale, w1, w2, w1_scale, w2_scale, topk_weights, topk_ids, out, T, topk, E, H, I,
                                     no_combine, apply_router_weight_on_input, routed_scaling_factor, ws, st);
  set_error_detail("fused_experts: hidden dtype code %d is not bf16/f16", h_dtype);
  return B200_E_UNSUPPORTED;
}

extern "C" int b200_fused_experts_fp8_scatter(const void* hidden_q, const float* hidden_scale, int out_dtype, const void* w1,
                                              const void* w2, const float* w1_scale, const float* w2_scale,
                                              const float* topk_weights, const int32_t* topk_ids, void* const* dests,
                                              int n_dest, int64_t rows_per_dest, int64_t T, int topk, int E, int64_t H,
                                              int64_t I, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace b200;
  B200_CHECK_ARG(T >= 0 && topk > 0 && E > 0 && H > 0 && I > 0, "fused_experts_scatter: bad shape");
  if (T == 0) return B200_OK;
  B200_CHECK_ARG(hidden_q && hidden_scale && w1 && w2 && w1_scale && w2_scale && topk_weights && topk_ids && dests,
                 "fused_experts_scatter: null pointer (rows arrive quantised: FP8 bytes + scales)");
  B200_CHECK_ARG(n_dest >= 1 && n_dest <= 8 && rows_per_dest > 0 && rows_per_dest < (1LL << 30) &&
                     (int64_t)n_dest * rows_per_dest >= T * topk,
                 "fused_experts_scatter: %d destinations x %lld rows do not cover %lld pairs", n_dest,
                 (long long)rows_per_dest, (long long)(T * topk));
  B200_UNSUPPORTED(H % 128 != 0 || I % 128 != 0, "fused_experts_scatter: H=%lld and I=%lld must be multiples of 128",
                   (long long)H, (long long)I);
  B200_UNSUPPORTED(E + 1 > 1025, "fused_experts_scatter: more than 1024 experts");
  B200_UNSUPPORTED(T * topk >= (1LL << 30), "fused_experts_scatter: too many (token, slot) pairs");
  ScatterDests sd = {};
  sd.n = n_dest;
  sd.rows_per_dest = rows_per_dest;
  for (int d = 0; d < n_dest; ++d) {
    B200_CHECK_ARG(dests[d] && ((uintptr_t)dests[d] & 15) == 0, "fused_experts_scatter: destination %d null or unaligned", d);
    sd.dest[d] = dests[d];
  }
  B200_CHECK_ARG(((uintptr_t)hidden_q & 15) == 0 && ((uintptr_t)w1 & 15) == 0 && ((uintptr_t)w2 & 15) == 0,
                 "fused_experts_scatter: tensors must be 16-byte aligned");
  const size_t need = b200_fused_experts_fp8_workspace_bytes(T, topk, E, H, I);
  if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255) != 0) {
    set_error_detail("fused_experts_scatter: workspace %zu < %zu bytes or not 256-byte aligned", workspace_bytes, need);
    return B200_E_WORKSPACE;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  if (out_dtype == B200_BF16)
    return run_fused_experts<__nv_bfloat16>(hidden_q, hidden_scale, w1, w2, w1_scale, w2_scale, topk_weights, topk_ids, nullptr, T,
                                            topk, E, H, I, B200_COMBINE_NONE, 0, 1.0f, ws, st, &sd);
  if (out_dtype == B200_F16)
    return run_fused_experts<__half>(hidden_q, hidden_scale, w1, w2, w1_scale, w2_scale, topk_weights, topk_ids, nullptr, T, topk,
                                     E, H, I, B200_COMBINE_NONE, 0, 1.0f, ws, st, &sd);
  set_error_detail("fused_experts_scatter: output dtype code %d is not bf16/f16", out_dtype);
  return B200_E_UNSUPPORTED;
}

extern "C" int b200_moe_sum_reduce(const void* rows, const int32_t* topk_ids, void* out, int dtype, int64_t T, int topk, int E,
                                   int64_t H, float scale, int skip_unrouted, int poison_on_status, void* stream) {
  using namespace b200;
  B200_CHECK_ARG(T >= 0 && topk > 0 && E > 0 && H > 0 && H % 8 == 0, "moe_sum_reduce: bad shape");
  if (T == 0) return B200_OK;
  B200_CHECK_ARG(rows && topk_ids && out && ((uintptr_t)rows & 15) == 0 && ((uintptr_t)out & 15) == 0,
                 "moe_sum_reduce: null or unaligned pointer");
  B200_UNSUPPORTED(topk > kSumReduceMaxSlots, "moe_sum_reduce: more than %d experts per token", kSumReduceMaxSlots);
  B200_UNSUPPORTED(T >= (1LL << 31), "moe_sum_reduce: too many tokens");
  const int* status = poison_on_status ? device_status_word() : nullptr;
  if (poison_on_status && !status) {
    set_error_detail("cannot resolve the device status word");
    return B200_E_LAUNCH;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == B200_BF16)
    moe_sum_reduce_kernel<__nv_bfloat16><<<(unsigned)T, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(rows), topk_ids,
                                                                       static_cast<__nv_bfloat16*>(out), topk, E, H, scale,
                                                                       skip_unrouted, status);
  else if (dtype == B200_F16)
    moe_sum_reduce_kernel<__half><<<(unsigned)T, 256, 0, st>>>(static_cast<const __half*>(rows), topk_ids,
                                                                static_cast<__half*>(out), topk, E, H, scale, skip_unrouted, status);
  else {
    set_error_detail("moe_sum_reduce: dtype code %d is not bf16/f16", dtype);
    return B200_E_UNSUPPORTED;
  }
  return check_launch("moe_sum_reduce");
}
