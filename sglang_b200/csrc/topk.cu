// Expert routing: scores -> (top-k weights fp32, top-k expert ids int32) for the fused MoE layer.
//
// One warp per token. Lane l owns the `vpl` consecutive experts [l*vpl, (l+1)*vpl) in registers
// (vpl = ceil(E/32) <= 32), so the row is read once and every step after the load is register
// and shuffle work:
//   scores   softmax over the row, or sigmoid per element (fp32)
//   choice   scores + correction bias (when given): what the selection compares
//   groups   (optional) experts form n_group equal groups; a group's score is the maximum, or
//            the sum of the two largest, of its choice values; only the topk_group best groups
//            stay eligible
//   top-k    k rounds of warp argmax over the eligible choice values, lower index first on ties;
//            the weight is the (unbiased) score of the chosen expert; results are in
//            descending order of choice
//   renorm   weights / their sum, optionally times a routed scaling factor
// Rows at or beyond *num_token_non_padded (when given) get id -1.
#include "common.cuh"

namespace b200 {

struct RouteParams {
  const void* logits;
  const float* bias;            // [E] or nullptr
  const int32_t* num_valid;     // device scalar or nullptr
  float* weights;               // [T, topk]
  int32_t* ids;                 // [T, topk]
  int64_t T;
  int E, vpl, topk;
  int sigmoid;                  // 0: softmax, 1: sigmoid
  int n_group, topk_group;      // n_group <= 1: no grouping
  int group_top2;               // group score: 1 = sum of the two largest, 0 = maximum
  int renormalize;
  float out_scale;              // multiplies the weights after renormalisation (1 = none)
  float softcap;                // != 0: logits become tanh(x / softcap) * softcap before scoring
  const float* logit_bias;      // [E] or nullptr: added to the (soft-capped) logits before scoring
};

constexpr float kNegInf = -__builtin_huge_valf();

// float -> uint32 whose unsigned order is the float order (-inf lowest)
__device__ __forceinline__ uint32_t ordered_key(float v) {
  const uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// (a, b) = two largest of {a, b, c, d}, a >= b, given a >= b and c >= d
__device__ __forceinline__ void merge_top2(float& a, float& b, float c, float d) {
  const float hi = fmaxf(a, c);
  const float lo = fmaxf(fminf(a, c), a >= c ? b : d);
  a = hi;
  b = lo;
}

template <typename T, int VMAX>
__global__ void __launch_bounds__(128) route_topk_kernel(const RouteParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t tok = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (tok >= p.T) return;
  const unsigned full = 0xffffffffu;
  const int vpl = p.vpl, E = p.E;
  const int e0 = lane * vpl;
  const T* row = static_cast<const T*>(p.logits) + tok * E;

  float s[VMAX], c[VMAX];
#pragma unroll
  for (int j = 0; j < VMAX; ++j) {
    const bool valid = j < vpl && e0 + j < E;
    s[j] = valid ? to_f32<T>(row[e0 + j]) : kNegInf;
  }
  if (p.softcap != 0.f || p.logit_bias != nullptr) {
#pragma unroll
    for (int j = 0; j < VMAX; ++j) {
      if (j < vpl && e0 + j < E) {
        float v = s[j];
        if (p.softcap != 0.f) v = tanhf(v / p.softcap) * p.softcap;
        if (p.logit_bias != nullptr) v += __ldg(p.logit_bias + e0 + j);
        s[j] = v;
      }
    }
  }
  if (p.sigmoid) {
#pragma unroll
    for (int j = 0; j < VMAX; ++j) s[j] = 1.0f / (1.0f + expf(-s[j]));  // slots past E: 1/(1+inf) = 0
  } else {
    float m = kNegInf;
#pragma unroll
    for (int j = 0; j < VMAX; ++j) m = fmaxf(m, s[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(full, m, o));
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < VMAX; ++j) {
      s[j] = expf(s[j] - m);  // exp(-inf) = 0 for the slots past E
      sum += s[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(full, sum, o);
#pragma unroll
    for (int j = 0; j < VMAX; ++j) s[j] = __fdiv_rn(s[j], sum);
  }
#pragma unroll
  for (int j = 0; j < VMAX; ++j) {
    const bool valid = j < vpl && e0 + j < E;
    c[j] = valid ? s[j] + (p.bias ? __ldg(p.bias + e0 + j) : 0.f) : kNegInf;
  }

  if (p.n_group > 1) {
    const int gs = E / p.n_group;  // experts per group
    const int lpg = gs / vpl;      // lanes per group when groups are whole lanes
    if (gs % vpl == 0 && (lpg & (lpg - 1)) == 0) {
      // groups are aligned power-of-two runs of lanes: all groups reduce at once
      float a = kNegInf, b = kNegInf;
#pragma unroll
      for (int j = 0; j < VMAX; ++j) merge_top2(a, b, c[j], kNegInf);
      for (int o = 1; o < lpg; o <<= 1) {
        const float oa = __shfl_xor_sync(full, a, o), ob = __shfl_xor_sync(full, b, o);
        merge_top2(a, b, oa, ob);
      }
      const float mine = p.group_top2 ? a + b : a;
      const int g = lane / lpg;
      int rank = 0;
      for (int o = 0; o < p.n_group; ++o) {
        const float other = __shfl_sync(full, mine, o * lpg);
        rank += (other > mine || (other == mine && o < g)) ? 1 : 0;
      }
      if (rank >= p.topk_group || g >= p.n_group) {
#pragma unroll
        for (int j = 0; j < VMAX; ++j) c[j] = kNegInf;
      }
    } else {
      // any other group size (n_group <= 32): one full-warp reduction per group, lane g keeps
      // the score of group g
      float mine = kNegInf;
      for (int g = 0; g < p.n_group; ++g) {
        float a = kNegInf, b = kNegInf;
#pragma unroll
        for (int j = 0; j < VMAX; ++j) merge_top2(a, b, (e0 + j) / gs == g ? c[j] : kNegInf, kNegInf);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float oa = __shfl_xor_sync(full, a, o), ob = __shfl_xor_sync(full, b, o);
          merge_top2(a, b, oa, ob);
        }
        if (lane == g) mine = p.group_top2 ? a + b : a;
      }
      int rank = 0;
      for (int o = 0; o < p.n_group; ++o) {
        const float other = __shfl_sync(full, mine, o);
        rank += (other > mine || (other == mine && o < lane)) ? 1 : 0;
      }
      const int keep = lane < p.n_group && rank < p.topk_group;
#pragma unroll
      for (int j = 0; j < VMAX; ++j) {
        const int g = min((e0 + j) / gs, 31);
        if (!__shfl_sync(full, keep, g)) c[j] = kNegInf;
      }
    }
  }

  float my_w = 0.f;
  int my_id = 0;
  for (int t = 0; t < p.topk; ++t) {
    float bv = kNegInf;
    int bi = E;  // no candidate
#pragma unroll
    for (int j = 0; j < VMAX; ++j) {
      if (j < vpl && e0 + j < E && (c[j] > bv || bi == E)) {
        bv = c[j];
        bi = e0 + j;
      }
    }
    // warp argmax in three instructions: redux.sync max over order-preserving integer keys, a
    // ballot of the lanes that hold the maximum, and the lowest such lane wins (lanes own
    // ascending expert ranges and each lane already kept its lowest index, so this is the
    // lowest expert index among equal values)
    const uint32_t key = ordered_key(bv);
    const uint32_t kmax = __reduce_max_sync(full, key);
    const int winner = __ffs(__ballot_sync(full, key == kmax)) - 1;
    bi = __shfl_sync(full, bi, winner);
    // the owner hands out the unbiased score and retires the expert
    const int owner = bi / vpl, slot = bi - owner * vpl;
    float wv = 0.f;
#pragma unroll
    for (int j = 0; j < VMAX; ++j) {
      if (lane == owner && j == slot) {
        wv = s[j];
        c[j] = kNegInf;
      }
    }
    wv = __shfl_sync(full, wv, owner & 31);
    if (lane == t) {
      my_w = wv;
      my_id = bi;
    }
  }
  if (p.renormalize) {
    float sum = lane < p.topk ? my_w : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(full, sum, o);
    my_w = __fdiv_rn(my_w, sum);
  }
  my_w *= p.out_scale;
  if (p.num_valid != nullptr && tok >= *p.num_valid) my_id = -1;
  if (lane < p.topk) {
    p.weights[tok * p.topk + lane] = my_w;
    p.ids[tok * p.topk + lane] = my_id;
  }
}

template <typename T>
static int launch_route(const RouteParams& p, cudaStream_t st) {
  const unsigned grid = (unsigned)cdiv(p.T, 4);
  if (p.vpl <= 1) route_topk_kernel<T, 1><<<grid, 128, 0, st>>>(p);
  else if (p.vpl <= 2) route_topk_kernel<T, 2><<<grid, 128, 0, st>>>(p);
  else if (p.vpl <= 4) route_topk_kernel<T, 4><<<grid, 128, 0, st>>>(p);
  else if (p.vpl <= 8) route_topk_kernel<T, 8><<<grid, 128, 0, st>>>(p);
  else if (p.vpl <= 16) route_topk_kernel<T, 16><<<grid, 128, 0, st>>>(p);
  else route_topk_kernel<T, 32><<<grid, 128, 0, st>>>(p);
  return check_launch("route_topk_kernel");
}

static int launch_route_dtype(const RouteParams& p, int logits_dtype, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (logits_dtype == B200_F32) return launch_route<float>(p, st);
  if (logits_dtype == B200_BF16) return launch_route<__nv_bfloat16>(p, st);
  if (logits_dtype == B200_F16) return launch_route<__half>(p, st);
  set_error_detail("route_topk: logits dtype code %d is not f32/bf16/f16", logits_dtype);
  return B200_E_UNSUPPORTED;
}

}  // namespace b200

extern "C" int b200_route_topk(const void* logits, int logits_dtype, const float* correction_bias, int64_t T, int E,
                               int topk, int scoring, int n_group, int topk_group, int group_score, int renormalize,
                               float output_scale, const int32_t* num_token_non_padded, float* topk_weights,
                               int32_t* topk_ids, void* stream) {
  using namespace b200;
  B200_CHECK_ARG(T >= 0 && E > 0 && topk > 0, "route_topk: bad shape T=%lld E=%d topk=%d", (long long)T, E, topk);
  if (T == 0) return B200_OK;
  B200_CHECK_ARG(logits && topk_weights && topk_ids, "route_topk: null pointer");
  B200_CHECK_ARG(scoring == B200_SCORE_SOFTMAX || scoring == B200_SCORE_SIGMOID, "route_topk: unknown scoring %d", scoring);
  B200_CHECK_ARG(topk <= E, "route_topk: topk=%d > E=%d", topk, E);
  B200_UNSUPPORTED(E > 1024 || topk > 32, "route_topk: E=%d > 1024 or topk=%d > 32", E, topk);
  if (n_group > 1) {
    B200_CHECK_ARG(E % n_group == 0 && topk_group >= 1 && topk_group <= n_group,
                   "route_topk: E=%d n_group=%d topk_group=%d", E, n_group, topk_group);
    B200_CHECK_ARG(group_score == B200_GROUP_MAX || group_score == B200_GROUP_TOP2_SUM, "route_topk: group_score %d",
                   group_score);
    B200_UNSUPPORTED(n_group > 32, "route_topk: more than 32 expert groups");
    B200_CHECK_ARG(topk <= topk_group * (E / n_group), "route_topk: topk=%d exceeds the experts of %d groups", topk,
                   topk_group);
  }
  RouteParams p = {};
  p.logits = logits; p.bias = correction_bias; p.num_valid = num_token_non_padded;
  p.weights = topk_weights; p.ids = topk_ids; p.T = T; p.E = E; p.vpl = (E + 31) / 32; p.topk = topk;
  p.sigmoid = scoring == B200_SCORE_SIGMOID; p.n_group = n_group; p.topk_group = topk_group;
  p.group_top2 = group_score == B200_GROUP_TOP2_SUM; p.renormalize = renormalize; p.out_scale = output_scale;
  return b200::launch_route_dtype(p, logits_dtype, stream);
}

extern "C" int b200_route_topk_softmax_capped(const void* logits, int logits_dtype, float softcap, const float* logit_bias,
                                              int64_t T, int E, int topk, int renormalize, float* topk_weights,
                                              int32_t* topk_ids, void* stream) {
  using namespace b200;
  B200_CHECK_ARG(T >= 0 && E > 0 && topk > 0, "route_topk: bad shape T=%lld E=%d topk=%d", (long long)T, E, topk);
  if (T == 0) return B200_OK;
  B200_CHECK_ARG(logits && topk_weights && topk_ids, "route_topk: null pointer");
  B200_CHECK_ARG(topk <= E, "route_topk: topk=%d > E=%d", topk, E);
  B200_CHECK_ARG(softcap >= 0.f, "route_topk: negative softcap");
  B200_UNSUPPORTED(E > 1024 || topk > 32, "route_topk: E=%d > 1024 or topk=%d > 32", E, topk);
  RouteParams p = {};
  p.logits = logits; p.weights = topk_weights; p.ids = topk_ids; p.T = T; p.E = E; p.vpl = (E + 31) / 32; p.topk = topk;
  p.renormalize = renormalize; p.out_scale = 1.0f; p.softcap = softcap; p.logit_bias = logit_bias;
  return launch_route_dtype(p, logits_dtype, stream);
}
