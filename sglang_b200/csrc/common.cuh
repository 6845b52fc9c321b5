// Shared helpers for the sm_100a block-FP8 kernels: status codes, error detail,
// the per-device status word and small device utilities.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include "../../include/b200_blockfp8.h"

namespace b200 {

// Thread-local text describing the last failed call (read by b200_last_error_detail).
void set_error_detail(const char* fmt, ...);

// Address of this device's status word (a __device__ int in status.cu); nullptr on failure.
int* device_status_word();

#define B200_CHECK_ARG(cond, ...)                 \
  do {                                            \
    if (!(cond)) {                                \
      ::b200::set_error_detail(__VA_ARGS__);      \
      return B200_E_BAD_ARG;                      \
    }                                             \
  } while (0)

#define B200_UNSUPPORTED(cond, ...)               \
  do {                                            \
    if (cond) {                                   \
      ::b200::set_error_detail(__VA_ARGS__);      \
      return B200_E_UNSUPPORTED;                  \
    }                                             \
  } while (0)

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error_detail("%s: %s", what, cudaGetErrorString(e));
    return B200_E_LAUNCH;
  }
  return B200_OK;
}

// Process-wide knobs set through b200_set_tuning (tests force a kernel path, tuning sweeps try a
// setting); -1 = decide automatically. Product calls read this struct, never the environment.
struct Tuning {
  long gemm_bn = -1;            // 128 / 256: tile width of the dense GEMM
  long gemm_skinny = -1;        // 0: never use the decode (swapped-operand) kernel
  long gemm_skinny_max_m = -1;  // rows up to which the decode kernel is used
  long gemm_splitk = -1;        // > 0: forced K split
  long gemm_2cta = -1;          // 0: never, 1: CTA-pair kernel whenever legal
  long gemm_ue8m0 = -1;          // 0: packed power-of-two scales never take the block-scaled MMA kernel
  long linear_decode_fused = -1; // 0: callers keep quantiser + GEMM as separate launches at decode sizes
  long moe_decode = -1;         // 1: fused_experts takes the few-token (swapped-operand) path for T <= 64
  long moe_down_splitk = -1;    // 0: the down GEMM never splits K
  long moe_zero_pads = -1;      // 0 / 1: whether the gather pass zeroes pad rows
  long peer_wait_ms = -1;       // limit of a device-side wait for another GPU
};
Tuning& tuning();

// Limit of a device-side wait for another GPU (handshakes of the peer-memory collectives), in
// nanoseconds: 2 s unless the peer_wait_ms knob says otherwise (clamped to 100 ms .. 60 s). Ranks
// that can drift further apart than this on the host must synchronise on the host first.
inline unsigned long long peer_wait_ns() {
  long ms = tuning().peer_wait_ms > 0 ? tuning().peer_wait_ms : 2000;
  if (ms < 100) ms = 100;
  if (ms > 60000) ms = 60000;
  return (unsigned long long)ms * 1000000ull;
}

inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// ---------------------------------------------------------------- device utilities
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// 16-byte read-only global load (bypasses L1 allocation: streamed once).
__device__ __forceinline__ uint4 ld_nc_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Four consecutive floats from shared memory, read at this point of the program (never cached in
// registers across a barrier wait): for tables another warp fills while this one waits on an mbarrier.
__device__ __forceinline__ float4 ld_shared_f4(const float* p) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(p)))
               : "memory");
  return v;
}

// Four floats -> four E4M3 bytes (round-to-nearest-even, saturate to +-448), packed little-endian.
__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
  __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return (uint32_t)lo | ((uint32_t)hi << 16);
}

// Unpack 16 elements of type T held in 16-byte registers into fp32.
template <typename T>
struct Vec16;
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int kLoads = 2;  // 16-byte loads per 16 elements
  __device__ static void load(const __nv_bfloat16* p, float (&f)[16]) {
    uint4 r[2] = {ld_nc_16(p), ld_nc_16(p + 8)};
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(r);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float2 t = __bfloat1622float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
};
template <>
struct Vec16<__half> {
  __device__ static void load(const __half* p, float (&f)[16]) {
    uint4 r[2] = {ld_nc_16(p), ld_nc_16(p + 8)};
    const __half2* h = reinterpret_cast<const __half2*>(r);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float2 t = __half22float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
};
template <>
struct Vec16<float> {
  __device__ static void load(const float* p, float (&f)[16]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 r = ld_nc_16(p + 4 * i);
      f[4 * i] = __uint_as_float(r.x);
      f[4 * i + 1] = __uint_as_float(r.y);
      f[4 * i + 2] = __uint_as_float(r.z);
      f[4 * i + 3] = __uint_as_float(r.w);
    }
  }
};

// Quantise 16 fp32 values that share `amax` (already reduced over the group and floored at
// eps) into 16 E4M3 bytes; returns the stored scale. `formula` as in the C ABI.
__device__ __forceinline__ float quant16(const float (&f)[16], float amax, int formula, uint4& out) {
  float s, q[16];
  if (formula == B200_QUANT_V2) {
    s = amax * (1.0f / 448.0f);
    float r = __fdiv_rn(448.0f, amax);
#pragma unroll
    for (int i = 0; i < 16; ++i) q[i] = f[i] * r;
  } else if (formula == B200_QUANT_RECIP) {
    s = __fdiv_rn(amax, 448.0f);
    float r = __fdiv_rn(1.0f, s);
#pragma unroll
    for (int i = 0; i < 16; ++i) q[i] = f[i] * r;
  } else if (formula == B200_QUANT_DIV_CORRECTED) {
    s = __fdiv_rn(amax, 448.0f);
    const float r = __frcp_rn(s);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float q0 = f[i] * r;
      // one residual step towards the rounded quotient; a zero result takes the sign of x as x / s does
      q[i] = copysignf(fmaf(fmaf(-q0, s, f[i]), r, q0), f[i]);
    }
  } else {
    s = __fdiv_rn(amax, 448.0f);
#pragma unroll
    for (int i = 0; i < 16; ++i) q[i] = __fdiv_rn(f[i], s);
  }
  // no explicit clamp to +-448: the conversion below saturates finite values to the same result
  out.x = pack4_e4m3(q[0], q[1], q[2], q[3]);
  out.y = pack4_e4m3(q[4], q[5], q[6], q[7]);
  out.z = pack4_e4m3(q[8], q[9], q[10], q[11]);
  out.w = pack4_e4m3(q[12], q[13], q[14], q[15]);
  return s;
}

// max over the LPG (power of two <= 32) consecutive lanes that share one group.
template <int LPG>
__device__ __forceinline__ float group_max(float v) {
#pragma unroll
  for (int o = LPG / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace b200
