// Status strings, thread-local error detail and the per-device status word.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

namespace b200 {

static thread_local char g_detail[512] = "";

void set_error_detail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_detail, sizeof(g_detail), fmt, ap);
  va_end(ap);
}

Tuning& tuning() {
  static Tuning t;
  return t;
}

// One word per device that loads the library. Kernels with bounded waits write a non-zero
// code here (atomicCAS from 0, so the first failure is kept) and return normally.
__device__ int g_device_status = 0;

int* device_status_word() {
  // The symbol's device address differs per device; resolve it with that device current.
  static thread_local int cached_dev = -1;
  static thread_local int* cached_ptr = nullptr;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  if (dev != cached_dev) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
    cached_ptr = static_cast<int*>(p);
    cached_dev = dev;
  }
  return cached_ptr;
}

}  // namespace b200

extern "C" {

const char* b200_status_string(int status) {
  switch (status) {
    case B200_OK: return "ok";
    case B200_E_BAD_ARG: return "bad argument";
    case B200_E_UNSUPPORTED: return "unsupported configuration";
    case B200_E_LAUNCH: return "CUDA launch / descriptor error";
    case B200_E_WORKSPACE: return "workspace missing or too small";
    case B200_E_TIMEOUT: return "device-side wait timed out";
    default: return "unknown status";
  }
}

const char* b200_last_error_detail(void) { return b200::g_detail; }

int b200_abi_version(void) { return 2; }

static long* tuning_slot(const char* name) {
  b200::Tuning& t = b200::tuning();
  struct { const char* n; long* p; } table[] = {
      {"gemm_bn", &t.gemm_bn}, {"gemm_skinny", &t.gemm_skinny}, {"gemm_skinny_max_m", &t.gemm_skinny_max_m},
      {"gemm_splitk", &t.gemm_splitk}, {"gemm_2cta", &t.gemm_2cta}, {"gemm_ue8m0", &t.gemm_ue8m0}, {"linear_decode_fused", &t.linear_decode_fused}, {"moe_decode", &t.moe_decode}, {"moe_down_splitk", &t.moe_down_splitk},
      {"moe_zero_pads", &t.moe_zero_pads}, {"peer_wait_ms", &t.peer_wait_ms}};
  for (auto& e : table)
    if (name && strcmp(name, e.n) == 0) return e.p;
  return nullptr;
}

int b200_set_tuning(const char* name, long value) {
  long* slot = tuning_slot(name);
  B200_CHECK_ARG(slot != nullptr, "unknown tuning knob '%s'", name ? name : "(null)");
  *slot = value;
  return B200_OK;
}

int b200_get_tuning(const char* name, long* value) {
  long* slot = tuning_slot(name);
  B200_CHECK_ARG(slot != nullptr && value != nullptr, "unknown tuning knob '%s'", name ? name : "(null)");
  *value = *slot;
  return B200_OK;
}

int b200_read_device_status(int* out, void* stream) {
  B200_CHECK_ARG(out != nullptr, "out is null");
  int* word = b200::device_status_word();
  if (!word) {
    b200::set_error_detail("cannot resolve the device status word");
    return B200_E_LAUNCH;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(out, word, sizeof(int), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaMemsetAsync(word, 0, sizeof(int), st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) {
    b200::set_error_detail("read_device_status: %s", cudaGetErrorString(e));
    return B200_E_LAUNCH;
  }
  return B200_OK;
}

}  // extern "C"
