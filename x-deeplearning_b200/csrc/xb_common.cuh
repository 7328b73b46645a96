// Shared helpers for the sm_100a kernel library: error reporting, dtype
// dispatch and scalar load/store with conversion.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "xdlb200.h"

namespace xb {

// Thread-local reason of the last rejected call (returned by xb_last_error()).
int fail(int code, const char* fmt, ...);
void clear_error();

#define XB_REQUIRE(cond, code, ...)              \
  do {                                           \
    if (!(cond)) return xb::fail(code, __VA_ARGS__); \
  } while (0)

#define XB_CUDA(call)                                                            \
  do {                                                                           \
    cudaError_t e__ = (call);                                                    \
    if (e__ != cudaSuccess)                                                      \
      return xb::fail(XB_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e__)); \
  } while (0)

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(XB_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
  return 0;
}

inline size_t dtype_size(int dt) {
  switch (dt) {
    case XB_F32: case XB_I32: return 4;
    case XB_I64: return 8;
    case XB_F16: case XB_BF16: return 2;
    default: return 0;
  }
}

// Number of SMs of the current device (cached per device).
int sm_count();

// A launch attribute such as cudaFuncAttributeMaxDynamicSharedMemorySize belongs to one device, and one process
// may serve several (one workspace per device, blaze/blaze/api/cpp_api/predictor_manager_impl.cc:142-177): this
// remembers, per launcher, on which devices the attribute was set. Safe for concurrent serving threads: two
// threads that both find the bit clear both set the (idempotent) attribute.
struct PerDeviceOnce {
  std::atomic<uint64_t> bits{0};
  // true when the caller still has to do the set-up on the current device (ordinal above 63: always)
  bool needed(int* dev) {
    *dev = 0;
    if (cudaGetDevice(dev) != cudaSuccess || *dev < 0 || *dev >= 64) { *dev = -1; return true; }
    return ((bits.load(std::memory_order_acquire) >> *dev) & 1u) == 0;
  }
  void done(int dev) {
    if (dev >= 0) bits.fetch_or(uint64_t(1) << dev, std::memory_order_release);
  }
};
#define XB_SET_MAX_SMEM_ONCE(once, bytes, ...)                                                        \
  do {                                                                                                \
    int dev__;                                                                                        \
    if ((once).needed(&dev__)) {                                                                      \
      const void* fns__[] = {__VA_ARGS__};                                                            \
      for (const void* f__ : fns__)                                                                   \
        XB_CUDA(cudaFuncSetAttribute(f__, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(bytes))); \
      (once).done(dev__);                                                                             \
    }                                                                                                 \
  } while (0)

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Load/store through a runtime dtype (used by the low-rate glue kernels).
__device__ __forceinline__ float load_as_f32(const void* p, int64_t i, int dt) {
  if (dt == XB_F32) return reinterpret_cast<const float*>(p)[i];
  if (dt == XB_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
  if (dt == XB_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  if (dt == XB_I32) return (float)reinterpret_cast<const int32_t*>(p)[i];
  return 0.f;
}
__device__ __forceinline__ void store_from_f32(void* p, int64_t i, int dt, float v) {
  if (dt == XB_F32) reinterpret_cast<float*>(p)[i] = v;
  else if (dt == XB_F16) reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
  else if (dt == XB_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else if (dt == XB_I32) reinterpret_cast<int32_t*>(p)[i] = (int32_t)v;
}

// Activation epilogues, restating blaze/blaze/math/activation.h:36-68.
struct EpiParams {
  int kind;            // XB_EPI_*
  const float* a;      // prelu slopes / dice gamma
  const float* b;      // dice mean
  const float* c;      // dice var
  int count;           // prelu slope count
  int nosqrt;
};

__device__ __forceinline__ float dice_rstd(float var, int nosqrt) {
  return nosqrt ? 1.f / var : 1.f / sqrtf(var + 1e-8f);
}
__device__ __forceinline__ float act_dice(float x, float gamma, float mean, float rstd) {
  float p = 1.f / (1.f + __expf(-(x - mean) * rstd));
  return (1.f - p) * gamma * x + p * x;
}
__device__ __forceinline__ float act_prelu(float x, float w) {
  return x * ((x > 0.f ? 1.f : 0.f) + (x < 0.f ? w : 0.f));
}
__device__ __forceinline__ float act_sigmoid(float x) { return 1.f / (1.f + __expf(-x)); }

__device__ __forceinline__ float apply_epilogue(const EpiParams& e, float v, int col) {
  switch (e.kind) {
    case XB_EPI_PRELU: return act_prelu(v, e.a[e.count == 1 ? 0 : col]);
    case XB_EPI_DICE: return act_dice(v, e.a[col], e.b[col], dice_rstd(e.c[col], e.nosqrt));
    case XB_EPI_SIGMOID: return act_sigmoid(v);
    default: return v;
  }
}

}  // namespace xb
