// Shared host/device helpers of libgmb200: status codes, the per-thread error
// message, launch checks, element-type traits (storage type vs compute type)
// and small complex helpers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <type_traits>
#include <cstdint>
#include <cstdio>

#include "../../include/gm_b200.h"

namespace gmb {

// ---- error reporting (never throws across the C ABI) ----
char* error_buffer();
int fail(int code, const char* fmt, ...);

#define GM_REQUIRE(cond, code, ...)                 \
  do {                                              \
    if (!(cond)) return ::gmb::fail(code, __VA_ARGS__); \
  } while (0)

#define GM_CUDA(call)                                                                              \
  do {                                                                                             \
    cudaError_t err__ = (call);                                                                    \
    if (err__ != cudaSuccess) return ::gmb::fail(GM_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(err__)); \
  } while (0)

inline int launch_status(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(GM_ERR_CUDA, "%s: %s", what, cudaGetErrorString(err));
  return GM_OK;
}

// SMs of the current device
inline int sm_count() {
  int device = 0, n = 148;
  if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device);
  return n;
}

// Opt a kernel in to `bytes` of dynamic shared memory (needed above 48 KiB).
template <typename Kernel>
inline int allow_smem(Kernel kernel, size_t bytes, const char* what) {
  cudaFuncAttributes attr;
  GM_CUDA(cudaFuncGetAttributes(&attr, kernel));
  if (bytes + attr.sharedSizeBytes <= 48 * 1024) return GM_OK;  // static + dynamic fit the default limit
  int device = 0, limit = 0;
  GM_CUDA(cudaGetDevice(&device));
  GM_CUDA(cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
  if ((size_t)limit < bytes) return fail(GM_ERR_LIMIT, "%s needs %zu bytes of shared memory, the device grants %d", what, bytes, limit);
  GM_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return GM_OK;
}

// ---- element types: S = storage, compute type = Compute<S>::type ----
template <typename S> struct Compute { using type = S; };
template <> struct Compute<__nv_bfloat16> { using type = float; };

template <typename C, typename S> __device__ __forceinline__ C ld(const S* p) { return (C)(*p); }
template <> __device__ __forceinline__ float ld<float, __nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename S, typename C> __device__ __forceinline__ void st(S* p, C v) { *p = (S)v; }
template <> __device__ __forceinline__ void st<__nv_bfloat16, float>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float gm_exp(float x) { return expf(x); }
__device__ __forceinline__ double gm_exp(double x) { return exp(x); }
__device__ __forceinline__ float gm_log(float x) { return logf(x); }
__device__ __forceinline__ double gm_log(double x) { return log(x); }
template <typename T> __device__ __forceinline__ T neg_inf() { return -(T)INFINITY; }

template <typename T>
__device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
template <typename T>
__device__ __forceinline__ T warp_max(T v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    T other = __shfl_xor_sync(0xffffffffu, v, o);
    v = other > v ? other : v;
  }
  return v;
}

}  // namespace gmb
