// Shared helpers of the sm_100a kernels: element types, 16-byte vectors, reductions with a
// fixed order, and the error convention of the exported C entry points.
//
// Every exported function returns 0 on success or a negative code after storing a message
// that kvb_last_error() hands to the Python side, which raises.  Kernels never trap; a
// device-side problem (a token id outside the table, a page id outside the pool) sets a
// bit in a status word that kvb_read_status() reads back.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define KVB_F32 0
#define KVB_BF16 1

#define KVB_STATUS_BAD_TOKEN 1
#define KVB_STATUS_BAD_PAGE 2
#define KVB_STATUS_WAIT_TIMEOUT 4

extern "C" int kvb_fail(int code, const char* what, const char* file, int line);
// Device address of the current device's status word (allocated once per device).
extern "C" int* kvb_status_word();

#define KVB_REQUIRE(cond, msg)                                   \
  do {                                                           \
    if (!(cond)) return kvb_fail(-1, msg, __FILE__, __LINE__);   \
  } while (0)

#define KVB_CHECK_LAUNCH()                                                        \
  do {                                                                            \
    cudaError_t kvb_err__ = cudaGetLastError();                                   \
    if (kvb_err__ != cudaSuccess)                                                 \
      return kvb_fail(-2, cudaGetErrorString(kvb_err__), __FILE__, __LINE__);     \
  } while (0)

#define KVB_CHECK_CUDA(call)                                                      \
  do {                                                                            \
    cudaError_t kvb_err__ = (call);                                               \
    if (kvb_err__ != cudaSuccess)                                                 \
      return kvb_fail(-2, cudaGetErrorString(kvb_err__), __FILE__, __LINE__);     \
  } while (0)

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

// A 16-byte vector of T: 4 floats or 8 bf16.
template <typename T>
struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  uint4 raw;
  __device__ __forceinline__ void load(const T* p) { raw = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void store(T* p) const { *reinterpret_cast<uint4*>(p) = raw; }
  __device__ __forceinline__ float get(int i) const {
    return to_float(reinterpret_cast<const T*>(&raw)[i]);
  }
  __device__ __forceinline__ void set(int i, float v) {
    reinterpret_cast<T*>(&raw)[i] = from_float<T>(v);
  }
};

__host__ __device__ __forceinline__ bool aligned16(const void* p) {
  return (reinterpret_cast<uintptr_t>(p) & 15) == 0;
}

// Butterfly reductions: every lane ends with the same value, combined in a fixed order.
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats. All threads get the sum.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = (lane < nwarps) ? scratch[lane] : 0.0f;
  return warp_sum(total);
}
