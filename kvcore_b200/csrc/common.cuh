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

// Most chunks a request's keys may be cut into by the split-KV attention entry points (sizes of
// their scratch are products with this count; the bound keeps them far inside 64 bits).
#define KVB_MAX_SPLITS 1024

extern "C" int kvb_fail(int code, const char* what, const char* file, int line);
// Device address of the current device's status word (allocated once per device).
extern "C" int* kvb_status_word();
// Multiprocessors of the current device (0 if the driver cannot be asked).
extern "C" int kvb_sm_count();

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

// ---- programmatic dependent launch --------------------------------------------------------------
// A kernel launched with the attribute below may start while the kernel before it in the stream
// is still running: it runs its prologue (barrier set-up, loads of data that no earlier kernel of
// the step writes: weights, the cached keys of earlier steps), then kvb_grid_wait() returns once
// the earlier kernel has completed and its writes are visible.  kvb_grid_launch_dependents() tells
// the scheduler that the next kernel may be brought in.  Both are no-ops in a plain launch.
// Rule for every kernel that uses them: nothing that an earlier kernel writes is read, and nothing
// in global memory is written, before kvb_grid_wait().
__device__ __forceinline__ void kvb_grid_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void kvb_grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

// ---- kernel timeline trace ----------------------------------------------------------------------
// When a trace buffer is set, the first and the last block of every kernel of this library append
// one event {tag, first/last/other, SM, block index, time at entry, time after kvb_grid_wait(), time
// at exit} (nanoseconds of the GPU's global timer).  Word 0 of the buffer counts events, word 1 is the capacity in events
// (its top bit set: every block records, not only the first and the last).
// The pointer lives once per translation unit (set through KVB_TRACE_TU's setter); null = off.
static __device__ unsigned long long* kvb_trace_buffer = nullptr;

__device__ __forceinline__ unsigned long long kvb_global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

struct KvbTrace {
  unsigned long long* buffer;
  unsigned long long entry, waited;
  int tag;
  __device__ __forceinline__ explicit KvbTrace(int kernel_tag) : buffer(nullptr), entry(0), waited(0), tag(kernel_tag) {
    unsigned long long* b = kvb_trace_buffer;
    if (b != nullptr && threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) {
      const bool first = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
      const bool last = blockIdx.x == gridDim.x - 1 && blockIdx.y == gridDim.y - 1 && blockIdx.z == gridDim.z - 1;
      if (first || last || (b[1] >> 63)) {
        buffer = b;
        entry = kvb_global_ns();
      }
    }
  }
  __device__ __forceinline__ void after_wait() {
    if (buffer != nullptr) waited = kvb_global_ns();
  }
  __device__ __forceinline__ ~KvbTrace() {
    if (buffer != nullptr) {
      const unsigned long long slot = atomicAdd(buffer, 1ull);
      if (slot < (buffer[1] & ~(1ull << 63))) {
        unsigned long long* e = buffer + 2 + slot * 4;
        const bool first = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
        const bool last = blockIdx.x == gridDim.x - 1 && blockIdx.y == gridDim.y - 1 && blockIdx.z == gridDim.z - 1;
        // word 0: tag (8 bits) | first/last/other (2 bits at 8) | SM (10 bits at 12) | linear block index (at 32)
        const unsigned long long index = blockIdx.x + (unsigned long long)gridDim.x * (blockIdx.y + (unsigned long long)gridDim.y * blockIdx.z);
        unsigned sm;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
        e[0] = (unsigned long long)(tag & 0xff) | (first ? 0ull : last ? 1ull << 8 : 2ull << 8) |
               ((unsigned long long)(sm & 0x3ff) << 12) | (index << 32);
        e[1] = entry;
        e[2] = waited;
        e[3] = kvb_global_ns();
      }
    }
  }
};

// First statements of every kernel: trace scope, wait for the kernel in front, let the next one in.
#define KVB_KERNEL_PROLOGUE(tag)                                                               \
  KvbTrace kvb_trace_scope__(tag);                                                             \
  kvb_grid_wait();               /* ordered after the kernel in front (dependent launch) */    \
  kvb_trace_scope__.after_wait();                                                              \
  kvb_grid_launch_dependents()   /* the kernel behind may be brought in; it waits the same way */

// One per .cu file: the setter through which the host hands this file's kernels the trace buffer.
#define KVB_TRACE_TU(name)                                                                     \
  extern "C" int kvb_trace_set_##name(unsigned long long* buffer) {                            \
    return (int)cudaMemcpyToSymbol(kvb_trace_buffer, &buffer, sizeof(buffer));                 \
  }

// Kernel tags of the trace.
#define KVB_TAG_GATHER 1
#define KVB_TAG_RMSNORM 2
#define KVB_TAG_SILU_MUL 3
#define KVB_TAG_ROPE_TABLE 4
#define KVB_TAG_ROPE_KV_WRITE 5
#define KVB_TAG_ATTN_ROWS 6
#define KVB_TAG_FLASH 7
#define KVB_TAG_FLASH_COMBINE 8
#define KVB_TAG_DECODE_TMA 9
#define KVB_TAG_DECODE_COMBINE 10
#define KVB_TAG_PREFILL_TC5 11
#define KVB_TAG_GEMM_F32 12
#define KVB_TAG_GEMM_STREAM 13
#define KVB_TAG_SAMPLE 14
#define KVB_TAG_FEED_TOKENS 16

// 1 when launches should carry the programmatic-serialization attribute (set by the host side).
extern "C" int kvb_pdl_enabled();

template <typename... Params, typename... Args>
static inline cudaError_t kvb_launch(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, bool overlap, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = (overlap && kvb_pdl_enabled()) ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

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

// SiLU of an activation whose result is rounded to bf16 by the caller: the fast exponential and
// division are within ~1e-6 of the exact ones, three orders inside the rounding, and cost a fifth
// of the instructions (the activation kernel of a prompt is bound by instruction issue, not memory).
// The 32-bit path uses the exact form.
__device__ __forceinline__ float kvb_silu_for_bf16(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

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
