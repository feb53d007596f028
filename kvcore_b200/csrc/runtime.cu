// Error reporting and the per-device status word shared by all kernels of the library.
#include <stdio.h>
#include <string.h>

#include "common.cuh"

static thread_local char g_last_error[512] = "";
// The status word lives in pinned host memory that the device sees too: kernels set bits in it
// (on their error paths only), the host reads it without a copy or a synchronisation.
static int* g_status_words[64] = {nullptr};        // device view
static volatile int* g_status_host[64] = {nullptr};  // host view of the same word

extern "C" int kvb_fail(int code, const char* what, const char* file, int line) {
  const char* base = strrchr(file, '/');
  snprintf(g_last_error, sizeof(g_last_error), "%s (%s:%d)", what, base ? base + 1 : file, line);
  return code;
}

extern "C" const char* kvb_last_error() { return g_last_error; }

extern "C" int* kvb_status_word() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
  if (g_status_words[device] == nullptr) {
    int* host = nullptr;
    int* seen_by_device = nullptr;
    if (cudaHostAlloc(&host, sizeof(int), cudaHostAllocMapped) != cudaSuccess) return nullptr;
    *host = 0;
    if (cudaHostGetDevicePointer(&seen_by_device, host, 0) != cudaSuccess) {
      cudaFreeHost(host);
      return nullptr;
    }
    g_status_host[device] = host;
    g_status_words[device] = seen_by_device;
  }
  return g_status_words[device];
}

// Reads the status bits kernels have set since the last reset, after everything launched so far
// has finished (synchronises the device).
extern "C" int kvb_read_status(int reset, int* out) {
  int* word = kvb_status_word();
  KVB_REQUIRE(word != nullptr, "cannot allocate the status word");
  int device = 0;
  KVB_CHECK_CUDA(cudaGetDevice(&device));
  KVB_CHECK_CUDA(cudaDeviceSynchronize());
  *out = *g_status_host[device];
  if (reset) *g_status_host[device] = 0;
  return 0;
}

// The same bits without waiting for anything: what the kernels that have finished so far reported.
// For a caller that has just synchronised on its own (it read a step's tokens back).
extern "C" int kvb_peek_status() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64 || g_status_host[device] == nullptr) return 0;
  return *g_status_host[device];
}

extern "C" int kvb_abi_version() { return 1; }

// Multiprocessors of the current device, asked from the driver once per device (0 if that fails).
extern "C" int kvb_sm_count() {
  static int counts[64] = {0};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
  if (counts[device] == 0) {
    int value = 0;
    if (cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    counts[device] = value;
  }
  return counts[device];
}

// Whether launches carry the programmatic-serialization attribute (kernels overlap their prologue
// with the tail of the kernel before them).  Off by default; the host side switches it on.
static int g_pdl_enabled = 0;
extern "C" int kvb_pdl_enabled() { return g_pdl_enabled; }
extern "C" void kvb_set_pdl(int enabled) { g_pdl_enabled = enabled; }
