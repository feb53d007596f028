// Error reporting and the per-device status word shared by all kernels of the library.
#include <stdio.h>
#include <string.h>

#include "common.cuh"

static thread_local char g_last_error[512] = "";
static int* g_status_words[64] = {nullptr};

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
    int* word = nullptr;
    if (cudaMalloc(&word, sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(word, 0, sizeof(int));
    g_status_words[device] = word;
  }
  return g_status_words[device];
}

// Reads the status bits kernels have set since the last reset (synchronises the device).
extern "C" int kvb_read_status(int reset, int* out) {
  int* word = kvb_status_word();
  KVB_REQUIRE(word != nullptr, "cannot allocate the device status word");
  KVB_CHECK_CUDA(cudaMemcpy(out, word, sizeof(int), cudaMemcpyDeviceToHost));
  if (reset) KVB_CHECK_CUDA(cudaMemset(word, 0, sizeof(int)));
  return 0;
}

extern "C" int kvb_abi_version() { return 1; }

// Whether launches carry the programmatic-serialization attribute (kernels overlap their prologue
// with the tail of the kernel before them).  Off by default; the host side switches it on.
static int g_pdl_enabled = 0;
extern "C" int kvb_pdl_enabled() { return g_pdl_enabled; }
extern "C" void kvb_set_pdl(int enabled) { g_pdl_enabled = enabled; }
