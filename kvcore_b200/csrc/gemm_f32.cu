// True 32-bit linear layer: out[m, n] = sum_k x[m, k] * w[n, k] (+ bias[n]), FMA on the CUDA
// cores only, no tensor cores and no reduced-precision mode.
//
// 64x64 output tile per block of 256 threads, 4x4 outputs per thread, K walked in slabs of
// 16 through shared memory.  Each output element is one accumulator that takes its products
// in ascending k, so its value does not depend on M, on the tile it falls in, or on the
// rest of the batch: the 32-bit path is bit-identical under any cutting of the work.
// Every M, N, K is accepted (edges are zero-filled in shared memory, adding exact zeros).
#include "common.cuh"

#define GT 64
#define GK 16

__global__ void __launch_bounds__(256)
gemm_f32_kernel(float* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w,
                const float* __restrict__ bias, int M, int N, int K, long long ldx, long long ldo) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_GEMM_F32);
  __shared__ float xs[GK][GT + 4];
  __shared__ float ws[GK][GT + 4];
  const int m0 = blockIdx.y * GT, n0 = blockIdx.x * GT;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // thread's 4x4 patch: rows ty*4.., cols tx*4..
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < K; k0 += GK) {
    // 64 rows x 16 k of each operand: 1024 elements, 4 per thread
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int idx = threadIdx.x + r * 256;
      const int row = idx >> 4, kk = idx & 15;
      const int k = k0 + kk;
      const int m = m0 + row, n = n0 + row;
      xs[kk][row] = (m < M && k < K) ? x[(size_t)m * ldx + k] : 0.0f;
      ws[kk][row] = (n < N && k < K) ? w[(size_t)n * K + k] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) out[(size_t)m * ldo + n] = acc[i][j] + (bias ? bias[n] : 0.0f);
    }
  }
}

extern "C" int kvb_gemm_f32(float* out, const float* x, const float* w, const float* bias, int M,
                            int N, int K, long long ldx, long long ldo, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  KVB_REQUIRE(K > 0, "gemm_f32: K must be positive");
  dim3 grid((N + GT - 1) / GT, (M + GT - 1) / GT);
  KVB_REQUIRE(grid.y <= 65535, "gemm_f32: too many rows for one launch");
  KVB_CHECK_CUDA(kvb_launch((gemm_f32_kernel), dim3(grid), dim3(256), 0, stream, true, out, x, w, bias, M, N, K, ldx, ldo));
  KVB_CHECK_LAUNCH();
  return 0;
}

KVB_TRACE_TU(gemm_f32)
