// Next-token sampling over 32-bit logits, one block per row of the batch.
//
// Per row: temperature < eps -> argmax (lowest index among equals).  Otherwise x = logit / T;
// top-k keeps x >= (k-th largest x); top-p then drops the low-probability tail whose
// cumulative probability stays <= 1 - p (the largest is always kept); the token is
// argmax_i (x_i - max) - log(q_i) with q_i ~ Exp(1), which is argmax softmax(x)_i / q_i.
// Thresholds are found by bisection over the order-preserving integer image of the floats
// (32 passes over the row each), which needs no sort and no scratch memory.
//
// Noise: Philox4x32-10 keyed by the request's 64-bit seed, counter = (vocabulary index / 4,
// index of the token being sampled, 0, 0); the four outputs serve four consecutive
// vocabulary entries.  u = (r + 0.5) * 2^-32 lies in (0, 1), q = -log(u).
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ uint32_t float_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                              uint32_t k0, uint32_t k1, uint32_t out[4]) {
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

struct ArgMax {
  float value;
  int index;
};

__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
  return a;
}

__device__ ArgMax block_argmax(ArgMax v, ArgMax* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other;
    other.value = __shfl_xor_sync(0xffffffffu, v.value, o);
    other.index = __shfl_xor_sync(0xffffffffu, v.index, o);
    v = better(v, other);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  ArgMax r = scratch[lane < (SAMPLE_THREADS / 32) ? lane : 0];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other;
    other.value = __shfl_xor_sync(0xffffffffu, r.value, o);
    other.index = __shfl_xor_sync(0xffffffffu, r.index, o);
    r = better(r, other);
  }
  return r;
}

__device__ float block_max_f(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  return warp_max(scratch[lane]);
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits, const double* __restrict__ params,
              int V, float eps) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_SAMPLE);
  __shared__ float fscratch[32];
  __shared__ ArgMax ascratch[32];
  const int row = blockIdx.x;
  const float* lg = logits + (size_t)row * V;
  const double* pr = params + (size_t)row * 6;
  const float temperature = (float)pr[0];
  const int top_k = (int)pr[1];
  const float top_p = (float)pr[2];
  const uint32_t seed_lo = (uint32_t)pr[3], seed_hi = (uint32_t)pr[4];
  const uint32_t token_index = (uint32_t)pr[5];
  const int tid = threadIdx.x;
  const ArgMax none = {-INFINITY, 0x7fffffff};

  if (temperature < eps) {
    // greedy: one pass; 16-byte loads, four of them in flight per thread (the row is read by one
    // block, so the pass is bound by the latency of its loads)
    ArgMax best = none;
    int done = 0;
    if ((reinterpret_cast<uintptr_t>(lg) & 15) == 0) {
      const int quads = V / 4;
      const float4* lg4 = reinterpret_cast<const float4*>(lg);
      for (int i0 = tid; i0 < quads; i0 += 4 * SAMPLE_THREADS) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i0 + u * SAMPLE_THREADS;
          v[u] = i < quads ? lg4[i] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (i0 + u * SAMPLE_THREADS >= quads) break;
          const int i = 4 * (i0 + u * SAMPLE_THREADS);
          best = better(best, ArgMax{v[u].x, i});
          best = better(best, ArgMax{v[u].y, i + 1});
          best = better(best, ArgMax{v[u].z, i + 2});
          best = better(best, ArgMax{v[u].w, i + 3});
        }
      }
      done = quads * 4;
    }
    for (int i = done + tid; i < V; i += SAMPLE_THREADS) best = better(best, ArgMax{lg[i], i});
    best = block_argmax(best, ascratch);
    if (tid == 0) out[row] = best.index;
    return;
  }

  // top-k: key of the k-th largest x
  uint32_t keep_from = 0;  // keep keys >= keep_from
  if (top_k < V) {
    uint32_t lo = 0, hi = 0xFFFFFFFFu;
    while (lo < hi) {
      const uint32_t mid = lo + (hi - lo) / 2 + ((hi - lo) & 1);  // upper middle
      float count = 0.0f;
      for (int i = tid; i < V; i += SAMPLE_THREADS) count += float_key(lg[i] / temperature) >= mid ? 1.0f : 0.0f;
      count = block_sum(count, fscratch);  // counts stay exact in float up to 2^24 entries
      if (count >= (float)top_k) lo = mid; else hi = mid - 1;
    }
    keep_from = lo;
  }

  float row_max = -INFINITY;
  for (int i = tid; i < V; i += SAMPLE_THREADS) row_max = fmaxf(row_max, lg[i] / temperature);
  row_max = block_max_f(row_max, fscratch);

  // top-p: drop keys <= drop_upto (none when top_p == 1)
  bool use_drop = false;
  uint32_t drop_upto = 0;
  if (top_p < 1.0f) {
    float z = 0.0f;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
      const float x = lg[i] / temperature;
      if (float_key(x) >= keep_from) z += expf(x - row_max);
    }
    z = block_sum(z, fscratch);
    const float target = (1.0f - top_p) * z;
    // Largest t below the key of the maximum whose mass of kept keys <= t stays <= target.
    // t = 0 always qualifies (no finite float maps to key 0), so `lo` is valid throughout.
    uint32_t lo = 0, hi = float_key(row_max) - 1;  // the largest is always kept
    while (lo < hi) {
      const uint32_t mid = lo + (hi - lo) / 2 + ((hi - lo) & 1);  // upper middle
      float mass = 0.0f;
      for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float x = lg[i] / temperature;
        const uint32_t key = float_key(x);
        if (key >= keep_from && key <= mid) mass += expf(x - row_max);
      }
      mass = block_sum(mass, fscratch);
      if (mass <= target) lo = mid; else hi = mid - 1;
    }
    use_drop = lo > 0;
    drop_upto = lo;
  }

  ArgMax best = none;
  const int groups = (V + 3) / 4;
  for (int g = tid; g < groups; g += SAMPLE_THREADS) {
    uint32_t r[4];
    philox4x32_10((uint32_t)g, token_index, 0u, 0u, seed_lo, seed_hi, r);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = g * 4 + j;
      if (i >= V) break;
      const float x = lg[i] / temperature;
      const uint32_t key = float_key(x);
      if (key < keep_from || (use_drop && key <= drop_upto)) continue;
      const float u = ((float)r[j] + 0.5f) * 2.3283064365386963e-10f;
      const float q = -logf(fminf(u, 0.99999994f));
      best = better(best, ArgMax{(x - row_max) - logf(q), i});
    }
  }
  best = block_argmax(best, ascratch);
  if (tid == 0) out[row] = best.index;
}

extern "C" int kvb_sample(int* out, const float* logits, const double* params, int rows, int V,
                          float eps, cudaStream_t stream) {
  if (rows == 0) return 0;
  KVB_REQUIRE(V > 0 && V < (1 << 24), "sample: vocabulary must be in [1, 2^24)");
  KVB_CHECK_CUDA(kvb_launch((sample_kernel), dim3(rows), dim3(SAMPLE_THREADS), 0, stream, true, out, logits, params, V, eps));
  KVB_CHECK_LAUNCH();
  return 0;
}

KVB_TRACE_TU(sampling)
