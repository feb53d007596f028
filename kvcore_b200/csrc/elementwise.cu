// Memory-bound kernels of the step: row gather (token embedding, logits rows), RMS norm with
// the residual sum folded in, SiLU(gate)*up, and rotary encoding fused with the cache write.
// Each is templated on the activation type (float for the 32-bit path, bf16 for serving) and
// does its arithmetic in 32-bit.  16-byte vector loads are used when the row size and the
// pointers allow, scalar loops otherwise, so every width is accepted.
#include "common.cuh"

// ------------------------------------------------------------------------------------------
// Row gather: out[i, :] = table[ids[i], :].  An id outside [0, rows) writes zeros and sets the
// BAD_TOKEN status bit instead of reading out of bounds.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* __restrict__ table,
                                   const int* __restrict__ ids, int width, int rows, int vec_ok,
                                   int* status) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_GATHER);
  const int row = blockIdx.x;
  const int id = ids[row];
  const bool valid = id >= 0 && id < rows;
  if (!valid && threadIdx.x == 0) atomicOr(status, KVB_STATUS_BAD_TOKEN);
  T* dst = out + (size_t)row * width;
  const T* src = table + (size_t)(valid ? id : 0) * width;
  if (vec_ok) {
    constexpr int N = Vec16<T>::N;
    for (int i = threadIdx.x * N; i < width; i += blockDim.x * N) {
      Vec16<T> v;
      if (valid) v.load(src + i); else v.raw = make_uint4(0, 0, 0, 0);
      v.store(dst + i);
    }
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x)
      dst[i] = valid ? src[i] : from_float<T>(0.0f);
  }
}

extern "C" int kvb_gather_rows(void* out, const void* table, const int* ids, int count, int width,
                               int rows, int dtype, cudaStream_t stream) {
  if (count == 0) return 0;
  KVB_REQUIRE(width > 0 && rows > 0, "gather_rows: empty table");
  int* status = kvb_status_word();
  KVB_REQUIRE(status != nullptr, "gather_rows: no status word");
  const int esize = dtype == KVB_F32 ? 4 : 2;
  const int vec_ok = ((size_t)width * esize) % 16 == 0 && aligned16(out) && aligned16(table);
  const int threads = 128;
  if (dtype == KVB_F32)
    KVB_CHECK_CUDA(kvb_launch((gather_rows_kernel<float>), dim3(count), dim3(threads), 0, stream, true, (float*)out, (const float*)table, ids,
                                                             width, rows, vec_ok, status));
  else
    KVB_CHECK_CUDA(kvb_launch((gather_rows_kernel<bf16>), dim3(count), dim3(threads), 0, stream, true, (bf16*)out, (const bf16*)table, ids,
                                                           width, rows, vec_ok, status));
  KVB_CHECK_LAUNCH();
  return 0;
}

// ------------------------------------------------------------------------------------------
// Token feedback: token_ids[t] = sampled[source[t]] where source[t] >= 0.  Lets a decode step be
// launched before the host has seen the tokens that the step in front sampled: the host packs a
// placeholder id and names the row of the earlier sampler output that holds the real one.
// ------------------------------------------------------------------------------------------
__global__ void feed_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ source,
                                   const int* __restrict__ sampled, int count, int sampled_rows,
                                   int* status) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_FEED_TOKENS);
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= count) return;
  const int row = source[t];
  if (row < 0) return;
  if (row >= sampled_rows) {   // never reads outside the sampler's output
    atomicOr(status, KVB_STATUS_BAD_TOKEN);
    return;
  }
  token_ids[t] = sampled[row];
}

extern "C" int kvb_feed_tokens(int* token_ids, const int* source, const int* sampled, int count,
                               int sampled_rows, cudaStream_t stream) {
  if (count == 0) return 0;
  KVB_REQUIRE(sampled_rows > 0, "feed_tokens: no sampled tokens to take from");
  int* status = kvb_status_word();
  KVB_REQUIRE(status != nullptr, "feed_tokens: no status word");
  const int threads = 128;
  KVB_CHECK_CUDA(kvb_launch((feed_tokens_kernel), dim3((count + threads - 1) / threads), dim3(threads), 0,
                            stream, true, token_ids, source, sampled, count, sampled_rows, status));
  KVB_CHECK_LAUNCH();
  return 0;
}

// ------------------------------------------------------------------------------------------
// RMS norm.  One block of 256 threads per row, whatever the batch: the reduction tree depends
// on the width only, so a row's result does not depend on what else is in the batch.
//   ADD: s = h + residual (rounded to T, stored back as the new residual), else s = h
//   out = T( w * (s * rsqrt(mean(s^2) + eps)) ), everything between in 32-bit.
// ------------------------------------------------------------------------------------------
template <typename T, typename W, bool ADD, bool VEC>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(T* __restrict__ out, T* __restrict__ residual, const T* __restrict__ h,
               const W* __restrict__ weight, int width, float eps) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_RMSNORM);
  __shared__ float scratch[32];
  const size_t base = (size_t)blockIdx.x * width;
  const T* hr = h + base;
  T* rr = ADD ? residual + base : nullptr;
  T* orow = out + base;
  float sq = 0.0f;
  if (VEC) {
    constexpr int N = Vec16<T>::N;
    constexpr int KEEP = 4;                       // vectors a thread keeps in registers between the passes
    const bool kept = width <= 256 * N * KEEP;    // rows up to 8,192 bf16 (4,096 float) values wide
    Vec16<T> mine[KEEP];
    int slot = 0;
    for (int i = threadIdx.x * N; i < width; i += 256 * N, ++slot) {
      Vec16<T> a;
      a.load(hr + i);
      if (ADD) {
        Vec16<T> r;
        r.load(rr + i);
#pragma unroll
        for (int j = 0; j < N; ++j) a.set(j, a.get(j) + r.get(j));
        a.store(rr + i);
      }
#pragma unroll
      for (int j = 0; j < N; ++j) { const float x = a.get(j); sq += x * x; }
      if (kept) {
#pragma unroll
        for (int s = 0; s < KEEP; ++s) if (s == slot) mine[s] = a;
      }
    }
    const float total = block_sum(sq, scratch);
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
    const T* src = ADD ? rr : hr;  // each thread re-reads exactly what it wrote itself
    slot = 0;
    for (int i = threadIdx.x * N; i < width; i += 256 * N, ++slot) {
      Vec16<T> a, o;
      if (kept) {
#pragma unroll
        for (int s = 0; s < KEEP; ++s) if (s == slot) a = mine[s];
      } else {
        a.load(src + i);
      }
      if (sizeof(W) == sizeof(T)) {
        Vec16<W> g;
        g.load(weight + i);
#pragma unroll
        for (int j = 0; j < N; ++j) o.set(j, g.get(j) * (a.get(j) * inv));
      } else {
#pragma unroll
        for (int j = 0; j < N; ++j) o.set(j, to_float(weight[i + j]) * (a.get(j) * inv));
      }
      o.store(orow + i);
    }
  } else {
    for (int i = threadIdx.x; i < width; i += 256) {
      float x = to_float(hr[i]);
      if (ADD) {
        const T s = from_float<T>(x + to_float(rr[i]));
        rr[i] = s;
        x = to_float(s);
      }
      sq += x * x;
    }
    const float total = block_sum(sq, scratch);
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
    const T* src = ADD ? rr : hr;  // each thread re-reads exactly what it wrote itself
    for (int i = threadIdx.x; i < width; i += 256)
      orow[i] = from_float<T>(to_float(weight[i]) * (to_float(src[i]) * inv));
  }
}

template <typename T, typename W>
static int launch_rmsnorm(void* out, void* residual, const void* h, const void* w, int rows,
                          int width, float eps, bool add, bool vec, cudaStream_t stream) {
#define KVB_RMS(ADD_, VEC_)                                                                       \
  KVB_CHECK_CUDA(kvb_launch((rmsnorm_kernel<T, W, ADD_, VEC_>), dim3(rows), dim3(256), 0, stream, true, \
                            (T*)out, (T*)residual, (const T*)h, (const W*)w, width, eps))
  if (add) { if (vec) KVB_RMS(true, true); else KVB_RMS(true, false); }
  else { if (vec) KVB_RMS(false, true); else KVB_RMS(false, false); }
#undef KVB_RMS
  return 0;
}

// residual == nullptr: plain norm of h.  Otherwise residual is updated in place to h + residual.
extern "C" int kvb_rmsnorm(void* out, void* residual, const void* h, const void* weight, int rows,
                           int width, float eps, int dtype, int weight_dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  KVB_REQUIRE(width > 0, "rmsnorm: width must be positive");
  const int esize = dtype == KVB_F32 ? 4 : 2;
  const bool add = residual != nullptr;
  const bool vec = ((size_t)width * esize) % 16 == 0 && aligned16(out) && aligned16(h) &&
                   (!add || aligned16(residual));
  if (dtype == KVB_F32) {
    KVB_REQUIRE(weight_dtype == KVB_F32, "rmsnorm: a 32-bit model needs 32-bit norm weights");
    if (int rc = launch_rmsnorm<float, float>(out, residual, h, weight, rows, width, eps, add, vec, stream)) return rc;
  } else if (weight_dtype == KVB_F32) {
    if (int rc = launch_rmsnorm<bf16, float>(out, residual, h, weight, rows, width, eps, add, vec, stream)) return rc;
  } else {
    if (int rc = launch_rmsnorm<bf16, bf16>(out, residual, h, weight, rows, width, eps, add, vec, stream)) return rc;
  }
  KVB_CHECK_LAUNCH();
  return 0;
}

// ------------------------------------------------------------------------------------------
// out[t, i] = silu(gate(t, i)) * up(t, i).  group == 0: gate(t, i) = gu[t, i], up(t, i) = gu[t, inter + i].
// group > 0: gate and up alternate in runs of `group` columns (gate 0..g-1, up 0..g-1, gate g..2g-1, ...),
// the layout a feed-forward keeps when its gate/up matrix is packed for the fused decode kernel.
// ------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float silu(float x);
template <>
__device__ __forceinline__ float silu<float>(float x) { return x / (1.0f + expf(-x)); }
template <>
__device__ __forceinline__ float silu<bf16>(float x) { return kvb_silu_for_bf16(x); }

template <typename T, bool VEC>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, int inter, int group,
                                long long total_vecs) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_SILU_MUL);
  constexpr int N = VEC ? Vec16<T>::N : 1;
  const int per_row = inter / N;
  // (row, vector of the row) of this thread's items, stepped without a division per item
  const long long first = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long step = (long long)gridDim.x * blockDim.x;
  long long row = first / per_row;
  int vec = (int)(first % per_row);
  const long long row_step = step / per_row;
  const int vec_step = (int)(step % per_row);
  const bool pow2 = group > 0 && (group & (group - 1)) == 0;   // runs of a power of two: shifts
  const int shift = pow2 ? __ffs(group) - 1 : 0;
  for (long long v = first; v < total_vecs; v += step) {
    const int col = vec * N;
    const int gate_col = group == 0 ? col
                         : pow2 ? ((col >> shift) << (shift + 1)) + (col & (group - 1))
                                : (col / group) * 2 * group + col % group;
    const T* g = gu + row * 2 * inter + gate_col;
    const int up = group > 0 ? group : inter;
    T* o = out + row * inter + col;
    if (VEC) {
      Vec16<T> a, b, r;
      a.load(g);
      b.load(g + up);
#pragma unroll
      for (int j = 0; j < Vec16<T>::N; ++j) {
        // the product is formed from the rounded activation, as silu(gate) * up in T would be
        const float s = to_float(from_float<T>(silu<T>(a.get(j))));
        r.set(j, s * b.get(j));
      }
      r.store(o);
    } else {
      const float s = to_float(from_float<T>(silu<T>(to_float(g[0]))));
      o[0] = from_float<T>(s * to_float(g[up]));
    }
    row += row_step;
    vec += vec_step;
    if (vec >= per_row) {
      vec -= per_row;
      ++row;
    }
  }
}

extern "C" int kvb_silu_mul(void* out, const void* gate_up, int rows, int inter, int group, int dtype,
                            cudaStream_t stream) {
  if (rows == 0) return 0;
  KVB_REQUIRE(inter > 0, "silu_mul: width must be positive");
  KVB_REQUIRE(group >= 0 && (group == 0 || inter % group == 0), "silu_mul: the group must divide the width");
  const int esize = dtype == KVB_F32 ? 4 : 2;
  const bool vec = ((size_t)inter * esize) % 16 == 0 && aligned16(out) && aligned16(gate_up) &&
                   (group == 0 || ((size_t)group * esize) % 16 == 0);
  const int n = vec ? 16 / esize : 1;
  const long long total = (long long)rows * (inter / n);
  const int threads = 256;
  const long long wanted = (total + threads - 1) / threads;
  const long long resident = (long long)(kvb_sm_count() > 0 ? kvb_sm_count() : 1) * 16;  // a grid-stride loop beyond that
  const int blocks = (int)(wanted < resident ? wanted : resident);
  if (dtype == KVB_F32) {
    if (vec) KVB_CHECK_CUDA(kvb_launch((silu_mul_kernel<float, true>), dim3(blocks), dim3(threads), 0, stream, true, (float*)out, (const float*)gate_up, inter, group, total));
    else KVB_CHECK_CUDA(kvb_launch((silu_mul_kernel<float, false>), dim3(blocks), dim3(threads), 0, stream, true, (float*)out, (const float*)gate_up, inter, group, total));
  } else {
    if (vec) KVB_CHECK_CUDA(kvb_launch((silu_mul_kernel<bf16, true>), dim3(blocks), dim3(threads), 0, stream, true, (bf16*)out, (const bf16*)gate_up, inter, group, total));
    else KVB_CHECK_CUDA(kvb_launch((silu_mul_kernel<bf16, false>), dim3(blocks), dim3(threads), 0, stream, true, (bf16*)out, (const bf16*)gate_up, inter, group, total));
  }
  KVB_CHECK_LAUNCH();
  return 0;
}

// ------------------------------------------------------------------------------------------
// cos/sin of every (token, frequency) of the step: table[t, j] = (cos, sin)(float(pos_t) * inv_freq[j]).
// Computed once per step and shared by all layers with the same frequency table.
// ------------------------------------------------------------------------------------------
__global__ void rope_table_kernel(float2* __restrict__ table, const int* __restrict__ positions,
                                  const float* __restrict__ inv_freq, int tokens, int half) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_ROPE_TABLE);
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= tokens * half) return;
  const int t = i / half, j = i % half;
  float s, c;
  sincosf((float)positions[t] * inv_freq[j], &s, &c);
  table[i] = make_float2(c, s);
}

extern "C" int kvb_rope_table(float* table, const int* positions, const float* inv_freq, int tokens,
                              int half, cudaStream_t stream) {
  if (tokens == 0) return 0;
  KVB_REQUIRE(half > 0, "rope_table: head_dim must be positive");
  const long long total = (long long)tokens * half;
  KVB_CHECK_CUDA(kvb_launch((rope_table_kernel), dim3((int)((total + 255) / 256)), dim3(256), 0, stream, true, (float2*)table, positions, inv_freq,
                                                                    tokens, half));
  KVB_CHECK_LAUNCH();
  return 0;
}

// ------------------------------------------------------------------------------------------
// Rotary encoding of q and k (half-rotation layout) fused with the write of k and v into the
// paged cache.  qkv is [T, (H + 2*KVH) * D]: q heads, then k heads, then v heads.
//   (c, s) = cos_sin[token, j]   (32-bit, from rope_table_kernel), j in [0, D/2)
//   x'[j] = x[j]*c - x[j+D/2]*s ;  x'[j+D/2] = x[j+D/2]*c + x[j]*s
// q and k are rotated in place; rotated k and v go to page table[req, pos / page] at offset
// pos % page of a cache laid out [pages, KVH, page, D].  cos_sin == nullptr: no rotation.
// k_cache == nullptr: nothing is written (an entry that reads another entry's cache).
// grid (tokens, head groups): threadIdx.x = j, threadIdx.y = head within the group; the
// blocks of a token share the copy of its v heads.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, long long qkv_stride,
                                     const int* __restrict__ positions,
                                     const int* __restrict__ req_index,
                                     const float2* __restrict__ cos_sin,
                                     const int* __restrict__ table, int table_stride,
                                     T* __restrict__ k_cache, T* __restrict__ v_cache, int H, int KVH,
                                     int D, int page_size, int num_pages, int* status) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_ROPE_KV_WRITE);
  const int token = blockIdx.x;
  const int half = D >> 1;
  const int pos = positions[token];
  T* row = qkv + (size_t)token * qkv_stride;

  size_t cache_base = 0;
  bool write = k_cache != nullptr;
  if (write) {
    const int page = table[(size_t)req_index[token] * table_stride + pos / page_size];
    if (page <= 0 || page >= num_pages) {
      if (threadIdx.x == 0 && threadIdx.y == 0 && blockIdx.y == 0) atomicOr(status, KVB_STATUS_BAD_PAGE);
      write = false;
    }
    cache_base = ((size_t)page * KVH * page_size + (pos % page_size)) * D;
  }
  const size_t head_stride = (size_t)page_size * D;  // between kv heads inside a page

  const int j = threadIdx.x;
  const int head = blockIdx.y * blockDim.y + threadIdx.y;
  if (j < half && head < H + KVH) {
    T* x = row + (size_t)head * D;
    float a = to_float(x[j]), b = to_float(x[j + half]);
    if (cos_sin != nullptr) {
      const float2 cs = cos_sin[(size_t)token * half + j];
      const float ra = a * cs.x - b * cs.y;
      const float rb = b * cs.x + a * cs.y;
      x[j] = from_float<T>(ra);
      x[j + half] = from_float<T>(rb);
      a = to_float(from_float<T>(ra));
      b = to_float(from_float<T>(rb));
    }
    if (head >= H && write) {
      T* dst = k_cache + cache_base + (size_t)(head - H) * head_stride;
      dst[j] = from_float<T>(a);
      dst[j + half] = from_float<T>(b);
    }
  }
  if (write) {
    const T* v = row + (size_t)(H + KVH) * D;
    const int tid = (blockIdx.y * blockDim.y + threadIdx.y) * blockDim.x + threadIdx.x;
    const int nthreads = gridDim.y * blockDim.y * blockDim.x;
    for (int i = tid; i < KVH * D; i += nthreads) {
      const int vh = i / D, d = i % D;
      v_cache[cache_base + (size_t)vh * head_stride + d] = v[i];
    }
  }
}

// Vector form of the kernel above for bf16 rows whose halves are multiples of 8 elements: a
// thread rotates 8 consecutive pairs (x[j..j+7], x[j+D/2..j+D/2+7]) with 16-byte accesses, and
// the v heads are copied 16 bytes at a time.  grid (tokens), any block size.
__global__ void rope_kv_write_vec_kernel(bf16* __restrict__ qkv, long long qkv_stride,
                                         const int* __restrict__ positions,
                                         const int* __restrict__ req_index,
                                         const float2* __restrict__ cos_sin,
                                         const int* __restrict__ table, int table_stride,
                                         bf16* __restrict__ k_cache, bf16* __restrict__ v_cache, int H,
                                         int KVH, int D, int page_size, int num_pages, int* status) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_ROPE_KV_WRITE);
  const int token = blockIdx.x;
  const int half = D >> 1;
  const int groups = half >> 3;                 // 16-byte groups per half
  const int pos = positions[token];
  bf16* row = qkv + (size_t)token * qkv_stride;
  size_t cache_base = 0;
  bool write = k_cache != nullptr;
  if (write) {
    const int page = table[(size_t)req_index[token] * table_stride + pos / page_size];
    if (page <= 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(status, KVB_STATUS_BAD_PAGE);
      write = false;
    }
    cache_base = ((size_t)page * KVH * page_size + (pos % page_size)) * D;
  }
  const size_t head_stride = (size_t)page_size * D;
  const int rotate_items = (H + KVH) * groups;
  const int copy_items = write ? KVH * (D >> 3) : 0;
  for (int item = threadIdx.x; item < rotate_items + copy_items; item += blockDim.x) {
    if (item < rotate_items) {
      const int head = item / groups, g = item % groups;
      bf16* x = row + (size_t)head * D + g * 8;
      Vec16<bf16> lo, hi;
      lo.load(x);
      hi.load(x + half);
      if (cos_sin != nullptr) {
        const float2* cs = cos_sin + (size_t)token * half + g * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float2 t = cs[i];
          const float a = lo.get(i), b = hi.get(i);
          lo.set(i, a * t.x - b * t.y);
          hi.set(i, b * t.x + a * t.y);
        }
        lo.store(x);
        hi.store(x + half);
      }
      if (head >= H && write) {
        bf16* dst = k_cache + cache_base + (size_t)(head - H) * head_stride + g * 8;
        lo.store(dst);
        hi.store(dst + half);
      }
    } else {
      const int i = item - rotate_items;
      const int vh = i / (D >> 3), g = i % (D >> 3);
      Vec16<bf16> v;
      v.load(row + (size_t)(H + KVH) * D + (size_t)vh * D + g * 8);
      v.store(v_cache + cache_base + (size_t)vh * head_stride + g * 8);
    }
  }
}

extern "C" int kvb_rope_kv_write(void* qkv, long long qkv_stride, const int* positions,
                                 const int* req_index, const float* cos_sin, const int* table,
                                 int table_stride, void* k_cache, void* v_cache, int tokens, int H,
                                 int KVH, int D, int page_size, int num_pages, int dtype,
                                 cudaStream_t stream) {
  if (tokens == 0) return 0;
  KVB_REQUIRE(D > 0 && D % 2 == 0 && D <= 1024, "rope_kv_write: head_dim must be even and <= 1024");
  KVB_REQUIRE(H >= 0 && KVH >= 0 && H + KVH > 0, "rope_kv_write: no heads to encode");
  KVB_REQUIRE(KVH > 0 || k_cache == nullptr, "rope_kv_write: a cache write needs kv heads");
  KVB_REQUIRE(qkv_stride >= (long long)(H + 2 * KVH) * D || (k_cache == nullptr && qkv_stride >= (long long)(H + KVH) * D),
              "rope_kv_write: row stride is smaller than the row");
  KVB_REQUIRE((k_cache == nullptr) == (v_cache == nullptr), "rope_kv_write: give both caches or none");
  KVB_REQUIRE(k_cache == nullptr || (table != nullptr && page_size > 0), "rope_kv_write: a cache write needs a block table");
  int* status = kvb_status_word();
  KVB_REQUIRE(status != nullptr, "rope_kv_write: no status word");
  const int half = D / 2;
  if (dtype == KVB_BF16 && D % 16 == 0 && qkv_stride % 8 == 0 && aligned16(qkv) &&
      (k_cache == nullptr || (aligned16(k_cache) && aligned16(v_cache)))) {
    const int items = (H + KVH) * (half / 8) + (k_cache ? KVH * (D / 8) : 0);
    int threads = 32;
    while (threads < items && threads < 256) threads <<= 1;
    KVB_CHECK_CUDA(kvb_launch((rope_kv_write_vec_kernel), dim3(tokens), dim3(threads), 0, stream, true, 
        (bf16*)qkv, qkv_stride, positions, req_index, (const float2*)cos_sin, table, table_stride,
        (bf16*)k_cache, (bf16*)v_cache, H, KVH, D, page_size, num_pages, status));
    KVB_CHECK_LAUNCH();
    return 0;
  }
  int tx = 1;
  while (tx < half) tx <<= 1;           // threads along j, a power of two >= D/2
  int ty = 128 / tx;
  if (ty < 1) ty = 1;
  if (ty > H + KVH) ty = H + KVH;
  dim3 block(tx, ty);
  dim3 grid(tokens, (H + KVH + ty - 1) / ty);
  KVB_REQUIRE(grid.y <= 65535, "rope_kv_write: too many heads");
  if (dtype == KVB_F32)
    KVB_CHECK_CUDA(kvb_launch((rope_kv_write_kernel<float>), dim3(grid), dim3(block), 0, stream, true, 
        (float*)qkv, qkv_stride, positions, req_index, (const float2*)cos_sin, table, table_stride,
        (float*)k_cache, (float*)v_cache, H, KVH, D, page_size, num_pages, status));
  else
    KVB_CHECK_CUDA(kvb_launch((rope_kv_write_kernel<bf16>), dim3(grid), dim3(block), 0, stream, true, 
        (bf16*)qkv, qkv_stride, positions, req_index, (const float2*)cos_sin, table, table_stride,
        (bf16*)k_cache, (bf16*)v_cache, H, KVH, D, page_size, num_pages, status));
  KVB_CHECK_LAUNCH();
  return 0;
}

KVB_TRACE_TU(elementwise)
