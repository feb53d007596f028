// Paged attention, general kernel: any head size up to 256, any head counts, any mix of
// prompt portions and decode tokens, optional sliding window, float or bf16 storage.
//
// One warp owns one (token, query head) row and walks the request's keys from the first
// visible position to the token's own position in steps of 32 keys: each lane scores one key
// (a full dot product over the head, in ascending order), the warp keeps a running maximum
// and sum (online softmax, 32-bit), and every lane accumulates its own slice of the output
// over the 32 values.  The walk depends only on the token's position, never on how the
// step was cut or batched, so a row's result is bit-identical under any cutting.  This is
// the kernel of the 32-bit path; the bf16 path uses it for shapes its faster kernels refuse.
//
// Cache layout: [pages, KVH, page_size, D]; page ids come from table[req, pos / page_size].
#include "common.cuh"

#define ATT_MAX_D 256
#define ATT_WARPS 4

template <typename T>
__device__ __forceinline__ float dot_row(const T* __restrict__ k, const float* __restrict__ q, int D,
                                         bool vec) {
  float acc = 0.0f;
  if (vec) {
    constexpr int N = Vec16<T>::N;
    for (int d = 0; d < D; d += N) {
      Vec16<T> kv;
      kv.load(k + d);
#pragma unroll
      for (int j = 0; j < N; ++j) acc = fmaf(kv.get(j), q[d + j], acc);
    }
  } else {
    for (int d = 0; d < D; ++d) acc = fmaf(to_float(k[d]), q[d], acc);
  }
  return acc;
}

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
paged_attention_rows_kernel(T* __restrict__ out, int out_stride, const T* __restrict__ q,
                            int q_stride, const T* __restrict__ k_cache,
                            const T* __restrict__ v_cache, const int* __restrict__ table,
                            int table_stride, const int* __restrict__ positions,
                            const int* __restrict__ req_index, int num_rows, int H, int KVH, int D,
                            int page_size, int num_pages, float scale, int window, int vec,
                            int* status) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_ATTN_ROWS);
  __shared__ float q_smem[ATT_WARPS][ATT_MAX_D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * ATT_WARPS + warp;
  if (row >= num_rows) return;
  const int token = row / H, head = row % H;
  const int kvh = head / (H / KVH);
  const int pos = positions[token];
  const int* pages = table + (size_t)req_index[token] * table_stride;

  const T* qrow = q + (size_t)token * q_stride + (size_t)head * D;
  for (int d = lane; d < D; d += 32) q_smem[warp][d] = to_float(qrow[d]);
  __syncwarp();

  constexpr int SLICES = ATT_MAX_D / 32;
  float acc[SLICES];
#pragma unroll
  for (int i = 0; i < SLICES; ++i) acc[i] = 0.0f;
  float running_max = -INFINITY, running_sum = 0.0f;
  const size_t head_off = (size_t)kvh * page_size * D;
  const size_t page_elems = (size_t)KVH * page_size * D;
  const int first = window > 0 ? max(0, pos - window + 1) : 0;

  for (int base = first; base <= pos; base += 32) {
    const int key = base + lane;
    const bool valid = key <= pos;
    float score = -INFINITY;
    int page = 0;
    if (valid) {
      page = pages[key / page_size];
      if (page <= 0 || page >= num_pages) {
        atomicOr(status, KVB_STATUS_BAD_PAGE);
        page = 0;
      } else {
        const T* krow = k_cache + (size_t)page * page_elems + head_off + (size_t)(key % page_size) * D;
        score = dot_row<T>(krow, q_smem[warp], D, vec) * scale;
      }
    }
    const float chunk_max = warp_max(score);
    const float new_max = fmaxf(running_max, chunk_max);
    // new_max is finite whenever the chunk holds one readable key; key `base` always is
    const float p = (score == -INFINITY) ? 0.0f : expf(score - new_max);
    const float correction = (running_max == -INFINITY) ? 0.0f : expf(running_max - new_max);
    running_sum = running_sum * correction + warp_sum(p);
    running_max = new_max;
#pragma unroll
    for (int i = 0; i < SLICES; ++i) acc[i] *= correction;
    const int count = min(32, pos - base + 1);
    for (int kk = 0; kk < count; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, p, kk);
      const int pg = __shfl_sync(0xffffffffu, page, kk);
      if (pg == 0) continue;  // uniform across the warp
      const T* vrow = v_cache + (size_t)pg * page_elems + head_off + (size_t)((base + kk) % page_size) * D;
#pragma unroll
      for (int i = 0; i < SLICES; ++i) {
        const int d = lane + 32 * i;
        if (d < D) acc[i] = fmaf(pk, to_float(vrow[d]), acc[i]);
      }
    }
  }
  const float inv = running_sum > 0.0f ? 1.0f / running_sum : 0.0f;
  T* orow = out + (size_t)token * out_stride + (size_t)head * D;
#pragma unroll
  for (int i = 0; i < SLICES; ++i) {
    const int d = lane + 32 * i;
    if (d < D) orow[d] = from_float<T>(acc[i] * inv);
  }
}

extern "C" int kvb_paged_attention_rows(void* out, int out_stride, const void* q, int q_stride,
                                        const void* k_cache, const void* v_cache, const int* table,
                                        int table_stride, const int* positions, const int* req_index,
                                        int tokens, int H, int KVH, int D, int page_size,
                                        int num_pages, float scale, int window, int dtype,
                                        cudaStream_t stream) {
  if (tokens == 0) return 0;
  KVB_REQUIRE(D > 0 && D <= ATT_MAX_D, "paged_attention: head_dim must be in [1, 256]");
  KVB_REQUIRE(H > 0 && KVH > 0 && H % KVH == 0, "paged_attention: H must be a multiple of KVH");
  KVB_REQUIRE(page_size > 0 && num_pages > 1, "paged_attention: empty cache");
  int* status = kvb_status_word();
  KVB_REQUIRE(status != nullptr, "paged_attention: no status word");
  const int esize = dtype == KVB_F32 ? 4 : 2;
  const int vec = ((size_t)D * esize) % 16 == 0 && aligned16(k_cache);
  const long long rows = (long long)tokens * H;
  KVB_REQUIRE(rows < (1ll << 31), "paged_attention: too many rows");
  const int blocks = (int)((rows + ATT_WARPS - 1) / ATT_WARPS);
  if (dtype == KVB_F32)
    KVB_CHECK_CUDA(kvb_launch((paged_attention_rows_kernel<float>), dim3(blocks), dim3(ATT_WARPS * 32), 0, stream, true, 
        (float*)out, out_stride, (const float*)q, q_stride, (const float*)k_cache,
        (const float*)v_cache, table, table_stride, positions, req_index, (int)rows, H, KVH, D,
        page_size, num_pages, scale, window, vec, status));
  else
    KVB_CHECK_CUDA(kvb_launch((paged_attention_rows_kernel<bf16>), dim3(blocks), dim3(ATT_WARPS * 32), 0, stream, true, 
        (bf16*)out, out_stride, (const bf16*)q, q_stride, (const bf16*)k_cache,
        (const bf16*)v_cache, table, table_stride, positions, req_index, (int)rows, H, KVH, D,
        page_size, num_pages, scale, window, vec, status));
  KVB_CHECK_LAUNCH();
  return 0;
}

KVB_TRACE_TU(attention_generic)
