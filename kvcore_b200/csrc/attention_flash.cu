// Paged flash attention for bf16 on tensor cores (mma.sync m16n8k16, fp32 accumulate), head
// sizes in steps of 16 up to 128.  One kernel body, two shapes:
//
//  * TILE mode (prompt portions, mixed batches): a block of 4 warps owns 64 query rows of one
//    (request, kv head); a row is a (token, query head of the group) pair, so the G heads that
//    share a kv head reuse every K/V tile.  Each warp owns 16 rows and walks all 64 keys of
//    each K/V tile.
//  * SPLIT mode (decode: at most 16 rows per request and kv head): the key range of a request
//    is cut into `num_splits` contiguous chunks, one block each; inside a block the 4 warps
//    take 16 keys each of every 64-key tile and merge their partial (max, sum, output)
//    through shared memory.  With more than one split the block writes its partial result to
//    scratch and a second kernel combines the splits.
//
// K/V tiles of 64 keys are gathered page by page through the block table with 16-byte
// cp.async copies into padded shared-memory rows (double buffered); fragments come from
// ldmatrix.  Scores, softmax and accumulation are 32-bit.  Keys outside the request, pages
// that were handed back (table entry 0) and rows beyond the batch are zero-filled or masked,
// never read as garbage.
//
// Cache layout [pages, KVH, page_size, D]; q rows at q + token*q_stride + head*D.
#include "common.cuh"

#define FA_KEYS 64          // keys per K/V tile
#define FA_THREADS 128
#define FA_PAD 8            // bf16 elements of padding per shared-memory row (16 bytes)
#define FA_PAGE_IDS 1024    // block-table entries staged in shared memory at a time

struct FlashParams {
  bf16* out; long long out_stride;
  const bf16* q; long long q_stride;
  const bf16* k_cache; const bf16* v_cache;
  const int* table; int table_stride;
  const int* query_start; const int* context_lens;
  int num_reqs, H, KVH, G, page_size, num_pages, window;
  float scale_log2;          // scale * log2(e)
  int num_splits;
  float* partial_o;          // [reqs, KVH, splits, 16, D]
  float* partial_ml;         // [reqs, KVH, splits, 16, 2]
  int* status;
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&v);
}

// Stage the block-table entries [first, first + FA_PAGE_IDS) of this request in shared memory
// (one coalesced sweep by the whole block), so that no tile waits on a table lookup.
__device__ __forceinline__ void stage_page_ids(int* ids, const FlashParams& p, const int* pages, int first) {
  for (int i = threadIdx.x; i < FA_PAGE_IDS; i += FA_THREADS) {
    const int index = first + i;
    ids[i] = index < p.table_stride ? pages[index] : 0;
  }
}

// Element offset of every key row of a 64-key tile inside the cache (or -1: zero-fill), from
// the staged page ids; done by the first 64 threads, one row each.
template <int D>
__device__ __forceinline__ void lookup_tile_rows(long long* rows, const FlashParams& p, const int* ids,
                                                 int ids_first, int kvh, int key0, int key_lo, int key_hi) {
  if (threadIdx.x >= FA_KEYS) return;
  const int key = key0 + threadIdx.x;
  long long off = -1;
  if (key >= key_lo && key < key_hi) {
    const int page = ids[key / p.page_size - ids_first];
    if (page > 0 && page < p.num_pages)
      off = ((long long)page * p.KVH + kvh) * p.page_size * D + (long long)(key % p.page_size) * D;
    else if (page != 0)
      atomicOr(p.status, KVB_STATUS_BAD_PAGE);
  }
  rows[threadIdx.x] = off;
}

// Copy one 64-key tile of K and V into shared memory, 16 bytes per cp.async.
template <int D>
__device__ __forceinline__ void load_kv_tile(bf16* ks, bf16* vs, const FlashParams& p,
                                             const long long* rows) {
  constexpr int ROW = D + FA_PAD;
  constexpr int CHUNKS = D / 8;
#pragma unroll 4
  for (int i = threadIdx.x; i < FA_KEYS * CHUNKS; i += FA_THREADS) {
    const int row = i / CHUNKS, chunk = i % CHUNKS;
    const long long base = rows[row];
    const bool valid = base >= 0;
    const long long off = valid ? base + chunk * 8 : 0;
    cp_async16(ks + row * ROW + chunk * 8, p.k_cache + off, valid);
    cp_async16(vs + row * ROW + chunk * 8, p.v_cache + off, valid);
  }
}

template <int D, bool SPLIT>
__global__ void __launch_bounds__(FA_THREADS)
flash_paged_kernel(const FlashParams p) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_FLASH);
  constexpr int ROW = D + FA_PAD;
  constexpr int TILE_M = SPLIT ? 16 : 64;
  constexpr int KSTEPS = D / 16;   // k-steps of Q.K^T
  constexpr int DBLOCKS = D / 8;   // n-blocks of the output
  constexpr int WARP_KEYS = SPLIT ? 16 : 64;   // keys of a tile one warp scores
  constexpr int NB = WARP_KEYS / 8;            // score n-blocks per warp

  extern __shared__ __align__(16) unsigned char smem_raw[];
  long long* tile_rows = reinterpret_cast<long long*>(smem_raw);  // [2][FA_KEYS] row offsets
  int* page_ids = reinterpret_cast<int*>(smem_raw + 2 * FA_KEYS * sizeof(long long));  // [FA_PAGE_IDS]
  bf16* qs = reinterpret_cast<bf16*>(smem_raw + 2 * FA_KEYS * sizeof(long long) + FA_PAGE_IDS * sizeof(int));
  bf16* ks = qs + TILE_M * ROW;
  bf16* vs = ks + 2 * FA_KEYS * ROW;

  const int req = blockIdx.z, kvh = blockIdx.y;
  const int tile = SPLIT ? 0 : gridDim.x - 1 - blockIdx.x;   // heaviest (latest) query tiles first
  const int split = SPLIT ? blockIdx.x : 0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_begin = p.query_start[req];
  const int q_len = p.query_start[req + 1] - q_begin;
  const int context = p.context_lens[req];
  const int rows_total = q_len * p.G;
  const int row0 = tile * TILE_M;
  if (row0 >= rows_total) return;  // whole block: this request has fewer rows
  const int* pages = p.table + (size_t)req * p.table_stride;

  // rows of this block: flat row r -> token r / G, head kvh*G + r % G
  const int last_row = min(row0 + TILE_M, rows_total) - 1;
  const int first_pos = context + row0 / p.G;
  const int last_pos = context + last_row / p.G;
  int key_lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  int key_hi = last_pos + 1;
  if (SPLIT) {
    const int tiles = (key_hi - (key_lo / FA_KEYS) * FA_KEYS + FA_KEYS - 1) / FA_KEYS;
    const int per = (tiles + p.num_splits - 1) / p.num_splits;
    const int base = (key_lo / FA_KEYS) * FA_KEYS;
    const int lo = base + split * per * FA_KEYS;
    const int hi = min(key_hi, lo + per * FA_KEYS);
    key_lo = max(key_lo, lo);
    key_hi = hi;
  }
  const int tile_begin = key_lo / FA_KEYS;
  const int tile_end = key_hi > key_lo ? (key_hi + FA_KEYS - 1) / FA_KEYS : tile_begin;

  // ---- Q tile into shared memory, then into A fragments --------------------------------
  for (int i = threadIdx.x; i < TILE_M * (D / 8); i += FA_THREADS) {
    const int r = i / (D / 8), chunk = i % (D / 8);
    const int flat = row0 + r;
    const bool valid = flat < rows_total;
    const int token = q_begin + (valid ? flat / p.G : 0);
    const int head = kvh * p.G + (valid ? flat % p.G : 0);
    cp_async16(qs + r * ROW + chunk * 8, p.q + (size_t)token * p.q_stride + (size_t)head * D + chunk * 8, valid);
  }
  cp_async_commit();
  // Page ids are staged FA_PAGE_IDS entries at a time; tiles_per_stage tiles fit one staging.
  const int tiles_per_staging = FA_PAGE_IDS * p.page_size / FA_KEYS;
  int ids_first = (tile_begin * FA_KEYS) / p.page_size;   // table entry held in page_ids[0]
  int restage_tile = tile_begin + tiles_per_staging;       // first tile that needs the next staging
  if (p.page_size > FA_KEYS || FA_KEYS % p.page_size) restage_tile = tile_begin + max(1, tiles_per_staging - 1);
  if (tile_begin < tile_end) {
    stage_page_ids(page_ids, p, pages, ids_first);
    __syncthreads();
    lookup_tile_rows<D>(tile_rows, p, page_ids, ids_first, kvh, tile_begin * FA_KEYS, key_lo, key_hi);
    if (tile_begin + 1 < tile_end)
      lookup_tile_rows<D>(tile_rows + FA_KEYS, p, page_ids, ids_first, kvh, (tile_begin + 1) * FA_KEYS, key_lo, key_hi);
    __syncthreads();
    load_kv_tile<D>(ks, vs, p, tile_rows);
  }
  cp_async_commit();
  cp_async_wait<1>();
  __syncthreads();

  const int wrow = SPLIT ? 0 : warp * 16;  // first row of this warp inside the block's tile
  unsigned qf[KSTEPS][4];
#pragma unroll
  for (int k = 0; k < KSTEPS; ++k) {
    const int r = wrow + (lane & 7) + 8 * ((lane >> 3) & 1);
    const int c = k * 16 + 8 * (lane >> 4);
    ldmatrix_x4(qf[k], qs + r * ROW + c);
  }
  // positions of this lane's two rows (lane/4 and lane/4 + 8)
  int row_pos[2];
  bool row_valid[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int flat = row0 + wrow + (lane >> 2) + 8 * h;
    row_valid[h] = flat < rows_total;
    row_pos[h] = context + (row_valid[h] ? flat / p.G : 0);
  }

  float o[DBLOCKS][4];
#pragma unroll
  for (int j = 0; j < DBLOCKS; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
  float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};

  for (int t = tile_begin; t < tile_end; ++t) {
    const int buf = (t - tile_begin) & 1;
    bf16* kt = ks + buf * FA_KEYS * ROW;
    bf16* vt = vs + buf * FA_KEYS * ROW;
    if (t + 1 < tile_end)
      load_kv_tile<D>(ks + (buf ^ 1) * FA_KEYS * ROW, vs + (buf ^ 1) * FA_KEYS * ROW, p,
                      tile_rows + (buf ^ 1) * FA_KEYS);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();  // tile t has landed; the row offsets of tile t (slot buf) are spent
    if (t + 2 < tile_end) {  // offsets of tile t+2 go to slot buf; published by the barrier that ends this turn
      if (t + 2 >= restage_tile) {  // uniform: the staged ids run out, fetch the next stretch
        ids_first = ((t + 2) * FA_KEYS) / p.page_size;
        restage_tile = t + 2 + max(1, tiles_per_staging - 1);
        __syncthreads();
        stage_page_ids(page_ids, p, pages, ids_first);
        __syncthreads();
      }
      lookup_tile_rows<D>(tile_rows + buf * FA_KEYS, p, page_ids, ids_first, kvh, (t + 2) * FA_KEYS, key_lo, key_hi);
    }

    const int wkey = SPLIT ? warp * 16 : 0;  // first key of the tile this warp scores
    float s[NB][4];
#pragma unroll
    for (int j = 0; j < NB; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
    for (int k = 0; k < KSTEPS; ++k) {
#pragma unroll
      for (int j = 0; j < NB; j += 2) {
        unsigned kb[4];
        const int key = wkey + j * 8 + (lane & 7) + 8 * (lane >> 4);
        const int c = k * 16 + 8 * ((lane >> 3) & 1);
        ldmatrix_x4(kb, kt + key * ROW + c);
        mma_bf16(s[j], qf[k], kb[0], kb[1]);
        mma_bf16(s[j + 1], qf[k], kb[2], kb[3]);
      }
    }
    // mask and online softmax (base-2 exponent)
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < NB; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        const int key = t * FA_KEYS + wkey + j * 8 + (lane & 3) * 2 + (e & 1);
        const bool seen = row_valid[h] && key >= key_lo && key < key_hi && key <= row_pos[h] &&
                          (p.window <= 0 || key > row_pos[h] - p.window);
        const float v = seen ? s[j][e] * p.scale_log2 : -INFINITY;
        s[j][e] = v;
        tile_max[h] = fmaxf(tile_max[h], v);
      }
    }
    float correction[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float m = tile_max[h];
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
      const float new_max = fmaxf(row_max[h], m);
      correction[h] = (row_max[h] == -INFINITY) ? 0.0f : exp2f(row_max[h] - new_max);
      row_max[h] = new_max;
      row_sum[h] *= correction[h];
    }
#pragma unroll
    for (int j = 0; j < DBLOCKS; ++j) {
      o[j][0] *= correction[0]; o[j][1] *= correction[0];
      o[j][2] *= correction[1]; o[j][3] *= correction[1];
    }
#pragma unroll
    for (int j = 0; j < NB; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        const float pv = (s[j][e] == -INFINITY) ? 0.0f : exp2f(s[j][e] - row_max[h]);
        s[j][e] = pv;
        row_sum[h] += pv;
      }
    }
    // O += P V over this warp's keys, 16 keys per step
#pragma unroll
    for (int kk = 0; kk < NB / 2; ++kk) {
      unsigned pa[4];
      pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int j = 0; j < DBLOCKS; j += 2) {
        unsigned vb[4];
        const int key = wkey + kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
        const int c = j * 8 + 8 * (lane >> 4);
        ldmatrix_x4_trans(vb, vt + key * ROW + c);
        mma_bf16(o[j], pa, vb[0], vb[1]);
        mma_bf16(o[j + 1], pa, vb[2], vb[3]);
      }
    }
    __syncthreads();  // everyone is done with this buffer before it is refilled
  }
  cp_async_wait<0>();

  // row sums live spread over the 4 lanes of a quad
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 1);
    row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 2);
  }

  if (!SPLIT) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (!row_valid[h]) continue;
      const int flat = row0 + wrow + (lane >> 2) + 8 * h;
      const int token = q_begin + flat / p.G;
      const int head = kvh * p.G + flat % p.G;
      const float inv = row_sum[h] > 0.0f ? 1.0f / row_sum[h] : 0.0f;
      bf16* dst = p.out + (size_t)token * p.out_stride + (size_t)head * D + (lane & 3) * 2;
#pragma unroll
      for (int j = 0; j < DBLOCKS; ++j)
        *reinterpret_cast<unsigned*>(dst + j * 8) = pack_bf16(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
    }
    return;
  }

  // ---- SPLIT: merge the four warps (each saw other keys of the same 16 rows) -------------
  __syncthreads();
  float* merge_o = reinterpret_cast<float*>(ks);            // [4 warps][16 rows][D]
  float* merge_ml = merge_o + 4 * 16 * D;                   // [4 warps][16 rows][2]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = (lane >> 2) + 8 * h;
#pragma unroll
    for (int j = 0; j < DBLOCKS; ++j) {
      float* dst = merge_o + ((size_t)(warp * 16 + r)) * D + j * 8 + (lane & 3) * 2;
      dst[0] = o[j][2 * h];
      dst[1] = o[j][2 * h + 1];
    }
    if ((lane & 3) == 0) {
      merge_ml[(warp * 16 + r) * 2 + 0] = row_max[h];
      merge_ml[(warp * 16 + r) * 2 + 1] = row_sum[h];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 16 * D; i += FA_THREADS) {
    const int r = i / D, d = i % D;
    if (r >= rows_total) continue;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, merge_ml[(w * 16 + r) * 2]);
    float total = 0.0f, acc = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = merge_ml[(w * 16 + r) * 2];
      const float f = (mw == -INFINITY) ? 0.0f : exp2f(mw - m);
      total += merge_ml[(w * 16 + r) * 2 + 1] * f;
      acc += merge_o[((size_t)(w * 16 + r)) * D + d] * f;
    }
    if (p.num_splits == 1) {
      const int token = q_begin + r / p.G;
      const int head = kvh * p.G + r % p.G;
      p.out[(size_t)token * p.out_stride + (size_t)head * D + d] =
          __float2bfloat16_rn(total > 0.0f ? acc / total : 0.0f);
    } else {
      const size_t slot = ((size_t)req * p.KVH + kvh) * p.num_splits + split;
      p.partial_o[(slot * 16 + r) * D + d] = acc;
      if (d == 0) {
        p.partial_ml[(slot * 16 + r) * 2 + 0] = m;
        p.partial_ml[(slot * 16 + r) * 2 + 1] = total;
      }
    }
  }
}

// Merge the splits of every (request, kv head, row): out = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M).
// One thread per output element; grid.x covers the 16 rows x D elements of a (request, kv head).
template <int D>
__global__ void flash_combine_kernel(const FlashParams p) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_FLASH_COMBINE);
  const int req = blockIdx.z, kvh = blockIdx.y;
  const int q_begin = p.query_start[req];
  const int rows_total = (p.query_start[req + 1] - q_begin) * p.G;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = i / D, d = i % D;
  if (r >= rows_total || r >= 16) return;
  const size_t base = ((size_t)req * p.KVH + kvh) * p.num_splits;
  // One trip to memory per eight splits: their maxima, sums and outputs are asked for together and
  // merged into the running triple (m, total, acc), rescaled when a later batch raises the maximum.
  // The splits are still added in their own order.
  float m = -INFINITY, total = 0.0f, acc = 0.0f;
  for (int s0 = 0; s0 < p.num_splits; s0 += 8) {
    float ms[8], ls[8], os[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool live = s0 + j < p.num_splits;
      const float2 ml = live ? *reinterpret_cast<const float2*>(p.partial_ml + ((base + s0 + j) * 16 + r) * 2)
                             : make_float2(-INFINITY, 0.0f);
      ms[j] = ml.x;
      ls[j] = ml.y;
      os[j] = live ? p.partial_o[((base + s0 + j) * 16 + r) * D + d] : 0.0f;
    }
    float batch_max = m;
#pragma unroll
    for (int j = 0; j < 8; ++j) batch_max = fmaxf(batch_max, ms[j]);
    if (batch_max > m) {
      const float keep = (m == -INFINITY) ? 0.0f : exp2f(m - batch_max);
      total *= keep;
      acc *= keep;
      m = batch_max;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float f = (ms[j] == -INFINITY) ? 0.0f : exp2f(ms[j] - m);
      total += ls[j] * f;
      acc += os[j] * f;
    }
  }
  const int token = q_begin + r / p.G;
  const int head = kvh * p.G + r % p.G;
  p.out[(size_t)token * p.out_stride + (size_t)head * D + d] =
      __float2bfloat16_rn(total > 0.0f ? acc / total : 0.0f);
}

template <int D>
static int launch_flash(const FlashParams& p, bool split_mode, int max_rows, cudaStream_t stream) {
  constexpr int ROW = D + FA_PAD;
  if (split_mode) {
    const size_t rows_bytes = 2 * FA_KEYS * sizeof(long long) + FA_PAGE_IDS * sizeof(int);
    size_t smem = rows_bytes + (size_t)(16 + 4 * FA_KEYS) * ROW * sizeof(bf16);
    const size_t merge = (size_t)(4 * 16 * D + 4 * 16 * 2) * sizeof(float);
    if (smem < rows_bytes + 16 * ROW * sizeof(bf16) + merge) smem = rows_bytes + 16 * ROW * sizeof(bf16) + merge;
    static bool configured_split = false;  // set once (the first call is never inside a graph capture)
    if (!configured_split) {
      KVB_CHECK_CUDA(cudaFuncSetAttribute(flash_paged_kernel<D, true>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      configured_split = true;
    }
    dim3 grid(p.num_splits, p.KVH, p.num_reqs);
    KVB_CHECK_CUDA(kvb_launch((flash_paged_kernel<D, true>), dim3(grid), dim3(FA_THREADS), smem, stream, true, p));
    KVB_CHECK_LAUNCH();
    if (p.num_splits > 1) {
      const int rows = max_rows < 16 ? max_rows : 16;
      dim3 cgrid((rows * D + 127) / 128, p.KVH, p.num_reqs);
      KVB_CHECK_CUDA(kvb_launch((flash_combine_kernel<D>), dim3(cgrid), dim3(128), 0, stream, true, p));
      KVB_CHECK_LAUNCH();
    }
  } else {
    const size_t smem = 2 * FA_KEYS * sizeof(long long) + FA_PAGE_IDS * sizeof(int) +
                        (size_t)(64 + 4 * FA_KEYS) * ROW * sizeof(bf16);
    static bool configured_tile = false;
    if (!configured_tile) {
      KVB_CHECK_CUDA(cudaFuncSetAttribute(flash_paged_kernel<D, false>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      configured_tile = true;
    }
    dim3 grid((max_rows + 63) / 64, p.KVH, p.num_reqs);
    KVB_CHECK_CUDA(kvb_launch((flash_paged_kernel<D, false>), dim3(grid), dim3(FA_THREADS), smem, stream, true, p));
    KVB_CHECK_LAUNCH();
  }
  return 0;
}

// Scratch floats needed for `num_splits` splits: partial outputs then partial (max, sum).
extern "C" long long kvb_flash_scratch_floats(int num_reqs, int KVH, int num_splits, int D) {
  if (num_splits <= 1) return 0;
  return (long long)num_reqs * KVH * num_splits * 16 * (D + 2);
}

// max_query_len: the longest portion in the batch.  split mode is used when every request has
// at most 16 (token, head) rows per kv head; otherwise num_splits must be 1.
extern "C" int kvb_flash_paged_attention(void* out, long long out_stride, const void* q,
                                         long long q_stride, const void* k_cache, const void* v_cache,
                                         const int* table, int table_stride, const int* query_start,
                                         const int* context_lens, int num_reqs, int max_query_len,
                                         int H, int KVH, int D, int page_size, int num_pages,
                                         float scale, int window, int num_splits, float* scratch,
                                         cudaStream_t stream) {
  if (num_reqs == 0) return 0;
  KVB_REQUIRE(D % 16 == 0 && D >= 16 && D <= 128, "flash attention: head_dim must be a multiple of 16 up to 128");
  KVB_REQUIRE(H > 0 && KVH > 0 && H % KVH == 0, "flash attention: H must be a multiple of KVH");
  KVB_REQUIRE(page_size > 0 && num_pages > 1, "flash attention: empty cache");
  KVB_REQUIRE(num_reqs <= 65535 && KVH <= 65535, "flash attention: batch too large for one launch");
  KVB_REQUIRE(aligned16(q) && aligned16(k_cache) && aligned16(v_cache) && (q_stride % 8) == 0,
              "flash attention: q and the caches must be 16-byte aligned");
  FlashParams p;
  p.out = (bf16*)out; p.out_stride = out_stride;
  p.q = (const bf16*)q; p.q_stride = q_stride;
  p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
  p.table = table; p.table_stride = table_stride;
  p.query_start = query_start; p.context_lens = context_lens;
  p.num_reqs = num_reqs; p.H = H; p.KVH = KVH; p.G = H / KVH;
  p.page_size = page_size; p.num_pages = num_pages; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = kvb_status_word();
  KVB_REQUIRE(p.status != nullptr, "flash attention: no status word");
  const int max_rows = max_query_len * p.G;
  const bool split_mode = max_rows <= 16;
  KVB_REQUIRE(split_mode || num_splits <= 1, "flash attention: splits need at most 16 rows per kv head");
  KVB_REQUIRE(num_splits <= KVB_MAX_SPLITS, "flash attention: at most 1024 splits");
  p.num_splits = num_splits < 1 ? 1 : num_splits;
  KVB_REQUIRE(p.num_splits == 1 || scratch != nullptr, "flash attention: splits need scratch memory");
  p.partial_o = scratch;
  p.partial_ml = scratch ? scratch + (size_t)num_reqs * KVH * p.num_splits * 16 * D : nullptr;
  switch (D) {
    case 16: return launch_flash<16>(p, split_mode, max_rows, stream);
    case 32: return launch_flash<32>(p, split_mode, max_rows, stream);
    case 48: return launch_flash<48>(p, split_mode, max_rows, stream);
    case 64: return launch_flash<64>(p, split_mode, max_rows, stream);
    case 80: return launch_flash<80>(p, split_mode, max_rows, stream);
    case 96: return launch_flash<96>(p, split_mode, max_rows, stream);
    case 112: return launch_flash<112>(p, split_mode, max_rows, stream);
    case 128: return launch_flash<128>(p, split_mode, max_rows, stream);
  }
  return kvb_fail(-1, "flash attention: unsupported head_dim", __FILE__, __LINE__);
}

// ------------------------------------------------------------------------------------------
// The same attention for callers that must not allocate (see no_alloc_api.h): scratch and
// status word live in this file's own device arrays.
// ------------------------------------------------------------------------------------------
#include "no_alloc_api.h"

static __device__ __align__(256) float kvb_static_scratch[KVB_STATIC_SCRATCH_FLOATS];
static __device__ __align__(256) int kvb_static_status_word[64];

// In host code the two names above are only stand-ins for the device arrays; the addresses a
// kernel can use come from cudaGetSymbolAddress, looked up once per device.
static float* g_static_scratch_ptr[64] = {nullptr};
static int* g_static_status_ptr[64] = {nullptr};

static int static_arrays(float** scratch, int** status) {
  int device = 0;
  KVB_CHECK_CUDA(cudaGetDevice(&device));
  KVB_REQUIRE(device >= 0 && device < 64, "static attention: device index out of range");
  if (g_static_scratch_ptr[device] == nullptr) {
    void* ptr = nullptr;
    KVB_CHECK_CUDA(cudaGetSymbolAddress(&ptr, kvb_static_scratch));
    KVB_REQUIRE(ptr != nullptr, "static attention: no device address for the scratch array");
    void* word = nullptr;
    KVB_CHECK_CUDA(cudaGetSymbolAddress(&word, kvb_static_status_word));
    KVB_REQUIRE(word != nullptr, "static attention: no device address for the status word");
    g_static_status_ptr[device] = static_cast<int*>(word);
    g_static_scratch_ptr[device] = static_cast<float*>(ptr);
  }
  *scratch = g_static_scratch_ptr[device];
  *status = g_static_status_ptr[device];
  return 0;
}

extern "C" int kvb_flash_paged_attention_static(void* out, long long out_stride, const void* q,
                                                long long q_stride, const void* k_cache, const void* v_cache,
                                                const int* table, int table_stride, const int* query_start,
                                                const int* context_lens, int num_reqs, int max_query_len,
                                                int H, int KVH, int D, int page_size, int num_pages,
                                                float scale, int window, int num_splits, cudaStream_t stream) {
  if (num_reqs == 0) return 0;
  KVB_REQUIRE(D % 16 == 0 && D >= 16 && D <= 128, "static attention: head_dim must be a multiple of 16 up to 128");
  KVB_REQUIRE(H > 0 && KVH > 0 && H % KVH == 0, "static attention: H must be a multiple of KVH");
  KVB_REQUIRE(page_size > 0 && num_pages > 1, "static attention: empty cache");
  KVB_REQUIRE(num_reqs <= 65535 && KVH <= 65535, "static attention: batch too large for one launch");
  KVB_REQUIRE(aligned16(q) && aligned16(k_cache) && aligned16(v_cache) && (q_stride % 8) == 0,
              "static attention: q and the caches must be 16-byte aligned");
  KVB_REQUIRE(num_splits <= KVB_MAX_SPLITS, "static attention: at most 1024 splits");
  const int splits = num_splits < 1 ? 1 : num_splits;
  const int max_rows = max_query_len * (H / KVH);
  const bool split_mode = max_rows <= 16;
  KVB_REQUIRE(split_mode || splits == 1, "static attention: splits need at most 16 rows per kv head");
  const long long needed = splits > 1 ? (long long)num_reqs * KVH * splits * 16 * (D + 2) : 0;
  KVB_REQUIRE(needed <= (long long)KVB_STATIC_SCRATCH_FLOATS,
              "static attention: num_reqs * KVH * num_splits * 16 * (D + 2) exceeds the built-in scratch "
              "of KVB_STATIC_SCRATCH_FLOATS floats");
  float* scratch = nullptr;
  int* status = nullptr;
  if (int rc = static_arrays(&scratch, &status)) return rc;
  // Nothing in the arrays has to be cleared per call: the kernels write every partial result they
  // later read, and the status word starts at zero with the library image and is cleared by
  // kvb_static_status, so that a bit set by one call is still there after the calls behind it.
  FlashParams p;
  p.out = (bf16*)out; p.out_stride = out_stride;
  p.q = (const bf16*)q; p.q_stride = q_stride;
  p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
  p.table = table; p.table_stride = table_stride;
  p.query_start = query_start; p.context_lens = context_lens;
  p.num_reqs = num_reqs; p.H = H; p.KVH = KVH; p.G = H / KVH;
  p.page_size = page_size; p.num_pages = num_pages; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  p.num_splits = splits;
  p.partial_o = scratch;
  p.partial_ml = scratch + (size_t)num_reqs * KVH * splits * 16 * D;
  switch (D) {
    case 16: return launch_flash<16>(p, split_mode, max_rows, stream);
    case 32: return launch_flash<32>(p, split_mode, max_rows, stream);
    case 48: return launch_flash<48>(p, split_mode, max_rows, stream);
    case 64: return launch_flash<64>(p, split_mode, max_rows, stream);
    case 80: return launch_flash<80>(p, split_mode, max_rows, stream);
    case 96: return launch_flash<96>(p, split_mode, max_rows, stream);
    case 112: return launch_flash<112>(p, split_mode, max_rows, stream);
    case 128: return launch_flash<128>(p, split_mode, max_rows, stream);
  }
  return kvb_fail(-1, "static attention: unsupported head_dim", __FILE__, __LINE__);
}

extern "C" int kvb_static_status(int* out) {
  float* scratch = nullptr;
  int* status = nullptr;
  if (int rc = static_arrays(&scratch, &status)) return rc;
  KVB_CHECK_CUDA(cudaMemcpy(out, status, sizeof(int), cudaMemcpyDeviceToHost));
  KVB_CHECK_CUDA(cudaMemset(status, 0, sizeof(int)));
  return 0;
}

KVB_TRACE_TU(attention_flash)
