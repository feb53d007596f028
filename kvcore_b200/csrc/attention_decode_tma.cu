// Split-KV paged attention for decode, fed by TMA (sm_100a).
//
// Decode reads every cached key and value once and does little arithmetic on them, so the
// kernel is built to keep as many bytes in flight as one SM can hold.  The work is cut into items,
// (request, kv head, split) triples; a block (two a SM) takes the item of its index and, when there are
// more items than blocks that fit the GPU at once, stays and takes further ones from a counter.  A
// producer warp walks an item's key range in tiles of 64 keys and, for each tile, looks the pages up in
// the block table and issues one tiled TMA copy per page (cp.async.bulk.tensor.2d, 128-byte swizzle;
// the block of one page and kv head is contiguous in the cache) for K and for V into a ring of STAGES
// shared-memory stages; each stage has a "full" mbarrier that the copies complete, an "empty"
// mbarrier that the consumers release, and a header that says which item and tile it holds.  The
// ring runs on from one item into the next: the next item's first tiles are on their way while the
// consumers still merge and store the last one.  Four consumer warps follow the headers; each
// warp scores 16 keys of a tile against the (at most 16) query rows of the request
// with mma.sync m16n8k16, keeps a running 32-bit softmax, and accumulates its part of the
// output; after an item's last tile the warps merge through shared memory (where q lay) and write
// either the final rows (one split) or a partial (max, sum, output) to scratch that a second kernel
// merges over the splits.
//
// Every wait on an mbarrier is bounded: when the bound is hit the thread sets the
// WAIT_TIMEOUT bit of the status word, the block stops waiting, drains the copies it
// issued (bounded again) and returns, so a fault in the pipeline cannot hang the GPU.
//
// Whole pages are copied, so slots of a request's last page beyond its length and the null
// page reach shared memory; their scores are masked and their probability is exactly zero.
// Cache memory is zero-initialised and only ever holds finite values, so 0 * value = 0.
#include <cuda.h>
#include <string.h>

#include "common.cuh"
#include "sm100.cuh"

#define TD_KEYS 64
#define TD_STAGES 3
#define TD_GROUPS 1        // consumer groups; group g takes the tiles t with t % TD_GROUPS == g
#define TD_GROUP_WARPS 4   // warps of a group; warp w of a group scores keys [16w, 16w+16) of a tile
#define TD_CONSUMERS (TD_GROUPS * TD_GROUP_WARPS)
#define TD_THREADS ((TD_CONSUMERS + 1) * 32)
#define TD_SPIN_LIMIT (1u << 20)

struct DecodeParams {
  bf16* out; long long out_stride;
  const bf16* q; long long q_stride;
  const int* table; int table_stride;
  const int* query_start; const int* context_lens;
  int num_reqs, H, KVH, G, page_size, num_pages, window;
  float scale_log2;
  int num_splits;
  float* partial_o;   // [reqs, KVH, splits, 16, D]
  float* partial_ml;  // [reqs, KVH, splits, 16, 2]
  int* status;
  // Rotation and cache write of this step's tokens done here instead of in a kernel in front
  // cos_sin != null: q rows are rotated on their way into shared memory.  k_cache != null: the
  // block whose key range holds a new token rotates its key (if cos_sin), writes key and value into
  // the cache page and lays them over the tile that TMA brought, which holds that slot's old bytes.
  const float2* cos_sin;      // [tokens, D / 2] (cos, sin)
  const bf16* k_new;          // this step's keys, row stride q_stride, [tokens][KVH][D] inside the qkv rows
  const bf16* v_new;
  bf16* k_cache; bf16* v_cache;   // [pages, KVH, page, D]
  // Work items are (request, kv head, split) triples, numbered in that order.  work == null: one item
  // a block.  Else blocks stay and take further items from work[0] (work[1] counts the blocks that
  // have seen the end; the last one puts both back to zero, where they must be before a launch).
  int total_items;
  int* work;
};

__device__ __forceinline__ void td_ldmatrix_x4(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void td_ldmatrix_x4_trans(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void td_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned td_pack(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&v);
}

// Byte offset of element (key, d) inside one stage's K (or V) area.  The cache is described to
// TMA as rows of 64 elements (128 bytes), so a key of D = 64*HALVES elements is HALVES
// consecutive rows and a whole page of a head is one contiguous box.  Shared-memory row
// r = key*HALVES + d/64 holds 8 chunks of 16 bytes, XOR-swizzled with r (128-byte swizzle).
template <int HALVES>
__device__ __forceinline__ unsigned swz(int key, int d) {
  const int r = key * HALVES + (d >> 6), chunk = (d & 63) >> 3;
  return (unsigned)(r * 128 + ((chunk ^ (r & 7)) << 4));
}

// What the producer tells the consumers about a stage of the ring: the work item it belongs to
// (a (request, kv head, split) triple; -1: no more items), the tile's index in the item's key range
// and what the consumers need to set the item up, so that they load nothing but q themselves.
struct TdStageHeader {
  int item, it, num_tiles, q_begin, q_len, context, key_lo, key_hi;
};

// Work item `item` = (request, kv head, split), numbered in that order: its query rows and the
// range of keys its split covers.
__device__ __forceinline__ TdStageHeader td_describe_item(const DecodeParams& p, int item) {
  TdStageHeader h;
  h.item = item;
  h.it = 0;
  const int req = item / (p.KVH * p.num_splits);
  const int split = item % p.num_splits;
  h.q_begin = p.query_start[req];
  h.q_len = p.query_start[req + 1] - h.q_begin;
  h.context = p.context_lens[req];
  const int rows_total = min(h.q_len * p.G, 16);
  const int last_pos = h.context + (rows_total - 1) / p.G;
  int key_lo = p.window > 0 ? max(0, h.context - p.window + 1) : 0;
  int key_hi = last_pos + 1;
  const int first_tile_key = (key_lo / TD_KEYS) * TD_KEYS;
  const int tiles = (key_hi - first_tile_key + TD_KEYS - 1) / TD_KEYS;
  const int per = (tiles + p.num_splits - 1) / p.num_splits;
  const int lo = first_tile_key + split * per * TD_KEYS;
  key_hi = min(key_hi, lo + per * TD_KEYS);
  key_lo = max(key_lo, lo);
  const int tile_begin = key_lo / TD_KEYS;
  const int tile_end = key_hi > key_lo ? (key_hi + TD_KEYS - 1) / TD_KEYS : tile_begin;
  h.num_tiles = tile_end - tile_begin;
  h.key_lo = key_lo;
  h.key_hi = key_hi;
  return h;
}

template <int D>
__global__ void __launch_bounds__(TD_THREADS, 2)
flash_decode_tma_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                        const DecodeParams p) {
  // No wait at the top: the pages of keys cached by earlier steps, the block table and the lengths
  // are written by no kernel of this step, so the producer warp starts its ring while the kernel
  // in front (the rotation and cache write of this step's tokens) still runs.  It waits before
  // the first tile that reaches this step's tokens; the other warps wait before they read q.
  KvbTrace kvb_trace_scope__(KVB_TAG_DECODE_TMA);
  kvb_grid_launch_dependents();
  static_assert(TD_GROUPS == 1, "the consumers follow the ring's headers together");
  constexpr int HALVES = D / 64;
  constexpr int KV_BYTES = TD_KEYS * D * 2;        // one of K or V of a stage
  constexpr int STAGE_BYTES = 2 * KV_BYTES;
  constexpr int QROW = D + 8;
  constexpr int KSTEPS = D / 16, DBLOCKS = D / 8;

  extern __shared__ unsigned char smem_dyn[];
  // 1024-byte alignment for the swizzled stages
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* stages = base;
  bf16* qs = reinterpret_cast<bf16*>(base + TD_STAGES * STAGE_BYTES);
  bf16* new_kv = qs + 16 * QROW;                               // fused rotation: [16 tokens][K, V][D]
  TdStageHeader* headers = reinterpret_cast<TdStageHeader*>(new_kv + 16 * 2 * D);
  unsigned long long* full_bar = reinterpret_cast<unsigned long long*>(headers + TD_STAGES);
  unsigned long long* empty_bar = full_bar + TD_STAGES;
  int* abort_flag = reinterpret_cast<int*>(empty_bar + TD_STAGES);
  // q and the new tokens' keys and values are dead once an item's last tile is done: the four consumer
  // warps merge through that memory, four rows at a time (the stages belong to the next item by then)
  float* merge_o = reinterpret_cast<float*>(qs);                // [4 warps][4 rows][D]
  float* merge_ml = merge_o + TD_CONSUMERS * 4 * D;             // [4 warps][4 rows][2]
  static_assert(16 * QROW * 2 + 16 * 2 * D * 2 >= (TD_CONSUMERS * 4 * D + TD_CONSUMERS * 4 * 2) * 4, "merge area");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < TD_STAGES; ++s) {
      kvb_mbar_init(&full_bar[s], 1);
      kvb_mbar_init(&empty_bar[s], TD_GROUP_WARPS);
    }
    *abort_flag = 0;
    kvb_mbar_init_fence();
  }
  __syncthreads();

  if (warp == TD_CONSUMERS) {
    // ---------------- producer ----------------
    // The whole warp walks the block's work items and, inside an item, its tiles; the ring of stages
    // runs on from one item into the next, so the first tiles of the next item are on their way while
    // the consumers still merge and store the last one.  The first item is the block's index; with a
    // work counter the following ones are taken from it (blocks stay until the work is gone), else
    // there is one item a block.  Page ids are fetched 32 table entries at a time, one lane each (a
    // coalesced load), a batch ahead of their use, so no copy waits on a table lookup.  Lane 0 owns
    // the barriers and writes the headers; lanes 0..pages_per_tile-1 each issue one page's copies.
    const int ppt = TD_KEYS / p.page_size;            // pages per tile: 1, 2, 4 or 8
    bool waited = false, reached_end = false;
    int g = 0;                                        // stages pushed so far
    int item = blockIdx.x;
    while (true) {
      if (item >= p.total_items) item = -1;
      TdStageHeader h;
      h.item = -1; h.it = 0; h.num_tiles = 0; h.q_begin = 0; h.q_len = 0; h.context = 0; h.key_lo = 0; h.key_hi = 0;
      if (item >= 0) h = td_describe_item(p, item);
      const int req = item >= 0 ? item / (p.KVH * p.num_splits) : 0;
      const int kvh = item >= 0 ? (item / p.num_splits) % p.KVH : 0;
      const int tile_begin = h.key_lo / TD_KEYS;
      const int* pages = p.table + (size_t)req * p.table_stride;
      const int first_entry = tile_begin * ppt;
      const int total_entries = h.num_tiles * ppt;
      const int key_hi = h.key_hi;
      auto fetch = [&](int entry) -> int {             // table entry `entry` of this item, 0 beyond it
        if (entry >= total_entries) return 0;
        const int index = first_entry + entry;
        if (index >= p.table_stride || index * p.page_size >= key_hi) return 0;
        const int page = pages[index];
        if (page < 0 || page >= p.num_pages) {
          atomicOr(p.status, KVB_STATUS_BAD_PAGE);
          return 0;
        }
        return page;
      };
      int cur = fetch(lane), nxt = fetch(32 + lane);
      // an item without keys (an empty split) and the end of the work still get a stage: a header alone
      const int pushes = h.num_tiles > 0 ? h.num_tiles : 1;
      int ok = 1;
      for (int it = 0; it < pushes && ok; ++it, ++g) {
        const int stage = g % TD_STAGES;
        const bool data = h.num_tiles > 0;
        const int e0 = it * ppt;
        // a tile that holds keys written in this step by a kernel in front (with the cache write done
        // here, the consumers lay those keys over the tile themselves)
        if (data && !waited && p.k_cache == nullptr && (tile_begin + it + 1) * TD_KEYS > h.context) {
          kvb_grid_wait();
          waited = true;
        }
        if (e0 > 0 && (e0 & 31) == 0) {                 // crossed into the next batch of entries
          cur = nxt;
          nxt = fetch(e0 + 32 + lane);
        }
        if (lane == 0) {
          if (g >= TD_STAGES && !kvb_mbar_wait<TD_SPIN_LIMIT, 64>(&empty_bar[stage], ((g / TD_STAGES) & 1) ^ 1)) {
            atomicOr(p.status, KVB_STATUS_WAIT_TIMEOUT);
            atomicExch(abort_flag, 1);
            ok = 0;
          }
          if (ok && *reinterpret_cast<volatile int*>(abort_flag)) ok = 0;
          if (ok) {
            h.it = it;
            headers[stage] = h;                         // released to the consumers by the arrival below
            if (data) kvb_mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
            else kvb_mbar_arrive(&full_bar[stage]);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        if (data) {
          const int page = __shfl_sync(0xffffffffu, cur, (e0 + lane) & 31);
          if (lane < ppt) {
            unsigned char* kdst = stages + stage * STAGE_BYTES;
            unsigned char* vdst = kdst + KV_BYTES;
            const int row = (page * p.KVH + kvh) * p.page_size * HALVES;   // in rows of 64 elements
            const int dst_off = lane * p.page_size * HALVES * 128;
            kvb_tma_2d(kdst + dst_off, &k_map, 0, row, &full_bar[stage]);     // one contiguous page of a head
            kvb_tma_2d(vdst + dst_off, &v_map, 0, row, &full_bar[stage]);
          }
        }
      }
      if (!ok) break;
      if (item < 0) {
        reached_end = true;
        break;
      }
      if (p.work == nullptr) {
        item = p.total_items;                           // one item a block: the end comes next
      } else {
        // the counter is shared with the launch in front if that is this kernel too: not before it is done
        if (!waited) {
          kvb_grid_wait();
          waited = true;
        }
        int next = 0;
        if (lane == 0) next = gridDim.x + atomicAdd(&p.work[0], 1);
        item = __shfl_sync(0xffffffffu, next, 0);
      }
    }
    if (!waited) kvb_grid_wait();
    // the last block to see the end of the work puts the counters back for the next launch
    if (p.work != nullptr && reached_end && lane == 0) {
      __threadfence();
      if (atomicAdd(&p.work[1], 1) == (int)gridDim.x - 1) {
        p.work[0] = 0;
        p.work[1] = 0;
        __threadfence();
      }
    }
    // on an aborted run, let the copies already issued land before the block may exit
    if (lane == 0 && *reinterpret_cast<volatile int*>(abort_flag)) {
      for (int s = max(0, g - TD_STAGES); s < g; ++s)
        kvb_mbar_wait<TD_SPIN_LIMIT, 64>(&full_bar[s % TD_STAGES], (s / TD_STAGES) & 1);
    }
    return;
  }

  // ---------------- consumers ----------------
  // They follow the headers of the ring: the first tile of an item sets the item up (q rows into
  // shared memory, rotated here if asked; this step's keys and values into the cache), every tile is
  // scored and accumulated, the last one is followed by the merge of the four warps and the store.
  float o[DBLOCKS][4];
  float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};
  unsigned qf[KSTEPS][4];
  int row_pos[2] = {0, 0};
  bool row_valid[2] = {false, false};
  int req = 0, kvh = 0, split = 0, q_begin = 0, q_len = 0, context = 0, key_lo = 0, key_hi = 0, tile_begin = 0,
      rows_total = 0;
  bool waited = false;
  const int wkey = warp * 16;
  auto begin_item = [&](const TdStageHeader& h) {
    // ---- a new item ----
    req = h.item / (p.KVH * p.num_splits);
    const int rest = h.item - req * (p.KVH * p.num_splits);
    kvh = rest / p.num_splits;
    split = rest - kvh * p.num_splits;
    q_begin = h.q_begin; q_len = h.q_len; context = h.context; key_lo = h.key_lo; key_hi = h.key_hi;
    tile_begin = key_lo / TD_KEYS;
    rows_total = min(q_len * p.G, 16);
    if (!waited) {
      kvb_grid_wait();                 // q is the output of the kernels in front
      kvb_trace_scope__.after_wait();
      waited = true;
    }
    // query rows -> padded shared memory (flat row r -> token r / G, head kvh*G + r % G), rotated on
    // the way when the rotation is done here: an item is the two 16-byte pieces (d, d + D/2)
    constexpr int PAIRS = D / 16;
    for (int i = threadIdx.x; i < 16 * PAIRS; i += TD_CONSUMERS * 32) {
      const int r = i / PAIRS, gq = i % PAIRS;
      Vec16<bf16> lo, hi;
      lo.raw = make_uint4(0, 0, 0, 0);
      hi.raw = make_uint4(0, 0, 0, 0);
      if (r < rows_total) {
        const int token = q_begin + r / p.G, head = kvh * p.G + r % p.G;
        const bf16* x = p.q + (size_t)token * p.q_stride + (size_t)head * D + gq * 8;
        lo.load(x);
        hi.load(x + D / 2);
        if (p.cos_sin != nullptr) {
          const float2* cs = p.cos_sin + (size_t)token * (D / 2) + gq * 8;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float2 t = cs[e];
            const float a = lo.get(e), b = hi.get(e);
            lo.set(e, a * t.x - b * t.y);
            hi.set(e, b * t.x + a * t.y);
          }
        }
      }
      *reinterpret_cast<uint4*>(qs + r * QROW + gq * 8) = lo.raw;
      *reinterpret_cast<uint4*>(qs + r * QROW + D / 2 + gq * 8) = hi.raw;
    }
    // this step's keys and values whose positions fall into this item's key range: rotate the key,
    // write both into the cache, keep them to lay over the tile that holds their (old) slots
    if (p.k_cache != nullptr) {
      const int new_tokens = q_len < 16 ? q_len : 16;
      // (dealt out from the last thread downwards: the first threads are the ones with query rows to
      // fetch, and the two fetches then wait for memory side by side instead of one after the other)
      for (int i = TD_CONSUMERS * 32 - 1 - (int)threadIdx.x; i < new_tokens * 2 * PAIRS; i += TD_CONSUMERS * 32) {
        const int t = i / (2 * PAIRS), which = (i / PAIRS) & 1, gq = i % PAIRS;   // which: 0 key, 1 value
        const int pos = context + t;
        if (pos < key_lo || pos >= key_hi) continue;
        const int token = q_begin + t;
        const bf16* x = (which ? p.v_new : p.k_new) + (size_t)token * p.q_stride + (size_t)kvh * D + gq * 8;
        Vec16<bf16> lo, hi;
        lo.load(x);
        hi.load(x + D / 2);
        if (!which && p.cos_sin != nullptr) {
          const float2* cs = p.cos_sin + (size_t)token * (D / 2) + gq * 8;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float2 c = cs[e];
            const float a = lo.get(e), b = hi.get(e);
            lo.set(e, a * c.x - b * c.y);
            hi.set(e, b * c.x + a * c.y);
          }
        }
        bf16* keep = new_kv + ((size_t)t * 2 + which) * D + gq * 8;
        *reinterpret_cast<uint4*>(keep) = lo.raw;
        *reinterpret_cast<uint4*>(keep + D / 2) = hi.raw;
        const int page = p.table[(size_t)req * p.table_stride + pos / p.page_size];
        if (page <= 0 || page >= p.num_pages) {
          atomicOr(p.status, KVB_STATUS_BAD_PAGE);
        } else {
          bf16* dst = (which ? p.v_cache : p.k_cache) +
                      (((size_t)page * p.KVH + kvh) * p.page_size + pos % p.page_size) * D + gq * 8;
          lo.store(dst);
          hi.store(dst + D / 2);
        }
      }
    }
    asm volatile("bar.sync 1, %0;\n" ::"n"(TD_CONSUMERS * 32));
#pragma unroll
    for (int k = 0; k < KSTEPS; ++k) {
      const int r = (lane & 7) + 8 * ((lane >> 3) & 1);
      const int c = k * 16 + 8 * (lane >> 4);
      td_ldmatrix_x4(qf[k], kvb_smem(qs + r * QROW + c));
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int r = (lane >> 2) + 8 * hh;
      row_valid[hh] = r < rows_total;
      row_pos[hh] = context + (row_valid[hh] ? r / p.G : 0);
      row_max[hh] = -INFINITY;
      row_sum[hh] = 0.0f;
    }
#pragma unroll
    for (int j = 0; j < DBLOCKS; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
  };
  // The block's first item is its index: q is loaded (and this step's keys written) while the first
  // tiles are on their way.  Later items are known from the header of their first stage.
  begin_item(td_describe_item(p, blockIdx.x));
  for (int g = 0;; ++g) {
    const int stage = g % TD_STAGES;
    if (!kvb_mbar_wait<TD_SPIN_LIMIT, 64>(&full_bar[stage], (g / TD_STAGES) & 1)) {
      atomicOr(p.status, KVB_STATUS_WAIT_TIMEOUT);
      atomicExch(abort_flag, 1);
      break;
    }
    const TdStageHeader h = headers[stage];
    if (h.item < 0) break;                              // the end of the work
    const int it = h.it;
    if (it == 0 && g > 0) begin_item(h);
    if (h.num_tiles > 0) {
      // ---- one tile of 64 keys ----
      const unsigned kbase = kvb_smem(stages + stage * STAGE_BYTES);
      const unsigned vbase = kbase + KV_BYTES;
      if (p.k_cache != nullptr) {
        // a tile that holds slots of this step's tokens: lay the fresh keys and values over them
        const int tile_lo = (tile_begin + it) * TD_KEYS;
        const int first_new = max(max(context, key_lo), tile_lo), end_new = min(min(context + q_len, key_hi), tile_lo + TD_KEYS);
        if (first_new < end_new) {
          const int count = (end_new - first_new) * 2 * (D / 8);
          for (int i = threadIdx.x; i < count; i += TD_CONSUMERS * 32) {
            const int t = i / (2 * (D / 8)), which = (i / (D / 8)) & 1, chunk = i % (D / 8);
            const int pos = first_new + t;
            const uint4 v = *reinterpret_cast<const uint4*>(new_kv + ((size_t)(pos - context) * 2 + which) * D + chunk * 8);
            unsigned char* area = stages + stage * STAGE_BYTES + (which ? KV_BYTES : 0);
            *reinterpret_cast<uint4*>(area + swz<HALVES>(pos - tile_lo, chunk * 8)) = v;
          }
          kvb_fence_async_shared();   // a later copy may reuse the stage
          asm volatile("bar.sync 1, %0;\n" ::"n"(TD_CONSUMERS * 32));
        }
      }
      float s[2][4], s2[2][4];  // two accumulation chains (even and odd k-steps) halve the latency
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
        s2[j][0] = s2[j][1] = s2[j][2] = s2[j][3] = 0.0f;
      }
#pragma unroll
      for (int k = 0; k < KSTEPS; ++k) {
        unsigned kb[4];
        const int key = wkey + (lane & 7) + 8 * (lane >> 4);
        const int d = k * 16 + 8 * ((lane >> 3) & 1);
        td_ldmatrix_x4(kb, kbase + swz<HALVES>(key, d));
        if (k & 1) {
          td_mma(s2[0], qf[k], kb[0], kb[1]);
          td_mma(s2[1], qf[k], kb[2], kb[3]);
        } else {
          td_mma(s[0], qf[k], kb[0], kb[1]);
          td_mma(s[1], qf[k], kb[2], kb[3]);
        }
      }
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[j][e] += s2[j][e];
      float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int hh = e >> 1;
          const int key = (tile_begin + it) * TD_KEYS + wkey + j * 8 + (lane & 3) * 2 + (e & 1);
          const bool seen = row_valid[hh] && key >= key_lo && key < key_hi && key <= row_pos[hh] &&
                            (p.window <= 0 || key > row_pos[hh] - p.window);
          const float v = seen ? s[j][e] * p.scale_log2 : -INFINITY;
          s[j][e] = v;
          tile_max[hh] = fmaxf(tile_max[hh], v);
        }
      }
      float correction[2];
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        float m = tile_max[hh];
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
        const float new_max = fmaxf(row_max[hh], m);
        correction[hh] = (row_max[hh] == -INFINITY) ? 0.0f : exp2f(row_max[hh] - new_max);
        row_max[hh] = new_max;
        row_sum[hh] *= correction[hh];
      }
#pragma unroll
      for (int j = 0; j < DBLOCKS; ++j) {
        o[j][0] *= correction[0]; o[j][1] *= correction[0];
        o[j][2] *= correction[1]; o[j][3] *= correction[1];
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int hh = e >> 1;
          const float pv = (s[j][e] == -INFINITY) ? 0.0f : exp2f(s[j][e] - row_max[hh]);
          s[j][e] = pv;
          row_sum[hh] += pv;
        }
      }
      unsigned pa[4];
      pa[0] = td_pack(s[0][0], s[0][1]);
      pa[1] = td_pack(s[0][2], s[0][3]);
      pa[2] = td_pack(s[1][0], s[1][1]);
      pa[3] = td_pack(s[1][2], s[1][3]);
#pragma unroll
      for (int j = 0; j < DBLOCKS; j += 2) {
        unsigned vb[4];
        const int key = wkey + (lane & 7) + 8 * ((lane >> 3) & 1);
        const int d = j * 8 + 8 * (lane >> 4);
        td_ldmatrix_x4_trans(vb, vbase + swz<HALVES>(key, d));
        td_mma(o[j], pa, vb[0], vb[1]);
        td_mma(o[j + 1], pa, vb[2], vb[3]);
      }
    }
    __syncwarp();
    if (lane == 0) kvb_mbar_arrive(&empty_bar[stage]);
    if (it + 1 < h.num_tiles) continue;

    // ---- the item's last tile is done: merge the four warps (four rows at a time) and store ----
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      row_sum[hh] += __shfl_xor_sync(0xffffffffu, row_sum[hh], 1);
      row_sum[hh] += __shfl_xor_sync(0xffffffffu, row_sum[hh], 2);
    }
    const int chunks = (rows_total + 3) / 4;
    for (int c = 0; c < chunks; ++c) {
      // all warps are past their last use of q and of the new keys (first chunk) or of the chunk before
      asm volatile("bar.sync 1, %0;\n" ::"n"(TD_CONSUMERS * 32));
      const int hh = c >> 1;
      if (((lane >> 4) & 1) == (c & 1)) {               // lanes that hold rows [4c, 4c + 4)
        const int r4 = (lane >> 2) & 3;
#pragma unroll
        for (int j = 0; j < DBLOCKS; ++j) {
          float* dst = merge_o + ((size_t)(warp * 4 + r4)) * D + j * 8 + (lane & 3) * 2;
          dst[0] = hh ? o[j][2] : o[j][0];
          dst[1] = hh ? o[j][3] : o[j][1];
        }
        if ((lane & 3) == 0) {
          merge_ml[(warp * 4 + r4) * 2 + 0] = hh ? row_max[1] : row_max[0];
          merge_ml[(warp * 4 + r4) * 2 + 1] = hh ? row_sum[1] : row_sum[0];
        }
      }
      asm volatile("bar.sync 1, %0;\n" ::"n"(TD_CONSUMERS * 32));
      const int rows_here = min(4, rows_total - 4 * c);
      // a thread takes four neighbouring columns of one row (D / 4 threads a row)
      const int r4 = threadIdx.x / (D / 4), d = (threadIdx.x % (D / 4)) * 4, r = 4 * c + r4;
      if (r4 < rows_here) {
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < TD_CONSUMERS; ++w) m = fmaxf(m, merge_ml[(w * 4 + r4) * 2]);
        float total = 0.0f;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int w = 0; w < TD_CONSUMERS; ++w) {
          const float mw = merge_ml[(w * 4 + r4) * 2];
          const float f = (mw == -INFINITY) ? 0.0f : exp2f(mw - m);
          total += merge_ml[(w * 4 + r4) * 2 + 1] * f;
          const float4 part = *reinterpret_cast<const float4*>(merge_o + ((size_t)(w * 4 + r4)) * D + d);
          acc.x += part.x * f; acc.y += part.y * f; acc.z += part.z * f; acc.w += part.w * f;
        }
        if (p.num_splits == 1) {
          const int token = q_begin + r / p.G, head = kvh * p.G + r % p.G;
          if (!(total > 0.0f)) { acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f); total = 1.0f; }
          __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x / total, acc.y / total), hi = __floats2bfloat162_rn(acc.z / total, acc.w / total);
          uint2 packed;
          packed.x = *reinterpret_cast<unsigned*>(&lo);
          packed.y = *reinterpret_cast<unsigned*>(&hi);
          *reinterpret_cast<uint2*>(p.out + (size_t)token * p.out_stride + (size_t)head * D + d) = packed;
        } else {
          const size_t slot = ((size_t)req * p.KVH + kvh) * p.num_splits + split;
          *reinterpret_cast<float4*>(p.partial_o + (slot * 16 + r) * D + d) = acc;
          if (d == 0) {
            p.partial_ml[(slot * 16 + r) * 2 + 0] = m;
            p.partial_ml[(slot * 16 + r) * 2 + 1] = total;
          }
        }
      }
    }
    // the next item's q goes where the merge just read
    asm volatile("bar.sync 1, %0;\n" ::"n"(TD_CONSUMERS * 32));
  }
}

// Same merge of splits as the cp.async kernel's, for this kernel's scratch layout.
template <int D>
__global__ void flash_decode_combine_kernel(const DecodeParams p) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_DECODE_COMBINE);
  const int req = blockIdx.z, kvh = blockIdx.y;
  const int q_begin = p.query_start[req];
  const int rows_total = min((p.query_start[req + 1] - q_begin) * p.G, 16);
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = i / D, d = i % D;
  if (r >= rows_total) return;
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
  const int token = q_begin + r / p.G, head = kvh * p.G + r % p.G;
  p.out[(size_t)token * p.out_stride + (size_t)head * D + d] =
      __float2bfloat16_rn(total > 0.0f ? acc / total : 0.0f);
}

// ---- host side -----------------------------------------------------------------------------
// Writes a 128-byte tensor map describing one layer's K (or V) cache [pages, KVH, page, D] bf16
// as a 2-D tensor of 64-element rows [pages*KVH*page*(D/64) rows, 64 columns] with boxes of
// [page*(D/64) rows, 64 columns]: one box is the contiguous block of one page and kv head.
extern "C" int kvb_make_kv_tensor_map(void* map_out, const void* cache, long long num_pages, int KVH,
                                      int page_size, int D) {
  KVB_REQUIRE(D == 64 || D == 128, "kv tensor map: head_dim must be 64 or 128");
  KVB_REQUIRE(page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64,
              "kv tensor map: page size must be 8, 16, 32 or 64");
  KVB_REQUIRE(aligned16(cache), "kv tensor map: the cache must be 16-byte aligned");
  KvbEncodeTiledFn encode = kvb_encode_tiled_fn();
  KVB_REQUIRE(encode != nullptr, "kv tensor map: the driver does not export cuTensorMapEncodeTiled");
  alignas(64) CUtensorMap map;
  const int halves = D / 64;
  const cuuint64_t dims[2] = {64, (cuuint64_t)num_pages * KVH * page_size * halves};
  const cuuint64_t strides[1] = {64 * sizeof(bf16)};
  const cuuint32_t box[2] = {64, (cuuint32_t)(page_size * halves)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult rc = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides,
                             box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  KVB_REQUIRE(rc == CUDA_SUCCESS, "kv tensor map: cuTensorMapEncodeTiled failed");
  memcpy(map_out, &map, sizeof(map));
  return 0;
}

template <int D>
static int launch_decode_tma(const CUtensorMap& k_map, const CUtensorMap& v_map, const DecodeParams& p,
                             int max_rows, int blocks, cudaStream_t stream) {
  constexpr size_t SMEM = 1024 + TD_STAGES * 2 * TD_KEYS * D * 2 + 16 * (D + 8) * 2 +
                          16 * 2 * D * 2 +   // the new tokens' keys and values (fused rotation)
                          TD_STAGES * sizeof(TdStageHeader) + 2 * TD_STAGES * 8 + 16;
  static bool configured = false;
  if (!configured) {
    KVB_CHECK_CUDA(cudaFuncSetAttribute(flash_decode_tma_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)SMEM));
    configured = true;
  }
  dim3 grid(blocks);
  KVB_CHECK_CUDA(kvb_launch((flash_decode_tma_kernel<D>), dim3(grid), dim3(TD_THREADS), SMEM, stream, true, k_map, v_map, p));
  KVB_CHECK_LAUNCH();
  if (p.num_splits > 1) {
    const int rows = max_rows < 16 ? max_rows : 16;
    dim3 cgrid((rows * D + 127) / 128, p.KVH, p.num_reqs);
    KVB_CHECK_CUDA(kvb_launch((flash_decode_combine_kernel<D>), dim3(cgrid), dim3(128), 0, stream, true, p));
    KVB_CHECK_LAUNCH();
  }
  return 0;
}

extern "C" int kvb_flash_decode_tma(void* out, long long out_stride, const void* q, long long q_stride,
                                    const void* k_map_host, const void* v_map_host, const int* table,
                                    int table_stride, const int* query_start, const int* context_lens,
                                    int num_reqs, int max_query_len, int H, int KVH, int D, int page_size,
                                    int num_pages, float scale, int window, int num_splits, float* scratch,
                                    const float* cos_sin, void* k_cache, void* v_cache, int* work, int max_blocks,
                                    cudaStream_t stream) {
  if (num_reqs == 0) return 0;
  KVB_REQUIRE(D == 64 || D == 128, "decode attention (TMA): head_dim must be 64 or 128");
  KVB_REQUIRE((k_cache == nullptr) == (v_cache == nullptr), "decode attention (TMA): give both caches or none");
  KVB_REQUIRE(page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64,
              "decode attention (TMA): page size must be 8, 16, 32 or 64");
  KVB_REQUIRE(H > 0 && KVH > 0 && H % KVH == 0, "decode attention (TMA): H must be a multiple of KVH");
  KVB_REQUIRE(max_query_len * (H / KVH) <= 16, "decode attention (TMA): at most 16 rows per request and kv head");
  KVB_REQUIRE(num_splits <= KVB_MAX_SPLITS, "decode attention (TMA): at most 1024 splits");
  KVB_REQUIRE((long long)num_reqs * KVH * (num_splits < 1 ? 1 : num_splits) < (1ll << 30),
              "decode attention (TMA): batch too large for one launch");
  KVB_REQUIRE(aligned16(q) && (q_stride % 8) == 0, "decode attention (TMA): q must be 16-byte aligned");
  KVB_REQUIRE(aligned16(out) && (out_stride % 8) == 0, "decode attention (TMA): out must be 16-byte aligned");
  KVB_REQUIRE(k_map_host != nullptr && v_map_host != nullptr, "decode attention (TMA): tensor maps are missing");
  DecodeParams p;
  p.out = (bf16*)out; p.out_stride = out_stride;
  p.q = (const bf16*)q; p.q_stride = q_stride;
  p.table = table; p.table_stride = table_stride;
  p.query_start = query_start; p.context_lens = context_lens;
  p.num_reqs = num_reqs; p.H = H; p.KVH = KVH; p.G = H / KVH;
  p.page_size = page_size; p.num_pages = num_pages; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.num_splits = num_splits < 1 ? 1 : num_splits;
  KVB_REQUIRE(p.num_splits == 1 || scratch != nullptr, "decode attention (TMA): splits need scratch memory");
  p.partial_o = scratch;
  p.partial_ml = scratch ? scratch + (size_t)num_reqs * KVH * p.num_splits * 16 * D : nullptr;
  p.status = kvb_status_word();
  KVB_REQUIRE(p.status != nullptr, "decode attention (TMA): no status word");
  // q points at the qkv rows [q heads | k heads | v heads]
  p.cos_sin = (const float2*)cos_sin;
  p.k_new = (const bf16*)q + (size_t)H * D;
  p.v_new = (const bf16*)q + (size_t)(H + KVH) * D;
  p.k_cache = (bf16*)k_cache; p.v_cache = (bf16*)v_cache;
  alignas(64) CUtensorMap k_map, v_map;
  memcpy(&k_map, k_map_host, sizeof(CUtensorMap));
  memcpy(&v_map, v_map_host, sizeof(CUtensorMap));
  const int max_rows = max_query_len * p.G;
  // With a work counter and more items than `max_blocks`, that many blocks stay and share the items;
  // else one block an item.
  p.total_items = num_reqs * KVH * p.num_splits;
  const bool shared = work != nullptr && max_blocks > 0 && p.total_items > max_blocks;
  p.work = shared ? work : nullptr;
  const int blocks = shared ? max_blocks : p.total_items;
  if (D == 64) return launch_decode_tma<64>(k_map, v_map, p, max_rows, blocks, stream);
  return launch_decode_tma<128>(k_map, v_map, p, max_rows, blocks, stream);
}

KVB_TRACE_TU(attention_decode_tma)
