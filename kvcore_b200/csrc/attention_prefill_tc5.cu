// Paged flash attention for prompt portions on the 5th-generation tensor cores (sm_100a):
// tcgen05.mma with accumulators in tensor memory, operands staged by TMA.  bf16, head size 128.
//
// A block owns TWO tiles of 128 query rows of one (request, kv head), A and B, one behind the other;
// a row is a (token, query head of the group) pair, so the G heads that share a kv head reuse every
// K/V tile, and every K/V tile that TMA brings is used by both query tiles.  The block walks the
// keys in tiles of 128.  Eleven warps:
//   warps 0-3  softmax of tile A, warps 4-7 softmax of tile B: thread t of a warpgroup owns row t
//              of its tile (= TMEM lane t) and the whole of it, so nothing is exchanged between
//              threads.  Per key tile it reads its row of S = Q.K^T from tensor memory (tcgen05.ld,
//              128 columns), masks where the tile needs it, keeps a running maximum and sum in 32-bit,
//              writes P = exp2(...) as packed bf16 over the columns it read S from (tcgen05.st: the
//              A operand of the second product is read from tensor memory, so P never touches shared
//              memory), and rescales its row of O when its maximum moved by more than 2^8.
//              The two warps of a scheduler belong to different query tiles: while one waits for
//              tensor memory or for the tensor pipe, the other works.
//   warps 8, 9 producers of K and of V (separate, so that a wait for a V stage never holds back
//              the next K tile): each looks pages up in the block table (batched, a batch ahead)
//              and issues the tiled TMA copies (two 64-column boxes per page, 128-byte swizzle)
//              into its two-stage ring.
//   warp 10    one thread issues the MMAs, alternating between the tiles so that the products of one
//              run under the softmax of the other:
//                S_A(0), S_B(0); then per key tile j:  O_A += P_A(j).V(j), S_A(j+1) = Q_A.K(j+1)^T,
//                O_B += P_B(j).V(j), S_B(j+1) = Q_B.K(j+1)^T
//              (P from tensor memory, V from shared memory as an MN-major operand).  S_X(j+1) goes
//              into the columns that held S_X(j) and P_X(j): the tensor pipe takes its instructions
//              in order, so it has read P_X(j) by then.
// The query tiles come by TMA too when the group size divides 128 (a 4-D map over [token, kv head,
// head of the group, 64 columns] lands the rows of a tile in (token, head) order); otherwise the softmax
// threads copy their rows.
// mbarriers: q_full, k_full/k_empty, v_full/v_empty (TMA <-> MMA, two stages each), and per query tile
// s_full (MMA -> softmax), p_ready (softmax -> MMA), pv_done (MMA -> softmax, the last product).
// tcgen05.commit arrives on the barriers that follow MMAs.  Every wait is bounded: on a time-out the
// thread sets the WAIT_TIMEOUT status bit and the block drains and frees its tensor memory before it
// returns.
//
// Tensor memory: 512 columns = S_A [0,128) | S_B [128,256) | O_A [256,384) | O_B [384,512); P_X lies
// over the first 64 columns of S_X (two bf16 a column).
// Shared memory: Q_A, Q_B 32 KB each | K 2x32 KB | V 2x32 KB (all 1024-byte aligned, 128B swizzle).
#include <cuda.h>
#include <string.h>

#include "common.cuh"
#include "sm100.cuh"

#define T5_BM 128
#define T5_BN 128
#define T5_D 128
#define T5_THREADS 352
#define T5_SPIN_LIMIT (1u << 20)
#define T5_HALF_BYTES (128 * 128)        // one 64-column half of a 128-row operand tile
#define T5_TILE_BYTES (2 * T5_HALF_BYTES)

struct Tc5Params {
  bf16* out; long long out_stride;
  const bf16* q; long long q_stride;
  const int* table; int table_stride;
  const int* query_start; const int* context_lens;
  int num_reqs, H, KVH, G, page_size, num_pages, window;
  float scale_log2;
  int* status;
  int q_by_tma;                // the query tiles are brought by TMA (q_map is valid)
};

// Byte offset of the 16-byte chunk `chunk16` (0..15 across the 128 columns) of row `r` in a
// [128 rows x 128 columns] bf16 operand tile stored as two swizzled 64-column halves.
__device__ __forceinline__ unsigned t5_chunk_off(int r, int chunk16) {
  return (unsigned)((chunk16 >> 3) * T5_HALF_BYTES + r * 128 + (((chunk16 & 7) ^ (r & 7)) << 4));
}

// max(a, b, c) in one instruction.
__device__ __forceinline__ float t5_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// (d0, d1) = (a0, a1) * b + c: one packed instruction for two elements.
__device__ __forceinline__ void t5_fma2(float& d0, float& d1, float a0, float a1, float b, float c) {
  asm("{.reg .b64 ra, rb, rc, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %4};\n mov.b64 rc, {%5, %5};\n"
      " fma.rn.f32x2 rd, ra, rb, rc;\n mov.b64 {%0, %1}, rd;}\n"
      : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
// (s0, s1) += (a0, a1), packed.
__device__ __forceinline__ void t5_add2(float& s0, float& s1, float a0, float a1) {
  asm("{.reg .b64 ra, rb, rd;\n mov.b64 ra, {%0, %1};\n mov.b64 rb, {%2, %3};\n add.rn.f32x2 rd, ra, rb;\n"
      " mov.b64 {%0, %1}, rd;}\n"
      : "+f"(s0), "+f"(s1) : "f"(a0), "f"(a1));
}

// P is cut to bf16, not rounded, and to make up for it every exponent gets log2(1 + 2^-9) added: the
// cut value is then off by at most half a bf16 step either way, as a rounded one would be, and it takes
// one byte permutation for two values instead of two additions and a permutation.  The row sum is taken
// of the same (raised) values, so the output is divided by sum / (1 + 2^-9).
#define T5_ROUND_SHIFT 0.0028150156f          // log2(1 + 2^-9)
#define T5_ROUND_FACTOR 1.001953125f          // 1 + 2^-9

__global__ void __launch_bounds__(T5_THREADS, 1)
flash_prefill_tc5_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                         const __grid_constant__ CUtensorMap q_map, const Tc5Params p) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_PREFILL_TC5);
  extern __shared__ __align__(1024) unsigned char t5_dyn[];
  unsigned char* base = t5_dyn;   // the swizzled tiles need 1024-byte alignment (checked below)
  unsigned char* q_smem = base;                              // tile A, tile B
  unsigned char* k_smem = q_smem + 2 * T5_TILE_BYTES;       // 2 stages
  unsigned char* v_smem = k_smem + 2 * T5_TILE_BYTES;       // 2 stages
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(v_smem + 2 * T5_TILE_BYTES);
  unsigned long long* k_full = bars;        // [2 stages]
  unsigned long long* k_empty = bars + 2;   // [2]
  unsigned long long* v_full = bars + 4;    // [2]
  unsigned long long* v_empty = bars + 6;   // [2]
  unsigned long long* s_full = bars + 8;    // [2 query tiles]
  unsigned long long* p_ready = bars + 10;  // [2 query tiles]
  unsigned long long* pv_done = bars + 12;  // [2 query tiles]
  unsigned long long* q_full = bars + 14;   // [1]: the query tiles have landed (TMA)
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 15);
  int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);

  // Later query tiles see more keys: they are handed out first, for all kv heads and requests (the
  // pair index is the slowest of the grid), so that the long blocks do not form the tail.
  const int req = blockIdx.y, kvh = blockIdx.x, pair = gridDim.z - 1 - blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_begin = p.query_start[req];
  const int q_len = p.query_start[req + 1] - q_begin;
  const int context = p.context_lens[req];
  const int rows_total = q_len * p.G;
  const int row0 = pair * 2 * T5_BM;
  if (row0 >= rows_total) return;  // whole block, before any barrier or allocation
  if (kvb_smem(base) & 1023u) {     // cannot happen with the alignment asked for; never run misaligned
    if (threadIdx.x == 0) atomicOr(p.status, KVB_STATUS_WAIT_TIMEOUT);
    return;
  }

  // keys of the two tiles: tile X sees [lo_X, hi_X); both walk the key tiles from tile_begin (the
  // first tile of A, whose rows come first), tile X through n_X of them
  const bool has_b = row0 + T5_BM < rows_total;
  const int last_row_a = min(row0 + T5_BM, rows_total) - 1;
  const int last_row_b = min(row0 + 2 * T5_BM, rows_total) - 1;
  const int first_pos_a = context + row0 / p.G;
  const int key_lo = p.window > 0 ? max(0, first_pos_a - p.window + 1) : 0;
  const int tile_begin = key_lo / T5_BN;
  const int n_a = (context + last_row_a / p.G + T5_BN) / T5_BN - tile_begin;             // >= 1
  const int n_b = has_b ? (context + last_row_b / p.G + T5_BN) / T5_BN - tile_begin : 0; // >= n_a when tile B exists
  const int num_tiles = max(n_a, n_b);
  const int key_hi = context + (has_b ? last_row_b : last_row_a) / p.G + 1;

  // the fifteen barriers, one thread each (p_ready counts the 128 threads of a softmax warpgroup)
  if (threadIdx.x < 15) {
    kvb_mbar_init(&bars[threadIdx.x], (threadIdx.x == 10 || threadIdx.x == 11) ? 128u : 1u);
    if (threadIdx.x == 0) *abort_flag = 0;
    kvb_mbar_init_fence();
  }
  if (warp == 8 && lane < 3) {   // the tensor maps are fetched while the block sets up
    const CUtensorMap* which = lane == 0 ? &k_map : lane == 1 ? &v_map : &q_map;
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<unsigned long long>(which)) : "memory");
  }
  if (warp == 10) {  // tensor memory: 512 columns for this block
    kvb_tc5_alloc(tmem_slot, 512u);
  }
  // Q rows -> shared memory in the swizzled K-major operand layout (thread t of warpgroup X: row t of tile X)
  if (warp < 8 && !p.q_by_tma) {
    const int r = threadIdx.x & 127, x = threadIdx.x >> 7;
    const int flat = row0 + x * T5_BM + r;
    const bool valid = flat < rows_total;
    const bf16* src = p.q + (size_t)(q_begin + (valid ? flat / p.G : 0)) * p.q_stride +
                      (size_t)(kvh * p.G + (valid ? flat % p.G : 0)) * T5_D;
    unsigned char* dst = q_smem + x * T5_TILE_BYTES;
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (valid) v = *reinterpret_cast<const uint4*>(src + c * 8);
      *reinterpret_cast<uint4*>(dst + t5_chunk_off(r, c)) = v;
    }
    kvb_fence_async_shared();  // generic writes -> visible to the MMA's reads
  }
  // the producers look their first pages up before the block meets, so that the first copies leave
  // right behind the barrier
  const int* pages = p.table + (size_t)req * p.table_stride;
  const int ppt = T5_BN / p.page_size;          // pages per tile: 2..16
  const int first_entry = tile_begin * ppt;
  const int total_entries = num_tiles * ppt;
  auto fetch = [&](int entry) -> int {
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
  int cur = 0, nxt = 0;
  if (warp == 8 || warp == 9) {
    cur = fetch(lane);
    nxt = fetch(32 + lane);
  }
  kvb_tc5_fence_before();
  __syncthreads();
  kvb_tc5_fence_after();
  const unsigned tmem_base = *tmem_slot;

  if (warp == 8 || warp == 9) {
    // ================= producers: warp 8 streams K tiles, warp 9 streams V tiles =================
    const bool is_k = warp == 8;
    const CUtensorMap* map = is_k ? &k_map : &v_map;
    unsigned char* ring = is_k ? k_smem : v_smem;
    unsigned long long* full = is_k ? k_full : v_full;
    unsigned long long* empty = is_k ? k_empty : v_empty;
    if (is_k && lane == 0 && p.q_by_tma) {
      // the query tiles: rows in (token, head of the group) order, 128 / G tokens a tile, as two boxes
      // of 64 columns each; tokens beyond the batch arrive as zeros
      const int tokens_per_tile = T5_BM / p.G;
      const int token0 = q_begin + row0 / p.G;
      kvb_mbar_expect_tx(q_full, (has_b ? 2u : 1u) * T5_TILE_BYTES);
      for (int x = 0; x < (has_b ? 2 : 1); ++x) {
        kvb_tma_4d(q_smem + x * T5_TILE_BYTES, &q_map, 0, 0, kvh, token0 + x * tokens_per_tile, q_full);
        kvb_tma_4d(q_smem + x * T5_TILE_BYTES + T5_HALF_BYTES, &q_map, 64, 0, kvh, token0 + x * tokens_per_tile, q_full);
      }
    }
    int issued = 0;
    for (int j = 0; j < num_tiles; ++j) {
      const int s = j & 1;
      const int e0 = j * ppt;
      if (e0 > 0 && (e0 & 31) == 0) {
        cur = nxt;
        nxt = fetch(e0 + 32 + lane);
      }
      const int page = __shfl_sync(0xffffffffu, cur, (e0 + lane) & 31);
      const int row = (page * p.KVH + kvh) * p.page_size;
      int ok = 1;
      if (lane == 0) {
        if (j >= 2 && !kvb_mbar_wait<T5_SPIN_LIMIT, 4096>(&empty[s], ((j >> 1) - 1) & 1)) ok = 0;
        if (ok && *reinterpret_cast<volatile int*>(abort_flag)) ok = 0;
        if (ok) kvb_mbar_expect_tx(&full[s], T5_TILE_BYTES);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane < ppt) {
        unsigned char* dst = ring + s * T5_TILE_BYTES + lane * p.page_size * 128;
        kvb_tma_2d(dst, map, 0, row, &full[s]);
        kvb_tma_2d(dst + T5_HALF_BYTES, map, 64, row, &full[s]);
      }
      issued = j + 1;
    }
    if (lane == 0 && issued < num_tiles) {
      atomicOr(p.status, KVB_STATUS_WAIT_TIMEOUT);
      atomicExch(abort_flag, 1);
    }
    if (lane == 0 && *reinterpret_cast<volatile int*>(abort_flag)) {
      // let the copies that were issued land before the block may exit
      for (int j = max(0, issued - 2); j < issued; ++j) kvb_mbar_wait<T5_SPIN_LIMIT, 4096>(&full[j & 1], (j >> 1) & 1);
      if (is_k && p.q_by_tma) kvb_mbar_wait<T5_SPIN_LIMIT, 4096>(q_full, 0);
    }
  } else if (warp == 10) {
    // ================= MMA issuer =================
    if (lane == 0) {
      // instruction descriptors: f32 accumulate, bf16 x bf16, M = 128, N = 128
      const unsigned idesc_s = kvb_tc5_idesc(T5_BM, T5_BN, false);   // A, B both K-major
      const unsigned idesc_pv = kvb_tc5_idesc(T5_BM, T5_BN, true);   // B (= V) MN-major
      bool ok = true;
      // The operand descriptors of a tile differ from step to step only in their address field (bits
      // 0-13, in units of 16 bytes; shared memory ends below 256 KB, so the field never overflows): the
      // six bases are made once and a step adds a constant.  This thread issues 32 MMAs per key tile and
      // is on the critical path of both query tiles: with the descriptors built per MMA it needed ~90
      // cycles an instruction, more than the 64 the tensor pipe takes.
      const unsigned long long q_desc[2] = {kvb_tc5_desc(kvb_smem(q_smem), 16, 1024),
                                            kvb_tc5_desc(kvb_smem(q_smem + T5_TILE_BYTES), 16, 1024)};
      const unsigned long long k_desc[2] = {kvb_tc5_desc(kvb_smem(k_smem), 16, 1024),
                                            kvb_tc5_desc(kvb_smem(k_smem + T5_TILE_BYTES), 16, 1024)};
      const unsigned long long v_desc[2] = {kvb_tc5_desc(kvb_smem(v_smem), T5_HALF_BYTES, 1024),
                                            kvb_tc5_desc(kvb_smem(v_smem + T5_TILE_BYTES), T5_HALF_BYTES, 1024)};
      auto issue_s = [&](int x, int j) {   // S_x(j) = Q_x . K(j)^T
        // 32 bytes (2 units) a step of 16 columns; after four steps on to the other 64-column half
        constexpr int HALF16 = T5_HALF_BYTES >> 4;
        kvb_tc5_mma8_ss<2, HALF16 - 6, 2, HALF16 - 6>(tmem_base + x * T5_BN, q_desc[x], k_desc[j & 1], idesc_s, 0u);
        kvb_tc5_commit(&s_full[x]);
      };
      auto issue_pv = [&](int x, int j) {  // O_x += P_x(j) . V(j): 16 keys per MMA (8 columns of P, 16 key rows of V)
        // 16 keys a step: 8 columns of P, 16 key rows (2,048 bytes = 128 units) of V
        kvb_tc5_mma8_ts<8, 128>(tmem_base + 256 + x * T5_D, tmem_base + x * T5_BN, v_desc[j & 1], idesc_pv, j > 0 ? 1u : 0u);
        kvb_tc5_commit(&pv_done[x]);
      };
      if (p.q_by_tma && !kvb_mbar_wait<T5_SPIN_LIMIT, 4096>(q_full, 0)) ok = false;
      if (ok && !kvb_mbar_wait<T5_SPIN_LIMIT, 4096>(&k_full[0], 0)) ok = false;
      if (ok) {
        kvb_tc5_fence_after();
        issue_s(0, 0);
        if (has_b) issue_s(1, 0);
        kvb_tc5_commit(&k_empty[0]);
      }
      int j = 0;
      // Pairs of key tiles well inside the block's run, where both query tiles are at work and nothing ends:
      // the ring places, barriers and phases of a pair are constants, so that this thread, which alone feeds
      // the tensor pipe, runs next to nothing between two groups of products.
      if (has_b) {
        unsigned ph = 0;
        for (; j + 3 < n_a && ok; j += 2, ph ^= 1u) {
#define T5_HALF_STEP(ST, PPAR, KPAR, ACC)                                                                  \
          {                                                                                               \
            if (!kvb_mbar_wait<T5_SPIN_LIMIT, 4096>(&v_full[ST], ph)) { ok = false; break; }              \
            if (!kvb_mbar_wait<T5_SPIN_LIMIT, 4096>(&p_ready[0], PPAR)) { ok = false; break; }            \
            kvb_tc5_fence_after();                                                                        \
            kvb_tc5_mma8_ts<8, 128>(tmem_base + 256, tmem_base, v_desc[ST], idesc_pv, ACC);               \
            kvb_tc5_commit(&pv_done[0]);                                                                  \
            if (!kvb_mbar_wait<T5_SPIN_LIMIT, 4096>(&k_full[(ST) ^ 1], KPAR)) { ok = false; break; }      \
            kvb_tc5_fence_after();                                                                        \
            kvb_tc5_mma8_ss<2, (T5_HALF_BYTES >> 4) - 6, 2, (T5_HALF_BYTES >> 4) - 6>(tmem_base, q_desc[0], k_desc[(ST) ^ 1], idesc_s, 0u); \
            kvb_tc5_commit(&s_full[0]);                                                                   \
            if (!kvb_mbar_wait<T5_SPIN_LIMIT, 4096>(&p_ready[1], PPAR)) { ok = false; break; }            \
            kvb_tc5_fence_after();                                                                        \
            kvb_tc5_mma8_ts<8, 128>(tmem_base + 256 + T5_D, tmem_base + T5_BN, v_desc[ST], idesc_pv, ACC); \
            kvb_tc5_commit(&pv_done[1]);                                                                  \
            kvb_tc5_commit(&v_empty[ST]);                                                                 \
            kvb_tc5_mma8_ss<2, (T5_HALF_BYTES >> 4) - 6, 2, (T5_HALF_BYTES >> 4) - 6>(tmem_base + T5_BN, q_desc[1], k_desc[(ST) ^ 1], idesc_s, 0u); \
            kvb_tc5_commit(&s_full[1]);                                                                   \
            kvb_tc5_commit(&k_empty[(ST) ^ 1]);                                                           \
          }
          T5_HALF_STEP(0, 0u, ph, j > 0 ? 1u : 0u)
          T5_HALF_STEP(1, 1u, ph ^ 1u, 1u)
#undef T5_HALF_STEP
        }
      }
      for (; j < num_tiles && ok; ++j) {
        const int st = j & 1, par = (j >> 1) & 1;
        const bool more = j + 1 < num_tiles;
        if (!kvb_mbar_wait<T5_SPIN_LIMIT, 4096>(&v_full[st], par)) { ok = false; break; }
        if (j < n_a) {
          if (!kvb_mbar_wait<T5_SPIN_LIMIT, 4096>(&p_ready[0], j & 1)) { ok = false; break; }
          kvb_tc5_fence_after();
          issue_pv(0, j);
        }
        if (more && !kvb_mbar_wait<T5_SPIN_LIMIT, 4096>(&k_full[st ^ 1], ((j + 1) >> 1) & 1)) { ok = false; break; }
        if (more) kvb_tc5_fence_after();
        if (j + 1 < n_a) issue_s(0, j + 1);
        if (j < n_b) {
          if (!kvb_mbar_wait<T5_SPIN_LIMIT, 4096>(&p_ready[1], j & 1)) { ok = false; break; }
          kvb_tc5_fence_after();
          issue_pv(1, j);
        }
        kvb_tc5_commit(&v_empty[st]);
        if (more) {
          if (j + 1 < n_b) issue_s(1, j + 1);
          kvb_tc5_commit(&k_empty[st ^ 1]);
        }
      }
      if (!ok) {
        atomicOr(p.status, KVB_STATUS_WAIT_TIMEOUT);
        atomicExch(abort_flag, 1);
      }
    }
  } else {
    // ================= softmax: thread t of warpgroup X owns row t of query tile X =================
    // The row of S is read from TMEM once and kept in registers: pass 1 finds its maximum, pass 2 forms
    // P = 2^(s*scale - m), sums it and writes it as bf16 over the columns S was read from.  Masks are
    // applied only on tiles that need them (the diagonal, a window, rows beyond the batch).  The running
    // maximum m is moved (and O rescaled) only when some row of the warp would grow by more than 2^8:
    // until then P may exceed 1, which bf16 and the 32-bit sums hold easily, and O and the row sum stay
    // consistent because both are taken against the same m.
    const int r = threadIdx.x & 127;
    const int x = threadIdx.x >> 7;                       // which query tile
    const int n_mine = x == 0 ? n_a : n_b;
    const int flat = row0 + x * T5_BM + r;
    const bool row_valid = flat < rows_total;
    const int pos = context + (row_valid ? flat / p.G : 0);
    const int row_lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int first_pos = context + (row0 + x * T5_BM) / p.G;   // position of the tile's first row
    const unsigned lane_addr = ((unsigned)((warp & 3) * 32) << 16);
    const bool ragged = row0 + (x + 1) * T5_BM > rows_total;     // the tile holds rows beyond the batch
    const unsigned s_addr = tmem_base + lane_addr + x * T5_BN;
    const unsigned o_addr = tmem_base + lane_addr + 256 + x * T5_D;
    float row_max = -INFINITY, row_sum = 0.0f;            // row_max in the scaled (log2) domain
    bool ok = true;
    for (int j = 0; j < n_mine; ++j) {
      if (!kvb_mbar_wait<T5_SPIN_LIMIT, 4096>(&s_full[x], j & 1)) { ok = false; break; }
      kvb_tc5_fence_after();
      const int key0 = (tile_begin + j) * T5_BN;
      const bool need_mask = ragged || p.window > 0 || key0 + T5_BN - 1 > first_pos;
      float s[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) kvb_tc5_ld32(s_addr + c * 32, s[c]);
      kvb_tc5_wait_ld();
      // ---- pass 1: maximum of the raw scores of the row ----
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (need_mask) {
        // keys of this tile the row sees: indices [lo, hi] within the tile (none if the row is beyond the batch)
        const int hi = row_valid ? pos - key0 : -1;
        const int lo = row_lo - key0;
        if (p.window > 0) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i > hi || c * 32 + i < lo) s[c][i] = -INFINITY;
          }
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i > hi) s[c][i] = -INFINITY;
          }
        }
      }
      {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) mx[(i >> 1) & 3] = t5_max3(mx[(i >> 1) & 3], s[c][i], s[c][i + 1]);
        }
      }
      const float tile_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;   // scale > 0; -inf stays -inf
      const float new_max = fmaxf(row_max, tile_max);
      const bool grows = new_max > row_max + 8.0f || (row_max == -INFINITY && new_max > -INFINITY);
      const bool move = __any_sync(0xffffffffu, grows);
      float correction = 1.0f;
      if (move) {
        correction = (row_max == -INFINITY) ? 0.0f : exp2f(row_max - new_max);
        row_max = new_max;
      }
      const float shift = ((row_max == -INFINITY) ? 0.0f : -row_max) + T5_ROUND_SHIFT;
      // ---- pass 2: P = 2^(s*scale - m), row sum, packed bf16 into tensor memory, 32 keys at a time ----
      // (the softmax warps are bound by instruction issue, not by the exp2 unit: the scaling and the sums
      // are packed two elements an instruction, and the conversion is one byte permutation for two)
      float sm[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float packed[16];                            // 32 keys, two bf16 a register
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float a0, a1, e0, e1;
          t5_fma2(a0, a1, s[c][i], s[c][i + 1], p.scale_log2, shift);      // masked entries stay -inf
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(a0));
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(a1));
          t5_add2(sm[i & 2], sm[(i & 2) + 1], e0, e1);
          // two bf16 in a register, the lower key in the lower half (cut: see T5_ROUND_SHIFT)
          packed[i / 2] = __uint_as_float(__byte_perm(__float_as_uint(e0), __float_as_uint(e1), 0x7632));
        }
        // P(j) lies over the first half of the columns S(j) was read from; S(j+1) is written there only
        // after the tensor pipe has taken P(j)
        kvb_tc5_st16(s_addr + c * 16, packed);
      }
      row_sum = row_sum * correction + ((sm[0] + sm[1]) + (sm[2] + sm[3]));
      if (move && j > 0) {
        // rescale this thread's row of O.  The product P(j-1).V(j-1) has landed: it was issued before
        // S(j), whose arrival this thread has seen, and the tensor pipe finishes in order.
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          float o[32];
          kvb_tc5_ld32(o_addr + c * 32, o);
          kvb_tc5_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= correction;
          kvb_tc5_st32(o_addr + c * 32, o);
        }
      }
      kvb_tc5_wait_st();
      kvb_tc5_fence_before();
      kvb_mbar_arrive(&p_ready[x]);
    }
    if (ok && n_mine > 0 && !kvb_mbar_wait<T5_SPIN_LIMIT, 4096>(&pv_done[x], (n_mine - 1) & 1)) ok = false;
    if (ok && n_mine > 0) {
      kvb_tc5_fence_after();
      const float inv = row_sum > 0.0f ? T5_ROUND_FACTOR / row_sum : 0.0f;
      bf16* dst = nullptr;
      if (row_valid)
        dst = p.out + (size_t)(q_begin + flat / p.G) * p.out_stride + (size_t)(kvh * p.G + flat % p.G) * T5_D;
      float o[4][32];                               // the whole row at once: one round trip to tensor memory
#pragma unroll
      for (int c = 0; c < 4; ++c) kvb_tc5_ld32(o_addr + c * 32, o[c]);
      kvb_tc5_wait_ld();
      if (row_valid) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 packed;
            __nv_bfloat162 t0 = __floats2bfloat162_rn(o[c][i] * inv, o[c][i + 1] * inv);
            __nv_bfloat162 t1 = __floats2bfloat162_rn(o[c][i + 2] * inv, o[c][i + 3] * inv);
            __nv_bfloat162 t2 = __floats2bfloat162_rn(o[c][i + 4] * inv, o[c][i + 5] * inv);
            __nv_bfloat162 t3 = __floats2bfloat162_rn(o[c][i + 6] * inv, o[c][i + 7] * inv);
            packed.x = *reinterpret_cast<unsigned*>(&t0);
            packed.y = *reinterpret_cast<unsigned*>(&t1);
            packed.z = *reinterpret_cast<unsigned*>(&t2);
            packed.w = *reinterpret_cast<unsigned*>(&t3);
            *reinterpret_cast<uint4*>(dst + c * 32 + i) = packed;
          }
        }
      }
    } else if (!ok) {
      atomicOr(p.status, KVB_STATUS_WAIT_TIMEOUT);
      atomicExch(abort_flag, 1);
    }
  }

  // ---- everyone meets; the allocating warp frees the tensor memory ----
  kvb_tc5_fence_before();
  __syncthreads();
  if (warp == 10) {
    kvb_tc5_fence_after();
    kvb_tc5_dealloc(tmem_base, 512u);
  }
}

// ---- host side -----------------------------------------------------------------------------
// Tensor map of one layer's K (or V) cache [pages, KVH, page, 128] bf16 as [rows, 128 columns] with
// boxes of [page rows, 64 columns] (one 64-column half of a page of a head), 128-byte swizzle.
extern "C" int kvb_make_kv_half_tensor_map(void* map_out, const void* cache, long long num_pages, int KVH,
                                           int page_size, int D) {
  KVB_REQUIRE(D == T5_D, "kv half tensor map: head_dim must be 128");
  KVB_REQUIRE(page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64,
              "kv half tensor map: page size must be 8, 16, 32 or 64");
  KVB_REQUIRE(aligned16(cache), "kv half tensor map: the cache must be 16-byte aligned");
  KvbEncodeTiledFn encode = kvb_encode_tiled_fn();
  KVB_REQUIRE(encode != nullptr, "kv half tensor map: the driver does not export cuTensorMapEncodeTiled");
  alignas(64) CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)num_pages * KVH * page_size};
  const cuuint64_t strides[1] = {(cuuint64_t)D * sizeof(bf16)};
  const cuuint32_t box[2] = {64, (cuuint32_t)page_size};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult rc = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides,
                             box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  KVB_REQUIRE(rc == CUDA_SUCCESS, "kv half tensor map: cuTensorMapEncodeTiled failed");
  memcpy(map_out, &map, sizeof(map));
  return 0;
}

// q [num_tokens, >= H * 128] bf16 with row stride q_stride (elements): the step's queries, rotated already.
extern "C" int kvb_flash_prefill_tc5(void* out, long long out_stride, const void* q, long long q_stride,
                                     const void* k_map_host, const void* v_map_host, const int* table,
                                     int table_stride, const int* query_start, const int* context_lens,
                                     int num_reqs, int max_query_len, int num_tokens, int H, int KVH, int D,
                                     int page_size, int num_pages, float scale, int window, cudaStream_t stream) {
  if (num_reqs == 0) return 0;
  KVB_REQUIRE(D == T5_D, "prefill attention (tcgen05): head_dim must be 128");
  KVB_REQUIRE(page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64,
              "prefill attention (tcgen05): page size must be 8, 16, 32 or 64");
  KVB_REQUIRE(H > 0 && KVH > 0 && H % KVH == 0, "prefill attention (tcgen05): H must be a multiple of KVH");
  KVB_REQUIRE(num_reqs <= 65535 && KVH <= 65535, "prefill attention (tcgen05): batch too large for one launch");
  KVB_REQUIRE(aligned16(q) && aligned16(out) && (q_stride % 8) == 0 && (out_stride % 8) == 0,
              "prefill attention (tcgen05): q and out must be 16-byte aligned");
  KVB_REQUIRE(k_map_host != nullptr && v_map_host != nullptr, "prefill attention (tcgen05): tensor maps are missing");
  Tc5Params p;
  p.out = (bf16*)out; p.out_stride = out_stride;
  p.q = (const bf16*)q; p.q_stride = q_stride;
  p.table = table; p.table_stride = table_stride;
  p.query_start = query_start; p.context_lens = context_lens;
  p.num_reqs = num_reqs; p.H = H; p.KVH = KVH; p.G = H / KVH;
  p.page_size = page_size; p.num_pages = num_pages; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = kvb_status_word();
  KVB_REQUIRE(p.status != nullptr, "prefill attention (tcgen05): no status word");
  alignas(64) CUtensorMap k_map, v_map, q_map;
  memcpy(&k_map, k_map_host, sizeof(CUtensorMap));
  memcpy(&v_map, v_map_host, sizeof(CUtensorMap));
  // The queries as [token][kv head][head of the group][128] with boxes of [128 / G tokens][1][G][64 columns]:
  // a box is one 64-column half of a query tile, its rows in (token, head) order.  Needs G to divide 128.
  memset(&q_map, 0, sizeof(q_map));
  p.q_by_tma = 0;
  if (T5_BM % p.G == 0 && num_tokens > 0) {
    KvbEncodeTiledFn encode = kvb_encode_tiled_fn();
    KVB_REQUIRE(encode != nullptr, "prefill attention (tcgen05): the driver does not export cuTensorMapEncodeTiled");
    const cuuint64_t dims[4] = {(cuuint64_t)T5_D, (cuuint64_t)p.G, (cuuint64_t)KVH, (cuuint64_t)num_tokens};
    const cuuint64_t strides[3] = {(cuuint64_t)T5_D * sizeof(bf16), (cuuint64_t)p.G * T5_D * sizeof(bf16),
                                   (cuuint64_t)q_stride * sizeof(bf16)};
    const cuuint32_t box[4] = {64, (cuuint32_t)p.G, 1, (cuuint32_t)(T5_BM / p.G)};
    const cuuint32_t elem[4] = {1, 1, 1, 1};
    const CUresult rc = encode(&q_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(q), dims, strides, box,
                               elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    KVB_REQUIRE(rc == CUDA_SUCCESS, "prefill attention (tcgen05): cuTensorMapEncodeTiled failed for the queries");
    p.q_by_tma = 1;
  }
  constexpr size_t SMEM = 6 * T5_TILE_BYTES + 16 * 8;
  static bool configured = false;
  if (!configured) {
    KVB_CHECK_CUDA(cudaFuncSetAttribute(flash_prefill_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
    configured = true;
  }
  const int max_rows = max_query_len * p.G;
  const int pairs = (max_rows + 2 * T5_BM - 1) / (2 * T5_BM);            // a block takes two query tiles
  KVB_REQUIRE(pairs <= 65535, "prefill attention (tcgen05): portion too long for one launch");
  dim3 grid(KVH, num_reqs, pairs);
  KVB_CHECK_CUDA(kvb_launch((flash_prefill_tc5_kernel), dim3(grid), dim3(T5_THREADS), SMEM, stream, true, k_map, v_map, q_map, p));
  KVB_CHECK_LAUNCH();
  return 0;
}

KVB_TRACE_TU(attention_prefill_tc5)
