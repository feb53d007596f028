// Weight-streaming linear layer for decode batches of 17 to 128 tokens on the 5th-generation
// tensor cores (sm_100a): out[M, N] = x[M, K] . W[N, K]^T (+ bias), bf16 in, 32-bit accumulate in
// tensor memory, K a multiple of 64.
//
// With this few tokens the layer is still one pass over the weight matrix, so the kernel is the
// streaming kernel of the smallest batches (gemm_stream.cu) with the product moved to tcgen05.mma.
// The tokens are the A operand: token m is lane m of the accumulator, the 256 weight rows of a
// tile are its columns.  A thread of the epilogue therefore holds one token's run of output rows,
// which is how the output, the residual and the gated pairs lie in memory: 16-byte stores, the
// sum of squares of a piece without a shuffle, gate and up of a pair in the same thread.
//
//  * A stage is the MT (32, 64 or 128) token rows of 64 k-values (4 to 16 KB) followed by 256 weight
//    rows of the same k-values (32 KB, ONE 2-D TMA box, 128-byte swizzle).  Five stages (four at
//    MT = 128): 160 KB of weights in flight per SM, which is what keeps DRAM busy.  The MMA always
//    reads 128 A rows; beyond MT they are the weight bytes that follow, and no one reads those lanes.
//  * One block per SM.  Stages are numbered tile by tile (k fastest) and dealt to the blocks as
//    equal contiguous ranges.  A tile that lies in one block's range is finished from tensor
//    memory.  A tile shared by P blocks: every block leaves its sums in scratch and raises a flag;
//    when all P flags are up, block i of the P adds rows [32 * floor(8 i / P), 32 * floor(8 (i+1) / P))
//    of all P parts in k order (the parts come into the idle stage memory by bulk copies, all in
//    flight together) and finishes those rows, so the fix-up traffic is spread over the blocks
//    that share the tile instead of landing on one owner.  The last block through a tile lowers
//    the flags again.  The result does not depend on timing.
//  * Warps: 0 producer (TMA), 1 MMA issuer (one thread; owns the tensor memory), 2-5 epilogue
//    (warp w reads accumulator lanes [32 (w mod 4), +32)), 6-9 (NORMED only) normalise each
//    stage's token rows in shared memory before the MMA reads them.
//  * Two accumulator buffers of 256 columns: the MMAs of the next tile run while the epilogue warps
//    finish the last one.
//  * Programmatic dependent launch: the whole ring of weight boxes is asked for before the wait
//    for the kernel in front.
//  * Epilogues as in gemm_stream.cu: plain, gated pairs (rows in runs of 8 gate, 8 up), residual
//    stream (adds into the residual in place and leaves sums of squares, here 32 columns a piece).
//
// Every wait is bounded (status bit WAIT_TIMEOUT; the block drains its copies, frees its tensor
// memory and returns).
#include <cuda.h>
#include <string.h>

#include "common.cuh"
#include "sm100.cuh"

#define TS_NT 256              // weight rows per tile: two MMA halves of 128
#define TS_KS 64               // k-values per stage
#define TS_W_BYTES (TS_NT * TS_KS * 2)
#define TS_EPI_WARPS 4
#define TS_NORM_WARPS 4
#define TS_THREADS ((2 + TS_EPI_WARPS) * 32)
#define TS_SPIN_LIMIT (1u << 22)
#define TS_NORM_W_BYTES (16 * 1024)
#define TS_MAX_TILES 4096      // done counters behind the flags

struct TsParams {
  void* out; int out_f32; long long ldo;
  const bf16* bias;
  int M, N, K;
  int n_tiles, kchunks, units;       // kchunks = K / 64; units = n_tiles * kchunks
  float* partial;                    // [blocks][2 slots][8 groups of 32 W rows][MT tokens][32]
  int* flags;                        // [blocks][2 slots] then [TS_MAX_TILES] counters; zero between launches
  int* status;
  const float* sumsq_in; int sumsq_pieces; const void* norm_weight; int norm_weight_f32; float eps;
  bf16* residual; float* sumsq_out;  // sumsq_out [M][ceil(N / 32)]
  int silu_pairs;
};

__device__ __forceinline__ float ts_round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// First stage of block b when `units` stages are dealt to `blocks` blocks, and the block that holds stage u.
__device__ __forceinline__ int ts_range_start(int units, int blocks, int b) {
  return (int)(((long long)units * b) / blocks);
}
__device__ __forceinline__ int ts_block_of(int units, int blocks, int u) {
  int b = (int)(((long long)u * blocks) / units);
  if (b >= blocks) b = blocks - 1;
  while (b + 1 < blocks && ts_range_start(units, blocks, b + 1) <= u) ++b;
  while (b > 0 && ts_range_start(units, blocks, b) > u) --b;
  return b;
}

// ---- epilogues -----------------------------------------------------------------------------
// Both take the sums of one token m for a run of output rows (W rows n), with the bias still to
// be added, and do one of: gated pairs, residual stream, plain store.  `vector_ok` says that the
// rows of out / residual may be written in 16-byte pieces.
struct TsOutput {
  bool vector_ok;     // 16-byte stores are aligned (leading dimensions and bases)
  int pieces;         // sums of squares per token: ceil(N / 32)
};

__device__ __forceinline__ unsigned ts_pack2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&v);
}
__device__ __forceinline__ float ts_silu_mul(float gate, float up) {
  // rounded as the unfused path rounds: the products to bf16, the activation to bf16, the result
  const float g = ts_round_bf16(gate), u = ts_round_bf16(up);
  const float act = ts_round_bf16(kvb_silu_for_bf16(g));
  return act * u;
}

// 32 rows n0 .. n0+31 (n0 a multiple of 32) of token m, all in this thread.
__device__ __forceinline__ void ts_finish_row32(const TsParams& p, const TsOutput& o, int m, int n0, float (&v)[32]) {
  const bool full = n0 + 32 <= p.N;
  if (p.bias != nullptr) {
    if (full) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        Vec16<bf16> b;
        b.load(p.bias + n0 + i * 8);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i * 8 + j] += b.get(j);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (n0 + j < p.N) v[j] += __bfloat162float(p.bias[n0 + j]);
    }
  }
  if (p.silu_pairs) {
    // rows in runs of 8 gate, 8 up (N is a multiple of 16): two runs of 8 outputs
    bf16* out = reinterpret_cast<bf16*>(p.out) + (size_t)m * p.ldo + (n0 >> 1);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (n0 + r * 16 >= p.N) break;
      float y[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = ts_silu_mul(v[r * 16 + j], v[r * 16 + 8 + j]);
      if (o.vector_ok) {
        *reinterpret_cast<uint4*>(out + r * 8) =
            make_uint4(ts_pack2(y[0], y[1]), ts_pack2(y[2], y[3]), ts_pack2(y[4], y[5]), ts_pack2(y[6], y[7]));
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) out[r * 8 + j] = __float2bfloat16_rn(y[j]);
      }
    }
  } else if (p.residual != nullptr) {
    bf16* slot = p.residual + (size_t)m * p.N + n0;
    float sq = 0.0f;
    if (full && o.vector_ok) {
      Vec16<bf16> old[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) old[i].load(slot + i * 8);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        Vec16<bf16> s;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          s.set(j, ts_round_bf16(v[i * 8 + j]) + old[i].get(j));
          const float kept = s.get(j);
          sq += kept * kept;
        }
        s.store(slot + i * 8);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (n0 + j < p.N) {
          const float kept = ts_round_bf16(ts_round_bf16(v[j]) + __bfloat162float(slot[j]));
          slot[j] = __float2bfloat16_rn(kept);
          sq += kept * kept;
        }
      }
    }
    p.sumsq_out[(size_t)m * o.pieces + (n0 >> 5)] = sq;
  } else if (p.out_f32) {
    float* out = reinterpret_cast<float*>(p.out) + (size_t)m * p.ldo + n0;
    if (full && o.vector_ok) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        *reinterpret_cast<float4*>(out + i * 4) = make_float4(v[i * 4], v[i * 4 + 1], v[i * 4 + 2], v[i * 4 + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (n0 + j < p.N) out[j] = v[j];
    }
  } else {
    bf16* out = reinterpret_cast<bf16*>(p.out) + (size_t)m * p.ldo + n0;
    if (full && o.vector_ok) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        *reinterpret_cast<uint4*>(out + i * 8) =
            make_uint4(ts_pack2(v[i * 8], v[i * 8 + 1]), ts_pack2(v[i * 8 + 2], v[i * 8 + 3]),
                       ts_pack2(v[i * 8 + 4], v[i * 8 + 5]), ts_pack2(v[i * 8 + 6], v[i * 8 + 7]));
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (n0 + j < p.N) out[j] = __float2bfloat16_rn(v[j]);
    }
  }
}

// 4 rows n .. n+3 (n a multiple of 4) of token m in this thread; the 8 threads that hold the 32 rows
// of a group sit in 8 neighbouring lanes (quad = lane & 7), the whole warp calls together.
__device__ __forceinline__ void ts_finish_quad(const TsParams& p, const TsOutput& o, int m, int n, int lane, bool token_live,
                                               float (&v)[4]) {
  if (p.bias != nullptr) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (n + j < p.N) v[j] += __bfloat162float(p.bias[n + j]);
  }
  if (p.silu_pairs) {
    // gates are quads 0, 1 of every 4 (rows 0-7 of 16); their ups sit two lanes on
    float up[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) up[j] = __shfl_down_sync(0xffffffffu, v[j], 2);
    if (token_live && (lane & 2) == 0 && n < p.N) {
      bf16* out = reinterpret_cast<bf16*>(p.out) + (size_t)m * p.ldo + (n >> 4) * 8 + (n & 7);
      float y[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) y[j] = ts_silu_mul(v[j], up[j]);
      if (o.vector_ok) {
        *reinterpret_cast<uint2*>(out) = make_uint2(ts_pack2(y[0], y[1]), ts_pack2(y[2], y[3]));
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) out[j] = __float2bfloat16_rn(y[j]);
      }
    }
  } else if (p.residual != nullptr) {
    float sq = 0.0f;
    if (token_live) {
      bf16* slot = p.residual + (size_t)m * p.N + n;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (n + j < p.N) {
          const float kept = ts_round_bf16(ts_round_bf16(v[j]) + __bfloat162float(slot[j]));
          slot[j] = __float2bfloat16_rn(kept);
          sq += kept * kept;
        }
      }
    }
    sq += __shfl_xor_sync(0xffffffffu, sq, 1);
    sq += __shfl_xor_sync(0xffffffffu, sq, 2);
    sq += __shfl_xor_sync(0xffffffffu, sq, 4);
    if (token_live && (lane & 7) == 0 && n < p.N) p.sumsq_out[(size_t)m * o.pieces + (n >> 5)] = sq;
  } else if (token_live) {
    if (p.out_f32) {
      float* out = reinterpret_cast<float*>(p.out) + (size_t)m * p.ldo + n;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (n + j < p.N) out[j] = v[j];
    } else {
      bf16* out = reinterpret_cast<bf16*>(p.out) + (size_t)m * p.ldo + n;
      if (o.vector_ok && n + 4 <= p.N) {
        *reinterpret_cast<uint2*>(out) = make_uint2(ts_pack2(v[0], v[1]), ts_pack2(v[2], v[3]));
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (n + j < p.N) out[j] = __float2bfloat16_rn(v[j]);
      }
    }
  }
}

template <int MT, bool NORMED>
__global__ void __launch_bounds__(TS_THREADS + TS_NORM_WARPS * 32, 1)
gemm_stream_tc5_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map,
                       const TsParams p) {
  constexpr int X_BYTES = MT * TS_KS * 2;
  constexpr int STAGE_BYTES = X_BYTES + TS_W_BYTES;            // token rows first, then the weights; a multiple of 1,024
  constexpr int STAGES = MT == 128 ? 4 : 5;
  constexpr unsigned TMEM_COLS = 512;                          // 2 buffers x 256 columns (W rows)
  constexpr int PART_FLOATS = 8 * MT * 32;                     // one slot: [8 groups of 32 W rows][MT tokens][32]

  extern __shared__ __align__(1024) unsigned char ts_dyn[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(ts_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* tail = base + STAGES * STAGE_BYTES;
  unsigned long long* full_bar = reinterpret_cast<unsigned long long*>(tail);   // [STAGES] weights (and x, unless NORMED) landed
  unsigned long long* empty_bar = full_bar + STAGES;                            // [STAGES] the MMAs that read the stage are done
  unsigned long long* xraw_bar = empty_bar + STAGES;                            // [STAGES] NORMED: raw token rows landed
  unsigned long long* xready_bar = xraw_bar + STAGES;                           // [STAGES] NORMED: token rows normalised
  unsigned long long* acc_full = xready_bar + STAGES;                           // [2] a segment's sums are complete
  unsigned long long* acc_free = acc_full + 2;                                  // [2] the epilogue has read them
  unsigned long long* mma_done = acc_free + 2;                                  // [1] every MMA of the block has retired
  unsigned long long* fix_bar = mma_done + 1;                                   // [1] the parts of shared tiles have arrived in shared memory
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(fix_bar + 1);
  int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);
  int* epi_abort = abort_flag + 1;   // written by the epilogue warps only, read by them behind their own barrier
  float* inv_rms = reinterpret_cast<float*>(tail + 512);                        // [MT] NORMED
  unsigned char* norm_w = tail + 1024;                                          // NORMED: the norm weights, as stored

  KvbTrace trace(KVB_TAG_GEMM_STREAM_TC5);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int blocks = gridDim.x, me = blockIdx.x;
  const int u_begin = ts_range_start(p.units, blocks, me), u_end = ts_range_start(p.units, blocks, me + 1);
  const int total = u_end - u_begin;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      kvb_mbar_init(&full_bar[s], 1);
      kvb_mbar_init(&empty_bar[s], 1);
      kvb_mbar_init(&xraw_bar[s], 1);
      kvb_mbar_init(&xready_bar[s], TS_NORM_WARPS);
    }
    for (int b = 0; b < 2; ++b) {
      kvb_mbar_init(&acc_full[b], 1);
      kvb_mbar_init(&acc_free[b], TS_EPI_WARPS);
    }
    kvb_mbar_init(mma_done, 1);
    kvb_mbar_init(fix_bar, 1);
    *abort_flag = 0;
    *epi_abort = 0;
    kvb_mbar_init_fence();
  }
  if (warp == 1) {
    kvb_tc5_alloc(tmem_slot, TMEM_COLS);
  }
  kvb_tc5_fence_before();
  __syncthreads();
  kvb_tc5_fence_after();
  kvb_grid_launch_dependents();
  const unsigned tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      const int pre = total < STAGES ? total : STAGES;
      // before the kernel in front has finished: the whole ring of weight boxes (weights are
      // written by no kernel of the step)
      for (int i = 0; i < pre; ++i) {
        const int u = u_begin + i;
        kvb_mbar_expect_tx(&full_bar[i], (unsigned)(NORMED ? TS_W_BYTES : STAGE_BYTES));
        kvb_tma_2d(base + i * STAGE_BYTES + X_BYTES, &w_map, (u % p.kchunks) * TS_KS, (u / p.kchunks) * TS_NT, &full_bar[i]);
      }
      kvb_grid_wait();                            // x is the output of the kernel in front
      trace.after_wait();
      int issued = 0;
      for (int it = 0; it < total; ++it) {
        const int stage = it % STAGES;
        if (it >= STAGES && !kvb_mbar_wait<TS_SPIN_LIMIT, 1024>(&empty_bar[stage], ((it / STAGES) & 1) ^ 1)) {
          atomicOr(p.status, KVB_STATUS_WAIT_TIMEOUT);
          atomicExch(abort_flag, 1);
          break;
        }
        if (*reinterpret_cast<volatile int*>(abort_flag)) break;
        const int u = u_begin + it;
        const int k0 = (u % p.kchunks) * TS_KS;
        unsigned char* xdst = base + stage * STAGE_BYTES;
        if (it >= pre) {
          kvb_mbar_expect_tx(&full_bar[stage], (unsigned)(NORMED ? TS_W_BYTES : STAGE_BYTES));
          kvb_tma_2d(xdst + X_BYTES, &w_map, k0, (u / p.kchunks) * TS_NT, &full_bar[stage]);
        }
        if (NORMED) {
          kvb_mbar_expect_tx(&xraw_bar[stage], (unsigned)X_BYTES);
          kvb_tma_2d(xdst, &x_map, k0, 0, &xraw_bar[stage]);
        } else {
          kvb_tma_2d(xdst, &x_map, k0, 0, &full_bar[stage]);
        }
        issued = it + 1;
      }
      if (*reinterpret_cast<volatile int*>(abort_flag)) {   // gave up: let the copies in flight land
        for (int j = max(0, issued - STAGES); j < issued; ++j) {
          kvb_mbar_wait<TS_SPIN_LIMIT, 1024>(&full_bar[j % STAGES], (j / STAGES) & 1);
          if (NORMED) kvb_mbar_wait<TS_SPIN_LIMIT, 1024>(&xraw_bar[j % STAGES], (j / STAGES) & 1);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      // instruction descriptor: f32 accumulate, bf16 x bf16, both K-major, M = 128 (token lanes), N = 256 (W rows)
      const unsigned idesc = kvb_tc5_idesc(128, TS_NT, false);
      bool ok = true;
      int it = 0, seg = 0, u = u_begin;
      while (u < u_end && ok) {
        const int n_tile = u / p.kchunks;
        const int tile_end = (n_tile + 1) * p.kchunks;
        const int seg_end = tile_end < u_end ? tile_end : u_end;
        const int buf = seg & 1;
        if (seg >= 2 && !kvb_mbar_wait<TS_SPIN_LIMIT, 1024>(&acc_free[buf], ((seg >> 1) - 1) & 1)) { ok = false; break; }
        bool first = true;
        for (; u < seg_end; ++u, ++it) {
          const int stage = it % STAGES;
          if (!kvb_mbar_wait<TS_SPIN_LIMIT, 1024>(&full_bar[stage], (it / STAGES) & 1)) { ok = false; break; }
          if (NORMED && !kvb_mbar_wait<TS_SPIN_LIMIT, 1024>(&xready_bar[stage], (it / STAGES) & 1)) { ok = false; break; }
          if (*reinterpret_cast<volatile int*>(abort_flag)) { ok = false; break; }
          kvb_tc5_fence_after();
          // A: the MT token rows (the MMA reads 128 rows: lanes beyond MT see the bytes that follow,
          // which stay inside the stage, and no one reads those lanes); B: the 256 weight rows
          const unsigned xbase = kvb_smem(base + stage * STAGE_BYTES);
          const unsigned wbase = xbase + X_BYTES;
#pragma unroll
          for (int kk = 0; kk < TS_KS / 16; ++kk)
            kvb_tc5_mma(tmem_base + buf * TS_NT, kvb_tc5_desc(xbase + kk * 32, 16, 1024), kvb_tc5_desc(wbase + kk * 32, 16, 1024), idesc,
                   (first && kk == 0) ? 0u : 1u);
          first = false;
          kvb_tc5_commit(&empty_bar[stage]);           // the stage may be refilled once these MMAs have read it
        }
        if (!ok) break;
        kvb_tc5_commit(&acc_full[buf]);
        ++seg;
      }
      if (!ok) {
        atomicOr(p.status, KVB_STATUS_WAIT_TIMEOUT);
        atomicExch(abort_flag, 1);
      }
      // nothing of this block may still be running on the tensor cores when the memory is freed
      kvb_tc5_commit(mma_done);
      kvb_mbar_wait<TS_SPIN_LIMIT, 1024>(mma_done, 0);
    }
  } else if (warp < 2 + TS_EPI_WARPS) {
    // ---------------- epilogue: thread = token (accumulator lane); warp w reads lanes [32 (w mod 4), +32) ----------------
    kvb_grid_wait();   // nothing is written to global memory before the kernel in front has finished
    const int q = warp & 3;
    const int tid = q * 32 + lane;                       // token of this thread
    const unsigned lane_addr = ((unsigned)(q * 32)) << 16;
    const bool warp_live = q * 32 < p.M;                 // some token of the warp exists
    TsOutput o;
    o.pieces = (p.N + 31) / 32;
    {
      const int esize = p.out_f32 ? 4 : 2;
      o.vector_ok = p.residual != nullptr
                        ? (p.N % 8 == 0 && aligned16(p.residual))
                        : (((size_t)p.ldo * esize) % 16 == 0 && aligned16(p.out));
    }
    int shared_tile[2] = {-1, -1};                       // tiles this block shares with others: [slot]
    bool ok = true;
    int seg = 0, u = u_begin;
    while (u < u_end && ok) {
      const int n_tile = u / p.kchunks, kc0 = u % p.kchunks;
      const int tile_end = (n_tile + 1) * p.kchunks;
      const int seg_end = tile_end < u_end ? tile_end : u_end;
      const int buf = seg & 1;
      const bool whole = kc0 == 0 && seg_end == tile_end;
      const int slot = kc0 == 0 ? 1 : 0;
      // the four warps decide together whether to go on: a wait that ran out in one of them ends all
      if (!kvb_mbar_wait<TS_SPIN_LIMIT, 1024>(&acc_full[buf], (seg >> 1) & 1)) *reinterpret_cast<volatile int*>(epi_abort) = 1;
      asm volatile("bar.sync 1, %0;\n" ::"n"(TS_EPI_WARPS * 32));
      if (*reinterpret_cast<volatile int*>(epi_abort)) { ok = false; break; }
      kvb_tc5_fence_after();
      float* part = p.partial + ((size_t)me * 2 + slot) * PART_FLOATS;
      if (warp_live) {
#pragma unroll 1
        for (int g = 0; g < 8; ++g) {
          if (n_tile * TS_NT + g * 32 >= p.N) break;       // rows beyond N: zeros, never read
          float v[32];
          kvb_tc5_ld32(tmem_base + lane_addr + buf * TS_NT + g * 32, v);
          kvb_tc5_wait_ld();
          if (tid < p.M) {
            if (whole) {
              ts_finish_row32(p, o, tid, n_tile * TS_NT + g * 32, v);
            } else if (tid < MT) {
              float4* dst = reinterpret_cast<float4*>(part + ((size_t)g * MT + tid) * 32);
#pragma unroll
              for (int i = 0; i < 8; ++i) __stcg(dst + i, make_float4(v[i * 4], v[i * 4 + 1], v[i * 4 + 2], v[i * 4 + 3]));
            }
          }
        }
      }
      kvb_tc5_fence_before();
      __syncwarp();
      if (lane == 0) kvb_mbar_arrive(&acc_free[buf]);
      if (!whole) {
        shared_tile[slot] = n_tile;
        __threadfence();
        asm volatile("bar.sync 1, %0;\n" ::"n"(TS_EPI_WARPS * 32));
        if (tid == 0) kvb_st_release(&p.flags[me * 2 + slot], 1);
      }
      u = seg_end;
      ++seg;
    }
    if (!ok) {
      atomicOr(p.status, KVB_STATUS_WAIT_TIMEOUT);
      atomicExch(abort_flag, 1);
    }
    // ---- tiles shared with other blocks: when all parts are there, this block finishes its rows ----
    // Part j of a tile lies in block b_first + j (slot 1 for the tile's first block, slot 0 for the
    // others), laid out [8 groups of 32 W rows][MT tokens][32].  Of the 8 groups this block takes
    // [g_lo, g_hi): that run of every part is one contiguous piece, which a bulk copy brings into the
    // (now idle) stage memory, all pieces of both tiles in flight together; the sums are then formed
    // from shared memory in k order.  Pieces that do not fit are read from global memory instead.
    asm volatile("bar.sync 1, %0;\n" ::"n"(TS_EPI_WARPS * 32));
    constexpr unsigned CAP = STAGES * STAGE_BYTES;
    constexpr unsigned GROUP_BYTES = MT * 32 * 4;
    int first_of[2] = {0, 0}, parts_of[2] = {0, 0}, g_lo[2] = {0, 0}, g_hi[2] = {0, 0};
    unsigned need[2] = {0, 0};
    if (ok) {
      bool seen_all = true;
#pragma unroll
      for (int slot = 0; slot < 2; ++slot) {
        const int n_tile = shared_tile[slot];
        if (n_tile < 0) continue;
        first_of[slot] = ts_block_of(p.units, blocks, n_tile * p.kchunks);
        parts_of[slot] = ts_block_of(p.units, blocks, (n_tile + 1) * p.kchunks - 1) - first_of[slot] + 1;
        const int mine = me - first_of[slot];
        g_lo[slot] = (8 * mine) / parts_of[slot];
        g_hi[slot] = (8 * (mine + 1)) / parts_of[slot];
        need[slot] = (unsigned)parts_of[slot] * (unsigned)(g_hi[slot] - g_lo[slot]) * GROUP_BYTES;
        for (int j = tid; j < parts_of[slot]; j += TS_EPI_WARPS * 32) {
          const int* flag = &p.flags[(first_of[slot] + j) * 2 + (j == 0 ? 1 : 0)];
          int seen = 0;
          for (unsigned spin = 0; spin < TS_SPIN_LIMIT && !seen; ++spin) {
            seen = kvb_ld_acquire(flag);
            if (!seen && spin > 4096) __nanosleep(64);   // the blocks finish together: spin first
          }
          if (!seen) seen_all = false;
        }
      }
      if (!seen_all) {
        atomicOr(p.status, KVB_STATUS_WAIT_TIMEOUT);
        atomicExch(abort_flag, 1);
        *reinterpret_cast<volatile int*>(epi_abort) = 1;
      }
    }
    asm volatile("bar.sync 1, %0;\n" ::"n"(TS_EPI_WARPS * 32));
    if (*reinterpret_cast<volatile int*>(epi_abort)) ok = false;
    if (ok && (shared_tile[0] >= 0 || shared_tile[1] >= 0)) {
      __threadfence();
      const bool together = need[0] + need[1] <= CAP;
      unsigned phase = 0;
#pragma unroll 1
      for (int round = 0; round < 2 && ok; ++round) {
        const int s_lo = round == 0 ? 0 : (together ? 2 : 1), s_hi = round == 0 ? (together ? 2 : 1) : 2;
        unsigned offset[2] = {0, 0}, staged = 0;
        for (int slot = s_lo; slot < s_hi; ++slot) {
          offset[slot] = staged;
          if (need[slot] <= CAP - staged) staged += need[slot];
          else offset[slot] = 0xffffffffu;               // does not fit: read from global memory
        }
        if (staged > 0) {
          if (tid == 0) {
            kvb_fence_async_shared();
            kvb_mbar_expect_tx(fix_bar, staged);
            for (int slot = s_lo; slot < s_hi; ++slot) {
              if (offset[slot] == 0xffffffffu || need[slot] == 0) continue;
              const unsigned piece = (unsigned)(g_hi[slot] - g_lo[slot]) * GROUP_BYTES;
              for (int j = 0; j < parts_of[slot]; ++j) {
                const float* src = p.partial + ((size_t)(first_of[slot] + j) * 2 + (j == 0 ? 1 : 0)) * PART_FLOATS +
                                   (size_t)g_lo[slot] * MT * 32;
                kvb_bulk_copy(base + offset[slot] + j * piece, src, piece, fix_bar);
              }
            }
          }
          if (!kvb_mbar_wait<TS_SPIN_LIMIT, 1024>(fix_bar, phase)) *reinterpret_cast<volatile int*>(epi_abort) = 1;
          phase ^= 1;
          asm volatile("bar.sync 1, %0;\n" ::"n"(TS_EPI_WARPS * 32));
          if (*reinterpret_cast<volatile int*>(epi_abort)) {
            if (tid == 0) {
              atomicOr(p.status, KVB_STATUS_WAIT_TIMEOUT);
              atomicExch(abort_flag, 1);
            }
            ok = false;
            break;
          }
        }
        // thread = (token of a pass of 16, 4 rows of the group's 32): a warp reads 4 tokens x 128 bytes in a row
        const int quad = tid & 7, sub = tid >> 3;
        for (int slot = s_lo; slot < s_hi; ++slot) {
          if (shared_tile[slot] < 0) continue;
          const int parts = parts_of[slot];
          const int groups = g_hi[slot] - g_lo[slot];
          const bool in_smem = offset[slot] != 0xffffffffu;
          const size_t part_stride = in_smem ? (size_t)groups * MT * 32 : 0;
#pragma unroll 1
          for (int item = 0; item < groups * (MT / 16); ++item) {
            const int g = item / (MT / 16), m = (item % (MT / 16)) * 16 + sub;
            if ((item % (MT / 16)) * 16 >= p.M) continue;       // the whole pass lies beyond the batch
            const int n = shared_tile[slot] * TS_NT + (g_lo[slot] + g) * 32 + quad * 4;
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (in_smem) {
              const float4* src = reinterpret_cast<const float4*>(base + offset[slot]) + (((size_t)g * MT + m) * 32 + quad * 4) / 4;
#pragma unroll 1
              for (int j0 = 0; j0 < parts; j0 += 4) {      // four parts in flight together, added in k order
                float4 vals[4];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  vals[j] = j0 + j < parts ? src[(size_t)(j0 + j) * part_stride / 4] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  if (j0 + j < parts) { acc[0] += vals[j].x; acc[1] += vals[j].y; acc[2] += vals[j].z; acc[3] += vals[j].w; }
                }
              }
            } else {
              const size_t within = ((size_t)(g_lo[slot] + g) * MT + m) * 32 + quad * 4;
#pragma unroll 1
              for (int j0 = 0; j0 < parts; j0 += 4) {
                float4 vals[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const int part_index = j0 + j;
                  vals[j] = part_index < parts
                                ? __ldcg(reinterpret_cast<const float4*>(p.partial + ((size_t)(first_of[slot] + part_index) * 2 + (part_index == 0 ? 1 : 0)) * PART_FLOATS + within))
                                : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  if (j0 + j < parts) { acc[0] += vals[j].x; acc[1] += vals[j].y; acc[2] += vals[j].z; acc[3] += vals[j].w; }
                }
              }
            }
            ts_finish_quad(p, o, m, n, lane, m < p.M, acc);
          }
        }
        // the pieces have been read: the memory may be filled again, the flags may go down
        asm volatile("bar.sync 1, %0;\n" ::"n"(TS_EPI_WARPS * 32));
      }
      // the last block through a tile lowers its flags for the next launch
      if (ok && tid == 0) {
        for (int slot = 0; slot < 2; ++slot) {
          if (shared_tile[slot] < 0) continue;
          int* counter = &p.flags[blocks * 2 + shared_tile[slot]];
          if (atomicAdd(counter, 1) == parts_of[slot] - 1) {
            *counter = 0;
            for (int j = 0; j < parts_of[slot]; ++j) p.flags[(first_of[slot] + j) * 2 + (j == 0 ? 1 : 0)] = 0;
          }
        }
      }
    }
  } else {
    // ---------------- NORMED: the normaliser warps ----------------
    if (NORMED) {
      const int nt = (warp - 2 - TS_EPI_WARPS) * 32 + lane;       // 0..127
      // the norm weights (written by no kernel of the step) into shared memory, before the wait
      const int w_bytes = p.K * (p.norm_weight_f32 ? 4 : 2);
      for (int i = nt * 16; i < w_bytes; i += TS_NORM_WARPS * 32 * 16)
        *reinterpret_cast<uint4*>(norm_w + i) = *reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(p.norm_weight) + i);
      kvb_grid_wait();
      // 1 / rms of this warp's MT / 4 token rows from the pieces of their sums of squares: every lane
      // adds its pieces in order, the lanes are added by a butterfly, so the value depends on the
      // pieces alone; the rows' loads go out together
      {
        constexpr int TW = MT / TS_NORM_WARPS;
        const int first = (warp - 2 - TS_EPI_WARPS) * TW;
        float part[TW];
#pragma unroll
        for (int i = 0; i < TW; ++i) part[i] = 0.0f;
        for (int t = lane; t < p.sumsq_pieces; t += 32) {
#pragma unroll
          for (int i = 0; i < TW; ++i)
            if (first + i < p.M) part[i] += __ldcg(p.sumsq_in + (size_t)(first + i) * p.sumsq_pieces + t);
        }
#pragma unroll
        for (int i = 0; i < TW; ++i) {
          const float sum = warp_sum(part[i]);
          if (lane == 0) inv_rms[first + i] = 1.0f / sqrtf(sum / (float)p.K + p.eps);
        }
      }
      asm volatile("bar.sync 2, %0;\n" ::"n"(TS_NORM_WARPS * 32));
      const int chunk = nt & 7, row0 = nt >> 3;            // 16 bytes of a row; rows row0, row0 + 16, ...
      for (int it = 0; it < total; ++it) {
        const int stage = it % STAGES;
        int fine = kvb_mbar_wait<TS_SPIN_LIMIT, 1024>(&xraw_bar[stage], (it / STAGES) & 1) ? 1 : 0;
        fine = __all_sync(0xffffffffu, fine);
        if (!fine) {
          if (lane == 0) {
            atomicOr(p.status, KVB_STATUS_WAIT_TIMEOUT);
            atomicExch(abort_flag, 1);
          }
          break;
        }
        if (*reinterpret_cast<volatile int*>(abort_flag)) break;
        const int k = ((u_begin + it) % p.kchunks) * TS_KS + chunk * 8;   // this thread's 8 k-values of the stage
        unsigned char* xs = base + stage * STAGE_BYTES;
        float g[8];
        if (p.norm_weight_f32) {
          const float4 lo = *reinterpret_cast<const float4*>(norm_w + (size_t)k * 4);
          const float4 hi = *reinterpret_cast<const float4*>(norm_w + (size_t)k * 4 + 16);
          g[0] = lo.x; g[1] = lo.y; g[2] = lo.z; g[3] = lo.w; g[4] = hi.x; g[5] = hi.y; g[6] = hi.z; g[7] = hi.w;
        } else {
          Vec16<bf16> gw;
          gw.raw = *reinterpret_cast<const uint4*>(norm_w + (size_t)k * 2);
#pragma unroll
          for (int j = 0; j < 8; ++j) g[j] = gw.get(j);
        }
        constexpr int PASSES = MT / 16;
        uint4 raw[PASSES];
#pragma unroll
        for (int i = 0; i < PASSES; ++i) {
          const int r = row0 + i * 16;
          raw[i] = *reinterpret_cast<const uint4*>(xs + r * 128 + ((chunk ^ (r & 7)) << 4));
        }
#pragma unroll
        for (int i = 0; i < PASSES; ++i) {
          const int r = row0 + i * 16;
          const float inv = inv_rms[r];
          Vec16<bf16> v, o;
          v.raw = raw[i];
#pragma unroll
          for (int j = 0; j < 8; ++j) o.set(j, g[j] * (v.get(j) * inv));
          *reinterpret_cast<uint4*>(xs + r * 128 + ((chunk ^ (r & 7)) << 4)) = o.raw;
        }
        // these writes come before the MMAs that read the stage and the TMA box that will reuse it
        kvb_fence_async_shared();
        __syncwarp();
        if (lane == 0) kvb_mbar_arrive(&xready_bar[stage]);
      }
    }
  }

  // ---- everyone meets; the allocating warp frees the tensor memory ----
  kvb_tc5_fence_before();
  __syncthreads();
  if (warp == 1) {
    kvb_tc5_fence_after();
    kvb_tc5_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- host side -----------------------------------------------------------------------------
// 2-D bf16 tensor map over a row-major [rows, cols] matrix with leading dimension ld (elements):
// boxes of [box_rows][64 columns], 128-byte swizzle, zero fill outside.
static int ts_make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols, long long ld, int box_rows) {
  KvbEncodeTiledFn encode = kvb_encode_tiled_fn();
  KVB_REQUIRE(encode != nullptr, "stream gemm (tcgen05): the driver does not export cuTensorMapEncodeTiled");
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(bf16)};
  const cuuint32_t box[2] = {TS_KS, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  KVB_REQUIRE(rc == CUDA_SUCCESS, "stream gemm (tcgen05): cuTensorMapEncodeTiled failed");
  return 0;
}

// Scratch floats (for the largest token block) and flag ints (zero before the first launch; the
// kernel leaves them zero) for `blocks` blocks.
extern "C" long long kvb_gemm_stream_tc5_scratch_floats(int blocks) { return (long long)blocks * 2 * 2 * 128 * 128; }
extern "C" long long kvb_gemm_stream_tc5_flag_ints(int blocks) { return (long long)blocks * 2 + TS_MAX_TILES; }
extern "C" int kvb_gemm_stream_tc5_norm_max_k() { return TS_NORM_W_BYTES / 4; }
extern "C" int kvb_gemm_stream_tc5_max_rows() { return 128; }

template <int MT, bool NORMED>
static int ts_launch(const void* w, const void* x, long long ldx, TsParams& p, int sms, cudaStream_t stream) {
  constexpr int STAGES = MT == 128 ? 4 : 5;
  constexpr size_t SMEM = 1024 + (size_t)STAGES * (TS_W_BYTES + MT * TS_KS * 2) + 1024 + (NORMED ? TS_NORM_W_BYTES : 0);
  static bool configured = false;
  if (!configured) {
    KVB_CHECK_CUDA(cudaFuncSetAttribute(gemm_stream_tc5_kernel<MT, NORMED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
    configured = true;
  }
  alignas(64) CUtensorMap w_map, x_map;
  if (int rc = ts_make_map(&w_map, w, p.N, p.K, p.K, TS_NT)) return rc;
  if (int rc = ts_make_map(&x_map, x, p.M, p.K, ldx, MT)) return rc;
  const int blocks = p.units < sms ? p.units : sms;
  const int threads = NORMED ? TS_THREADS + TS_NORM_WARPS * 32 : TS_THREADS;
  KVB_CHECK_CUDA(kvb_launch(gemm_stream_tc5_kernel<MT, NORMED>, dim3(blocks), dim3(threads), SMEM, stream, true, w_map,
                            x_map, p));
  return 0;
}

// out[M, N] = x[M, K] . w[N, K]^T (+ bias), 1 <= M <= 128, K a multiple of 64.  Arguments as
// kvb_gemm_stream_bf16, except: scratch holds kvb_gemm_stream_tc5_scratch_floats(sms) floats, flags
// kvb_gemm_stream_tc5_flag_ints(sms) ints (zero before the first launch); with the residual epilogue
// sumsq_out is [M, ceil(N / 32)] (32 columns a piece).  `sms` must not exceed the number of blocks
// that run at the same time (one per SM): blocks that share a tile wait for one another.
extern "C" int kvb_gemm_stream_tc5_bf16(void* out, int out_f32, long long ldo, const void* x, long long ldx,
                                        const void* w, const void* bias, int M, int N, int K, int silu_pairs,
                                        const void* norm_weight, int norm_weight_f32, float eps,
                                        const float* sumsq_in, int sumsq_pieces, void* residual, float* sumsq_out,
                                        float* scratch, int* flags, int sms, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  KVB_REQUIRE(M > 0 && M <= 128, "stream gemm (tcgen05): takes 1 to 128 rows of x");
  KVB_REQUIRE(K > 0 && K % 64 == 0 && ldx % 8 == 0,
              "stream gemm (tcgen05): K must be a multiple of 64 and the row stride of x of 8");
  KVB_REQUIRE(aligned16(x) && aligned16(w) && aligned16(bias), "stream gemm (tcgen05): x, w and bias must be 16-byte aligned");
  KVB_REQUIRE(scratch != nullptr && flags != nullptr && sms > 0, "stream gemm (tcgen05): needs scratch and flags");
  KVB_REQUIRE(!silu_pairs || (N % 16 == 0 && !out_f32),
              "stream gemm (tcgen05): gated pairs need N a multiple of 16 and a bf16 result");
  KVB_REQUIRE(residual == nullptr || (!silu_pairs && !out_f32 && sumsq_out != nullptr),
              "stream gemm (tcgen05): the residual epilogue needs a plain bf16 product and a place for the squares");
  KVB_REQUIRE(norm_weight == nullptr || (sumsq_in != nullptr && sumsq_pieces > 0 && aligned16(norm_weight) &&
                                         (size_t)K * (norm_weight_f32 ? 4 : 2) <= TS_NORM_W_BYTES),
              "stream gemm (tcgen05): the fused norm needs the sums of squares and K small enough for shared memory");
  TsParams p;
  memset(&p, 0, sizeof(p));
  p.out = out; p.out_f32 = out_f32; p.ldo = ldo;
  p.bias = (const bf16*)bias;
  p.M = M; p.N = N; p.K = K;
  p.silu_pairs = silu_pairs;
  p.norm_weight = norm_weight; p.norm_weight_f32 = norm_weight_f32; p.eps = eps;
  p.sumsq_in = sumsq_in; p.sumsq_pieces = sumsq_pieces;
  p.residual = (bf16*)residual; p.sumsq_out = sumsq_out;
  p.n_tiles = (N + TS_NT - 1) / TS_NT;
  p.kchunks = K / TS_KS;
  KVB_REQUIRE(p.n_tiles <= TS_MAX_TILES, "stream gemm (tcgen05): N is too large");
  KVB_REQUIRE((long long)p.n_tiles * p.kchunks < (1ll << 30), "stream gemm (tcgen05): the matrix is too large");
  p.units = p.n_tiles * p.kchunks;
  p.partial = scratch;
  p.flags = flags;
  p.status = kvb_status_word();
  KVB_REQUIRE(p.status != nullptr, "stream gemm (tcgen05): no status word");
  const bool normed = norm_weight != nullptr;
  if (M <= 32) return normed ? ts_launch<32, true>(w, x, ldx, p, sms, stream) : ts_launch<32, false>(w, x, ldx, p, sms, stream);
  if (M <= 64) return normed ? ts_launch<64, true>(w, x, ldx, p, sms, stream) : ts_launch<64, false>(w, x, ldx, p, sms, stream);
  return normed ? ts_launch<128, true>(w, x, ldx, p, sms, stream) : ts_launch<128, false>(w, x, ldx, p, sms, stream);
}

KVB_TRACE_TU(gemm_stream_tc5)
