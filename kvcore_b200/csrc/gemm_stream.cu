// Weight-streaming linear layer for decode: out[M, N] = x[M, K] . W[N, K]^T (+ bias), bf16 in,
// 32-bit accumulate, M <= 16 tokens, K a multiple of 64 (sm_100a).
//
// With so few tokens the layer is one pass over the weight matrix, so the kernel is built around
// keeping DRAM busy.  What was measured on B200 while building it: the access pattern of the
// boxes does not matter (rows of 128 bytes 8 KB apart stream as fast as contiguous runs); what
// matters is the number of bytes in flight per SM (about 180 KB) and the number of 128-byte lines
// the SM's TMA unit has to move (token rows that travel with every stage are not free; an L2
// prefetch of each box costs as much as the box and made the kernel slower).
//
//  * A stage is 64 weight rows x 256 k-values (32 KB), brought by ONE 3-D TMA box laid out as
//    [4 slabs of 64 k][64 rows][128 bytes] with the 128-byte swizzle; one more box brings the
//    token rows of x for the same k-values (rows beyond M and k beyond K arrive as zeros).  The
//    ring holds five stages.
//  * One block per SM.  The stages of the layer are numbered tile by tile (k fastest) and dealt to
//    the blocks as equal contiguous ranges, so every SM streams the same number of bytes whatever
//    N and K are.  A range that starts inside a tile is a "part": the block adds it up and leaves
//    it in scratch; the block that holds the tile's first stage (the owner) adds the parts in k
//    order, adds the bias and stores.  Each block writes at most one part (the first thing it
//    does) and waits only for blocks that run beside it, with a bounded spin.  There is no flag:
//    scratch holds a marker (a NaN that no sum can be) between launches, the owner reads the
//    values of a part until none is the marker, and puts the marker back.
//  * Programmatic dependent launch: weights are written by no kernel of a step, so the whole ring
//    of weight boxes is asked for before waiting for the kernel in front (whose output x is):
//    when this kernel follows another in a stream, its blocks fill their rings while the other's
//    last blocks finish and while small kernels in between run.
//  * Eight consumer warps: warp w owns weight rows [16 (w mod 4), +16) and one half of the stage's
//    k-values (ldmatrix the W rows as the A operand and the token rows as the B operand of
//    mma.sync m16n8k16); the two halves are added in a fixed order when a tile (or the block's
//    share of it) ends.
//
// The result does not depend on timing: halves and parts are added in a fixed order.  All waits
// are bounded (status bit WAIT_TIMEOUT, then drain and return).
#include <cuda.h>
#include <string.h>

#include "common.cuh"
#include "sm100.cuh"

#define GS_NT 64            // weight rows per tile
#define GS_KG 4             // slabs of 64 k-values per stage
#define GS_CONSUMERS 8
#define GS_THREADS ((GS_CONSUMERS + 1) * 32)
#define GS_STAGES 5
#define GS_SPIN_LIMIT (1u << 20)
#define GS_NORM_W_BYTES (16 * 1024)   // norm weights a NORMED kernel keeps in shared memory
#define GS_NORMALISERS 4               // NORMED: warps that normalise the token rows of each stage
#define GS_SCRATCH_MARKER 0x7FC0DEADu  // every word of scratch between launches: a NaN no sum can be (sums that are NaN are 0x7FFFFFFF)

struct StreamParams {
  void* out; int out_f32; long long ldo;
  const bf16* bias;
  int M, N, K;
  int n_tiles, kchunks, units;       // kchunks = ceil(K / 256); units = n_tiles * kchunks
  float* partial;                    // [blocks][MBLK * 4][128]; GS_SCRATCH_MARKER everywhere between launches
  int* status;
  // NORMED kernels: the rows of x are sums s that still need their RMS norm.  Every token's sum
  // of squares arrives in pieces, sumsq_in[m * sumsq_pieces + t] (added in a fixed order); a warp
  // of its own turns each stage's token rows into bf16(norm_weight[k] * (s * rsqrt(mean + eps)))
  // before the consumers use them.
  const float* sumsq_in; int sumsq_pieces; const void* norm_weight; int norm_weight_f32; float eps;
  // Epilogue with the residual stream (residual != null, [M, N] bf16): s = bf16(bf16(out) + residual)
  // written over residual (every tile its own columns), and the sum of its squares over the tile's
  // 64 columns to sumsq_out[m * n_tiles + tile].  out itself is not written.
  bf16* residual; float* sumsq_out;
  int silu_pairs;                    // 1: rows n and n+8 of every 16 are a (gate, up) pair: out[m, .] = silu(gate) * up
  unsigned spin_limit;               // polls after which a wait gives up
  // Test of the give-up path (kvb_gemm_stream_test_give_up): block test_skip_block never asks for the
  // copies of its stage test_skip_stage, so that everyone who waits for them runs out of polls.  -1: off.
  int test_skip_block, test_skip_stage;
};

__device__ __forceinline__ void gs_ldmatrix_x4(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void gs_ldmatrix_x2(unsigned (&r)[2], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void gs_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Byte offset of (row, k) in an operand area made of [rows][128-byte] slabs, one per 64 k-values,
// 16-byte chunks XOR-swizzled with the row as TMA's 128-byte swizzle lays them out.
__device__ __forceinline__ unsigned gs_swz(int row, int k, int rows) {
  const int slab = k >> 6, chunk = (k & 63) >> 3;
  return (unsigned)(slab * rows * 128 + row * 128 + ((chunk ^ (row & 7)) << 4));
}

// A bounded wait with the launch's limit (GS_SPIN_LIMIT polls unless a test lowered it).
__device__ __forceinline__ bool gs_wait(const StreamParams& p, unsigned long long* bar, unsigned parity) {
  return kvb_mbar_wait_n(bar, parity, p.spin_limit, 64);
}

// Named barrier ID of THREADS threads that also tells everyone whether anyone brought `mine`: the way the
// warps of a role leave together when one of them has given up (a plain barrier followed by a look at a
// flag lets one warp leave and another stay, and the one that stays then waits at the next barrier for good).
template <int ID, int THREADS>
__device__ __forceinline__ bool gs_bar_any(bool mine) {
  unsigned any;
  asm volatile("{\n.reg .pred p, q;\nsetp.ne.u32 p, %1, 0;\nbar.red.or.pred q, %2, %3, p;\nselp.u32 %0, 1, 0, q;\n}\n"
               : "=r"(any) : "r"((unsigned)mine), "n"(ID), "n"(THREADS) : "memory");
  return any != 0;
}

// First stage of block b when `units` stages are dealt to `blocks` blocks.
__device__ __forceinline__ int gs_range_start(int units, int blocks, int b) {
  return (int)(((long long)units * b) / blocks);
}

template <int MBLK, bool NORMED>   // MB = 8 * MBLK token rows; NORMED: x is normalised on the way (see StreamParams)
__global__ void __launch_bounds__(GS_THREADS + GS_NORMALISERS * 32, 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map,
                   const StreamParams p) {
  constexpr int MB = 8 * MBLK;
  constexpr int KB = 64 * GS_KG;
  constexpr int W_BYTES = GS_NT * KB * 2;
  constexpr int X_BYTES = MB * KB * 2;
  constexpr int STAGE_BYTES = W_BYTES + X_BYTES;      // a multiple of 1,024
  constexpr int STAGES = GS_STAGES;

  extern __shared__ __align__(1024) unsigned char gs_dyn[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(gs_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* tail = base + STAGES * STAGE_BYTES;
  unsigned long long* full_bar = reinterpret_cast<unsigned long long*>(tail);   // weights (and x, unless NORMED) landed
  unsigned long long* empty_bar = full_bar + STAGES;
  unsigned long long* xraw_bar = empty_bar + STAGES;            // NORMED: the raw token rows landed
  unsigned long long* xready_bar = xraw_bar + STAGES;           // NORMED: the token rows are normalised
  int* flags = reinterpret_cast<int*>(tail + 512);              // [0] abort
  float* halves = reinterpret_cast<float*>(tail + 1024);        // [MBLK * 4][128 threads]
  // the finished tile, [MB tokens][64 rows] in the output's type, so that it leaves in whole lines
  unsigned char* out_tile = tail + 1024 + MBLK * 4 * 128 * sizeof(float);
  unsigned char* norm_w = out_tile + MB * GS_NT * sizeof(float);   // NORMED: the norm weights, as stored

  KvbTrace trace(KVB_TAG_GEMM_STREAM);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int blocks = gridDim.x, me = blockIdx.x;
  const int u_begin = gs_range_start(p.units, blocks, me), u_end = gs_range_start(p.units, blocks, me + 1);
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      kvb_mbar_init(&full_bar[s], 1);
      kvb_mbar_init(&empty_bar[s], GS_CONSUMERS);
      kvb_mbar_init(&xraw_bar[s], 1);
      kvb_mbar_init(&xready_bar[s], GS_NORMALISERS);
    }
    flags[0] = 0;
    kvb_mbar_init_fence();
  }
  __syncthreads();
  kvb_grid_launch_dependents();

  if (warp == GS_CONSUMERS) {
    // ---------------- producer ----------------
    if (lane == 0) {
      const int total = u_end - u_begin;
      const int pre = total < STAGES ? total : STAGES;
      // before the kernel in front has finished: the whole ring of weight boxes (weights are
      // written by no kernel of the step)
      for (int i = 0; i < pre; ++i) {
        const int u = u_begin + i;
        if (me == p.test_skip_block && i == p.test_skip_stage) continue;
        kvb_mbar_expect_tx(&full_bar[i], (unsigned)(NORMED ? W_BYTES : STAGE_BYTES));
        kvb_tma_3d(base + i * STAGE_BYTES, &w_map, 0, (u / p.kchunks) * GS_NT, (u % p.kchunks) * GS_KG, &full_bar[i]);
      }
      kvb_grid_wait();                            // x is the output of the kernel in front
      int issued = 0;
      for (int it = 0; it < total; ++it) {
        const int stage = it % STAGES;
        if (it >= STAGES && !gs_wait(p, &empty_bar[stage], ((it / STAGES) & 1) ^ 1)) {
          atomicOr(p.status, KVB_STATUS_WAIT_TIMEOUT);
          atomicExch(&flags[0], 1);
          break;
        }
        if (*reinterpret_cast<volatile int*>(&flags[0])) break;
        const int u = u_begin + it;
        const int slab = (u % p.kchunks) * GS_KG;
        unsigned char* wdst = base + stage * STAGE_BYTES;
        issued = it + 1;
        if (me == p.test_skip_block && it == p.test_skip_stage) continue;
        if (it >= pre) {
          kvb_mbar_expect_tx(&full_bar[stage], (unsigned)(NORMED ? W_BYTES : STAGE_BYTES));
          kvb_tma_3d(wdst, &w_map, 0, (u / p.kchunks) * GS_NT, slab, &full_bar[stage]);
        }
        if (NORMED) {
          kvb_mbar_expect_tx(&xraw_bar[stage], (unsigned)X_BYTES);
          kvb_tma_3d(wdst + W_BYTES, &x_map, 0, 0, slab, &xraw_bar[stage]);
        } else {
          kvb_tma_3d(wdst + W_BYTES, &x_map, 0, 0, slab, &full_bar[stage]);
        }
      }
      if (*reinterpret_cast<volatile int*>(&flags[0])) {   // gave up: let the copies in flight land
        for (int j = max(0, issued - STAGES); j < issued; ++j) {
          gs_wait(p, &full_bar[j % STAGES], (j / STAGES) & 1);
          if (NORMED) gs_wait(p, &xraw_bar[j % STAGES], (j / STAGES) & 1);
        }
      }
    }
  } else if (warp > GS_CONSUMERS) {
    // ---------------- NORMED: the normaliser warps; warp n takes token rows n, n + 4, ... ----------------
    if (NORMED) {
      const int nw = warp - GS_CONSUMERS - 1;
      // the norm weights (written by no kernel of the step) into shared memory, before the wait
      const int w_bytes = p.K * (p.norm_weight_f32 ? 4 : 2);
      for (int i = (nw * 32 + lane) * 16; i < w_bytes; i += GS_NORMALISERS * 32 * 16)
        *reinterpret_cast<uint4*>(norm_w + i) = *reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(p.norm_weight) + i);
      asm volatile("bar.sync 3, %0;\n" ::"n"(GS_NORMALISERS * 32));
      kvb_grid_wait();
      // 1 / rms of this warp's token rows from the pieces of their sums of squares: every lane adds
      // its pieces in order, the lanes are added by a butterfly, so the value depends on the pieces alone
      // (the pieces of all of this warp's rows are asked for before any of them is added: one trip to L2,
      // not one a row, between the end of the kernel in front and the first normalised stage)
      constexpr int ROWS = MB / GS_NORMALISERS;
      float inv[ROWS], part[ROWS];
#pragma unroll
      for (int i = 0; i < ROWS; ++i) part[i] = 0.0f;
      for (int t = lane; t < p.sumsq_pieces; t += 32) {
        float piece[ROWS];
#pragma unroll
        for (int i = 0; i < ROWS; ++i) {
          const int m = nw + i * GS_NORMALISERS;
          piece[i] = m < p.M ? __ldcg(p.sumsq_in + (size_t)m * p.sumsq_pieces + t) : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < ROWS; ++i) part[i] += piece[i];
      }
#pragma unroll
      for (int i = 0; i < ROWS; ++i) inv[i] = 1.0f / sqrtf(warp_sum(part[i]) / (float)p.K + p.eps);
      const int total = u_end - u_begin;
      for (int it = 0; it < total; ++it) {
        const int stage = it % STAGES;
        int fine = gs_wait(p, &xraw_bar[stage], (it / STAGES) & 1) ? 1 : 0;
        fine = __all_sync(0xffffffffu, fine);
        if (!fine) {
          if (lane == 0) {
            atomicOr(p.status, KVB_STATUS_WAIT_TIMEOUT);
            atomicExch(&flags[0], 1);
          }
          break;
        }
        if (*reinterpret_cast<volatile int*>(&flags[0])) break;
        const int k = ((u_begin + it) % p.kchunks) * KB + lane * 8;   // this lane's 8 k-values of the stage
        unsigned char* xs = base + stage * STAGE_BYTES + W_BYTES;
        if (k < p.K) {                                               // beyond K the rows are zeros
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
          uint4 raw[ROWS];
#pragma unroll
          for (int i = 0; i < ROWS; ++i)
            raw[i] = *reinterpret_cast<const uint4*>(xs + gs_swz(nw + i * GS_NORMALISERS, lane * 8, MB));
#pragma unroll
          for (int i = 0; i < ROWS; ++i) {
            Vec16<bf16> v, o;
            v.raw = raw[i];
#pragma unroll
            for (int j = 0; j < 8; ++j) o.set(j, g[j] * (v.get(j) * inv[i]));
            *reinterpret_cast<uint4*>(xs + gs_swz(nw + i * GS_NORMALISERS, lane * 8, MB)) = o.raw;
          }
        }
        // these writes come before the TMA box that will reuse the stage
        kvb_fence_async_shared();
        __syncwarp();
        if (lane == 0) kvb_mbar_arrive(&xready_bar[stage]);
      }
    }
  } else {
    // ---------------- consumers: warp w owns rows [16 (w & 3), +16) and k-half (w >> 2) of every stage ----------------
    kvb_grid_wait();   // nothing is written to global memory before the kernel in front has finished
    trace.after_wait();
    const int rg = warp & 3, kh = warp >> 2;
    const int tid = rg * 32 + lane;               // 0..127 within the k-half
    const int a_row = rg * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), a_k = kh * (KB / 2) + 8 * (lane >> 4);
    const int b_row = lane & 7, b_k = kh * (KB / 2) + 8 * ((lane >> 3) & 1);
    int it = 0;
    int u = u_begin;
    while (u < u_end) {
      const int n_tile = u / p.kchunks, kc0 = u % p.kchunks;
      const int tile_end = (n_tile + 1) * p.kchunks;
      const int seg_end = tile_end < u_end ? tile_end : u_end;
      float acc[2][MBLK][4];
#pragma unroll
      for (int j = 0; j < MBLK; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[0][j][e] = acc[1][j][e] = 0.0f;
      }
      for (; u < seg_end; ++u, ++it) {
        const int stage = it % STAGES;
        bool landed = gs_wait(p, &full_bar[stage], (it / STAGES) & 1);
        if (NORMED && landed) landed = gs_wait(p, &xready_bar[stage], (it / STAGES) & 1);
        if (!__all_sync(0xffffffffu, landed)) {
          atomicOr(p.status, KVB_STATUS_WAIT_TIMEOUT);
          atomicExch(&flags[0], 1);
          break;
        }
        const unsigned wbase = kvb_smem(base + stage * STAGE_BYTES);
        const unsigned xbase = wbase + W_BYTES;
        // fragments of step kk+1 are fetched while the products of step kk are issued; two
        // accumulator chains (even and odd steps) halve the dependent-issue latency
        unsigned a[2][4], b[2][MBLK][2];
        gs_ldmatrix_x4(a[0], wbase + gs_swz(a_row, a_k, GS_NT));
#pragma unroll
        for (int j = 0; j < MBLK; ++j) gs_ldmatrix_x2(b[0][j], xbase + gs_swz(j * 8 + b_row, b_k, MB));
#pragma unroll
        for (int kk = 0; kk < KB / 32; ++kk) {
          const int cur = kk & 1, nxt = cur ^ 1;
          if (kk + 1 < KB / 32) {
            gs_ldmatrix_x4(a[nxt], wbase + gs_swz(a_row, a_k + (kk + 1) * 16, GS_NT));
#pragma unroll
            for (int j = 0; j < MBLK; ++j)
              gs_ldmatrix_x2(b[nxt][j], xbase + gs_swz(j * 8 + b_row, b_k + (kk + 1) * 16, MB));
          }
#pragma unroll
          for (int j = 0; j < MBLK; ++j) gs_mma(acc[cur][j], a[cur], b[cur][j][0], b[cur][j][1]);
        }
        __syncwarp();
        if (lane == 0) kvb_mbar_arrive(&empty_bar[stage]);
      }
#pragma unroll
      for (int j = 0; j < MBLK; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[0][j][e] += acc[1][j][e];
      }
      // ---- the two k-halves meet: warps 4-7 hand theirs to warps 0-3 ----
      if (kh == 1) {
#pragma unroll
        for (int j = 0; j < MBLK; ++j) {
#pragma unroll
          for (int e = 0; e < 4; ++e) halves[(j * 4 + e) * 128 + tid] = acc[0][j][e];
        }
      }
      if (gs_bar_any<1, GS_CONSUMERS * 32>(*reinterpret_cast<volatile int*>(&flags[0]) != 0)) break;   // somebody gave up waiting
      if (kh == 0) {
#pragma unroll
        for (int j = 0; j < MBLK; ++j) {
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[0][j][e] += halves[(j * 4 + e) * 128 + tid];
        }
        if (kc0 != 0) {
          // ---- a part: the tile's first stage is another block's; leave the sums in scratch ----
          float* dst = p.partial + (size_t)me * (MBLK * 4 * 128) + tid;
#pragma unroll
          for (int j = 0; j < MBLK; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) __stcg(dst + (j * 4 + e) * 128, acc[0][j][e]);
          }
          // no fence and no flag: between launches every word of scratch holds a marker (a NaN that
          // no sum can be), and the owner reads each value until it is there
        } else {
          // ---- the owner: add the parts of the blocks behind (in k order), then store ----
          // (residual epilogue: this thread's 8 columns of the residual are asked for now, so that
          // their trip to L2 runs beside the wait for the parts)
          Vec16<bf16> res_early;
          const int res_m = tid >> 3, res_col = n_tile * GS_NT + (tid & 7) * 8;
          const bool res_mine = p.residual != nullptr && res_m < p.M && res_col < p.N;
          if (res_mine) res_early.load(p.residual + (size_t)res_m * p.N + res_col);
          bool complete = true;
          if (seg_end < tile_end) {
            // the blocks behind that hold stages of this tile: their sums are fetched together, every
            // thread reading its own values until none is the marker any more (one trip to L2 when the
            // parts are there, as they are whenever those blocks did them first), then added in k order;
            // the marker goes back in for the next launch
            int parts = 0;
            while (me + 1 + parts < blocks && gs_range_start(p.units, blocks, me + 1 + parts) < tile_end) ++parts;
            for (int c0 = 0; c0 < parts; c0 += 4) {
              const int batch = parts - c0 < 4 ? parts - c0 : 4;
              float part[4][MBLK][4];
              bool there = false;
              for (unsigned spin = 0; spin < p.spin_limit && !there; ++spin) {
                if (spin > 256) __nanosleep(64);               // the blocks finish together: spin first
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                  if (c < batch) {
                    const float* src = p.partial + (size_t)(me + 1 + c0 + c) * (MBLK * 4 * 128) + tid;
#pragma unroll
                    for (int j = 0; j < MBLK; ++j) {
#pragma unroll
                      for (int e = 0; e < 4; ++e) part[c][j][e] = __ldcg(src + (j * 4 + e) * 128);
                    }
                  }
                }
                there = true;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                  if (c < batch) {
#pragma unroll
                    for (int j = 0; j < MBLK; ++j) {
#pragma unroll
                      for (int e = 0; e < 4; ++e) there = there && __float_as_uint(part[c][j][e]) != GS_SCRATCH_MARKER;
                    }
                  }
                }
              }
              if (!there) {
                atomicOr(p.status, KVB_STATUS_WAIT_TIMEOUT);
                atomicExch(&flags[0], 1);
              }
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                if (c < batch) {
                  float* src = p.partial + (size_t)(me + 1 + c0 + c) * (MBLK * 4 * 128) + tid;
#pragma unroll
                  for (int j = 0; j < MBLK; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                      acc[0][j][e] += part[c][j][e];
                      if (there) __stcg(src + (j * 4 + e) * 128, __uint_as_float(GS_SCRATCH_MARKER));
                    }
                  }
                }
              }
            }
            if (gs_bar_any<2, 128>(*reinterpret_cast<volatile int*>(&flags[0]) != 0)) complete = false;
          }
          if (complete) {
            // ---- bias, activation, then through shared memory: the tile leaves as whole 128-byte runs ----
            const int r_lo = rg * 16 + (lane >> 2);               // row of the tile (and r_lo + 8)
            const int width = p.silu_pairs ? GS_NT / 2 : GS_NT;   // output columns this tile makes
            if (!p.silu_pairs) {
#pragma unroll
              for (int j = 0; j < MBLK; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const int r = r_lo + 8 * (e >> 1);
                  const int m = j * 8 + (lane & 3) * 2 + (e & 1);
                  const int n = n_tile * GS_NT + r;
                  float v = acc[0][j][e];
                  if (p.bias && n < p.N) v += __bfloat162float(p.bias[n]);
                  if (p.out_f32) reinterpret_cast<float*>(out_tile)[m * GS_NT + r] = v;
                  else reinterpret_cast<bf16*>(out_tile)[m * GS_NT + r] = __float2bfloat16_rn(v);
                }
              }
            } else {
              // gated pairs: this thread holds gate (row r) and up (row r + 8) of the same output column.
              // Rounded as the unfused path rounds: the products to bf16, the activation to bf16, the result.
              const int n = n_tile * GS_NT + r_lo;                 // the gate row
              const int col = rg * 8 + (lane >> 2);                // the output column inside the tile
#pragma unroll
              for (int j = 0; j < MBLK; ++j) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                  const int m = j * 8 + (lane & 3) * 2 + e;
                  float g = acc[0][j][e], u = acc[0][j][e + 2];
                  if (p.bias && n + 8 < p.N) { g += __bfloat162float(p.bias[n]); u += __bfloat162float(p.bias[n + 8]); }
                  g = __bfloat162float(__float2bfloat16_rn(g));
                  u = __bfloat162float(__float2bfloat16_rn(u));
                  const float act = __bfloat162float(__float2bfloat16_rn(kvb_silu_for_bf16(g)));
                  reinterpret_cast<bf16*>(out_tile)[m * (GS_NT / 2) + col] = __float2bfloat16_rn(act * u);
                }
              }
            }
            asm volatile("bar.sync 2, 128;\n");
            if (p.residual != nullptr) {
              // the tile joins the residual stream: thread (m, piece) adds 8 columns and their squares
              const int m = tid >> 3, piece = tid & 7;
              float sq = 0.0f;
              const int col = n_tile * GS_NT + piece * 8;
              if (res_mine) {                                    // N is a multiple of 8 here
                bf16* rrow = p.residual + (size_t)m * p.N + col;
                Vec16<bf16> o, r = res_early;
                o.raw = *reinterpret_cast<const uint4*>(out_tile + ((size_t)m * GS_NT + piece * 8) * 2);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  r.set(j, o.get(j) + r.get(j));
                  const float v = r.get(j);
                  sq += v * v;
                }
                r.store(rrow);
              }
              // the eight pieces of a token sit in eight neighbouring lanes
              sq += __shfl_xor_sync(0xffffffffu, sq, 1);
              sq += __shfl_xor_sync(0xffffffffu, sq, 2);
              sq += __shfl_xor_sync(0xffffffffu, sq, 4);
              if (piece == 0 && m < p.M) p.sumsq_out[(size_t)m * p.n_tiles + n_tile] = sq;
            } else {
              const int esize = p.out_f32 ? 4 : 2;
              const int col0 = n_tile * width;                       // first output column of the tile
              const int n_out = p.silu_pairs ? p.N / 2 : p.N;
              const int per_row = width * esize / 16;                // 16-byte pieces of a token's run
              unsigned char* gout = reinterpret_cast<unsigned char*>(p.out);
              const bool whole = col0 + width <= n_out && ((size_t)p.ldo * esize) % 16 == 0 &&
                                 (reinterpret_cast<uintptr_t>(gout) + (size_t)col0 * esize) % 16 == 0;
              if (whole) {
                for (int i = tid; i < p.M * per_row; i += 128) {
                  const int m = i / per_row, piece = i % per_row;
                  *reinterpret_cast<uint4*>(gout + ((size_t)m * p.ldo + col0) * esize + piece * 16) =
                      *reinterpret_cast<const uint4*>(out_tile + (size_t)m * width * esize + piece * 16);
                }
              } else {
                for (int i = tid; i < p.M * width; i += 128) {
                  const int m = i / width, c = i % width;
                  if (col0 + c < n_out) {
                    if (p.out_f32) reinterpret_cast<float*>(gout)[(size_t)m * p.ldo + col0 + c] = reinterpret_cast<const float*>(out_tile)[i];
                    else reinterpret_cast<bf16*>(gout)[(size_t)m * p.ldo + col0 + c] = reinterpret_cast<const bf16*>(out_tile)[i];
                  }
                }
              }
            }
            asm volatile("bar.sync 2, 128;\n");   // the tile buffer is free again
          }
        }
      }
      // warps 0-3 have read the halves before they are written again
      if (gs_bar_any<1, GS_CONSUMERS * 32>(*reinterpret_cast<volatile int*>(&flags[0]) != 0)) break;
    }
  }
}

// ---- host side -----------------------------------------------------------------------------
// 3-D bf16 tensor map over a row-major [rows, cols] matrix with leading dimension ld (elements),
// seen as [cols / 64 slabs][rows][64]: boxes of [GS_KG slabs][box_rows][64], 128-byte swizzle, zero
// fill outside.  cols must be a multiple of 64.
static int gs_make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols, long long ld,
                       int box_rows) {
  KvbEncodeTiledFn encode = kvb_encode_tiled_fn();
  KVB_REQUIRE(encode != nullptr, "stream gemm: the driver does not export cuTensorMapEncodeTiled");
  const cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(cols / 64)};
  const cuuint64_t strides[2] = {(cuuint64_t)ld * sizeof(bf16), 64 * sizeof(bf16)};
  const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, GS_KG};
  const cuuint32_t elem[3] = {1, 1, 1};
  const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box,
                             elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  KVB_REQUIRE(rc == CUDA_SUCCESS, "stream gemm: cuTensorMapEncodeTiled failed");
  return 0;
}

// Scratch words for `blocks` blocks (the largest token block).  Before the first launch every word
// holds kvb_gemm_stream_scratch_marker(); the kernel leaves them so.
extern "C" long long kvb_gemm_stream_scratch_floats(int blocks) { return (long long)blocks * 2 * 4 * 128; }
extern "C" unsigned kvb_gemm_stream_scratch_marker() { return GS_SCRATCH_MARKER; }

template <int MBLK, bool NORMED>
static int gs_launch(const void* w, const void* x, long long ldx, StreamParams& p, int sms, cudaStream_t stream) {
  constexpr int MB = 8 * MBLK;
  constexpr size_t SMEM = 1024 + (size_t)GS_STAGES * (GS_NT + MB) * GS_KG * 128 + 1024 +
                          MBLK * 4 * 128 * sizeof(float) + MB * GS_NT * sizeof(float) + (NORMED ? GS_NORM_W_BYTES : 0);
  static bool configured = false;
  if (!configured) {
    KVB_CHECK_CUDA(cudaFuncSetAttribute(gemm_stream_kernel<MBLK, NORMED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
    configured = true;
  }
  alignas(64) CUtensorMap w_map, x_map;
  if (int rc = gs_make_map(&w_map, w, p.N, p.K, p.K, GS_NT)) return rc;
  if (int rc = gs_make_map(&x_map, x, p.M, p.K, ldx, MB)) return rc;
  const int blocks = p.units < sms ? p.units : sms;
  const int threads = NORMED ? GS_THREADS + GS_NORMALISERS * 32 : GS_THREADS;    // NORMED: the normaliser warps
  KVB_CHECK_CUDA(kvb_launch(gemm_stream_kernel<MBLK, NORMED>, dim3(blocks), dim3(threads), SMEM, stream, true, w_map,
                            x_map, p));
  return 0;
}

// For the test of the give-up path only: the NEXT launch of kvb_gemm_stream_bf16 gives up waiting
// after `spin_limit` polls instead of GS_SPIN_LIMIT, and its block `block` never asks for the copies
// of its stage `stage`.  The consumers of that block, and the owners of tiles it shares, then run
// out of polls: they set the status bit KVB_STATUS_WAIT_TIMEOUT, let the copies in flight land and
// return, leaving wrong values in `out`.  Nothing faults and nothing waits without a limit.
static int g_gs_test_block = -1, g_gs_test_stage = -1;
static unsigned g_gs_test_limit = 0;
extern "C" void kvb_gemm_stream_test_give_up(int block, int stage, unsigned spin_limit) {
  g_gs_test_block = block;
  g_gs_test_stage = stage;
  g_gs_test_limit = spin_limit;
}

// Largest K whose norm weights (taken as 32-bit) a NORMED launch keeps in shared memory.
extern "C" int kvb_gemm_stream_norm_max_k() { return GS_NORM_W_BYTES / 4; }

// out[M, N] = x[M, K] . w[N, K]^T (+ bias), 1 <= M <= 16, K a multiple of 64.
//   scratch: kvb_gemm_stream_scratch_floats(sms) words, each holding kvb_gemm_stream_scratch_marker()
//   before the first launch.  Launches that share scratch must be ordered in one stream.
//   silu_pairs: the rows of w come in runs of 8 gate rows, 8 up rows, ...; out is [M, N / 2] with
//   out[m, c] = silu(gate_c(m)) * up_c(m) (the feed-forward's activation fused into the epilogue).
//   norm_weight != null: the rows of x are sums that still need their RMS norm; sumsq_in holds
//   every token's sum of squares in sumsq_pieces pieces ([M, sumsq_pieces]); the kernel uses
//   x' = bf16(norm_weight[k] * (x * rsqrt(sum / K + eps))).  K * (4 or 2 bytes) must fit 16 KB.
//   residual != null ([M, N] bf16, contiguous, N a multiple of 8): the result joins the residual
//   stream: residual = bf16(bf16(out) + residual) in place, and sumsq_out[m, tile] (M x ceil(N / 64)
//   floats) gets the squares of the new sums, 64 columns a piece; out is not written.
extern "C" int kvb_gemm_stream_bf16(void* out, int out_f32, long long ldo, const void* x, long long ldx,
                                    const void* w, const void* bias, int M, int N, int K, int silu_pairs,
                                    const void* norm_weight, int norm_weight_f32, float eps, const float* sumsq_in,
                                    int sumsq_pieces, void* residual, float* sumsq_out, float* scratch, int sms,
                                    cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  KVB_REQUIRE(M > 0 && M <= 16, "stream gemm: takes 1 to 16 rows of x");
  KVB_REQUIRE(K > 0 && K % 64 == 0 && ldx % 8 == 0, "stream gemm: K must be a multiple of 64 and the row stride of x of 8");
  KVB_REQUIRE(aligned16(x) && aligned16(w), "stream gemm: x and w must be 16-byte aligned");
  KVB_REQUIRE(scratch != nullptr && sms > 0, "stream gemm: needs scratch");
  KVB_REQUIRE(!silu_pairs || (N % 16 == 0 && !out_f32), "stream gemm: gated pairs need N a multiple of 16 and a bf16 result");
  KVB_REQUIRE(residual == nullptr || (!silu_pairs && !out_f32 && N % 8 == 0 && sumsq_out != nullptr && aligned16(residual)),
              "stream gemm: the residual epilogue needs a plain bf16 product, N a multiple of 8 and a place for the squares");
  KVB_REQUIRE(norm_weight == nullptr || (sumsq_in != nullptr && sumsq_pieces > 0 && aligned16(norm_weight) &&
                                         (size_t)K * (norm_weight_f32 ? 4 : 2) <= GS_NORM_W_BYTES),
              "stream gemm: the fused norm needs the sums of squares and K small enough for shared memory");
  StreamParams p;
  memset(&p, 0, sizeof(p));
  p.out = out; p.out_f32 = out_f32; p.ldo = ldo;
  p.bias = (const bf16*)bias;
  p.M = M; p.N = N; p.K = K;
  p.silu_pairs = silu_pairs;
  p.norm_weight = norm_weight; p.norm_weight_f32 = norm_weight_f32; p.eps = eps;
  p.sumsq_in = sumsq_in; p.sumsq_pieces = sumsq_pieces;
  p.residual = (bf16*)residual; p.sumsq_out = sumsq_out;
  p.n_tiles = (N + GS_NT - 1) / GS_NT;
  p.kchunks = (K / 64 + GS_KG - 1) / GS_KG;
  KVB_REQUIRE((long long)p.n_tiles * p.kchunks < (1ll << 30), "stream gemm: the matrix is too large");
  p.units = p.n_tiles * p.kchunks;
  p.partial = scratch;
  p.status = kvb_status_word();
  KVB_REQUIRE(p.status != nullptr, "stream gemm: no status word");
  p.spin_limit = g_gs_test_limit ? g_gs_test_limit : GS_SPIN_LIMIT;
  p.test_skip_block = g_gs_test_block;
  p.test_skip_stage = g_gs_test_stage;
  g_gs_test_block = g_gs_test_stage = -1;      // armed for one launch
  g_gs_test_limit = 0;
  if (norm_weight != nullptr) {
    if (M <= 8) return gs_launch<1, true>(w, x, ldx, p, sms, stream);
    return gs_launch<2, true>(w, x, ldx, p, sms, stream);
  }
  if (M <= 8) return gs_launch<1, false>(w, x, ldx, p, sms, stream);
  return gs_launch<2, false>(w, x, ldx, p, sms, stream);
}

KVB_TRACE_TU(gemm_stream)
