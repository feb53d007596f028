// Weight-streaming linear layer for decode: out[M, N] = x[M, K] . W[N, K]^T (+ bias), bf16 in,
// 32-bit accumulate, M <= 64 tokens.  With so few tokens the layer is a stream of the weight
// matrix through the SM, so the kernel is a TMA pipeline with a little tensor-core work hung
// on it (sm_100a).
//
// Persistent blocks walk work items (a tile of 64 weight rows, a chunk of K).  A producer warp
// issues, per stage of 128 k-values, two swizzled TMA boxes of W [64 rows x 64 k] and two of x
// [MB rows x 64 k] (rows beyond M are zero-filled by TMA) into a ring of stages guarded by
// full/empty mbarriers.  Four consumer warps own 16 weight rows each: ldmatrix the W rows as
// the A operand and the token rows as the B operand of mma.sync m16n8k16, so the accumulator
// is [16 weight rows x tokens].  When K is cut into chunks (to have enough items for 148 SMs)
// each item writes its 32-bit partial tile to scratch and bumps the tile's counter; the block
// that arrives last adds the partials in chunk order (so the result does not depend on
// timing), adds the bias and stores.  Counters reset themselves.
//
// All mbarrier waits are bounded (status bit WAIT_TIMEOUT, then drain and return).
#include <cuda.h>
#include <string.h>

#include "common.cuh"

#define SK_NT 64            // weight rows per tile
#define SK_KB 128           // k-values per stage
#define SK_STAGES(MBLK) ((MBLK) == 8 ? 6 : (MBLK) == 4 ? 8 : 10)   // ring depth that fits shared memory
#define SK_CONSUMERS 4
#define SK_THREADS ((SK_CONSUMERS + 1) * 32)
#define SK_SPIN_LIMIT (1u << 22)

struct SkinnyParams {
  void* out; int out_f32; long long ldo;
  const bf16* bias;
  int M, N, K;
  int n_tiles, ksplit, kblocks;      // kblocks = ceil(K / SK_KB)
  float* partial;                    // [ksplit, MB*8 tokens, n_tiles*64]  (ksplit > 1)
  int* counters;                     // [n_tiles], zero between launches
  int* status;
};

__device__ __forceinline__ unsigned sk_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void sk_mbar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(sk_smem(bar)), "r"(count));
}
__device__ __forceinline__ void sk_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(sk_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void sk_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(sk_smem(bar)) : "memory");
}
__device__ __forceinline__ bool sk_wait_bounded(unsigned long long* bar, unsigned parity) {
  for (unsigned spin = 0; spin < SK_SPIN_LIMIT; ++spin) {
    unsigned done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.b32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(sk_smem(bar)), "r"(parity) : "memory");
    if (done) return true;
    if (spin > 64) __nanosleep(64);
  }
  return false;
}
__device__ __forceinline__ void sk_tma_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
      ::"r"(sk_smem(dst)), "l"(reinterpret_cast<unsigned long long>(map)), "r"(x), "r"(y), "r"(sk_smem(bar))
      : "memory");
}
__device__ __forceinline__ void sk_ldmatrix_x4(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void sk_ldmatrix_x2(unsigned (&r)[2], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void sk_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Byte offset of (row, k) in a stage area made of two [rows][128-byte] halves (k 0..63, 64..127),
// 16-byte chunks XOR-swizzled with the row as TMA's 128-byte swizzle lays them out.
__device__ __forceinline__ unsigned sk_swz(int row, int k, int rows) {
  const int half = k >> 6, chunk = (k & 63) >> 3;
  return (unsigned)(half * rows * 128 + row * 128 + ((chunk ^ (row & 7)) << 4));
}

// First k-block and number of k-blocks of chunk `ks` when `kblocks` are dealt to `ksplit` chunks.
__device__ __forceinline__ void sk_chunk(int kblocks, int ksplit, int ks, int& first, int& count) {
  const int base = kblocks / ksplit, extra = kblocks % ksplit;
  first = ks * base + min(ks, extra);
  count = base + (ks < extra ? 1 : 0);
}

template <int MBLK>   // token blocks of 8: MB = 8 * MBLK rows of x per stage
__global__ void __launch_bounds__(SK_THREADS, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map,
                   const SkinnyParams p) {
  constexpr int MB = 8 * MBLK;
  constexpr int W_BYTES = SK_NT * SK_KB * 2;      // 16 KB
  constexpr int X_BYTES = MB * SK_KB * 2;
  constexpr int STAGE_BYTES = W_BYTES + ((X_BYTES + 1023) / 1024) * 1024;
  constexpr int STAGES = SK_STAGES(MBLK);

  extern __shared__ unsigned char sk_dyn[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(sk_dyn) + 1023) & ~uintptr_t(1023));
  unsigned long long* full_bar = reinterpret_cast<unsigned long long*>(base + STAGES * STAGE_BYTES);
  unsigned long long* empty_bar = full_bar + STAGES;
  int* flags = reinterpret_cast<int*>(empty_bar + STAGES);   // [0] abort, [1] "this block reduces"

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_items = p.n_tiles * p.ksplit;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      sk_mbar_init(&full_bar[s], 1);
      sk_mbar_init(&empty_bar[s], SK_CONSUMERS);
    }
    flags[0] = 0;
    flags[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  __syncthreads();

  if (warp == SK_CONSUMERS) {
    // ---------------- producer ----------------
    if (lane == 0) {
      int it = 0, issued = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        const int n_tile = item / p.ksplit, ks = item % p.ksplit;
        int kb0, kbn;
        sk_chunk(p.kblocks, p.ksplit, ks, kb0, kbn);
        for (int kb = kb0; kb < kb0 + kbn; ++kb, ++it) {
          const int stage = it % STAGES;
          if (it >= STAGES && !sk_wait_bounded(&empty_bar[stage], ((it / STAGES) & 1) ^ 1)) {
            atomicOr(p.status, KVB_STATUS_WAIT_TIMEOUT);
            atomicExch(&flags[0], 1);
            ok = false;
            break;
          }
          if (*reinterpret_cast<volatile int*>(&flags[0])) { ok = false; break; }
          unsigned char* wdst = base + stage * STAGE_BYTES;
          unsigned char* xdst = wdst + W_BYTES;
          sk_expect_tx(&full_bar[stage], W_BYTES + X_BYTES);
          const int k = kb * SK_KB;
          sk_tma_2d(wdst, &w_map, k, n_tile * SK_NT, &full_bar[stage]);
          sk_tma_2d(wdst + SK_NT * 128, &w_map, k + 64, n_tile * SK_NT, &full_bar[stage]);
          sk_tma_2d(xdst, &x_map, k, 0, &full_bar[stage]);
          sk_tma_2d(xdst + MB * 128, &x_map, k + 64, 0, &full_bar[stage]);
          issued = it + 1;
        }
      }
      if (*reinterpret_cast<volatile int*>(&flags[0])) {
        for (int j = max(0, issued - STAGES); j < issued; ++j)
          sk_wait_bounded(&full_bar[j % STAGES], (j / STAGES) & 1);
      }
    }
  } else {
    // ---------------- consumers: warp w owns weight rows [16w, 16w+16) of the tile ----------------
    int it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
      const int n_tile = item / p.ksplit, ks = item % p.ksplit;
      int kb0, kbn;
      sk_chunk(p.kblocks, p.ksplit, ks, kb0, kbn);
      float acc[MBLK][4];
#pragma unroll
      for (int j = 0; j < MBLK; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
      for (int kb = 0; kb < kbn; ++kb, ++it) {
        const int stage = it % STAGES;
        if (!sk_wait_bounded(&full_bar[stage], (it / STAGES) & 1)) {
          atomicOr(p.status, KVB_STATUS_WAIT_TIMEOUT);
          atomicExch(&flags[0], 1);
          ok = false;
          break;
        }
        const unsigned wbase = sk_smem(base + stage * STAGE_BYTES);
        const unsigned xbase = wbase + W_BYTES;
#pragma unroll
        for (int kk = 0; kk < SK_KB / 16; ++kk) {
          unsigned a[4];
          {
            const int row = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
            const int k = kk * 16 + 8 * (lane >> 4);
            sk_ldmatrix_x4(a, wbase + sk_swz(row, k, SK_NT));
          }
#pragma unroll
          for (int j = 0; j < MBLK; ++j) {
            unsigned b[2];
            const int row = j * 8 + (lane & 7);
            const int k = kk * 16 + 8 * ((lane >> 3) & 1);
            sk_ldmatrix_x2(b, xbase + sk_swz(row, k, MB));
            sk_mma(acc[j], a, b[0], b[1]);
          }
        }
        __syncwarp();
        if (lane == 0) sk_arrive(&empty_bar[stage]);
      }
      // the consumer warps leave together if any of them gave up waiting
      asm volatile("bar.sync 1, %0;\n" ::"n"(SK_CONSUMERS * 32));
      if (*reinterpret_cast<volatile int*>(&flags[0])) break;
      // ---- this warp's [16 rows x MB tokens] tile: store, or hand to the split-K reduction ----
      const int n_lo = n_tile * SK_NT + warp * 16 + (lane >> 2);
      if (p.ksplit == 1) {
#pragma unroll
        for (int j = 0; j < MBLK; ++j) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int n = n_lo + 8 * (e >> 1);
            const int m = j * 8 + (lane & 3) * 2 + (e & 1);
            if (n < p.N && m < p.M) {
              float v = acc[j][e];
              if (p.bias) v += __bfloat162float(p.bias[n]);
              if (p.out_f32) reinterpret_cast<float*>(p.out)[(size_t)m * p.ldo + n] = v;
              else reinterpret_cast<bf16*>(p.out)[(size_t)m * p.ldo + n] = __float2bfloat16_rn(v);
            }
          }
        }
      } else {
        const size_t plane = (size_t)MB * p.n_tiles * SK_NT;
        float* dst = p.partial + (size_t)ks * plane;
#pragma unroll
        for (int j = 0; j < MBLK; ++j) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int n = n_lo + 8 * (e >> 1);
            const int m = j * 8 + (lane & 3) * 2 + (e & 1);
            dst[(size_t)m * p.n_tiles * SK_NT + n] = acc[j][e];
          }
        }
        // the four consumer warps of this item meet, then one thread counts the item in
        __threadfence();
        asm volatile("bar.sync 1, %0;\n" ::"n"(SK_CONSUMERS * 32));
        if (threadIdx.x == 0) {
          const int seen = atomicAdd(&p.counters[n_tile], 1);
          flags[1] = (seen == p.ksplit - 1);
          if (seen == p.ksplit - 1) p.counters[n_tile] = 0;  // ready for the next launch
        }
        asm volatile("bar.sync 1, %0;\n" ::"n"(SK_CONSUMERS * 32));
        if (flags[1]) {
          __threadfence();
          // last to arrive: add the chunks in order for the 64 rows x MB tokens of the tile
          for (int i = threadIdx.x; i < SK_NT * MB; i += SK_CONSUMERS * 32) {
            const int m = i / SK_NT, n = n_tile * SK_NT + i % SK_NT;
            if (n >= p.N || m >= p.M) continue;
            float v = 0.0f;
            for (int c = 0; c < p.ksplit; ++c)
              v += __ldcg(p.partial + (size_t)c * plane + (size_t)m * p.n_tiles * SK_NT + n);
            if (p.bias) v += __bfloat162float(p.bias[n]);
            if (p.out_f32) reinterpret_cast<float*>(p.out)[(size_t)m * p.ldo + n] = v;
            else reinterpret_cast<bf16*>(p.out)[(size_t)m * p.ldo + n] = __float2bfloat16_rn(v);
          }
        }
        asm volatile("bar.sync 1, %0;\n" ::"n"(SK_CONSUMERS * 32));
      }
    }
  }
}

// ---- host side -----------------------------------------------------------------------------
typedef CUresult (*SkEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static SkEncodeFn sk_encode_fn() {
  static SkEncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<SkEncodeFn>(ptr);
  }
  return fn;
}

// 2-D bf16 tensor map over a row-major [rows, cols] matrix with leading dimension ld (elements),
// boxes of [box_rows, 64 columns], 128-byte swizzle, zero fill outside.
static int sk_make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols, long long ld,
                       int box_rows) {
  SkEncodeFn encode = sk_encode_fn();
  KVB_REQUIRE(encode != nullptr, "skinny gemm: the driver does not export cuTensorMapEncodeTiled");
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(bf16)};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
                             elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  KVB_REQUIRE(rc == CUDA_SUCCESS, "skinny gemm: cuTensorMapEncodeTiled failed");
  return 0;
}

// How K is cut so that there are enough work items for `sms` SMs (each chunk at least 4 stages).
extern "C" int kvb_gemm_skinny_ksplit(int N, int K, int sms) {
  const int n_tiles = (N + SK_NT - 1) / SK_NT;
  const int kblocks = (K + SK_KB - 1) / SK_KB;
  int ksplit = (2 * sms + n_tiles - 1) / n_tiles;
  if (ksplit > kblocks / 4) ksplit = kblocks / 4;
  if (ksplit < 1) ksplit = 1;
  if (ksplit > 16) ksplit = 16;
  return ksplit;
}

// Scratch floats the split-K reduction needs (0 when K is not cut).
extern "C" long long kvb_gemm_skinny_scratch_floats(int M, int N, int ksplit) {
  if (ksplit <= 1) return 0;
  const int mb = M <= 8 ? 8 : M <= 16 ? 16 : M <= 32 ? 32 : 64;
  const long long n_pad = (long long)((N + SK_NT - 1) / SK_NT) * SK_NT;
  return (long long)ksplit * mb * n_pad;
}

template <int MBLK>
static int sk_launch(const CUtensorMap& w_map, const CUtensorMap& x_map, const SkinnyParams& p, int blocks,
                     cudaStream_t stream) {
  constexpr int MB = 8 * MBLK;
  constexpr int STAGE = SK_NT * SK_KB * 2 + ((MB * SK_KB * 2 + 1023) / 1024) * 1024;
  constexpr size_t SMEM = 1024 + (size_t)SK_STAGES(MBLK) * STAGE + 2 * SK_STAGES(MBLK) * 8 + 16;
  static bool configured = false;
  if (!configured) {
    KVB_CHECK_CUDA(cudaFuncSetAttribute(gemm_skinny_kernel<MBLK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
    configured = true;
  }
  gemm_skinny_kernel<MBLK><<<blocks, SK_THREADS, SMEM, stream>>>(w_map, x_map, p);
  KVB_CHECK_LAUNCH();
  return 0;
}

// counters: at least ceil(N/64) ints, zero before the first launch (the kernel leaves them zero).
// scratch: kvb_gemm_skinny_scratch_floats(M, N, ksplit) floats when ksplit > 1.
extern "C" int kvb_gemm_skinny_bf16(void* out, int out_f32, long long ldo, const void* x, long long ldx,
                                    const void* w, const void* bias, int M, int N, int K, int ksplit,
                                    float* scratch, int* counters, int sms, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  KVB_REQUIRE(M > 0 && M <= 64, "skinny gemm: takes 1 to 64 rows of x");
  KVB_REQUIRE(K > 0 && K % 8 == 0 && ldx % 8 == 0, "skinny gemm: K and the row stride of x must be multiples of 8");
  KVB_REQUIRE(aligned16(x) && aligned16(w), "skinny gemm: x and w must be 16-byte aligned");
  KVB_REQUIRE(ksplit >= 1 && ksplit <= 16, "skinny gemm: ksplit must be in [1, 16]");
  SkinnyParams p;
  p.out = out; p.out_f32 = out_f32; p.ldo = ldo;
  p.bias = (const bf16*)bias;
  p.M = M; p.N = N; p.K = K;
  p.n_tiles = (N + SK_NT - 1) / SK_NT;
  p.kblocks = (K + SK_KB - 1) / SK_KB;
  p.ksplit = ksplit > p.kblocks ? p.kblocks : ksplit;
  KVB_REQUIRE(p.ksplit == 1 || (scratch != nullptr && counters != nullptr), "skinny gemm: split K needs scratch and counters");
  p.partial = scratch;
  p.counters = counters;
  p.status = kvb_status_word();
  KVB_REQUIRE(p.status != nullptr, "skinny gemm: no status word");
  const int mblk = M <= 8 ? 1 : M <= 16 ? 2 : M <= 32 ? 4 : 8;
  alignas(64) CUtensorMap w_map, x_map;
  if (int rc = sk_make_map(&w_map, w, N, K, K, SK_NT)) return rc;
  if (int rc = sk_make_map(&x_map, x, M, K, ldx, 8 * mblk)) return rc;
  const int items = p.n_tiles * p.ksplit;
  const int blocks = items < sms ? items : sms;
  switch (mblk) {
    case 1: return sk_launch<1>(w_map, x_map, p, blocks, stream);
    case 2: return sk_launch<2>(w_map, x_map, p, blocks, stream);
    case 4: return sk_launch<4>(w_map, x_map, p, blocks, stream);
    default: return sk_launch<8>(w_map, x_map, p, blocks, stream);
  }
}
