// The asynchronous machinery of sm_100a as inline PTX, shared by the kernels that use it:
// mbarriers (every wait bounded), TMA tensor copies, shared-memory descriptors and the tcgen05
// instructions (MMA with accumulators in tensor memory, commit, loads and stores of tensor
// memory), and the acquire/release accesses used to hand data from block to block.
#pragma once

#include <cuda.h>

#include "common.cuh"

__device__ __forceinline__ unsigned kvb_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

// ---- mbarriers ------------------------------------------------------------------------------
__device__ __forceinline__ void kvb_mbar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(kvb_smem(bar)), "r"(count));
}
// After the barriers of a block are initialised: visible to the async proxy (TMA, tcgen05.commit).
__device__ __forceinline__ void kvb_mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}
__device__ __forceinline__ void kvb_mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(kvb_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void kvb_mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(kvb_smem(bar)) : "memory");
}
__device__ __forceinline__ bool kvb_mbar_try_wait(unsigned long long* bar, unsigned parity) {
  unsigned done;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n}\n"
      : "=r"(done) : "r"(kvb_smem(bar)), "r"(parity) : "memory");
  return done != 0;
}
// Waits for the phase of `parity` to complete; gives up (false) after LIMIT polls.  The first
// SPIN polls follow each other directly (short hand-offs), the later ones sleep 64 ns between.
template <unsigned LIMIT, unsigned SPIN>
__device__ __forceinline__ bool kvb_mbar_wait(unsigned long long* bar, unsigned parity) {
  for (unsigned poll = 0; poll < LIMIT; ++poll) {
    if (kvb_mbar_try_wait(bar, parity)) return true;
    if (poll > SPIN) __nanosleep(64);
  }
  return false;
}
// The same with the limit chosen at run time.
__device__ __forceinline__ bool kvb_mbar_wait_n(unsigned long long* bar, unsigned parity, unsigned limit, unsigned spin) {
  for (unsigned poll = 0; poll < limit; ++poll) {
    if (kvb_mbar_try_wait(bar, parity)) return true;
    if (poll > spin) __nanosleep(64);
  }
  return false;
}
// Generic-proxy writes to shared memory made visible to the async proxy (TMA, tensor cores).
__device__ __forceinline__ void kvb_fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// ---- TMA ------------------------------------------------------------------------------------
__device__ __forceinline__ void kvb_tma_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
      ::"r"(kvb_smem(dst)), "l"(reinterpret_cast<unsigned long long>(map)), "r"(x), "r"(y), "r"(kvb_smem(bar))
      : "memory");
}
__device__ __forceinline__ void kvb_tma_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2,
                                           unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
      ::"r"(kvb_smem(dst)), "l"(reinterpret_cast<unsigned long long>(map)), "r"(c0), "r"(c1), "r"(c2),
        "r"(kvb_smem(bar))
      : "memory");
}
__device__ __forceinline__ void kvb_tma_4d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                           unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];\n"
      ::"r"(kvb_smem(dst)), "l"(reinterpret_cast<unsigned long long>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
        "r"(kvb_smem(bar))
      : "memory");
}
// Untiled copy of `bytes` (a multiple of 16, both addresses 16-byte aligned) from global to shared memory.
__device__ __forceinline__ void kvb_bulk_copy(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
               ::"r"(kvb_smem(dst)), "l"(src), "r"(bytes), "r"(kvb_smem(bar)) : "memory");
}

// ---- block-to-block hand-over through global memory -------------------------------------------
__device__ __forceinline__ int kvb_ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void kvb_st_release(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}

// ---- tcgen05 --------------------------------------------------------------------------------
// Shared-memory matrix descriptor: 128-byte swizzle, version 1 (sm_100); leading and stride byte offsets.
__device__ __forceinline__ unsigned long long kvb_tc5_desc(unsigned addr, unsigned lbo_bytes, unsigned sbo_bytes) {
  return (unsigned long long)((addr & 0x3FFFFu) >> 4) | ((unsigned long long)(lbo_bytes >> 4) << 16) |
         ((unsigned long long)(sbo_bytes >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: f32 accumulate, bf16 x bf16, M x N; b_mn_major: B is MN-major (else both K-major).
__device__ __forceinline__ unsigned kvb_tc5_idesc(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((unsigned)(n >> 3) << 17) |
         ((unsigned)(m >> 4) << 24);
}
// D[tmem] (+)= A[smem] . B[smem], issued by one thread.
__device__ __forceinline__ void kvb_tc5_mma(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc,
                                            unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// D[tmem] (+)= A[tmem] . B[smem]: A is 128 lanes x 8 columns (16 bf16 a lane, two to a column).
__device__ __forceinline__ void kvb_tc5_mma_ts(unsigned tmem_d, unsigned tmem_a, unsigned long long bdesc,
                                               unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// Eight MMAs of one 128-wide k-range in ONE instruction sequence: D[tmem] (+)= A . B with the operands'
// descriptors advanced by constants (in units of 16 bytes) from step to step: a_step / b_step per k-step of
// 16, and a_jump / b_jump added once after the fourth step (the second 64-column half of a swizzled tile).
// The first product overwrites D unless `accumulate`; the others add.  Written as one block so that the
// issuing thread, which is alone in its warp and pays several cycles for every dependent instruction, has
// nothing but eight tcgen05.mma and their descriptor additions to execute.
template <int A_STEP, int A_JUMP, int B_STEP, int B_JUMP>
__device__ __forceinline__ void kvb_tc5_mma8_ss(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc,
                                                unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n.reg .pred p, q;\n.reg .b64 a, b;\n"
      "setp.ne.b32 p, %4, 0;\nsetp.eq.b32 q, 0, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "add.u64 a, %1, %5;\nadd.u64 b, %2, %7;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, q;\n"
      "add.u64 a, a, %5;\nadd.u64 b, b, %7;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, q;\n"
      "add.u64 a, a, %5;\nadd.u64 b, b, %7;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, q;\n"
      "add.u64 a, a, %6;\nadd.u64 b, b, %8;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, q;\n"
      "add.u64 a, a, %5;\nadd.u64 b, b, %7;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, q;\n"
      "add.u64 a, a, %5;\nadd.u64 b, b, %7;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, q;\n"
      "add.u64 a, a, %5;\nadd.u64 b, b, %7;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, q;\n}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate),
        "n"(A_STEP), "n"(A_JUMP), "n"(B_STEP), "n"(B_JUMP) : "memory");
}
// The same with A in tensor memory: its address advances by A_COLS columns a step, B's descriptor by B_STEP.
template <int A_COLS, int B_STEP>
__device__ __forceinline__ void kvb_tc5_mma8_ts(unsigned tmem_d, unsigned tmem_a, unsigned long long bdesc,
                                                unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n.reg .pred p, q;\n.reg .b64 b;\n.reg .b32 a;\n"
      "setp.ne.b32 p, %4, 0;\nsetp.eq.b32 q, 0, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "add.u32 a, %1, %5;\nadd.u64 b, %2, %6;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, q;\n"
      "add.u32 a, a, %5;\nadd.u64 b, b, %6;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, q;\n"
      "add.u32 a, a, %5;\nadd.u64 b, b, %6;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, q;\n"
      "add.u32 a, a, %5;\nadd.u64 b, b, %6;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, q;\n"
      "add.u32 a, a, %5;\nadd.u64 b, b, %6;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, q;\n"
      "add.u32 a, a, %5;\nadd.u64 b, b, %6;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, q;\n"
      "add.u32 a, a, %5;\nadd.u64 b, b, %6;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, q;\n}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate), "n"(A_COLS), "n"(B_STEP) : "memory");
}
// The barrier gets an arrival when every MMA issued so far by this thread has finished.
__device__ __forceinline__ void kvb_tc5_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(kvb_smem(bar)) : "memory");
}
__device__ __forceinline__ void kvb_tc5_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void kvb_tc5_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// Whole warp: `columns` (a power of two, 32..512) of tensor memory for this block; the address lands in *slot (shared).
__device__ __forceinline__ void kvb_tc5_alloc(unsigned* slot, unsigned columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(kvb_smem(slot)), "r"(columns));
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
}
__device__ __forceinline__ void kvb_tc5_dealloc(unsigned tmem_base, unsigned columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(columns));
}
// Warp w of a warpgroup reads / writes lanes [32 (w mod 4), +32): 32 consecutive columns of this thread's lane.
__device__ __forceinline__ void kvb_tc5_ld32(unsigned taddr, float (&v)[32]) {
  unsigned* r = reinterpret_cast<unsigned*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void kvb_tc5_st32(unsigned taddr, const float (&v)[32]) {
  const unsigned* r = reinterpret_cast<const unsigned*>(v);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void kvb_tc5_st16(unsigned taddr, const float (&v)[16]) {
  const unsigned* r = reinterpret_cast<const unsigned*>(v);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void kvb_tc5_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void kvb_tc5_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// ---- host side: tensor maps -------------------------------------------------------------------
// cuTensorMapEncodeTiled through the runtime's driver entry point (the library does not link the
// driver); null if the driver does not export it.
typedef CUresult (*KvbEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                     CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline KvbEncodeTiledFn kvb_encode_tiled_fn() {
  static KvbEncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<KvbEncodeTiledFn>(ptr);
  }
  return fn;
}
