// Thin wrappers over the Blackwell (sm_100a) instructions the GEMM kernels are built from: mbarrier,
// TMA tiled loads (never with cluster multicast), tcgen05 tensor-memory allocation, MMA issue, commit and
// tensor-memory loads, plus the shared-memory and instruction descriptors tcgen05.mma consumes.
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace mccl {
namespace umma {

__device__ __forceinline__ uint32_t smemAddr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// ---- mbarrier ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbarInit(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smemAddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbarExpectTx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smemAddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbarArrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smemAddr(bar)) : "memory");
}
__device__ __forceinline__ bool mbarTryWait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.b32 %0, 1, 0, p;\n}"
      : "=r"(done) : "r"(smemAddr(bar)), "r"(parity) : "memory");
  return done != 0;
}
// Bounded wait: gives up after `budgetNs` and returns false (the caller records the failure and unwinds).
__device__ __forceinline__ bool mbarWait(uint64_t* bar, uint32_t parity, uint64_t budgetNs) {
  if (mbarTryWait(bar, parity)) return true;
  uint64_t t0;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
  for (uint32_t spins = 1;; ++spins) {
    if (mbarTryWait(bar, parity)) return true;
    if ((spins & 0xff) == 0) {
      uint64_t t;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
      if (t - t0 > budgetNs) return false;
    }
  }
}
// The same for roles with slack (producer, epilogue): each probe lets the hardware park the thread for up to
// about a microsecond (it resumes as soon as the phase completes), so a waiting warp takes next to no issue
// slots from the MMA-issuing warp on its scheduler.
__device__ __forceinline__ bool mbarWaitParked(uint64_t* bar, uint32_t parity, uint64_t budgetNs) {
  uint64_t t0 = 0;
  for (uint32_t spins = 0;; ++spins) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.b32 %0, 1, 0, p;\n}"
        : "=r"(done) : "r"(smemAddr(bar)), "r"(parity), "r"(1000u) : "memory");
    if (done) return true;
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    if (spins == 0) t0 = t;
    else if (t - t0 > budgetNs) return false;
  }
}
__device__ __forceinline__ void fenceBarrierInit() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// Make generic-proxy writes to global memory visible to the async proxy (TMA) of this thread.
__device__ __forceinline__ void fenceProxyAsyncGlobal() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// ---- TMA ----------------------------------------------------------------------------------------------------
// 2-D tiled load global -> shared, completion signalled on `bar` in bytes.  x = innermost coordinate: its
// byte offset must be a multiple of 16 (here always a multiple of 64 bf16 = 128 bytes).
__device__ __forceinline__ void tmaLoad2d(void* smemDst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :: "r"(smemAddr(smemDst)), "l"(map), "r"(smemAddr(bar)), "r"(x), "r"(y) : "memory");
}
// 2-D tiled store shared -> global (bulk async-group completion).  x = innermost coordinate, a multiple of 64
// bf16 here; the source tile is laid out with the map's 128-byte swizzle.
__device__ __forceinline__ void tmaStore2d(const CUtensorMap* map, const void* smemSrc, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               :: "l"(map), "r"(smemAddr(smemSrc)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmaStoreCommit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until at most N of this thread's store groups still READ their shared-memory source (the buffer may be reused).
template <int N> __device__ __forceinline__ void tmaStoreWaitRead() { asm volatile("cp.async.bulk.wait_group.read %0;" :: "n"(N) : "memory"); }
// Wait until every store group of this thread has completed (its global writes are performed).
__device__ __forceinline__ void tmaStoreWaitAll() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Shared-memory writes of this thread become visible to the async proxy (TMA) after this fence.
__device__ __forceinline__ void fenceProxyAsyncShared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void prefetchTensorMap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" :: "l"(map) : "memory");
}

// ---- tensor memory -------------------------------------------------------------------------------------------
// Whole-warp calls.  `cols` is a power of two >= 32; the base address lands in *smemSlot.
__device__ __forceinline__ void tmemAlloc(uint32_t* smemSlot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smemAddr(smemSlot)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmemRelinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmemDealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- descriptors ----------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor for a K-major bf16 tile written by TMA with the 128-byte swizzle: rows
// of 64 elements (128 bytes), groups of 8 rows 1024 bytes apart.  Fields (16-byte units): start address
// [0,14), leading byte offset [16,30) = 1 (unused for swizzled K-major), stride byte offset [32,46) = 64,
// descriptor version [46,48) = 1, layout type [61,64) = 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smemDescSw128(const void* tile) {
  uint64_t d = 0;
  d |= (uint64_t)((smemAddr(tile) & 0x3ffff) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor of tcgen05.mma.kind::f16 with bf16 A/B (both K-major), fp32 accumulate, M x N.
__host__ __device__ constexpr uint32_t instrDescBf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
__device__ __forceinline__ void mmaBf16(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      :: "r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrive on `bar` once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mmaCommit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smemAddr(bar)) : "memory");
}

// 32 lanes x 32 columns of fp32: thread t of the warp gets row (lane base + t), v[j] = column (col base + j).
__device__ __forceinline__ void tmemLoad32x32(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
        "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
        "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmemLoadWait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace umma
}  // namespace mccl
