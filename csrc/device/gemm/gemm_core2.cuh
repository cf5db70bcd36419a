// Two-SM form of the bf16 GEMM: a cluster of two CTAs works on one 256 x BN output tile with
// tcgen05.mma.cta_group::2 (M = 256).  Each CTA stages its own 128 rows of A and its own half of the B tile
// (BN/2 rows), so a pair moves half the B bytes through shared memory per FLOP that two independent CTAs
// would, and the stage is small enough for a ring of seven or eight stages.
//
//   CTA 0 of the pair ("leader")            CTA 1
//   warp 0  TMA: A rows [0,128), B rows      TMA: A rows [128,256), B rows [BN/2, BN) of the tile; all four
//           [0, BN/2) of the tile             loads of a stage complete on the LEADER's full barrier
//   warp 1  issues the MMAs for both CTAs,   idle
//           commits to the empty / tmemFull
//           barriers of both CTAs
//   warp 2  allocates / frees tensor memory (cta_group::2: one warp of each CTA takes part)
//   warps 4-7 epilogue of the CTA's own 128 rows; both CTAs release the accumulator on the leader's barrier
//
// Each CTA fetches what it needs itself: no load is shared between the CTAs of a pair.  Every wait is bounded, as in
// the one-SM kernel; a CTA that gives up leaves its loops, and its partner then runs into its own time limit
// before both meet at the closing cluster barrier.  No counterpart in the reference.
#pragma once

#include "gemm_core.cuh"

namespace mccl {
namespace gemm {

constexpr int BM2 = 256;               // rows of a pair's tile
constexpr int kThreadsGemm2 = 256;

template <int BN> struct Smem2 {
  static constexpr int A_BYTES = BM * BK * 2;              // this CTA's 128 rows
  static constexpr int B_BYTES = (BN / 2) * BK * 2;        // this CTA's half of the B tile
  // Epilogue staging: per epilogue warp two buffers of 32 rows x 128 bytes (64 bf16), from which TMA stores go out.
  static constexpr int EPI_BYTES = 4 * 2 * 32 * 128;
  // as many stages as fit beside that and the barriers in the 227 KB a CTA may use, eight at most (BN 256 and 224: six)
  static constexpr int FIT = (232448 - 1536 - EPI_BYTES) / (A_BYTES + B_BYTES);
  static constexpr int STAGES = FIT > 8 ? 8 : FIT;
  static constexpr int TILE_BYTES = STAGES * (A_BYTES + B_BYTES);
  static constexpr int TOTAL = TILE_BYTES + EPI_BYTES + 512 + 1024;    // + barriers + alignment slack
};

namespace umma2 {

__device__ __forceinline__ uint32_t clusterCtaRank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of `localAddr` (a shared::cta address) in the shared memory of CTA `cta` of this cluster.
__device__ __forceinline__ uint32_t mapToCta(uint32_t localAddr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(localAddr), "r"(cta));
  return r;
}
// Barrier over all threads of both CTAs (the form that does not require converged warps).
__device__ __forceinline__ void clusterSync() {
  asm volatile("barrier.cluster.arrive.release;\n barrier.cluster.wait.acquire;" ::: "memory");
}
// Arrive on a barrier that may live in the partner CTA (shared::cluster address).
__device__ __forceinline__ void mbarArriveCluster(uint32_t clusterAddr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" :: "r"(clusterAddr) : "memory");
}
// 2-D tiled load into this CTA's shared memory whose completion bytes are counted on a barrier of either CTA
// of the pair (shared::cluster address).
__device__ __forceinline__ void tmaLoad2dPair(void* smemDst, const CUtensorMap* map, uint32_t barClusterAddr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :: "r"(umma::smemAddr(smemDst)), "l"(map), "r"(barClusterAddr), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmemAlloc(uint32_t* smemSlot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(umma::smemAddr(smemSlot)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmemRelinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmemDealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(cols) : "memory");
}
// D (128 lanes in each CTA's tensor memory) (+)= A (128 rows from each CTA) * B (BN/2 rows from each CTA).
__device__ __forceinline__ void mmaBf16(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
      :: "r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with the descriptors given as (low word, high word): stepping along K only changes the low word,
// which saves the 64-bit additions in the one thread that issues every MMA of the pair.
__device__ __forceinline__ void mmaBf16Split(uint32_t tmemD, uint32_t aLo, uint32_t bLo, uint32_t descHi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n .reg .b64 da, db;\n mov.b64 da, {%1, %3};\n mov.b64 db, {%2, %3};\n setp.ne.b32 p, %5, 0;\n"
      " tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n}"
      :: "r"(tmemD), "r"(aLo), "r"(bLo), "r"(descHi), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mmaCommitMaskAddr(uint32_t barAddr, uint16_t mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               :: "r"(barAddr), "h"(mask) : "memory");
}
// Four fp32 added to global memory in one instruction (performed at L2).
__device__ __forceinline__ void redAddF32x4(float* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" :: "l"(p), "f"(__uint_as_float(a)), "f"(__uint_as_float(b)),
               "f"(__uint_as_float(c)), "f"(__uint_as_float(d)) : "memory");
}
// Arrive on the barrier at this offset in both CTAs once every MMA issued so far has completed: one commit per
// CTA, each naming that CTA's barrier by its shared::cluster address (a commit tracks all earlier MMAs of the
// issuing thread, so the two are independent observers of the same work).
__device__ __forceinline__ void mmaCommitTo(uint32_t barClusterAddr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(barClusterAddr) : "memory");
}
// One instruction that arrives on the barrier at this offset in every CTA of `mask` (a commit, not a load).
__device__ __forceinline__ void mmaCommitMask(uint64_t* bar, uint16_t mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               :: "r"(umma::smemAddr(bar)), "h"(mask) : "memory");
}
__device__ __forceinline__ void mmaCommitBoth(uint64_t* bar) {
  const uint32_t local = umma::smemAddr(bar);
  mmaCommitTo(mapToCta(local, 0));
  mmaCommitTo(mapToCta(local, 1));
}

}  // namespace umma2

// Launched as clusters of two CTAs (cluster dimension attribute of the launch).  Threads: 256 in the plain
// mode, 384 (communication warps 8-11) in the fused modes.
// VAR selects how the MMA thread is written (bit 0: one commit instruction for both CTAs' barriers instead of
// two; bit 1: wait for the next stage between the MMAs of the current one).
template <int BN, int MODE, int VAR>
__global__ void __launch_bounds__(MODE == MODE_PLAIN ? kThreadsGemm2 : kThreadsGemm, 1) tpGemm2Kernel(const __grid_constant__ GemmArgs a) {
  using S = Smem2<BN>;
  constexpr int STAGES2 = S::STAGES;
  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES2 * S::A_BYTES;
  uint8_t* sEpi = smem + S::TILE_BYTES;            // 1024-byte aligned: every tile size is a multiple of 1024
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::TILE_BYTES + S::EPI_BYTES);
  uint64_t* full = bars;                          // [STAGES2] used in the leader: all four loads of a stage
  uint64_t* empty = bars + STAGES2;               // [STAGES2] in each CTA: the MMAs have read the stage
  uint64_t* tmemFull = bars + 2 * STAGES2;        // [2] in each CTA: accumulator complete
  uint64_t* tmemEmpty = bars + 2 * STAGES2 + 2;   // [2] used in the leader: both epilogues have drained it
  uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES2 + 4);
  volatile int* sFail = reinterpret_cast<volatile int*>(tmemSlot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t ctaRank = umma2::clusterCtaRank();
  const int pair = blockIdx.x >> 1, numPairs = gridDim.x >> 1;
  const int tilesN = a.N / BN, stripes = a.M / BM2, kBlocks = a.K / BK;     // stripes of 256 rows
  const int totalTiles = tilesN * stripes;
  const int n = (MODE == MODE_PLAIN) ? 1 : a.peers.n, rank = (MODE == MODE_PLAIN) ? 0 : a.peers.rank;
  const int stripesPerBlock = stripes / n;          // 256-row stripes of one rank's row block
  const uint64_t budget = a.budgetNs;
  // Split tail (see GemmArgs): this pair's slice of one of the last tiles, if any.
  const int mainTiles = totalTiles - a.tailTiles;
  const bool hasTail = a.tailTiles > 0 && pair < a.tailTiles * a.tailSlices;
  const int tailIdx = hasTail ? pair / a.tailSlices : 0;                       // which of the tail tiles
  const int tailSlice = hasTail ? pair - tailIdx * a.tailSlices : 0;
  const int tailKb0 = hasTail ? (int)((long long)tailSlice * kBlocks / a.tailSlices) : 0;
  const int tailLen = hasTail ? (int)((long long)(tailSlice + 1) * kBlocks / a.tailSlices) - tailKb0 : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2; ++s) { umma::mbarInit(&full[s], 1); umma::mbarInit(&empty[s], 1); }
    for (int i = 0; i < 2; ++i) { umma::mbarInit(&tmemFull[i], 1); umma::mbarInit(&tmemEmpty[i], 8); }
    *sFail = 0;
    umma::fenceBarrierInit();
    umma::prefetchTensorMap(&a.mapA);
    umma::prefetchTensorMap(&a.mapB);
    if (a.tmaStore) umma::prefetchTensorMap(&a.mapC);
  }
  if (warp == 2) { umma2::tmemAlloc(tmemSlot, kTmemCols); umma2::tmemRelinquish(); }
  umma::tcFenceBefore();
  __syncthreads();
  umma2::clusterSync();                            // both CTAs' barriers exist before anything signals them
  umma::tcFenceAfter();
  const uint32_t tmemBase = *tmemSlot;

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer (both CTAs)
    int stage = 0; uint32_t phase = 0;
    const bool noLoads = a.debug & 1;
    // main tiles, whole K each; then this pair's slice of a tail tile
    for (int t = pair, turn = 0; *sFail == 0; t += numPairs, ++turn) {
      const bool tail = t >= mainTiles;
      if (tail && !hasTail) break;
      const int tile = tail ? mainTiles + tailIdx : t;
      int stripe, nt;
      tileCoords<MODE>(tile, tilesN, a.panel, stripesPerBlock, rank, n, &stripe, &nt);
      if (MODE == MODE_AG) {
        const int shard = stripe / stripesPerBlock;
        if (!waitGpuFlag(&a.shardReady[shard], (uint64_t)gridDim.x, budget)) { *sFail = 1; atomicExch(a.errFlag, 20); break; }
        umma::fenceProxyAsyncGlobal();
      }
      const int kbLo = tail ? tailKb0 : 0, kbHi = tail ? tailKb0 + tailLen : kBlocks;
      for (int kb = kbLo; kb < kbHi; ++kb) {
        if (!umma::mbarWaitParked(&empty[stage], phase ^ 1, budget)) { *sFail = 1; atomicExch(a.errFlag, 21); break; }
        if (noLoads && (turn != 0 || kb >= STAGES2)) {       // tuning aid: the whole handshake, no data
          if (ctaRank == 0) umma::mbarArrive(&full[stage]);
          if (++stage == STAGES2) { stage = 0; phase ^= 1; }
          continue;
        }
        if (ctaRank == 0) umma::mbarExpectTx(&full[stage], 2 * (S::A_BYTES + S::B_BYTES));
        const uint32_t leaderFull = umma2::mapToCta(umma::smemAddr(&full[stage]), 0);
        umma2::tmaLoad2dPair(sA + stage * S::A_BYTES, &a.mapA, leaderFull, kb * BK, stripe * BM2 + (int)ctaRank * BM);
        umma2::tmaLoad2dPair(sB + stage * S::B_BYTES, &a.mapB, leaderFull, kb * BK, nt * BN + (int)ctaRank * (BN / 2));
        if (++stage == STAGES2) { stage = 0; phase ^= 1; }
      }
      if (tail) break;
    }
  } else if (warp == 1 && lane == 0 && ctaRank == 0) {
    // ---------------- MMA issuer (leader only)
    // This one thread feeds the tensor cores of both SMs, and what it executes between two MMAs is time in
    // which nothing new gets queued, so the loop is kept short: one flat count of (tile, k block) steps, the ring
    // of stages unrolled so that every barrier and descriptor is the base plus a constant, descriptors stepped
    // in their low word only, and (VAR bit 1) the wait for the NEXT stage placed between the second and the
    // third MMA of the current one, where two queued MMAs hide the barrier's round trip.
    constexpr uint32_t idesc = umma::instrDescBf16(BM2, BN);
    constexpr bool kMcCommit = (VAR & 1) != 0, kEarlyWait = (VAR & 2) != 0;
    const uint64_t descA0 = umma::smemDescSw128(sA), descB0 = umma::smemDescSw128(sB);
    const uint32_t aLo0 = (uint32_t)descA0, bLo0 = (uint32_t)descB0, descHi = (uint32_t)(descA0 >> 32);
    const uint32_t emptyAddr = umma::smemAddr(empty), tmemFullAddr = umma::smemAddr(tmemFull);
    const uint32_t emptyPeer = umma2::mapToCta(emptyAddr, 1), tmemFullPeer = umma2::mapToCta(tmemFullAddr, 1);
    const int myTiles = pair < mainTiles ? (mainTiles - pair + numPairs - 1) / numPairs : 0;
    int remaining = myTiles * kBlocks + tailLen;
    int tilesStarted = 0, curLen = kBlocks;          // k blocks of the tile being accumulated (the tail slice is shorter)
    int kb = 0, acc = 0; uint32_t phase = 0, accPhase = 0;
    uint32_t d = tmemBase;
    bool fail = false;
    if (kEarlyWait && remaining > 0 && !umma::mbarWait(&full[0], 0, budget)) { fail = true; *sFail = 1; atomicExch(a.errFlag, 23); }
    while (remaining > 0 && !fail) {
#pragma unroll
      for (int s = 0; s < STAGES2; ++s) {
        if (remaining == 0) break;
        if (kb == 0) {
          if (*sFail != 0) { fail = true; break; }
          if (!umma::mbarWait(&tmemEmpty[acc], accPhase ^ 1, budget)) { fail = true; *sFail = 1; atomicExch(a.errFlag, 22); break; }
          d = tmemBase + (uint32_t)acc * 256u;
          curLen = tilesStarted < myTiles ? kBlocks : tailLen;
          ++tilesStarted;
        }
        if (!kEarlyWait && !umma::mbarWait(&full[s], phase, budget)) { fail = true; *sFail = 1; atomicExch(a.errFlag, 23); break; }
        umma::tcFenceAfter();
        const uint32_t aLo = aLo0 + (uint32_t)(s * (S::A_BYTES >> 4)), bLo = bLo0 + (uint32_t)(s * (S::B_BYTES >> 4));
        umma2::mmaBf16Split(d, aLo, bLo, descHi, idesc, (uint32_t)kb);
        umma2::mmaBf16Split(d, aLo + 2, bLo + 2, descHi, idesc, 1);
        if (kEarlyWait && remaining > 1) {
          const int ns = (s + 1) % STAGES2;
          if (!umma::mbarWait(&full[ns], ns == 0 ? phase ^ 1 : phase, budget)) { fail = true; *sFail = 1; atomicExch(a.errFlag, 23); }
        }
        umma2::mmaBf16Split(d, aLo + 4, bLo + 4, descHi, idesc, 1);
        umma2::mmaBf16Split(d, aLo + 6, bLo + 6, descHi, idesc, 1);
        if (kMcCommit) umma2::mmaCommitMaskAddr(emptyAddr + 8u * s, 3);
        else { umma2::mmaCommitTo(emptyAddr + 8u * s); umma2::mmaCommitTo(emptyPeer + 8u * s); }
        --remaining;
        if (++kb == curLen) {
          kb = 0;
          if (kMcCommit) umma2::mmaCommitMaskAddr(tmemFullAddr + 8u * acc, 3);
          else { umma2::mmaCommitTo(tmemFullAddr + 8u * acc); umma2::mmaCommitTo(tmemFullPeer + 8u * acc); }
          acc ^= 1; if (acc == 0) accPhase ^= 1;
        }
        if (fail) break;
      }
      phase ^= 1;
    }
  } else if (warp >= 4 && warp < 8) {
    // ---------------- epilogue (both CTAs, own 128 rows)
    const int q = warp - 4;
    int acc = 0; uint32_t accPhase = 0;
    uint32_t epiCount = 0;                          // chunks staged so far: consecutive chunks alternate buffers, across tiles too
    for (int t = pair; t < mainTiles; t += numPairs) {
      int stripe, nt;
      tileCoords<MODE>(t, tilesN, a.panel, stripesPerBlock, rank, n, &stripe, &nt);
      bool good = *sFail == 0 && umma::mbarWaitParked(&tmemFull[acc], accPhase, budget);
      if (!good && *sFail == 0) { *sFail = 1; atomicExch(a.errFlag, 24); }
      if (MODE == MODE_RS) good = !namedBarrierOr(1, 128, !good);     // the four warps meet at a barrier below
      if (!good) break;
      umma::tcFenceAfter();
      const int stripe128 = stripe * 2 + (int)ctaRank;                 // this CTA's 128 rows of the pair's tile
      const size_t row = (size_t)stripe128 * BM + q * 32 + lane;
      __nv_bfloat16* dstRow = a.C + row * (size_t)a.N + (size_t)nt * BN;
      // Whole 64-column chunks leave through shared memory and one TMA store per warp and chunk (each warp its 32
      // rows: no barrier between warps); a 32-column remainder of BN, and everything when the tuning aid asks
      // for it, takes the per-thread stores below.
      const bool viaTma = a.tmaStore && !(a.debug & 4);
      int cDone = 0;
      if (viaTma) {
        uint8_t* myEpi = sEpi + q * 8192;
#pragma unroll 1
        for (int c64 = 0; c64 < BN / 64; ++c64) {
          uint8_t* buf = myEpi + (epiCount++ & 1) * 4096;
          uint32_t v[64];
          const uint32_t taddr = tmemBase + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * 256u + (uint32_t)c64 * 64u;
          umma::tmemLoad32x32(taddr, v);
          umma::tmemLoad32x32(taddr + 32u, v + 32);
          if (lane == 0) umma::tmaStoreWaitRead<1>();          // the store that read this buffer two chunks ago is done with it
          umma::tmemLoadWait();
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 o;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float x0 = __uint_as_float(v[8 * j + 2 * e]), x1 = __uint_as_float(v[8 * j + 2 * e + 1]);
              if (a.epilogue == EPI_SILU) { x0 = silu(x0); x1 = silu(x1); }
              o2[e] = __floats2bfloat162_rn(x0, x1);
            }
            // 128-byte swizzle: 16-byte chunk j of row r sits at chunk j ^ (r % 8)
            *reinterpret_cast<uint4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) = o;
          }
          umma::fenceProxyAsyncShared();
          __syncwarp();
          if (lane == 0 && !(a.debug & 2)) {
            umma::tmaStore2d(&a.mapC, buf, nt * BN + c64 * 64, stripe128 * BM + q * 32);
            umma::tmaStoreCommit();
          }
        }
        cDone = (BN / 64) * 2;
      }
#pragma unroll 1
      for (int c = cDone; c < BN / 32; ++c) {
        uint32_t v[32];
        umma::tmemLoad32x32(tmemBase + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * 256u + (uint32_t)c * 32u, v);
        umma::tmemLoadWait();
        uint4 outv[4];
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(outv);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float x0 = __uint_as_float(v[2 * j]), x1 = __uint_as_float(v[2 * j + 1]);
          if (a.epilogue == EPI_SILU) { x0 = silu(x0); x1 = silu(x1); }
          o2[j] = __floats2bfloat162_rn(x0, x1);
        }
        uint4* dst = reinterpret_cast<uint4*>(dstRow + c * 32);
        if (a.debug & 2) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) dst[j] = outv[j];
      }
      umma::tcFenceBefore();
      __syncwarp();
      if (lane == 0) umma2::mbarArriveCluster(umma2::mapToCta(umma::smemAddr(&tmemEmpty[acc]), 0));
      acc ^= 1; if (acc == 0) accPhase ^= 1;
      if (MODE == MODE_RS) {
        // Count the tile towards its 128-row stripe; tell the owner of the row block when the stripe is whole.
        if (viaTma && lane == 0) { umma::tmaStoreWaitAll(); umma::fenceProxyAsyncGlobal(); }   // this warp's rows of the tile are written
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 4 && lane == 0) {
          __threadfence_system();
          const unsigned long long doneNow = atomicAdd(reinterpret_cast<unsigned long long*>(&a.stripeCount[stripe128]), 1ull) + 1ull;
          if (doneNow == (uint64_t)tilesN) {
            const int per128 = 2 * stripesPerBlock;
            const int owner = stripe128 / per128, within = stripe128 - owner * per128;
            __threadfence_system();
            stReleaseSys(&a.tileReadyPeer[owner][(size_t)rank * per128 + within], a.callIndex);
          }
        }
      }
    }
    if (hasTail && MODE != MODE_RS) {
      // ---- this pair's K slice of a tail tile: add the fp32 partial into the workspace; the CTA that adds last
      // turns the sum into C and leaves the workspace and its counter zero for the next launch.
      int stripe, nt;
      tileCoords<MODE>(mainTiles + tailIdx, tilesN, a.panel, stripesPerBlock, rank, n, &stripe, &nt);
      bool good = *sFail == 0 && umma::mbarWaitParked(&tmemFull[acc], accPhase, budget);
      if (!good && *sFail == 0) { *sFail = 1; atomicExch(a.errFlag, 24); }
      good = !namedBarrierOr(1, 128, !good);
      if (good) {
        umma::tcFenceAfter();
        // This CTA's 128 rows of the tile's sum, kept as [column quad][row][4]: the 32 lanes of one `red` (32 rows,
        // one quad) touch 512 contiguous bytes instead of 32 rows a kilobyte apart.
        float* half = a.tailWs + ((size_t)tailIdx * BM2 + (size_t)ctaRank * BM) * BN;
        float* wsRow = half + (size_t)(q * 32 + lane) * 4;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          umma::tmemLoad32x32(tmemBase + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * 256u + (uint32_t)c * 32u, v);
          umma::tmemLoadWait();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            umma2::redAddF32x4(wsRow + (size_t)(c * 8 + j) * (BM * 4), v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
        umma::tcFenceBefore();
        __threadfence();
        int last = 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 4 && lane == 0) last = atomicAdd(&a.tailCount[tailIdx * 2 + (int)ctaRank], 1u) == (unsigned)(a.tailSlices - 1);
        if (namedBarrierOr(1, 128, last != 0)) {
          __threadfence();
          const int row = threadIdx.x - 128;                  // one output row per thread, 16 columns (one 32-byte sector) at a time
          __nv_bfloat16* cRow = a.C + ((size_t)(stripe * 2 + (int)ctaRank) * BM + row) * (size_t)a.N + (size_t)nt * BN;
          float4* sum4 = reinterpret_cast<float4*>(half) + row;
          // Eight loads in flight per thread: with one, the 128 threads would spend the L2 latency 64 times over.
#pragma unroll 1
          for (int c16 = 0; c16 < BN / 16; c16 += 2) {
            float4 x[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) x[u] = __ldcg(sum4 + (size_t)(c16 * 4 + u) * BM);
#pragma unroll
            for (int u = 0; u < 8; ++u) __stcg(sum4 + (size_t)(c16 * 4 + u) * BM, make_float4(0.f, 0.f, 0.f, 0.f));
#pragma unroll
            for (int h = 0; h < 4; ++h) {                     // two quads = 8 columns = one 16-byte store
              uint32_t o[4];
#pragma unroll
              for (int k = 0; k < 2; ++k) {
                float4 y = x[h * 2 + k];
                if (a.epilogue == EPI_SILU) { y.x = silu(y.x); y.y = silu(y.y); y.z = silu(y.z); y.w = silu(y.w); }
                __nv_bfloat162 lo = __floats2bfloat162_rn(y.x, y.y), hi = __floats2bfloat162_rn(y.z, y.w);
                o[k * 2] = *reinterpret_cast<uint32_t*>(&lo);
                o[k * 2 + 1] = *reinterpret_cast<uint32_t*>(&hi);
              }
              *reinterpret_cast<uint4*>(cRow + c16 * 16 + h * 8) = make_uint4(o[0], o[1], o[2], o[3]);
            }
          }
          if (row == 0) a.tailCount[tailIdx * 2 + (int)ctaRank] = 0u;
        }
      }
    }
    if (a.tmaStore && lane == 0) umma::tmaStoreWaitAll();      // shared memory stays valid until the stores have read it
  } else if (warp >= 8 && MODE != MODE_PLAIN) {
    commWarps<MODE>(a, sFail, n, rank, 2 * stripesPerBlock);
  }

  umma::tcFenceBefore();
  __syncthreads();
  umma2::clusterSync();                            // neither CTA frees tensor memory the other still uses
  if (warp == 2) umma2::tmemDealloc(tmemBase, kTmemCols);
}

}  // namespace gemm
}  // namespace mccl
