// Persistent, warp-specialised bf16 GEMM for sm_100a with the tensor-parallel collectives fused in.
//
//   C[M,N] = A[M,K] * B[N,K]^T      A, B row-major (K contiguous), fp32 accumulation in tensor memory
//
// One CTA per SM walks output tiles of 128 x BN.  Warp roles:
//   warp 0      TMA producer: 128x64 A tiles and BNx64 B tiles into a 4-stage shared-memory ring
//               (cp.async.bulk.tensor, 128-byte swizzle, no cluster multicast)
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16) four times per stage into one
//               of two TMEM accumulators and commits to mbarriers
//   warp 2      allocates and frees the 512 TMEM columns
//   warps 4-7   epilogue: tcgen05.ld the finished accumulator (each warp its 32 lanes), activation, bf16
//               pack, 16-byte stores; overlaps the next tile's MMAs thanks to the second accumulator
//   warps 8-11  communication, in the fused modes:
//     MODE_AG   all-gather -> GEMM: copy the peers' activation shards into this GPU's full activation
//               buffer over NVLink (plain peer loads) and publish a counter per shard; the producer waits for
//               the shard a tile's rows belong to, so tiles of the own shard start at once and the rest
//               follow in arrival order.  TMA only ever reads local memory.
//     MODE_RS   GEMM -> reduce-scatter: the epilogue writes bf16 partial tiles to a peer-visible staging
//               buffer, row blocks of other ranks first, and pushes a flag to the owner when a 128-row
//               stripe is complete; the owner's communication warps pull the eight partial stripes, add
//               them in fp32 in rank order and write the reduced rows.
// Every wait (mbarrier, flag) is bounded: on expiry the role records an error code and all roles unwind,
// tensor memory is freed and the kernel returns.
// Neither the GEMM nor the fused forms exist in the reference (it has no tensor-parallel code).
#pragma once

#include <cuda_bf16.h>

#include "../common.cuh"
#include "umma.cuh"

namespace mccl {
namespace gemm {

constexpr int BM = 128, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int kThreadsGemm = 384;
constexpr int kCommThreads = 128;
constexpr int kTmemCols = 512;
enum Mode { MODE_PLAIN = 0, MODE_AG = 1, MODE_RS = 2 };
enum Epilogue { EPI_NONE = 0, EPI_SILU = 1 };

struct GemmArgs {
  CUtensorMap mapA;            // A: [M, K] bf16, box 64 x 128
  CUtensorMap mapB;            // B: [N, K] bf16, box 64 x BN
  int M, N, K;
  __nv_bfloat16* C;            // [M, N] output (plain / AG) or partial staging (RS)
  int epilogue;
  int* errFlag;                // device-visible int, 0 = fine
  uint64_t budgetNs;
  // fused modes
  DevPeers peers;
  uint64_t callIndex;          // 1, 2, 3 ... per flags buffer
  uint64_t* shardReady;        // AG: local counters [n]
  const char* xPeer[MCCL_MAX_RANKS];   // AG: every rank's activation shard [M/n, K]
  char* xFull;                 // AG: local [M, K]
  const char* partialPeer[MCCL_MAX_RANKS];   // RS: every rank's staging [M, N]
  uint64_t* tileReadyPeer[MCCL_MAX_RANKS];   // RS: every rank's flags [n][stripes per block]
  uint64_t* stripeCount;       // RS: local counters [M/128]: tiles of the stripe stored so far
  __nv_bfloat16* out;          // RS: [M/n, N]
  float* accum;                // RS: [M/n, N] fp32 running sum of the partials that have arrived
  int panel;                   // stripes per rasterisation panel (divides the stripes of a row block)
  // Two-SM kernel, split tail: when the tiles do not fill the last wave, the last `tailTiles` tiles are cut along K
  // into `tailSlices` slices each, one slice per SM pair, so the last wave costs 1 / tailSlices of a tile instead of
  // a whole one.  The slices add their fp32 partial tiles into `tailWs` (zero between launches: the CTA that adds
  // last converts the sum to C and clears what it read); `tailCount` counts arrivals per (tile, half).
  int tailTiles, tailSlices;
  float* tailWs;
  unsigned int* tailCount;
  CUtensorMap mapC;            // two-SM kernel: C as [M, N] bf16, box 64 x 32, for the epilogue's TMA stores
  int tmaStore;                // 1: mapC is valid
  int debug;                   // tuning aid of the two-SM kernel (MCCL_GEMM_DEBUG): bit 0 = skip the loads after the
                               // first ring fill, bit 1 = skip the epilogue's global stores (results are then meaningless), bit 2 = per-thread
                               // 16-byte stores instead of the TMA store
};

template <int BN> struct Smem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int TILE_BYTES = STAGES * (A_BYTES + B_BYTES);
  static constexpr int TOTAL = TILE_BYTES + 256 + 1024;     // barriers + alignment slack
};

__device__ __forceinline__ float silu(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

__device__ __forceinline__ uint64_t ldAcquireGpu(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ bool waitGpuFlag(const uint64_t* flag, uint64_t want, uint64_t budgetNs) {
  if (ldAcquireGpu(flag) >= want) return true;
  const uint64_t t0 = globalTimerNs();
  for (uint32_t spins = 1;; ++spins) {
    if (ldAcquireGpu(flag) >= want) return true;
    if ((spins & 0xff) == 0 && globalTimerNs() - t0 > budgetNs) return false;
  }
}

// Named barrier over `count` threads that also ORs a predicate: every participant gets the same answer, so
// all of them leave a loop together (a plain flag read could differ between warps and strand one of them at
// the next barrier).
__device__ __forceinline__ bool namedBarrierOr(int id, int count, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n .reg .pred p, q;\n setp.ne.b32 p, %1, 0;\n barrier.cta.red.or.pred q, %2, %3, p;\n selp.b32 %0, 1, 0, q;\n}"
      : "=r"(r) : "r"((uint32_t)pred), "r"(id), "r"(count) : "memory");
  return r != 0;
}

// Barrier among the communication warps (128 threads, named barrier 2) of the CTAs with this blockIdx.x
// on every rank; same flag protocol as ctaBarrier.
__device__ __forceinline__ bool commBarrier(const DevPeers& P, uint64_t& epoch, volatile int* sFail, int ct) {
  const int cta = blockIdx.x;
  asm volatile("bar.sync 2, 128;" ::: "memory");
  ++epoch;
  if (ct < P.n && ct != P.rank) {
    __threadfence_system();
    stReleaseSys(&flagsOf(P, ct)->bar[cta][P.rank], epoch);
    if (!waitFlag(&flagsOf(P, P.rank)->bar[cta][ct], epoch, P, 1u, ct, (int)(epoch & 0xffff))) *sFail = 1;
  }
  return !namedBarrierOr(2, kCommThreads, *sFail != 0);
}

// Tile t -> (row stripe, column tile).  Tiles are walked panel by panel: a panel is `panel` consecutive
// stripes, and inside it the stripe index runs fastest, so the CTAs that run together share a few B tiles and
// `panel` A stripes (both stay in L2) instead of one A stripe and every B tile.  The order of the row blocks:
// AG starts with the own shard and continues in the order the shards arrive; RS starts with the block of
// rank+1 and ends with the own block, so partial results for the peers leave early.
template <int MODE>
__host__ __device__ __forceinline__ void tileCoords(int t, int tilesN, int panel, int stripesPerBlock, int rank, int n, int* stripe, int* nt) {
  const int perPanel = panel * tilesN;
  const int p = t / perPanel, within = t - p * perPanel;
  const int ord = p * panel + within % panel;
  *nt = within / panel;
  if (MODE == MODE_PLAIN) { *stripe = ord; return; }
  const int blockOrd = ord / stripesPerBlock, inBlock = ord - blockOrd * stripesPerBlock;
  const int block = (MODE == MODE_AG) ? (rank + blockOrd) % n : (rank + 1 + blockOrd) % n;
  *stripe = block * stripesPerBlock + inBlock;
}

// The communication warps (threads 256..383, named barrier 2) of the fused modes; `stripesPerBlock` counts
// 128-row stripes of one rank's row block.
template <int MODE>
__device__ __forceinline__ void commWarps(const GemmArgs& a, volatile int* sFail, int n, int rank, int stripesPerBlock) {
  const int ct = threadIdx.x - 256;
  const DevPeers& P = a.peers;
  CtrlFlags* mine = flagsOf(P, P.rank);
  uint64_t epoch = mine->epoch[blockIdx.x];
  bool ok = commBarrier(P, epoch, sFail, ct);              // peers' inputs exist, their buffers are free
  const int G = gridDim.x, cta = blockIdx.x;
  if (MODE == MODE_AG && ok) {
    const uint64_t shardBytes = (uint64_t)(a.M / n) * a.K * 2, V = shardBytes / 16;
    const uint64_t lo = sliceLo(V, G, cta), hi = sliceLo(V, G, cta + 1);
    for (int i = 0; i < n; ++i) {
      const int s = (rank + i) % n;
      const char* src = a.xPeer[s];
      char* dst = a.xFull + (uint64_t)s * shardBytes;
      if (src != dst) copyVecs(src, dst, lo, hi, ct, kCommThreads);
      if (namedBarrierOr(2, kCommThreads, *sFail != 0)) break;
      if (ct == 0) { __threadfence(); atomicAdd(reinterpret_cast<unsigned long long*>(&a.shardReady[s]), 1ull); }
    }
  }
  if (MODE == MODE_RS && ok) {
    // Partials for this rank's row block arrive in a fixed order: rank-1 computes the block first, then
    // rank-2, ..., and the own GEMM last.  Each arrival is folded into an fp32 running sum as soon as its
    // stripe flag is up, so the NVLink reads spread over the whole GEMM and only the last fold (own
    // partial, local) remains at the end.  The fold order is the same on every run.
    const uint64_t stripeBytes = (uint64_t)BM * a.N * 2, V = stripeBytes / 16;
    const uint64_t* ready = a.tileReadyPeer[rank];
    bool failed = false;
    for (int ord = 0; ord < n && !failed; ++ord) {
      const int src = (ord == n - 1) ? rank : (rank - 1 - ord + 2 * n) % n;
      for (int lt = 0; lt < stripesPerBlock; ++lt) {
        if (ct == 0 && !waitFlag(&ready[(size_t)src * stripesPerBlock + lt], a.callIndex, P, 2u, src, lt)) *sFail = 1;
        if (namedBarrierOr(2, kCommThreads, *sFail != 0)) { failed = true; break; }
        const char* part = a.partialPeer[src] + ((uint64_t)rank * stripesPerBlock + lt) * stripeBytes;
        float4* acc4 = reinterpret_cast<float4*>(a.accum) + (uint64_t)lt * V * 2;
        char* dst = reinterpret_cast<char*>(a.out) + (uint64_t)lt * stripeBytes;
        // Eight remote vectors in flight per thread: with one, the 148 x 128 communication threads keep
        // only 0.3 MB on the wire and the pull runs at a tenth of the link rate.
        constexpr int U = 8;
        forTiles(V, G, cta, [&](uint64_t lo, uint64_t hi) {
          for (uint64_t i = lo + ct; i < hi; i += (uint64_t)U * kCommThreads) {
            uint4 pv[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const uint64_t idx = i + (uint64_t)u * kCommThreads;
              if (idx < hi) pv[u] = ldSys128(part + idx * 16);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const uint64_t idx = i + (uint64_t)u * kCommThreads;
              if (idx >= hi) continue;
              float acc[8];
              accInit<__nv_bfloat16>(acc, pv[u]);
              if (ord > 0) {
                const float4 x = acc4[2 * idx], y = acc4[2 * idx + 1];
                acc[0] += x.x; acc[1] += x.y; acc[2] += x.z; acc[3] += x.w;
                acc[4] += y.x; acc[5] += y.y; acc[6] += y.z; acc[7] += y.w;
              }
              if (ord == n - 1) {
                stLocal128(dst + idx * 16, accFinish<__nv_bfloat16>(acc, 1));
              } else {
                acc4[2 * idx] = make_float4(acc[0], acc[1], acc[2], acc[3]);
                acc4[2 * idx + 1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
              }
            }
          }
        });
      }
    }
  }
  if (!namedBarrierOr(2, kCommThreads, !ok || *sFail != 0)) commBarrier(P, epoch, sFail, ct);   // nobody still reads this rank's buffers
  if (ct == 0) mine->epoch[blockIdx.x] = epoch;
  if (*sFail && ct == 0) atomicCAS(a.errFlag, 0, 15);
}

template <int BN, int MODE>
__global__ void __launch_bounds__(kThreadsGemm, 1) tpGemmKernel(const __grid_constant__ GemmArgs a) {
  using S = Smem<BN>;
  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * S::A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::TILE_BYTES);
  uint64_t* full = bars;                 // [STAGES] TMA -> MMA
  uint64_t* empty = bars + STAGES;       // [STAGES] MMA -> TMA
  uint64_t* tmemFull = bars + 2 * STAGES;     // [2] MMA -> epilogue
  uint64_t* tmemEmpty = bars + 2 * STAGES + 2; // [2] epilogue -> MMA
  uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* sFail = reinterpret_cast<volatile int*>(tmemSlot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tilesN = a.N / BN, stripes = a.M / BM, kBlocks = a.K / BK;
  const int totalTiles = tilesN * stripes;
  const int n = (MODE == MODE_PLAIN) ? 1 : a.peers.n, rank = (MODE == MODE_PLAIN) ? 0 : a.peers.rank;
  const int stripesPerBlock = stripes / n;
  const uint64_t budget = a.budgetNs;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { umma::mbarInit(&full[s], 1); umma::mbarInit(&empty[s], 1); }
    for (int i = 0; i < 2; ++i) { umma::mbarInit(&tmemFull[i], 1); umma::mbarInit(&tmemEmpty[i], 4); }
    *sFail = 0;
    umma::fenceBarrierInit();
    umma::prefetchTensorMap(&a.mapA);
    umma::prefetchTensorMap(&a.mapB);
  }
  if (warp == 2) { umma::tmemAlloc(tmemSlot, kTmemCols); umma::tmemRelinquish(); }
  umma::tcFenceBefore();
  __syncthreads();
  umma::tcFenceAfter();
  const uint32_t tmemBase = *tmemSlot;

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer
    int stage = 0; uint32_t phase = 0;
    for (int t = blockIdx.x; t < totalTiles && *sFail == 0; t += gridDim.x) {
      int stripe, nt;
      tileCoords<MODE>(t, tilesN, a.panel, stripesPerBlock, rank, n, &stripe, &nt);
      if (MODE == MODE_AG) {
        const int shard = stripe / stripesPerBlock;
        if (!waitGpuFlag(&a.shardReady[shard], (uint64_t)gridDim.x, budget)) { *sFail = 1; atomicExch(a.errFlag, 10); break; }
        umma::fenceProxyAsyncGlobal();
      }
      for (int kb = 0; kb < kBlocks; ++kb) {
        if (!umma::mbarWait(&empty[stage], phase ^ 1, budget)) { *sFail = 1; atomicExch(a.errFlag, 11); break; }
        umma::mbarExpectTx(&full[stage], S::A_BYTES + S::B_BYTES);
        umma::tmaLoad2d(sA + stage * S::A_BYTES, &a.mapA, &full[stage], kb * BK, stripe * BM);
        umma::tmaLoad2d(sB + stage * S::B_BYTES, &a.mapB, &full[stage], kb * BK, nt * BN);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer
    constexpr uint32_t idesc = umma::instrDescBf16(BM, BN);
    int stage = 0; uint32_t phase = 0; int acc = 0; uint32_t accPhase = 0;
    for (int t = blockIdx.x; t < totalTiles && *sFail == 0; t += gridDim.x) {
      if (!umma::mbarWait(&tmemEmpty[acc], accPhase ^ 1, budget)) { *sFail = 1; atomicExch(a.errFlag, 12); break; }
      umma::tcFenceAfter();
      const uint32_t d = tmemBase + (uint32_t)acc * 256u;
      for (int kb = 0; kb < kBlocks; ++kb) {
        if (!umma::mbarWait(&full[stage], phase, budget)) { *sFail = 1; atomicExch(a.errFlag, 13); break; }
        umma::tcFenceAfter();
        const uint64_t da = umma::smemDescSw128(sA + stage * S::A_BYTES), db = umma::smemDescSw128(sB + stage * S::B_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          umma::mmaBf16(d, da + (uint64_t)(k * UMMA_K * 2 / 16), db + (uint64_t)(k * UMMA_K * 2 / 16), idesc, (kb | k) != 0);
        umma::mmaCommit(&empty[stage]);          // the stage is free once these MMAs have read it
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      if (*sFail) break;
      umma::mmaCommit(&tmemFull[acc]);           // accumulator complete
      acc ^= 1; if (acc == 0) accPhase ^= 1;
    }
  } else if (warp >= 4 && warp < 8) {
    // ---------------- epilogue
    const int q = warp - 4;                      // == warp % 4: the TMEM lane quarter this warp may read
    int acc = 0; uint32_t accPhase = 0;
    for (int t = blockIdx.x; t < totalTiles; t += gridDim.x) {
      int stripe, nt;
      tileCoords<MODE>(t, tilesN, a.panel, stripesPerBlock, rank, n, &stripe, &nt);
      bool good = *sFail == 0 && umma::mbarWait(&tmemFull[acc], accPhase, budget);
      if (!good && *sFail == 0) { *sFail = 1; atomicExch(a.errFlag, 14); }
      // In RS mode the four warps meet at a named barrier below, so they must agree on leaving.
      if (MODE == MODE_RS) good = !namedBarrierOr(1, 128, !good);
      if (!good) break;
      umma::tcFenceAfter();
      const size_t row = (size_t)stripe * BM + q * 32 + lane;
      __nv_bfloat16* dstRow = a.C + row * (size_t)a.N + (size_t)nt * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
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
#pragma unroll
        for (int j = 0; j < 4; ++j) dst[j] = outv[j];
      }
      umma::tcFenceBefore();
      __syncwarp();
      if (lane == 0) umma::mbarArrive(&tmemEmpty[acc]);
      acc ^= 1; if (acc == 0) accPhase ^= 1;
      if (MODE == MODE_RS) {
        // All four warps have stored their rows of this tile; count it towards the stripe and tell the
        // owner of the row block when the stripe is whole.
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 4 && lane == 0) {
          __threadfence_system();
          const unsigned long long doneNow = atomicAdd(reinterpret_cast<unsigned long long*>(&a.stripeCount[stripe]), 1ull) + 1ull;
          if (doneNow == (uint64_t)tilesN) {
            const int owner = stripe / stripesPerBlock, within = stripe - owner * stripesPerBlock;
            __threadfence_system();
            stReleaseSys(&a.tileReadyPeer[owner][(size_t)rank * stripesPerBlock + within], a.callIndex);
          }
        }
      }
    }
  } else if (warp >= 8 && MODE != MODE_PLAIN) {
    commWarps<MODE>(a, sFail, n, rank, stripesPerBlock);
  }

  umma::tcFenceBefore();
  __syncthreads();
  if (warp == 2) umma::tmemDealloc(tmemBase, kTmemCols);
}

}  // namespace gemm
}  // namespace mccl
