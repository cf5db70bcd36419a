// Expert-parallel token exchange fused with the gather / scatter by routing index.
//
// A mixture-of-experts layer sends token t of rank r to expert e = flat[t] / capacity, slot s = flat[t] %
// capacity.  Expert e lives on rank e / expertsPerRank, whose exchange buffer is laid out as
// [source rank][local expert][slot][row].  The usual form packs the tokens into a send buffer by index, runs an
// all-to-all of equal blocks and unpacks; here one kernel does the whole thing:
//
//   scatter (dispatch, and the backward pass of combine): every token row is read once from local memory,
//            optionally scaled, and stored straight into its slot of the destination rank's buffer over NVLink;
//   gather  (combine, and the backward pass of dispatch): every token reads its row back from the slot in the
//            expert's rank over NVLink, optionally scaled by its gate, into the local output; dropped tokens
//            (flat < 0) produce zero rows.
//
// Both are bracketed by the cross-GPU barrier of the collective kernels (same CTA count on every rank), so a
// buffer is complete when the kernel ends and nobody reads or writes it across kernels.  Slots that receive no
// token must read as zero (their rows meet zero gradients in the expert's weight gradient, and 0 x garbage may be
// NaN), so scatter is preceded by a clear of this rank's own buffer on the same stream.
// The reference's AllToAll (src/coll/coll.cc:90-106) is the unfused primitive; it has no routing.
#include <cuda_runtime.h>

#include "../comm/comm.h"
#include "../transport/cuda_mem.h"
#include "common.cuh"
#include "mccl_ops.h"

namespace mccl {
namespace {

constexpr int kMoeThreads = 512;
constexpr int kMoeWarps = kMoeThreads / 32;

struct MoeArgs {
  DevPeers peers;
  char* exch[MCCL_MAX_RANKS];     // every rank's exchange buffer as mapped here
  const char* tokens;             // scatter: local rows in; gather: unused
  char* out;                      // gather: local rows out
  const int32_t* flat;            // [nTokens] expert * capacity + slot, or < 0 for a dropped token
  const float* scale;             // [nTokens] or null
  int nTokens;
  int rowBytes;                   // multiple of 16
  int expertsPerRank;
  int capacity;
};

template <typename T>
__device__ __forceinline__ uint4 scaleVec(uint4 v, float s) {
  Pack<T> p; p.v = v;
#pragma unroll
  for (int i = 0; i < Pack<T>::N; ++i) p.e[i] = narrow<T>(widen<T>(p.e[i]) * s);
  return p.v;
}

// Row of (source rank, expert, slot) inside a rank's exchange buffer.
__device__ __forceinline__ uint64_t slotRow(int srcRank, int f, int expertsPerRank, int capacity, int* dstRank) {
  const int e = f / capacity, s = f - e * capacity;
  *dstRank = e / expertsPerRank;
  const int el = e - *dstRank * expertsPerRank;
  return ((uint64_t)srcRank * expertsPerRank + el) * capacity + s;
}

template <typename T, bool GATHER>
__global__ void __launch_bounds__(kMoeThreads, 1) moeKernel(const __grid_constant__ MoeArgs a) {
  __shared__ int sFail;
  const DevPeers& P = a.peers;
  const int cta = blockIdx.x, G = gridDim.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, me = P.rank;
  if (tid == 0) sFail = 0;
  CtrlFlags* mine = flagsOf(P, me);
  uint64_t epoch = mine->epoch[cta];
  bool ok = P.n == 1 || ctaBarrier(P, epoch, &sFail);     // buffers cleared / filled on every rank
  if (ok) {
    const int vecs = a.rowBytes / 16;
    const int nExperts = a.expertsPerRank * P.n;
    for (int t = cta * kMoeWarps + warp; t < a.nTokens; t += G * kMoeWarps) {
      const int f = a.flat[t];
      const bool kept = f >= 0 && f < nExperts * a.capacity;      // an index outside the grid is treated as dropped
      if (!kept) {
        if (GATHER) for (int v = lane; v < vecs; v += 32) stLocal128(a.out + (uint64_t)t * a.rowBytes + v * 16, make_uint4(0, 0, 0, 0));
        continue;
      }
      int peer;
      const uint64_t row = slotRow(me, f, a.expertsPerRank, a.capacity, &peer);
      char* remote = a.exch[peer] + row * (uint64_t)a.rowBytes;
      const float s = a.scale ? a.scale[t] : 1.0f;
      // Eight 16-byte pieces in flight per lane: with one, a row's trip over NVLink (a few microseconds for a
      // remote load) is paid 28 times in a row for a 14 KB row.
      constexpr int U = 8;
      const char* from = GATHER ? remote : a.tokens + (uint64_t)t * a.rowBytes;
      char* to = GATHER ? a.out + (uint64_t)t * a.rowBytes : remote;
      const bool farLoad = GATHER && peer != me, farStore = !GATHER && peer != me;
      for (int v0 = lane; v0 < vecs; v0 += 32 * U) {
        uint4 x[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int v = v0 + u * 32;
          if (v < vecs) x[u] = farLoad ? ldSys128(from + v * 16) : ldLocal128(from + v * 16);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int v = v0 + u * 32;
          if (v >= vecs) continue;
          if (a.scale) x[u] = scaleVec<T>(x[u], s);
          if (farStore) stSys128(to + v * 16, x[u]); else stLocal128(to + v * 16, x[u]);
        }
      }
    }
  }
  if (ok && P.n > 1) ok = ctaBarrier(P, epoch, &sFail);   // scatter: every row has landed; gather: nobody still reads
  if (tid == 0) mine->epoch[cta] = epoch;
}

template <bool GATHER>
mcclResult_t launchMoe(mcclComm* c, const MoeArgs& a, int dt, int ctas, cudaStream_t s) {
  switch (dt) {
    case mcclFloat32:  moeKernel<float, GATHER><<<ctas, kMoeThreads, 0, s>>>(a); break;
    case mcclBfloat16: moeKernel<__nv_bfloat16, GATHER><<<ctas, kMoeThreads, 0, s>>>(a); break;
    case mcclFloat16:  moeKernel<__half, GATHER><<<ctas, kMoeThreads, 0, s>>>(a); break;
    default: return mcclInvalidArgument;
  }
  if (cudaGetLastError() != cudaSuccess) return mcclSystemError;
  c->launches.fetch_add(1);
  return mcclSuccess;
}

mcclResult_t prepare(mcclComm_t comm, void* exchange, int rowBytes, int expertsPerRank, int capacity, MoeArgs* a, size_t* bytes) {
  if (comm == nullptr || !comm->cuda || comm->cu == nullptr || exchange == nullptr) return mcclInvalidArgument;
  if (rowBytes <= 0 || rowBytes % 16 || expertsPerRank <= 0 || capacity <= 0) return mcclInvalidArgument;
  if (comm->nRanks > MCCL_MAX_RANKS) return mcclInvalidArgument;
  *bytes = (size_t)comm->nRanks * expertsPerRank * capacity * rowBytes;
  Segment* seg = segmentFind(comm->cu, exchange, *bytes);
  if (seg == nullptr) {
    MCCL_WARN("the expert exchange buffer must live in symmetric memory (mcclMemAlloc) and hold ranks x experts x capacity rows");
    return mcclInvalidArgument;
  }
  memset(a, 0, sizeof(*a));
  a->peers = comm->cu->peers;
  const size_t off = (size_t)(static_cast<char*>(exchange) - seg->local);
  for (int p = 0; p < comm->nRanks; ++p) a->exch[p] = seg->peer[p] + off;
  a->rowBytes = rowBytes;
  a->expertsPerRank = expertsPerRank;
  a->capacity = capacity;
  return mcclSuccess;
}

// The same CTA count on every rank (the barrier pairs CTAs by index): it depends on the communicator's limit only.
int moeCtas(const mcclComm* c) {
  int g = 64;
  if (c->maxCtas > 0) g = std::min(g, c->maxCtas);
  return std::max(1, std::min(g, MCCL_MAX_CTAS));
}

}  // namespace
}  // namespace mccl

using namespace mccl;

extern "C" {

// Dispatch: rows of `tokens` ([nTokens, rowBytes], local memory) go to their slots of the destination ranks'
// `exchange` buffers (symmetric memory, [ranks][expertsPerRank][capacity][rowBytes] on every rank), each row
// multiplied by scale[t] when `scale` is given.  Collective over `comm`; every rank's buffer is cleared first.
mcclResult_t mcclMoeScatter(mcclComm_t comm, const void* tokens, const int32_t* flat, const float* scale, void* exchange,
                            int nTokens, int rowBytes, int expertsPerRank, int capacity, mcclDataType_t dt, mcclStream_t stream) {
  MoeArgs a;
  size_t bytes = 0;
  MCCLCHECK(prepare(comm, exchange, rowBytes, expertsPerRank, capacity, &a, &bytes));
  if (nTokens < 0 || (nTokens > 0 && (tokens == nullptr || flat == nullptr))) return mcclInvalidArgument;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  CUDACHECK(cudaSetDevice(comm->device));
  CUDACHECK(cudaMemsetAsync(exchange, 0, bytes, s));
  a.tokens = static_cast<const char*>(tokens);
  a.flat = flat;
  a.scale = scale;
  a.nTokens = nTokens;
  return launchMoe<false>(comm, a, dt, moeCtas(comm), s);
}

// Combine: out[t] = scale[t] x (the row in token t's slot of the expert's rank), zero for dropped tokens.
mcclResult_t mcclMoeGather(mcclComm_t comm, const void* exchange, const int32_t* flat, const float* scale, void* out,
                           int nTokens, int rowBytes, int expertsPerRank, int capacity, mcclDataType_t dt, mcclStream_t stream) {
  MoeArgs a;
  size_t bytes = 0;
  MCCLCHECK(prepare(comm, const_cast<void*>(exchange), rowBytes, expertsPerRank, capacity, &a, &bytes));
  if (nTokens < 0 || (nTokens > 0 && (out == nullptr || flat == nullptr))) return mcclInvalidArgument;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  CUDACHECK(cudaSetDevice(comm->device));
  a.out = static_cast<char*>(out);
  a.flat = flat;
  a.scale = scale;
  a.nTokens = nTokens;
  return launchMoe<true>(comm, a, dt, moeCtas(comm), s);
}

}  // extern "C"
