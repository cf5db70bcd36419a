// Device-side building blocks of the collective kernels: 128-bit loads/stores at system scope, the typed
// fold (fp32 accumulation for 16-bit floats), release/acquire flag operations, bounded waits that give up
// into a status word instead of hanging, the cross-GPU barrier, and the NVLS multimem instructions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "devcomm.h"
#include "mccl.h"

namespace mccl {

// ---- memory operations ------------------------------------------------------------------------------
// Data that another GPU produced or will read is accessed at system scope; L1 is bypassed.
__device__ __forceinline__ uint4 ldSys128(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void stSys128(void* p, uint4 v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ldLocal128(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void stLocal128(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }

__device__ __forceinline__ uint64_t ldAcquireSys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void stReleaseSys(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" :: "l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t globalTimerNs() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ---- bounded wait -------------------------------------------------------------------------------------
// Spins until *flag >= want.  After `timeoutNs`, or as soon as the host raises status->abort, it records
// (code, peer, cta, step) in the status word and returns false; the caller then leaves the kernel.
__device__ __forceinline__ bool waitFlag(const uint64_t* flag, uint64_t want, const DevPeers& P, uint32_t code, int peer, int step) {
  if (ldAcquireSys(flag) >= want) return true;
  const uint64_t t0 = globalTimerNs();
  uint32_t spins = 0;
  for (;;) {
    if (ldAcquireSys(flag) >= want) return true;
    if ((++spins & 0x3ff) == 0) {
      if (P.status->abort != 0 || globalTimerNs() - t0 > P.timeoutNs) {
        if (atomicCAS((unsigned int*)&P.status->code, 0u, P.status->abort ? 3u : code) == 0u) {
          P.status->peer = (uint32_t)peer;
          P.status->cta = blockIdx.x;
          P.status->step = (uint32_t)step;
          __threadfence_system();
        }
        return false;
      }
    }
  }
}

__device__ __forceinline__ CtrlFlags* flagsOf(const DevPeers& P, int r) {
  return reinterpret_cast<CtrlFlags*>(P.ctrl[r] + P.layout.flagsOff);
}

// Barrier among the CTAs with this blockIdx.x on every rank.  `epoch` is the CTA's running barrier count
// (kept in a register, loaded from flags->epoch at entry and stored back at exit).  Everything the CTA
// wrote before the barrier is visible to every peer CTA that leaves it.  Returns false on timeout.
__device__ __forceinline__ bool ctaBarrier(const DevPeers& P, uint64_t& epoch, int* sFail) {
  const int cta = blockIdx.x, t = threadIdx.x;
  __syncthreads();
  ++epoch;
  if (t < P.n && t != P.rank) {
    __threadfence_system();
    stReleaseSys(&flagsOf(P, t)->bar[cta][P.rank], epoch);
    if (!waitFlag(&flagsOf(P, P.rank)->bar[cta][t], epoch, P, 1u, t, (int)(epoch & 0xffff))) *sFail = 1;
  }
  __syncthreads();
  return *sFail == 0;
}

// ---- typed fold -----------------------------------------------------------------------------------------
template <typename T> struct Acc { using type = T; };
template <> struct Acc<__half> { using type = float; };
template <> struct Acc<__nv_bfloat16> { using type = float; };
template <> struct Acc<int8_t> { using type = int32_t; };
template <> struct Acc<uint8_t> { using type = uint32_t; };

template <typename T> __device__ __forceinline__ typename Acc<T>::type widen(T v) { return (typename Acc<T>::type)v; }
template <> __device__ __forceinline__ float widen<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float widen<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T narrow(typename Acc<T>::type v) { return (T)v; }
template <> __device__ __forceinline__ __half narrow<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename A> __device__ __forceinline__ A foldOp(A a, A b, int op) {
  switch (op) {
    case mcclProd: return a * b;
    case mcclMax:  return a > b ? a : b;
    case mcclMin:  return a < b ? a : b;
    default:       return a + b;
  }
}

// avg: floats multiply by 1/n, integers divide (after wrapping to the element type, as the host path does).
template <typename T> __device__ __forceinline__ T finish(typename Acc<T>::type a, int divisor) {
  if (divisor > 1) return (T)(narrow<T>(a) / (T)divisor);
  return narrow<T>(a);
}
template <> __device__ __forceinline__ float finish<float>(float a, int divisor) { return divisor > 1 ? a * (1.0f / (float)divisor) : a; }
template <> __device__ __forceinline__ double finish<double>(double a, int divisor) { return divisor > 1 ? a * (1.0 / (double)divisor) : a; }
template <> __device__ __forceinline__ __half finish<__half>(float a, int divisor) { return __float2half_rn(divisor > 1 ? a * (1.0f / (float)divisor) : a); }
template <> __device__ __forceinline__ __nv_bfloat16 finish<__nv_bfloat16>(float a, int divisor) { return __float2bfloat16_rn(divisor > 1 ? a * (1.0f / (float)divisor) : a); }

template <typename T> struct Pack {
  static constexpr int N = 16 / sizeof(T);
  union { uint4 v; T e[16 / sizeof(T)]; };
};

// acc[] <- widen(first source)
template <typename T> __device__ __forceinline__ void accInit(typename Acc<T>::type* acc, uint4 v) {
  Pack<T> p; p.v = v;
#pragma unroll
  for (int i = 0; i < Pack<T>::N; ++i) acc[i] = widen<T>(p.e[i]);
}
template <typename T> __device__ __forceinline__ void accFold(typename Acc<T>::type* acc, uint4 v, int op) {
  Pack<T> p; p.v = v;
#pragma unroll
  for (int i = 0; i < Pack<T>::N; ++i) acc[i] = foldOp<typename Acc<T>::type>(acc[i], widen<T>(p.e[i]), op);
}
template <typename T> __device__ __forceinline__ uint4 accFinish(const typename Acc<T>::type* acc, int divisor) {
  Pack<T> p;
#pragma unroll
  for (int i = 0; i < Pack<T>::N; ++i) p.e[i] = finish<T>(acc[i], divisor);
  return p.v;
}

// ---- NVLS multimem (NVSwitch reduces / replicates) -------------------------------------------------------
__device__ __forceinline__ uint4 mmLdReduceAddF32(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ uint4 mmLdReduceAddBf16(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ uint4 mmLdReduceAddF16(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ uint4 mmLdReduceMinBf16(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.min.v4.bf16x2 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ uint4 mmLdReduceMaxBf16(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.max.v4.bf16x2 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ uint4 mmLdReduceMinF16(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.min.v4.f16x2 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ uint4 mmLdReduceMaxF16(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.max.v4.f16x2 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
// Replicated store: the bits land in every rank's copy.  Typed .f32 only because the instruction wants a
// type; no arithmetic happens.
__device__ __forceinline__ void mmStore128(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" :: "l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Copy vectors [lo, hi) (16-byte units) from src to dst, eight loads in flight per thread.
__device__ __forceinline__ void copyVecs(const char* src, char* dst, uint64_t lo, uint64_t hi, int tid, int nthreads) {
  constexpr int U = 8;
  uint64_t i = lo + tid;
  for (; i + (uint64_t)(U - 1) * nthreads < hi; i += (uint64_t)U * nthreads) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = ldSys128(src + (i + (uint64_t)u * nthreads) * 16);
#pragma unroll
    for (int u = 0; u < U; ++u) stLocal128(dst + (i + (uint64_t)u * nthreads) * 16, v[u]);
  }
  for (; i < hi; i += nthreads) stLocal128(dst + i * 16, ldSys128(src + i * 16));
}

// Work split of V units over G CTAs.  Up to 16384 units (256 KB of 16-byte vectors) per CTA it is one
// contiguous slice each; beyond that the CTAs take 256 KB tiles round-robin, so at any moment all CTAs of a
// GPU work inside one window of G x 256 KB.  (With one huge contiguous slice per CTA, a 32 GB all-reduce
// touched 32 windows 128 MB apart on every GPU at once and lost a fifth of its bandwidth.)  The split
// depends on (V, G) only, so CTA b covers the same units on every rank and in every phase.
__host__ __device__ __forceinline__ uint64_t tileUnits(uint64_t V, int G) {
  uint64_t per = (V + (uint64_t)G - 1) / (uint64_t)G;
  per = (per + 511) / 512 * 512;
  return per > 16384 ? 16384 : (per < 512 ? 512 : per);
}
template <typename F>
__device__ __forceinline__ void forTiles(uint64_t V, int G, int cta, F&& body) {
  const uint64_t tile = tileUnits(V, G);
  for (uint64_t lo = (uint64_t)cta * tile; lo < V; lo += (uint64_t)G * tile) body(lo, lo + tile < V ? lo + tile : V);
}

// Slice [lo, hi) of `total` units for part `i` of `parts`.
__device__ __forceinline__ uint64_t sliceLo(uint64_t total, int parts, int i) {
  return (uint64_t)(((unsigned __int128)total * (unsigned)i) / (unsigned)parts);
}

}  // namespace mccl
