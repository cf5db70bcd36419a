#include "host_reduce.h"

#include <cstring>

#include "../os/pool.h"

namespace mccl {

uint16_t floatToBf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);  // NaN stays NaN
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
float bf16ToFloat(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

namespace {

struct Bf16 { uint16_t bits; };

template <typename T> struct Wide { using type = T; };
template <> struct Wide<_Float16> { using type = float; };

template <typename T> inline T applyOp(T a, T b, mcclRedOp_t op) {
  switch (op) {
    case mcclProd: return (T)(a * b);
    case mcclMax:  return a > b ? a : b;
    case mcclMin:  return a < b ? a : b;
    default:       return (T)(a + b);
  }
}
template <> inline Bf16 applyOp<Bf16>(Bf16 a, Bf16 b, mcclRedOp_t op) {
  return Bf16{floatToBf16(applyOp<float>(bf16ToFloat(a.bits), bf16ToFloat(b.bits), op))};
}
template <> inline _Float16 applyOp<_Float16>(_Float16 a, _Float16 b, mcclRedOp_t op) {
  return (_Float16)applyOp<float>((float)a, (float)b, op);
}

// The op switch is hoisted out of the loop so each instantiation vectorises.
template <typename T, int OP>
void foldLoop(T* dst, const T* a, const T* b, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = applyOp<T>(a[i], b[i], (mcclRedOp_t)OP);
}

template <typename T>
void fold(T* dst, const T* a, const T* b, size_t n, mcclRedOp_t op) {
  switch (op) {
    case mcclProd: foldLoop<T, mcclProd>(dst, a, b, n); break;
    case mcclMax:  foldLoop<T, mcclMax>(dst, a, b, n); break;
    case mcclMin:  foldLoop<T, mcclMin>(dst, a, b, n); break;
    default:       foldLoop<T, mcclSum>(dst, a, b, n); break;
  }
}

constexpr size_t kParallelBytes = 4u << 20;

template <typename T>
mcclResult_t foldTyped(void* dst, const void* a, const void* b, size_t count, mcclRedOp_t op) {
  T* d = static_cast<T*>(dst);
  const T* x = static_cast<const T*>(a);
  const T* y = static_cast<const T*>(b);
  if (count * sizeof(T) < kParallelBytes) {
    fold<T>(d, x, y, count, op);
    return mcclSuccess;
  }
  const int parts = 8;
  return parallelFor(stripePool(), parts, [&](int i) -> mcclResult_t {
    const size_t lo = chunkOff(count, parts, i), hi = chunkOff(count, parts, i + 1);
    fold<T>(d + lo, x + lo, y + lo, hi - lo, op);
    return mcclSuccess;
  });
}

mcclResult_t dispatch(void* dst, const void* a, const void* b, size_t count, mcclDataType_t dt, mcclRedOp_t op) {
  if ((unsigned)op >= (unsigned)mcclNumOps) MCCLFAIL(mcclInvalidArgument);
  switch (dt) {
    case mcclInt8:     return foldTyped<int8_t>(dst, a, b, count, op);
    case mcclUint8:    return foldTyped<uint8_t>(dst, a, b, count, op);
    case mcclInt32:    return foldTyped<int32_t>(dst, a, b, count, op);
    case mcclUint32:   return foldTyped<uint32_t>(dst, a, b, count, op);
    case mcclInt64:    return foldTyped<int64_t>(dst, a, b, count, op);
    case mcclUint64:   return foldTyped<uint64_t>(dst, a, b, count, op);
    case mcclFloat16:  return foldTyped<_Float16>(dst, a, b, count, op);
    case mcclBfloat16: return foldTyped<Bf16>(dst, a, b, count, op);
    case mcclFloat32:  return foldTyped<float>(dst, a, b, count, op);
    case mcclFloat64:  return foldTyped<double>(dst, a, b, count, op);
    default: MCCLFAIL(mcclInvalidArgument);
  }
}

template <typename T> void scaleInt(T* p, size_t n, int div) { for (size_t i = 0; i < n; ++i) p[i] = (T)(p[i] / (T)div); }
template <typename T> void scaleFp(T* p, size_t n, T s) { for (size_t i = 0; i < n; ++i) p[i] = (T)(p[i] * s); }

mcclResult_t scaleRange(char* base, size_t lo, size_t hi, mcclDataType_t dt, int n) {
  const size_t cnt = hi - lo;
  switch (dt) {
    case mcclInt8:    scaleInt(reinterpret_cast<int8_t*>(base) + lo, cnt, n); break;
    case mcclUint8:   scaleInt(reinterpret_cast<uint8_t*>(base) + lo, cnt, n); break;
    case mcclInt32:   scaleInt(reinterpret_cast<int32_t*>(base) + lo, cnt, n); break;
    case mcclUint32:  scaleInt(reinterpret_cast<uint32_t*>(base) + lo, cnt, n); break;
    case mcclInt64:   scaleInt(reinterpret_cast<int64_t*>(base) + lo, cnt, n); break;
    case mcclUint64:  scaleInt(reinterpret_cast<uint64_t*>(base) + lo, cnt, n); break;
    case mcclFloat32: scaleFp(reinterpret_cast<float*>(base) + lo, cnt, 1.0f / (float)n); break;
    case mcclFloat64: scaleFp(reinterpret_cast<double*>(base) + lo, cnt, 1.0 / (double)n); break;
    case mcclFloat16: {
      _Float16* p = reinterpret_cast<_Float16*>(base) + lo;
      const float s = 1.0f / (float)n;
      for (size_t i = 0; i < cnt; ++i) p[i] = (_Float16)((float)p[i] * s);
      break;
    }
    case mcclBfloat16: {
      uint16_t* p = reinterpret_cast<uint16_t*>(base) + lo;
      const float s = 1.0f / (float)n;
      for (size_t i = 0; i < cnt; ++i) p[i] = floatToBf16(bf16ToFloat(p[i]) * s);
      break;
    }
    default: MCCLFAIL(mcclInvalidArgument);
  }
  return mcclSuccess;
}

}  // namespace

mcclResult_t hostReduce(void* dst, const void* src, size_t count, mcclDataType_t dt, mcclRedOp_t op) {
  return dispatch(dst, dst, src, count, dt, op);
}

mcclResult_t hostReduceOut(void* dst, const void* a, const void* b, size_t count, mcclDataType_t dt, mcclRedOp_t op) {
  return dispatch(dst, a, b, count, dt, op);
}

mcclResult_t hostReduceMulti(void* dst, const void* src, size_t count, int nSrc, size_t strideElems,
                             mcclDataType_t dt, mcclRedOp_t op) {
  const size_t es = mcclDataSize(dt);
  if (es == 0) MCCLFAIL(mcclInvalidArgument);
  for (int k = 0; k < nSrc; ++k)
    MCCLCHECK(hostReduce(dst, static_cast<const char*>(src) + (size_t)k * strideElems * es, count, dt, op));
  return mcclSuccess;
}

mcclResult_t hostScale(void* buf, size_t count, mcclDataType_t dt, int nRanks) {
  if (nRanks <= 1) return mcclSuccess;
  const size_t es = mcclDataSize(dt);
  if (es == 0) MCCLFAIL(mcclInvalidArgument);
  char* base = static_cast<char*>(buf);
  if (count * es < kParallelBytes) return scaleRange(base, 0, count, dt, nRanks);
  const int parts = 8;
  return parallelFor(stripePool(), parts, [&](int i) -> mcclResult_t {
    return scaleRange(base, chunkOff(count, parts, i), chunkOff(count, parts, i + 1), dt, nRanks);
  });
}

}  // namespace mccl
