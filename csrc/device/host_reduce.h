// Host reductions for the CPU transport; also the oracle the GPU kernels are tested against.
// dst = op(dst, src) for all 10 dtypes and sum/prod/max/min (avg travels as sum and is finished by
// hostScale).  bf16 widens to fp32, applies the op and narrows with round-to-nearest-even (NaN kept
// quiet); fp16 uses the compiler's _Float16.
// Parity: src/device/reduce_kernel.h:18-173 of the reference (cpuReduceT, cpuReduceOutT, reduceMulti,
// chunkOffElems, scaleBuf/cpuScale).  Difference: integer avg divides (truncating, as NCCL does) instead
// of returning mcclInvalidUsage after the reduction already ran.
#pragma once

#include <cstddef>
#include <cstdint>

#include "../core/core.h"

namespace mccl {

mcclResult_t hostReduce(void* dst, const void* src, size_t count, mcclDataType_t dt, mcclRedOp_t op);
mcclResult_t hostReduceOut(void* dst, const void* a, const void* b, size_t count, mcclDataType_t dt, mcclRedOp_t op);
// dst = op(dst, src[0], src[1*stride], ...), folded in ascending source order.
mcclResult_t hostReduceMulti(void* dst, const void* src, size_t count, int nSrc, size_t strideElems,
                             mcclDataType_t dt, mcclRedOp_t op);
// Finish an average: floats *= 1/n, integers /= n.
mcclResult_t hostScale(void* buf, size_t count, mcclDataType_t dt, int nRanks);

// Element offset of chunk i when `count` elements are cut into n chunks (no padding, handles remainders).
inline size_t chunkOff(size_t count, int n, int i) { return (size_t)((__uint128_t)count * (unsigned)i / (unsigned)n); }

uint16_t floatToBf16(float f);
float    bf16ToFloat(uint16_t h);

}  // namespace mccl
