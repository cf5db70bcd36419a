// Optional per-call tracing: with MCCL_TRACE=<path prefix> every collective / point-to-point batch is
// recorded (name, bytes, algorithm, host enqueue time, and on the cuda transport the device time between two
// CUDA events on the caller's stream) and written as Chrome-trace JSON to <prefix>.<rank>.json when the
// communicator is destroyed.  The reference has no tracing (no timers or trace files anywhere in it).
#pragma once

#include <cstddef>
#include <cstdint>

struct mcclComm;

namespace mccl {

struct TraceSpan {
  int index = -1;      // slot in the communicator's trace, -1 = tracing is off
};

bool      traceEnabled();
TraceSpan traceBegin(mcclComm* c, const char* name, size_t bytes, int algo, void* stream);
void      traceEnd(mcclComm* c, TraceSpan span, void* stream);
void      traceFlush(mcclComm* c);     // resolve event times and write the file (called by destroy)

}  // namespace mccl
