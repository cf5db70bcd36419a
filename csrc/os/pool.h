// Persistent worker pools for the CPU/TCP path and for parallel handle exchange at init.
// Two singletons at distinct nesting levels (outer fan-out, inner stripe) so a job that blocks on I/O in
// one pool can start jobs in the other without starving itself.
// Parity: src/pool.h:10-18, src/pool.cc:16-106 of the reference.
#pragma once

#include <functional>

#include "../core/core.h"

namespace mccl {

class ThreadPool;
ThreadPool* stripePool();   // leaf level: per-socket shards of one message
ThreadPool* fanoutPool();   // outer level: per-peer transfers, send||recv pairs
MCCL_PARAM(PoolThreads);

// Run fn(0..count-1); returns the first non-success result.  Work items are claimed from a shared
// counter and the caller claims too, so progress never depends on a free pool thread (safe for blocking
// I/O and for nested calls into the other pool).
mcclResult_t parallelFor(ThreadPool* pool, int count, const std::function<mcclResult_t(int)>& fn);

}  // namespace mccl
