// A pool on top of the symmetric allocator: ONE collective allocation (mcclMemAlloc: handle exchange, peer
// mappings, multicast binding, barriers), then sub-allocations that are local bookkeeping.  First fit over a free
// list kept sorted by offset, neighbours merged on free: the result depends only on the sequence of calls, so ranks
// that make the same calls get the same offsets, which is what makes a sub-allocation "the same part of the same
// allocation on every rank" for the kernels.
// Role parity: mcclMemPool of the reference (src/allocator.cc:38-77), a freelist over page-aligned host buffers;
// here the buffers are ranges of one registered device segment (or of one page-aligned host block on the tcp transport).
#include <algorithm>
#include <mutex>
#include <vector>

#include "../comm/comm.h"

struct mcclSymPool {
  mcclComm* comm = nullptr;
  char* base = nullptr;
  size_t bytes = 0;
  std::mutex mu;
  struct Range { size_t off, len; };
  std::vector<Range> freeList;     // sorted by offset, no two adjacent
  std::vector<Range> live;         // handed out, unsorted
};

namespace {
constexpr size_t kAlign = 256;
size_t roundUp(size_t v) { return (v + kAlign - 1) / kAlign * kAlign; }
}  // namespace

using namespace mccl;

extern "C" {

mcclResult_t mcclSymPoolCreate(mcclComm_t comm, size_t bytes, mcclSymPool_t* pool) {
  if (comm == nullptr || pool == nullptr || bytes == 0) MCCLFAIL(mcclInvalidArgument);
  void* p = nullptr;
  const size_t total = roundUp(bytes);
  MCCLCHECK(mcclMemAlloc(comm, total, &p));
  mcclSymPool* s = new mcclSymPool();
  s->comm = comm;
  s->base = static_cast<char*>(p);
  s->bytes = total;
  s->freeList.push_back({0, total});
  *pool = s;
  return mcclSuccess;
}

mcclResult_t mcclSymPoolAlloc(mcclSymPool_t pool, size_t bytes, void** ptr) {
  if (pool == nullptr || ptr == nullptr || bytes == 0) MCCLFAIL(mcclInvalidArgument);
  const size_t need = roundUp(bytes);
  std::lock_guard<std::mutex> lk(pool->mu);
  for (size_t i = 0; i < pool->freeList.size(); ++i) {
    mcclSymPool::Range& f = pool->freeList[i];
    if (f.len < need) continue;
    const size_t off = f.off;
    if (f.len == need) pool->freeList.erase(pool->freeList.begin() + i);
    else { f.off += need; f.len -= need; }
    pool->live.push_back({off, need});
    *ptr = pool->base + off;
    return mcclSuccess;
  }
  *ptr = nullptr;
  MCCL_WARN("symmetric pool of %zu bytes has no free range of %zu bytes", pool->bytes, need);
  return mcclSystemError;
}

mcclResult_t mcclSymPoolFree(mcclSymPool_t pool, void* ptr) {
  if (pool == nullptr) MCCLFAIL(mcclInvalidArgument);
  if (ptr == nullptr) return mcclSuccess;
  std::lock_guard<std::mutex> lk(pool->mu);
  const size_t off = (size_t)(static_cast<char*>(ptr) - pool->base);
  for (size_t i = 0; i < pool->live.size(); ++i) {
    if (pool->live[i].off != off) continue;
    mcclSymPool::Range r = pool->live[i];
    pool->live.erase(pool->live.begin() + i);
    auto it = std::lower_bound(pool->freeList.begin(), pool->freeList.end(), r,
                               [](const mcclSymPool::Range& a, const mcclSymPool::Range& b) { return a.off < b.off; });
    it = pool->freeList.insert(it, r);
    if (it + 1 != pool->freeList.end() && it->off + it->len == (it + 1)->off) { it->len += (it + 1)->len; pool->freeList.erase(it + 1); }
    if (it != pool->freeList.begin() && (it - 1)->off + (it - 1)->len == it->off) { (it - 1)->len += it->len; pool->freeList.erase(it); }
    return mcclSuccess;
  }
  MCCLFAIL(mcclInvalidArgument);     // not a live sub-allocation of this pool
}

mcclResult_t mcclSymPoolStats(mcclSymPool_t pool, size_t* total, size_t* inUse, size_t* largestFree) {
  if (pool == nullptr) MCCLFAIL(mcclInvalidArgument);
  std::lock_guard<std::mutex> lk(pool->mu);
  size_t used = 0, largest = 0;
  for (const auto& r : pool->live) used += r.len;
  for (const auto& r : pool->freeList) largest = std::max(largest, r.len);
  if (total) *total = pool->bytes;
  if (inUse) *inUse = used;
  if (largestFree) *largestFree = largest;
  return mcclSuccess;
}

mcclResult_t mcclSymPoolDestroy(mcclSymPool_t pool) {
  if (pool == nullptr) return mcclSuccess;
  mcclResult_t rc = mcclMemFree(pool->comm, pool->base);     // collective
  delete pool;
  return rc;
}

}  // extern "C"
