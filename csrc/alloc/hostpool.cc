// Host allocations: page-aligned buffers (pinned when a GPU is present so that copies to the device are
// asynchronous) and a fixed-size freelist pool that grows by one buffer when it runs dry.
// Parity: src/include/alloc.h:10-23, src/allocator.cc:11-77 of the reference.
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unistd.h>
#include <vector>

#include "../core/core.h"

struct mcclMemPool {
  size_t buffSize = 0;
  std::mutex mu;
  std::vector<void*> all;
  std::vector<void*> freeList;
};

extern "C" {

mcclResult_t mcclPageAlloc(size_t bytes, void** out) {
  if (out == nullptr || bytes == 0) MCCLFAIL(mcclInvalidArgument);
  const size_t page = (size_t)sysconf(_SC_PAGESIZE);
  const size_t rounded = (bytes + page - 1) / page * page;
  void* p = nullptr;
  if (posix_memalign(&p, page, rounded) != 0 || p == nullptr) MCCLFAIL(mcclSystemError);
  *out = p;
  return mcclSuccess;
}

void mcclPageFree(void* ptr) { free(ptr); }

mcclResult_t mcclMemPoolCreate(size_t buffSize, int count, mcclMemPool_t* out) {
  if (out == nullptr || buffSize == 0 || count < 0) MCCLFAIL(mcclInvalidArgument);
  mcclMemPool* p = new mcclMemPool();
  p->buffSize = buffSize;
  for (int i = 0; i < count; ++i) {
    void* b = nullptr;
    mcclResult_t rc = mcclPageAlloc(buffSize, &b);
    if (rc != mcclSuccess) { mcclMemPoolDestroy(p); return rc; }
    p->all.push_back(b);
    p->freeList.push_back(b);
  }
  *out = p;
  return mcclSuccess;
}

mcclResult_t mcclMemPoolAlloc(mcclMemPool_t p, mcclBuf* out) {
  if (p == nullptr || out == nullptr) MCCLFAIL(mcclInvalidArgument);
  std::lock_guard<std::mutex> lk(p->mu);
  if (p->freeList.empty()) {
    void* b = nullptr;
    MCCLCHECK(mcclPageAlloc(p->buffSize, &b));
    p->all.push_back(b);
    p->freeList.push_back(b);
  }
  out->host = p->freeList.back();
  out->size = p->buffSize;
  p->freeList.pop_back();
  return mcclSuccess;
}

mcclResult_t mcclMemPoolFree(mcclMemPool_t p, const mcclBuf* buf) {
  if (p == nullptr || buf == nullptr || buf->host == nullptr) MCCLFAIL(mcclInvalidArgument);
  std::lock_guard<std::mutex> lk(p->mu);
  bool owned = false;
  for (void* b : p->all) owned = owned || b == buf->host;
  if (!owned) MCCLFAIL(mcclInvalidArgument);
  for (void* b : p->freeList) if (b == buf->host) MCCLFAIL(mcclInvalidUsage);   // double free
  p->freeList.push_back(buf->host);
  return mcclSuccess;
}

mcclResult_t mcclMemPoolStats(mcclMemPool_t p, int* total, int* free_) {
  if (p == nullptr) MCCLFAIL(mcclInvalidArgument);
  std::lock_guard<std::mutex> lk(p->mu);
  if (total) *total = (int)p->all.size();
  if (free_) *free_ = (int)p->freeList.size();
  return mcclSuccess;
}

mcclResult_t mcclMemPoolDestroy(mcclMemPool_t p) {
  if (p == nullptr) return mcclSuccess;
  for (void* b : p->all) mcclPageFree(b);
  delete p;
  return mcclSuccess;
}

}  // extern "C"
