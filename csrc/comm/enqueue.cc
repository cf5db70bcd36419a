// Launch policy and the per-communicator worker of the tcp transport.
// A non-blocking communicator owns one thread and a FIFO; a fatal result (system/internal/remote) latches
// and every later job is skipped, because a channel that failed mid-message is desynchronised.  Usage
// errors do not latch.  On the cuda transport the stream is the queue and no worker exists.
// Parity: src/enqueue.cc:11-106, src/include/comm.h:106-121 of the reference.
#include <condition_variable>
#include <deque>
#include <thread>

#include "comm.h"

namespace mccl {

struct WorkQueue {
  std::thread thread;
  std::mutex mu;
  std::condition_variable cv, idle;
  std::deque<std::function<mcclResult_t()>> jobs;
  bool stop = false;
  bool running = false;
  int firstError = (int)mcclSuccess;
};

static void workerLoop(mcclComm* comm) {
  WorkQueue* w = comm->work;
  std::unique_lock<std::mutex> lk(w->mu);
  for (;;) {
    w->cv.wait(lk, [&] { return w->stop || !w->jobs.empty(); });
    if (w->jobs.empty()) break;                       // stop requested and everything drained
    std::function<mcclResult_t()> job = std::move(w->jobs.front());
    w->jobs.pop_front();
    const bool skip = resultFatal((mcclResult_t)w->firstError) || comm->aborted.load();
    w->running = true;
    lk.unlock();
    mcclResult_t rc = skip ? mcclSuccess : job();
    lk.lock();
    w->running = false;
    if (resultFatal(rc) && !resultFatal((mcclResult_t)w->firstError)) {
      w->firstError = (int)rc;
      comm->asyncState.store((int)rc);
    }
    if (w->jobs.empty()) w->idle.notify_all();
  }
  w->idle.notify_all();
}

mcclResult_t workerStart(mcclComm* comm) {
  if (comm->work) return mcclSuccess;
  comm->work = new WorkQueue();
  comm->work->thread = std::thread(workerLoop, comm);
  return mcclSuccess;
}

void workerStop(mcclComm* comm) {
  WorkQueue* w = comm->work;
  if (w == nullptr) return;
  {
    std::lock_guard<std::mutex> lk(w->mu);
    w->stop = true;
  }
  w->cv.notify_all();
  if (w->thread.joinable()) w->thread.join();
  delete w;
  comm->work = nullptr;
}

mcclResult_t workerSync(mcclComm* comm) {
  WorkQueue* w = comm->work;
  std::unique_lock<std::mutex> lk(w->mu);
  w->idle.wait(lk, [&] { return w->jobs.empty() && !w->running; });
  const mcclResult_t e = (mcclResult_t)w->firstError;
  return resultFatal(e) ? e : mcclSuccess;
}

mcclResult_t workerAsyncError(mcclComm* comm, mcclResult_t* out) {
  WorkQueue* w = comm->work;
  std::lock_guard<std::mutex> lk(w->mu);
  if (resultFatal((mcclResult_t)w->firstError)) *out = (mcclResult_t)w->firstError;
  else if (!w->jobs.empty() || w->running) *out = mcclInProgress;
  else *out = mcclSuccess;
  return mcclSuccess;
}

mcclResult_t commLaunch(mcclComm* comm, std::function<mcclResult_t()> op) {
  if (comm == nullptr) MCCLFAIL(mcclInvalidArgument);
  if (comm->aborted.load()) MCCLFAIL(mcclInvalidUsage);
  if (comm->work == nullptr) {
    const mcclResult_t latched = (mcclResult_t)comm->asyncState.load();
    if (resultFatal(latched)) return latched;
    const mcclResult_t rc = op();
    if (resultFatal(rc)) comm->asyncState.store((int)rc);
    return rc;
  }
  WorkQueue* w = comm->work;
  {
    std::lock_guard<std::mutex> lk(w->mu);
    if (resultFatal((mcclResult_t)w->firstError)) return (mcclResult_t)w->firstError;
    if (w->stop) MCCLFAIL(mcclInvalidUsage);
    w->jobs.push_back(std::move(op));
  }
  w->cv.notify_one();
  return mcclSuccess;
}

}  // namespace mccl
