#include "pool.h"

#include <atomic>
#include <condition_variable>
#include <deque>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

namespace mccl {

DEFINE_MCCL_PARAM(PoolThreads, "POOL_THREADS", 0);

class ThreadPool {
 public:
  explicit ThreadPool(int n) {
    for (int i = 0; i < n; ++i) workers_.emplace_back([this] { loop(); });
  }
  ~ThreadPool() {
    {
      std::lock_guard<std::mutex> lk(mu_);
      stop_ = true;
    }
    cv_.notify_all();
    for (auto& t : workers_) t.join();
  }
  void post(std::function<void()> job) {
    {
      std::lock_guard<std::mutex> lk(mu_);
      jobs_.push_back(std::move(job));
    }
    cv_.notify_one();
  }
  int size() const { return (int)workers_.size(); }

 private:
  void loop() {
    for (;;) {
      std::function<void()> job;
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [this] { return stop_ || !jobs_.empty(); });
        if (jobs_.empty()) return;
        job = std::move(jobs_.front());
        jobs_.pop_front();
      }
      job();
    }
  }
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<std::function<void()>> jobs_;
  std::vector<std::thread> workers_;
  bool stop_ = false;
};

static int poolThreads() {
  int64_t n = mcclParamPoolThreads();
  if (n <= 0) {
    n = (int64_t)std::thread::hardware_concurrency();
    if (n < 16) n = 16;
    if (n > 64) n = 64;
  }
  return (int)n;
}

// Leaked on purpose: worker threads may still be parked in I/O when static destructors run.
ThreadPool* stripePool() { static ThreadPool* p = new ThreadPool(poolThreads()); return p; }
ThreadPool* fanoutPool() { static ThreadPool* p = new ThreadPool(poolThreads()); return p; }

namespace {
struct Share {
  std::atomic<int> next{0};
  std::atomic<int> done{0};
  std::atomic<int> firstErr{(int)mcclSuccess};
  int count = 0;
  std::function<mcclResult_t(int)> fn;
  std::mutex mu;
  std::condition_variable cv;
  void drain() {
    for (;;) {
      int i = next.fetch_add(1);
      if (i >= count) return;
      mcclResult_t rc = fn(i);
      if (rc != mcclSuccess) {
        int expect = (int)mcclSuccess;
        firstErr.compare_exchange_strong(expect, (int)rc);
      }
      if (done.fetch_add(1) + 1 == count) {
        std::lock_guard<std::mutex> lk(mu);
        cv.notify_all();
      }
    }
  }
};
}  // namespace

mcclResult_t parallelFor(ThreadPool* pool, int count, const std::function<mcclResult_t(int)>& fn) {
  if (count <= 0) return mcclSuccess;
  if (count == 1) return fn(0);
  auto sh = std::make_shared<Share>();
  sh->count = count;
  sh->fn = fn;
  int helpers = count - 1;
  int pooled = helpers < pool->size() ? helpers : pool->size();
  for (int i = 0; i < pooled; ++i) pool->post([sh] { sh->drain(); });
  // Items may block on one another (a send completes only once the peer's matching recv runs), so every
  // item needs its own thread: whatever the pool cannot cover gets a temporary one.
  std::vector<std::thread> extra;
  for (int i = pooled; i < helpers; ++i) extra.emplace_back([sh] { sh->drain(); });
  sh->drain();
  {
    std::unique_lock<std::mutex> lk(sh->mu);
    sh->cv.wait(lk, [&] { return sh->done.load() >= count; });
  }
  for (auto& t : extra) t.join();
  return (mcclResult_t)sh->firstErr.load();
}

}  // namespace mccl
