#include "trace.h"

#include <chrono>
#include <cstdio>
#include <cuda_runtime.h>
#include <mutex>
#include <string>
#include <vector>

#include "../comm/comm.h"

namespace mccl {

namespace {
struct Record {
  std::string name;
  size_t bytes;
  int algo;
  double hostBeginUs, hostEndUs;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
};
struct Trace {
  std::mutex mu;
  std::vector<Record> recs;
  cudaEvent_t origin = nullptr;     // device time zero, recorded with the first traced call
  double originHostUs = 0;
};
std::mutex gMu;
std::vector<std::pair<mcclComm*, Trace*>> gTraces;
constexpr size_t kMaxRecords = 1u << 16;

double nowUs() {
  return std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
Trace* traceOf(mcclComm* c, bool create) {
  std::lock_guard<std::mutex> lk(gMu);
  for (auto& kv : gTraces) if (kv.first == c) return kv.second;
  if (!create) return nullptr;
  gTraces.emplace_back(c, new Trace());
  return gTraces.back().second;
}
}  // namespace

bool traceEnabled() {
  static const bool on = envStr("MCCL_TRACE") != nullptr;
  return on;
}

TraceSpan traceBegin(mcclComm* c, const char* name, size_t bytes, int algo, void* stream) {
  TraceSpan s;
  if (!traceEnabled()) return s;
  Trace* t = traceOf(c, true);
  std::lock_guard<std::mutex> lk(t->mu);
  if (t->recs.size() >= kMaxRecords) return s;
  Record r;
  r.name = name;
  r.bytes = bytes;
  r.algo = algo;
  r.hostBeginUs = r.hostEndUs = nowUs();
  if (c->cuda) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (t->origin == nullptr && cudaEventCreate(&t->origin) == cudaSuccess) {
      cudaEventRecord(t->origin, st);
      t->originHostUs = r.hostBeginUs;
    }
    if (cudaEventCreate(&r.e0) == cudaSuccess && cudaEventCreate(&r.e1) == cudaSuccess) cudaEventRecord(r.e0, st);
    cudaGetLastError();
  }
  t->recs.push_back(r);
  s.index = (int)t->recs.size() - 1;
  return s;
}

void traceEnd(mcclComm* c, TraceSpan span, void* stream) {
  if (span.index < 0) return;
  Trace* t = traceOf(c, false);
  if (t == nullptr) return;
  std::lock_guard<std::mutex> lk(t->mu);
  Record& r = t->recs[span.index];
  r.hostEndUs = nowUs();
  r.algo = c->lastAlgo.load();      // the planner's final choice is known once the call has been issued
  if (r.e1) cudaEventRecord(r.e1, static_cast<cudaStream_t>(stream));
  cudaGetLastError();
}

void traceFlush(mcclComm* c) {
  Trace* t = nullptr;
  {
    std::lock_guard<std::mutex> lk(gMu);
    for (size_t i = 0; i < gTraces.size(); ++i)
      if (gTraces[i].first == c) { t = gTraces[i].second; gTraces.erase(gTraces.begin() + i); break; }
  }
  if (t == nullptr) return;
  const char* prefix = envStr("MCCL_TRACE");
  char path[512];
  snprintf(path, sizeof(path), "%s.%d.json", prefix ? prefix : "mccl_trace", c->rank);
  FILE* f = fopen(path, "w");
  if (f != nullptr) {
    fprintf(f, "{\"traceEvents\":[\n");
    bool first = true;
    for (Record& r : t->recs) {
      // host track: the enqueue call; device track: the time between the two events on the stream
      fprintf(f, "%s{\"name\":\"%s\",\"cat\":\"enqueue\",\"ph\":\"X\",\"pid\":%d,\"tid\":0,\"ts\":%.3f,\"dur\":%.3f,"
                 "\"args\":{\"bytes\":%zu,\"algo\":\"%s\"}}", first ? "" : ",\n", r.name.c_str(), c->rank,
              r.hostBeginUs - t->recs[0].hostBeginUs, r.hostEndUs - r.hostBeginUs, r.bytes, mcclAlgoStr(r.algo));
      first = false;
      if (r.e0 && r.e1 && cudaEventSynchronize(r.e1) == cudaSuccess) {
        float startMs = 0.f, durMs = 0.f;
        if (cudaEventElapsedTime(&startMs, t->origin, r.e0) == cudaSuccess && cudaEventElapsedTime(&durMs, r.e0, r.e1) == cudaSuccess)
          fprintf(f, ",\n{\"name\":\"%s\",\"cat\":\"device\",\"ph\":\"X\",\"pid\":%d,\"tid\":1,\"ts\":%.3f,\"dur\":%.3f,"
                     "\"args\":{\"bytes\":%zu,\"algo\":\"%s\"}}", r.name.c_str(), c->rank, startMs * 1e3, durMs * 1e3, r.bytes,
                  mcclAlgoStr(r.algo));
      }
      if (r.e0) cudaEventDestroy(r.e0);
      if (r.e1) cudaEventDestroy(r.e1);
    }
    fprintf(f, "\n]}\n");
    fclose(f);
  }
  if (t->origin) cudaEventDestroy(t->origin);
  cudaGetLastError();
  delete t;
}

}  // namespace mccl
