// Base layer shared by every translation unit: result checks, leveled logging and cached env params.
// Parity: the reference's checks (src/include/checks.h:7-25), debug switch (src/misc/checks.cc:8-11) and
// param cache (src/include/param.h:17-30, src/misc/param.cc:9-22).
#pragma once

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <string>

#include "mccl.h"

namespace mccl {

enum LogLevel { LOG_NONE = 0, LOG_WARN = 1, LOG_INFO = 2, LOG_TRACE = 3 };

// Level from MCCL_DEBUG (WARN|INFO|TRACE, or any other non-empty value = WARN), read once.
int  logLevel();
void logSetRank(int rank);
void logMsg(int level, const char* file, int line, const char* fmt, ...) __attribute__((format(printf, 4, 5)));

#define MCCL_WARN(...)  do { if (::mccl::logLevel() >= ::mccl::LOG_WARN)  ::mccl::logMsg(::mccl::LOG_WARN,  __FILE__, __LINE__, __VA_ARGS__); } while (0)
#define MCCL_INFO(...)  do { if (::mccl::logLevel() >= ::mccl::LOG_INFO)  ::mccl::logMsg(::mccl::LOG_INFO,  __FILE__, __LINE__, __VA_ARGS__); } while (0)
#define MCCL_TRACE(...) do { if (::mccl::logLevel() >= ::mccl::LOG_TRACE) ::mccl::logMsg(::mccl::LOG_TRACE, __FILE__, __LINE__, __VA_ARGS__); } while (0)

// Records `r` as the calling thread's last error and logs the site; returns r.
mcclResult_t noteFailure(mcclResult_t r, const char* file, int line);

inline bool resultFatal(mcclResult_t r) {
  return r == mcclSystemError || r == mcclInternalError || r == mcclRemoteError;
}

// mcclInProgress is not a failure: a non-blocking call that has been queued reports it.
#define MCCLCHECK(call)                                                         \
  do {                                                                          \
    mcclResult_t rc_ = (call);                                                  \
    if (rc_ != mcclSuccess && rc_ != mcclInProgress)                            \
      return ::mccl::noteFailure(rc_, __FILE__, __LINE__);                      \
  } while (0)

#define MCCLCHECKGOTO(call, res, label)                                         \
  do {                                                                          \
    (res) = (call);                                                             \
    if ((res) != mcclSuccess && (res) != mcclInProgress) {                      \
      ::mccl::noteFailure((res), __FILE__, __LINE__);                           \
      goto label;                                                               \
    }                                                                           \
  } while (0)

#define MCCLFAIL(code) return ::mccl::noteFailure((code), __FILE__, __LINE__)

// Cached integer env params.  DEFINE_MCCL_PARAM(Name, "SUFFIX", default) defines
// int64_t mcclParam<Name>() that reads MCCL_<SUFFIX> once (strtoll base 0).  INT64_MIN marks "not read
// yet"; the cache is atomic because transport threads read it while another thread may do the first load.
int64_t loadParam(const char* env, int64_t deflt);

#define MCCL_PARAM(name) int64_t mcclParam##name()
#define DEFINE_MCCL_PARAM(name, env, deflt)                                     \
  int64_t mcclParam##name() {                                                   \
    static std::atomic<int64_t> cache{INT64_MIN};                               \
    int64_t v = cache.load(std::memory_order_acquire);                          \
    if (__builtin_expect(v == INT64_MIN, 0)) {                                  \
      v = ::mccl::loadParam("MCCL_" env, (deflt));                              \
      cache.store(v, std::memory_order_release);                                \
    }                                                                           \
    return v;                                                                   \
  }

// Uncached reads for strings/floats and for knobs that tests flip at run time.
const char* envStr(const char* name);
double      envDouble(const char* name, double deflt);
int64_t     envInt(const char* name, int64_t deflt);

// Host-side fault injection: MCCL_FAULT_INJECT="<site>:<nth>" makes the nth pass through the named site
// (counted per process) fail.  Sites are plain names used by the socket and bootstrap layers.
bool faultInject(const char* site);

// GPU facts used as the node score and as the "B200 required" gate of the cuda transport.
struct GpuInfo {
  int      device = -1;
  char     name[128] = {0};
  int      ccMajor = 0, ccMinor = 0;
  int      smCount = 0;
  uint64_t hbmBytes = 0;
  int      l2Bytes = 0;
  int      multicast = 0;   // CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED
  int      vmm = 0;         // virtual memory management + POSIX fd handles
  char     busId[32] = {0};
  char     uuid[16] = {0};
};
int          cudaDeviceCountSafe();          // 0 when no driver / no device
mcclResult_t discoverGpu(int device, GpuInfo* out);
bool         gpuSupported(const GpuInfo& g); // compute capability 10.x
std::string  gpuDescribe(const GpuInfo& g);

}  // namespace mccl
