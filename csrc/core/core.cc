// Type helpers, logging, env params and the host-side fault-injection hook.
// Parity: src/misc/types.cc:5-64, src/misc/param.cc:9-22, src/misc/checks.cc:8-11 of the reference.
#include "core.h"

#include <cerrno>
#include <cstdarg>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unistd.h>

namespace mccl {

static thread_local mcclResult_t tlsLastError = mcclSuccess;
static std::atomic<int> gLogRank{-1};

int logLevel() {
  static std::atomic<int> level{-1};
  int v = level.load(std::memory_order_acquire);
  if (v >= 0) return v;
  const char* e = getenv("MCCL_DEBUG");
  if (e == nullptr || *e == '\0') v = LOG_NONE;
  else if (!strcasecmp(e, "TRACE")) v = LOG_TRACE;
  else if (!strcasecmp(e, "INFO")) v = LOG_INFO;
  else if (!strcasecmp(e, "NONE") || !strcmp(e, "0")) v = LOG_NONE;
  else v = LOG_WARN;
  level.store(v, std::memory_order_release);
  return v;
}

void logSetRank(int rank) { gLogRank.store(rank); }

void logMsg(int level, const char* file, int line, const char* fmt, ...) {
  static const char* tag[] = {"", "WARN", "INFO", "TRACE"};
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  const char* base = strrchr(file, '/');
  fprintf(stderr, "mccl[%d:%d] %s %s:%d %s\n", (int)getpid(), gLogRank.load(), tag[level & 3],
          base ? base + 1 : file, line, buf);
}

mcclResult_t noteFailure(mcclResult_t r, const char* file, int line) {
  tlsLastError = r;
  if (logLevel() >= LOG_WARN) logMsg(LOG_WARN, file, line, "-> %s", mcclResultStr(r));
  return r;
}

int64_t loadParam(const char* env, int64_t deflt) {
  const char* s = getenv(env);
  if (s == nullptr || *s == '\0') return deflt;
  errno = 0;
  char* end = nullptr;
  long long v = strtoll(s, &end, 0);
  if (errno != 0 || end == s) {
    MCCL_WARN("ignoring %s=%s (not an integer)", env, s);
    return deflt;
  }
  if (v == INT64_MIN) v = INT64_MIN + 1;
  return v;
}

const char* envStr(const char* name) {
  const char* s = getenv(name);
  return (s && *s) ? s : nullptr;
}
double envDouble(const char* name, double deflt) {
  const char* s = envStr(name);
  if (!s) return deflt;
  char* end = nullptr;
  double v = strtod(s, &end);
  return end == s ? deflt : v;
}
int64_t envInt(const char* name, int64_t deflt) {
  const char* s = envStr(name);
  if (!s) return deflt;
  char* end = nullptr;
  long long v = strtoll(s, &end, 0);
  return end == s ? deflt : v;
}

bool faultInject(const char* site) {
  static std::mutex mu;
  static std::string armedSite;
  static long long nth = -1;
  static long long seen = 0;
  static bool parsed = false;
  std::lock_guard<std::mutex> lk(mu);
  if (!parsed) {
    parsed = true;
    const char* s = envStr("MCCL_FAULT_INJECT");
    if (s) {
      const char* colon = strchr(s, ':');
      armedSite = colon ? std::string(s, colon - s) : std::string(s);
      nth = colon ? atoll(colon + 1) : 1;
    }
  }
  if (nth < 0 || armedSite != site) return false;
  return ++seen == nth;
}

}  // namespace mccl

using namespace mccl;

extern "C" {

mcclResult_t mcclGetVersion(int* version) {
  if (version == nullptr) return mcclInvalidArgument;
  *version = MCCL_VERSION_CODE;
  return mcclSuccess;
}

size_t mcclDataSize(mcclDataType_t t) {
  switch (t) {
    case mcclInt8: case mcclUint8: return 1;
    case mcclFloat16: case mcclBfloat16: return 2;
    case mcclInt32: case mcclUint32: case mcclFloat32: return 4;
    case mcclInt64: case mcclUint64: case mcclFloat64: return 8;
    default: return 0;
  }
}

const char* mcclDataTypeStr(mcclDataType_t t) {
  static const char* names[] = {"int8", "uint8", "int32", "uint32", "int64", "uint64",
                                "float16", "bfloat16", "float32", "float64"};
  return ((unsigned)t < (unsigned)mcclNumTypes) ? names[t] : "invalid";
}

const char* mcclRedOpStr(mcclRedOp_t op) {
  static const char* names[] = {"sum", "prod", "max", "min", "avg"};
  return ((unsigned)op < (unsigned)mcclNumOps) ? names[op] : "invalid";
}

const char* mcclResultStr(mcclResult_t r) {
  static const char* names[] = {"success", "unspecified error", "system error", "internal error",
                                "invalid argument", "invalid usage", "remote error", "in progress"};
  return ((unsigned)r < (unsigned)mcclNumResults) ? names[r] : "invalid result";
}
const char* mcclGetErrorString(mcclResult_t r) { return mcclResultStr(r); }
int mcclResultFatal(mcclResult_t r) { return mccl::resultFatal(r) ? 1 : 0; }

const char* mcclAlgoStr(int algo) {
  static const char* names[] = {"ring", "tree", "oneshot", "twoshot", "nvls"};
  if (algo == mcclAlgoAuto) return "auto";
  return ((unsigned)algo < (unsigned)mcclNumAlgos) ? names[algo] : "invalid";
}

const char* mcclCollStr(int coll) {
  static const char* names[] = {"allreduce", "allgather", "reducescatter", "broadcast", "reduce", "alltoall"};
  return ((unsigned)coll < (unsigned)mcclNumColls) ? names[coll] : "invalid";
}

mcclResult_t mcclGetLastError(mcclComm_t) { return tlsLastError; }
mcclResult_t mcclSetLastError(mcclResult_t r) { tlsLastError = r; return mcclSuccess; }

void mcclFreeString(char* s) { free(s); }

}  // extern "C"
