// Cost model and algorithm choice.
//
//   time_us = alpha[algo] + step[algo] * steps(algo, n) + bytes * traffic(algo, coll, n) / (1000 * bw[algo])
//
// steps() counts dependent link crossings, traffic() the bytes that cross a rank's busiest direction per
// payload byte.  Unlike the reference's model (src/graph/tuning.cc:16-31), whose bandwidth term is the same
// for ring and tree, the traffic factor differs per algorithm, which is what separates one-shot (latency
// optimal, (n-1)x traffic) from two-shot/ring (2(n-1)/n) and NVLS (about 1: the switch reduces and
// replicates).  alpha/step/bw start from the topology (measured where calibration ran) and can be
// overridden from a cache file.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>

#include <sys/stat.h>
#include <unistd.h>
#include <string>
#include <ctype.h>
#include "graph.h"

namespace mccl {

static int ceilLog2(int n) { int l = 0; while ((1 << l) < n) ++l; return l; }

int algoSteps(int algo, int n) {
  if (n <= 1) return 0;
  switch (algo) {
    case mcclAlgoRing:    return 2 * (n - 1);
    case mcclAlgoTree:    return 2 * ceilLog2(n);
    case mcclAlgoOneShot: return 1;
    case mcclAlgoTwoShot: return 2;
    case mcclAlgoNvls:    return 2;
    default:              return 0;
  }
}

double algoTraffic(int algo, int coll, int n) {
  if (n <= 1) return 0.0;
  const double f = (double)(n - 1) / n;
  switch (coll) {
    case mcclCollAllReduce:
      switch (algo) {
        case mcclAlgoRing: case mcclAlgoTwoShot: return 2.0 * f;
        case mcclAlgoTree:    return 2.0;
        case mcclAlgoOneShot: return (double)(n - 1);
        case mcclAlgoNvls:    return 1.0 + 1.0 / n;
      }
      break;
    case mcclCollAllGather:      // bytes = total gathered size
    case mcclCollReduceScatter:  // bytes = total input size
    case mcclCollAllToAll:
      switch (algo) {
        case mcclAlgoTree: return 1.0 + f;        // everything through the hub
        default:           return f;
      }
    case mcclCollBroadcast:
      switch (algo) {
        case mcclAlgoRing: return 1.0;
        case mcclAlgoTree: return 2.0;            // an interior node forwards to two children
        case mcclAlgoNvls: return 1.0;
        case mcclAlgoTwoShot: return 2.0 * f;     // scatter from the root, then all-gather
        default:           return (double)(n - 1); // root writes every peer
      }
    case mcclCollReduce:
      switch (algo) {
        case mcclAlgoRing: return f + 1.0 / n;
        case mcclAlgoTree: return 2.0;
        case mcclAlgoNvls: return 1.0;
        case mcclAlgoTwoShot: return 2.0 * f;     // every rank folds a shard, the root collects them
        default:           return (double)(n - 1); // root reads every peer
      }
  }
  return 1.0;
}

mcclResult_t tunerInit(const TopoSystem& sys, const TopoGraph graphs[mcclNumAlgos], bool cudaTransport, TunerModel* out) {
  if (out == nullptr) MCCLFAIL(mcclInvalidArgument);
  (void)sys;
  out->cuda = cudaTransport;
  for (int a = 0; a < mcclNumAlgos; ++a) {
    out->viable[a] = graphs[a].viable;
    out->bw[a] = graphs[a].bw;
    out->stepUs[a] = graphs[a].latencyUs;
    out->alphaUs[a] = 0.f;
  }
  if (cudaTransport) {
    // Defaults fitted to this library's kernels on B200 (2 and 8 GPUs, bf16 sum, back-to-back launches):
    // alpha grows with the number of peers a CTA signals and waits for; the bandwidth fractions are what
    // each algorithm sustains of the 900 GB/s port at 1 GiB once its traffic factor is taken out.
    // MCCL_CALIBRATE=1 or MCCL_TUNER_CACHE replace them with values measured on the machine at hand.
    const float n = (float)sys.nodes.size();
    out->alphaUs[mcclAlgoOneShot] = 8.f + 2.1f * n;
    out->alphaUs[mcclAlgoNvls] = 15.f + 1.3f * n;
    out->alphaUs[mcclAlgoTwoShot] = 17.f + 4.2f * n;
    out->alphaUs[mcclAlgoRing] = 12.f;
    out->alphaUs[mcclAlgoTree] = 12.f;
    out->stepUs[mcclAlgoOneShot] = out->stepUs[mcclAlgoNvls] = out->stepUs[mcclAlgoTwoShot] = 0.f;
    out->stepUs[mcclAlgoRing] = 9.6f;
    out->stepUs[mcclAlgoTree] = 9.0f;
    out->bw[mcclAlgoTwoShot] *= 0.60f;
    out->bw[mcclAlgoOneShot] *= 0.145f;
    out->bw[mcclAlgoRing] *= 0.23f;
    out->bw[mcclAlgoTree] *= 0.047f;
    out->bw[mcclAlgoNvls] *= 0.60f;
    out->oneShotMaxBytes = (size_t)envInt("MCCL_DIRECT_MAX_BYTES", 2 << 20);
    out->oneShotMaxRanks = (int)envInt("MCCL_DIRECT_MAX_RANKS", 16);
  } else {
    out->oneShotMaxBytes = (size_t)envInt("MCCL_DIRECT_MAX_BYTES", 2 << 20);
    out->oneShotMaxRanks = (int)envInt("MCCL_DIRECT_MAX_RANKS", 8);
  }
  const char* cache = envStr("MCCL_TUNER_CACHE");
  if (cache) tunerLoadCache(out, cache);
  return mcclSuccess;
}

std::string tunerCachePath(int nRanks, const char* gpuName) {
  const char* forced = envStr("MCCL_TUNER_CACHE");
  if (forced && *forced) return forced;
  const char* home = envStr("HOME");
  std::string dir = std::string(home && *home ? home : "/tmp") + "/.cache/mccl_b200";
  std::string gpu;
  for (const char* p = gpuName ? gpuName : "gpu"; *p; ++p) gpu += (isalnum((unsigned char)*p) ? *p : '_');
  return dir + "/tuner-" + std::to_string(nRanks) + "x" + gpu + ".txt";
}

mcclResult_t tunerLoadCache(TunerModel* m, const char* path) {
  FILE* f = fopen(path, "r");
  if (f == nullptr) return mcclSuccess;  // nothing cached yet
  m->measured = true;
  char name[32];
  float alpha, step, bw;
  while (fscanf(f, "%31s %f %f %f", name, &alpha, &step, &bw) == 4) {
    for (int a = 0; a < mcclNumAlgos; ++a)
      if (!strcmp(name, mcclAlgoStr(a))) { m->alphaUs[a] = alpha; m->stepUs[a] = step; if (bw > 0.f) m->bw[a] = bw; }
  }
  fclose(f);
  return mcclSuccess;
}

mcclResult_t tunerSaveCache(const TunerModel& m, const char* path) {
  std::string dir(path);
  const size_t slash = dir.rfind('/');
  if (slash != std::string::npos && slash > 0) {       // mkdir -p of the parent
    dir.resize(slash);
    for (size_t i = 1; i <= dir.size(); ++i)
      if (i == dir.size() || dir[i] == '/') { std::string part = dir.substr(0, i); mkdir(part.c_str(), 0755); }
  }
  // Written beside the target and renamed into place, so a reader never sees half a file.
  const std::string tmp = std::string(path) + ".tmp" + std::to_string((long)getpid());
  FILE* f = fopen(tmp.c_str(), "w");
  if (f == nullptr) MCCLFAIL(mcclSystemError);
  for (int a = 0; a < mcclNumAlgos; ++a) fprintf(f, "%s %g %g %g\n", mcclAlgoStr(a), m.alphaUs[a], m.stepUs[a], m.bw[a]);
  fclose(f);
  if (rename(tmp.c_str(), path) != 0) { remove(tmp.c_str()); MCCLFAIL(mcclSystemError); }
  return mcclSuccess;
}

mcclResult_t tunerAlgoTime(const TunerModel& m, int algo, int coll, int n, size_t bytes, float* us) {
  if (us == nullptr || (unsigned)algo >= (unsigned)mcclNumAlgos) MCCLFAIL(mcclInvalidArgument);
  if (!m.viable[algo] || m.bw[algo] <= 0.f) { *us = INFINITY; return mcclSuccess; }
  // bw[oneshot] describes the push all-reduce.  The "direct" forms of the other collectives on the cuda transport
  // are plain peer copies / folds in the pull kernel, which sustains what two-shot's phases do.
  const float bw = (m.cuda && algo == mcclAlgoOneShot && coll != mcclCollAllReduce && m.bw[mcclAlgoTwoShot] > 0.f)
                       ? m.bw[mcclAlgoTwoShot] : m.bw[algo];
  *us = m.alphaUs[algo] + m.stepUs[algo] * (float)algoSteps(algo, n) +
        (float)((double)bytes * algoTraffic(algo, coll, n) / (1000.0 * bw));
  return mcclSuccess;
}

// The switch hands back a 16-bit sum already rounded to the element type; the 1/n of an average is applied to
// that.  With n a power of two the scale is exact, so the result equals the once-rounded average the peer-load
// kernels produce; for other n the average would be rounded twice, and such calls are left to two-shot.
bool nvlsAvgExact(int dt, int op, int n) {
  if (op != mcclAvg || (dt != mcclFloat16 && dt != mcclBfloat16)) return true;
  return n > 0 && (n & (n - 1)) == 0;
}

bool algoSupports(int algo, int coll, int dt, int op, bool cudaTransport) {
  if (!cudaTransport) {
    if (algo == mcclAlgoTwoShot || algo == mcclAlgoNvls) return false;
    if (algo == mcclAlgoOneShot) return coll != mcclCollBroadcast;   // broadcast has ring and tree only
    return coll != mcclCollAllToAll;
  }
  const bool gpuType = dt == mcclFloat32 || dt == mcclFloat16 || dt == mcclBfloat16 || dt == mcclInt32 ||
                       dt == mcclUint32 || dt == mcclInt64 || dt == mcclUint64 || dt == mcclInt8 ||
                       dt == mcclUint8 || dt == mcclFloat64;
  if (!gpuType) return false;
  const bool reducing = coll == mcclCollAllReduce || coll == mcclCollReduceScatter || coll == mcclCollReduce;
  switch (algo) {
    case mcclAlgoNvls:
      if (coll == mcclCollAllToAll) return false;
      if (!reducing) return true;
      // The vector forms of multimem.ld_reduce the kernels use: add for f32, add / min / max for f16 and bf16.
      // (Integer types only have scalar forms, which the peer-load kernels beat; they are left to two-shot.)
      if (dt == mcclFloat32) return op == mcclSum || op == mcclAvg;
      if (dt == mcclFloat16 || dt == mcclBfloat16) return op == mcclSum || op == mcclAvg || op == mcclMax || op == mcclMin;
      return false;
    case mcclAlgoRing:    // the ring kernel's reduce steps / gather steps, with a scatter before or a collect after
    case mcclAlgoTree:    // the tree kernel's up phase / down phase, likewise
      return coll != mcclCollAllToAll;
    case mcclAlgoTwoShot:
      return coll == mcclCollAllReduce || coll == mcclCollBroadcast || coll == mcclCollReduce;
    case mcclAlgoOneShot:
      return true;   // "direct": every rank reads/writes every peer once
    default: return false;
  }
}

mcclResult_t tunerPick(const TunerModel& m, int coll, int n, size_t bytes, int dt, int op, const int enabled[mcclNumAlgos],
                       bool cudaTransport, int* algo) {
  if (algo == nullptr) MCCLFAIL(mcclInvalidArgument);
  // Measured on 2 and 8 B200: for all-gather, reduce-scatter, broadcast and reduce the NVLS form is at
  // least as fast as the peer-load form at every size, so the model is only consulted for all-reduce.
  // Exception, measured on 4 B200: multicast delivers about 505 GB/s into each GPU, peer loads 650 and more, so from
  // 64 MB up all-gather and reduce-scatter are faster in the peer-load ("direct") form there (64 MB, us: all-gather
  // 111.7 direct / 120.7 NVLS / 116.8 NCCL; reduce-scatter 107.0 / 124.8 / 118.2).  On 8 GPUs the two forms measured
  // the same, so the rule is kept to small worlds.
  if (cudaTransport && (coll == mcclCollAllGather || coll == mcclCollReduceScatter) && n <= 4 && bytes >= ((size_t)64 << 20) &&
      (enabled == nullptr || enabled[mcclAlgoOneShot]) && m.viable[mcclAlgoOneShot]) {
    *algo = mcclAlgoOneShot;
    return mcclSuccess;
  }
  if (cudaTransport && coll != mcclCollAllReduce && (enabled == nullptr || enabled[mcclAlgoNvls]) && m.viable[mcclAlgoNvls] &&
      algoSupports(mcclAlgoNvls, coll, dt, op, true) && nvlsAvgExact(dt, op, n)) {
    *algo = mcclAlgoNvls;
    return mcclSuccess;
  }
  int best = -1;
  float bestUs = INFINITY;
  // Ties go to the lower-numbered algorithm (ring), as in the reference.
  for (int a = 0; a < mcclNumAlgos; ++a) {
    if (enabled != nullptr && !enabled[a]) continue;
    if (!m.viable[a] || !algoSupports(a, coll, dt, op, cudaTransport)) continue;
    if (a == mcclAlgoNvls && !nvlsAvgExact(dt, op, n)) continue;
    if (a == mcclAlgoOneShot && coll == mcclCollAllReduce &&
        (bytes > m.oneShotMaxBytes || n > m.oneShotMaxRanks)) continue;
    if (!cudaTransport && a == mcclAlgoOneShot && (bytes > m.oneShotMaxBytes || n > m.oneShotMaxRanks)) continue;
    float us;
    tunerAlgoTime(m, a, coll, n, bytes, &us);
    if (us < bestUs) { bestUs = us; best = a; }
  }
  if (best < 0) {
    // The allow-list left nothing that can run this call: fall back to anything viable rather than fail.
    for (int a = 0; a < mcclNumAlgos && best < 0; ++a)
      if (m.viable[a] && algoSupports(a, coll, dt, op, cudaTransport) &&
          !(a == mcclAlgoOneShot && coll == mcclCollAllReduce && bytes > m.oneShotMaxBytes && cudaTransport)) best = a;
  }
  if (best < 0) MCCLFAIL(mcclInternalError);
  *algo = best;
  return mcclSuccess;
}

mcclResult_t parseList(const char* str, const char* const names[], int n, int* enabled) {
  if (str == nullptr || *str == '\0') { for (int i = 0; i < n; ++i) enabled[i] = 1; return mcclSuccess; }
  const bool invert = str[0] == '^';
  if (invert) ++str;
  for (int i = 0; i < n; ++i) enabled[i] = invert ? 1 : 0;
  std::string s(str);
  size_t pos = 0;
  while (pos <= s.size()) {
    size_t comma = s.find(',', pos);
    if (comma == std::string::npos) comma = s.size();
    std::string tok = s.substr(pos, comma - pos);
    pos = comma + 1;
    if (tok.empty()) continue;
    bool known = false;
    for (int i = 0; i < n; ++i)
      if (!strcasecmp(tok.c_str(), names[i])) { enabled[i] = invert ? 0 : 1; known = true; }
    if (!known) {
      MCCL_WARN("unknown name '%s' in list '%s'", tok.c_str(), str);
      return mcclInvalidArgument;
    }
  }
  return mcclSuccess;
}

mcclResult_t getEnabledAlgos(int enabled[mcclNumAlgos]) {
  static const char* const names[] = {"ring", "tree", "oneshot", "twoshot", "nvls"};
  mcclResult_t rc = parseList(envStr("MCCL_ALGO"), names, mcclNumAlgos, enabled);
  if (rc != mcclSuccess) for (int i = 0; i < mcclNumAlgos; ++i) enabled[i] = 1;
  return mcclSuccess;
}

}  // namespace mccl
