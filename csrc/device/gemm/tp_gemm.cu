// Host side of the tcgen05 GEMM and its fused tensor-parallel forms: tensor-map encoding, shape checks,
// argument set-up and launch.  C ABI so the Python layer can call it with raw pointers.
#include <cuda.h>
#include <cuda_runtime.h>
#include <mutex>

#include "../../comm/comm.h"
#include "../../transport/cuda_mem.h"
#include "gemm_core.cuh"
#include "mccl_ops.h"
#include "gemm_core2.cuh"

using namespace mccl;
using namespace mccl::gemm;

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encodeTiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess) fn = reinterpret_cast<EncodeTiledFn>(p);
    cudaGetLastError();
  });
  return fn;
}

// Row-major [rows, cols] bf16 matrix, box = 64 columns (128 bytes, the swizzle width) x boxRows rows.
mcclResult_t makeMap(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t boxRows) {
  EncodeTiledFn fn = encodeTiled();
  if (fn == nullptr) MCCLFAIL(mcclSystemError);
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, boxRows};
  const cuuint32_t elemStrides[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elemStrides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    MCCL_WARN("cuTensorMapEncodeTiled failed with %d (base %p rows %llu cols %llu box %u)", (int)r, base,
              (unsigned long long)rows, (unsigned long long)cols, boxRows);
    return mcclInvalidArgument;
  }
  return mcclSuccess;
}

// Widest tile width that divides N and fills the machine's last wave best.
int pickBN(int M, int N, int sms) {
  const int cand[] = {256, 224, 192, 160, 128, 96, 64};
  int best = 0;
  double bestEff = -1.0;
  for (int bn : cand) {
    if (N % bn) continue;
    const long tiles = (long)(M / BM) * (N / bn);
    const long waves = (tiles + sms - 1) / sms;
    // Fraction of issued tile slots doing work, discounted for narrow tiles (less reuse of the A tile).
    const double eff = (double)tiles / (double)(waves * sms) * (bn >= 192 ? 1.0 : (bn >= 128 ? 0.92 : 0.75));
    if (eff > bestEff + 1e-9) { bestEff = eff; best = bn; }
  }
  return best;
}

// Tile width of the two-SM kernel for `stripes` 256-row stripes on `pairs` SM pairs.  An MMA over 128 rows per SM
// takes the same time for every N up to 256, so the time of a tile hardly depends on its width (a 224-wide tile
// measured 0.965 of a 256-wide one: less operand traffic): minimise waves x tile time.
// Split tail of the two-SM kernel: with `tiles` tiles on `pairs` SM pairs, how many of the last tiles are cut along
// K and into how many slices (0 / 0: none).  Used when the last wave would be less than half full and a slice keeps
// at least two k blocks.
void tailSplit(long tiles, int pairs, int kBlocks, bool allowed, int* tailTiles, int* tailSlices) {
  *tailTiles = *tailSlices = 0;
  static const bool on = envInt("MCCL_GEMM_SPLIT_TAIL", 1) != 0;
  if (!allowed || !on || tiles <= pairs) return;
  const int rem = (int)(tiles % pairs);
  if (rem == 0 || rem * 2 > pairs) return;
  int slices = pairs / rem;
  static const int cap = (int)envInt("MCCL_GEMM_TAIL_SLICES", 0);      // tuning: at most this many slices per tile
  if (cap > 0 && slices > cap) slices = cap;
  if (slices < 2 || kBlocks / slices < 2) return;
  *tailTiles = rem;
  *tailSlices = slices;
}

int pickBN2(int stripes, int N, int pairs, int kBlocks = 0, bool tailAllowed = false) {
  const int cand[] = {256, 224, 192, 160, 128, 96, 64};
  int best = 0;
  double bestCost = 1e30;
  for (int bn : cand) {
    if (N % bn) continue;
    const long tiles = (long)stripes * (N / bn);
    double waves = (double)((tiles + pairs - 1) / pairs);
    int tt, ts;
    tailSplit(tiles, pairs, kBlocks, tailAllowed, &tt, &ts);
    if (tt > 0) waves = (double)(tiles / pairs) + 1.0 / ts + 0.05;      // the slice wave and the fp32 fix-up
    const double cost = waves * (0.72 + 0.28 * bn / 256.0);
    if (cost < bestCost - 1e-9) { bestCost = cost; best = bn; }
  }
  return best;
}

// fp32 workspace and arrival counters of the split tail, one per (device, stream), zero between launches.
struct TailWs { float* ws; unsigned int* count; };
bool tailWorkspace(int device, cudaStream_t s, TailWs* out) {
  static std::mutex mu;
  static std::vector<std::pair<std::pair<int, cudaStream_t>, TailWs>> all;
  // A launch that is being recorded into a CUDA graph keeps whole tiles: the workspace belongs to a stream, and a
  // graph's kernels run wherever the graph is replayed, possibly beside a launch that uses the same workspace;
  // nor may memory be allocated and the device synchronised while a stream records.
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(s, &capturing) != cudaSuccess) { cudaGetLastError(); return false; }
  if (capturing != cudaStreamCaptureStatusNone) return false;
  std::lock_guard<std::mutex> lk(mu);
  for (auto& e : all) if (e.first.first == device && e.first.second == s) { *out = e.second; return true; }
  const size_t tilesMax = 80, wsBytes = tilesMax * BM2 * 256 * sizeof(float), cntBytes = tilesMax * 2 * sizeof(unsigned int);
  char* p = nullptr;
  if (cudaMalloc((void**)&p, wsBytes + cntBytes) != cudaSuccess || cudaMemset(p, 0, wsBytes + cntBytes) != cudaSuccess ||
      cudaDeviceSynchronize() != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  TailWs w{reinterpret_cast<float*>(p), reinterpret_cast<unsigned int*>(p + wsBytes)};
  all.push_back({{device, s}, w});
  *out = w;
  return true;
}

int* errFlagFor(int device) {
  static std::mutex mu;
  static int* flags[64] = {nullptr};
  std::lock_guard<std::mutex> lk(mu);
  if (device < 0 || device >= 64) return nullptr;
  if (flags[device] == nullptr) {
    int* host = nullptr;
    if (cudaHostAlloc((void**)&host, 64, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    *host = 0;
    flags[device] = host;
  }
  return flags[device];
}

template <int MODE>
mcclResult_t launchMode(const GemmArgs& a, int bn, int grid, cudaStream_t s) {
#define MCCL_GEMM_CASE(BN_)                                                                                          \
  case BN_: {                                                                                                        \
    auto kern = tpGemmKernel<BN_, MODE>;                                                                             \
    static bool attr[64] = {false};                                                                                  \
    int dev = 0; cudaGetDevice(&dev);                                                                                \
    if (!attr[dev & 63]) {                                                                                           \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<BN_>::TOTAL) != cudaSuccess) {  \
        cudaGetLastError(); return mcclSystemError; }                                                                \
      attr[dev & 63] = true;                                                                                         \
    }                                                                                                                \
    kern<<<grid, kThreadsGemm, Smem<BN_>::TOTAL, s>>>(a);                                                             \
    break;                                                                                                           \
  }
  switch (bn) {
    MCCL_GEMM_CASE(256) MCCL_GEMM_CASE(224) MCCL_GEMM_CASE(192) MCCL_GEMM_CASE(160) MCCL_GEMM_CASE(128) MCCL_GEMM_CASE(96)
    MCCL_GEMM_CASE(64)
    default: return mcclInvalidArgument;
  }
#undef MCCL_GEMM_CASE
  return cudaGetLastError() == cudaSuccess ? mcclSuccess : mcclSystemError;
}

int smCount() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

// ---- two-SM kernel: clusters of two CTAs ------------------------------------------------------------------------
bool twoSmWanted() {
  static const bool on = envInt("MCCL_GEMM_2SM", 1) != 0;     // 8192 x 3584 x 8192: 328 us against 369 us for the one-SM kernel
  return on;
}

// Form of the MMA thread the two-SM kernels are built with (see tpGemm2Kernel); the plain GEMM can be switched
// to the others with MCCL_GEMM_VAR for timing comparisons.
constexpr int kGemm2Var = 1;

template <int MODE, int VAR>
bool pairKernelVar(int bn, const void** fn, int* smem) {
#define MCCL_GEMM2_CASE(BN_) case BN_: *fn = reinterpret_cast<const void*>(&tpGemm2Kernel<BN_, MODE, VAR>); *smem = Smem2<BN_>::TOTAL; return true;
  switch (bn) {
    MCCL_GEMM2_CASE(256) MCCL_GEMM2_CASE(224) MCCL_GEMM2_CASE(192) MCCL_GEMM2_CASE(160) MCCL_GEMM2_CASE(128) MCCL_GEMM2_CASE(96)
    MCCL_GEMM2_CASE(64)
    default: return false;
  }
#undef MCCL_GEMM2_CASE
}

template <int MODE>
bool pairKernel(int bn, const void** fn, int* smem) {
  if (MODE == MODE_PLAIN) {
    static const int var = (int)envInt("MCCL_GEMM_VAR", kGemm2Var);
    if (var == 0) return pairKernelVar<MODE_PLAIN, 0>(bn, fn, smem);
    if (var == 2) return pairKernelVar<MODE_PLAIN, 2>(bn, fn, smem);
    if (var == 3) return pairKernelVar<MODE_PLAIN, 3>(bn, fn, smem);
  }
  return pairKernelVar<MODE, kGemm2Var>(bn, fn, smem);
}

void pairConfig(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr, int pairs, int threads, int smem, cudaStream_t s) {
  *cfg = cudaLaunchConfig_t{};
  cfg->gridDim = dim3(2 * pairs, 1, 1);
  cfg->blockDim = dim3(threads, 1, 1);
  cfg->dynamicSmemBytes = smem;
  cfg->stream = s;
  attr->id = cudaLaunchAttributeClusterDimension;
  attr->val.clusterDim.x = 2; attr->val.clusterDim.y = 1; attr->val.clusterDim.z = 1;
  cfg->attrs = attr;
  cfg->numAttrs = 1;
}

mcclResult_t pairPrepare(const void* fn, int smem) {
  if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) { cudaGetLastError(); return mcclSystemError; }
  return mcclSuccess;
}

// Clusters of two that can be resident at once (the fused modes need every CTA of the grid running).
int residentPairs(const void* fn, int threads, int smem) {
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr;
  pairConfig(&cfg, &attr, smCount() / 2, threads, smem, nullptr);
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, fn, &cfg) != cudaSuccess) { cudaGetLastError(); return 0; }
  return n;
}

mcclResult_t launchPairs(const void* fn, int threads, int smem, int pairs, const GemmArgs& a, cudaStream_t s) {
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr;
  pairConfig(&cfg, &attr, pairs, threads, smem, s);
  void* args[1] = {const_cast<GemmArgs*>(&a)};
  if (cudaLaunchKernelExC(&cfg, fn, args) != cudaSuccess) {
    MCCL_WARN("launch of the two-SM GEMM failed: %s", cudaGetErrorString(cudaGetLastError()));
    return mcclSystemError;
  }
  return mcclSuccess;
}

mcclResult_t checkShapes(int M, int N, int K, int nRanks) {
  if (M <= 0 || N <= 0 || K <= 0 || M % (BM * nRanks) || K % BK || N % 64) {
    MCCL_WARN("tcgen05 GEMM needs M %% %d == 0, N %% 64 == 0, K %% 64 == 0 (got %d x %d x %d)", BM * nRanks, M, N, K);
    return mcclInvalidArgument;
  }
  return mcclSuccess;
}

// Largest panel height (in stripes) not above 8 that divides the stripes of one row block.
int pickPanel(int stripesPerBlock) {
  for (int p = 8; p > 1; --p) if (stripesPerBlock % p == 0) return p;
  return 1;
}

}  // namespace

extern "C" {

// Last error code recorded by a GEMM kernel on the current device (0 = none); reading clears it.
int mcclTpGemmLastError(void) {
  int dev = 0;
  cudaGetDevice(&dev);
  int* f = errFlagFor(dev);
  if (f == nullptr) return -1;
  const int v = *f;
  *f = 0;
  return v;
}

// Index-arithmetic probe (host only): the (row stripe, column tile) the t-th tile of a GEMM maps to, for
// mode 0 = plain, 1 = all-gather, 2 = reduce-scatter.  Also reports the tile width the launcher would pick.
int mcclDbgGemmTile(int mode, int M, int N, int nRanks, int rank, int sms, int t, int* stripe, int* nt, int* bn, int* panel) {
  if (M % (BM * nRanks) || N % 64) return -1;
  *bn = pickBN(M, N, sms);
  if (*bn == 0) return -1;
  const int stripes = M / BM, stripesPerBlock = stripes / nRanks, tilesN = N / *bn;
  *panel = pickPanel(stripesPerBlock);
  if (t < 0 || t >= stripes * tilesN) return -1;
  if (mode == 0) tileCoords<MODE_PLAIN>(t, tilesN, *panel, stripesPerBlock, rank, nRanks, stripe, nt);
  else if (mode == 1) tileCoords<MODE_AG>(t, tilesN, *panel, stripesPerBlock, rank, nRanks, stripe, nt);
  else tileCoords<MODE_RS>(t, tilesN, *panel, stripesPerBlock, rank, nRanks, stripe, nt);
  return stripes * tilesN;
}

// C[M,N] = act(A[M,K] * B[N,K]^T), bf16 in and out, on the current device.
mcclResult_t mcclTpGemm(const void* A, const void* B, void* C, int M, int N, int K, int epilogue, int maxCtas, mcclStream_t stream) {
  if (A == nullptr || B == nullptr || C == nullptr) return mcclInvalidArgument;
  MCCLCHECK(checkShapes(M, N, K, 1));
  const int sms = maxCtas > 0 ? maxCtas : smCount();
  const int bn = pickBN(M, N, sms);
  if (bn == 0) return mcclInvalidArgument;
  GemmArgs a;
  memset(&a, 0, sizeof(a));
  MCCLCHECK(makeMap(&a.mapA, A, M, K, BM));
  MCCLCHECK(makeMap(&a.mapB, B, N, K, bn));
  a.M = M; a.N = N; a.K = K;
  a.C = static_cast<__nv_bfloat16*>(C);
  a.epilogue = epilogue;
  int dev = 0;
  cudaGetDevice(&dev);
  int* hostFlag = errFlagFor(dev);
  if (hostFlag == nullptr || cudaHostGetDevicePointer((void**)&a.errFlag, hostFlag, 0) != cudaSuccess) return mcclSystemError;
  a.budgetNs = 2000000000ull;
  a.panel = pickPanel(M / BM);
  const int tiles = (M / BM) * (N / bn);
  return launchMode<MODE_PLAIN>(a, bn, tiles < sms ? tiles : sms, reinterpret_cast<cudaStream_t>(stream));
}

// The same product computed by pairs of SMs (tcgen05.mma.cta_group::2 on 256-row tiles); needs M % 256 == 0.
mcclResult_t mcclTpGemm2(const void* A, const void* B, void* C, int M, int N, int K, int epilogue, int maxCtas, mcclStream_t stream) {
  if (A == nullptr || B == nullptr || C == nullptr) return mcclInvalidArgument;
  MCCLCHECK(checkShapes(M, N, K, 1));
  if (M % BM2) {
    MCCL_WARN("the two-SM GEMM needs M %% %d == 0 (got %d)", BM2, M);
    return mcclInvalidArgument;
  }
  const int pairsMax = std::max(1, (maxCtas > 0 ? maxCtas : smCount()) / 2);
  int bn = pickBN2(M / BM2, N, pairsMax, K / BK, true);
  const int forcedBn = (int)envInt("MCCL_GEMM_BN", 0);          // tuning aid: a tile width that divides N
  if (forcedBn > 0 && N % forcedBn == 0) bn = forcedBn;
  const void* fn = nullptr;
  int smem = 0;
  if (bn == 0 || !pairKernel<MODE_PLAIN>(bn, &fn, &smem)) return mcclInvalidArgument;
  MCCLCHECK(pairPrepare(fn, smem));
  GemmArgs a;
  memset(&a, 0, sizeof(a));
  MCCLCHECK(makeMap(&a.mapA, A, M, K, BM));
  MCCLCHECK(makeMap(&a.mapB, B, N, K, bn / 2));
  a.M = M; a.N = N; a.K = K;
  a.C = static_cast<__nv_bfloat16*>(C);
  a.epilogue = epilogue;
  int dev = 0;
  cudaGetDevice(&dev);
  int* hostFlag = errFlagFor(dev);
  if (hostFlag == nullptr || cudaHostGetDevicePointer((void**)&a.errFlag, hostFlag, 0) != cudaSuccess) return mcclSystemError;
  a.budgetNs = 2000000000ull;
  a.debug = (int)envInt("MCCL_GEMM_DEBUG", 0);
  MCCLCHECK(makeMap(&a.mapC, C, M, N, 32));
  a.tmaStore = 1;
  {
    TailWs w;
    tailSplit((long)(M / BM2) * (N / bn), pairsMax, K / BK, true, &a.tailTiles, &a.tailSlices);
    if (a.tailTiles > 0 && a.tailTiles <= 80 && tailWorkspace(dev, reinterpret_cast<cudaStream_t>(stream), &w)) { a.tailWs = w.ws; a.tailCount = w.count; }
    else a.tailTiles = a.tailSlices = 0;
  }
  a.panel = pickPanel(M / BM2);
  if (envInt("MCCL_GEMM_PANEL", 0) > 0) a.panel = (int)envInt("MCCL_GEMM_PANEL", 0);
  const int tiles = (M / BM2) * (N / bn);
  return launchPairs(fn, kThreadsGemm2, smem, tiles < pairsMax ? tiles : pairsMax, a, reinterpret_cast<cudaStream_t>(stream));
}

// Fused all-gather -> GEMM -> activation.  xShard: this rank's [M/n, K] activations in symmetric memory;
// xFull: local [M, K] workspace; W: [N, K] local weight shard; out: [M, N]; flags: >= 16 uint64 of device
// memory (zeroed by this call).  Collective over `comm`.
mcclResult_t mcclTpAllGatherGemm(mcclComm_t comm, const void* xShard, void* xFull, const void* W, void* out, void* flags,
                                 int M, int N, int K, int epilogue, mcclStream_t stream) {
  if (comm == nullptr || !comm->cuda || comm->cu == nullptr || xShard == nullptr || xFull == nullptr || W == nullptr ||
      out == nullptr || flags == nullptr) return mcclInvalidArgument;
  const int n = comm->nRanks;
  MCCLCHECK(checkShapes(M, N, K, n));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  CUDACHECK(cudaSetDevice(comm->device));
  const size_t shardBytes = (size_t)(M / n) * K * 2;
  Segment* seg = segmentFind(comm->cu, xShard, shardBytes);
  if (seg == nullptr) {
    MCCL_WARN("mcclTpAllGatherGemm: the activation shard must live in symmetric memory (mcclMemAlloc)");
    return mcclInvalidArgument;
  }
  // Two-SM form: every rank must take the same branch, which it does because the decision depends on the
  // shape, an environment variable and the GPU model only.
  const bool two = twoSmWanted() && (M / n) % BM2 == 0;
  const void* fn2 = nullptr;
  int smem2 = 0, pairs = 0;
  int sms = std::min(smCount(), MCCL_MAX_CTAS);
  int bn = 0;
  if (two) {
    bn = pickBN2(M / BM2, N, sms / 2, K / BK, true);
    if (bn == 0 || !pairKernel<MODE_AG>(bn, &fn2, &smem2)) return mcclInvalidArgument;
    MCCLCHECK(pairPrepare(fn2, smem2));
    pairs = std::min(residentPairs(fn2, kThreadsGemm, smem2), sms / 2);
    if (pairs <= 0) return mcclSystemError;
    if (pairs != sms / 2) bn = pickBN2(M / BM2, N, pairs, K / BK, true);
    if (bn == 0 || !pairKernel<MODE_AG>(bn, &fn2, &smem2)) return mcclInvalidArgument;
    MCCLCHECK(pairPrepare(fn2, smem2));
  } else {
    bn = pickBN(M, N, sms);
    if (bn == 0) return mcclInvalidArgument;
  }
  GemmArgs a;
  memset(&a, 0, sizeof(a));
  MCCLCHECK(makeMap(&a.mapA, xFull, M, K, BM));
  MCCLCHECK(makeMap(&a.mapB, W, N, K, two ? bn / 2 : bn));
  a.M = M; a.N = N; a.K = K;
  a.C = static_cast<__nv_bfloat16*>(out);
  a.epilogue = epilogue;
  if (two) {
    MCCLCHECK(makeMap(&a.mapC, out, M, N, 32));
    a.tmaStore = 1;
    TailWs w;
    tailSplit((long)(M / BM2) * (N / bn), pairs, K / BK, true, &a.tailTiles, &a.tailSlices);
    if (a.tailTiles > 0 && a.tailTiles <= 80 && tailWorkspace(comm->device, s, &w)) { a.tailWs = w.ws; a.tailCount = w.count; }
    else a.tailTiles = a.tailSlices = 0;
  }
  int* hostFlag = errFlagFor(comm->device);
  if (hostFlag == nullptr || cudaHostGetDevicePointer((void**)&a.errFlag, hostFlag, 0) != cudaSuccess) return mcclSystemError;
  a.peers = comm->cu->peers;
  a.budgetNs = 2 * a.peers.timeoutNs;
  a.callIndex = 1;
  a.panel = pickPanel(M / (two ? BM2 : BM) / n);
  a.shardReady = static_cast<uint64_t*>(flags);
  const size_t off = (size_t)(static_cast<const char*>(xShard) - seg->local);
  for (int p = 0; p < n; ++p) a.xPeer[p] = seg->peer[p] + off;
  a.xFull = static_cast<char*>(xFull);
  CUDACHECK(cudaMemsetAsync(flags, 0, MCCL_MAX_RANKS * sizeof(uint64_t), s));
  // Every CTA's communication warps take part in the copy and in the cross-GPU barriers, so the grid is
  // the same on every rank and never larger than what is resident at once.
  mcclResult_t rc;
  if (two) {
    const int tiles = (M / BM2) * (N / bn);
    rc = launchPairs(fn2, kThreadsGemm, smem2, tiles < pairs ? tiles : pairs, a, s);
  } else {
    const int tiles = (M / BM) * (N / bn);
    rc = launchMode<MODE_AG>(a, bn, tiles < sms ? tiles : sms, s);
  }
  if (rc == mcclSuccess) comm->launches.fetch_add(1);
  return rc;
}

// Fused GEMM -> reduce-scatter over the row (token) dimension.  H: [M, K] local activations; W: [N, K] local
// weight shard; partial: [M, N] staging in symmetric memory; flags: symmetric memory of at least
// (16 + M/128 + n * M/(128 n)) uint64, zeroed once at allocation; out: [M/n, N] reduced rows of this rank's
// block; accum: [M/n, N] fp32 local workspace.  callIndex counts the calls made with this flags buffer (1, 2, ...).  Collective over `comm`.
mcclResult_t mcclTpGemmReduceScatter(mcclComm_t comm, const void* H, const void* W, void* partial, void* flags, void* out,
                                     float* accum, int M, int N, int K, uint64_t callIndex, mcclStream_t stream) {
  if (comm == nullptr || !comm->cuda || comm->cu == nullptr || H == nullptr || W == nullptr || partial == nullptr ||
      flags == nullptr || out == nullptr || accum == nullptr || callIndex == 0) return mcclInvalidArgument;
  const int n = comm->nRanks;
  MCCLCHECK(checkShapes(M, N, K, n));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  CUDACHECK(cudaSetDevice(comm->device));
  const int stripes = M / BM, stripesPerBlock = stripes / n;
  const size_t flagWords = 16 + (size_t)stripes + (size_t)n * stripesPerBlock;
  Segment* pseg = segmentFind(comm->cu, partial, (size_t)M * N * 2);
  Segment* fseg = segmentFind(comm->cu, flags, flagWords * 8);
  if (pseg == nullptr || fseg == nullptr) {
    MCCL_WARN("mcclTpGemmReduceScatter: staging and flags must live in symmetric memory (mcclMemAlloc)");
    return mcclInvalidArgument;
  }
  const bool two = twoSmWanted() && (M / n) % BM2 == 0;
  const void* fn2 = nullptr;
  int smem2 = 0, pairs = 0;
  int sms = std::min(smCount(), MCCL_MAX_CTAS);
  int bn = 0;
  if (two) {
    bn = pickBN2(M / BM2, N, sms / 2);
    if (bn == 0 || !pairKernel<MODE_RS>(bn, &fn2, &smem2)) return mcclInvalidArgument;
    MCCLCHECK(pairPrepare(fn2, smem2));
    pairs = std::min(residentPairs(fn2, kThreadsGemm, smem2), sms / 2);
    if (pairs <= 0) return mcclSystemError;
    if (pairs != sms / 2) bn = pickBN2(M / BM2, N, pairs);
    if (bn == 0 || !pairKernel<MODE_RS>(bn, &fn2, &smem2)) return mcclInvalidArgument;
    MCCLCHECK(pairPrepare(fn2, smem2));
  } else {
    bn = pickBN(M, N, sms);
    if (bn == 0) return mcclInvalidArgument;
  }
  GemmArgs a;
  memset(&a, 0, sizeof(a));
  MCCLCHECK(makeMap(&a.mapA, H, M, K, BM));
  MCCLCHECK(makeMap(&a.mapB, W, N, K, two ? bn / 2 : bn));
  a.M = M; a.N = N; a.K = K;
  a.C = static_cast<__nv_bfloat16*>(partial);
  a.epilogue = EPI_NONE;
  if (two) { MCCLCHECK(makeMap(&a.mapC, partial, M, N, 32)); a.tmaStore = 1; }
  int* hostFlag = errFlagFor(comm->device);
  if (hostFlag == nullptr || cudaHostGetDevicePointer((void**)&a.errFlag, hostFlag, 0) != cudaSuccess) return mcclSystemError;
  a.peers = comm->cu->peers;
  a.budgetNs = 2 * a.peers.timeoutNs;
  a.callIndex = callIndex;
  const size_t poff = (size_t)(static_cast<char*>(partial) - pseg->local), foff = (size_t)(static_cast<char*>(flags) - fseg->local);
  uint64_t* localFlags = static_cast<uint64_t*>(flags);
  a.stripeCount = localFlags + 16;
  for (int p = 0; p < n; ++p) {
    a.partialPeer[p] = pseg->peer[p] + poff;
    a.tileReadyPeer[p] = reinterpret_cast<uint64_t*>(fseg->peer[p] + foff) + 16 + stripes;
  }
  a.out = static_cast<__nv_bfloat16*>(out);
  a.accum = accum;
  a.panel = pickPanel(two ? stripesPerBlock / 2 : stripesPerBlock);
  CUDACHECK(cudaMemsetAsync(a.stripeCount, 0, (size_t)stripes * sizeof(uint64_t), s));   // local counters only
  mcclResult_t rc;
  if (two) {
    const int tiles = (M / BM2) * (N / bn);
    rc = launchPairs(fn2, kThreadsGemm, smem2, tiles < pairs ? tiles : pairs, a, s);
  } else {
    const int tiles = (M / BM) * (N / bn);
    rc = launchMode<MODE_RS>(a, bn, tiles < sms ? tiles : sms, s);
  }
  if (rc == mcclSuccess) comm->launches.fetch_add(1);
  return rc;
}

}  // extern "C"
