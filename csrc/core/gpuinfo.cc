// GPU discovery through the CUDA runtime (statically linked, so the library loads on hosts that have no
// driver: every entry point here degrades to "no device").
// Role parity: mcclDiscoverChip (src/misc/utils.h:8-28, src/misc/utils.cpp:18-114) of the reference.
#include <cstring>
#include <cuda.h>
#include <cuda_runtime.h>

#include "core.h"

namespace mccl {

int cudaDeviceCountSafe() {
  static int cached = -1;
  if (cached >= 0) return cached;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) { n = 0; cudaGetLastError(); }
  cached = n;
  return n;
}

mcclResult_t discoverGpu(int device, GpuInfo* out) {
  if (out == nullptr) MCCLFAIL(mcclInvalidArgument);
  if (cudaDeviceCountSafe() <= 0) MCCLFAIL(mcclInvalidUsage);
  if (device < 0 && cudaGetDevice(&device) != cudaSuccess) MCCLFAIL(mcclSystemError);
  cudaDeviceProp p;
  if (cudaGetDeviceProperties(&p, device) != cudaSuccess) MCCLFAIL(mcclSystemError);
  *out = GpuInfo();
  out->device = device;
  snprintf(out->name, sizeof(out->name), "%s", p.name);
  out->ccMajor = p.major;
  out->ccMinor = p.minor;
  out->smCount = p.multiProcessorCount;
  out->hbmBytes = p.totalGlobalMem;
  out->l2Bytes = p.l2CacheSize;
  memcpy(out->uuid, &p.uuid, sizeof(out->uuid));
  cudaDeviceGetPCIBusId(out->busId, sizeof(out->busId), device);
  int v = 0;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMemoryPoolsSupported, device) == cudaSuccess) out->vmm = v;
  // Multicast support is a driver attribute; ask through the runtime's driver entry point lookup.
  typedef CUresult (*GetAttr)(int*, CUdevice_attribute, CUdevice);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qr;
  if (cudaGetDriverEntryPoint("cuDeviceGetAttribute", &fn, cudaEnableDefault, &qr) == cudaSuccess && fn) {
    int mc = 0, vm = 0, fd = 0;
    ((GetAttr)fn)(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device);
    ((GetAttr)fn)(&vm, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, device);
    ((GetAttr)fn)(&fd, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, device);
    out->multicast = mc;
    out->vmm = vm && fd;
  }
  cudaGetLastError();
  return mcclSuccess;
}

bool gpuSupported(const GpuInfo& g) { return g.ccMajor == 10; }

std::string gpuDescribe(const GpuInfo& g) {
  char buf[256];
  snprintf(buf, sizeof(buf), "%s sm_%d%d %d SMs %.0f GiB %s multicast=%d vmm=%d", g.name, g.ccMajor, g.ccMinor, g.smCount,
           (double)g.hbmBytes / (1u << 30), g.busId, g.multicast, g.vmm);
  return buf;
}

}  // namespace mccl
