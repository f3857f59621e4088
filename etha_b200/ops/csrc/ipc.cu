// CUDA IPC plumbing: export the allocation behind a device pointer, map a peer's allocation into
// this process, enable peer access.  The reference gets the same effect through torch's CUDA-IPC
// pickling of whole tensors (src/etha/tensor_bus/client.py:314, src/etha/tensor_bus/utils.py:14-69);
// here handles are plain 64-byte blobs so that any agent can open any other agent's registration.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>

#include "common.h"
#include "m2n.h"

namespace {
int fail(cudaError_t e, const char* what) {
  snprintf(etha_err_buf(), ETHA_ERR_LEN, "%s: %s", what, cudaGetErrorString(e));
  return -(int)e - 1000;
}
typedef CUresult (*GetAddressRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
GetAddressRangeFn address_range_fn() {
  static GetAddressRangeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) == cudaSuccess && p)
      fn = reinterpret_cast<GetAddressRangeFn>(p);
  }
  return fn;
}
std::mutex g_mu;
struct Opened { uint64_t base; int refs; };
std::map<std::string, Opened> g_opened;      // handle bytes -> mapping
std::map<uint64_t, std::string> g_by_base;
}  // namespace

extern "C" {

int etha_ipc_export(uint64_t ptr, unsigned char* handle64, uint64_t* base, uint64_t* size) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  GetAddressRangeFn fn = address_range_fn();
  if (!fn) { snprintf(etha_err_buf(), ETHA_ERR_LEN, "cuMemGetAddressRange not available"); return -1; }
  CUdeviceptr b = 0;
  size_t n = 0;
  CUresult r = fn(&b, &n, (CUdeviceptr)ptr);
  if (r != CUDA_SUCCESS) { snprintf(etha_err_buf(), ETHA_ERR_LEN, "cuMemGetAddressRange failed (%d)", (int)r); return -2; }
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(b));
  if (e != cudaSuccess) return fail(e, "cudaIpcGetMemHandle");
  memcpy(handle64, &h, 64);
  *base = (uint64_t)b;
  *size = (uint64_t)n;
  return 0;
}

int etha_ipc_open(const unsigned char* handle64, uint64_t* mapped_base) {
  std::lock_guard<std::mutex> lock(g_mu);
  std::string key(reinterpret_cast<const char*>(handle64), 64);
  auto it = g_opened.find(key);
  if (it != g_opened.end()) {
    it->second.refs++;
    *mapped_base = it->second.base;
    return 0;
  }
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail(e, "cudaIpcOpenMemHandle");
  g_opened[key] = {(uint64_t)p, 1};
  g_by_base[(uint64_t)p] = key;
  *mapped_base = (uint64_t)p;
  return 0;
}

int etha_ipc_close(uint64_t mapped_base) {
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_by_base.find(mapped_base);
  if (it == g_by_base.end()) return -1;
  auto op = g_opened.find(it->second);
  if (--op->second.refs > 0) return 0;
  cudaError_t e = cudaIpcCloseMemHandle(reinterpret_cast<void*>(mapped_base));
  g_opened.erase(op);
  g_by_base.erase(it);
  return e == cudaSuccess ? 0 : fail(e, "cudaIpcCloseMemHandle");
}

// Copy-engine copy between two device addresses (either may be a mapped peer allocation): the DMA baseline the
// copy kernels are compared with.
int etha_copy_engine_d2d(uint64_t dst, uint64_t src, uint64_t bytes, void* stream) {
  cudaError_t e = cudaMemcpyAsync(reinterpret_cast<void*>(dst), reinterpret_cast<const void*>(src), bytes,
                                  cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
  return e == cudaSuccess ? 0 : fail(e, "cudaMemcpyAsync(device to device)");
}

int etha_enable_peer_access(int peer_device) {
  int cur = 0;
  cudaGetDevice(&cur);
  if (cur == peer_device) return 0;
  int can = 0;
  cudaError_t e = cudaDeviceCanAccessPeer(&can, cur, peer_device);
  if (e != cudaSuccess) return fail(e, "cudaDeviceCanAccessPeer");
  if (!can) { snprintf(etha_err_buf(), ETHA_ERR_LEN, "device %d cannot access device %d", cur, peer_device); return -1; }
  e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return 0; }
  return e == cudaSuccess ? 0 : fail(e, "cudaDeviceEnablePeerAccess");
}

int etha_device_info(int* sm_count, int* cc_major, int* cc_minor, int* multicast_supported) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(e, "cudaGetDevice");
  cudaDeviceGetAttribute(sm_count, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(cc_major, cudaDevAttrComputeCapabilityMajor, dev);
  cudaDeviceGetAttribute(cc_minor, cudaDevAttrComputeCapabilityMinor, dev);
  *multicast_supported = 0;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuDeviceGetAttribute", &p, cudaEnableDefault, &q) == cudaSuccess && p) {
    typedef CUresult (*Fn)(int*, CUdevice_attribute, CUdevice);
    int v = 0;
    if (reinterpret_cast<Fn>(p)(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) == CUDA_SUCCESS) *multicast_supported = v;
  }
  return 0;
}

}  // extern "C"
