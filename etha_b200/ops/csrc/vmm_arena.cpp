// VMM arena: device memory that can be shared by file descriptor and bound to an NVLS multicast object.
//
// `cudaMalloc` memory travels between processes as an IPC handle, but it cannot be bound to a multicast
// object; NVSwitch multicast (`multimem.st`, one store delivered to every replica) needs allocations made
// with the virtual-memory-management API.  This file wraps exactly the driver calls that takes:
// cuMemCreate / export / import / map, and cuMulticastCreate / AddDevice / BindMem / map.  The driver entry
// points are looked up through the runtime (`cudaGetDriverEntryPoint`), so the library does not link libcuda
// and still loads on a machine without a driver.
//
// The reference has no counterpart: it relies on torch's caching allocator and NCCL broadcast for Replicate
// targets (src/etha/comm/transfer.py:33-41).
#include <cuda.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include <cstdio>
#include <cstring>

#include "common.h"
#include "m2n.h"

namespace {

template <typename Fn>
Fn entry(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || !p) return nullptr;
  return reinterpret_cast<Fn>(p);
}

int drv_fail(CUresult r, const char* what) {
  snprintf(etha_err_buf(), ETHA_ERR_LEN, "%s failed with CUresult %d", what, (int)r);
  return -2000 - (int)r;
}

#define DRV(name, type) \
  static type fn_##name = entry<type>(#name); \
  if (!fn_##name) { snprintf(etha_err_buf(), ETHA_ERR_LEN, "driver entry point %s not available", #name); return -1999; }

typedef CUresult (*MemCreateFn)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
typedef CUresult (*MemReleaseFn)(CUmemGenericAllocationHandle);
typedef CUresult (*MemGranFn)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
typedef CUresult (*MemExportFn)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
typedef CUresult (*MemImportFn)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
typedef CUresult (*MemReserveFn)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
typedef CUresult (*MemMapFn)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
typedef CUresult (*MemSetAccessFn)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
typedef CUresult (*MemUnmapFn)(CUdeviceptr, size_t);
typedef CUresult (*MemAddrFreeFn)(CUdeviceptr, size_t);
typedef CUresult (*McCreateFn)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
typedef CUresult (*McAddDevFn)(CUmemGenericAllocationHandle, CUdevice);
typedef CUresult (*McBindFn)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
typedef CUresult (*McBindAddrFn)(CUmemGenericAllocationHandle, size_t, CUdeviceptr, size_t, unsigned long long);
typedef CUresult (*McUnbindFn)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
typedef CUresult (*McGranFn)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);

CUmemAllocationProp device_prop(int dev) {
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = dev;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

int map_rw(CUmemGenericAllocationHandle h, size_t size, size_t align, int dev, uint64_t* va_out) {
  DRV(cuMemAddressReserve, MemReserveFn)
  DRV(cuMemMap, MemMapFn)
  DRV(cuMemSetAccess, MemSetAccessFn)
  DRV(cuMemAddressFree, MemAddrFreeFn)
  CUdeviceptr va = 0;
  CUresult r = fn_cuMemAddressReserve(&va, size, align, 0, 0);
  if (r != CUDA_SUCCESS) return drv_fail(r, "cuMemAddressReserve");
  r = fn_cuMemMap(va, size, 0, h, 0);
  if (r != CUDA_SUCCESS) { fn_cuMemAddressFree(va, size); return drv_fail(r, "cuMemMap"); }
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = fn_cuMemSetAccess(va, size, &acc, 1);
  if (r != CUDA_SUCCESS) return drv_fail(r, "cuMemSetAccess");
  *va_out = (uint64_t)va;
  return 0;
}

}  // namespace

extern "C" {

// Granularity (bytes) every arena size must be a multiple of: the larger of the allocation and the multicast
// granularity for `n_devices` (0: allocation granularity only).
int etha_vmm_granularity(int n_devices, uint64_t* out) {
  DRV(cuMemGetAllocationGranularity, MemGranFn)
  int dev = 0;
  cudaGetDevice(&dev);
  cudaFree(0);  // make sure the primary context exists
  CUmemAllocationProp prop = device_prop(dev);
  size_t g = 0;
  CUresult r = fn_cuMemGetAllocationGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS) return drv_fail(r, "cuMemGetAllocationGranularity");
  if (n_devices > 1) {
    DRV(cuMulticastGetGranularity, McGranFn)
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = n_devices;
    mp.size = g;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    r = fn_cuMulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED);
    if (r != CUDA_SUCCESS) return drv_fail(r, "cuMulticastGetGranularity");
    if (mg > g) g = mg;
  }
  *out = g;
  return 0;
}

// Allocate `size` bytes (a multiple of the granularity) on the current device, map them read/write and export
// a POSIX file descriptor for other processes.
int etha_vmm_alloc(uint64_t size, uint64_t* handle, uint64_t* va, int* fd) {
  DRV(cuMemCreate, MemCreateFn)
  DRV(cuMemExportToShareableHandle, MemExportFn)
  DRV(cuMemRelease, MemReleaseFn)
  int dev = 0;
  cudaGetDevice(&dev);
  cudaFree(0);
  CUmemAllocationProp prop = device_prop(dev);
  CUmemGenericAllocationHandle h;
  CUresult r = fn_cuMemCreate(&h, size, &prop, 0);
  if (r != CUDA_SUCCESS) return drv_fail(r, "cuMemCreate");
  int rc = map_rw(h, size, 0, dev, va);
  if (rc != 0) { fn_cuMemRelease(h); return rc; }
  int out_fd = -1;
  r = fn_cuMemExportToShareableHandle(&out_fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) return drv_fail(r, "cuMemExportToShareableHandle");
  *handle = (uint64_t)h;
  *fd = out_fd;
  return 0;
}

// Map another process's allocation (received as a file descriptor) read/write on the current device.
int etha_vmm_import(int fd, uint64_t size, uint64_t* handle, uint64_t* va) {
  DRV(cuMemImportFromShareableHandle, MemImportFn)
  DRV(cuMemRelease, MemReleaseFn)
  int dev = 0;
  cudaGetDevice(&dev);
  cudaFree(0);
  CUmemGenericAllocationHandle h;
  CUresult r = fn_cuMemImportFromShareableHandle(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return drv_fail(r, "cuMemImportFromShareableHandle");
  int rc = map_rw(h, size, 0, dev, va);
  if (rc != 0) { fn_cuMemRelease(h); return rc; }
  *handle = (uint64_t)h;
  return 0;
}

int etha_vmm_unmap_release(uint64_t handle, uint64_t va, uint64_t size) {
  DRV(cuMemUnmap, MemUnmapFn)
  DRV(cuMemAddressFree, MemAddrFreeFn)
  DRV(cuMemRelease, MemReleaseFn)
  if (va) {
    fn_cuMemUnmap((CUdeviceptr)va, size);
    fn_cuMemAddressFree((CUdeviceptr)va, size);
  }
  if (handle) fn_cuMemRelease((CUmemGenericAllocationHandle)handle);
  return 0;
}

// ---- multicast -----------------------------------------------------------------------------------------
int etha_mc_create(int n_devices, uint64_t size, uint64_t* mc_handle, int* fd) {
  DRV(cuMulticastCreate, McCreateFn)
  DRV(cuMemExportToShareableHandle, MemExportFn)
  cudaFree(0);
  CUmulticastObjectProp mp;
  memset(&mp, 0, sizeof(mp));
  mp.numDevices = n_devices;
  mp.size = size;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle h;
  CUresult r = fn_cuMulticastCreate(&h, &mp);
  if (r != CUDA_SUCCESS) return drv_fail(r, "cuMulticastCreate");
  int out_fd = -1;
  r = fn_cuMemExportToShareableHandle(&out_fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) return drv_fail(r, "cuMemExportToShareableHandle(multicast)");
  *mc_handle = (uint64_t)h;
  *fd = out_fd;
  return 0;
}

int etha_mc_import(int fd, uint64_t* mc_handle) {
  DRV(cuMemImportFromShareableHandle, MemImportFn)
  cudaFree(0);
  CUmemGenericAllocationHandle h;
  CUresult r = fn_cuMemImportFromShareableHandle(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return drv_fail(r, "cuMemImportFromShareableHandle(multicast)");
  *mc_handle = (uint64_t)h;
  return 0;
}

// Every member calls this with its own device before anybody binds memory.
int etha_mc_add_device(uint64_t mc_handle) {
  DRV(cuMulticastAddDevice, McAddDevFn)
  int dev = 0;
  cudaGetDevice(&dev);
  CUresult r = fn_cuMulticastAddDevice((CUmemGenericAllocationHandle)mc_handle, (CUdevice)dev);
  return r == CUDA_SUCCESS ? 0 : drv_fail(r, "cuMulticastAddDevice");
}

// Bind `size` bytes of this device's allocation `mem_handle` at `offset` of the multicast object.
int etha_mc_bind(uint64_t mc_handle, uint64_t offset, uint64_t mem_handle, uint64_t mem_offset, uint64_t size) {
  DRV(cuMulticastBindMem, McBindFn)
  CUresult r = fn_cuMulticastBindMem((CUmemGenericAllocationHandle)mc_handle, offset, (CUmemGenericAllocationHandle)mem_handle,
                                     mem_offset, size, 0);
  return r == CUDA_SUCCESS ? 0 : drv_fail(r, "cuMulticastBindMem");
}

// Same, naming the memory by the address it is mapped at in this process instead of by its allocation handle:
// the form to use for an allocation this process imported from another one.
int etha_mc_bind_addr(uint64_t mc_handle, uint64_t offset, uint64_t va, uint64_t size) {
  DRV(cuMulticastBindAddr, McBindAddrFn)
  CUresult r = fn_cuMulticastBindAddr((CUmemGenericAllocationHandle)mc_handle, offset, (CUdeviceptr)va, size, 0);
  return r == CUDA_SUCCESS ? 0 : drv_fail(r, "cuMulticastBindAddr");
}

// Map the multicast object on the current device; stores to the returned address range must be multimem.st.
int etha_mc_map(uint64_t mc_handle, uint64_t size, uint64_t* va) {
  int dev = 0;
  cudaGetDevice(&dev);
  return map_rw((CUmemGenericAllocationHandle)mc_handle, size, 0, dev, va);
}

int etha_mc_unbind(uint64_t mc_handle, uint64_t offset, uint64_t size) {
  DRV(cuMulticastUnbind, McUnbindFn)
  int dev = 0;
  cudaGetDevice(&dev);
  CUresult r = fn_cuMulticastUnbind((CUmemGenericAllocationHandle)mc_handle, (CUdevice)dev, offset, size);
  return r == CUDA_SUCCESS ? 0 : drv_fail(r, "cuMulticastUnbind");
}

int etha_close_fd(int fd) { return close(fd); }

}  // extern "C"
