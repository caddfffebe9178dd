// Symmetric heap on the virtual-memory-management API, with an NVLink multicast (NVLS) view.
//
// Why not cudaMalloc + CUDA IPC alone: memory that is to be bound to a multicast object - so that one
// multimem.ld_reduce fetches the sum of all ranks' copies from the NVSwitch and one multimem.st writes all
// copies - has to come from cuMemCreate.  Every rank therefore creates its region as a physical allocation,
// shares it as a POSIX file descriptor (the Python side passes descriptors between rank processes over a
// Unix-domain socket; ranks that live in one process simply share the handle), maps all ranks' regions for
// plain peer loads / stores, and binds its own region into one multicast object that all ranks map as well:
//
//     base[r]   unicast mapping of rank r's region      (ld / st / red, as before)
//     mc_base   multicast mapping over all regions       (multimem.ld_reduce / multimem.st / multimem.red)
//
// Both views use the same offsets.  Every entry point returns a TPB_* code; none of them launches a kernel.
// The driver API is reached through cudaGetDriverEntryPoint, so the library keeps loading on a machine
// without a driver.  Teardown order matters on NVSwitch systems: unmap the multicast view and unbind before
// the memory is released, and do it on every rank before any rank exits.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "tpb_api.h"

namespace {

template <typename Fn>
Fn driver_fn(const char* name) {
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &ptr, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return nullptr;
  return reinterpret_cast<Fn>(ptr);
}

#define TPB_DRIVER(name, ...)                                         \
  typedef CUresult (*name##_t)(__VA_ARGS__);                          \
  static name##_t name##_p() {                                        \
    static name##_t fn = driver_fn<name##_t>(#name);                  \
    return fn;                                                        \
  }

TPB_DRIVER(cuMemCreate, CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long)
TPB_DRIVER(cuMemRelease, CUmemGenericAllocationHandle)
TPB_DRIVER(cuMemGetAllocationGranularity, size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags)
TPB_DRIVER(cuMemExportToShareableHandle, void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long)
TPB_DRIVER(cuMemImportFromShareableHandle, CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType)
TPB_DRIVER(cuMemAddressReserve, CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long)
TPB_DRIVER(cuMemAddressFree, CUdeviceptr, size_t)
TPB_DRIVER(cuMemMap, CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long)
TPB_DRIVER(cuMemUnmap, CUdeviceptr, size_t)
TPB_DRIVER(cuMemSetAccess, CUdeviceptr, size_t, const CUmemAccessDesc*, size_t)
TPB_DRIVER(cuMulticastCreate, CUmemGenericAllocationHandle*, const CUmulticastObjectProp*)
TPB_DRIVER(cuMulticastAddDevice, CUmemGenericAllocationHandle, CUdevice)
TPB_DRIVER(cuMulticastBindMem, CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long)
TPB_DRIVER(cuMulticastUnbind, CUmemGenericAllocationHandle, CUdevice, size_t, size_t)
TPB_DRIVER(cuMulticastGetGranularity, size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags)
TPB_DRIVER(cuDeviceGet, CUdevice*, int)
TPB_DRIVER(cuDeviceGetAttribute, int*, CUdevice_attribute, CUdevice)

CUmemAllocationProp region_prop(int device) {
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

CUmulticastObjectProp multicast_prop(int n_devices, size_t bytes) {
  CUmulticastObjectProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.numDevices = static_cast<unsigned>(n_devices);
  prop.size = bytes;
  prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

}  // namespace

// *vmm = 1 if `device` supports cuMemCreate with POSIX file descriptor handles, *multicast = 1 if it supports
// multicast objects.  Both 0 (and TPB_OK) when the driver is absent.
extern "C" int tpb_symm_support(int device, int* vmm, int* multicast) {
  if (!vmm || !multicast) return TPB_ERR_ARG;
  *vmm = *multicast = 0;
  if (!cuDeviceGet_p() || !cuDeviceGetAttribute_p() || !cuMemCreate_p()) return TPB_OK;
  cudaFree(0);  // make sure a context exists
  CUdevice dev;
  if (cuDeviceGet_p()(&dev, device) != CUDA_SUCCESS) return TPB_ERR_DRIVER;
  int v = 0, fd = 0, mc = 0;
  cuDeviceGetAttribute_p()(&v, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, dev);
  cuDeviceGetAttribute_p()(&fd, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev);
  cuDeviceGetAttribute_p()(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev);
  *vmm = (v && fd) ? 1 : 0;
  *multicast = (*vmm && mc && cuMulticastCreate_p()) ? 1 : 0;
  return TPB_OK;
}

// Size that a region of at least `bytes` must have: a multiple of the allocation granularity and (n_devices > 1) of the
// multicast granularity of an object over n_devices devices.
extern "C" int tpb_symm_round_size(int device, int n_devices, size_t bytes, size_t* rounded) {
  if (!rounded || !cuMemGetAllocationGranularity_p()) return TPB_ERR_DRIVER;
  CUmemAllocationProp prop = region_prop(device);
  size_t gran = 0;
  if (cuMemGetAllocationGranularity_p()(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || !gran) return TPB_ERR_DRIVER;
  if (n_devices > 1 && cuMulticastGetGranularity_p()) {
    CUmulticastObjectProp mp = multicast_prop(n_devices, bytes);
    size_t mg = 0;
    if (cuMulticastGetGranularity_p()(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > gran) gran = mg;
  }
  *rounded = (bytes + gran - 1) / gran * gran;
  return TPB_OK;
}

// Physical allocation of `bytes` (already rounded) on `device`.  *fd receives a POSIX descriptor of it when fd is not null
// (the caller closes it after the peers have imported it).
extern "C" int tpb_symm_create(int device, size_t bytes, unsigned long long* handle, int* fd) {
  if (!handle || !cuMemCreate_p()) return TPB_ERR_DRIVER;
  CUmemAllocationProp prop = region_prop(device);
  CUmemGenericAllocationHandle h;
  if (cuMemCreate_p()(&h, bytes, &prop, 0) != CUDA_SUCCESS) return TPB_ERR_DRIVER;
  if (fd) {
    int out = -1;
    if (cuMemExportToShareableHandle_p()(&out, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS) {
      cuMemRelease_p()(h);
      return TPB_ERR_DRIVER;
    }
    *fd = out;
  }
  *handle = static_cast<unsigned long long>(h);
  return TPB_OK;
}

// Handle of an allocation (or multicast object) that another process exported as descriptor `fd`.
extern "C" int tpb_symm_import(int fd, unsigned long long* handle) {
  if (!handle || !cuMemImportFromShareableHandle_p()) return TPB_ERR_DRIVER;
  CUmemGenericAllocationHandle h;
  if (cuMemImportFromShareableHandle_p()(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) !=
      CUDA_SUCCESS)
    return TPB_ERR_DRIVER;
  *handle = static_cast<unsigned long long>(h);
  return TPB_OK;
}

// Maps `handle` (an allocation or a multicast object) at a fresh virtual address with read / write access for the listed
// devices.
extern "C" int tpb_symm_map(unsigned long long handle, size_t bytes, const int* devices, int n_devices, void** ptr) {
  if (!ptr || !devices || n_devices < 1 || n_devices > 64 || !cuMemAddressReserve_p()) return TPB_ERR_DRIVER;
  CUdeviceptr va = 0;
  if (cuMemAddressReserve_p()(&va, bytes, 0, 0, 0) != CUDA_SUCCESS) return TPB_ERR_DRIVER;
  if (cuMemMap_p()(va, bytes, 0, static_cast<CUmemGenericAllocationHandle>(handle), 0) != CUDA_SUCCESS) {
    cuMemAddressFree_p()(va, bytes);
    return TPB_ERR_DRIVER;
  }
  CUmemAccessDesc access[64];
  for (int i = 0; i < n_devices; ++i) {
    access[i].location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access[i].location.id = devices[i];
    access[i].flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  }
  if (cuMemSetAccess_p()(va, bytes, access, static_cast<size_t>(n_devices)) != CUDA_SUCCESS) {
    cuMemUnmap_p()(va, bytes);
    cuMemAddressFree_p()(va, bytes);
    return TPB_ERR_DRIVER;
  }
  *ptr = reinterpret_cast<void*>(va);
  return TPB_OK;
}

extern "C" int tpb_symm_unmap(void* ptr, size_t bytes) {
  if (!ptr || !cuMemUnmap_p()) return TPB_ERR_DRIVER;
  const CUdeviceptr va = reinterpret_cast<CUdeviceptr>(ptr);
  CUresult r = cuMemUnmap_p()(va, bytes);
  cuMemAddressFree_p()(va, bytes);
  return r == CUDA_SUCCESS ? TPB_OK : TPB_ERR_DRIVER;
}

extern "C" int tpb_symm_release(unsigned long long handle) {
  if (!cuMemRelease_p()) return TPB_ERR_DRIVER;
  return cuMemRelease_p()(static_cast<CUmemGenericAllocationHandle>(handle)) == CUDA_SUCCESS ? TPB_OK : TPB_ERR_DRIVER;
}

// Multicast object over n_devices devices covering `bytes`; *fd as in tpb_symm_create.
extern "C" int tpb_mc_create(int n_devices, size_t bytes, unsigned long long* handle, int* fd) {
  if (!handle || !cuMulticastCreate_p()) return TPB_ERR_DRIVER;
  CUmulticastObjectProp prop = multicast_prop(n_devices, bytes);
  CUmemGenericAllocationHandle h;
  if (cuMulticastCreate_p()(&h, &prop) != CUDA_SUCCESS) return TPB_ERR_DRIVER;
  if (fd) {
    int out = -1;
    if (cuMemExportToShareableHandle_p()(&out, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS) {
      cuMemRelease_p()(h);
      return TPB_ERR_DRIVER;
    }
    *fd = out;
  }
  *handle = static_cast<unsigned long long>(h);
  return TPB_OK;
}

// Every participating device is added before any memory is bound.
extern "C" int tpb_mc_add_device(unsigned long long mc, int device) {
  if (!cuMulticastAddDevice_p()) return TPB_ERR_DRIVER;
  CUdevice dev;
  if (cuDeviceGet_p()(&dev, device) != CUDA_SUCCESS) return TPB_ERR_DRIVER;
  return cuMulticastAddDevice_p()(static_cast<CUmemGenericAllocationHandle>(mc), dev) == CUDA_SUCCESS ? TPB_OK : TPB_ERR_DRIVER;
}

// Binds the whole allocation `mem` (on a device that was added) at offset 0 of the multicast object.
extern "C" int tpb_mc_bind(unsigned long long mc, unsigned long long mem, size_t bytes) {
  if (!cuMulticastBindMem_p()) return TPB_ERR_DRIVER;
  return cuMulticastBindMem_p()(static_cast<CUmemGenericAllocationHandle>(mc), 0, static_cast<CUmemGenericAllocationHandle>(mem), 0, bytes, 0) ==
                 CUDA_SUCCESS
             ? TPB_OK
             : TPB_ERR_DRIVER;
}

extern "C" int tpb_mc_unbind(unsigned long long mc, int device, size_t bytes) {
  if (!cuMulticastUnbind_p()) return TPB_ERR_DRIVER;
  CUdevice dev;
  if (cuDeviceGet_p()(&dev, device) != CUDA_SUCCESS) return TPB_ERR_DRIVER;
  return cuMulticastUnbind_p()(static_cast<CUmemGenericAllocationHandle>(mc), dev, 0, bytes) == CUDA_SUCCESS ? TPB_OK : TPB_ERR_DRIVER;
}
