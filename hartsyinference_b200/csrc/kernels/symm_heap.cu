// Symmetric device heap: the same-sized allocation on every GPU of a group, mapped into every
// process of the group, so that a kernel on one GPU can store to / load from its peers over
// NVLink with plain pointers, plus (where the fabric supports it) ONE multicast mapping of all
// the ranks' allocations, through which `multimem` instructions reduce inside the NVSwitch or
// store to every rank at once. One process per GPU.
//
// Two transports for the handles:
//   * virtual memory management (preferred): cuMemCreate with a POSIX file-descriptor handle; the
//     descriptors travel between the processes as SCM_RIGHTS messages (Python side), peers import
//     and map them (cuMemMap); rank 0 creates the multicast object, every rank adds its device and
//     binds its own allocation at offset 0, then maps the multicast object like memory;
//   * CUDA IPC (fallback when descriptors cannot be exported): cudaMalloc + cudaIpcGetMemHandle,
//     no multicast mapping.
//
// The reference reaches peer memory only through cuMemcpyPeerAsync after cuCtxEnablePeerAccess
// (src/HartsyInference.Cuda/CudaPeerAccess.cs:23-42, CudaBackend.cs:10407-10483 CopyFromPeer) and
// probes the topology with cuDeviceCanAccessPeer / cuDeviceGetP2PAttribute
// (src/HartsyInference.Cuda/CudaTopology.cs:33-102); here peers are addressed from inside kernels.
#include "common.cuh"

#include <string.h>

using namespace b200;

// ---------------------------------------------------------------------------------------------
// CUDA IPC transport
// ---------------------------------------------------------------------------------------------
B200_API int b200_symm_alloc(void** out, long long bytes) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, static_cast<size_t>(bytes));
  if (e != cudaSuccess) return -static_cast<int>(e) - 100;
  e = cudaMemset(p, 0, static_cast<size_t>(bytes));
  if (e != cudaSuccess) return -static_cast<int>(e) - 200;
  e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return -static_cast<int>(e) - 300;
  *out = p;
  return 0;
}

B200_API int b200_symm_free(void* p) {
  return cudaFree(p) == cudaSuccess ? 0 : -1;
}

// handle_out: 64 bytes (cudaIpcMemHandle_t)
B200_API int b200_symm_export(void* p, void* handle_out) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return -static_cast<int>(e) - 100;
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}

B200_API int b200_symm_import(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return -static_cast<int>(e) - 100;
  *out = p;
  return 0;
}

B200_API int b200_symm_unmap(void* p) {
  return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : -1;
}

B200_API int b200_symm_memset(void* p, int value, long long bytes, cudaStream_t stream) {
  return cudaMemsetAsync(p, value, static_cast<size_t>(bytes), stream) == cudaSuccess ? 0 : -1;
}

// ---------------------------------------------------------------------------------------------
// Virtual-memory-management transport and the multicast mapping. Driver entry points are looked
// up at run time so that the library loads on machines without a driver.
// ---------------------------------------------------------------------------------------------
namespace {

template <typename Fn>
Fn driver_fn(const char* name) {
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint(name, &sym, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  return reinterpret_cast<Fn>(sym);
}

#define B200_DRV(name, ...)                                                              \
  typedef CUresult (*name##_t)(__VA_ARGS__);                                             \
  static name##_t p_##name() {                                                           \
    static name##_t f = driver_fn<name##_t>(#name);                                      \
    return f;                                                                            \
  }

B200_DRV(cuMemCreate, CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long)
B200_DRV(cuMemRelease, CUmemGenericAllocationHandle)
B200_DRV(cuMemGetAllocationGranularity, size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags)
B200_DRV(cuMemExportToShareableHandle, void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long)
B200_DRV(cuMemImportFromShareableHandle, CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType)
B200_DRV(cuMemAddressReserve, CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long)
B200_DRV(cuMemAddressFree, CUdeviceptr, size_t)
B200_DRV(cuMemMap, CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long)
B200_DRV(cuMemUnmap, CUdeviceptr, size_t)
B200_DRV(cuMemSetAccess, CUdeviceptr, size_t, const CUmemAccessDesc*, size_t)
B200_DRV(cuMulticastCreate, CUmemGenericAllocationHandle*, const CUmulticastObjectProp*)
B200_DRV(cuMulticastAddDevice, CUmemGenericAllocationHandle, CUdevice)
B200_DRV(cuMulticastBindMem, CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long)
B200_DRV(cuMulticastUnbind, CUmemGenericAllocationHandle, CUdevice, size_t, size_t)
B200_DRV(cuMulticastGetGranularity, size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags)
B200_DRV(cuDeviceGetAttribute, int*, CUdevice_attribute, CUdevice)

int rc_of(CUresult r, int base) { return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r) - base; }

CUmemAllocationProp device_prop(int dev) {
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = dev;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

}  // namespace

// Capabilities of the current device: bit 0 = allocations exportable as file descriptors,
// bit 1 = multicast objects (NVLS) supported. Negative on error.
B200_API int b200_vmm_caps() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (cudaFree(nullptr) != cudaSuccess) return -1;   // make sure the primary context exists
  if (!p_cuDeviceGetAttribute() || !p_cuMemCreate() || !p_cuMemMap()) return 0;
  int vmm = 0, fd = 0, mc = 0;
  p_cuDeviceGetAttribute()(&vmm, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, dev);
  p_cuDeviceGetAttribute()(&fd, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev);
  if (p_cuMulticastCreate()) p_cuDeviceGetAttribute()(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev);
  return ((vmm && fd) ? 1 : 0) | ((vmm && fd && mc) ? 2 : 0);
}

// Size that a heap of `bytes` is rounded up to so that it can be mapped (and bound to a multicast
// object of `ndev` devices when ndev > 1).
B200_API long long b200_vmm_round_size(long long bytes, int ndev) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || !p_cuMemGetAllocationGranularity()) return -1;
  CUmemAllocationProp prop = device_prop(dev);
  size_t gran = 0;
  if (p_cuMemGetAllocationGranularity()(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS) return -2;
  if (ndev > 1 && p_cuMulticastGetGranularity()) {
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = static_cast<unsigned>(ndev);
    mp.size = static_cast<size_t>(bytes);
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (p_cuMulticastGetGranularity()(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > gran)
      gran = mg;
  }
  if (gran == 0) return -3;
  return static_cast<long long>((static_cast<size_t>(bytes) + gran - 1) / gran * gran);
}

// Physical allocation on the current device (size from b200_vmm_round_size) + its descriptor.
B200_API int b200_vmm_create(long long size, unsigned long long* handle_out, int* fd_out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  CUmemAllocationProp prop = device_prop(dev);
  CUmemGenericAllocationHandle h = 0;
  CUresult r = p_cuMemCreate()(&h, static_cast<size_t>(size), &prop, 0);
  if (r != CUDA_SUCCESS) return rc_of(r, 100);
  int fd = -1;
  r = p_cuMemExportToShareableHandle()(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    p_cuMemRelease()(h);
    return rc_of(r, 200);
  }
  *handle_out = static_cast<unsigned long long>(h);
  *fd_out = fd;
  return 0;
}

// Descriptor received from a peer (a memory allocation or a multicast object) -> handle.
B200_API int b200_vmm_import(int fd, unsigned long long* handle_out) {
  CUmemGenericAllocationHandle h = 0;
  CUresult r = p_cuMemImportFromShareableHandle()(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                  CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return rc_of(r, 100);
  *handle_out = static_cast<unsigned long long>(h);
  return 0;
}

// Maps a handle (memory or multicast object) read-write into the current device's address space.
B200_API int b200_vmm_map(unsigned long long handle, long long size, void** va_out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  CUdeviceptr va = 0;
  CUresult r = p_cuMemAddressReserve()(&va, static_cast<size_t>(size), 0, 0, 0);
  if (r != CUDA_SUCCESS) return rc_of(r, 100);
  r = p_cuMemMap()(va, static_cast<size_t>(size), 0, static_cast<CUmemGenericAllocationHandle>(handle), 0);
  if (r != CUDA_SUCCESS) {
    p_cuMemAddressFree()(va, static_cast<size_t>(size));
    return rc_of(r, 200);
  }
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = p_cuMemSetAccess()(va, static_cast<size_t>(size), &acc, 1);
  if (r != CUDA_SUCCESS) {
    p_cuMemUnmap()(va, static_cast<size_t>(size));
    p_cuMemAddressFree()(va, static_cast<size_t>(size));
    return rc_of(r, 300);
  }
  *va_out = reinterpret_cast<void*>(va);
  return 0;
}

B200_API int b200_vmm_unmap(void* va, long long size) {
  CUresult r = p_cuMemUnmap()(reinterpret_cast<CUdeviceptr>(va), static_cast<size_t>(size));
  if (r != CUDA_SUCCESS) return rc_of(r, 100);
  return rc_of(p_cuMemAddressFree()(reinterpret_cast<CUdeviceptr>(va), static_cast<size_t>(size)), 200);
}

B200_API int b200_vmm_release(unsigned long long handle) {
  return rc_of(p_cuMemRelease()(static_cast<CUmemGenericAllocationHandle>(handle)), 100);
}

// Multicast object for `ndev` devices and `size` bytes (created by one rank) + its descriptor.
B200_API int b200_mc_create(int ndev, long long size, unsigned long long* handle_out, int* fd_out) {
  if (!p_cuMulticastCreate()) return -1;
  CUmulticastObjectProp mp;
  memset(&mp, 0, sizeof(mp));
  mp.numDevices = static_cast<unsigned>(ndev);
  mp.size = static_cast<size_t>(size);
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle h = 0;
  CUresult r = p_cuMulticastCreate()(&h, &mp);
  if (r != CUDA_SUCCESS) return rc_of(r, 100);
  int fd = -1;
  r = p_cuMemExportToShareableHandle()(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    p_cuMemRelease()(h);
    return rc_of(r, 200);
  }
  *handle_out = static_cast<unsigned long long>(h);
  *fd_out = fd;
  return 0;
}

// Every rank: add the current device to the object. All devices must be added before any binds.
B200_API int b200_mc_add_device(unsigned long long mc) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  return rc_of(p_cuMulticastAddDevice()(static_cast<CUmemGenericAllocationHandle>(mc), dev), 100);
}

// Every rank: bind its own allocation at offset 0 of the object.
B200_API int b200_mc_bind(unsigned long long mc, unsigned long long mem, long long size) {
  return rc_of(p_cuMulticastBindMem()(static_cast<CUmemGenericAllocationHandle>(mc), 0,
                                      static_cast<CUmemGenericAllocationHandle>(mem), 0,
                                      static_cast<size_t>(size), 0), 100);
}

// Every rank, before it frees its allocation or exits: take its memory out of the object.
B200_API int b200_mc_unbind(unsigned long long mc, long long size) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  return rc_of(p_cuMulticastUnbind()(static_cast<CUmemGenericAllocationHandle>(mc), dev, 0,
                                     static_cast<size_t>(size)), 100);
}

// Topology probe of the visible devices: out[i * n + j] = 1 when device i can address device j's
// memory, +2 when native atomics over the link are supported (NVLink), -1 on error.
B200_API int b200_topology_probe(int* out, int cap) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) return -1;
  if (n * n > cap) return -2;
  for (int i = 0; i < n; ++i)
    for (int j = 0; j < n; ++j) {
      int v = 0;
      if (i == j) {
        v = 3;
      } else {
        int can = 0, atom = 0;
        if (cudaDeviceCanAccessPeer(&can, i, j) != cudaSuccess) can = 0;
        if (can) cudaDeviceGetP2PAttribute(&atom, cudaDevP2PAttrNativeAtomicSupported, i, j);
        v = (can ? 1 : 0) + (atom ? 2 : 0);
      }
      out[i * n + j] = v;
    }
  return n;
}
