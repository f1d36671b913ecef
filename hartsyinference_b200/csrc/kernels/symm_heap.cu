// Symmetric device heap: the same-sized allocation on every GPU of a group, mapped into every
// process of the group, so that a kernel on one GPU can store to / load from its peers over
// NVLink with plain pointers. One process per GPU; the handles travel over the group's control
// plane (torch.distributed) and are opened with CUDA IPC.
//
// The reference reaches peer memory only through cuMemcpyPeerAsync after cuCtxEnablePeerAccess
// (src/HartsyInference.Cuda/CudaPeerAccess.cs:23-42, CudaBackend.cs:10407-10483 CopyFromPeer) and
// probes the topology with cuDeviceCanAccessPeer / cuDeviceGetP2PAttribute
// (src/HartsyInference.Cuda/CudaTopology.cs:33-102); here peers are addressed from inside kernels.
#include "common.cuh"

using namespace b200;

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
