// Peer-mapped device buffers for the fused compute+collective kernels: each rank allocates a buffer, exports a CUDA
// IPC handle, and maps every peer's buffer into its own address space (plain peer loads/stores over NVLink; no
// multicast objects are bound, so a rank that exits does not disturb its peers' mappings).
// The reference keeps all GPUs in one process and uses cudaDeviceEnablePeerAccess + NCCL
// (cpp_runtime/backends/cuda/storage/load_options.cpp:259-283).
#include <cuda_runtime.h>
#include <string.h>

extern "C" int mfq_ipc_alloc(size_t bytes, void** ptr, unsigned char* handle64) {
  if (!ptr || !handle64 || bytes == 0) return -1;
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return -2;
  if (cudaMemset(p, 0, bytes) != cudaSuccess) return -3;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) { cudaFree(p); return -4; }
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  *ptr = p;
  return cudaDeviceSynchronize() == cudaSuccess ? 0 : -5;
}

extern "C" int mfq_ipc_open(const unsigned char* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? 0 : -1;
}

extern "C" int mfq_ipc_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? 0 : -1; }
extern "C" int mfq_ipc_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? 0 : -1; }
