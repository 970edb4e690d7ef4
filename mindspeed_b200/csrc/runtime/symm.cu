// Symmetric memory runtime: device buffers that every rank of a group can address.
//
// Each rank allocates the same-sized buffer with cudaMalloc (not from the framework's caching allocator, so that an
// IPC handle can be exported), the 64-byte handles are exchanged by the host over the process group, and every rank
// maps its peers' buffers (cudaIpcOpenMemHandle enables peer access lazily).  Kernels then receive a table of base
// pointers and read or write peers with ordinary loads, stores and non-multicast TMA.
#include "msb_common.cuh"

MSB_API int msb_symm_alloc(size_t bytes, void** out) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) { msb_set_error("symm_alloc(%zu): %s", bytes, cudaGetErrorString(e)); return 1; }
  e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) { msb_set_error("symm_alloc memset: %s", cudaGetErrorString(e)); cudaFree(p); return 1; }
  *out = p;
  return 0;
}
MSB_API int msb_symm_free(void* p) {
  cudaError_t e = cudaFree(p);
  if (e != cudaSuccess) { msb_set_error("symm_free: %s", cudaGetErrorString(e)); return 1; }
  return 0;
}
MSB_API int msb_symm_export(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) { msb_set_error("symm_export: %s", cudaGetErrorString(e)); return 1; }
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
MSB_API int msb_symm_import(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) { msb_set_error("symm_import: %s", cudaGetErrorString(e)); return 1; }
  *out = p;
  return 0;
}
MSB_API int msb_symm_close(void* p) {
  cudaError_t e = cudaIpcCloseMemHandle(p);
  if (e != cudaSuccess) { msb_set_error("symm_close: %s", cudaGetErrorString(e)); return 1; }
  return 0;
}
MSB_API int msb_ipc_handle_bytes() { return (int)sizeof(cudaIpcMemHandle_t); }
