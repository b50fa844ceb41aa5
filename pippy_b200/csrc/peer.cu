// Peer (symmetric) memory: plain cudaMalloc allocations exported with CUDA IPC so that every rank of a node can map
// every other rank's buffer and kernels can load/store it directly over NVLink.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

extern "C" {

// Allocates `bytes` of zeroed device memory. Returns 0 on success.
int pb_peer_alloc(unsigned long long bytes, void** out) {
  cudaError_t e = cudaMalloc(out, bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(*out, 0, bytes);
  return (int)e;
}

int pb_peer_free(void* p) { return (int)cudaFree(p); }

// Writes the 64-byte IPC handle of allocation `p` to `handle_out`.
int pb_ipc_get_handle(void* p, void* handle_out) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}

int pb_ipc_open(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}

int pb_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }

int pb_ipc_handle_bytes() { return (int)sizeof(cudaIpcMemHandle_t); }

// Same-process "peers" (several devices driven by one process, used by tests): enable direct access.
int pb_enable_peer_access(int peer_device) {
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return 0;
  }
  return (int)e;
}

}  // extern "C"
