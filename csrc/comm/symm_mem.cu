// Symmetric peer memory for one node: every rank allocates the same buffers with
// cudaMalloc, exports them as CUDA IPC handles and maps its peers' buffers, so
// kernels can load and store across NVLink / NVSwitch directly.  Handles travel
// over the existing process group (Python side).  No multicast object is bound
// to these buffers, so a rank that leaves cannot fault its peers' GPUs.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

extern "C" {

// Zero-filled device allocation outside PyTorch's caching allocator (IPC handles
// need whole cudaMalloc allocations).  Returns nullptr on failure.
void* ft_symm_alloc(size_t nbytes) {
  void* p = nullptr;
  if (cudaMalloc(&p, nbytes) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  if (cudaMemset(p, 0, nbytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    cudaGetLastError();
    cudaFree(p);
    return nullptr;
  }
  return p;   // zeroed before any peer can learn the address
}

int ft_symm_free(void* p) { return (int)cudaFree(p); }

int ft_ipc_handle_size() { return (int)sizeof(cudaIpcMemHandle_t); }

// Writes the 64-byte IPC handle of `ptr` (a pointer returned by ft_symm_alloc).
int ft_ipc_get_handle(void* ptr, void* out_handle) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return (int)e;
  memcpy(out_handle, &h, sizeof(h));
  return 0;
}

// Maps a peer's allocation into this process; returns the local address or nullptr.
void* ft_ipc_open(const void* handle) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return p;
}

int ft_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }

// 1 when device `dev` can address device `peer` directly.
int ft_can_access_peer(int dev, int peer) {
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, dev, peer) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return ok;
}

}  // extern "C"
