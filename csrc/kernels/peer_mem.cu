// Peer-mapped device buffers for the fused tensor-parallel kernels, one process per GPU on
// one node.  A rank allocates its inbox with cudaMalloc, publishes the 64-byte CUDA IPC
// handle through the job's out-of-band channel (torch.distributed object gather), and maps
// every peer's buffer with cudaIpcOpenMemHandle.  Kernels then reach peers with plain
// loads/stores over NVLink.  This is the build's own symmetric-memory layer; it plays the
// role the HCCL communicator bootstrap plays in the reference
// (crates/orinfer-engine/src/backend/ascend/hccl.rs:97-156 RootInfo exchange).
#include <cuda_runtime.h>
#include <string.h>

#include "api.h"

extern "C" {

// Allocates `bytes` of zeroed device memory on the current device; returns the pointer
// (nullptr on failure).
void* orinfer_peer_alloc(size_t bytes) {
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return nullptr;
  if (cudaMemset(p, 0, bytes) != cudaSuccess) {
    cudaFree(p);
    return nullptr;
  }
  cudaDeviceSynchronize();
  return p;
}

int orinfer_peer_free(void* p) { return static_cast<int>(cudaFree(p)); }

// Writes the 64-byte IPC handle of an orinfer_peer_alloc buffer.
int orinfer_peer_export(void* p, unsigned char* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return static_cast<int>(e);
  static_assert(sizeof(h) == 64, "CUDA IPC handles are 64 bytes");
  memcpy(handle64, &h, 64);
  return 0;
}

// Maps a peer's buffer into this process; *out receives the device pointer.
int orinfer_peer_import(const unsigned char* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return static_cast<int>(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
}

int orinfer_peer_unmap(void* p) { return static_cast<int>(cudaIpcCloseMemHandle(p)); }

// Plain copy between (possibly peer-mapped) device buffers, for self-tests.
int orinfer_peer_copy(void* dst, const void* src, size_t bytes) {
  cudaError_t e = cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToDevice);
  return static_cast<int>(e);
}

}  // extern "C"
