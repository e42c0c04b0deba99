// Static-scratch variant of the greedy argmax: see argmax_noalloc.h for who needs it.
#include <mutex>

#include "api.h"
#include "argmax_kernels.cuh"
#include "argmax_noalloc.h"

namespace {

constexpr int kMaxRows = ORINFER_ARGMAX_NOALLOC_MAX_ROWS;
constexpr int kMaxParts = 64;                      // orinfer_argmax_parts() never exceeds this
constexpr int kMaxDevices = 64;

// rows x parts partial maxima followed by rows x parts partial indices (128 KiB).  In host
// code this name is only a handle for cudaGetSymbolAddress, never a pointer to pass on.
static __device__ __align__(256) unsigned char g_argmax_scratch[kMaxRows * kMaxParts * 8];

struct PerDevice {
  bool ready = false;
  float* values = nullptr;
  int* indices = nullptr;
};

std::mutex g_lock;
PerDevice g_devices[kMaxDevices];

// Resolves the scratch address once per device, with that device current.
cudaError_t scratch_for_current_device(PerDevice** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> guard(g_lock);
  PerDevice& slot = g_devices[dev];
  if (!slot.ready) {
    void* base = nullptr;
    e = cudaGetSymbolAddress(&base, g_argmax_scratch);
    if (e != cudaSuccess) return e;
    slot.values = static_cast<float*>(base);
    slot.indices = reinterpret_cast<int*>(static_cast<unsigned char*>(base) +
                                          static_cast<size_t>(kMaxRows) * kMaxParts * 4);
    slot.ready = true;
  }
  *out = &slot;
  return cudaSuccess;
}

}  // namespace

extern "C" int orinfer_argmax_noalloc(const float* logits, int rows, int vocab, int* token,
                                      cudaStream_t stream) {
  if (rows == 0) return 0;
  if (rows < 0 || rows > kMaxRows || vocab <= 0 || vocab > ORINFER_ARGMAX_NOALLOC_MAX_VOCAB ||
      logits == nullptr || token == nullptr)
    return -1;
  const int parts = orinfer_argmax_parts(vocab);
  if (parts > kMaxParts) return -1;
  PerDevice* dev = nullptr;
  cudaError_t e = scratch_for_current_device(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  orinfer::argmax_partial_kernel<<<dim3(parts, rows), 256, 0, stream>>>(logits, vocab, parts,
                                                                      dev->values, dev->indices);
  orinfer::argmax_merge_kernel<<<rows, 32, 0, stream>>>(dev->values, dev->indices, parts, token);
  return static_cast<int>(cudaGetLastError());
}
