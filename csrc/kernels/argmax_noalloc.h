// Greedy argmax for callers that are not allowed to allocate device memory.
//
// This entry point has no counterpart in the reference engine.  It exists for hosts
// that embed the kernel library where cudaMalloc is off limits: a real-time serving
// loop that must not take the allocator's lock, a process whose memory was handed out
// up front by another runtime, or a sandbox that forbids allocation calls after start.
// The ordinary entry point, orinfer_argmax(), asks such a caller for two scratch
// buffers it cannot provide; this one keeps its scratch inside the library instead.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest problem the built-in scratch can hold.
#define ORINFER_ARGMAX_NOALLOC_MAX_ROWS 256
#define ORINFER_ARGMAX_NOALLOC_MAX_VOCAB 1048576

// token[r] = index of the largest value of logits[r, 0..vocab) (lowest index on ties,
// -1 when the row holds a non-finite value).  Same result as orinfer_argmax().
//
// * Allocates nothing: the partial results live in a 128 KiB array that is part of the
//   library image, so every GPU that loads the library carries those 128 KiB until the
//   process exits.
// * rows must be within 1..ORINFER_ARGMAX_NOALLOC_MAX_ROWS (0 is a no-op) and vocab
//   within 1..ORINFER_ARGMAX_NOALLOC_MAX_VOCAB; anything larger is refused with -1 and
//   nothing is launched.
// * The first call on each device looks up the device address of the array (with that
//   device current).  Make that first call before starting any stream capture.
// * All calls on a device share the one array.  Calls that can overlap on the GPU
//   (different streams with no ordering between them) race on it; serialise them.
//   Nothing in the array has to be cleared between calls: every slot that a call reads
//   was written earlier by the same call.
//
// Returns 0, -1 for a rejected size, or the cudaError_t of the set-up or launch.
int orinfer_argmax_noalloc(const float* logits, int rows, int vocab, int* token,
                           cudaStream_t stream);

#ifdef __cplusplus
}
#endif
