// Greedy argmax kernels shared by the allocating-caller entry point (elementwise.cu)
// and the static-scratch entry point (argmax_noalloc.cu).  `static` gives each
// translation unit its own copy, so no relocatable device code is needed.
#pragma once

#include "common.cuh"

namespace orinfer {

// ------------------------------------------------------------------ argmax
// Pass 1: each block scans a slice of one row; pass 2 merges the partials.  Ties go
// to the lowest index; a non-finite maximum marks the row invalid (token -1).
static __global__ void argmax_partial_kernel(const float* __restrict__ logits, int vocab, int parts,
                                      float* __restrict__ pval, int* __restrict__ pidx) {
  const int row = blockIdx.y, part = blockIdx.x;
  const int chunk = (vocab + parts - 1) / parts;
  const int lo = part * chunk, hi = min(vocab, lo + chunk);
  const float* r = logits + static_cast<size_t>(row) * vocab;
  float best = -INFINITY;
  int bidx = 0x7fffffff;
  bool bad = false;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = r[i];
    if (!(fabsf(v) <= 3.4e38f)) bad = true;
    if (v > best) { best = v; bidx = i; }
  }
  __shared__ float sv[256];
  __shared__ int si[256];
  __shared__ int sbad;
  if (threadIdx.x == 0) sbad = 0;
  __syncthreads();
  if (bad) sbad = 1;
  sv[threadIdx.x] = best;
  si[threadIdx.x] = bidx;
  __syncthreads();
  for (int s = blockDim.x / 2; s > 0; s >>= 1) {
    if (threadIdx.x < s) {
      const float ov = sv[threadIdx.x + s];
      const int oi = si[threadIdx.x + s];
      if (ov > sv[threadIdx.x] || (ov == sv[threadIdx.x] && oi < si[threadIdx.x])) {
        sv[threadIdx.x] = ov;
        si[threadIdx.x] = oi;
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    pval[row * parts + part] = sbad ? NAN : sv[0];
    pidx[row * parts + part] = si[0];
  }
}

static __global__ void argmax_merge_kernel(const float* __restrict__ pval, const int* __restrict__ pidx,
                                    int parts, int* __restrict__ token) {
  const int row = blockIdx.x;
  if (threadIdx.x != 0) return;
  float best = -INFINITY;
  int bidx = 0x7fffffff;
  bool bad = false;
  for (int p = 0; p < parts; ++p) {
    const float v = pval[row * parts + p];
    const int i = pidx[row * parts + p];
    if (v != v) bad = true;
    if (v > best || (v == best && i < bidx)) { best = v; bidx = i; }
  }
  token[row] = bad ? -1 : bidx;
}

}  // namespace orinfer
