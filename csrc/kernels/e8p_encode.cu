// Exhaustive nearest-codeword search of the E8P lattice codebook: one thread per
// 8-vector scans the 256 basis rows for both parity shifts.  For a shift p the
// target is moved by -(1-2p); per basis row the best signs are the target's signs,
// but the flip mask must have even weight, so an odd mask pays for toggling its
// cheapest coordinate.  Same search as the reference's fused encoder
// (kernels/cuda/model/e8p_encode.py:61); used to quantise weights on the device.
#include "api.h"
#include "common.cuh"
#include "e8p_basis.h"

namespace orinfer {

struct EncodeTable {
  float mag[256][8];
  float norm[256];
  unsigned char negmask[256];     // bit d set when basis coordinate d is negative
};

__constant__ int c_coord_bit[8] = {0, 4, 1, 5, 2, 6, 3, 7};

__global__ void __launch_bounds__(128) e8p_encode_kernel(const float* __restrict__ x,
                                                         int* __restrict__ codes, long long vectors,
                                                         const EncodeTable* __restrict__ table) {
  __shared__ EncodeTable tab;
  {
    const float* src = reinterpret_cast<const float*>(table);
    float* dst = reinterpret_cast<float*>(&tab);
    for (int i = threadIdx.x; i < static_cast<int>(sizeof(EncodeTable) / 4); i += blockDim.x)
      dst[i] = src[i];
  }
  __syncthreads();
  const long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (v >= vectors) return;
  const float4 lo = *reinterpret_cast<const float4*>(x + v * 8);
  const float4 hi = *reinterpret_cast<const float4*>(x + v * 8 + 4);
  const float xs[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
  float best = INFINITY;
  int best_code = 0;
#pragma unroll 1
  for (int p = 0; p < 2; ++p) {
    const float shift = static_cast<float>(1 - 2 * p);
    float a[8];
    unsigned want = 0;
    float asq = 0.f;
#pragma unroll
    for (int d = 0; d < 8; ++d) {
      const float t = xs[d] - shift;
      if (t < 0.f) want |= 1u << d;
      a[d] = fabsf(t);
      asq += a[d] * a[d];
    }
    float pbest = INFINITY;
    int pidx = 0;
#pragma unroll 4
    for (int i = 0; i < 256; ++i) {
      float dot = 0.f;
#pragma unroll
      for (int d = 0; d < 8; ++d) dot += a[d] * tab.mag[i][d];
      float dist = asq - 2.f * dot + tab.norm[i];
      const unsigned flip = want ^ tab.negmask[i];
      if (__popc(flip) & 1) {
        float tmin = a[0] * tab.mag[i][0];
#pragma unroll
        for (int d = 1; d < 8; ++d) tmin = fminf(tmin, a[d] * tab.mag[i][d]);
        dist += 4.f * tmin;
      }
      if (dist < pbest) {
        pbest = dist;
        pidx = i;
      }
    }
    if (pbest < best) {
      unsigned flip = want ^ tab.negmask[pidx];
      if (__popc(flip) & 1) {
        int td = 0;
        float tmin = a[0] * tab.mag[pidx][0];
#pragma unroll
        for (int d = 1; d < 8; ++d) {
          const float c = a[d] * tab.mag[pidx][d];
          if (c < tmin) {
            tmin = c;
            td = d;
          }
        }
        flip ^= 1u << td;
      }
      unsigned low = 0;
#pragma unroll
      for (int d = 0; d < 8; ++d) low |= ((flip >> d) & 1u) << c_coord_bit[d];
      low ^= static_cast<unsigned>(p);
      best = pbest;
      best_code = (pidx << 8) | static_cast<int>(low);
    }
  }
  codes[v] = best_code;
}

namespace {
EncodeTable* g_encode_table = nullptr;
}

static cudaError_t ensure_encode_table() {
  if (g_encode_table) return cudaSuccess;
  int8_t basis[256][8];
  build_e8p_basis(basis);
  static EncodeTable host;
  for (int i = 0; i < 256; ++i) {
    float n = 0.f;
    unsigned char neg = 0;
    for (int d = 0; d < 8; ++d) {
      host.mag[i][d] = static_cast<float>(basis[i][d] < 0 ? -basis[i][d] : basis[i][d]);
      n += host.mag[i][d] * host.mag[i][d];
      if (basis[i][d] < 0) neg |= static_cast<unsigned char>(1u << d);
    }
    host.norm[i] = n;
    host.negmask[i] = neg;
  }
  cudaError_t e = cudaMalloc(&g_encode_table, sizeof(EncodeTable));
  if (e != cudaSuccess) return e;
  return cudaMemcpy(g_encode_table, &host, sizeof(EncodeTable), cudaMemcpyHostToDevice);
}

}  // namespace orinfer

extern "C" int orinfer_e8p_encode(const float* x, int* codes, long long vectors,
                                  cudaStream_t stream) {
  if (vectors <= 0) return 0;
  cudaError_t e = orinfer::ensure_encode_table();
  if (e != cudaSuccess) return static_cast<int>(e);
  const long long blocks = (vectors + 127) / 128;
  if (blocks > 2147483647LL) return -1;
  orinfer::e8p_encode_kernel<<<static_cast<unsigned>(blocks), 128, 0, stream>>>(
      x, codes, vectors, orinfer::g_encode_table);
  return static_cast<int>(cudaGetLastError());
}
