// Device top-k / top-p categorical sampler for rows whose options need no host state
// (temperature > 0, 1 <= top_k <= 64, no penalties, bias, mask or probability report).
// One CTA per row:
//   1. exact radix select (4 passes of 8-bit histograms over order-preserving keys) of the
//      top_k-th largest logit;
//   2. shortlist of every entry above the threshold plus the lowest-id ties at it;
//   3. rank sort by (logit descending, id ascending) - the host law's order;
//   4. one thread walks the host law in FP64: weights exp((s - max)/T), nucleus cut at
//      total * top_p, renormalise, draw with the caller's counter-RNG uniform.
// The uniform comes from the host (counter_uniform(seed, 0, step)), so a request samples the
// same stream whether a step runs here or through the host law.  A row the kernel cannot
// serve exactly (more ties at the threshold than the shortlist holds, non-finite logits)
// sets flag[row] = 1 and the host law takes that row.
// Replaces sampling.{scores,radix_histogram,radix_choose,shortlist_collect,shortlist_sample}
// (kernels/cuda/model/sampling.py:67-170,396-516 of the reference).
#include "api.h"
#include "common.cuh"

namespace orinfer {

constexpr int SAMPLE_THREADS = 1024;
constexpr int MAX_TOPK = 64;
constexpr int TIE_CAP = 256;

__device__ __forceinline__ uint32_t order_key(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_topk_kernel(
    const float* __restrict__ logits, int vocab, long long row_stride,
    const int* __restrict__ top_k, const double* __restrict__ temperature,
    const double* __restrict__ top_p, const double* __restrict__ uniform,
    int* __restrict__ token, int* __restrict__ flag) {
  const int row = blockIdx.x, tid = threadIdx.x;
  const float* lg = logits + static_cast<long long>(row) * row_stride;
  __shared__ unsigned int hist[256];
  __shared__ uint32_t s_prefix, s_mask;
  __shared__ int s_need, s_bad;
  __shared__ int n_above, n_tie;
  __shared__ float sl_val[MAX_TOPK];
  __shared__ int sl_id[MAX_TOPK];
  __shared__ int tie_id[TIE_CAP];
  __shared__ float so_val[MAX_TOPK];
  __shared__ int so_id[MAX_TOPK];
  const int k = min(max(top_k[row], 1), min(MAX_TOPK, vocab));
  if (tid == 0) {
    s_prefix = 0;
    s_mask = 0;
    s_need = k;
    s_bad = 0;
    n_above = 0;
    n_tie = 0;
  }
  __syncthreads();
  // ---- 1. radix select of the k-th largest key
  for (int pass = 3; pass >= 0; --pass) {
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix, mask = s_mask;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
      const float v = lg[i];
      if (pass == 3 && !isfinite(v)) s_bad = 1;
      const uint32_t key = order_key(v);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> (8 * pass)) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      int need = s_need, d = 255;
      for (; d > 0; --d) {
        const int c = static_cast<int>(hist[d]);
        if (c >= need) break;
        need -= c;
      }
      s_need = need;                                   // still needed inside digit d
      s_prefix = prefix | (static_cast<uint32_t>(d) << (8 * pass));
      s_mask = mask | (0xffu << (8 * pass));
    }
    __syncthreads();
  }
  const uint32_t thresh = s_prefix;                    // key of the k-th largest logit
  const int need_ties = s_need;                        // how many entries equal to it belong
  // ---- 2. shortlist
  for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
    const float v = lg[i];
    const uint32_t key = order_key(v);
    if (key > thresh) {
      const int slot = atomicAdd(&n_above, 1);
      if (slot < MAX_TOPK) {
        sl_val[slot] = v;
        sl_id[slot] = i;
      }
    } else if (key == thresh) {
      const int slot = atomicAdd(&n_tie, 1);
      if (slot < TIE_CAP) tie_id[slot] = i;
    }
  }
  __syncthreads();
  const int above = n_above, ties = n_tie;
  if (s_bad || above + need_ties != k || ties > TIE_CAP) {
    if (tid == 0) {
      flag[row] = 1;
      token[row] = -1;
    }
    return;
  }
  // the lowest-id ties complete the shortlist (rank by id among the ties)
  if (tid < ties) {
    const int id = tie_id[tid];
    int rank = 0;
    for (int j = 0; j < ties; ++j) rank += tie_id[j] < id;
    if (rank < need_ties) {
      sl_val[above + rank] = lg[id];
      sl_id[above + rank] = id;
    }
  }
  __syncthreads();
  // ---- 3. rank sort: logit descending, id ascending
  if (tid < k) {
    const float v = sl_val[tid];
    const int id = sl_id[tid];
    int rank = 0;
    for (int j = 0; j < k; ++j) rank += (sl_val[j] > v) || (sl_val[j] == v && sl_id[j] < id);
    so_val[rank] = v;
    so_id[rank] = id;
  }
  __syncthreads();
  // ---- 4. the law, in the host's order of operations
  if (tid == 0) {
    const double t = temperature[row], mx = static_cast<double>(so_val[0]);
    double w[MAX_TOPK];
    double total = 0.0;
    for (int i = 0; i < k; ++i) {
      w[i] = exp((static_cast<double>(so_val[i]) - mx) / t);
      total += w[i];
    }
    const double threshold = total * top_p[row];
    double mass = 0.0;
    int keep = k;
    for (int i = 0; i < k; ++i) {
      mass += w[i];
      if (mass >= threshold) {
        keep = i + 1;
        break;
      }
    }
    const double u = uniform[row];
    double acc = 0.0;
    int chosen = -1;
    for (int i = 0; i < keep; ++i) {
      acc += w[i] / mass;
      if (u < acc) {
        chosen = so_id[i];
        break;
      }
    }
    if (chosen < 0) {
      for (int i = keep - 1; i >= 0; --i)
        if (w[i] / mass > 0.0) {
          chosen = so_id[i];
          break;
        }
    }
    token[row] = chosen;
    flag[row] = chosen < 0 ? 1 : 0;
  }
}

}  // namespace orinfer

using namespace orinfer;

extern "C" {

// logits fp32 [rows, row_stride >= vocab]; per-row top_k (1..64), temperature (> 0), top_p
// (0..1], uniform [0,1).  token[row] receives the draw, flag[row] = 1 when the host law must
// serve the row instead.
int orinfer_sample_topk(const float* logits, int rows, int vocab, long long row_stride,
                        const int* top_k, const double* temperature, const double* top_p,
                        const double* uniform, int* token, int* flag, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || row_stride < vocab) return -1;
  sample_topk_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(logits, vocab, row_stride, top_k,
                                                         temperature, top_p, uniform, token, flag);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
