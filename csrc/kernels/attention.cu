// Causal GQA attention over the paged INT8 KV cache, row-at-a-time form: every query
// row is an independent problem against keys 0..pos of its request, so one kernel
// serves decode (one row per request), MTP verification (a few rows) and chunked
// prefill rows.  The query heads that share a KV head are processed together so the
// INT8 K/V rows are read once; long contexts are split along the key axis into
// partial (max, sum, out) records that a second kernel merges.  INT8 values are
// dequantised on the fly with their group-64 FP16 scales.  Replaces the decode
// configurations of causal_attention_int8 and merge_attention_int8
// (kernels/cuda/model/attention_rows.py:61-276,280-400).
#include "api.h"
#include "common.cuh"

namespace orinfer {

constexpr int ATTN_WARPS = 4;

template <int D, int REP>
__global__ void __launch_bounds__(ATTN_WARPS * 32) attn_rows_kernel(
    const __half* __restrict__ q, const __half* __restrict__ gate, const int* __restrict__ row_req,
    const int* __restrict__ row_pos, const int* __restrict__ page_table, int max_pages,
    const int8_t* __restrict__ kc, const int8_t* __restrict__ vc, const __half* __restrict__ ks,
    const __half* __restrict__ vs, __half* __restrict__ out, int qh, int kvh, int splits,
    float* __restrict__ scratch) {
  constexpr int EPL = D / 32;
  constexpr int GROUPS = D / 64;
  const int row = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int req = row_req[row];
  const int kv_len = row_pos[row] + 1;
  const int per = (kv_len + splits - 1) / splits;
  const int k_lo = split * per, k_hi = min(kv_len, k_lo + per);
  const int group = (lane * EPL) / 64;
  const float qscale = rsqrtf(static_cast<float>(D)) * 1.4426950408889634f;

  float qv[REP][EPL], acc[REP][EPL], mx[REP], sum[REP];
#pragma unroll
  for (int r = 0; r < REP; ++r) {
    const __half* qp = q + (static_cast<size_t>(row) * qh + h * REP + r) * D + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      qv[r][e] = __half2float(qp[e]) * qscale;
      acc[r][e] = 0.f;
    }
    mx[r] = -INFINITY;
    sum[r] = 0.f;
  }
  const int* pages = page_table + static_cast<size_t>(req) * max_pages;
  for (int key = k_lo + warp; key < k_hi; key += ATTN_WARPS) {
    const int page = pages[key >> 7];
    const size_t slot = (static_cast<size_t>(page) * 128 + (key & 127)) * kvh + h;
    const int8_t* kp = kc + slot * D + lane * EPL;
    const int8_t* vp = vc + slot * D + lane * EPL;
    const float ksc = __half2float(ks[slot * GROUPS + group]);
    const float vsc = __half2float(vs[slot * GROUPS + group]);
    float kf[EPL], vf[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      kf[e] = static_cast<float>(kp[e]) * ksc;
      vf[e] = static_cast<float>(vp[e]) * vsc;
    }
#pragma unroll
    for (int r = 0; r < REP; ++r) {
      float d = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) d += qv[r][e] * kf[e];
      d = warp_sum(d);
      const float mnew = fmaxf(mx[r], d);
      const float corr = exp2f(mx[r] - mnew);
      const float p = exp2f(d - mnew);
      sum[r] = sum[r] * corr + p;
#pragma unroll
      for (int e = 0; e < EPL; ++e) acc[r][e] = acc[r][e] * corr + p * vf[e];
      mx[r] = mnew;
    }
  }
  __shared__ float s_m[ATTN_WARPS][REP], s_l[ATTN_WARPS][REP];
  __shared__ float s_o[ATTN_WARPS][REP][D];
#pragma unroll
  for (int r = 0; r < REP; ++r) {
    if (lane == 0) {
      s_m[warp][r] = mx[r];
      s_l[warp][r] = sum[r];
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) s_o[warp][r][lane * EPL + e] = acc[r][e];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < REP * D; i += blockDim.x) {
    const int r = i / D, d = i % D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATTN_WARPS; ++w) m = fmaxf(m, s_m[w][r]);
    float l = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < ATTN_WARPS; ++w) {
      const float f = s_m[w][r] == -INFINITY ? 0.f : exp2f(s_m[w][r] - m);
      l += s_l[w][r] * f;
      o += s_o[w][r][d] * f;
    }
    const int head = h * REP + r;
    if (splits == 1) {
      float v = l > 0.f ? o / l : 0.f;
      if (gate) {
        const float g = __half2float(gate[(static_cast<size_t>(row) * qh + head) * D + d]);
        v *= __fdiv_rn(1.f, 1.f + expf(-g));
      }
      out[(static_cast<size_t>(row) * qh + head) * D + d] = __float2half_rn(v);
    } else {
      float* rec = scratch + ((static_cast<size_t>(row) * qh + head) * splits + split) * (D + 2);
      if (d == 0) {
        rec[0] = m;
        rec[1] = l;
      }
      rec[2 + d] = o;
    }
  }
}

template <int D>
__global__ void attn_merge_kernel(const float* __restrict__ scratch,
                                  const __half* __restrict__ gate, __half* __restrict__ out,
                                  int qh, int splits) {
  const int row = blockIdx.x, head = blockIdx.y;
  const float* rec = scratch + (static_cast<size_t>(row) * qh + head) * splits * (D + 2);
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, rec[s * (D + 2)]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float l = 0.f, o = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = rec[s * (D + 2)];
      const float f = ms == -INFINITY ? 0.f : exp2f(ms - m);
      l += rec[s * (D + 2) + 1] * f;
      o += rec[s * (D + 2) + 2 + d] * f;
    }
    float v = l > 0.f ? o / l : 0.f;
    if (gate) {
      const float g = __half2float(gate[(static_cast<size_t>(row) * qh + head) * D + d]);
      v *= __fdiv_rn(1.f, 1.f + expf(-g));
    }
    out[(static_cast<size_t>(row) * qh + head) * D + d] = __float2half_rn(v);
  }
}

template <int D, int REP>
static int launch_attn(const __half* q, const __half* gate, const int* row_req, const int* row_pos,
                       const int* page_table, int max_pages, const int8_t* kc, const int8_t* vc,
                       const __half* ks, const __half* vs, __half* out, int rows, int qh, int kvh,
                       int splits, float* scratch, cudaStream_t stream) {
  dim3 grid(rows, kvh, splits);
  attn_rows_kernel<D, REP><<<grid, ATTN_WARPS * 32, 0, stream>>>(
      q, gate, row_req, row_pos, page_table, max_pages, kc, vc, ks, vs, out, qh, kvh, splits,
      scratch);
  if (splits > 1)
    attn_merge_kernel<D><<<dim3(rows, qh), D < 128 ? 64 : 128, 0, stream>>>(scratch, gate, out, qh,
                                                                           splits);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace orinfer

using namespace orinfer;

extern "C" size_t orinfer_attention_scratch_bytes(int rows, int qh, int head_dim, int splits) {
  if (splits <= 1) return 0;
  return static_cast<size_t>(rows) * qh * splits * (head_dim + 2) * sizeof(float);
}

extern "C" int orinfer_attention(const __half* q, const __half* gate, const int* row_req,
                                 const int* row_pos, const int* page_table, int max_pages,
                                 const int8_t* kc, const int8_t* vc, const __half* ks,
                                 const __half* vs, __half* out, int rows, int qh, int kvh,
                                 int head_dim, int splits, float* scratch, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (splits < 1 || (splits > 1 && scratch == nullptr) || kvh <= 0 || qh % kvh) return -1;
  const int rep = qh / kvh;
#define CASE(DD, RR)                                                                         \
  if (head_dim == DD && rep == RR)                                                           \
    return launch_attn<DD, RR>(q, gate, row_req, row_pos, page_table, max_pages, kc, vc, ks, \
                               vs, out, rows, qh, kvh, splits, scratch, stream);
  CASE(64, 1) CASE(64, 2) CASE(64, 4) CASE(64, 8)
  CASE(128, 1) CASE(128, 2) CASE(128, 4) CASE(128, 5) CASE(128, 8)
  CASE(256, 4) CASE(256, 8)
#undef CASE
  return -1;
}
