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

__device__ __forceinline__ void unpack16(const int4& raw, float (&f)[16]) {
  const int w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[4 * i + 0] = static_cast<float>(static_cast<signed char>(w[i] & 0xff));
    f[4 * i + 1] = static_cast<float>(static_cast<signed char>((w[i] >> 8) & 0xff));
    f[4 * i + 2] = static_cast<float>(static_cast<signed char>((w[i] >> 16) & 0xff));
    f[4 * i + 3] = static_cast<float>(w[i] >> 24);
  }
}

// One CTA per (row, group of RPC query heads sharing a KV head, key split).  A key's D INT8
// channels are covered by D/16 lanes with one 16-byte load each, so a warp takes 32/(D/16)
// keys per step (4 at D = 128) and the four warps interleave.  Keys are processed in chunks
// of up to ATTN_CHUNK: pass 1 writes the scores of the chunk to shared memory, the softmax
// weights are formed there once per (head, key), and pass 2 accumulates weight x V.  No
// running rescale sits in the inner loops (only one per chunk), so both passes are streams
// of independent multiply-adds.
constexpr int ATTN_CHUNK = 512;

template <int D, int RPC>
__global__ void __launch_bounds__(ATTN_WARPS * 32) attn_rows_kernel(
    const __half* __restrict__ q, const __half* __restrict__ gate, const int* __restrict__ row_req,
    const int* __restrict__ row_pos, const int* __restrict__ page_table, int max_pages,
    const int8_t* __restrict__ kc, const int8_t* __restrict__ vc, const __half* __restrict__ ks,
    const __half* __restrict__ vs, __half* __restrict__ out, int qh, int kvh, int splits,
    float* __restrict__ scratch, int rep) {
  constexpr int LPK = D / 16;                  // lanes per key
  constexpr int KPW = 32 / LPK;                // keys per warp step
  constexpr int KPI = ATTN_WARPS * KPW;        // keys per CTA step
  constexpr int GROUPS = D / 64;
  constexpr int THREADS = ATTN_WARPS * 32;
  const int row = blockIdx.x, split = blockIdx.z;
  const int hgroups = rep / RPC;               // CTAs per KV head
  const int h = blockIdx.y / hgroups;          // KV head
  const int head0 = h * rep + (blockIdx.y % hgroups) * RPC;   // first query head of this CTA
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int sub = lane % LPK, kslot = lane / LPK;
  const int req = row_req[row];
  const int kv_len = row_pos[row] + 1;
  const int per = (kv_len + splits - 1) / splits;
  const int k_lo = split * per, k_hi = min(kv_len, k_lo + per);
  const int group = (sub * 16) / 64;
  const float qscale = rsqrtf(static_cast<float>(D)) * 1.4426950408889634f;

  // query heads (pre-scaled, FP32) in shared memory: every lane group reads the same slice,
  // so the loads are broadcasts, and the registers go to the accumulators
  __shared__ __align__(16) float s_q[RPC][D];
  __shared__ float s_p[RPC][ATTN_CHUNK];       // scores, then softmax weights, of the chunk
  __shared__ float s_red[ATTN_WARPS][RPC];
  __shared__ float s_m[RPC], s_l[RPC], s_corr[RPC];
  __shared__ float s_o[ATTN_WARPS][RPC][D];
  __shared__ int s_page[ATTN_CHUNK / 128 + 2];  // page ids covering the chunk
  for (int i = tid; i < RPC * D; i += THREADS)
    s_q[i / D][i % D] =
        __half2float(q[(static_cast<size_t>(row) * qh + head0 + i / D) * D + i % D]) * qscale;
  if (tid < RPC) {
    s_m[tid] = -INFINITY;
    s_l[tid] = 0.f;
  }
  float acc[RPC][16];
#pragma unroll
  for (int r = 0; r < RPC; ++r)
#pragma unroll
    for (int e = 0; e < 16; ++e) acc[r][e] = 0.f;
  __syncthreads();
  const int* pages = page_table + static_cast<size_t>(req) * max_pages;

  for (int c0 = k_lo; c0 < k_hi; c0 += ATTN_CHUNK) {
    const int n = min(ATTN_CHUNK, k_hi - c0);
    const int page0 = c0 >> 7;
    if (tid <= ((c0 + n - 1) >> 7) - page0) s_page[tid] = pages[page0 + tid];
    __syncthreads();
    // slot of chunk key kk in the paged cache (page ids come from shared memory, so a key's
    // address does not wait for a global load)
    auto slot_of = [&](int kk) {
      const int key = c0 + kk;
      return (static_cast<size_t>(s_page[(key >> 7) - page0]) * 128 + (key & 127)) * kvh + h;
    };
    // ---- pass 1: scores of the chunk (loop uniform over the warp: the shuffles need every
    // lane); the loads of the next step are issued before this step's arithmetic
    float lmax[RPC];
#pragma unroll
    for (int r = 0; r < RPC; ++r) lmax[r] = -INFINITY;
    int4 raw = make_int4(0, 0, 0, 0);
    float sc_next = 0.f;
    if (warp * KPW + kslot < n) {
      const size_t slot = slot_of(warp * KPW + kslot);
      raw = __ldg(reinterpret_cast<const int4*>(kc + slot * D + sub * 16));
      sc_next = __half2float(ks[slot * GROUPS + group]);
    }
    for (int base = warp * KPW; base < n; base += KPI) {
      const int kk = base + kslot;
      const bool valid = kk < n;
      float kf[16];
      unpack16(raw, kf);
      const float ksc = valid ? sc_next : 0.f;
      if (kk + KPI < n) {
        const size_t slot = slot_of(kk + KPI);
        raw = __ldg(reinterpret_cast<const int4*>(kc + slot * D + sub * 16));
        sc_next = __half2float(ks[slot * GROUPS + group]);
      }
#pragma unroll
      for (int r = 0; r < RPC; ++r) {
        float d = 0.f;
#pragma unroll
        for (int e4 = 0; e4 < 4; ++e4) {
          const float4 qq = *reinterpret_cast<const float4*>(&s_q[r][sub * 16 + e4 * 4]);
          d += qq.x * kf[e4 * 4] + qq.y * kf[e4 * 4 + 1] + qq.z * kf[e4 * 4 + 2] +
               qq.w * kf[e4 * 4 + 3];
        }
        d *= ksc;
#pragma unroll
        for (int o = 1; o < LPK; o <<= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        if (valid) {
          lmax[r] = fmaxf(lmax[r], d);
          if (sub == 0) s_p[r][kk] = d;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < RPC; ++r) {
      const float m = warp_max(lmax[r]);
      if (lane == 0) s_red[warp][r] = m;
    }
    __syncthreads();
    // ---- new running maximum, rescale factor of what was accumulated so far
    if (tid < RPC) {
      float m = s_m[tid];
#pragma unroll
      for (int w = 0; w < ATTN_WARPS; ++w) m = fmaxf(m, s_red[w][tid]);
      s_corr[tid] = s_m[tid] == -INFINITY ? 0.f : exp2f(s_m[tid] - m);
      s_m[tid] = m;
    }
    __syncthreads();
    // ---- softmax weights of the chunk, once per (head, key)
    float lsum[RPC];
#pragma unroll
    for (int r = 0; r < RPC; ++r) {
      const float m = s_m[r];
      float t = 0.f;
      for (int kk = tid; kk < n; kk += THREADS) {
        const float p = exp2f(s_p[r][kk] - m);
        s_p[r][kk] = p;
        t += p;
      }
      lsum[r] = warp_sum(t);
    }
    __syncthreads();                           // every warp is done with s_red's maxima
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < RPC; ++r) s_red[warp][r] = lsum[r];
    }
    __syncthreads();
    if (tid < RPC) {
      float l = s_l[tid] * s_corr[tid];
#pragma unroll
      for (int w = 0; w < ATTN_WARPS; ++w) l += s_red[w][tid];
      s_l[tid] = l;
    }
    if (c0 > k_lo) {
#pragma unroll
      for (int r = 0; r < RPC; ++r) {
        const float c = s_corr[r];
#pragma unroll
        for (int e = 0; e < 16; ++e) acc[r][e] *= c;
      }
    }
    // ---- pass 2: weight x V (same one-step-ahead loads)
    if (warp * KPW + kslot < n) {
      const size_t slot = slot_of(warp * KPW + kslot);
      raw = __ldg(reinterpret_cast<const int4*>(vc + slot * D + sub * 16));
      sc_next = __half2float(vs[slot * GROUPS + group]);
    }
    for (int base = warp * KPW; base < n; base += KPI) {
      const int kk = base + kslot;
      if (kk < n) {
        float vf[16];
        unpack16(raw, vf);
        const float vsc = sc_next;
        if (kk + KPI < n) {
          const size_t slot = slot_of(kk + KPI);
          raw = __ldg(reinterpret_cast<const int4*>(vc + slot * D + sub * 16));
          sc_next = __half2float(vs[slot * GROUPS + group]);
        }
#pragma unroll
        for (int r = 0; r < RPC; ++r) {
          const float pv = s_p[r][kk] * vsc;
#pragma unroll
          for (int e = 0; e < 16; ++e) acc[r][e] += pv * vf[e];
        }
      }
    }
    __syncthreads();                           // s_p is rewritten by the next chunk
  }
  // lanes that only differ in kslot hold sums over disjoint key sets (same reference maximum)
#pragma unroll
  for (int o = LPK; o < 32; o <<= 1) {
#pragma unroll
    for (int r = 0; r < RPC; ++r)
#pragma unroll
      for (int e = 0; e < 16; ++e) acc[r][e] += __shfl_xor_sync(0xffffffffu, acc[r][e], o);
  }
  if (kslot == 0) {
#pragma unroll
    for (int r = 0; r < RPC; ++r)
#pragma unroll
      for (int e = 0; e < 16; ++e) s_o[warp][r][sub * 16 + e] = acc[r][e];
  }
  __syncthreads();
  for (int i = tid; i < RPC * D; i += THREADS) {
    const int r = i / D, d = i % D;
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < ATTN_WARPS; ++w) o += s_o[w][r][d];
    const float m = s_m[r], l = s_l[r];
    const int head = head0 + r;
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

template <int D, int RPC>
static int launch_attn(const __half* q, const __half* gate, const int* row_req, const int* row_pos,
                       const int* page_table, int max_pages, const int8_t* kc, const int8_t* vc,
                       const __half* ks, const __half* vs, __half* out, int rows, int qh, int kvh,
                       int rep, int splits, float* scratch, cudaStream_t stream) {
  dim3 grid(rows, kvh * (rep / RPC), splits);
  attn_rows_kernel<D, RPC><<<grid, ATTN_WARPS * 32, 0, stream>>>(
      q, gate, row_req, row_pos, page_table, max_pages, kc, vc, ks, vs, out, qh, kvh, splits,
      scratch, rep);
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
  // query heads per CTA: all heads of a KV head up to 5; 8 run as two groups of 4 (their
  // accumulators would not fit the register file)
#define CASE(DD, RR, RPC)                                                                     \
  if (head_dim == DD && rep == RR)                                                            \
    return launch_attn<DD, RPC>(q, gate, row_req, row_pos, page_table, max_pages, kc, vc, ks, \
                                vs, out, rows, qh, kvh, rep, splits, scratch, stream);
  CASE(64, 1, 1) CASE(64, 2, 2) CASE(64, 4, 4) CASE(64, 8, 4)
  CASE(128, 1, 1) CASE(128, 2, 2) CASE(128, 4, 4) CASE(128, 5, 5) CASE(128, 8, 4)
  CASE(256, 1, 1) CASE(256, 2, 2) CASE(256, 4, 4) CASE(256, 8, 4)
#undef CASE
  return -1;
}
