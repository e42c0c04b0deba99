// Bandwidth-bound row kernels: W8 embedding gather, the fused
// residual-add / RMSNorm / SwiGLU / block-128 Hadamard rotation / per-token INT8
// quantiser, RoPE tables, q/k head-norm + RoPE + paged INT8 KV write, and greedy
// argmax.  They replace the reference's residual_norm_rotate_a8 /
// rotate_activation_a8 (kernels/cuda/model/rotation_a8.py:267,608),
// activation_quantization (kernels/cuda/operators/op30_activation_quantization.py:22),
// full_prepare_mrope_int8 (kernels/cuda/model/kv_int8.py:63) and greedy_partials /
// greedy_merge (kernels/cuda/model/greedy.py:11,83).
#include <cooperative_groups.h>

#include "common.cuh"
#include "api.h"
#include "argmax_kernels.cuh"
#include "tp_comm.cuh"

namespace cg = cooperative_groups;

namespace orinfer {

// ------------------------------------------------------------------ embedding
__global__ void embed_w8_kernel(const int* __restrict__ ids, const int8_t* __restrict__ table,
                                const __half* __restrict__ scales, __half* __restrict__ out,
                                int hidden, int vocab, int* status) {
  const int row = blockIdx.x;
  int id = ids[row];
  if (id < 0 || id >= vocab) {
    report_status(status, STATUS_BAD_INDEX, 1);
    id = 0;
  }
  const float s = __half2float(scales[id]);
  const int8_t* src = table + static_cast<size_t>(id) * hidden;
  __half* dst = out + static_cast<size_t>(row) * hidden;
  for (int i = threadIdx.x * 16; i < hidden; i += blockDim.x * 16) {
    const int4 raw = *reinterpret_cast<const int4*>(src + i);
    const int8_t* b = reinterpret_cast<const int8_t*>(&raw);
    __align__(16) __half h[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) h[j] = __float2half_rn(static_cast<float>(b[j]) * s);
    *reinterpret_cast<int4*>(dst + i) = *reinterpret_cast<const int4*>(h);
    *reinterpret_cast<int4*>(dst + i + 8) = *reinterpret_cast<const int4*>(h + 8);
  }
}

// ------------------------------------------------------------------ act_prep
constexpr int MAX_NORM_BLOCKS = 128;          // rows that are normalised have K <= 16384

template <int CL>
__device__ __forceinline__ float cluster_reduce(float v, float* slot, bool is_max) {
  if (CL == 1) return v;
  cg::cluster_group cluster = cg::this_cluster();
  if (threadIdx.x == 0) *slot = v;
  cluster.sync();
  float r = 0.f;
#pragma unroll
  for (int c = 0; c < CL; ++c) {
    const float o = *cluster.map_shared_rank(slot, c);
    r = is_max ? fmaxf(r, o) : r + o;
  }
  return r;
}

template <bool SWIGLU, int CL>
__global__ void __launch_bounds__(512) act_prep_kernel(
    const __half* __restrict__ x, float* __restrict__ resid, const __half* __restrict__ norm_w,
    const int8_t* __restrict__ signs, int8_t* __restrict__ q_out, float* __restrict__ scale_out,
    __half* __restrict__ y_out, int K, float eps, int zero_centered, InboxIn in, int* status,
    AgOut ag, int rows, const int* __restrict__ row_limit, int row_base) {
  extern __shared__ float rowbuf_raw[];
  __shared__ float red[32];
  __shared__ float cl_slot[2];
  __shared__ float blk_sum[MAX_NORM_BLOCKS];
  const int tid = threadIdx.x;
  const int crank = CL > 1 ? static_cast<int>(blockIdx.x) % CL : 0;
  const int nblk = K / 128;
  const int k_lo = (nblk * crank / CL) * 128, k_hi = (nblk * (crank + 1) / CL) * 128;
  float* rowbuf = rowbuf_raw - k_lo;           // indexed by the channel number
  // sequence-parallel form: this rank handles only the rows it owns and pushes the result
  const bool sp = !SWIGLU && ag.tp > 0;
  const int row = (sp ? ag.rank * ag.rows_per : row_base) + static_cast<int>(blockIdx.x) / CL;
  if (sp && row >= rows) {                 // tail of the last owner: nothing to do but count
    if (in.inbox != nullptr) inbox_consumed(in, gridDim.x);
    ag_signal_done(ag, gridDim.x);
    return;
  }
  // a device-side row count (rows routed to this rank's experts) bounds the useful work of a
  // launch that was sized for the worst case
  if (row_limit != nullptr && row >= *row_limit) return;
  if (SWIGLU) {
    const __half* g = x + static_cast<size_t>(row) * 2 * K;
    const __half* u = g + K;
    for (int i = k_lo + tid * 8; i < k_hi; i += blockDim.x * 8) {
      const int4 gr = *reinterpret_cast<const int4*>(g + i);
      const int4 ur = *reinterpret_cast<const int4*>(u + i);
      const __half* gh = reinterpret_cast<const __half*>(&gr);
      const __half* uh = reinterpret_cast<const __half*>(&ur);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gv = __half2float(gh[j]);
        const float sg = __fdiv_rn(1.f, 1.f + expf(-gv));
        rowbuf[i + j] = round_f16(__fmul_rn(__fmul_rn(gv, sg), __half2float(uh[j])));
      }
    }
  } else {
    const __half* xr = x ? x + static_cast<size_t>(row) * K : nullptr;
    float* rr = resid ? resid + static_cast<size_t>(row) * K : nullptr;
    const bool from_inbox = in.inbox != nullptr;
    const bool from_ll = in.ll != nullptr;
    const int ll_seq = from_ll ? *reinterpret_cast<volatile int*>(in.seen) + 1 : 0;
    if (from_inbox && !from_ll) inbox_wait(in, status);   // a timed-out wait is reported
    for (int i = k_lo + tid * 8; i < k_hi; i += blockDim.x * 8) {
      float v[8];
      if (from_ll) {
        // low-latency form: each unit carries its own sequence number; sum the sources in
        // fixed order as soon as their units have arrived
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = 0.f;
        for (int s = 0; s < in.tp; ++s) {
          const uint2* src = in.ll + (static_cast<size_t>(s) * LL_ROWS + row) * (K / 2) + i / 2;
          uint32_t w[4];
          ll_load4(src, ll_seq, w[0], w[1], status, s);
          ll_load4(src + 2, ll_seq, w[2], w[3], status, s);
          const __half* h = reinterpret_cast<const __half*>(w);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] += __half2float(h[j]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = round_f16(v[j]);
      } else if (from_inbox) {
        // sum the tp partial rows in fixed source order; bypass L1 (peers wrote this memory)
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = 0.f;
        for (int s = 0; s < in.tp; ++s) {
          const __half* src =
              in.inbox + (static_cast<size_t>(s) * in.rows_cap + row) * K + i;
          const int4 raw = __ldcg(reinterpret_cast<const int4*>(src));
          const __half* h = reinterpret_cast<const __half*>(&raw);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] += __half2float(h[j]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = round_f16(v[j]);
      } else if (xr) {
        const int4 raw = *reinterpret_cast<const int4*>(xr + i);
        const __half* h = reinterpret_cast<const __half*>(&raw);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __half2float(h[j]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = 0.f;
      }
      if (rr) {
        const float4 r0 = *reinterpret_cast<const float4*>(rr + i);
        const float4 r1 = *reinterpret_cast<const float4*>(rr + i + 4);
        v[0] += r0.x; v[1] += r0.y; v[2] += r0.z; v[3] += r0.w;
        v[4] += r1.x; v[5] += r1.y; v[6] += r1.z; v[7] += r1.w;
        *reinterpret_cast<float4*>(rr + i) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(rr + i + 4) = make_float4(v[4], v[5], v[6], v[7]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) rowbuf[i + j] = v[j];
    }
    if (norm_w) {
      // Sum of squares in a launch-independent order: one partial per 128-channel block
      // (fixed lane pattern), then the blocks added in channel order.  One row therefore
      // normalises to the same bits whether it runs alone (cluster form), in a large packet
      // or inside another kernel's prologue.
      __syncthreads();
      {
        const int warp = tid >> 5, lane = tid & 31, nw = blockDim.x >> 5;
        for (int b = k_lo / 128 + warp; b < k_hi / 128; b += nw) {
          const float s = block128_sumsq(rowbuf + b * 128, lane);
          if (lane == 0) blk_sum[b - k_lo / 128] = s;
        }
      }
      __syncthreads();
      float total = 0.f;
      if (CL == 1) {
        for (int b = 0; b < nblk; ++b) total = __fadd_rn(total, blk_sum[b]);
      } else {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        for (int c = 0; c < CL; ++c) {
          const float* remote = cluster.map_shared_rank(blk_sum, c);
          const int count = nblk * (c + 1) / CL - nblk * c / CL;
          for (int b = 0; b < count; ++b) total = __fadd_rn(total, remote[b]);
        }
      }
      const float r = rsqrtf(total / static_cast<float>(K) + eps);
      const float add = zero_centered ? 1.f : 0.f;
      for (int i = k_lo + tid * 8; i < k_hi; i += blockDim.x * 8) {
        const int4 wr = *reinterpret_cast<const int4*>(norm_w + i);
        const __half* wh = reinterpret_cast<const __half*>(&wr);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          rowbuf[i + j] =
              round_f16(__fmul_rn(__fmul_rn(rowbuf[i + j], r), __half2float(wh[j]) + add));
      }
    } else {
      for (int i = k_lo + tid * 8; i < k_hi; i += blockDim.x * 8)
#pragma unroll
        for (int j = 0; j < 8; ++j) rowbuf[i + j] = round_f16(rowbuf[i + j]);
    }
  }
  __syncthreads();
  if (y_out) {
    __half* yr = y_out + static_cast<size_t>(row) * K;
    for (int i = k_lo + tid * 8; i < k_hi; i += blockDim.x * 8) {
      __align__(16) __half h[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) h[j] = __float2half_rn(rowbuf[i + j]);
      *reinterpret_cast<int4*>(yr + i) = *reinterpret_cast<const int4*>(h);
    }
  }
  float amax = 0.f;
  if (signs) {
    // Each warp transforms whole 128-blocks; lane holds 4 consecutive values.
    const int warp = tid >> 5, lane = tid & 31, nw = blockDim.x >> 5;
    for (int b = k_lo / 128 + warp; b < k_hi / 128; b += nw) {
      amax = fmaxf(amax, hadamard128_inplace(rowbuf + b * 128, signs + b * 128, lane));
    }
  } else {
    for (int i = k_lo + tid; i < k_hi; i += blockDim.x) amax = fmaxf(amax, fabsf(rowbuf[i]));
  }
  amax = cluster_reduce<CL>(block_reduce(amax, red, true), &cl_slot[1], true);
  const float scale = a8_scale(amax);
  if (sp) {
    // all-gather by push: the INT8 row and its scale go to every rank's activation buffer
    if (tid < ag.tp) ag.scale[tid][row] = scale;
    for (int i = k_lo + tid * 16; i < k_hi; i += blockDim.x * 16) {
      __align__(16) signed char c[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) c[j] = static_cast<signed char>(a8_code(rowbuf[i + j], scale));
      for (int d = 0; d < ag.tp; ++d)
        *reinterpret_cast<int4*>(ag.q[d] + static_cast<size_t>(row) * K + i) =
            *reinterpret_cast<const int4*>(c);
    }
    if (in.inbox != nullptr) inbox_consumed(in, gridDim.x);
    ag_signal_done(ag, gridDim.x);
    return;
  }
  if (tid == 0 && crank == 0) scale_out[row] = scale;
  int8_t* qr = q_out + static_cast<size_t>(row) * K;
  for (int i = k_lo + tid * 4; i < k_hi; i += blockDim.x * 4) {
    char4 c;
    c.x = static_cast<signed char>(a8_code(rowbuf[i + 0], scale));
    c.y = static_cast<signed char>(a8_code(rowbuf[i + 1], scale));
    c.z = static_cast<signed char>(a8_code(rowbuf[i + 2], scale));
    c.w = static_cast<signed char>(a8_code(rowbuf[i + 3], scale));
    *reinterpret_cast<char4*>(qr + i) = c;
  }
  if (!SWIGLU && (in.inbox != nullptr || in.ll != nullptr)) inbox_consumed(in, gridDim.x);
  // a CTA's shared memory must outlive the cluster's reads of it
  if (CL > 1) cg::this_cluster().sync();
}

// One warp per row, the whole row in registers (K = 128 * NBLK <= 5120): no block barrier and
// no shared memory, only shuffles.  Serves the plain forms (x and / or residual, optional
// RMSNorm, optional rotation) of packets with many rows; same helpers and the same order of
// operations as the CTA-per-row kernel, so a row gives the same bits through either.
template <int NBLK>
__global__ void __launch_bounds__(128) act_prep_warp_kernel(
    const __half* __restrict__ x, float* __restrict__ resid, const __half* __restrict__ norm_w,
    const int8_t* __restrict__ signs, int8_t* __restrict__ q_out, float* __restrict__ scale_out,
    __half* __restrict__ y_out, int rows, float eps, int zero_centered) {
  constexpr int K = NBLK * 128;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  float v[NBLK][4];
  const __half* xr = x ? x + static_cast<size_t>(row) * K : nullptr;
  float* rr = resid ? resid + static_cast<size_t>(row) * K : nullptr;
#pragma unroll
  for (int b = 0; b < NBLK; ++b) {
    const int i = b * 128 + lane * 4;
    if (xr) {
      const uint2 raw = *reinterpret_cast<const uint2*>(xr + i);
      const __half* h = reinterpret_cast<const __half*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) v[b][j] = __half2float(h[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[b][j] = 0.f;
    }
    if (rr) {
      const float4 r = *reinterpret_cast<const float4*>(rr + i);
      v[b][0] += r.x; v[b][1] += r.y; v[b][2] += r.z; v[b][3] += r.w;
      *reinterpret_cast<float4*>(rr + i) = make_float4(v[b][0], v[b][1], v[b][2], v[b][3]);
    }
  }
  if (norm_w) {
    float total = 0.f;
#pragma unroll
    for (int b = 0; b < NBLK; ++b)
      total = __fadd_rn(total, block128_sumsq_regs(v[b][0], v[b][1], v[b][2], v[b][3]));
    const float r = rsqrtf(total / static_cast<float>(K) + eps);
    const float add = zero_centered ? 1.f : 0.f;
#pragma unroll
    for (int b = 0; b < NBLK; ++b) {
      const uint2 raw = *reinterpret_cast<const uint2*>(norm_w + b * 128 + lane * 4);
      const __half* wh = reinterpret_cast<const __half*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        v[b][j] = round_f16(__fmul_rn(__fmul_rn(v[b][j], r), __half2float(wh[j]) + add));
    }
  } else {
#pragma unroll
    for (int b = 0; b < NBLK; ++b)
#pragma unroll
      for (int j = 0; j < 4; ++j) v[b][j] = round_f16(v[b][j]);
  }
  if (y_out) {
    __half* yr = y_out + static_cast<size_t>(row) * K;
#pragma unroll
    for (int b = 0; b < NBLK; ++b) {
      __align__(8) __half h[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) h[j] = __float2half_rn(v[b][j]);
      *reinterpret_cast<uint2*>(yr + b * 128 + lane * 4) = *reinterpret_cast<const uint2*>(h);
    }
  }
  float amax = 0.f;
#pragma unroll
  for (int b = 0; b < NBLK; ++b) {
    if (signs) {
      const char4 sg = *reinterpret_cast<const char4*>(signs + b * 128 + lane * 4);
      amax = fmaxf(amax, hadamard128_regs(v[b][0], v[b][1], v[b][2], v[b][3], sg, lane));
    } else {
      amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[b][0]), fabsf(v[b][1])),
                               fmaxf(fabsf(v[b][2]), fabsf(v[b][3]))));
    }
  }
  amax = warp_max(amax);
  const float scale = a8_scale(amax);
  if (lane == 0) scale_out[row] = scale;
  int8_t* qr = q_out + static_cast<size_t>(row) * K;
#pragma unroll
  for (int b = 0; b < NBLK; ++b) {
    char4 c;
    c.x = static_cast<signed char>(a8_code(v[b][0], scale));
    c.y = static_cast<signed char>(a8_code(v[b][1], scale));
    c.z = static_cast<signed char>(a8_code(v[b][2], scale));
    c.w = static_cast<signed char>(a8_code(v[b][3], scale));
    *reinterpret_cast<char4*>(qr + b * 128 + lane * 4) = c;
  }
}

__global__ void ag_wait_kernel(AgIn in, int rows, int* status) {
  if (threadIdx.x == 0 && blockIdx.x == 0) ag_wait(in, 0, rows - 1, status);
}

// ------------------------------------------------------------------ RoPE tables
__global__ void rope_table_kernel(const int* __restrict__ positions, float* __restrict__ cosb,
                                  float* __restrict__ sinb, int rows, int half_dim, double theta) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * half_dim) return;
  const int r = idx / half_dim, j = idx % half_dim;
  const double inv = pow(theta, -static_cast<double>(2 * j) / static_cast<double>(2 * half_dim));
  const double ang = static_cast<double>(positions[r]) * inv;
  double s, c;
  sincos(ang, &s, &c);
  cosb[idx] = static_cast<float>(c);
  sinb[idx] = static_cast<float>(s);
}

// ------------------------------------------------------------------ q/k norm + RoPE + KV write
// One warp per (row, head).  Heads are ordered q[0..QH), k[0..KVH), v[0..KVH).
// Input row layout: q heads (D each, or 2D = query|gate when GATED), then K, then V.
template <int D, bool GATED>
__global__ void __launch_bounds__(256) qk_rope_kv_kernel(
    const __half* __restrict__ qkv, const __half* __restrict__ wq, const __half* __restrict__ wk,
    const float* __restrict__ cosb, const float* __restrict__ sinb,
    const int* __restrict__ row_req, const int* __restrict__ row_pos,
    const int* __restrict__ page_table, int max_pages, int qh, int kvh, float eps,
    int zero_centered, __half* __restrict__ q_out, __half* __restrict__ gate_out,
    int8_t* __restrict__ kcache, int8_t* __restrict__ vcache, __half* __restrict__ kscale,
    __half* __restrict__ vscale, int num_pages, int* status) {
  constexpr int HALF = D / 2;
  constexpr int PER = HALF / 32;          // pairs per lane
  constexpr int GROUPS = D / 64;
  const int row = blockIdx.x;
  const int head = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int heads = qh + 2 * kvh;
  if (head >= heads) return;
  const int qstride = GATED ? 2 * D : D;
  const int width = qh * qstride + 2 * kvh * D;
  const __half* src;
  const bool is_q = head < qh, is_k = !is_q && head < qh + kvh;
  if (is_q) src = qkv + static_cast<size_t>(row) * width + head * qstride;
  else src = qkv + static_cast<size_t>(row) * width + qh * qstride + (head - qh) * D;
  float a[PER], b[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    a[i] = __half2float(src[lane + 32 * i]);
    b[i] = __half2float(src[HALF + lane + 32 * i]);
  }
  if (is_q || is_k) {
    const __half* w = is_q ? wq : wk;
    if (w) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < PER; ++i) ss += a[i] * a[i] + b[i] * b[i];
      ss = warp_sum(ss);
      const float r = rsqrtf(ss / static_cast<float>(D) + eps);
      const float add = zero_centered ? 1.f : 0.f;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        a[i] = round_f16(__fmul_rn(__fmul_rn(a[i], r), __half2float(w[lane + 32 * i]) + add));
        b[i] = round_f16(
            __fmul_rn(__fmul_rn(b[i], r), __half2float(w[HALF + lane + 32 * i]) + add));
      }
    }
    const float* cr = cosb + static_cast<size_t>(row) * HALF;
    const float* sr = sinb + static_cast<size_t>(row) * HALF;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const float c = cr[lane + 32 * i], s = sr[lane + 32 * i];
      const float na = round_f16(__fsub_rn(__fmul_rn(a[i], c), __fmul_rn(b[i], s)));
      const float nb = round_f16(__fadd_rn(__fmul_rn(b[i], c), __fmul_rn(a[i], s)));
      a[i] = na;
      b[i] = nb;
    }
  }
  if (is_q) {
    __half* dst = q_out + (static_cast<size_t>(row) * qh + head) * D;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      dst[lane + 32 * i] = __float2half_rn(a[i]);
      dst[HALF + lane + 32 * i] = __float2half_rn(b[i]);
    }
    if (GATED) {
      __half* gd = gate_out + (static_cast<size_t>(row) * qh + head) * D;
      for (int i = lane; i < D; i += 32) gd[i] = src[D + i];
    }
    return;
  }
  // K or V: quantise per 64-channel group and write into the paged cache.
  const int req = row_req[row], pos = row_pos[row];
  const int page = page_table[static_cast<size_t>(req) * max_pages + (pos >> 7)];
  if (page < 0 || page >= num_pages) {
    if (lane == 0) report_status(status, STATUS_BAD_INDEX, 2);
    return;
  }
  const int kvhead = is_k ? head - qh : head - qh - kvh;
  const size_t slot = static_cast<size_t>(page) * 128 + (pos & 127);
  float gmax[GROUPS];
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) gmax[g] = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int ja = lane + 32 * i, jb = HALF + ja;
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) {
      if (ja / 64 == g) gmax[g] = fmaxf(gmax[g], fabsf(a[i]));
      if (jb / 64 == g) gmax[g] = fmaxf(gmax[g], fabsf(b[i]));
    }
  }
  float gscale[GROUPS];
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
    const float m = warp_max(gmax[g]);
    gscale[g] = round_f16(fmaxf(__fdiv_rn(m, 127.f), 5.9604644775390625e-08f));
  }
  int8_t* cdst = (is_k ? kcache : vcache) + (slot * kvh + kvhead) * D;
  __half* sdst = (is_k ? kscale : vscale) + (slot * kvh + kvhead) * GROUPS;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int ja = lane + 32 * i, jb = HALF + ja;
    float sa = gscale[0], sb = gscale[0];
#pragma unroll
    for (int g = 1; g < GROUPS; ++g) {
      if (ja / 64 == g) sa = gscale[g];
      if (jb / 64 == g) sb = gscale[g];
    }
    cdst[ja] = static_cast<int8_t>(a8_code(a[i], sa));
    cdst[jb] = static_cast<int8_t>(a8_code(b[i], sb));
  }
  if (lane < GROUPS) {
    float s = gscale[0];
#pragma unroll
    for (int g = 1; g < GROUPS; ++g)
      if (lane == g) s = gscale[g];
    sdst[lane] = __float2half_rn(s);
  }
}

}  // namespace orinfer

using namespace orinfer;

static int act_prep_launch(const __half* x, float* resid, const __half* norm_w, const int8_t* signs,
                           int8_t* q_out, float* scale_out, __half* y_out, int rows, int K,
                           float eps, int zero_centered, int swiglu, InboxIn in,
                           cudaStream_t stream, AgOut ag = AgOut{},
                           const int* row_limit = nullptr, int row_base = 0);

extern "C" {

int orinfer_embed_w8(const int* ids, const int8_t* table, const __half* scales, __half* out,
                     int rows, int hidden, int vocab, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hidden % 16) return -1;
  if (runtime_ensure_init() != cudaSuccess) return -2;
  embed_w8_kernel<<<rows, 128, 0, stream>>>(ids, table, scales, out, hidden, vocab,
                                            runtime_status_ptr());
  return static_cast<int>(cudaGetLastError());
}

int orinfer_act_prep(const __half* x, float* resid, const __half* norm_w, const int8_t* signs,
                     int8_t* q_out, float* scale_out, __half* y_out, int rows, int K, float eps,
                     int zero_centered, int swiglu, cudaStream_t stream) {
  InboxIn none{};
  return act_prep_launch(x, resid, norm_w, signs, q_out, scale_out, y_out, rows, K, eps,
                         zero_centered, swiglu, none, stream);
}

// Same as orinfer_act_prep for a launch sized for the worst case: rows at or beyond the
// device-side count *row_limit are skipped.
int orinfer_act_prep_limited(const __half* x, const int8_t* signs, int8_t* q_out,
                             float* scale_out, int rows, int K, int swiglu, const int* row_limit,
                             cudaStream_t stream) {
  InboxIn none{};
  return act_prep_launch(x, nullptr, nullptr, signs, q_out, scale_out, nullptr, rows, K, 1e-6f, 0,
                         swiglu, none, stream, AgOut{}, row_limit);
}

// Same, but the branch input is the sum of the tp partial rows in the local inbox.
int orinfer_act_prep_inbox(const OrinferInbox* inbox, float* resid, const __half* norm_w,
                           const int8_t* signs, int8_t* q_out, float* scale_out, __half* y_out,
                           int rows, int K, float eps, int zero_centered, cudaStream_t stream) {
  if (inbox == nullptr || inbox->tp < 1 || inbox->tp > TP_MAX || rows > inbox->rows_cap) return -1;
  InboxIn in{};
  in.inbox = reinterpret_cast<const __half*>(inbox->inbox);
  in.flag = inbox->flag;
  in.seen = inbox->seen;
  in.ticket = inbox->ticket;
  in.tp = inbox->tp;
  in.rows_cap = inbox->rows_cap;
  in.ll = nullptr;
  if (inbox->ll != nullptr) {             // low-latency form: decode-sized packets only
    if (rows > LL_ROWS) return -1;
    in.ll = reinterpret_cast<const uint2*>(inbox->ll);
    in.inbox = nullptr;
  }
  return act_prep_launch(nullptr, resid, norm_w, signs, q_out, scale_out, y_out, rows, K, eps,
                         zero_centered, 0, in, stream);
}

// Rows [row_base, row_base + count) only (the rows this rank owns after a reduce-scatter):
// sums the tp partial rows, adds the residual, normalises, rotates and quantises into the
// LOCAL buffers at the same row indices.  Every CTA still takes part in the inbox hand-shake.
int orinfer_act_prep_inbox_rows(const OrinferInbox* inbox, float* resid, const __half* norm_w,
                                const int8_t* signs, int8_t* q_out, float* scale_out,
                                __half* y_out, int row_base, int count, int K, float eps,
                                int zero_centered, cudaStream_t stream) {
  if (inbox == nullptr || inbox->tp < 1 || inbox->tp > TP_MAX || row_base < 0 || count < 1 ||
      row_base + count > inbox->rows_cap)
    return -1;
  InboxIn in{};
  in.inbox = reinterpret_cast<const __half*>(inbox->inbox);
  in.flag = inbox->flag;
  in.seen = inbox->seen;
  in.ticket = inbox->ticket;
  in.tp = inbox->tp;
  in.rows_cap = inbox->rows_cap;
  return act_prep_launch(nullptr, resid, norm_w, signs, q_out, scale_out, y_out, count, K, eps,
                         zero_centered, 0, in, stream, AgOut{}, nullptr, row_base);
}

// inbox == nullptr: the branch output of the owned rows is the local matrix x (indexed by
// global row), e.g. the combined expert output of a token-sharded MoE layer.
int orinfer_act_prep_sp(const OrinferInbox* inbox, const OrinferAgOut* agp, float* resid,
                        const __half* norm_w, const int8_t* signs, int rows, int K, float eps,
                        int zero_centered, cudaStream_t stream, const __half* x) {
  if (agp == nullptr || agp->tp < 1 || agp->tp > TP_MAX || agp->rows_per < 1 || K % 16 ||
      static_cast<long long>(agp->rows_per) * agp->tp < rows)
    return -1;
  if (inbox == nullptr && x == nullptr) return -1;
  if (inbox != nullptr && (agp->tp != inbox->tp || rows > inbox->rows_cap)) return -1;
  InboxIn in{};
  if (inbox != nullptr) {
    in.inbox = reinterpret_cast<const __half*>(inbox->inbox);
    in.flag = inbox->flag;
    in.seen = inbox->seen;
    in.ticket = inbox->ticket;
    in.tp = inbox->tp;
    in.rows_cap = inbox->rows_cap;
  }
  AgOut ag;
  for (int i = 0; i < TP_MAX; ++i) {
    ag.q[i] = reinterpret_cast<int8_t*>(agp->q[i]);
    ag.scale[i] = agp->scale[i];
    ag.flag[i] = agp->flag[i];
  }
  ag.sent = agp->sent;
  ag.ticket = agp->ticket;
  ag.tp = agp->tp;
  ag.rank = agp->rank;
  ag.rows_per = agp->rows_per;
  return act_prep_launch(inbox != nullptr ? nullptr : x, resid, norm_w, signs, nullptr, nullptr,
                         nullptr, rows, K, eps, zero_centered, 0, in, stream, ag);
}

int orinfer_ag_wait(const OrinferAgIn* agp, int rows, cudaStream_t stream) {
  if (agp == nullptr || agp->tp < 1 || agp->tp > TP_MAX || agp->rows_per < 1 || rows < 1) return -1;
  if (runtime_ensure_init() != cudaSuccess) return -2;
  AgIn in{agp->flag, agp->sent, agp->tp, agp->rows_per};
  ag_wait_kernel<<<1, 32, 0, stream>>>(in, rows, runtime_status_ptr());
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"

static int act_prep_launch(const __half* x, float* resid, const __half* norm_w, const int8_t* signs,
                           int8_t* q_out, float* scale_out, __half* y_out, int rows, int K,
                           float eps, int zero_centered, int swiglu, InboxIn in,
                           cudaStream_t stream, AgOut ag, const int* row_limit, int row_base) {
  if (rows <= 0) return 0;
  if (runtime_ensure_init() != cudaSuccess) return -2;
  int* status = runtime_status_ptr();
  if (K % 128) return -1;
  if (norm_w != nullptr && K / 128 > MAX_NORM_BLOCKS) return -1;
  const size_t smem = static_cast<size_t>(K) * sizeof(float);
  static const int slot = runtime_new_slot();
  if (runtime_first_use(slot)) {
    cudaFuncSetAttribute(act_prep_kernel<true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         200 * 1024);
    cudaFuncSetAttribute(act_prep_kernel<false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         200 * 1024);
  }
  if (smem > 200 * 1024) return -1;
  // A few rows (decode steps): one row would keep a single SM busy, so a cluster of CTAs
  // shares each row.  Not for the sequence-parallel and count-limited forms, whose CTAs may
  // leave early.
  constexpr int CL = 8;
  if (rows <= 16 && ag.tp == 0 && row_limit == nullptr && K / 128 >= CL) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows * CL);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = (static_cast<size_t>(K / 128 + CL - 1) / CL) * 128 * sizeof(float);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CL;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const AgOut no_ag{};
    const int* no_limit = nullptr;
    cudaError_t e;
    if (swiglu) {
      float* no_resid = nullptr;
      const __half* no_norm = nullptr;
      e = cudaLaunchKernelEx(&cfg, act_prep_kernel<true, CL>, x, no_resid, no_norm, signs, q_out,
                             scale_out, y_out, K, eps, zero_centered, in, status, no_ag, rows,
                             no_limit, 0);
    } else {
      e = cudaLaunchKernelEx(&cfg, act_prep_kernel<false, CL>, x, resid, norm_w, signs, q_out,
                             scale_out, y_out, K, eps, zero_centered, in, status, no_ag, rows,
                             no_limit, row_base);
    }
    return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
  }
  // Thousands of plain rows of moderate width: one warp per row, the row in registers.  With
  // fewer rows there are too few warps in flight to hide the latency of a row's loads, and
  // the CTA-per-row kernel below is more than twice as fast (512 rows of 2560: 11 us
  // against 27 us).
  if (!swiglu && rows >= 2048 && ag.tp == 0 && row_limit == nullptr && in.inbox == nullptr &&
      in.ll == nullptr && row_base == 0 && q_out != nullptr && scale_out != nullptr) {
#define WARP_ROWS(NB)                                                                         \
  if (K == NB * 128) {                                                                        \
    act_prep_warp_kernel<NB><<<(rows + 3) / 4, 128, 0, stream>>>(                             \
        x, resid, norm_w, signs, q_out, scale_out, y_out, rows, eps, zero_centered);          \
    return static_cast<int>(cudaGetLastError());                                              \
  }
    WARP_ROWS(2) WARP_ROWS(8) WARP_ROWS(16) WARP_ROWS(20) WARP_ROWS(32) WARP_ROWS(40)
#undef WARP_ROWS
  }
  // SwiGLU rows are wide and spend their time in exp / divide: more threads per row
  const int threads = swiglu && K >= 4096 ? 512 : 256;
  if (swiglu)
    act_prep_kernel<true, 1><<<rows, threads, smem, stream>>>(x, nullptr, nullptr, signs, q_out,
                                                          scale_out, y_out, K, eps, zero_centered,
                                                          in, status, AgOut{}, rows, row_limit, 0);
  else
    act_prep_kernel<false, 1><<<ag.tp > 0 ? ag.rows_per : rows, 256, smem, stream>>>(
        x, resid, norm_w, signs, q_out, scale_out, y_out, K, eps, zero_centered, in, status, ag,
        rows, row_limit, row_base);
  return static_cast<int>(cudaGetLastError());
}

extern "C" {

int orinfer_rope_table(const int* positions, float* cosb, float* sinb, int rows, int head_dim,
                       double theta, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int total = rows * (head_dim / 2);
  rope_table_kernel<<<(total + 255) / 256, 256, 0, stream>>>(positions, cosb, sinb, rows,
                                                             head_dim / 2, theta);
  return static_cast<int>(cudaGetLastError());
}

int orinfer_qk_rope_kv(const __half* qkv, const __half* wq, const __half* wk, const float* cosb,
                       const float* sinb, const int* row_req, const int* row_pos,
                       const int* page_table, int max_pages, int rows, int qh, int kvh,
                       int head_dim, int gated, float eps, int zero_centered, __half* q_out,
                       __half* gate_out, int8_t* kcache, int8_t* vcache, __half* kscale,
                       __half* vscale, int num_pages, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (runtime_ensure_init() != cudaSuccess) return -2;
  const int heads = qh + 2 * kvh;
  dim3 grid(rows, (heads + 7) / 8);
  int* st = runtime_status_ptr();
#define LAUNCH(DD, GG)                                                                          \
  qk_rope_kv_kernel<DD, GG><<<grid, 256, 0, stream>>>(                                          \
      qkv, wq, wk, cosb, sinb, row_req, row_pos, page_table, max_pages, qh, kvh, eps,           \
      zero_centered, q_out, gate_out, kcache, vcache, kscale, vscale, num_pages, st)
  if (head_dim == 64 && !gated) LAUNCH(64, false);
  else if (head_dim == 64 && gated) LAUNCH(64, true);
  else if (head_dim == 128 && !gated) LAUNCH(128, false);
  else if (head_dim == 128 && gated) LAUNCH(128, true);
  else if (head_dim == 256 && !gated) LAUNCH(256, false);
  else if (head_dim == 256 && gated) LAUNCH(256, true);
  else return -1;
#undef LAUNCH
  return static_cast<int>(cudaGetLastError());
}

int orinfer_argmax_parts(int vocab) { return vocab >= 65536 ? 64 : (vocab >= 4096 ? 8 : 1); }

int orinfer_argmax(const float* logits, int rows, int vocab, float* scratch_val, int* scratch_idx,
                   int* token, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int parts = orinfer_argmax_parts(vocab);
  argmax_partial_kernel<<<dim3(parts, rows), 256, 0, stream>>>(logits, vocab, parts, scratch_val,
                                                               scratch_idx);
  argmax_merge_kernel<<<rows, 32, 0, stream>>>(scratch_val, scratch_idx, parts, token);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
