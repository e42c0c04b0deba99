// Small-M quantised GEMM (decode path, M <= 8): weight-bandwidth bound.  Each CTA
// owns a few output rows and streams their codes once; warps split K, lanes decode
// E8P codes through a shared-memory value table and accumulate with dp4a against
// the INT8 activations staged in shared memory.  Replaces the reference's dp4a /
// gemv projections (kernels/cuda/model/integer_core.py:275,
// kernels/cuda/model/integer_vq.py:381 integer_e8p_gemv,
// kernels/cuda/model/int8_projection.py:66).
#include "api.h"
#include "common.cuh"
#include "tp_comm.cuh"

namespace orinfer {

constexpr int GEMV_WARPS = 8;

template <int MT>
__device__ __forceinline__ void stage_activations(int8_t* dst, const int8_t* __restrict__ a, int M,
                                                  int K) {
  const int chunks = MT * K / 16;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    const int m = (c * 16) / K;
    int4 v = make_int4(0, 0, 0, 0);
    if (m < M) v = *reinterpret_cast<const int4*>(a + static_cast<size_t>(c) * 16);
    *reinterpret_cast<int4*>(dst + static_cast<size_t>(c) * 16) = v;
  }
}

template <int MT>
__device__ __forceinline__ void store_row(void* out, int out_f32, int m, int n, int N, int acc,
                                          float sw, float sa, const PeerOut* po = nullptr) {
  const float v = (static_cast<float>(acc) * sw) * sa;
  if (po != nullptr) {
    // partial result -> slot [rank] of every rank's inbox (plain peer stores over NVLink)
    const __half hv = __float2half_rn(v);
    const size_t off = (static_cast<size_t>(po->rank) * po->rows_cap + m) * N + n;
    for (int d = 0; d < po->tp; ++d) po->inbox[d][off] = hv;
    return;
  }
  if (out_f32) reinterpret_cast<float*>(out)[static_cast<size_t>(m) * N + n] = v;
  else reinterpret_cast<__half*>(out)[static_cast<size_t>(m) * N + n] = __float2half_rn(v);
}

// FMT 1: Q4 (U32 codes, 8 output rows per group, 4 lanes per row); FMT 2: Q2 (U16 codes, 16
// rows, 2 lanes).  One persistent CTA per SM: the decode tables (32 interleaved copies, so a
// lane's lookups never meet another lane's on a bank) and the activations are staged once.
// The grid is n_parts x k_parts CTAs; a CTA owns a contiguous range of row groups and one
// range of k-blocks, its warps take contiguous runs of (group, k-block) units, every lane
// keeps DEPTH 16-byte code loads in flight, and the partial dot products meet in shared
// memory (integer atomics: exact, so the result does not depend on the order).
//
// The decode never forms the weights.  With v the 4-bit fields of a code (common.cuh), a Q4
// weight is 8*v0 + 2*v1 - 75, so
//     sum_k a_k w_k = 2 * sum_k a_k (4*v0 + v1)_k  -  75 * sum_k a_k
// and the first sum is one dp4a per four weights on bytes built with two masks and one
// multiply-add; sum_k a_k is computed once per activation row while it is staged.  Q2
// likewise with 2*v - 15.
//
// k_parts > 1 (projections too narrow for one CTA per SM): the CTAs of one n-part add their
// integers into a zeroed workspace; the last one to finish (ticket) applies the scales,
// writes the outputs and zeroes what it read.  Launches that use the workspace must not
// overlap on the device (they are issued on one stream).
constexpr int GEMV_COPIES = 32;
constexpr int GEMV_DEPTH = 4;

// Optional fusion of the decode step's row kernels into the projection (at most 8 rows, no
// peers).  `pre` builds the INT8 activations inside every CTA instead of reading them:
//   1: rows = resid (+ x), RMSNorm with norm_w, rotation, A8        (x and norm_w may be null)
//   2: rows = x (FP16 [M, K]), rotation, A8
//   3: rows = SwiGLU of x (FP16 [M, 2K]: gate | up), rotation, A8
// with exactly the arithmetic of act_prep_kernel (same helpers, same order), so a row gives
// the same bits through either path.  Every CTA repeats the (small) row preparation; CTA 0
// also stores what other kernels may read (y_out, q_out, scale_out).  `resid_accum` adds the
// FP16-rounded output into an FP32 matrix: the residual stream then already contains the
// branch output when the next prologue reads it, so no kernel both reads and writes it.
struct GemvFuse {
  int pre;
  const __half* x;
  const float* resid;
  const __half* norm_w;
  const int8_t* signs;
  float eps;
  int zero_centered;
  int8_t* q_out;
  float* scale_out;
  __half* y_out;
  float* resid_accum;
};

template <int MT>
struct GemvThreads {
  static constexpr int value = MT <= 2 ? 1024 : 512;
};

template <int FMT, int MT>
__global__ void __launch_bounds__(GemvThreads<MT>::value, 1) e8p_gemv_kernel(
    const int8_t* __restrict__ a, const float* __restrict__ a_scale, const uint4* __restrict__ w,
    const __half* __restrict__ w_scale, void* __restrict__ out, int M, int N, int K, int out_f32,
    const E8pTables* __restrict__ tables, PeerOut po, int n_parts, int k_parts, int max_groups,
    int* __restrict__ ws, GemvFuse fz) {
  constexpr int THREADS = GemvThreads<MT>::value;
  constexpr int ROWS = FMT == 1 ? 8 : 16;
  constexpr int LPR = 32 / ROWS;                 // lanes per row
  constexpr int WPL = 128 / LPR;                 // weights per lane per k-block
  constexpr int DEPTH = GEMV_DEPTH;
  using Lut = E8pLut<GEMV_COPIES>;
  const PeerOut* peer = po.tp > 0 ? &po : nullptr;
  const bool ll = peer != nullptr && po.rows_per == LL_MODE;
  const int ll_seq = ll ? *reinterpret_cast<volatile int*>(po.sent) + 1 : 0;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  Lut* lut = reinterpret_cast<Lut*>(smem_raw);
  int8_t* act = reinterpret_cast<int8_t*>(smem_raw) + sizeof(Lut);
  int* acc_s = reinterpret_cast<int*>(act + static_cast<size_t>(MT) * K);   // [groups][ROWS][MT]
  int* asum = acc_s + max_groups * ROWS * MT;                                // [MT]
  float* scale_s = reinterpret_cast<float*>(asum + MT);                      // [MT]
  float* fbuf = reinterpret_cast<float*>(                                    // [K], pre only
      (reinterpret_cast<uintptr_t>(scale_s + MT) + 15) & ~static_cast<uintptr_t>(15));
  __shared__ int last_flag;
  __shared__ float red[32];
  __shared__ float blk_sum[128];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  e8p_lut_init(lut, tables, tid, THREADS);
  for (int i = tid; i < max_groups * ROWS * MT + MT; i += THREADS) acc_s[i] = 0;
  __syncthreads();
  if (fz.pre == 0) {
    // stage the activations; their row sums ride along
    const int chunks = MT * K / 16;
    int part_sum[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) part_sum[m] = 0;
    for (int c = tid; c < chunks; c += THREADS) {
      const int m = (c * 16) / K;
      int4 v = make_int4(0, 0, 0, 0);
      if (m < M) v = *reinterpret_cast<const int4*>(a + static_cast<size_t>(c) * 16);
      *reinterpret_cast<int4*>(act + static_cast<size_t>(c) * 16) = v;
      int s = __dp4a(v.x, 0x01010101, 0);
      s = __dp4a(v.y, 0x01010101, s);
      s = __dp4a(v.z, 0x01010101, s);
      s = __dp4a(v.w, 0x01010101, s);
#pragma unroll
      for (int mm = 0; mm < MT; ++mm)
        if (mm == m) part_sum[mm] += s;
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      int s = part_sum[m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (lane == 0 && s != 0) atomicAdd(&asum[m], s);
    }
    if (tid < MT) scale_s[tid] = tid < M ? a_scale[tid] : 0.f;
  } else {
    // build the activations: the row kernels' work, repeated by every CTA
    constexpr int NWP = THREADS / 32;
    const bool first_cta = blockIdx.x == 0;
    for (int m = 0; m < MT; ++m) {
      int8_t* arow = act + static_cast<size_t>(m) * K;
      if (m >= M) {
        for (int i = tid * 16; i < K; i += THREADS * 16)
          *reinterpret_cast<int4*>(arow + i) = make_int4(0, 0, 0, 0);
        continue;
      }
      float* fb = fbuf;                          // one row at a time
      if (fz.pre == 3) {
        const __half* g = fz.x + static_cast<size_t>(m) * 2 * K;
        const __half* u = g + K;
        for (int i = tid * 8; i < K; i += THREADS * 8) {
          const int4 gr = *reinterpret_cast<const int4*>(g + i);
          const int4 ur = *reinterpret_cast<const int4*>(u + i);
          const __half* gh = reinterpret_cast<const __half*>(&gr);
          const __half* uh = reinterpret_cast<const __half*>(&ur);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float gv = __half2float(gh[j]);
            const float sg = __fdiv_rn(1.f, 1.f + expf(-gv));
            fb[i + j] = round_f16(__fmul_rn(__fmul_rn(gv, sg), __half2float(uh[j])));
          }
        }
      } else {
        const __half* xr = fz.x ? fz.x + static_cast<size_t>(m) * K : nullptr;
        const float* rr = (fz.pre == 1 && fz.resid) ? fz.resid + static_cast<size_t>(m) * K
                                                    : nullptr;
        for (int i = tid * 8; i < K; i += THREADS * 8) {
          float v[8];
          if (xr) {
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
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) fb[i + j] = v[j];
        }
        if (fz.norm_w) {
          __syncthreads();
          for (int b = warp; b < K / 128; b += NWP) {
            const float sq = block128_sumsq(fb + b * 128, lane);
            if (lane == 0) blk_sum[b] = sq;
          }
          __syncthreads();
          float total = 0.f;
          for (int b = 0; b < K / 128; ++b) total = __fadd_rn(total, blk_sum[b]);
          const float r = rsqrtf(total / static_cast<float>(K) + fz.eps);
          const float add = fz.zero_centered ? 1.f : 0.f;
          for (int i = tid * 8; i < K; i += THREADS * 8) {
            const int4 wr = *reinterpret_cast<const int4*>(fz.norm_w + i);
            const __half* wh = reinterpret_cast<const __half*>(&wr);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              fb[i + j] = round_f16(__fmul_rn(__fmul_rn(fb[i + j], r), __half2float(wh[j]) + add));
          }
        } else {
          for (int i = tid * 8; i < K; i += THREADS * 8)
#pragma unroll
            for (int j = 0; j < 8; ++j) fb[i + j] = round_f16(fb[i + j]);
        }
      }
      __syncthreads();
      if (fz.y_out != nullptr && first_cta) {
        __half* yr = fz.y_out + static_cast<size_t>(m) * K;
        for (int i = tid * 8; i < K; i += THREADS * 8) {
          __align__(16) __half h[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) h[j] = __float2half_rn(fb[i + j]);
          *reinterpret_cast<int4*>(yr + i) = *reinterpret_cast<const int4*>(h);
        }
      }
      float amax = 0.f;
      if (fz.signs) {
        for (int b = warp; b < K / 128; b += NWP)
          amax = fmaxf(amax, hadamard128_inplace(fb + b * 128, fz.signs + b * 128, lane));
      } else {
        for (int i = tid; i < K; i += THREADS) amax = fmaxf(amax, fabsf(fb[i]));
      }
      amax = block_reduce(amax, red, true);
      const float scale = a8_scale(amax);
      int psum = 0;
      for (int i = tid * 4; i < K; i += THREADS * 4) {
        char4 c;
        c.x = static_cast<signed char>(a8_code(fb[i + 0], scale));
        c.y = static_cast<signed char>(a8_code(fb[i + 1], scale));
        c.z = static_cast<signed char>(a8_code(fb[i + 2], scale));
        c.w = static_cast<signed char>(a8_code(fb[i + 3], scale));
        *reinterpret_cast<char4*>(arow + i) = c;
        if (fz.q_out != nullptr && first_cta)
          *reinterpret_cast<char4*>(fz.q_out + static_cast<size_t>(m) * K + i) = c;
        psum = __dp4a(*reinterpret_cast<const int*>(&c), 0x01010101, psum);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
      if (lane == 0 && psum != 0) atomicAdd(&asum[m], psum);
      if (tid == 0) {
        scale_s[m] = scale;
        if (fz.scale_out != nullptr && first_cta) fz.scale_out[m] = scale;
      }
      __syncthreads();
    }
  }
  __syncthreads();

  const int row = lane / LPR, part = lane % LPR;
  const int kb_all = K / 128;
  const int groups = (N + ROWS - 1) / ROWS;
  const int np = blockIdx.x % n_parts, kp = blockIdx.x / n_parts;
  const int g_lo = static_cast<int>(static_cast<long long>(groups) * np / n_parts);
  const int g_hi = static_cast<int>(static_cast<long long>(groups) * (np + 1) / n_parts);
  const int kb_lo = kb_all * kp / k_parts, kb_hi = kb_all * (kp + 1) / k_parts;
  const int kbs = kb_hi - kb_lo;
  const int units = (g_hi - g_lo) * kbs;
  constexpr int NW = THREADS / 32;
  const int u_lo = static_cast<int>(static_cast<long long>(units) * warp / NW);
  const int u_hi = static_cast<int>(static_cast<long long>(units) * (warp + 1) / NW);

  int acc[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m] = 0;
  const int copy = lane;                                   // GEMV_COPIES == 32

  if (u_lo < u_hi) {
    // (group, k-block) of the unit being loaded, and of the unit being consumed
    int lg = g_lo + u_lo / kbs, lkb = kb_lo + u_lo % kbs;
    int g = lg, kb = lkb;
    uint4 buf[DEPTH];
    auto fetch = [&](int uu) -> uint4 {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (uu < u_hi) {
        const int n = min(lg * ROWS + row, N - 1);
        v = __ldg(w + (static_cast<size_t>(lkb) * N + n) * LPR + part);
        if (++lkb == kb_hi) {
          lkb = kb_lo;
          ++lg;
        }
      }
      return v;
    };
#pragma unroll
    for (int i = 0; i < DEPTH; ++i) buf[i] = fetch(u_lo + i);
    for (int base = u_lo; base < u_hi; base += DEPTH) {
#pragma unroll
      for (int i = 0; i < DEPTH; ++i) {
        const uint4 cur = buf[i];
        buf[i] = fetch(base + i + DEPTH);
        if (base + i < u_hi) {
          const int8_t* abase = act + kb * 128 + part * WPL;
          const uint32_t words[4] = {cur.x, cur.y, cur.z, cur.w};
          if (FMT == 1) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t v0 = e8p_fields<GEMV_COPIES, 0>(words[j], lut, copy);
              const uint32_t v1 = e8p_fields<GEMV_COPIES, 1>(words[j], lut, copy);
              const int xlo = static_cast<int>((v0 & E8P_NIB) * 4u + (v1 & E8P_NIB));
              const int xhi = static_cast<int>(((v0 >> 4) & E8P_NIB) * 4u + ((v1 >> 4) & E8P_NIB));
#pragma unroll
              for (int m = 0; m < MT; ++m) {
                const int2 av = *reinterpret_cast<const int2*>(abase + m * K + j * 8);
                acc[m] = __dp4a(xlo, av.x, acc[m]);
                acc[m] = __dp4a(xhi, av.y, acc[m]);
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t v = (j & 1) ? e8p_fields<GEMV_COPIES, 1>(words[j >> 1], lut, copy)
                                         : e8p_fields<GEMV_COPIES, 0>(words[j >> 1], lut, copy);
              const int xlo = static_cast<int>(v & E8P_NIB);
              const int xhi = static_cast<int>((v >> 4) & E8P_NIB);
#pragma unroll
              for (int m = 0; m < MT; ++m) {
                const int2 av = *reinterpret_cast<const int2*>(abase + m * K + j * 8);
                acc[m] = __dp4a(xlo, av.x, acc[m]);
                acc[m] = __dp4a(xhi, av.y, acc[m]);
              }
            }
          }
          const bool last_of_group = kb + 1 == kb_hi, last_unit = base + i + 1 == u_hi;
          if (last_of_group || last_unit) {
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              int v = acc[m];
#pragma unroll
              for (int o = 1; o < LPR; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
              if (part == 0) atomicAdd(&acc_s[((g - g_lo) * ROWS + row) * MT + m], v);
              acc[m] = 0;
            }
          }
          if (last_of_group) {
            kb = kb_lo;
            ++g;
          } else {
            ++kb;
          }
        }
      }
    }
  }
  __syncthreads();

  // sum_k a_k w_k from the staged integers: Q4 2*acc - 75*S, Q2 2*acc - 15*S
  constexpr int BIAS = FMT == 1 ? 75 : 15;
  const int n_base = g_lo * ROWS;
  const int n_count = min(g_hi * ROWS, N) - n_base;        // output columns of this n-part
  bool finalize = true;
  if (k_parts > 1) {
    // add this CTA's integers to the workspace; the last CTA of the n-part finishes
    for (int i = tid; i < n_count * MT; i += THREADS) {
      const int m = i / n_count, r = i % n_count;
      const int v = acc_s[r * MT + m];
      if (m < M && v != 0) atomicAdd(ws + static_cast<size_t>(m) * GEMV_WS_COLS + n_base + r, v);
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      unsigned int* ticket = reinterpret_cast<unsigned int*>(ws + 8 * GEMV_WS_COLS) + np;
      const unsigned int t = atomicAdd(ticket, 1u);
      last_flag = t == static_cast<unsigned int>(k_parts - 1);
      if (last_flag) *ticket = 0;
    }
    __syncthreads();
    finalize = last_flag != 0;
    if (finalize) {
      __threadfence();
      for (int i = tid; i < n_count * MT; i += THREADS) {
        const int m = i / n_count, r = i % n_count;
        int v = 0;
        if (m < M) {
          int* p = ws + static_cast<size_t>(m) * GEMV_WS_COLS + n_base + r;
          v = __ldcg(p);
          *p = 0;
        }
        acc_s[r * MT + m] = v;
      }
      __syncthreads();
    }
  }
  if (finalize) {
    if (peer != nullptr && n_count % 8 == 0) {
      // peers get whole 16-byte segments (8 consecutive outputs of one row per store):
      // 2-byte remote stores would each become their own NVLink write
      const int segs = n_count / 8;
      for (int i = tid; i < segs * MT; i += THREADS) {
        const int m = i / segs, seg = i % segs;
        if (m < M) {
          __align__(16) __half h[8];
          const float sa = scale_s[m];
          const int bias = BIAS * asum[m];
#pragma unroll
          for (int r = 0; r < 8; ++r) {
            const int total = 2 * acc_s[(seg * 8 + r) * MT + m] - bias;
            h[r] = __float2half_rn(
                (static_cast<float>(total) * __half2float(w_scale[n_base + seg * 8 + r])) * sa);
          }
          if (ll) {
            ll_store8(po, ll_seq, m, n_base + seg * 8, N, h);
          } else {
            const size_t off =
                (static_cast<size_t>(po.rank) * po.rows_cap + m) * N + n_base + seg * 8;
            for (int d = 0; d < po.tp; ++d)
              *reinterpret_cast<int4*>(po.inbox[d] + off) = *reinterpret_cast<const int4*>(h);
          }
        }
      }
    } else {
      for (int i = tid; i < n_count * MT; i += THREADS) {
        const int m = i / n_count, r = i % n_count;
        if (m < M) {
          const int total = 2 * acc_s[r * MT + m] - BIAS * asum[m];
          const float sw = __half2float(w_scale[n_base + r]);
          if (fz.resid_accum != nullptr) {
            const __half hv = __float2half_rn((static_cast<float>(total) * sw) * scale_s[m]);
            float* dst = fz.resid_accum + static_cast<size_t>(m) * N + n_base + r;
            *dst = *dst + __half2float(hv);
            if (out != nullptr)
              reinterpret_cast<__half*>(out)[static_cast<size_t>(m) * N + n_base + r] = hv;
          } else {
            store_row<MT>(out, out_f32, m, n_base + r, N, total, sw, scale_s[m], peer);
          }
        }
      }
    }
  }
  if (ll) ll_done(po, ll_seq, gridDim.x);
  else if (peer != nullptr) peer_signal_done(po, gridDim.x);
}

// W8: one warp per output row, 16 weights per lane per step.
template <int MT>
__global__ void __launch_bounds__(GEMV_WARPS * 32) w8_gemv_kernel(
    const int8_t* __restrict__ a, const float* __restrict__ a_scale, const int8_t* __restrict__ w,
    const __half* __restrict__ w_scale, void* __restrict__ out, int M, int N, int K, int out_f32,
    PeerOut po) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int8_t* act = reinterpret_cast<int8_t*>(smem_raw);
  const PeerOut* peer = po.tp > 0 ? &po : nullptr;
  stage_activations<MT>(act, a, M, K);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * GEMV_WARPS + warp;
  if (n < N) {
  const int8_t* wr = w + static_cast<size_t>(n) * K;
  int acc[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m] = 0;
#pragma unroll 4
  for (int k = lane * 16; k < K; k += 512) {
    const int4 wv = __ldg(reinterpret_cast<const int4*>(wr + k));
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const int4 av = *reinterpret_cast<const int4*>(act + m * K + k);
      acc[m] = __dp4a(wv.x, av.x, acc[m]);
      acc[m] = __dp4a(wv.y, av.y, acc[m]);
      acc[m] = __dp4a(wv.z, av.z, acc[m]);
      acc[m] = __dp4a(wv.w, av.w, acc[m]);
    }
  }
  const float sw = __half2float(w_scale[n]);
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    int v = acc[m];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0 && m < M) store_row<MT>(out, out_f32, m, n, N, v, sw, a_scale[m], peer);
  }
  }
  if (peer != nullptr) peer_signal_done(po, gridDim.x);
}

// Grid shape of the E8P GEMV: n_parts x k_parts CTAs on the 148 SMs.  K is split (2, 4 or
// 8 ways, at least 4 k-blocks each) when whole row groups divide badly over the SMs.
struct GemvGrid {
  int n_parts, k_parts, max_groups;
};
static GemvGrid gemv_grid(int rows_per_group, int N, int K) {
  const int groups = (N + rows_per_group - 1) / rows_per_group, kb = K / 128;
  GemvGrid best{groups < 148 ? groups : 148, 1, 0};
  double best_eff = 0.0;
  for (int kp = 1; kp <= 8; kp *= 2) {
    if (kp > 1 && (kb / kp < 4 || N > GEMV_WS_COLS || 148 / kp > GEMV_WS_TICKETS)) break;
    const int np = groups < 148 / kp ? groups : 148 / kp;
    const int per = (groups + np - 1) / np;
    double eff = (static_cast<double>(groups) / np / per) * (static_cast<double>(np) * kp / 148.0);
    if (kp > 1) eff *= 0.97;                       // the workspace round trip is not free
    if (eff > best_eff + 1e-9) {
      best_eff = eff;
      best = GemvGrid{np, kp, 0};
    }
  }
  best.max_groups = (groups + best.n_parts - 1) / best.n_parts;
  return best;
}

constexpr size_t GEMV_SMEM_LIMIT = 220 * 1024;

// Dynamic shared memory of the E8P GEMV for `mt` staged activation rows.
static size_t e8p_gemv_smem(int fmt, int mt, int N, int K, bool fused) {
  const int rows = fmt == 1 ? 8 : 16;
  const GemvGrid g = gemv_grid(rows, N, K);
  size_t smem = sizeof(E8pLut<GEMV_COPIES>) + static_cast<size_t>(mt) * K +
                (static_cast<size_t>(g.max_groups) * rows * mt + 2 * mt) * sizeof(int) + 16;
  if (fused) smem += static_cast<size_t>(K) * sizeof(float);
  return smem;
}

template <int FMT, int MT>
static int launch_e8p(const int8_t* a, const float* as, const void* w, const __half* ws, void* out,
                      int M, int N, int K, int out_f32, cudaStream_t stream, const PeerOut& po,
                      const GemvFuse& fz = GemvFuse{}) {
  constexpr int ROWS = FMT == 1 ? 8 : 16;
  const GemvGrid g = gemv_grid(ROWS, N, K);
  const size_t smem = e8p_gemv_smem(FMT, MT, N, K, fz.pre != 0);
  if (smem > GEMV_SMEM_LIMIT) return -1;
  static const int slot = runtime_new_slot();
  if (runtime_first_use(slot)) {
    cudaError_t e = cudaFuncSetAttribute(e8p_gemv_kernel<FMT, MT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  e8p_gemv_kernel<FMT, MT><<<g.n_parts * g.k_parts, GemvThreads<MT>::value, smem, stream>>>(
      a, as, reinterpret_cast<const uint4*>(w), ws, out, M, N, K, out_f32, runtime_e8p_tables(),
      po, g.n_parts, g.k_parts, g.max_groups, runtime_gemv_workspace(), fz);
  return static_cast<int>(cudaGetLastError());
}

template <int MT>
static int launch_w8(const int8_t* a, const float* as, const void* w, const __half* ws, void* out,
                     int M, int N, int K, int out_f32, cudaStream_t stream, const PeerOut& po) {
  const size_t smem = static_cast<size_t>(MT) * K;
  if (smem > 200 * 1024) return -1;
  static const int slot = runtime_new_slot();
  if (runtime_first_use(slot))
    cudaFuncSetAttribute(w8_gemv_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         200 * 1024);
  w8_gemv_kernel<MT><<<(N + GEMV_WARPS - 1) / GEMV_WARPS, GEMV_WARPS * 32, smem, stream>>>(
      a, as, reinterpret_cast<const int8_t*>(w), ws, out, M, N, K, out_f32, po);
  return static_cast<int>(cudaGetLastError());
}

int qgemv_dispatch(int fmt, const int8_t* a, const float* as, const void* w, const __half* ws,
                   void* out, int M, int N, int K, int out_f32, cudaStream_t stream,
                   const PeerOut* peer) {
  PeerOut po{};
  if (peer != nullptr) po = *peer;
  if (M < 1 || M > 8 || K % 128) return -1;
  if (fmt != 0) {
    // Very long rows (K above about 19 000 at eight rows): the staged activations of all
    // rows do not fit beside the tables, so the rows go in several launches.
    int fit = 8;
    while (fit > 1 && e8p_gemv_smem(fmt, fit, N, K, false) > GEMV_SMEM_LIMIT) fit /= 2;
    if (M > fit) {
      if (peer != nullptr && peer->tp > 0) return -1;      // row indices of the push would shift
      const size_t out_row = static_cast<size_t>(N) * (out_f32 ? 4 : 2);
      for (int m0 = 0; m0 < M; m0 += fit) {
        const int rows = M - m0 < fit ? M - m0 : fit;
        const int r = qgemv_dispatch(fmt, a + static_cast<size_t>(m0) * K, as + m0, w, ws,
                                     static_cast<char*>(out) + m0 * out_row, rows, N, K, out_f32,
                                     stream, peer);
        if (r) return r;
      }
      return 0;
    }
  }
#define BY_M(FN, ...)                                            \
  (M == 1 ? FN<__VA_ARGS__ 1>(a, as, w, ws, out, M, N, K, out_f32, stream, po)  \
   : M == 2 ? FN<__VA_ARGS__ 2>(a, as, w, ws, out, M, N, K, out_f32, stream, po) \
   : M <= 4 ? FN<__VA_ARGS__ 4>(a, as, w, ws, out, M, N, K, out_f32, stream, po) \
            : FN<__VA_ARGS__ 8>(a, as, w, ws, out, M, N, K, out_f32, stream, po))
  if (fmt == 0) {
    if (K % 16) return -1;
    return BY_M(launch_w8, );
  }
  if (fmt == 1) return BY_M(launch_e8p, 1, );
  if (fmt == 2) return BY_M(launch_e8p, 2, );
#undef BY_M
  return -1;
}

// Projection of at most 8 rows with the row preparation fused in (see GemvFuse); E8P weights.
int qgemv_fused_dispatch(int fmt, const void* w, const __half* ws, void* out, int M, int N, int K,
                         cudaStream_t stream, const GemvFuse& fz) {
  if (M < 1 || M > 8 || K % 128 || fz.pre < 1 || fz.pre > 3 || (fmt != 1 && fmt != 2)) return -1;
  if (fz.norm_w != nullptr && K / 128 > 128) return -1;
  const PeerOut po{};
#define BY_M(F)                                                                                   \
  (M == 1 ? launch_e8p<F, 1>(nullptr, nullptr, w, ws, out, M, N, K, 0, stream, po, fz)            \
   : M == 2 ? launch_e8p<F, 2>(nullptr, nullptr, w, ws, out, M, N, K, 0, stream, po, fz)          \
   : M <= 4 ? launch_e8p<F, 4>(nullptr, nullptr, w, ws, out, M, N, K, 0, stream, po, fz)          \
            : launch_e8p<F, 8>(nullptr, nullptr, w, ws, out, M, N, K, 0, stream, po, fz))
  if (fmt == 1) return BY_M(1);
  return BY_M(2);
#undef BY_M
}

}  // namespace orinfer

using namespace orinfer;

// pre: 1 = resid (+ x) -> RMSNorm(norm_w) -> rotate(signs) -> A8; 2 = x -> rotate -> A8;
// 3 = SwiGLU(x [M, 2K]) -> rotate -> A8.  out: FP16 [M, N] or null; resid_accum: FP32 [M, N]
// that receives += the FP16-rounded output, or null.  Returns -1 when the shape does not fit
// the fused kernel (more than 8 rows, W8 weights, too much shared memory): the caller then
// uses the separate kernels.
extern "C" int orinfer_qgemv_fused(int fmt, int pre, const __half* x, const float* resid,
                                   const __half* norm_w, const int8_t* signs, float eps,
                                   int zero_centered, int8_t* q_out, float* scale_out,
                                   __half* y_out, const void* w, const __half* w_scale, void* out,
                                   float* resid_accum, int M, int N, int K, cudaStream_t stream) {
  if (runtime_ensure_init() != cudaSuccess) return -2;
  if (pre == 1 && resid == nullptr && x == nullptr) return -1;
  if ((pre == 2 || pre == 3) && x == nullptr) return -1;
  const GemvFuse fz{pre, x, resid, norm_w, signs, eps, zero_centered, q_out, scale_out, y_out,
                    resid_accum};
  return qgemv_fused_dispatch(fmt, w, w_scale, out, M, N, K, stream, fz);
}
