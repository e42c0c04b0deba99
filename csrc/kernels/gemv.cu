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

// FMT 1: Q4 (U32 codes, 8 rows per group, 4 lanes per row); FMT 2: Q2 (U16 codes, 16 rows,
// 2 lanes).  CTAs are persistent over row groups (decode tables and activations are staged
// once); inside a group the 8 warps split the k-blocks, and every lane keeps DEPTH 16-byte
// code loads of the next batch in flight while it decodes the current one.
// Decode tables replicated COPIES times with the copies interleaved word by word, so that
// lane l always reads copy l % COPIES.  The lookups of a warp are random in the entry index;
// with one copy they collide on the 32 banks about 3.5-fold, which made the kernel
// shared-memory bound.  With 16 interleaved copies only the two lanes sharing a copy can
// collide (entry parity equal), so a lookup costs ~1.5 wavefronts instead of ~3.5.
// A single row (MT = 1) keeps one copy: its launch is so short that filling 48 KiB of tables
// per CTA costs more than the conflicts it removes (measured: 19.9 us vs 22.2 us at
// N = 19456, K = 2560), while 8 rows gain 20 % (38 us -> 30 us).
template <int COPIES>
struct E8pBanked {
  uint32_t posx[256 * COPIES], posy[256 * COPIES], sel[256 * COPIES];
};

template <int COPIES>
__device__ __forceinline__ void banked_init(E8pBanked<COPIES>* sm,
                                            const E8pTables* __restrict__ g, int tid,
                                            int nthreads) {
  for (int j = tid; j < 256 * COPIES; j += nthreads) {
    const int i = j / COPIES;
    const uint2 p = g->pos[i];
    sm->posx[j] = p.x;
    sm->posy[j] = p.y;
    const uint32_t t = static_cast<uint32_t>(i) ^ (__popc(i) & 1u), t2 = t >> 2;
    const uint32_t lo = 0x3210u | ((t & 0x11u) << 2) | ((t & 0x22u) << 9);
    const uint32_t hi = 0x3210u | ((t2 & 0x11u) << 2) | ((t2 & 0x22u) << 9);
    sm->sel[j] = lo | (hi << 16);
  }
}

template <int COPIES>
__device__ __forceinline__ void banked_select(uint32_t code,
                                              const E8pBanked<COPIES>* __restrict__ sm, int copy,
                                              uint32_t& lo, uint32_t& hi, uint32_t& par) {
  const uint32_t s = code & 0xffu;
  par = __popc(s) & 1u;
  const uint32_t at = ((code >> 8) & 0xffu) * COPIES + copy;
  const uint32_t ex = sm->posx[at], ey = sm->posy[at];
  const uint32_t sl = sm->sel[s * COPIES + copy];
  lo = __byte_perm(ex, 0x30303030u - ex, sl);
  hi = __byte_perm(ey, 0x30303030u - ey, sl >> 16);
}

template <int COPIES>
__device__ __forceinline__ uint2 banked_decode8(uint32_t code,
                                                const E8pBanked<COPIES>* __restrict__ sm,
                                                int copy) {
  uint32_t lo, hi, par;
  banked_select(code, sm, copy, lo, hi, par);
  const uint32_t cw = 0x69696969u - par * 0x02020202u;
  return make_uint2((lo + cw) ^ 0x80808080u, (hi + cw) ^ 0x80808080u);
}

template <int COPIES>
__device__ __forceinline__ uint2 banked_decode_q4(uint32_t word,
                                                  const E8pBanked<COPIES>* __restrict__ sm,
                                                  int copy) {
  uint32_t l0, h0, p0, l1, h1, p1;
  banked_select(word & 0xffffu, sm, copy, l0, h0, p0);
  banked_select(word >> 16, sm, copy, l1, h1, p1);
  const uint32_t cw = 0x0d0d0d0du - p0 * 0x08080808u - p1 * 0x02020202u;
  return make_uint2(((l0 << 2) + l1 + cw) ^ 0x80808080u, ((h0 << 2) + h1 + cw) ^ 0x80808080u);
}

template <int FMT, int MT>
__global__ void __launch_bounds__(GEMV_WARPS * 32) e8p_gemv_kernel(
    const int8_t* __restrict__ a, const float* __restrict__ a_scale, const uint4* __restrict__ w,
    const __half* __restrict__ w_scale, void* __restrict__ out, int M, int N, int K, int out_f32,
    const E8pTables* __restrict__ tables, PeerOut po) {
  constexpr int ROWS = FMT == 1 ? 8 : 16;
  constexpr int LPR = 32 / ROWS;                 // lanes per row
  constexpr int WPL = 128 / LPR;                 // weights per lane per k-block
  constexpr int DEPTH = 4;
  const PeerOut* peer = po.tp > 0 ? &po : nullptr;
  const bool ll = peer != nullptr && po.rows_per == LL_MODE;
  const int ll_seq = ll ? *reinterpret_cast<volatile int*>(po.sent) + 1 : 0;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int COPIES = MT == 1 ? 1 : 16;
  using Table = E8pBanked<COPIES>;
  Table* table = reinterpret_cast<Table*>(smem_raw);
  int8_t* act = reinterpret_cast<int8_t*>(smem_raw) + sizeof(Table);
  __shared__ int red[2][GEMV_WARPS][ROWS][MT];

  banked_init(table, tables, threadIdx.x, blockDim.x);
  const int copy = threadIdx.x & (COPIES - 1);
  stage_activations<MT>(act, a, M, K);
  __syncthreads();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = lane / LPR, part = lane % LPR;
  const int kblocks = K / 128;
  const int groups = (N + ROWS - 1) / ROWS;
  int acc[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m] = 0;

  // position of this warp in its (group, k-block batch) sequence
  int g = blockIdx.x, kb0 = warp, parity = 0;
  auto load_batch = [&](int gg, int kk, uint4 (&dst)[DEPTH]) {
    const int n = min(gg * ROWS + row, N - 1);
#pragma unroll
    for (int i = 0; i < DEPTH; ++i) {
      const int kb = kk + GEMV_WARPS * i;
      dst[i] = make_uint4(0, 0, 0, 0);
      if (gg < groups && kb < kblocks)
        dst[i] = __ldg(w + (static_cast<size_t>(kb) * N + n) * LPR + part);
    }
  };
  uint4 cur[DEPTH], nxt[DEPTH];
  load_batch(g, kb0, cur);
  while (g < groups) {
    int ng = g, nkb = kb0 + GEMV_WARPS * DEPTH;
    if (nkb >= kblocks) {
      ng = g + gridDim.x;
      nkb = warp;
    }
    load_batch(ng, nkb, nxt);
#pragma unroll
    for (int i = 0; i < DEPTH; ++i) {
      const int kb = kb0 + GEMV_WARPS * i;
      if (kb < kblocks) {
        const int8_t* abase = act + kb * 128 + part * WPL;
        const uint32_t words[4] = {cur[i].x, cur[i].y, cur[i].z, cur[i].w};
        if (FMT == 1) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint2 q = banked_decode_q4(words[j], table, copy);
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              const int2 av = *reinterpret_cast<const int2*>(abase + m * K + j * 8);
              acc[m] = __dp4a(static_cast<int>(q.x), av.x, acc[m]);
              acc[m] = __dp4a(static_cast<int>(q.y), av.y, acc[m]);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t code = (words[j >> 1] >> ((j & 1) * 16)) & 0xffffu;
            const uint2 q = banked_decode8(code, table, copy);
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              const int2 av = *reinterpret_cast<const int2*>(abase + m * K + j * 8);
              acc[m] = __dp4a(static_cast<int>(q.x), av.x, acc[m]);
              acc[m] = __dp4a(static_cast<int>(q.y), av.y, acc[m]);
            }
          }
        }
      }
    }
    if (ng != g) {
      // group finished: combine lanes, then warps (double-buffered, one barrier per group)
#pragma unroll
      for (int m = 0; m < MT; ++m) {
#pragma unroll
        for (int o = 1; o < LPR; o <<= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
        if (part == 0) red[parity][warp][row][m] = acc[m];
        acc[m] = 0;
      }
      __syncthreads();
      const int n0 = g * ROWS;
      if (peer != nullptr && n0 + ROWS <= N) {
        // peers get whole 16-byte segments (8 consecutive outputs of one row per store):
        // 2-byte remote stores would each become their own NVLink write
        for (int i = threadIdx.x; i < (ROWS / 8) * MT; i += blockDim.x) {
          const int m = i % MT, seg = i / MT;
          if (m < M) {
            __align__(16) __half h[8];
            const float sa = a_scale[m];
#pragma unroll
            for (int r = 0; r < 8; ++r) {
              int total = 0;
#pragma unroll
              for (int wv = 0; wv < GEMV_WARPS; ++wv) total += red[parity][wv][seg * 8 + r][m];
              h[r] = __float2half_rn(
                  (static_cast<float>(total) * __half2float(w_scale[n0 + seg * 8 + r])) * sa);
            }
            if (ll) {
              ll_store8(po, ll_seq, m, n0 + seg * 8, N, h);
            } else {
              const size_t off =
                  (static_cast<size_t>(po.rank) * po.rows_cap + m) * N + n0 + seg * 8;
              for (int d = 0; d < po.tp; ++d)
                *reinterpret_cast<int4*>(po.inbox[d] + off) = *reinterpret_cast<const int4*>(h);
            }
          }
        }
      } else {
        for (int i = threadIdx.x; i < ROWS * MT; i += blockDim.x) {
          const int r = i / MT, m = i % MT;
          if (n0 + r < N && m < M) {
            int total = 0;
#pragma unroll
            for (int wv = 0; wv < GEMV_WARPS; ++wv) total += red[parity][wv][r][m];
            store_row<MT>(out, out_f32, m, n0 + r, N, total, __half2float(w_scale[n0 + r]),
                          a_scale[m], peer);
          }
        }
      }
      parity ^= 1;
    }
    g = ng;
    kb0 = nkb;
#pragma unroll
    for (int i = 0; i < DEPTH; ++i) cur[i] = nxt[i];
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

template <int FMT, int MT>
static int launch_e8p(const int8_t* a, const float* as, const void* w, const __half* ws, void* out,
                      int M, int N, int K, int out_f32, cudaStream_t stream, const PeerOut& po) {
  constexpr int ROWS = FMT == 1 ? 8 : 16;
  const size_t smem = sizeof(E8pBanked<(MT == 1 ? 1 : 16)>) + static_cast<size_t>(MT) * K;
  if (smem > 200 * 1024) return -1;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(e8p_gemv_kernel<FMT, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         200 * 1024);
    attr = true;
  }
  const int groups = (N + ROWS - 1) / ROWS;
  const int per_sm = smem > 110 * 1024 ? 1 : (smem > 72 * 1024 ? 2 : (smem > 54 * 1024 ? 3 : 4));
  const int grid = groups < 148 * per_sm ? groups : 148 * per_sm;
  e8p_gemv_kernel<FMT, MT><<<grid, GEMV_WARPS * 32, smem, stream>>>(
      a, as, reinterpret_cast<const uint4*>(w), ws, out, M, N, K, out_f32, runtime_e8p_tables(),
      po);
  return static_cast<int>(cudaGetLastError());
}

template <int MT>
static int launch_w8(const int8_t* a, const float* as, const void* w, const __half* ws, void* out,
                     int M, int N, int K, int out_f32, cudaStream_t stream, const PeerOut& po) {
  const size_t smem = static_cast<size_t>(MT) * K;
  if (smem > 200 * 1024) return -1;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(w8_gemv_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         200 * 1024);
    attr = true;
  }
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

}  // namespace orinfer
