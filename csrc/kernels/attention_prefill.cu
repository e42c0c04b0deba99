// Causal GQA flash attention for prefill chunks over the paged INT8 KV cache, on
// tcgen05 tensor cores with TMEM accumulators.
//
// One CTA owns a 128-row query tile: P = 128 / rep consecutive query positions of one
// request times the `rep` query heads that share one KV head (the heads are packed into
// the MMA M axis so each INT8 K/V page is dequantised once for all of them).  Per KV
// page (128 keys = one cache page):
//   * warps 6-9 read the INT8 page and its group-64 FP16 scales straight from global
//     memory, dequantise to FP16 and store K and V as 128-byte-swizzled tiles
//     (K is the K-major B operand of S = Q K^T, V the MN-major B operand of O += P V);
//   * warp 1 issues tcgen05.mma kind::f16: S (128x128 fp32) and O (128xD fp32) live in TMEM;
//   * warps 2-5 own one query row per thread: they read S from TMEM, apply scale and the
//     causal mask, keep the running max / sum, rescale O in TMEM when the max moved,
//     and write P as FP16 into shared memory for the second MMA;
//   * warp 0 loads the Q tile once with a 3-D TMA (d, head, position).
// Head size 256 walks the cache in half pages (KT = 64 keys per step): Q (64 KB), two K and
// two V buffers (32 KB each) and two P buffers then fill the 227 KB of one CTA exactly, and
// S0 | S1 | O (64 + 64 + 256 columns) still fit in TMEM.
// Output is O / sum, optionally times sigmoid(gate), in FP16.  Replaces the prefill
// configurations of causal_attention_int8 and dequantize_attention_kv
// (kernels/cuda/model/attention_rows.py:61-276, kernels/cuda/model/kv_int8.py:210-247).
#include <cuda.h>

#include "api.h"
#include "common.cuh"
#include "tma.h"

namespace orinfer {
namespace fa {

constexpr int THREADS = 320;                 // 10 warps
constexpr int TILE = 128;                    // query rows per CTA and keys per KV step

template <int D>
struct Smem {
  static constexpr int KT = D > 128 ? 64 : 128;          // keys per step
  static constexpr int SUB = TILE * 128;                 // one [128 x 64 fp16] sub-tile (Q, P)
  static constexpr int KSUB = KT * 128;                  // one [KT x 64 fp16] sub-tile (K, V)
  static constexpr int NSUB = D / 64;                    // sub-tiles per operand
  static constexpr int PSUB = KT / 64;                   // sub-tiles of one P buffer
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + NSUB * SUB;       // two K buffers
  static constexpr int V_OFF = K_OFF + 2 * NSUB * KSUB;  // two V buffers
  static constexpr int P_OFF = V_OFF + 2 * NSUB * KSUB;  // two P buffers of 128 x KT fp16
  static constexpr int BAR_OFF = P_OFF + 2 * PSUB * SUB;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
  static_assert(TOTAL <= 227 * 1024, "exceeds the shared memory of one CTA");
};

// Eight INT8 values (two words) -> eight FP16 values times an FP16 scale, exactly
// half(float(q) * float(scale)): build 1152 + q as a half via byte permute, subtract,
// multiply (one rounding, like the fp32 product rounded to half).
__device__ __forceinline__ uint4 dequant8(uint32_t w0, uint32_t w1, __half2 scale2) {
  const __half2 bias = __half2half2(__ushort_as_half(0x6480));     // 1152.0
  uint32_t x0 = w0 ^ 0x80808080u, x1 = w1 ^ 0x80808080u;
  uint32_t h[4];
  h[0] = __byte_perm(x0, 0x64646464u, 0x4140);
  h[1] = __byte_perm(x0, 0x64646464u, 0x4342);
  h[2] = __byte_perm(x1, 0x64646464u, 0x4140);
  h[3] = __byte_perm(x1, 0x64646464u, 0x4342);
  uint4 out;
  uint32_t* o = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __half2 v = *reinterpret_cast<__half2*>(&h[i]);
    v = __hmul2(__hsub2(v, bias), scale2);
    o[i] = *reinterpret_cast<uint32_t*>(&v);
  }
  return out;
}

struct Chunk {            // one prefill chunk of one request
  int row_start;          // first packed row
  int q_len;              // rows in the chunk
  int pos0;               // absolute position of the first row
  int slot;               // row of the page table
};

template <int D>
__global__ void __launch_bounds__(THREADS, 1) attn_prefill_kernel(
    const __grid_constant__ CUtensorMap tmap_q, const Chunk* __restrict__ chunks,
    const int* __restrict__ page_table, int max_pages, const int8_t* __restrict__ kc,
    const int8_t* __restrict__ vc, const __half* __restrict__ ks, const __half* __restrict__ vs,
    const __half* __restrict__ gate, __half* __restrict__ out, int qh, int kvh, int rep,
    int num_pages, int* status) {
  using L = Smem<D>;
  constexpr int NSUB = L::NSUB;
  constexpr int KT = L::KT;
  constexpr int GROUPS = D / 64;
  constexpr uint32_t TMEM_COLS = 512;          // S0 | S1 (128 columns each) | O (D columns)
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* q_full = bars;            // Q tile landed
  uint64_t* kv_ready = bars + 1;      // [2] dequantised K/V buffer filled (128 arrivals)
  uint64_t* s_full = bars + 3;        // [2] S[b] = QK^T finished
  uint64_t* p_ready = bars + 5;       // [2] P[b] written, S[b] consumed, O rescaled (128 arrivals)
  uint64_t* o_done = bars + 7;        // O += PV finished (O may be rescaled)
  uint64_t* kv_free = bars + 8;       // [2] the PV that read K/V buffer b finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Chunk ch = chunks[blockIdx.z];
  const int h = blockIdx.y;                       // kv head
  const int P = TILE / rep;                       // query positions per tile
  const int p_first = blockIdx.x * P;             // first chunk-relative position of this tile
  if (p_first >= ch.q_len) return;
  const int p_count = min(P, ch.q_len - p_first);
  const int last_pos = ch.pos0 + p_first + p_count - 1;
  const int n_tiles = last_pos / KT + 1;          // KV steps that any row of the tile can see

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(&kv_ready[0], 128);
    mbar_init(&kv_ready[1], 128);
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(&p_ready[0], 128);
    mbar_init(&p_ready[1], 128);
    mbar_init(o_done, 1);
    mbar_init(&kv_free[0], 1);
    mbar_init(&kv_free[1], 1);
    mbar_fence_init();
    prefetch_tmap(&tmap_q);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 256;   // S[b] at tmem_s + 128 * b
  const int* pages = page_table + static_cast<size_t>(ch.slot) * max_pages;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, static_cast<uint32_t>(NSUB) * 64 * 2 * rep * P);
      for (int s = 0; s < NSUB; ++s)
        tma_load_3d(smem + L::Q_OFF + s * L::SUB, &tmap_q, q_full, s * 64, h * rep,
                    ch.row_start + p_first);
      mbar_wait(q_full, 0, status, STATUS_TMA_WAIT, 1);     // our copy has landed before exit
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc(1, 0, 0, 0, 0, TILE, KT);
      constexpr uint32_t idesc_o = umma_idesc(1, 0, 0, 0, 1, TILE, D);
      const uint32_t q_addr = smem_u32(smem + L::Q_OFF);
      const uint32_t p_addr = smem_u32(smem + L::P_OFF);
      bool ok = mbar_wait(q_full, 0, status, STATUS_MMA_WAIT, 2);
      // S and P are double buffered: S(j+1) = Q K(j+1)^T is issued before O += P(j) V(j), so
      // the tensor core works on the next scores while the softmax warps turn S(j) into P(j).
      auto issue_qk = [&](int j) -> bool {
        const int b = j & 1;
        if (!mbar_wait(&kv_ready[b], (j >> 1) & 1, status, STATUS_MMA_WAIT, 0x100 | j))
          return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(smem + L::K_OFF + b * NSUB * L::KSUB);
#pragma unroll
        for (int i = 0; i < D / 16; ++i) {
          const uint32_t q_off = (i / 4) * L::SUB + (i % 4) * 32;
          const uint32_t k_off = (i / 4) * L::KSUB + (i % 4) * 32;
          mma_f16_ss(tmem_s + 128 * b, umma_desc(q_addr + q_off, 16, 1024),
                     umma_desc(k_addr + k_off, 16, 1024), idesc_s, i != 0 ? 1u : 0u);
        }
        tc_commit(&s_full[b]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int b = j & 1;
        // S[(j+1)&1] was last read by the softmax of tile j-1, whose p_ready this thread
        // waited for before issuing PV(j-1): program order makes the overwrite safe.
        if (j + 1 < n_tiles) ok = issue_qk(j + 1);
        if (!ok) break;
        const uint32_t v_addr = smem_u32(smem + L::V_OFF + b * NSUB * L::KSUB);
        const uint32_t pj_addr = p_addr + b * L::PSUB * L::SUB;
        ok = mbar_wait(&p_ready[b], (j >> 1) & 1, status, STATUS_MMA_WAIT, 0x200 | j);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int i = 0; i < KT / 16; ++i) {
          const uint32_t a_off = (i / 4) * L::SUB + (i % 4) * 32;
          mma_f16_ss(tmem_o, umma_desc(pj_addr + a_off, 16, 1024),
                     umma_desc(v_addr + i * 2048, L::KSUB, 1024), idesc_o, (j | i) != 0 ? 1u : 0u);
        }
        tc_commit(o_done);
        tc_commit(&kv_free[b]);
      }
    }
  } else if (warp >= 6) {
    // ---------------- dequant warps: INT8 page -> FP16 swizzled K / V tiles
    const int t = threadIdx.x - 192;                 // 0..127
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int b = j & 1;
      int page = pages[j * KT / TILE];
      const int key_base = j * KT % TILE;            // first key of this step inside the page
      if (page < 0 || page >= num_pages) {
        report_status(status, STATUS_BAD_INDEX, 3);
        page = 0;
      }
      unsigned char* kb = smem + L::K_OFF + b * NSUB * L::KSUB;
      unsigned char* vb = smem + L::V_OFF + b * NSUB * L::KSUB;
      constexpr int CPK = D / 16;                    // 16-byte chunks per key
      constexpr int ITERS = KT * CPK / 128;
      // every load of the page is issued before the first conversion: one memory round trip
      // per page instead of one per pair of chunks (the 128 dequant threads have no other
      // way to hide latency)
      uint4 kraw[ITERS], vraw[ITERS];
      __half ksc[ITERS], vsc[ITERS];
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        const int idx = it * 128 + t;
        const int key = idx / CPK, c = idx % CPK;
        const size_t slot = (static_cast<size_t>(page) * 128 + key_base + key) * kvh + h;
        kraw[it] = __ldg(reinterpret_cast<const uint4*>(kc + slot * D + c * 16));
        vraw[it] = __ldg(reinterpret_cast<const uint4*>(vc + slot * D + c * 16));
        ksc[it] = ks[slot * GROUPS + c / 4];
        vsc[it] = vs[slot * GROUPS + c / 4];
      }
      // buffer b was last read by the MMAs of tile j-2: wait for its PV to finish.  A
      // per-buffer barrier is used because a waiter two phases behind a shared barrier
      // would alias its parity.
      if (j >= 2)
        ok = mbar_wait(&kv_free[b], ((j >> 1) - 1) & 1, status, STATUS_DECODE_WAIT, j);
      if (!ok) break;
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        const int idx = it * 128 + t;
        const int key = idx / CPK, c = idx % CPK;
        const __half2 k2 = __half2half2(ksc[it]), v2 = __half2half2(vsc[it]);
        const int sub = c / 4, chunk = (c % 4) * 2;
        unsigned char* kd = kb + sub * L::KSUB;
        unsigned char* vd = vb + sub * L::KSUB;
        *reinterpret_cast<uint4*>(kd + swz128(key, chunk)) = dequant8(kraw[it].x, kraw[it].y, k2);
        *reinterpret_cast<uint4*>(kd + swz128(key, chunk + 1)) =
            dequant8(kraw[it].z, kraw[it].w, k2);
        *reinterpret_cast<uint4*>(vd + swz128(key, chunk)) = dequant8(vraw[it].x, vraw[it].y, v2);
        *reinterpret_cast<uint4*>(vd + swz128(key, chunk + 1)) =
            dequant8(vraw[it].z, vraw[it].w, v2);
      }
      fence_proxy_async();
      mbar_arrive(&kv_ready[b]);
    }
  } else {
    // ---------------- softmax warps: one query row per thread
    const int quad = warp & 3;
    const int row = quad * 32 + lane;                       // row of the tile = TMEM lane
    const int p_rel = row / rep, head = h * rep + row % rep;
    const bool valid = p_rel < p_count;
    const int q_pos = valid ? ch.pos0 + p_first + p_rel : -1;
    const float scale = rsqrtf(static_cast<float>(D)) * 1.4426950408889634f;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int sb = j & 1;
      const uint32_t tmem_sj = tmem_s + 128 * sb;
      unsigned char* pb = smem + L::P_OFF + sb * L::PSUB * L::SUB;
      ok = mbar_wait(&s_full[sb], (j >> 1) & 1, status, STATUS_EPILOGUE_WAIT, j);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int key0 = j * KT;
      // Only the last page of a row can hold keys beyond its position; every earlier page
      // takes the mask-free path (one FMNMX per score here, FFMA + EX2 per score below).
      const bool full = key0 + KT - 1 <= q_pos;
      // pass 1: row maximum (of the raw scores: the scale is positive)
      float m_raw = -INFINITY;
#pragma unroll 1
      for (int c0 = 0; c0 < KT; c0 += 64) {
        uint32_t r[32], r2[32];                           // two TMEM loads in flight
        tmem_ld_32x32(tmem_sj + lane_addr + c0, r);
        tmem_ld_32x32(tmem_sj + lane_addr + c0 + 32, r2);
        tc_wait_ld();
        if (full) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            m_raw = fmaxf(m_raw, fmaxf(__uint_as_float(r[i]), __uint_as_float(r2[i])));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (key0 + c0 + i <= q_pos) m_raw = fmaxf(m_raw, __uint_as_float(r[i]));
            if (key0 + c0 + 32 + i <= q_pos) m_raw = fmaxf(m_raw, __uint_as_float(r2[i]));
          }
        }
      }
      const float m_tile = m_raw * scale;               // -inf stays -inf
      const float m_new = fmaxf(m_run, m_tile);
      const float corr = (m_new == -INFINITY) ? 1.f : exp2f(m_run - m_new);
      // P buffer and O are free once PV of tile j-1 has finished
      if (j >= 1) {
        ok = mbar_wait(o_done, (j - 1) & 1, status, STATUS_EPILOGUE_WAIT, 0x100 | j);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (!__all_sync(0xffffffffu, corr == 1.f)) {
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_o + lane_addr + c0, r);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * corr);
            tmem_st_32x32(tmem_o + lane_addr + c0, r);
          }
          tc_wait_st();
        }
      }
      // pass 2: probabilities -> FP16 P tile, row sum
      float l_tile = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < KT; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_sj + lane_addr + c0, r);
        tc_wait_ld();
        uint32_t packed[16];
        if (full) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = exp2f(fmaf(__uint_as_float(r[i]), scale, -m_new));
            const float p1 = exp2f(fmaf(__uint_as_float(r[i + 1]), scale, -m_new));
            l_tile += p0 + p1;
            const __half2 hp = __floats2half2_rn(p0, p1);
            packed[i / 2] = *reinterpret_cast<const uint32_t*>(&hp);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = 0.f, p1 = 0.f;
            if (key0 + c0 + i <= q_pos) p0 = exp2f(fmaf(__uint_as_float(r[i]), scale, -m_new));
            if (key0 + c0 + i + 1 <= q_pos)
              p1 = exp2f(fmaf(__uint_as_float(r[i + 1]), scale, -m_new));
            l_tile += p0 + p1;
            const __half2 hp = __floats2half2_rn(p0, p1);
            packed[i / 2] = *reinterpret_cast<const uint32_t*>(&hp);
          }
        }
        // keys c0..c0+31 -> sub-tile c0/64, 16-byte chunks ((c0 % 64) / 8) .. +3
        unsigned char* dst = pb + (c0 / 64) * L::SUB;
        const int chunk0 = (c0 % 64) / 8;
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<uint4*>(dst + swz128(row, chunk0 + q)) =
              make_uint4(packed[q * 4], packed[q * 4 + 1], packed[q * 4 + 2], packed[q * 4 + 3]);
      }
      l_run = l_run * corr + l_tile;
      m_run = m_new;
      tc_fence_before();
      fence_proxy_async();
      mbar_arrive(&p_ready[sb]);
    }
    if (ok) {
      ok = mbar_wait(o_done, (n_tiles - 1) & 1, status, STATUS_EPILOGUE_WAIT, 0x300);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const size_t orow = static_cast<size_t>(ch.row_start + p_first + p_rel) * qh + head;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_o + lane_addr + c0, r);
        tc_wait_ld();
        if (valid) {
          __align__(16) __half hv[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float v = __uint_as_float(r[i]) * inv;
            if (gate) {
              const float g = __half2float(gate[orow * D + c0 + i]);
              v *= __fdiv_rn(1.f, 1.f + expf(-g));
            }
            hv[i] = __float2half_rn(v);
          }
          uint4* o = reinterpret_cast<uint4*>(out + orow * D + c0);
#pragma unroll
          for (int q = 0; q < 4; ++q) o[q] = reinterpret_cast<const uint4*>(hv)[q];
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int D>
int launch(const __half* q, const __half* gate, const Chunk* chunks, int n_chunks, int max_q_len,
           int total_rows, const int* page_table, int max_pages, const int8_t* kc,
           const int8_t* vc, const __half* ks, const __half* vs, __half* out, int qh, int kvh,
           int num_pages, cudaStream_t stream) {
  using L = Smem<D>;
  const int rep = qh / kvh;
  const int P = TILE / rep;
  PFN_encodeTiled enc = runtime_tma_encoder();
  if (!enc) return -3;
  CUtensorMap tq;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(qh),
                        static_cast<cuuint64_t>(total_rows)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(D) * 2, static_cast<cuuint64_t>(qh) * D * 2};
  cuuint32_t box[3] = {64, static_cast<cuuint32_t>(rep), static_cast<cuuint32_t>(P)};
  cuuint32_t estr[3] = {1, 1, 1};
  if (enc(&tq, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<__half*>(q), dims, strides, box,
          estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return -3;
  static const int slot = runtime_new_slot();
  if (runtime_first_use(slot)) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  dim3 grid((max_q_len + P - 1) / P, kvh, n_chunks);
  attn_prefill_kernel<D><<<grid, THREADS, L::TOTAL, stream>>>(
      tq, chunks, page_table, max_pages, kc, vc, ks, vs, gate, out, qh, kvh, rep, num_pages,
      runtime_status_ptr());
  return static_cast<int>(cudaGetLastError());
}

}  // namespace fa
}  // namespace orinfer

using namespace orinfer;

// chunks: int32 [n_chunks, 4] = (row_start, q_len, pos0, page-table row) on the device.
extern "C" int orinfer_attention_prefill(const __half* q, const __half* gate, const int* chunks,
                                         int n_chunks, int max_q_len, int total_rows,
                                         const int* page_table, int max_pages, const int8_t* kc,
                                         const int8_t* vc, const __half* ks, const __half* vs,
                                         __half* out, int qh, int kvh, int head_dim, int num_pages,
                                         cudaStream_t stream) {
  if (n_chunks <= 0 || max_q_len <= 0) return 0;
  if (kvh <= 0 || qh % kvh || qh / kvh > 16) return -1;
  if (runtime_ensure_init() != cudaSuccess) return -2;
  const fa::Chunk* ch = reinterpret_cast<const fa::Chunk*>(chunks);
  if (head_dim == 128)
    return fa::launch<128>(q, gate, ch, n_chunks, max_q_len, total_rows, page_table, max_pages, kc,
                           vc, ks, vs, out, qh, kvh, num_pages, stream);
  if (head_dim == 64)
    return fa::launch<64>(q, gate, ch, n_chunks, max_q_len, total_rows, page_table, max_pages, kc,
                          vc, ks, vs, out, qh, kvh, num_pages, stream);
  if (head_dim == 256)
    return fa::launch<256>(q, gate, ch, n_chunks, max_q_len, total_rows, page_table, max_pages,
                           kc, vc, ks, vs, out, qh, kvh, num_pages, stream);
  return -4;          // unsupported head size: caller falls back to the row kernel
}
