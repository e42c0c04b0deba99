// Quantised GEMM on the 5th-generation tensor cores: out[M,N] = (A8[M,K] . W[N,K]^T) * s_w * s_a.
//
// One CTA computes a (MT*128) x NB output tile: MT = 1, 2 or 4 accumulators in TMEM share
// every decoded weight tile (the lattice decode, not the MMA, is the scarce resource, so a
// weight tile should be decoded once and multiplied against as many rows as the packet has),
// and NB = 128, 64 or 32 weight rows per CTA spreads narrow projections over the 148 SMs.
// Warp 0 streams the activation tiles with TMA and warp 2 the weight side (INT8 weights by
// TMA for W8; the packed E8P codes as one contiguous bulk copy per k-block for Q4/Q2).
// Warps 3-18 expand the lattice codes into an INT8 weight tile in the 128-byte-swizzled
// K-major layout the tensor core reads, warp 1 issues tcgen05.mma kind::i8 into TMEM, and
// warps 3-18 finally read TMEM back, apply the two scales and
// store FP16/FP32.  INT4 tensor-core MMA (the reference's fastest path,
// kernels/cuda/model/e8p_core.py:15-33) does not exist on tcgen05, so both E8P formats go
// through INT8 operands.  Replaces e8p_q4.projection (kernels/cuda/model/e8p_q4.py:144-265),
// integer_vq (kernels/cuda/model/integer_vq.py:263) and int8_projection
// (kernels/cuda/model/int8_projection.py:15).
#include <cuda.h>
#include <mutex>

#include "api.h"
#include "common.cuh"
#include "tma.h"
#include "tp_comm.cuh"

namespace orinfer {

int qgemv_dispatch(int fmt, const int8_t* a, const float* as, const void* w, const __half* ws,
                   void* out, int M, int N, int K, int out_f32, cudaStream_t stream,
                   const PeerOut* peer);

namespace tc {

constexpr int BM = 128, BK = 128;
constexpr int TILE_BYTES = 128 * 128;        // one INT8 activation tile (128 rows x 128 k)
constexpr int PRODUCERS = 512;               // warps 3..18
constexpr int PWARPS = PRODUCERS / 32;
constexpr int NUM_SMS = 148;
// 0: persistent kernel; 1: one tile per CTA (default: the fastest measured so far); 2: CTA
// pairs (cta_group::2) where the shape allows, else persistent.  All give the same bits.
static int g_impl = 1;
static int g_probe = 0;      // timing experiments of the one-tile kernel (see its `probe`)
// warp 0: activation loader, warp 1: MMA issuer, warp 2: weight loader, warps 3..18: lattice
// decode and epilogue.  Each role has a warp of its own: two roles that wait on different
// barriers inside one warp would suspend each other.
constexpr int ROLE_THREADS = 96;
constexpr int THREADS = ROLE_THREADS + PRODUCERS;

template <int FMT, int MT, int NB>
struct Layout {
  static constexpr int ROW_CODE_BYTES = FMT == 1 ? 64 : (FMT == 2 ? 32 : 0);
  static constexpr int CODE_BYTES = NB * ROW_CODE_BYTES;
  static constexpr int B_BYTES = NB * BK;     // INT8 weight tile, 128-byte rows
  // Two rings of different depth: activation tiles are large (MT x 16 KiB per k-block), so
  // they get what is left after the weight side (codes + decoded INT8 tile) is 3-4 deep;
  // the decode then runs ahead of the tensor core while the next activation tiles land.
  static constexpr int A_BYTES = MT * TILE_BYTES;
  static constexpr int BC_BYTES = B_BYTES + CODE_BYTES;
  static constexpr int BUDGET = 216 * 1024;
  static constexpr int SB_FIT = (BUDGET - 2 * A_BYTES) / BC_BYTES;
  static constexpr int SB = SB_FIT >= 4 ? 4 : SB_FIT;
  static constexpr int SA_FIT = (BUDGET - SB * BC_BYTES) / A_BYTES;
  static constexpr int SA = SA_FIT >= 4 ? 4 : SA_FIT;
  static_assert(SA >= 2 && SB >= 2, "at least double buffering");
  static constexpr int LUT_COPIES = 4;
  static constexpr int LUT_BYTES = FMT == 0 ? 0 : static_cast<int>(sizeof(E8pLut<LUT_COPIES>));
  static constexpr int A_OFF = 0;
  static constexpr int B_OFF = A_OFF + SA * A_BYTES;
  static constexpr int CODE_OFF = B_OFF + SB * B_BYTES;
  static constexpr int LUT_OFF = CODE_OFF + SB * CODE_BYTES;
  static constexpr int BAR_OFF = LUT_OFF + LUT_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;   // barriers + alignment slack
  static_assert(TOTAL <= 227 * 1024, "exceeds the shared memory of one CTA");
};

// Grouped (mixture-of-experts) launch: blockIdx.y walks a device-side tile table
// (expert, first row, valid rows); each expert has its own weight bank and row scales.
struct GroupDesc {
  const int* tiles;            // int32 [max_tiles, 4]; nullptr = ordinary GEMM
  const int* meta;             // meta[0] = number of tiles
  long long w_stride;          // bytes between consecutive experts' weight banks
  int n_per_expert;            // rows of one expert's bank (= N)
};

template <int FMT, bool OUT_F32, int MT, int NB>
__global__ void __launch_bounds__(THREADS, 1) qgemm_tc_kernel(
    const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
    const unsigned char* __restrict__ w, const float* __restrict__ a_scale,
    const __half* __restrict__ w_scale, void* __restrict__ out, int M, int N, int K,
    const E8pTables* __restrict__ tables, int* status, PeerOut po, GroupDesc grp, AgIn ag,
    int* __restrict__ partial, int* __restrict__ tickets, int n_begin, int n_end, int probe) {
  // probe (timing experiments only; results are then meaningless): bit 0 = issue no MMAs,
  // bit 1 = copy no operands (the loaders only signal), bit 2 = decode nothing, bit 3 = the
  // epilogue stores nothing to global memory, bit 4 = no epilogue at all, bit 5 = no k-blocks,
  // bit 6 = leave at once, bit 7 = no TMEM allocation (with bits 0 and 4), bit 8 = no table copy, bit 9 = accumulators are reinterpreted, not converted
  using L = Layout<FMT, MT, NB>;
  constexpr int SA = L::SA, SB = L::SB;
  constexpr int BN = NB;
  if (probe & 64) return;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* a_s = smem + L::A_OFF;
  unsigned char* b_s = smem + L::B_OFF;
  unsigned char* code_s = smem + L::CODE_OFF;
  using Lut = E8pLut<L::LUT_COPIES>;
  Lut* lut = reinterpret_cast<Lut*>(smem + L::LUT_OFF);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* a_full = bars;                   // [SA] activation tiles landed (TMA)
  uint64_t* a_empty = bars + SA;             // [SA] tensor core done with the tiles
  uint64_t* c_full = bars + 2 * SA;          // [SB] packed codes landed (bulk copy)
  uint64_t* b_full = c_full + SB;            // [SB] INT8 weight tile ready (decode or TMA)
  uint64_t* b_empty = c_full + 2 * SB;       // [SB] tensor core done with the weight tile
  uint64_t* tmem_full = c_full + 3 * SB;     // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full + 1);
  int* ticket_slot = reinterpret_cast<int*>(tmem_slot + 1);
  bool writes_output = true;                   // false: another split finishes this tile

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = n_begin + blockIdx.x * BN;    // this launch covers columns [n_begin, n_end)
  int m0 = blockIdx.y * BM * MT, m_limit = M, b_row0 = n0;
  if (grp.tiles != nullptr) {
    if (static_cast<int>(blockIdx.y) >= grp.meta[0]) return;
    const int expert = grp.tiles[blockIdx.y * 4];
    m0 = grp.tiles[blockIdx.y * 4 + 1];
    m_limit = m0 + grp.tiles[blockIdx.y * 4 + 2];
    w += static_cast<long long>(expert) * grp.w_stride;
    w_scale += static_cast<long long>(expert) * grp.n_per_expert;
    b_row0 = expert * grp.n_per_expert + n0;
  }
  // split-K: blockIdx.z owns k-blocks [kb0, kb0 + kblocks).  Every CTA of a tile stores its raw
  // INT32 accumulators into partial[z][tile] and takes a ticket; the CTA that arrives last
  // adds the other splits to its own accumulators and runs the ordinary epilogue, so the
  // result is bit for bit the unsplit one (integer sums) and no second kernel is needed.
  const int kb_all = K / BK, kb_per = (kb_all + gridDim.z - 1) / gridDim.z;
  const int kb0 = blockIdx.z * kb_per;
  const int kblocks = (probe & 32) ? 0 : max(0, min(kb_all, kb0 + kb_per) - kb0);
  const int rows_valid = min(BN, n_end - n0);
  constexpr uint32_t TMEM_COLS = MT * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < SA; ++s) {
      mbar_init(&a_full[s], 1);
      mbar_init(&a_empty[s], 1);
    }
    for (int s = 0; s < SB; ++s) {
      mbar_init(&c_full[s], 1);
      mbar_init(&b_full[s], FMT == 0 ? 1 : PRODUCERS);
      mbar_init(&b_empty[s], 1);
    }
    mbar_init(tmem_full, 1);
    mbar_fence_init();
    prefetch_tmap(&tmap_a);
    if (FMT == 0) prefetch_tmap(&tmap_b);
  }
  if (warp == 1 && !(probe & 128)) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  if (FMT != 0 && warp >= 3 && !(probe & 256)) {
    e8p_lut_init(lut, tables, threadIdx.x - ROLE_THREADS, PRODUCERS);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // peer epilogue staging: one padded FP16 row per output row (pad keeps 16-byte stores of
  // 32 consecutive rows on distinct banks)
  constexpr int STAGE_ROW = BN * 2 + 16;
  static_assert(MT * BM * STAGE_ROW <= L::LUT_OFF, "staged tile must fit in the operand rings");

  if (warp == 0) {
    if (lane == 0) {
      // activation loader
      int issued = 0;
      bool a_ready = true;
      if (ag.tp > 0) {
        // all-gather fused into the GEMM: A rows of this M tile were pushed by their owner
        // ranks; wait for exactly those sources, then order the async-proxy loads after it
        a_ready = ag_wait(ag, m0, min(m0 + MT * BM, M) - 1, status);
        fence_proxy_async_all();
      }
      for (int kb = 0; a_ready && kb < kblocks; ++kb) {
        const int s = kb % SA;
        if (!mbar_wait(&a_empty[s], ((kb / SA) & 1) ^ 1, status, STATUS_TMA_WAIT, kb)) break;
        if (probe & 2) {
          mbar_arrive(&a_full[s]);
        } else {
          mbar_expect_tx(&a_full[s], MT * TILE_BYTES);
#pragma unroll
          for (int t = 0; t < MT; ++t)
            tma_load_2d(a_s + (s * MT + t) * TILE_BYTES, &tmap_a, &a_full[s], (kb0 + kb) * BK,
                        m0 + t * BM);
        }
        issued = kb + 1;
      }
      // Never leave the CTA with a copy of ours in flight: wait (bounded) for the
      // last copies issued into each stage.
      for (int kb = max(0, issued - SA); kb < issued; ++kb)
        mbar_wait(&a_full[kb % SA], (kb / SA) & 1, status, STATUS_TMA_WAIT, 0x4000 | kb);
    }
  } else if (warp == 2) {
    if (lane == 0) {
      // weight loader: INT8 tiles by TMA (W8) or the packed codes as one bulk copy
      int issued = 0;
      uint64_t* landed = FMT == 0 ? b_full : c_full;
      for (int kb = 0; kb < kblocks; ++kb) {
        const int s = kb % SB;
        if (!mbar_wait(&b_empty[s], ((kb / SB) & 1) ^ 1, status, STATUS_TMA_WAIT, 0x1000 | kb))
          break;
        if (probe & 2) {
          mbar_arrive(FMT == 0 ? &b_full[s] : &c_full[s]);
        } else if (FMT == 0) {
          mbar_expect_tx(&b_full[s], L::B_BYTES);
          tma_load_2d(b_s + s * L::B_BYTES, &tmap_b, &b_full[s], (kb0 + kb) * BK, b_row0);
        } else {
          const unsigned char* src =
              w + (static_cast<size_t>(kb0 + kb) * N + n0) * L::ROW_CODE_BYTES;
          mbar_expect_tx(&c_full[s], rows_valid * L::ROW_CODE_BYTES);
          bulk_load(code_s + s * L::CODE_BYTES, src, rows_valid * L::ROW_CODE_BYTES, &c_full[s]);
        }
        issued = kb + 1;
      }
      for (int kb = max(0, issued - SB); kb < issued; ++kb)
        mbar_wait(&landed[kb % SB], (kb / SB) & 1, status, STATUS_TMA_WAIT, 0x5000 | kb);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(2, 1, 1, 0, 0, BM, BN);
      bool ok = true;
      for (int kb = 0; kb < kblocks && ok; ++kb) {
        const int sa = kb % SA, sb = kb % SB;
        ok = mbar_wait(&a_full[sa], (kb / SA) & 1, status, STATUS_MMA_WAIT, kb);
        if (ok) ok = mbar_wait(&b_full[sb], (kb / SB) & 1, status, STATUS_MMA_WAIT, 0x2000 | kb);
        if (!ok) break;
        tc_fence_after();
        const uint32_t b_addr = smem_u32(b_s + sb * L::B_BYTES);
#pragma unroll
        for (int j = 0; j < BK / 32; ++j) {
          if (probe & 1) break;
          const uint64_t bdesc = umma_desc(b_addr + j * 32, 16, 1024);
#pragma unroll
          for (int t = 0; t < MT; ++t) {
            const uint32_t a_addr = smem_u32(a_s + (sa * MT + t) * TILE_BYTES);
            mma_i8_ss(tmem_base + t * BN, umma_desc(a_addr + j * 32, 16, 1024), bdesc, idesc,
                      (kb | j) != 0 ? 1u : 0u);
          }
        }
        tc_commit(&a_empty[sa]);
        tc_commit(&b_empty[sb]);
      }
      if (ok && kblocks > 0) tc_commit(tmem_full);
    }
  } else {
    const int t = threadIdx.x - ROLE_THREADS;                     // 0..511
    bool ok = true;
    if (FMT != 0) {
      const int chunk = t & 7, rbase = t >> 3;          // 64 weight rows per pass
      const int copy = t & (L::LUT_COPIES - 1);
      for (int kb = 0; kb < kblocks; ++kb) {
        const int s = kb % SB;
        // the codes of this phase are only requested after the tensor core released the
        // stage, so their arrival also means the INT8 tile of this stage may be overwritten
        ok = mbar_wait(&c_full[s], (kb / SB) & 1, status, STATUS_DECODE_WAIT, kb);
        if (!ok) break;
        const unsigned char* cs = code_s + s * L::CODE_BYTES;
        unsigned char* bs = b_s + s * L::B_BYTES;
#pragma unroll
        for (int i = 0; i < (BN + 63) / 64; ++i) {
          const int row = rbase + 64 * i;
          if ((BN < 64 && row >= BN) || (probe & 4)) break;
          uint4 v = make_uint4(0, 0, 0, 0);
          if (row < rows_valid) {
            if (FMT == 1) {
              const uint2 wd = *reinterpret_cast<const uint2*>(cs + row * 64 + chunk * 8);
              const uint2 q0 = e8p_decode_q4(wd.x, lut, copy);
              const uint2 q1 = e8p_decode_q4(wd.y, lut, copy);
              v = make_uint4(q0.x, q0.y, q1.x, q1.y);
            } else {
              const uint32_t wd = *reinterpret_cast<const uint32_t*>(cs + row * 32 + chunk * 4);
              const uint2 q0 = e8p_decode8<L::LUT_COPIES, 0>(wd, lut, copy);
              const uint2 q1 = e8p_decode8<L::LUT_COPIES, 1>(wd, lut, copy);
              v = make_uint4(q0.x, q0.y, q1.x, q1.y);
            }
          }
          *reinterpret_cast<uint4*>(bs + swz128(row, chunk)) = v;
        }
        fence_proxy_async();
        mbar_arrive(&b_full[s]);
      }
    }
    const int quad = warp & 3;                          // TMEM lane quadrant of this warp
    const int part = (warp - 3) >> 2;                   // 0..3: which 32-column chunks
    const int row = quad * 32 + lane;
    constexpr int CHUNKS = BN / 32;                     // 32-column chunks per accumulator
    // A warp's items all cover the same 32 columns (4 is a multiple of CHUNKS).  Their weight
    // scales, and the row scales of the warp's rows, are requested before the wait on the
    // accumulators: fetched one FP16 at a time inside the loop, their latency was most of
    // the epilogue (10 of 30 us per 512 x 128 tile).
    const int c_warp = (part % CHUNKS) * 32;
    uint4 wsv[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const int n = n0 + c_warp + g * 8;
      wsv[g] = n + 8 <= n_end ? *reinterpret_cast<const uint4*>(w_scale + n)
                              : make_uint4(0, 0, 0, 0);
    }
    float sa_pre[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int m = m0 + mt * BM + row;
      // gathered row scales are written by peers and only complete once the activation
      // loader has seen their flags: those are read after the accumulators are ready
      sa_pre[mt] = (ag.tp == 0 && m < m_limit) ? a_scale[m] : 0.f;
    }
    if (ok && kblocks > 0) ok = mbar_wait(tmem_full, 0, status, STATUS_EPILOGUE_WAIT, 0);
    ok = __all_sync(0xffffffffu, ok);        // tcgen05.ld needs the whole warp
    constexpr int TILE_INT4 = MT * BM * BN / 4;
    const size_t tile_id = static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x;
    const size_t tiles = static_cast<size_t>(gridDim.x) * gridDim.y;
    if (partial != nullptr && tickets == nullptr) {
      // Large tiles with many splits: the raw accumulators go to partial[z][M][width]
      // (compact over this launch's columns) and a second kernel, spread over all SMs, adds
      // the splits; one CTA reading every other split's tile would take longer than that.
      if (ok) {
        tc_fence_after();
        const int width = n_end - n_begin;
#pragma unroll 1
        for (int item = part; item < MT * CHUNKS; item += 4) {
          const int mt = item / CHUNKS, c0 = (item % CHUNKS) * 32;
          const int m = m0 + mt * BM + row;
          uint32_t r[32];
          if (kblocks > 0) {
            tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + mt * BN + c0, r);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0;         // an empty k range contributes zero
          }
          if (m < m_limit) {
            int* dst = partial + (static_cast<size_t>(blockIdx.z) * M + m) * width +
                       (n0 - n_begin) + c0;
#pragma unroll
            for (int g = 0; g < 8; ++g)
              if (n0 + c0 + g * 4 + 4 <= n_end)
                *reinterpret_cast<int4*>(dst + g * 4) =
                    make_int4(r[g * 4], r[g * 4 + 1], r[g * 4 + 2], r[g * 4 + 3]);
          }
        }
      }
      writes_output = false;
    } else if (partial != nullptr) {
      // Layout inside a tile: [item][group of 4 columns][row] as int4, so a warp instruction
      // writes (and the last arriver reads back) 512 contiguous bytes.
      if (ok) {
        tc_fence_after();
        int4* mine = reinterpret_cast<int4*>(partial) + (blockIdx.z * tiles + tile_id) * TILE_INT4;
#pragma unroll 1
        for (int item = part; item < MT * CHUNKS; item += 4) {
          const int mt = item / CHUNKS, c0 = (item % CHUNKS) * 32;
          uint32_t r[32];
          if (kblocks > 0) {
            tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + mt * BN + c0, r);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0;         // an empty k range contributes zero
          }
#pragma unroll
          for (int g = 0; g < 8; ++g)
            mine[(item * 8 + g) * BM + row] =
                make_int4(r[g * 4], r[g * 4 + 1], r[g * 4 + 2], r[g * 4 + 3]);
        }
      }
      // every producer warp takes part, also after a failed wait, so that the ticket count
      // of the tile stays whole and nobody is left at the barrier
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(PRODUCERS) : "memory");
      if (t == 0) {
        const int ticket = atomicAdd(tickets + tile_id, 1);
        if (ticket == static_cast<int>(gridDim.z) - 1) tickets[tile_id] = 0;
        __threadfence();
        *ticket_slot = ticket;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(PRODUCERS) : "memory");
      writes_output = *reinterpret_cast<volatile int*>(ticket_slot) ==
                      static_cast<int>(gridDim.z) - 1;
    }
    if (ok && writes_output && !(probe & 16)) {
      tc_fence_after();
      // Conversions run at a fraction of the FP32 rate: the 32 weight scales become FP32 once
      // per thread instead of once per item, and results are packed to FP16 two at a time.
      float ws[32];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const __half2* h2 = reinterpret_cast<const __half2*>(&wsv[g]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(h2[j]);
          ws[g * 8 + 2 * j] = f.x;
          ws[g * 8 + 2 * j + 1] = f.y;
        }
      }
#pragma unroll 1
      for (int item = part; item < MT * CHUNKS; item += 4) {
        const int mt = item / CHUNKS, c0 = (item % CHUNKS) * 32;
        const int m = m0 + mt * BM + row;
        // gathered row scales were written by peers: read them past L1
        float sa = 0.f;
#pragma unroll
        for (int q = 0; q < MT; ++q)
          if (q == mt) sa = sa_pre[q];                     // static indexing keeps it in registers
        if (ag.tp > 0 && m < m_limit) sa = __ldcg(a_scale + m);
        uint32_t r[32];
        if (kblocks > 0) {
          tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + mt * BN + c0, r);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0;           // an empty k range contributes zero
        }
        if (partial != nullptr) {
          for (int z = 0; z < static_cast<int>(gridDim.z); ++z) {
            if (z == static_cast<int>(blockIdx.z)) continue;
            const int4* theirs =
                reinterpret_cast<const int4*>(partial) + (z * tiles + tile_id) * TILE_INT4;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              const int4 v = __ldcg(theirs + (item * 8 + g) * BM + row);
              r[g * 4] += v.x; r[g * 4 + 1] += v.y; r[g * 4 + 2] += v.z; r[g * 4 + 3] += v.w;
            }
          }
        }
        if (m < m_limit) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int n = n0 + c0 + g * 8;
            if (n + 8 <= n_end) {
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j)
                v[j] = (((probe & 512) ? __uint_as_float(r[g * 8 + j])
                                       : static_cast<float>(static_cast<int>(r[g * 8 + j]))) *
                        ws[g * 8 + j]) * sa;
              if (po.tp > 0 || !OUT_F32) {
                // step 1: the FP16 tile is staged in the (now idle) operand rings so that it
                // leaves in whole rows: a warp storing 32 rows x 16 bytes straight from its
                // registers touches 32 lines per instruction, which made the epilogue cost
                // more than the main loop; peers get their partial tile the same way
                __align__(16) __half2 h[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
                *reinterpret_cast<int4*>(smem + static_cast<size_t>(mt * BM + row) * STAGE_ROW +
                                         (c0 + g * 8) * 2) = *reinterpret_cast<const int4*>(h);
              } else if (OUT_F32) {
                float* o = reinterpret_cast<float*>(out) + static_cast<size_t>(m) * N + n;
                *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<float4*>(o + 4) = make_float4(v[4], v[5], v[6], v[7]);
              } else {
                __align__(16) __half2 h[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
                __half* o = reinterpret_cast<__half*>(out) + static_cast<size_t>(m) * N + n;
                *reinterpret_cast<int4*>(o) = *reinterpret_cast<const int4*>(h);
              }
            }
          }
        }
      }
    }
  }
  if (warp >= 3 && (po.tp > 0 || !OUT_F32) && writes_output) {
    // step 2: every producer warp joins (also after a failed wait, so that nobody is left at
    // the barrier), then whole 16-byte segments of consecutive columns go out lane by lane:
    // a warp writes two complete 256-byte rows per instruction instead of 32 rows x 16
    // bytes, which keeps memory transactions (and NVLink packets) full.
    asm volatile("bar.sync 1, %0;" ::"n"(PRODUCERS) : "memory");
    constexpr int SEGS = BN / 8;                          // 16-byte segments per row
    const int t = threadIdx.x - ROLE_THREADS;
    for (int idx = t; idx < MT * BM * SEGS; idx += PRODUCERS) {
      const int r = idx / SEGS, seg = idx % SEGS;
      const int m = m0 + r, n = n0 + seg * 8;
      if (m < m_limit && n + 8 <= n_end && !(probe & 24)) {
        const int4 val = *reinterpret_cast<const int4*>(smem + static_cast<size_t>(r) * STAGE_ROW +
                                                        seg * 16);
        if (po.tp == 0) {
          *reinterpret_cast<int4*>(reinterpret_cast<__half*>(out) + static_cast<size_t>(m) * N +
                                   n) = val;
          continue;
        }
        const size_t off = (static_cast<size_t>(po.rank) * po.rows_cap + m) * N + n;
        if (po.rows_per > 0) {
          // reduce-scatter: only the owner of row m receives this partial
          *reinterpret_cast<int4*>(po.inbox[min(m / po.rows_per, po.tp - 1)] + off) = val;
        } else {
          for (int d = 0; d < po.tp; ++d) *reinterpret_cast<int4*>(po.inbox[d] + off) = val;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1 && !(probe & 128)) tmem_dealloc(tmem_base, TMEM_COLS);
  // (with a second pass adding the splits, that pass pushes to the peers and signals)
  if (po.tp > 0 && !(partial != nullptr && tickets == nullptr))
    peer_signal_done(po, gridDim.x * gridDim.y * gridDim.z);
}

// ---------------------------------------------------------------- persistent form
// One CTA per SM walks the tile list (tile = blockIdx.x + i * gridDim.x; m fastest, so the
// CTAs running together share a few weight tiles in L2).  What is paid once per CTA instead
// of once per tile: the decode tables, the TMEM allocation, the barriers and the pipeline
// fill.  Differences from the one-tile kernel above:
//   * activation tiles live in a ring of single 16 KiB slots (8 for MT = 4) with a barrier
//     pair each, so a slot is refilled as soon as its own MMAs retire instead of when the
//     whole MT-tile stage does; all rings and their phases run on across tiles;
//   * packed codes and decoded INT8 tiles have rings of their own depth;
//   * the epilogue of tile i runs while the tensor core already works on tile i+1: the
//     producer warps first decode the k-blocks of tile i+1 that fit in the ring, then drain
//     the accumulators of tile i one at a time, and the MMA warp waits per accumulator
//     (tmem_empty[t]) before it overwrites it;
//   * M sub-tiles past the last row are neither loaded nor multiplied;
//   * every wait polls a CTA-wide abort word, so that all roles leave together when one
//     bounded wait ran out.
// With peers (fused scatter) the FP16 tile is staged in the operand rings as before, so
// the loaders wait for the epilogue before they refill the rings (epi_done).
template <int FMT, int MT, int NB>
struct PsLayout {
  static constexpr int ROW_CODE_BYTES = FMT == 1 ? 64 : (FMT == 2 ? 32 : 0);
  static constexpr int CODE_BYTES = NB * ROW_CODE_BYTES;
  static constexpr int B_BYTES = NB * BK;
  static constexpr int NSLOT = MT == 4 ? 8 : (MT == 2 ? 6 : 4);
  static constexpr int SBD = FMT == 0 ? 4 : 3;          // decoded (or TMA-loaded) weight tiles
  static constexpr int SC = FMT == 0 ? 0 : 3;           // packed-code slabs
  static constexpr int LUT_COPIES = 8;
  static constexpr int LUT_BYTES = FMT == 0 ? 0 : static_cast<int>(sizeof(E8pLut<LUT_COPIES>));
  static constexpr int A_OFF = 0;
  static constexpr int B_OFF = A_OFF + NSLOT * TILE_BYTES;
  static constexpr int CODE_OFF = B_OFF + SBD * B_BYTES;
  static constexpr int LUT_OFF = CODE_OFF + SC * CODE_BYTES;
  static constexpr int BAR_OFF = LUT_OFF + LUT_BYTES;
  static constexpr int TOTAL = BAR_OFF + 512 + 1024;    // barriers + alignment slack
  static_assert(TOTAL <= 227 * 1024, "exceeds the shared memory of one CTA");
};

struct PsTile {
  int n0, m0, m_limit, b_row0, kb0, kblocks, rows_valid, z, mt_act;
  const unsigned char* w;
  const __half* w_scale;
};

template <int FMT, bool OUT_F32, int MT, int NB>
__global__ void __launch_bounds__(THREADS, 1) qgemm_ps_kernel(
    const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
    const unsigned char* __restrict__ w, const float* __restrict__ a_scale,
    const __half* __restrict__ w_scale, void* __restrict__ out, int M, int N, int K,
    const E8pTables* __restrict__ tables, int* status, PeerOut po, GroupDesc grp, AgIn ag,
    int* __restrict__ partial, int n_begin, int n_end, int splits) {
  using L = PsLayout<FMT, MT, NB>;
  constexpr int NSLOT = L::NSLOT, SBD = L::SBD, SC = L::SC > 0 ? L::SC : 1;
  constexpr int BN = NB;
  constexpr int CHUNKS = BN / 32;                      // 32-column chunks per accumulator
  constexpr uint32_t TMEM_COLS = MT * BN;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* a_s = smem + L::A_OFF;
  unsigned char* b_s = smem + L::B_OFF;
  unsigned char* code_s = smem + L::CODE_OFF;
  using Lut = E8pLut<L::LUT_COPIES>;
  Lut* lut = reinterpret_cast<Lut*>(smem + L::LUT_OFF);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* a_full = bars;                     // [NSLOT] activation tile landed (TMA)
  uint64_t* a_empty = a_full + NSLOT;          // [NSLOT] its MMAs retired
  uint64_t* c_full = a_empty + NSLOT;          // [SC]   packed codes landed (bulk copy)
  uint64_t* c_empty = c_full + SC;             // [SC]   every producer warp read them
  uint64_t* b_full = c_empty + SC;             // [SBD]  INT8 weight tile ready (decode or TMA)
  uint64_t* b_empty = b_full + SBD;            // [SBD]  its MMAs retired
  uint64_t* tmem_full = b_empty + SBD;         // [1]    all MMAs of the tile retired
  uint64_t* tmem_empty = tmem_full + 1;        // [MT]   accumulator read out by the epilogue
  uint64_t* epi_done = tmem_empty + MT;        // [1]    staged tile left for the peers
  uint64_t* stage_full = epi_done + 1;         // [1]    every producer warp staged its part
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(stage_full + 1);
  volatile int* abort_w = reinterpret_cast<volatile int*>(tmem_slot + 1);
  static_assert((2 * NSLOT + 2 * SC + 2 * SBD + MT + 3) * 8 + 8 <= 512, "barrier block");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool peer_stage = po.tp > 0 && partial == nullptr;
  const int n_tiles = (n_end - n_begin + BN - 1) / BN;
  const int m_tiles = grp.tiles != nullptr ? grp.meta[0] : (M + BM * MT - 1) / (BM * MT);
  const int total = n_tiles * m_tiles * splits;
  const int kb_all = K / BK, kb_per = (kb_all + splits - 1) / splits;

  auto tile_at = [&](int t) {
    PsTile T;
    T.z = t / (n_tiles * m_tiles);
    const int r = t - T.z * (n_tiles * m_tiles);
    const int nt = r / m_tiles, mi = r - nt * m_tiles;
    T.n0 = n_begin + nt * BN;
    T.m0 = mi * BM * MT;
    T.m_limit = M;
    T.b_row0 = T.n0;
    T.w = w;
    T.w_scale = w_scale;
    if (grp.tiles != nullptr) {
      const int expert = grp.tiles[mi * 4];
      T.m0 = grp.tiles[mi * 4 + 1];
      T.m_limit = T.m0 + grp.tiles[mi * 4 + 2];
      T.w = w + static_cast<long long>(expert) * grp.w_stride;
      T.w_scale = w_scale + static_cast<long long>(expert) * grp.n_per_expert;
      T.b_row0 = expert * grp.n_per_expert + T.n0;
    }
    T.kb0 = T.z * kb_per;
    T.kblocks = max(0, min(kb_all, T.kb0 + kb_per) - T.kb0);
    T.rows_valid = min(BN, n_end - T.n0);
    const int rows = min(T.m_limit, M) - T.m0;
    T.mt_act = rows <= 0 ? 0 : min(MT, (rows + BM - 1) / BM);
    return T;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSLOT; ++s) {
      mbar_init(&a_full[s], 1);
      mbar_init(&a_empty[s], 1);
    }
    for (int s = 0; s < SC; ++s) {
      mbar_init(&c_full[s], 1);
      mbar_init(&c_empty[s], PWARPS);
    }
    for (int s = 0; s < SBD; ++s) {
      mbar_init(&b_full[s], FMT == 0 ? 1 : PWARPS);
      mbar_init(&b_empty[s], 1);
    }
    mbar_init(tmem_full, 1);
    for (int t = 0; t < MT; ++t) mbar_init(&tmem_empty[t], 4 * CHUNKS);
    mbar_init(epi_done, PWARPS);
    mbar_init(stage_full, PWARPS);
    *abort_w = 0;
    mbar_fence_init();
    prefetch_tmap(&tmap_a);
    if (FMT == 0) prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  if (FMT != 0 && warp >= 3) e8p_lut_init(lut, tables, threadIdx.x - ROLE_THREADS, PRODUCERS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr int STAGE_ROW = BN * 2 + 16;
  static_assert(MT * BM * STAGE_ROW <= L::LUT_OFF, "staged tile must fit in the operand rings");

#define PS_WAIT(bar, par, code, detail) \
  mbar_wait_abortable((bar), (par), status, (code), (detail), abort_w)

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- activation loader
      uint32_t ca = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total; t += gridDim.x, ++it) {
        const PsTile T = tile_at(t);
        if (peer_stage && it > 0) ok = PS_WAIT(epi_done, (it - 1) & 1, STATUS_EPILOGUE_WAIT, 1);
        if (ok && ag.tp > 0 && T.mt_act > 0) {
          // all-gather fused into the GEMM: the rows of this M tile were pushed by their
          // owner ranks; wait for exactly those, then order the async-proxy loads after it
          ok = ag_wait(ag, T.m0, min(T.m0 + MT * BM, M) - 1, status);
          if (!ok) *abort_w = 1;
          fence_proxy_async_all();
        }
        for (int kb = 0; ok && kb < T.kblocks; ++kb) {
          for (int s = 0; s < T.mt_act; ++s, ++ca) {
            const uint32_t slot = ca % NSLOT;
            ok = PS_WAIT(&a_empty[slot], ((ca / NSLOT) & 1) ^ 1, STATUS_TMA_WAIT, kb);
            if (!ok) break;
            mbar_expect_tx(&a_full[slot], TILE_BYTES);
            tma_load_2d(a_s + slot * TILE_BYTES, &tmap_a, &a_full[slot], (T.kb0 + kb) * BK,
                        T.m0 + s * BM);
          }
        }
      }
      // never leave the CTA with a copy of ours in flight
      for (uint32_t c = ca > NSLOT ? ca - NSLOT : 0; c < ca; ++c)
        mbar_wait(&a_full[c % NSLOT], (c / NSLOT) & 1, status, STATUS_TMA_WAIT, 0x4000);
    }
  } else if (warp == 2) {
    if (lane == 0) {
      // ---------------- weight loader: INT8 tiles by TMA (W8) or packed codes as bulk copies
      uint32_t cw = 0;
      int it = 0;
      bool ok = true;
      constexpr int DEPTH = FMT == 0 ? SBD : SC;
      uint64_t* landed = FMT == 0 ? b_full : c_full;
      uint64_t* freed = FMT == 0 ? b_empty : c_empty;
      for (int t = blockIdx.x; ok && t < total; t += gridDim.x, ++it) {
        const PsTile T = tile_at(t);
        if (peer_stage && it > 0) ok = PS_WAIT(epi_done, (it - 1) & 1, STATUS_EPILOGUE_WAIT, 2);
        for (int kb = 0; ok && kb < T.kblocks && T.mt_act > 0; ++kb, ++cw) {
          const uint32_t s = cw % DEPTH;
          ok = PS_WAIT(&freed[s], ((cw / DEPTH) & 1) ^ 1, STATUS_TMA_WAIT, 0x1000 | kb);
          if (!ok) break;
          if (FMT == 0) {
            mbar_expect_tx(&b_full[s], L::B_BYTES);
            tma_load_2d(b_s + s * L::B_BYTES, &tmap_b, &b_full[s], (T.kb0 + kb) * BK, T.b_row0);
          } else {
            const unsigned char* src =
                T.w + (static_cast<size_t>(T.kb0 + kb) * N + T.n0) * L::ROW_CODE_BYTES;
            mbar_expect_tx(&c_full[s], T.rows_valid * L::ROW_CODE_BYTES);
            bulk_load(code_s + s * L::CODE_BYTES, src, T.rows_valid * L::ROW_CODE_BYTES,
                      &c_full[s]);
          }
        }
      }
      for (uint32_t c = cw > DEPTH ? cw - DEPTH : 0; c < cw; ++c)
        mbar_wait(&landed[c % DEPTH], (c / DEPTH) & 1, status, STATUS_TMA_WAIT, 0x5000);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer
      constexpr uint32_t idesc = umma_idesc(2, 1, 1, 0, 0, BM, BN);
      uint32_t ca = 0, cb = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total; t += gridDim.x, ++it) {
        const PsTile T = tile_at(t);
        const int kbs = T.mt_act > 0 ? T.kblocks : 0;
        for (int kb = 0; ok && kb < kbs; ++kb, ++cb) {
          const uint32_t sb = cb % SBD;
          ok = PS_WAIT(&b_full[sb], (cb / SBD) & 1, STATUS_MMA_WAIT, 0x2000 | kb);
          if (!ok) break;
          const uint32_t b_addr = smem_u32(b_s + sb * L::B_BYTES);
          uint32_t a_addr[MT];
#pragma unroll
          for (int s = 0; s < MT; ++s) {
            if (s < T.mt_act && ok) {
              // the epilogue of the previous tile must have read this accumulator out
              if (kb == 0 && it > 0)
                ok = PS_WAIT(&tmem_empty[s], (it - 1) & 1, STATUS_MMA_WAIT, 0x3000 | s);
              const uint32_t slot = (ca + s) % NSLOT;
              if (ok) ok = PS_WAIT(&a_full[slot], ((ca + s) / NSLOT) & 1, STATUS_MMA_WAIT, kb);
              a_addr[s] = smem_u32(a_s + slot * TILE_BYTES);
            }
          }
          if (!ok) break;
          tc_fence_after();
          // consecutive MMAs go to different accumulators: back-to-back accumulation into one
          // TMEM tile would serialise on it
#pragma unroll
          for (int j = 0; j < BK / 32; ++j) {
            const uint64_t bdesc = umma_desc(b_addr + j * 32, 16, 1024);
#pragma unroll
            for (int s = 0; s < MT; ++s)
              if (s < T.mt_act)
                mma_i8_ss(tmem_base + s * BN, umma_desc(a_addr[s] + j * 32, 16, 1024), bdesc,
                          idesc, (kb | j) != 0 ? 1u : 0u);
          }
          for (int s = 0; s < T.mt_act; ++s, ++ca) tc_commit(&a_empty[ca % NSLOT]);
          tc_commit(&b_empty[sb]);
        }
        if (ok) {
          if (kbs > 0) {
            tc_commit(tmem_full);
          } else {
            // nothing to multiply: still one tmem_full phase per tile, and never ahead of the
            // previous tile's epilogue (a phase must not complete before its waiters looked)
            if (it > 0) ok = PS_WAIT(&tmem_empty[0], (it - 1) & 1, STATUS_MMA_WAIT, 0x3800);
            if (ok) mbar_arrive(tmem_full);
          }
        }
      }
    }
  } else {
    // ---------------- producers (lattice decode) and epilogue
    const int t512 = threadIdx.x - ROLE_THREADS;                  // 0..511
    const int chunk = t512 & 7, rbase = t512 >> 3;      // 64 weight rows per pass
    const int copy = t512 & (L::LUT_COPIES - 1);
    const int quad = warp & 3;                          // TMEM lane quadrant of this warp
    const int part = (warp - 3) >> 2;                   // 0..3: which 32-column chunks
    const int row = quad * 32 + lane;
    bool ok = true;

    auto epilogue = [&](const PsTile& T, int it) {
      ok = PS_WAIT(tmem_full, it & 1, STATUS_EPILOGUE_WAIT, 0) && ok;
      ok = __all_sync(0xffffffffu, ok);                 // tcgen05.ld needs the whole warp
      if (!ok) return;
      tc_fence_after();
      const bool have_acc = T.kblocks > 0 && T.mt_act > 0;
#pragma unroll 1
      for (int item = part; item < MT * CHUNKS; item += 4) {
        const int mt = item / CHUNKS, c0 = (item % CHUNKS) * 32;
        const int m = T.m0 + mt * BM + row;
        uint32_t r[32];
        if (have_acc && mt < T.mt_act) {
          tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + mt * BN + c0, r);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0;        // nothing was accumulated
        }
        // this warp's share of accumulator mt is in registers: the tensor core may reuse it
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[mt]);
        // gathered row scales were written by peers: read them past L1
        const float sa = m < T.m_limit ? (ag.tp > 0 ? __ldcg(a_scale + m) : a_scale[m]) : 0.f;
        if (partial != nullptr) {
          if (m < T.m_limit) {
            // the workspace is compact over this launch's columns
            const int width = n_end - n_begin;
            int* dst = partial + (static_cast<size_t>(T.z) * M + m) * width +
                       (T.n0 - n_begin) + c0;
#pragma unroll
            for (int g = 0; g < 8; ++g)
              if (T.n0 + c0 + g * 4 + 4 <= n_end)
                *reinterpret_cast<int4*>(dst + g * 4) =
                    make_int4(r[g * 4], r[g * 4 + 1], r[g * 4 + 2], r[g * 4 + 3]);
          }
          continue;
        }
        if (m < T.m_limit) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int n = T.n0 + c0 + g * 8;
            if (n + 8 <= n_end) {
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j)
                v[j] = (static_cast<float>(static_cast<int>(r[g * 8 + j])) *
                        __half2float(T.w_scale[n + j])) * sa;
              if (peer_stage) {
                __align__(16) __half h[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) h[j] = __float2half_rn(v[j]);
                *reinterpret_cast<int4*>(smem + static_cast<size_t>(mt * BM + row) * STAGE_ROW +
                                         (c0 + g * 8) * 2) = *reinterpret_cast<const int4*>(h);
              } else if (OUT_F32) {
                float* o = reinterpret_cast<float*>(out) + static_cast<size_t>(m) * N + n;
                *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<float4*>(o + 4) = make_float4(v[4], v[5], v[6], v[7]);
              } else {
                __align__(16) __half h[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) h[j] = __float2half_rn(v[j]);
                __half* o = reinterpret_cast<__half*>(out) + static_cast<size_t>(m) * N + n;
                *reinterpret_cast<int4*>(o) = *reinterpret_cast<const int4*>(h);
              }
            }
          }
        }
      }
      if (peer_stage) {
        // fused scatter, step 2: when every producer warp has staged its part, whole 16-byte
        // segments of consecutive columns leave lane by lane (a warp writes complete rows per
        // instruction, which keeps NVLink packets full)
        __syncwarp();
        if (lane == 0) mbar_arrive(stage_full);
        ok = PS_WAIT(stage_full, it & 1, STATUS_EPILOGUE_WAIT, 3);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) return;
        constexpr int SEGS = BN / 8;
        for (int idx = t512; idx < MT * BM * SEGS; idx += PRODUCERS) {
          const int rr = idx / SEGS, seg = idx % SEGS;
          const int m = T.m0 + rr, n = T.n0 + seg * 8;
          if (m < T.m_limit && n + 8 <= n_end) {
            const int4 val = *reinterpret_cast<const int4*>(
                smem + static_cast<size_t>(rr) * STAGE_ROW + seg * 16);
            const size_t off = (static_cast<size_t>(po.rank) * po.rows_cap + m) * N + n;
            if (po.rows_per > 0) {
              // reduce-scatter: only the owner of row m receives this partial
              *reinterpret_cast<int4*>(po.inbox[min(m / po.rows_per, po.tp - 1)] + off) = val;
            } else {
              for (int d = 0; d < po.tp; ++d) *reinterpret_cast<int4*>(po.inbox[d] + off) = val;
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(epi_done);           // the rings may be refilled
      }
    };

    uint32_t cc = 0, cb = 0;
    int it = 0;
    bool have_prev = false;
    PsTile prev{};
    for (int t = blockIdx.x; ok && t < total; t += gridDim.x, ++it) {
      const PsTile T = tile_at(t);
      const int kbs = T.mt_act > 0 ? T.kblocks : 0;
      bool prev_pending = have_prev;
      // where the previous tile's epilogue runs: after the k-blocks that fit in the ring
      // have been decoded (they are all the tensor core can use before it is drained anyway)
      const int epos = (peer_stage || FMT == 0) ? -1 : min(SBD, kbs) - 1;
      if (prev_pending && epos < 0) {
        epilogue(prev, it - 1);
        prev_pending = false;
      }
      if (FMT != 0) {
        for (int kb = 0; ok && kb < kbs; ++kb, ++cc, ++cb) {
          const uint32_t sc = cc % SC, sb = cb % SBD;
          ok = PS_WAIT(&c_full[sc], (cc / SC) & 1, STATUS_DECODE_WAIT, kb);
          if (ok) ok = PS_WAIT(&b_empty[sb], ((cb / SBD) & 1) ^ 1, STATUS_DECODE_WAIT, 0x800 | kb);
          if (!ok) break;
          const unsigned char* cs = code_s + sc * L::CODE_BYTES;
          unsigned char* bs = b_s + sb * L::B_BYTES;
#pragma unroll
          for (int i = 0; i < (BN + 63) / 64; ++i) {
            const int wrow = rbase + 64 * i;
            if (BN < 64 && wrow >= BN) break;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (wrow < T.rows_valid) {
              if (FMT == 1) {
                const uint2 wd = *reinterpret_cast<const uint2*>(cs + wrow * 64 + chunk * 8);
                const uint2 q0 = e8p_decode_q4(wd.x, lut, copy);
                const uint2 q1 = e8p_decode_q4(wd.y, lut, copy);
                v = make_uint4(q0.x, q0.y, q1.x, q1.y);
              } else {
                const uint32_t wd = *reinterpret_cast<const uint32_t*>(cs + wrow * 32 + chunk * 4);
                const uint2 q0 = e8p_decode8<L::LUT_COPIES, 0>(wd, lut, copy);
                const uint2 q1 = e8p_decode8<L::LUT_COPIES, 1>(wd, lut, copy);
                v = make_uint4(q0.x, q0.y, q1.x, q1.y);
              }
            }
            *reinterpret_cast<uint4*>(bs + swz128(wrow, chunk)) = v;
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(&b_full[sb]);
            mbar_arrive(&c_empty[sc]);
          }
          if (prev_pending && kb == epos) {
            epilogue(prev, it - 1);
            prev_pending = false;
          }
        }
      }
      if (ok && prev_pending) epilogue(prev, it - 1);
      prev = T;
      have_prev = true;
    }
    if (ok && have_prev) epilogue(prev, it - 1);
  }
#undef PS_WAIT
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
  if (peer_stage) peer_signal_done(po, gridDim.x);
}

// ---------------------------------------------------------------- CTA-pair form
// Two CTAs (a cluster of 2, neighbouring SMs) share one output tile of 512 rows x 256
// columns through tcgen05 cta_group::2: every MMA covers 256 rows x 256 columns, CTA r of
// the pair holds rows [r*128, r*128+128) of each 256-row A sub-tile and weight rows
// [r*128, r*128+128) of the 256-row B tile in its own shared memory, and its TMEM receives
// its 128 rows of both accumulators.  Per MAC a CTA therefore streams half the activation
// bytes and decodes half the weight rows of the one-CTA kernel with the same TMEM budget,
// which is what the L2-to-SM bandwidth (the limiter of the one-CTA kernel) needed.
// The even CTA issues the MMAs.  Barriers that the MMA thread waits on live in the even
// CTA and collect both CTAs' arrivals (TMA bytes through the pair form of the tile load,
// producer and epilogue warps through cluster-scope arrives); barriers that it signals are
// signalled in both CTAs at once with tcgen05.commit ... multicast::cluster (a barrier
// signal; every load in this file is unicast).  Persistent over pair tiles like the kernel
// above; fused scatter (peers) and fused all-gather wait are kept.
template <int FMT>
struct PairLayout {
  static constexpr int MT = 2, BN = 256, HALF_N = 128;
  static constexpr int ROW_CODE_BYTES = FMT == 1 ? 64 : (FMT == 2 ? 32 : 0);
  static constexpr int CODE_BYTES = HALF_N * ROW_CODE_BYTES;
  static constexpr int B_BYTES = HALF_N * BK;
  static constexpr int NSLOT = 8;                        // 4 k-blocks of 2 sub-tiles
  static constexpr int SBD = FMT == 0 ? 4 : 3;
  static constexpr int SC = FMT == 0 ? 0 : 3;
  static constexpr int LUT_COPIES = 8;
  static constexpr int LUT_BYTES = FMT == 0 ? 0 : static_cast<int>(sizeof(E8pLut<LUT_COPIES>));
  static constexpr int A_OFF = 0;
  static constexpr int B_OFF = A_OFF + NSLOT * TILE_BYTES;
  static constexpr int CODE_OFF = B_OFF + SBD * B_BYTES;
  static constexpr int LUT_OFF = CODE_OFF + SC * CODE_BYTES;
  static constexpr int BAR_OFF = LUT_OFF + LUT_BYTES;
  static constexpr int TOTAL = BAR_OFF + 512 + 1024;
  static_assert(TOTAL <= 227 * 1024, "exceeds the shared memory of one CTA");
};

template <int FMT, bool OUT_F32>
__global__ void __launch_bounds__(THREADS, 1) qgemm_pair_kernel(
    const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
    const unsigned char* __restrict__ w, const float* __restrict__ a_scale,
    const __half* __restrict__ w_scale, void* __restrict__ out, int M, int N, int K,
    const E8pTables* __restrict__ tables, int* status, PeerOut po, AgIn ag) {
  using L = PairLayout<FMT>;
  constexpr int MT = L::MT, BN = L::BN, HALF_N = L::HALF_N;
  constexpr int NSLOT = L::NSLOT, SBD = L::SBD, SC = L::SC > 0 ? L::SC : 1;
  constexpr int CHUNKS = BN / 32;
  constexpr uint32_t TMEM_COLS = MT * BN;               // 512
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* a_s = smem + L::A_OFF;
  unsigned char* b_s = smem + L::B_OFF;
  unsigned char* code_s = smem + L::CODE_OFF;
  using Lut = E8pLut<L::LUT_COPIES>;
  Lut* lut = reinterpret_cast<Lut*>(smem + L::LUT_OFF);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* a_full = bars;                     // [NSLOT] even CTA: both halves landed
  uint64_t* a_empty = a_full + NSLOT;          // [NSLOT] both CTAs: MMAs retired
  uint64_t* c_full = a_empty + NSLOT;          // [SC]    local: packed codes landed
  uint64_t* c_empty = c_full + SC;             // [SC]    local: producer warps read them
  uint64_t* b_full = c_empty + SC;             // [SBD]   even CTA: both halves decoded / landed
  uint64_t* b_empty = b_full + SBD;            // [SBD]   both CTAs: MMAs retired
  uint64_t* tmem_full = b_empty + SBD;         // [1]     both CTAs
  uint64_t* tmem_empty = tmem_full + 1;        // [MT]    even CTA: both epilogues read it out
  uint64_t* epi_done = tmem_empty + MT;        // [1]     local
  uint64_t* stage_full = epi_done + 1;         // [1]     local
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(stage_full + 1);
  volatile int* abort_w = reinterpret_cast<volatile int*>(tmem_slot + 1);
  static_assert((2 * NSLOT + 2 * SC + 2 * SBD + MT + 3) * 8 + 8 <= 512, "barrier block");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t crank = cluster_ctarank();              // 0: issues the MMAs
  const bool leader = crank == 0;
  const bool peer_stage = po.tp > 0;
  const int n_tiles = (N + BN - 1) / BN;
  const int m_tiles = (M + 2 * BM * MT - 1) / (2 * BM * MT);       // 512 rows per pair tile
  const int total = n_tiles * m_tiles;
  const int kblocks = K / BK;
  const int pair_id = blockIdx.x >> 1, pairs = gridDim.x >> 1;

  struct Tile {
    int n0, m0, mt_act, rows_valid;
  };
  auto tile_at = [&](int t) {
    Tile T;
    const int nt = t / m_tiles, mi = t - nt * m_tiles;
    T.n0 = nt * BN;
    T.m0 = mi * 2 * BM * MT;
    const int rows = M - T.m0;
    T.mt_act = rows <= 0 ? 0 : min(MT, (rows + 2 * BM - 1) / (2 * BM));
    T.rows_valid = max(0, min(HALF_N, N - (T.n0 + static_cast<int>(crank) * HALF_N)));
    return T;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSLOT; ++s) {
      mbar_init(&a_full[s], 1);
      mbar_init(&a_empty[s], 1);
    }
    for (int s = 0; s < SC; ++s) {
      mbar_init(&c_full[s], 1);
      mbar_init(&c_empty[s], PWARPS);
    }
    for (int s = 0; s < SBD; ++s) {
      mbar_init(&b_full[s], FMT == 0 ? 1 : 2 * PWARPS);
      mbar_init(&b_empty[s], 1);
    }
    mbar_init(tmem_full, 1);
    for (int t = 0; t < MT; ++t) mbar_init(&tmem_empty[t], 2 * 4 * CHUNKS);
    mbar_init(epi_done, PWARPS);
    mbar_init(stage_full, PWARPS);
    *abort_w = 0;
    mbar_fence_init();
    prefetch_tmap(&tmap_a);
    if (FMT == 0) prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, TMEM_COLS);
    tmem_relinquish2();
  }
  if (FMT != 0 && warp >= 3) e8p_lut_init(lut, tables, threadIdx.x - ROLE_THREADS, PRODUCERS);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                          // the peer's barriers exist before anyone signals
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr int STAGE_ROW = BN * 2 + 16;
  static_assert(MT * BM * STAGE_ROW <= L::LUT_OFF, "staged tile must fit in the operand rings");

#define PR_WAIT(bar, par, code, detail) \
  mbar_wait_abortable((bar), (par), status, (code), (detail), abort_w)

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- activation loader (both CTAs): this CTA's 128 rows of each sub-tile
      uint32_t ca = 0;
      int it = 0;
      bool ok = true;
      for (int t = pair_id; ok && t < total; t += pairs, ++it) {
        const Tile T = tile_at(t);
        if (peer_stage && it > 0) ok = PR_WAIT(epi_done, (it - 1) & 1, STATUS_EPILOGUE_WAIT, 1);
        if (ok && ag.tp > 0 && T.mt_act > 0) {
          ok = ag_wait(ag, T.m0, min(T.m0 + 2 * BM * MT, M) - 1, status);
          if (!ok) *abort_w = 1;
          fence_proxy_async_all();
        }
        for (int kb = 0; ok && kb < kblocks; ++kb) {
          for (int s = 0; s < T.mt_act; ++s, ++ca) {
            const uint32_t slot = ca % NSLOT;
            ok = PR_WAIT(&a_empty[slot], ((ca / NSLOT) & 1) ^ 1, STATUS_TMA_WAIT, kb);
            if (!ok) break;
            const uint32_t full0 = mapa_u32(smem_u32(&a_full[slot]), 0);
            if (leader) mbar_expect_tx(&a_full[slot], 2 * TILE_BYTES);
            tma_load_2d_pair(a_s + slot * TILE_BYTES, &tmap_a, full0, kb * BK,
                             T.m0 + s * 2 * BM + static_cast<int>(crank) * BM);
          }
        }
      }
      // the even CTA's barriers count both CTAs' copies: wait for the last ones before the
      // pair leaves (the odd CTA is held by the cluster barrier at the end)
      if (leader)
        for (uint32_t c = ca > NSLOT ? ca - NSLOT : 0; c < ca; ++c)
          mbar_wait(&a_full[c % NSLOT], (c / NSLOT) & 1, status, STATUS_TMA_WAIT, 0x4000);
    }
  } else if (warp == 2) {
    if (lane == 0) {
      // ---------------- weight loader (both CTAs): its 128 weight rows
      uint32_t cw = 0;
      int it = 0;
      bool ok = true;
      constexpr int DEPTH = FMT == 0 ? SBD : SC;
      uint64_t* freed = FMT == 0 ? b_empty : c_empty;
      for (int t = pair_id; ok && t < total; t += pairs, ++it) {
        const Tile T = tile_at(t);
        const int nrow0 = T.n0 + static_cast<int>(crank) * HALF_N;
        if (peer_stage && it > 0) ok = PR_WAIT(epi_done, (it - 1) & 1, STATUS_EPILOGUE_WAIT, 2);
        for (int kb = 0; ok && kb < kblocks && T.mt_act > 0; ++kb, ++cw) {
          const uint32_t s = cw % DEPTH;
          ok = PR_WAIT(&freed[s], ((cw / DEPTH) & 1) ^ 1, STATUS_TMA_WAIT, 0x1000 | kb);
          if (!ok) break;
          if (FMT == 0) {
            const uint32_t full0 = mapa_u32(smem_u32(&b_full[s]), 0);
            if (leader) mbar_expect_tx(&b_full[s], 2 * L::B_BYTES);
            tma_load_2d_pair(b_s + s * L::B_BYTES, &tmap_b, full0, kb * BK, nrow0);
          } else {
            // a slab past the last weight row is not loaded: its waiters get an empty phase
            const uint32_t bytes = T.rows_valid * L::ROW_CODE_BYTES;
            mbar_expect_tx(&c_full[s], bytes);
            if (bytes > 0)
              bulk_load(code_s + s * L::CODE_BYTES,
                        w + (static_cast<size_t>(kb) * N + nrow0) * L::ROW_CODE_BYTES, bytes,
                        &c_full[s]);
          }
        }
      }
      if (FMT != 0 || leader) {
        uint64_t* landed = FMT == 0 ? b_full : c_full;
        for (uint32_t c = cw > DEPTH ? cw - DEPTH : 0; c < cw; ++c)
          mbar_wait(&landed[c % DEPTH], (c / DEPTH) & 1, status, STATUS_TMA_WAIT, 0x5000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // ---------------- MMA issuer (even CTA only)
      constexpr uint32_t idesc = umma_idesc(2, 1, 1, 0, 0, 2 * BM, BN);
      uint32_t ca = 0, cb = 0;
      int it = 0;
      bool ok = true;
      for (int t = pair_id; ok && t < total; t += pairs, ++it) {
        const Tile T = tile_at(t);
        const int kbs = T.mt_act > 0 ? kblocks : 0;
        for (int kb = 0; ok && kb < kbs; ++kb, ++cb) {
          const uint32_t sb = cb % SBD;
          ok = PR_WAIT(&b_full[sb], (cb / SBD) & 1, STATUS_MMA_WAIT, 0x2000 | kb);
          if (!ok) break;
          const uint32_t b_addr = smem_u32(b_s + sb * L::B_BYTES);
          uint32_t a_addr[MT];
#pragma unroll
          for (int s = 0; s < MT; ++s) {
            if (s < T.mt_act && ok) {
              if (kb == 0 && it > 0)
                ok = PR_WAIT(&tmem_empty[s], (it - 1) & 1, STATUS_MMA_WAIT, 0x3000 | s);
              const uint32_t slot = (ca + s) % NSLOT;
              if (ok) ok = PR_WAIT(&a_full[slot], ((ca + s) / NSLOT) & 1, STATUS_MMA_WAIT, kb);
              a_addr[s] = smem_u32(a_s + slot * TILE_BYTES);
            }
          }
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int j = 0; j < BK / 32; ++j) {
            const uint64_t bdesc = umma_desc(b_addr + j * 32, 16, 1024);
#pragma unroll
            for (int s = 0; s < MT; ++s)
              if (s < T.mt_act)
                mma_i8_ss_pair(tmem_base + s * BN, umma_desc(a_addr[s] + j * 32, 16, 1024), bdesc,
                               idesc, (kb | j) != 0 ? 1u : 0u);
          }
          for (int s = 0; s < T.mt_act; ++s, ++ca) tc_commit_pair(&a_empty[ca % NSLOT], 3);
          tc_commit_pair(&b_empty[sb], 3);
        }
        if (ok) {
          if (kbs > 0) {
            tc_commit_pair(tmem_full, 3);
          } else {
            if (it > 0) ok = PR_WAIT(&tmem_empty[0], (it - 1) & 1, STATUS_MMA_WAIT, 0x3800);
            if (ok) {
              mbar_arrive(tmem_full);
              mbar_arrive_cluster(mapa_u32(smem_u32(tmem_full), 1));
            }
          }
        }
      }
    }
  } else {
    // ---------------- producers (lattice decode of this CTA's weight rows) and epilogue
    const int t512 = threadIdx.x - ROLE_THREADS;
    const int chunk = t512 & 7, rbase = t512 >> 3;
    const int copy = t512 & (L::LUT_COPIES - 1);
    const int quad = warp & 3;
    const int part = (warp - 3) >> 2;
    const int row = quad * 32 + lane;
    bool ok = true;

    auto epilogue = [&](const Tile& T, int it) {
      ok = PR_WAIT(tmem_full, it & 1, STATUS_EPILOGUE_WAIT, 0) && ok;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) return;
      tc_fence_after();
#pragma unroll 1
      for (int item = part; item < MT * CHUNKS; item += 4) {
        const int mt = item / CHUNKS, c0 = (item % CHUNKS) * 32;
        const int m = T.m0 + mt * 2 * BM + static_cast<int>(crank) * BM + row;
        uint32_t r[32];
        if (mt < T.mt_act) {
          tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + mt * BN + c0, r);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tmem_empty[mt]), 0));
        const float sa = m < M ? (ag.tp > 0 ? __ldcg(a_scale + m) : a_scale[m]) : 0.f;
        if (m < M) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int n = T.n0 + c0 + g * 8;
            if (n + 8 <= N) {
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j)
                v[j] = (static_cast<float>(static_cast<int>(r[g * 8 + j])) *
                        __half2float(w_scale[n + j])) * sa;
              if (peer_stage) {
                __align__(16) __half h[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) h[j] = __float2half_rn(v[j]);
                *reinterpret_cast<int4*>(smem + static_cast<size_t>(mt * BM + row) * STAGE_ROW +
                                         (c0 + g * 8) * 2) = *reinterpret_cast<const int4*>(h);
              } else if (OUT_F32) {
                float* o = reinterpret_cast<float*>(out) + static_cast<size_t>(m) * N + n;
                *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<float4*>(o + 4) = make_float4(v[4], v[5], v[6], v[7]);
              } else {
                __align__(16) __half h[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) h[j] = __float2half_rn(v[j]);
                __half* o = reinterpret_cast<__half*>(out) + static_cast<size_t>(m) * N + n;
                *reinterpret_cast<int4*>(o) = *reinterpret_cast<const int4*>(h);
              }
            }
          }
        }
      }
      if (peer_stage) {
        __syncwarp();
        if (lane == 0) mbar_arrive(stage_full);
        ok = PR_WAIT(stage_full, it & 1, STATUS_EPILOGUE_WAIT, 3);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) return;
        constexpr int SEGS = BN / 8;
        for (int idx = t512; idx < MT * BM * SEGS; idx += PRODUCERS) {
          const int rr = idx / SEGS, seg = idx % SEGS;
          const int m = T.m0 + (rr / BM) * 2 * BM + static_cast<int>(crank) * BM + rr % BM;
          const int n = T.n0 + seg * 8;
          if (m < M && n + 8 <= N) {
            const int4 val = *reinterpret_cast<const int4*>(
                smem + static_cast<size_t>(rr) * STAGE_ROW + seg * 16);
            const size_t off = (static_cast<size_t>(po.rank) * po.rows_cap + m) * N + n;
            if (po.rows_per > 0) {
              *reinterpret_cast<int4*>(po.inbox[min(m / po.rows_per, po.tp - 1)] + off) = val;
            } else {
              for (int d = 0; d < po.tp; ++d) *reinterpret_cast<int4*>(po.inbox[d] + off) = val;
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(epi_done);
      }
    };

    uint32_t cc = 0, cb = 0;
    int it = 0;
    bool have_prev = false;
    Tile prev{};
    for (int t = pair_id; ok && t < total; t += pairs, ++it) {
      const Tile T = tile_at(t);
      const int kbs = T.mt_act > 0 ? kblocks : 0;
      bool prev_pending = have_prev;
      const int epos = (peer_stage || FMT == 0) ? -1 : min(SBD, kbs) - 1;
      if (prev_pending && epos < 0) {
        epilogue(prev, it - 1);
        prev_pending = false;
      }
      if (FMT != 0) {
        for (int kb = 0; ok && kb < kbs; ++kb, ++cc, ++cb) {
          const uint32_t sc = cc % SC, sb = cb % SBD;
          ok = PR_WAIT(&c_full[sc], (cc / SC) & 1, STATUS_DECODE_WAIT, kb);
          if (ok) ok = PR_WAIT(&b_empty[sb], ((cb / SBD) & 1) ^ 1, STATUS_DECODE_WAIT, 0x800 | kb);
          if (!ok) break;
          const unsigned char* cs = code_s + sc * L::CODE_BYTES;
          unsigned char* bs = b_s + sb * L::B_BYTES;
#pragma unroll
          for (int i = 0; i < HALF_N / 64; ++i) {
            const int wrow = rbase + 64 * i;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (wrow < T.rows_valid) {
              if (FMT == 1) {
                const uint2 wd = *reinterpret_cast<const uint2*>(cs + wrow * 64 + chunk * 8);
                const uint2 q0 = e8p_decode_q4(wd.x, lut, copy);
                const uint2 q1 = e8p_decode_q4(wd.y, lut, copy);
                v = make_uint4(q0.x, q0.y, q1.x, q1.y);
              } else {
                const uint32_t wd = *reinterpret_cast<const uint32_t*>(cs + wrow * 32 + chunk * 4);
                const uint2 q0 = e8p_decode8<L::LUT_COPIES, 0>(wd, lut, copy);
                const uint2 q1 = e8p_decode8<L::LUT_COPIES, 1>(wd, lut, copy);
                v = make_uint4(q0.x, q0.y, q1.x, q1.y);
              }
            }
            *reinterpret_cast<uint4*>(bs + swz128(wrow, chunk)) = v;
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive_cluster(mapa_u32(smem_u32(&b_full[sb]), 0));
            mbar_arrive(&c_empty[sc]);
          }
          if (prev_pending && kb == epos) {
            epilogue(prev, it - 1);
            prev_pending = false;
          }
        }
      }
      if (ok && prev_pending) epilogue(prev, it - 1);
      prev = T;
      have_prev = true;
    }
    if (ok && have_prev) epilogue(prev, it - 1);
  }
#undef PR_WAIT
  // nobody leaves while its pair may still signal its barriers or read its shared memory
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) tmem_dealloc2(tmem_base, TMEM_COLS);
  if (peer_stage) peer_signal_done(po, gridDim.x);
}

template <int FMT, bool OUT_F32>
int launch_pair(const int8_t* a, const float* a_scale, const void* w, const __half* w_scale,
                void* out, int M, int N, int K, cudaStream_t stream, const PeerOut& po,
                const AgIn& ag) {
  using L = PairLayout<FMT>;
  CUtensorMap ta, tb;
  if (!make_tmap_2d(&ta, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, K, BM, BK)) return -3;
  if (FMT == 0) {
    if (!make_tmap_2d(&tb, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, K, L::HALF_N, BK)) return -3;
  } else {
    tb = ta;
    if (reinterpret_cast<uintptr_t>(w) % 16) return -1;
  }
  static const int slot = runtime_new_slot();
  if (runtime_first_use(slot)) {
    cudaError_t e = cudaFuncSetAttribute(qgemm_pair_kernel<FMT, OUT_F32>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  const long tiles = static_cast<long>((N + L::BN - 1) / L::BN) * ((M + 511) / 512);
  const int pairs = static_cast<int>(tiles < NUM_SMS / 2 ? tiles : NUM_SMS / 2);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = L::TOTAL;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(
      &cfg, qgemm_pair_kernel<FMT, OUT_F32>, ta, tb, reinterpret_cast<const unsigned char*>(w),
      a_scale, w_scale, out, M, N, K, runtime_e8p_tables(), runtime_status_ptr(), po, ag);
  return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}

// out[m][n] = (float(sum_z partial[z][m][n]) * w_scale[n]) * a_scale[m], as FP16 into `out`
// or, with peers, into the inboxes (all ranks, or the row's owner when rows_per > 0).
// One thread per 8 columns; the arithmetic is the GEMM epilogue's, so a split GEMM returns
// bit for bit what the unsplit one does.
__global__ void __launch_bounds__(256) splitk_finalize_kernel(
    const int* __restrict__ partial, int splits, const float* __restrict__ a_scale,
    const __half* __restrict__ w_scale, __half* __restrict__ out, int M, int N, PeerOut po,
    int ag_scales, int n_begin, int width) {
  const int groups = width / 8;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx < static_cast<long long>(M) * groups) {
    const int m = static_cast<int>(idx / groups), c = static_cast<int>(idx % groups) * 8;
    const int n = n_begin + c;
    int acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int z = 0; z < splits; ++z) {
      const int4* src = reinterpret_cast<const int4*>(
          partial + (static_cast<size_t>(z) * M + m) * width + c);
      const int4 a = src[0], b = src[1];
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    const float sa = ag_scales ? __ldcg(a_scale + m) : a_scale[m];
    __align__(16) __half h[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      h[j] = __float2half_rn((static_cast<float>(acc[j]) * __half2float(w_scale[n + j])) * sa);
    if (po.tp > 0) {
      const size_t off = (static_cast<size_t>(po.rank) * po.rows_cap + m) * N + n;
      if (po.rows_per > 0) {
        *reinterpret_cast<int4*>(po.inbox[min(m / po.rows_per, po.tp - 1)] + off) =
            *reinterpret_cast<const int4*>(h);
      } else {
        for (int d = 0; d < po.tp; ++d)
          *reinterpret_cast<int4*>(po.inbox[d] + off) = *reinterpret_cast<const int4*>(h);
      }
    } else {
      *reinterpret_cast<int4*>(out + static_cast<size_t>(m) * N + n) =
          *reinterpret_cast<const int4*>(h);
    }
  }
  if (po.tp > 0) peer_signal_done(po, gridDim.x);
}


// Split-K sums inside the GEMM kernel (one-tile form) when the last arriver has at most
// 512 KiB of other splits' accumulators to read.
inline bool splitk_in_kernel(int mt, int nb, int splits) {
  return splits > 1 && static_cast<long>(splits - 1) * mt * BM * nb * 4 <= 512 * 1024;
}

template <int FMT, bool OUT_F32, int MT, int NB>
int launch_ps(const int8_t* a, const float* a_scale, const void* w, const __half* w_scale,
              void* out, int M, int N, int K, cudaStream_t stream, const PeerOut& po,
              const GroupDesc& grp, int experts, int max_tiles, const AgIn& ag, int splits,
              int n_begin, int n_end) {
  using L = PsLayout<FMT, MT, NB>;
  CUtensorMap ta, tb;
  if (!make_tmap_2d(&ta, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, K, BM, BK)) return -3;
  if (FMT == 0) {
    if (!make_tmap_2d(&tb, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1,
                      static_cast<uint64_t>(N) * experts, K, K, NB, BK))
      return -3;
  } else {
    tb = ta;
    if (reinterpret_cast<uintptr_t>(w) % 16) return -1;
  }
  static const int slot = runtime_new_slot();
  if (runtime_first_use(slot)) {
    cudaError_t e = cudaFuncSetAttribute(qgemm_ps_kernel<FMT, OUT_F32, MT, NB>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  const int width = n_end - n_begin;
  if (width <= 0) return 0;
  const long n_tiles = (width + NB - 1) / NB;
  const long m_tiles = grp.tiles ? max_tiles : (M + BM * MT - 1) / (BM * MT);
  const long total = n_tiles * m_tiles * splits;
  const int grid = static_cast<int>(total < NUM_SMS ? total : NUM_SMS);
  int* partial = splits > 1 ? runtime_splitk_workspace() : nullptr;
  if (splits > 1 && static_cast<size_t>(splits) * M * width * 4 > SPLITK_WORKSPACE_BYTES) return -1;
  qgemm_ps_kernel<FMT, OUT_F32, MT, NB><<<grid, THREADS, L::TOTAL, stream>>>(
      ta, tb, reinterpret_cast<const unsigned char*>(w), a_scale, w_scale, out, M, N, K,
      runtime_e8p_tables(), runtime_status_ptr(), po, grp, ag, partial, n_begin, n_end, splits);
  if (splits > 1) {
    const long long items = static_cast<long long>(M) * (width / 8);
    splitk_finalize_kernel<<<static_cast<unsigned>((items + 255) / 256), 256, 0, stream>>>(
        partial, splits, a_scale, w_scale, reinterpret_cast<__half*>(out), M, N, po,
        ag.tp > 0 ? 1 : 0, n_begin, width);
  }
  return static_cast<int>(cudaGetLastError());
}

template <int FMT, bool OUT_F32, int MT, int NB>
int launch(const int8_t* a, const float* a_scale, const void* w, const __half* w_scale, void* out,
           int M, int N, int K, cudaStream_t stream, const PeerOut& po,
           const GroupDesc& grp = GroupDesc{nullptr, nullptr, 0, 0}, int experts = 1,
           int max_tiles = 0, const AgIn& ag = AgIn{nullptr, nullptr, 0, 0}, int splits = 1,
           int n_begin = 0, int n_end = -1) {
  using L = Layout<FMT, MT, NB>;
  if (n_end < 0) n_end = N;
  if (g_impl != 1)
    return launch_ps<FMT, OUT_F32, MT, NB>(a, a_scale, w, w_scale, out, M, N, K, stream, po, grp,
                                           experts, max_tiles, ag, splits, n_begin, n_end);
  CUtensorMap ta, tb;
  if (!make_tmap_2d(&ta, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, K, BM, BK)) return -3;
  if (FMT == 0) {
    if (!make_tmap_2d(&tb, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1,
                      static_cast<uint64_t>(N) * experts, K, K, NB, BK))
      return -3;
  } else {
    tb = ta;
    if (reinterpret_cast<uintptr_t>(w) % 16) return -1;
  }
  static const int slot = runtime_new_slot();
  if (runtime_first_use(slot)) {
    cudaError_t e = cudaFuncSetAttribute(qgemm_tc_kernel<FMT, OUT_F32, MT, NB>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  const int width = n_end - n_begin;
  if (width <= 0) return 0;
  dim3 grid((width + NB - 1) / NB, grp.tiles ? max_tiles : (M + BM * MT - 1) / (BM * MT), splits);
  int* partial = splits > 1 ? runtime_splitk_workspace() : nullptr;
  const size_t tiles = static_cast<size_t>(grid.x) * grid.y;
  // The CTA that arrives last at a tile adds the other splits itself when that is little to
  // read; otherwise a second kernel, spread over every SM, adds them.
  const bool in_kernel = splitk_in_kernel(MT, NB, splits);
  if (splits > 1 && (tiles > static_cast<size_t>(SPLITK_TICKETS) ||
                     tiles * splits * MT * BM * NB * 4 > SPLITK_WORKSPACE_BYTES))
    return -1;
  qgemm_tc_kernel<FMT, OUT_F32, MT, NB><<<grid, THREADS, L::TOTAL, stream>>>(
      ta, tb, reinterpret_cast<const unsigned char*>(w), a_scale, w_scale, out, M, N, K,
      runtime_e8p_tables(), runtime_status_ptr(), po, grp, ag, partial,
      in_kernel ? runtime_splitk_tickets() : nullptr, n_begin, n_end, g_probe);
  if (splits > 1 && !in_kernel) {
    const long long items = static_cast<long long>(M) * (width / 8);
    splitk_finalize_kernel<<<static_cast<unsigned>((items + 255) / 256), 256, 0, stream>>>(
        partial, splits, a_scale, w_scale, reinterpret_cast<__half*>(out), M, N, po,
        ag.tp > 0 ? 1 : 0, n_begin, width);
  }
  return static_cast<int>(cudaGetLastError());
}

// Tile choice.  Rows: as many accumulators as the packet fills (each decoded weight tile is
// then multiplied against up to 512 rows).  Weight rows per CTA: the widest tile that still
// gives the grid about one CTA per SM, so narrow projections (N = hidden) do not leave most
// of the machine idle.  FP32 output is only used by the (very wide) vocabulary head.
// Cells of the split-K workspace one split of an M x N product needs: its tiles are stored
// whole, so both extents round up to the largest tile.
inline size_t padded_cells(int M, int N) {
  return static_cast<size_t>((M + 4 * BM - 1) / (4 * BM)) * (4 * BM) * ((N + 127) / 128) * 128;
}

inline int plan_splits(int M, int N, int K, int out_f32) {
  const int mt = M > 2 * BM ? 4 : (M > BM ? 2 : 1);
  const long c128 = static_cast<long>((M + BM * mt - 1) / (BM * mt)) * ((N + 127) / 128);
  int splits = 1;
  if (!out_f32 && c128 <= 74 && K / BK >= 8 && N % 8 == 0) {
    splits = static_cast<int>(148 / c128);
    splits = splits > K / BK / 8 ? K / BK / 8 : splits;          // at least 8 k-blocks each
    splits = splits > 8 ? 8 : splits;
    while (splits > 1 && static_cast<size_t>(splits) * padded_cells(M, N) * 4 > SPLITK_WORKSPACE_BYTES)
      --splits;
  }
  return splits < 1 ? 1 : splits;
}

// ---------------------------------------------------------------- launch plan
// What launch_fmt decides for a shape: M-tile factor, weight-tile width, K splits and whether
// the wave tail is peeled off into a split-K launch of its own.  The defaults below are the
// heuristics; a tuned table (orinfer_qgemm_set_variant: per format, projection shape and row
// range) overrides them.  The role of the reference's per-row-range kernel variants
// (crates/orinfer-model-sdk/src/operators/rows.rs:10-60) and of its offline projection tuner
// (python/orinfer_build/tuning/).
struct Plan {
  int mt, nb, splits, tail_splits;   // tail_splits > 0: peel ntiles % 148 weight tiles
};

struct Variant {
  int fmt, m_lo, m_hi, n, k, mt, nb, splits;
};
constexpr int MAX_VARIANTS = 512;
static Variant g_variants[MAX_VARIANTS];
static int g_variant_count = 0;
static std::mutex g_variant_mutex;            // the table may change while other threads launch

inline bool variant_valid(const Variant& v) {
  if (v.fmt < 0 || v.fmt > 2 || v.m_lo < 1 || v.m_hi < v.m_lo || v.n < 8 || v.k < BK) return false;
  if (v.mt != 1 && v.mt != 2 && v.mt != 4) return false;
  if (v.nb != 128 && v.nb != 64 && v.nb != 32) return false;
  if (v.splits < 1 || v.splits > 16 || v.splits > v.k / BK) return false;
  if (v.splits > 1 && (v.nb != 128 || v.n % 8)) return false;
  if (v.splits > 1 &&
      static_cast<size_t>(v.splits) * padded_cells(v.m_hi, v.n) * 4 > SPLITK_WORKSPACE_BYTES)
    return false;
  return true;
}

inline Plan make_plan(int fmt, int M, int N, int K, int out_f32, bool fused) {
  Plan p{};
  p.mt = M > 2 * BM ? 4 : (M > BM ? 2 : 1);
  if (!out_f32) {
    std::lock_guard<std::mutex> lock(g_variant_mutex);
    for (int i = 0; i < g_variant_count; ++i) {
      const Variant& v = g_variants[i];
      if (v.fmt == fmt && v.n == N && v.k == K && M >= v.m_lo && M <= v.m_hi) {
        p.mt = v.mt;
        p.nb = v.nb;
        p.splits = v.splits;
        return p;
      }
    }
  }
  long mtiles = (M + BM * p.mt - 1) / (BM * p.mt);
  const long ntiles = (N + 127) / 128;
  auto ctas = [&](int nb) { return mtiles * ((N + nb - 1) / nb); };
  // A projection too narrow to give every SM a CTA (at most half a wave of 128-wide tiles):
  //  * up to 128 rows it is split along K: thin tiles would make every CTA stream the whole
  //    activation matrix, K splits share it, and the INT32 partials make the result
  //    independent of the split.  Two k-blocks per split are enough to pay for the finalize
  //    pass at these row counts;
  //  * above 128 rows the finalize pass (rows x N x splits INT32) costs more than it saves
  //    unless K is long: thinner weight tiles under a smaller M tile win instead.
  // (Measured over 18 projection shapes x 15 row buckets by the tuner in
  // orinfer_b200/tuning/gemm_tuner.py; a tuned table still overrides these.)
  const long c128 = ctas(128);
  p.splits = 1;
  const bool narrow = !out_f32 && c128 <= 74 && K / BK >= 8 && N % 8 == 0;
  if (narrow && M > BM && K / BK <= 48) {
    p.mt = M <= 6 * BM ? 2 : 4;
    p.nb = M <= 2 * BM ? 32 : 64;
    return p;
  }
  if (narrow) {
    int splits = static_cast<int>(148 / c128);
    const int per = M <= BM ? 2 : 8;                    // k-blocks a split must keep
    splits = splits > K / BK / per ? K / BK / per : splits;
    splits = splits > 8 ? 8 : splits;
    while (splits > 1 && static_cast<size_t>(splits) * padded_cells(M, N) * 4 > SPLITK_WORKSPACE_BYTES)
      --splits;
    p.splits = splits < 1 ? 1 : splits;
  }
  // With four or more 512-row tiles, halving the weight tile doubles the activation traffic
  // and the weight decode work for no gain: 128-wide tiles won every such case measured.
  p.nb = (out_f32 || p.splits > 1 || c128 >= 120 || (p.mt == 4 && mtiles >= 4)) ? 128
                                                                 : (ctas(64) >= 120 ? 64 : 32);
  // Wave quantisation: a grid of one M tile that is a few CTAs larger than the machine would
  // run a second, almost empty wave.  The full wave runs as one launch; the last few weight
  // tiles follow as a split-K launch of their own, which occupies the SMs the tail left idle.
  if (!out_f32 && p.splits == 1 && p.nb == 128 && mtiles == 1 && !fused && ntiles > 148 &&
      ntiles % 148 > 0 && ntiles % 148 <= 40 && K / BK >= 8 && N % 128 == 0) {
    int ts = static_cast<int>(148 / (ntiles % 148));
    ts = ts > K / BK / 4 ? K / BK / 4 : ts;
    p.tail_splits = ts > 8 ? 8 : (ts < 1 ? 1 : ts);
  }
  return p;
}

// K splits of the tail launch (128-row tiles): fill the machine once, keep at least four
// k-blocks per split.
inline int tail_splits_for(int M, int K, int tail_tiles) {
  const long ctas = static_cast<long>(tail_tiles) * ((M + BM - 1) / BM);
  long ts = 148 / (ctas > 0 ? ctas : 1);
  ts = ts > K / BK / 4 ? K / BK / 4 : ts;
  return static_cast<int>(ts > 8 ? 8 : (ts < 1 ? 1 : ts));
}

template <int FMT>
int launch_fmt(const int8_t* a, const float* a_scale, const void* w, const __half* w_scale,
               void* out, int M, int N, int K, int out_f32, cudaStream_t stream,
               const PeerOut& po, const AgIn& ag = AgIn{nullptr, nullptr, 0, 0}) {
  const GroupDesc none{nullptr, nullptr, 0, 0};
  if (g_impl == 2 && M > BM && N >= 256) {
    if (out_f32) return launch_pair<FMT, true>(a, a_scale, w, w_scale, out, M, N, K, stream, po, ag);
    return launch_pair<FMT, false>(a, a_scale, w, w_scale, out, M, N, K, stream, po, ag);
  }
  const Plan plan = make_plan(FMT, M, N, K, out_f32, po.tp != 0);
  const int mt = plan.mt, nb = plan.nb, splits = plan.splits;
  if (plan.tail_splits > 0) {
    const long ntiles = (N + 127) / 128;
    const int tail_tiles = static_cast<int>(ntiles % 148);
    const int cut = static_cast<int>(ntiles - tail_tiles) * 128;
    // the tail runs as 128-row tiles: more CTAs of less work each, and small accumulator
    // tiles whose splits are added inside the kernel
    const int ts = tail_splits_for(M, K, tail_tiles);
#define ORINFER_TWO(MTV)                                                                        \
  {                                                                                             \
    const int r = launch<FMT, false, MTV, 128>(a, a_scale, w, w_scale, out, M, N, K, stream, po, \
                                               none, 1, 0, ag, 1, 0, cut);                     \
    if (r) return r;                                                                            \
    return launch<FMT, false, 1, 128>(a, a_scale, w, w_scale, out, M, N, K, stream, po, none,  \
                                      1, 0, ag, ts, cut, N);                                   \
  }
    if (mt == 4) ORINFER_TWO(4)
    if (mt == 2) ORINFER_TWO(2)
    ORINFER_TWO(1)
#undef ORINFER_TWO
  }
#define ORINFER_GO(F32, MTV, NBV)                                                              \
  return launch<FMT, F32, MTV, NBV>(a, a_scale, w, w_scale, out, M, N, K, stream, po, none, 1, \
                                    0, ag, splits)
  if (out_f32) {
    if (mt == 4) ORINFER_GO(true, 4, 128);
    if (mt == 2) ORINFER_GO(true, 2, 128);
    ORINFER_GO(true, 1, 128);
  }
  if (mt == 4) {
    if (nb == 128) ORINFER_GO(false, 4, 128);
    if (nb == 64) ORINFER_GO(false, 4, 64);
    ORINFER_GO(false, 4, 32);
  }
  if (mt == 2) {
    if (nb == 128) ORINFER_GO(false, 2, 128);
    if (nb == 64) ORINFER_GO(false, 2, 64);
    ORINFER_GO(false, 2, 32);
  }
  if (nb == 128) ORINFER_GO(false, 1, 128);
  if (nb == 64) ORINFER_GO(false, 1, 64);
  ORINFER_GO(false, 1, 32);
#undef ORINFER_GO
}

}  // namespace tc
}  // namespace orinfer

using namespace orinfer;

static int qgemm_any(int fmt, const int8_t* a, const float* a_scale, const void* w,
                     const __half* w_scale, void* out, int M, int N, int K, int out_f32,
                     int force_path, cudaStream_t stream, const PeerOut* peer) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 128 || N % 8 || fmt < 0 || fmt > 2) return -1;
  if (runtime_ensure_init() != cudaSuccess) return -2;
  const bool simt = force_path == 1 || (force_path == 0 && M <= 8);
  if (simt) {
    // The SIMT kernel takes at most 8 rows per launch (one launch when fused with peers,
    // because every launch bumps the peers' sequence flags).
    if (peer != nullptr && M > 8) return -1;
    for (int m = 0; m < M; m += 8) {
      const int rows = M - m < 8 ? M - m : 8;
      void* o = out_f32 ? static_cast<void*>(reinterpret_cast<float*>(out) + (size_t)m * N)
                        : static_cast<void*>(reinterpret_cast<__half*>(out) + (size_t)m * N);
      int r = qgemv_dispatch(fmt, a + (size_t)m * K, a_scale + m, w, w_scale, o, rows, N, K,
                             out_f32, stream, peer);
      if (r) return r;
    }
    return 0;
  }
  PeerOut po{};
  if (peer != nullptr) po = *peer;
  if (fmt == 0)
    return tc::launch_fmt<0>(a, a_scale, w, w_scale, out, M, N, K, out_f32, stream, po);
  if (fmt == 1)
    return tc::launch_fmt<1>(a, a_scale, w, w_scale, out, M, N, K, out_f32, stream, po);
  return tc::launch_fmt<2>(a, a_scale, w, w_scale, out, M, N, K, out_f32, stream, po);
}

// Number of kernel launches orinfer_qgemm makes for this shape and format.
extern "C" int orinfer_qgemm_launches_fmt(int fmt, int M, int N, int K, int out_f32,
                                          int force_path) {
  if (force_path == 1 || (force_path == 0 && M <= 8)) return (M + 7) / 8;
  const tc::Plan p = tc::make_plan(fmt, M, N, K, out_f32, false);
  // K splits are added up inside the one-tile kernel when the tiles are small; otherwise,
  // and in the persistent forms, a second pass adds them
  if (p.tail_splits > 0) {
    const int ts = tc::g_impl == 1
                       ? tc::tail_splits_for(M, K, static_cast<int>(((N + 127) / 128) % 148))
                       : p.tail_splits;
    const bool second = ts > 1 && !(tc::g_impl == 1 && tc::splitk_in_kernel(1, 128, ts));
    return second ? 3 : 2;
  }
  const bool second = p.splits > 1 && !(tc::g_impl == 1 && tc::splitk_in_kernel(p.mt, 128, p.splits));
  return second ? 2 : 1;
}

extern "C" int orinfer_qgemm_launches(int M, int N, int K, int out_f32, int force_path) {
  return orinfer_qgemm_launches_fmt(1, M, N, K, out_f32, force_path);
}

// Tuned launch variants: rows m_lo..m_hi of projection (fmt, N, K) run with M-tile factor mt
// (1, 2, 4), weight-tile width nb (128, 64, 32) and `splits` K splits.  Earlier entries win.
// The table is guarded by a mutex: launches on other threads read a consistent table.
extern "C" int orinfer_qgemm_set_variant(int fmt, int m_lo, int m_hi, int n, int k, int mt,
                                         int nb, int splits) {
  const tc::Variant v{fmt, m_lo, m_hi, n, k, mt, nb, splits};
  if (!tc::variant_valid(v)) return -1;
  std::lock_guard<std::mutex> lock(tc::g_variant_mutex);
  if (tc::g_variant_count >= tc::MAX_VARIANTS) return -2;
  tc::g_variants[tc::g_variant_count++] = v;
  return 0;
}

extern "C" void orinfer_qgemm_clear_variants() {
  std::lock_guard<std::mutex> lock(tc::g_variant_mutex);
  tc::g_variant_count = 0;
}

// 0 = persistent kernel, 1 = one tile per CTA (default), 2 = CTA pairs; for comparisons and tests.
// Timing experiments of the one-tile kernel: bit 0 no MMAs, bit 1 no operand copies, bit 2
// no lattice decode.  Outputs are meaningless while a bit is set.
extern "C" int orinfer_qgemm_set_probe(int bits) {
  tc::g_probe = bits & 1023;
  return 0;
}

extern "C" int orinfer_qgemm_set_impl(int impl) {
  if (impl < 0 || impl > 2) return -1;
  tc::g_impl = impl;
  return 0;
}

// The plan for a shape: out[0..3] = mt, nb, splits, tail_splits.
extern "C" void orinfer_qgemm_plan(int fmt, int M, int N, int K, int out_f32, int* out) {
  const tc::Plan p = tc::make_plan(fmt, M, N, K, out_f32, false);
  out[0] = p.mt;
  out[1] = p.nb;
  out[2] = p.splits;
  out[3] = p.tail_splits;
}

extern "C" int orinfer_qgemm(int fmt, const int8_t* a, const float* a_scale, const void* w,
                             const __half* w_scale, void* out, int M, int N, int K, int out_f32,
                             int force_path, cudaStream_t stream) {
  return qgemm_any(fmt, a, a_scale, w, w_scale, out, M, N, K, out_f32, force_path, stream,
                   nullptr);
}

extern "C" int orinfer_qgemm_peer(int fmt, const int8_t* a, const float* a_scale, const void* w,
                                  const __half* w_scale, const OrinferPeerOut* peer, int M, int N,
                                  int K, int force_path, cudaStream_t stream) {
  if (peer == nullptr || peer->tp < 1 || peer->tp > TP_MAX || M > peer->rows_cap) return -1;
  PeerOut po;
  for (int i = 0; i < TP_MAX; ++i) {
    po.inbox[i] = reinterpret_cast<__half*>(peer->inbox[i]);
    po.flag[i] = peer->flag[i];
  }
  po.sent = peer->sent;
  po.ticket = peer->ticket;
  po.tp = peer->tp;
  po.rank = peer->rank;
  po.rows_cap = peer->rows_cap;
  po.rows_per = peer->rows_per;
  if (po.rows_per < LL_MODE || (po.rows_per > 0 && (M <= 8 || force_path == 1))) return -1;
  if (po.rows_per == LL_MODE && (M > LL_ROWS || fmt == 0 || N % 16 || force_path == 2)) return -1;
  return qgemm_any(fmt, a, a_scale, w, w_scale, nullptr, M, N, K, 0, force_path, stream, &po);
}

extern "C" int orinfer_qgemm_ag(int fmt, const int8_t* a, const float* a_scale, const void* w,
                                const __half* w_scale, void* out, const OrinferAgIn* agp, int M,
                                int N, int K, int out_f32, cudaStream_t stream) {
  if (agp == nullptr || agp->tp < 1 || agp->tp > TP_MAX || agp->rows_per < 1) return -1;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 128 || N % 8 || fmt < 0 || fmt > 2) return -1;
  if (runtime_ensure_init() != cudaSuccess) return -2;
  const AgIn ag{agp->flag, agp->sent, agp->tp, agp->rows_per};
  const PeerOut po{};
  if (fmt == 0)
    return tc::launch_fmt<0>(a, a_scale, w, w_scale, out, M, N, K, out_f32, stream, po, ag);
  if (fmt == 1)
    return tc::launch_fmt<1>(a, a_scale, w, w_scale, out, M, N, K, out_f32, stream, po, ag);
  return tc::launch_fmt<2>(a, a_scale, w, w_scale, out, M, N, K, out_f32, stream, po, ag);
}

// Grouped expert GEMM: rows of `a` are sorted by expert; tile t of the table covers rows
// [first, first + valid) of expert e, multiplied with that expert's bank.  out is fp16 [S, N].
extern "C" int orinfer_qgemm_grouped(int fmt, const int8_t* a, const float* a_scale, const void* w,
                                     const __half* w_scale, void* out, int S, int N, int K,
                                     int experts, const int* tiles, const int* meta,
                                     int max_tiles, cudaStream_t stream) {
  if (S <= 0 || max_tiles <= 0) return 0;
  if (K <= 0 || K % 128 || N % 128 || fmt < 0 || fmt > 2 || experts < 1) return -1;
  if (runtime_ensure_init() != cudaSuccess) return -2;
  const long long bank = fmt == 0 ? static_cast<long long>(N) * K
                                  : static_cast<long long>(K / 128) * N * (fmt == 1 ? 64 : 32);
  tc::GroupDesc g{tiles, meta, bank, N};
  PeerOut po{};
  if (fmt == 0)
    return tc::launch<0, false, 1, 128>(a, a_scale, w, w_scale, out, S, N, K, stream, po, g, experts,
                                   max_tiles);
  if (fmt == 1)
    return tc::launch<1, false, 1, 128>(a, a_scale, w, w_scale, out, S, N, K, stream, po, g, experts,
                                   max_tiles);
  return tc::launch<2, false, 1, 128>(a, a_scale, w, w_scale, out, S, N, K, stream, po, g, experts,
                                 max_tiles);
}
