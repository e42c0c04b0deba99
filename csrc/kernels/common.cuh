// Shared device helpers for the sm_100a kernels: bounded mbarrier waits, TMA and
// tcgen05 PTX wrappers, UMMA descriptors, the E8P lattice decoder and small math
// utilities.  Every wait in this file is bounded: after WAIT_LIMIT_CYCLES it
// records an error code in g_orinfer_status and returns false so the caller can
// leave its loop, drain its copies and free its TMEM instead of spinning forever.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace orinfer {

// Status word (device memory owned by the host runtime, passed to kernels that
// can wait): 0 = ok, otherwise (code << 16) | detail of the first failed bounded
// wait or rejected index.  Read back with orinfer_read_status().

// Bounded waits give up after status[2] * 1024 clock cycles (set at start-up and by
// orinfer_set_wait_limit_us; about one second by default); kernels that get no status pointer
// use the default.
constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;   // about one second
constexpr int STATUS_LIMIT_WORD = 2;

__device__ __forceinline__ long long wait_limit(const int* status) {
  if (status == nullptr) return WAIT_LIMIT_CYCLES;
  const int k = *reinterpret_cast<const volatile int*>(status + STATUS_LIMIT_WORD);
  return k > 0 ? static_cast<long long>(k) << 10 : WAIT_LIMIT_CYCLES;
}

enum StatusCode : int {
  STATUS_OK = 0,
  STATUS_TMA_WAIT = 1,
  STATUS_MMA_WAIT = 2,
  STATUS_EPILOGUE_WAIT = 3,
  STATUS_DECODE_WAIT = 4,
  STATUS_PEER_WAIT = 5,
  STATUS_BAD_INDEX = 6,
};

__device__ __forceinline__ void report_status(int* status, int code, int detail) {
  if (status != nullptr) atomicCAS(status, 0, (code << 16) | (detail & 0xffff));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait; false (and a status record) when the phase never completes.  The clock and
// the limit (a global load) are only touched every 256 failed polls, so a wait that is
// satisfied within microseconds costs nothing but the polls.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code,
                                          int detail) {
  long long start = 0, limit = 0;
  for (uint32_t spins = 1;; ++spins) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spins & 255u) == 0) {
      if (limit == 0) {
        limit = wait_limit(status);
        start = clock64();
      } else if (clock64() - start > limit) {
        report_status(status, code, detail);
        return false;
      }
    }
  }
}
// Same, for kernels whose roles must all leave when one of them gave up: `abort` is a word
// in shared memory that the first failed wait sets and every other wait polls.
__device__ __forceinline__ bool mbar_wait_abortable(uint64_t* bar, uint32_t parity, int* status,
                                                    int code, int detail, volatile int* abort) {
  long long start = 0, limit = 0;
  for (uint32_t spins = 1;; ++spins) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spins & 63u) == 0) {
      if (*abort != 0) return false;
      if ((spins & 255u) == 0) {
        if (limit == 0) {
          limit = wait_limit(status);
          start = clock64();
        } else if (clock64() - start > limit) {
          report_status(status, code, detail);
          *abort = 1;
          return false;
        }
      }
    }
  }
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, uint64_t* bar, int x,
                                            int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* tmap, uint64_t* bar, int x,
                                            int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// Untiled bulk copy global -> shared; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(smem_u32(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
// Make generic-proxy shared-memory writes visible to the async proxy (TMA / tcgen05).
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Order earlier generic-proxy accesses (here: an acquire of data that peers stored to global
// memory) before later async-proxy accesses (TMA loads of that memory), all state spaces.
__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

// ---------------------------------------------------------------- tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_slot)),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; one thread issues for the whole CTA.
__device__ __forceinline__ void mma_i8_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_f16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// ---------------------------------------------------------------- CTA pairs (cta_group::2)
// Two CTAs of a cluster drive one MMA of 256 rows: each holds its 128 rows of A and its half
// of the B rows in its own shared memory, the even CTA issues the instruction, and each
// CTA's TMEM receives its 128 rows of the accumulator.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local` (a shared::cta address) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(
                   cluster_addr),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_slot)),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void mma_i8_ss_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Completion of all earlier MMAs of this thread arrives on the barrier at the same offset in
// every CTA of `cta_mask` (no data moves: this is a barrier signal, not a multicast load).
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(smem_u32(bar)),
      "h"(cta_mask)
      : "memory");
}
// TMA tile load of a CTA pair: the data lands in this CTA's shared memory, the bytes are
// counted on the barrier `bar_cluster_addr` (the even CTA's).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const void* tmap,
                                                 uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns; thread i of the warp receives lane
// (taddr.lane + i).  A warp may only touch the lane quadrant (warp_id % 4).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(
          taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
      "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
      "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
      "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// Shared-memory matrix descriptor (SM100 format, version 1).  Byte offsets are
// stored without their four low bits.
//   K-major  SWIZZLE_128B: rows are 128 bytes, 8-row groups 1024 bytes apart (SBO).
//   MN-major SWIZZLE_128B: LBO = distance between 64-element MN blocks,
//                          SBO = distance between 8-row K groups.
constexpr uint64_t UMMA_SWIZZLE_128B = 2;
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes,
                                              uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3ffff) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= 1ull << 46;                       // descriptor version for sm_100
  d |= UMMA_SWIZZLE_128B << 61;
  return d;
}

// Instruction descriptor (dense, no negate, no saturate).
//   c_format: 0 F16, 1 F32, 2 S32;  a/b_format: i8 kind 1 = signed; f16 kind 0 = F16, 1 = BF16
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t c_fmt, uint32_t a_fmt, uint32_t b_fmt,
                                                  uint32_t a_mn_major, uint32_t b_mn_major,
                                                  uint32_t m, uint32_t n) {
  return (c_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16) |
         ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Byte offset of logical (row, 16-byte chunk) inside a 128-byte-swizzled tile
// whose rows are 128 bytes and whose base is 1024-byte aligned.
__device__ __forceinline__ uint32_t swz128(uint32_t row, uint32_t chunk) {
  return row * 128u + ((chunk ^ (row & 7u)) << 4);
}

// ---------------------------------------------------------------- E8P decode
// A 16-bit code is (basis index << 8) | sign byte.  Two 256-entry tables of 32-bit words hold
// eight 4-bit fields each, one per coordinate: field 2j is coordinate j, field 2j+1 is
// coordinate 4+j, so that `v & 0x0f0f0f0f` and `(v >> 4) & 0x0f0f0f0f` are the two groups
// of four coordinates as bytes in k order.
//   e2[index]: 2*u per coordinate, u = (basis + 14) / 4 in 1..6; negating a coordinate is
//              u -> 7 - u = u ^ 7
//   sg[signs]: 0xE per flipped coordinate, plus (1 - parity) in bit 0 of every field
//   v = e2[index] ^ sg[signs] = 2*(u ^ 7*flip) + (1 - parity)   and the decoded coordinate
//   is 2*v - 15 (the +/-1 parity shift is folded into bit 0).
// One lookup pair and one XOR decode a code; the formats then combine whole words:
//   Q4 weight 4*c0 + c1 = 8*v0 + 2*v1 - 75,   Q2 weight = 2*v - 15.
struct E8pTables {
  uint32_t e2[256];
  uint32_t sg[256];
};

// Shared-memory working copy: COPIES replicas interleaved word by word, lane l reads replica
// l % COPIES.  The lookups of a warp are random in the entry index; with one copy they
// collide on the 32 banks about 3.5-fold, with 8 copies about 2-fold, with 32 copies never.
template <int COPIES>
struct E8pLut {
  uint32_t e2[256 * COPIES];
  uint32_t sg[256 * COPIES];
};

template <int COPIES>
__device__ __forceinline__ void e8p_lut_init(E8pLut<COPIES>* sm, const E8pTables* __restrict__ g,
                                             int tid, int nthreads) {
  static_assert(COPIES % 4 == 0, "filled with 16-byte stores");
  constexpr int PER = COPIES / 4;                       // 16-byte stores per entry
  for (int j = tid; j < 256 * PER; j += nthreads) {
    const int i = j / PER;
    const uint32_t a = g->e2[i], b = g->sg[i];
    reinterpret_cast<uint4*>(sm->e2)[j] = make_uint4(a, a, a, a);
    reinterpret_cast<uint4*>(sm->sg)[j] = make_uint4(b, b, b, b);
  }
}

// The 4-bit fields v of the code in the low (HALF = 0) or high (HALF = 1) half of `word`.
template <int COPIES, int HALF>
__device__ __forceinline__ uint32_t e8p_fields(uint32_t word, const E8pLut<COPIES>* __restrict__ sm,
                                               int copy) {
  const uint32_t idx = __byte_perm(word, 0, HALF ? 0x4443 : 0x4441);
  const uint32_t sgn = __byte_perm(word, 0, HALF ? 0x4442 : 0x4440);
  return sm->e2[idx * COPIES + copy] ^ sm->sg[sgn * COPIES + copy];
}

constexpr uint32_t E8P_NIB = 0x0f0f0f0fu;

// One Q4 word (coarse U16 low, residual U16 high) -> eight INT8 weights 4*c0 + c1.
template <int COPIES>
__device__ __forceinline__ uint2 e8p_decode_q4(uint32_t word, const E8pLut<COPIES>* __restrict__ sm,
                                               int copy) {
  const uint32_t v0 = e8p_fields<COPIES, 0>(word, sm, copy);
  const uint32_t v1 = e8p_fields<COPIES, 1>(word, sm, copy);
  // biased byte 8*v0 + 2*v1 + (128 - 75) is in 73..183: no carries; XOR 0x80 -> two's complement
  uint32_t lo = (v0 & E8P_NIB) * 8u + 0x35353535u;
  lo = ((v1 & E8P_NIB) * 2u + lo) ^ 0x80808080u;
  uint32_t hi = ((v0 >> 4) & E8P_NIB) * 8u + 0x35353535u;
  hi = (((v1 >> 4) & E8P_NIB) * 2u + hi) ^ 0x80808080u;
  return make_uint2(lo, hi);
}

// One Q2 code (HALF of `word`) -> eight INT8 weights 2*v - 15.
template <int COPIES, int HALF>
__device__ __forceinline__ uint2 e8p_decode8(uint32_t word, const E8pLut<COPIES>* __restrict__ sm,
                                             int copy) {
  const uint32_t v = e8p_fields<COPIES, HALF>(word, sm, copy);
  return make_uint2(((v & E8P_NIB) * 2u + 0x71717171u) ^ 0x80808080u,
                    (((v >> 4) & E8P_NIB) * 2u + 0x71717171u) ^ 0x80808080u);
}

// Host-side runtime state, one set per device (runtime.cu): the status word that bounded
// waits report into, the decode tables, and start-up workspaces (no launch ever allocates,
// so captured graphs keep the addresses).  The accessors return the current device's set.
int* runtime_status_ptr();
// INT32 partial accumulators of split-K GEMMs: [splits][M][N].
constexpr size_t SPLITK_WORKSPACE_BYTES = 96ull << 20;
int* runtime_splitk_workspace();
// One arrival counter per output tile of a split-K GEMM whose last-arriving CTA adds the
// splits itself; zero between launches (the last arriver clears its counter).
constexpr int SPLITK_TICKETS = 1 << 14;
int* runtime_splitk_tickets();
// Zero-initialised INT32 accumulators [8][GEMV_WS_COLS] + tickets of the K-split GEMV; every
// launch leaves them zero again.
constexpr int GEMV_WS_COLS = 1 << 18;
constexpr int GEMV_WS_TICKETS = 1024;
int* runtime_gemv_workspace();
const E8pTables* runtime_e8p_tables();
cudaError_t runtime_ensure_init();
// True the first time it is called for (current device, slot); kernels use it to set their
// dynamic shared-memory attribute once per device.
bool runtime_first_use(int slot);
int runtime_new_slot();

// ---------------------------------------------------------------- math
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Sum or maximum over the CTA; `red` is 32 floats of shared memory.  Every thread gets the
// result.  (For maxima of non-negative values.)
__device__ __forceinline__ float block_reduce(float v, float* red, bool is_max) {
  v = is_max ? warp_max(v) : warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = (lane < nw) ? red[lane] : 0.f;
  r = is_max ? warp_max(r) : warp_sum(r);
  return r;
}

// Signed block-128 Hadamard rotation of one block held as floats, in place: lane l holds
// channels 4l..4l+3.  Returns the largest magnitude of the lane's four results.  Shared by
// every kernel that rotates activations, so the bits do not depend on the kernel.
__device__ __forceinline__ float hadamard128_regs(float& v0, float& v1, float& v2, float& v3,
                                                  char4 sg, int lane) {
  v0 *= sg.x; v1 *= sg.y; v2 *= sg.z; v3 *= sg.w;
  float t0 = v0 + v1, t1 = v0 - v1, t2 = v2 + v3, t3 = v2 - v3;      // h = 1
  v0 = t0 + t2; v2 = t0 - t2; v1 = t1 + t3; v3 = t1 - t3;            // h = 2
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {                                   // h = 4 .. 64
    const float o0 = __shfl_xor_sync(0xffffffffu, v0, m);
    const float o1 = __shfl_xor_sync(0xffffffffu, v1, m);
    const float o2 = __shfl_xor_sync(0xffffffffu, v2, m);
    const float o3 = __shfl_xor_sync(0xffffffffu, v3, m);
    const bool hi = (lane & m) != 0;
    v0 = hi ? o0 - v0 : v0 + o0;
    v1 = hi ? o1 - v1 : v1 + o1;
    v2 = hi ? o2 - v2 : v2 + o2;
    v3 = hi ? o3 - v3 : v3 + o3;
  }
  const float c = 0.08838834764831845f;                                // 128^-1/2
  v0 *= c; v1 *= c; v2 *= c; v3 *= c;
  return fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3)));
}
__device__ __forceinline__ float hadamard128_inplace(float* block, const int8_t* signs, int lane) {
  float* p = block + lane * 4;
  const char4 sg = *reinterpret_cast<const char4*>(signs + lane * 4);
  float v0 = p[0], v1 = p[1], v2 = p[2], v3 = p[3];
  const float amax = hadamard128_regs(v0, v1, v2, v3, sg, lane);
  p[0] = v0; p[1] = v1; p[2] = v2; p[3] = v3;
  return amax;
}

// Sum of squares of the lane's four values of a block (same order as block128_sumsq).
__device__ __forceinline__ float block128_sumsq_regs(float v0, float v1, float v2, float v3) {
  float s = __fmul_rn(v0, v0);
  s = __fmaf_rn(v1, v1, s);
  s = __fmaf_rn(v2, v2, s);
  s = __fmaf_rn(v3, v3, s);
  return warp_sum(s);
}

// Sum of squares of one 128-channel block held as floats: lane l covers channels 4l..4l+3
// in order, then a butterfly over the warp.  Every kernel that normalises rows uses this
// function, so the sum does not depend on which kernel (or launch shape) computed it.
__device__ __forceinline__ float block128_sumsq(const float* block, int lane) {
  const float4 v = *reinterpret_cast<const float4*>(block + lane * 4);
  float s = __fmul_rn(v.x, v.x);
  s = __fmaf_rn(v.y, v.y, s);
  s = __fmaf_rn(v.z, v.z, s);
  s = __fmaf_rn(v.w, v.w, s);
  return warp_sum(s);
}
__device__ __forceinline__ float round_f16(float v) { return __half2float(__float2half_rn(v)); }

// Activation scale law: FP16 value of max(amax/127, 2^-24), or 1 for an all-zero row.
__device__ __forceinline__ float a8_scale(float amax) {
  if (!(amax > 0.f)) return 1.f;
  return round_f16(fmaxf(__fdiv_rn(amax, 127.f), 5.9604644775390625e-08f));
}
__device__ __forceinline__ int a8_code(float v, float scale) {
  float r = rintf(__fdiv_rn(v, scale));
  r = fminf(127.f, fmaxf(-127.f, r));
  return static_cast<int>(r);
}

}  // namespace orinfer
