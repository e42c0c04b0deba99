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

constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;   // about one second

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
// Bounded wait; false (and a status record) when the phase never completes.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code,
                                          int detail) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - start > WAIT_LIMIT_CYCLES) {
      report_status(status, code, detail);
      return false;
    }
  }
  return true;
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
// Global table (2 KiB): pos[index] = {lo, hi}, four packed bytes each, holding basis + 24,
// so every byte is in 14..34 and whole-word arithmetic never carries between bytes; the
// negated coordinates are 48 - pos, again without borrows.  A code's sign byte picks
// pos/neg per coordinate with one PRMT per half; the selectors come from a 256-entry
// table indexed by the sign byte.  The +/-1 parity shift and the re-centring are one
// constant added afterwards, and XOR 0x80 turns the biased byte into two's complement.
struct E8pTables {
  uint2 pos[256];
};

// Shared-memory working copy: the value table plus PRMT selectors per sign byte
// (low half-word: coordinates 0-3, high half-word: coordinates 4-7).
struct E8pSmem {
  uint2 pos[256];
  uint32_t sel[256];
};

// Host-side runtime singletons (runtime.cu): device status word and decode tables.
int* runtime_status_ptr();
// INT32 partial accumulators of split-K GEMMs: [splits][M][N], allocated once at start-up so
// that no launch ever allocates (captured graphs keep the address).
constexpr size_t SPLITK_WORKSPACE_BYTES = 96ull << 20;
int* runtime_splitk_workspace();
const E8pTables* runtime_e8p_tables();
cudaError_t runtime_ensure_init();

__device__ __forceinline__ void e8p_smem_init(E8pSmem* sm, const E8pTables* __restrict__ g,
                                              int tid, int nthreads) {
  for (int i = tid; i < 256; i += nthreads) {
    sm->pos[i] = g->pos[i];
    const uint32_t t = static_cast<uint32_t>(i) ^ (__popc(i) & 1u), t2 = t >> 2;
    // coordinate c flips with bit {0,4,1,5,2,6,3,7}[c]; nibble j of a PRMT selector is
    // j (take the "pos" byte) or j + 4 (take the "neg" byte)
    const uint32_t lo = 0x3210u | ((t & 0x11u) << 2) | ((t & 0x22u) << 9);
    const uint32_t hi = 0x3210u | ((t2 & 0x11u) << 2) | ((t2 & 0x22u) << 9);
    sm->sel[i] = lo | (hi << 16);
  }
}

// -> biased coordinate bytes (+/-basis + 24) and the parity bit of one 16-bit code
__device__ __forceinline__ void e8p_select(uint32_t code, const E8pSmem* __restrict__ sm,
                                           uint32_t& lo, uint32_t& hi, uint32_t& par) {
  const uint32_t s = code & 0xffu;
  par = __popc(s) & 1u;
  const uint2 e = sm->pos[(code >> 8) & 0xffu];
  const uint32_t sl = sm->sel[s];
  lo = __byte_perm(e.x, 0x30303030u - e.x, sl);
  hi = __byte_perm(e.y, 0x30303030u - e.y, sl >> 16);
}

// One 16-bit code -> eight INT8 weights  (+/-basis) + (1 - 2*parity).
__device__ __forceinline__ uint2 e8p_decode8(uint32_t code, const E8pSmem* __restrict__ sm) {
  uint32_t lo, hi, par;
  e8p_select(code, sm, lo, hi, par);
  const uint32_t cw = 0x69696969u - par * 0x02020202u;          // 128 - 24 + shift
  return make_uint2((lo + cw) ^ 0x80808080u, (hi + cw) ^ 0x80808080u);
}

// One Q4 word (coarse U16 low, residual U16 high) -> eight INT8 weights 4*q0 + q1.
__device__ __forceinline__ uint2 e8p_decode_q4(uint32_t word, const E8pSmem* __restrict__ sm) {
  uint32_t l0, h0, p0, l1, h1, p1;
  e8p_select(word & 0xffffu, sm, l0, h0, p0);
  e8p_select(word >> 16, sm, l1, h1, p1);
  // 4*(b0+24) + (b1+24) + c = 4*q0 + q1 + 128  with  c = 128 - 120 + 4*s0 + s1
  const uint32_t cw = 0x0d0d0d0du - p0 * 0x08080808u - p1 * 0x02020202u;
  return make_uint2(((l0 << 2) + l1 + cw) ^ 0x80808080u, ((h0 << 2) + h1 + cw) ^ 0x80808080u);
}

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
