// Device-side plumbing of the fused tensor-parallel kernels: peer inboxes reached with
// plain stores over NVLink (no TMA multicast anywhere), per-source sequence flags, and
// bounded waits.  Protocol for one fused "row-parallel GEMM -> all-reduce" step:
//   producer (GEMM epilogue, every rank): write the FP16 partial tile into slot [my rank] of
//     every peer's inbox; fence; the last CTA of the grid bumps its local `sent` counter and
//     stores the new value into flag[my rank] on every peer (release, system scope);
//   consumer (the next norm/quantise kernel, every rank): wait (bounded, acquire, system
//     scope) until flag[src] > seen for every src, then sum the tp partial rows in fixed
//     source order (bit-reproducible) with L1-bypassing loads; its last CTA bumps `seen`.
// Every rank runs the same sequence of fused ops, so the counters stay aligned without
// any reset, also across CUDA-graph replays (all counters live in device memory).
#pragma once

#include "common.cuh"

namespace orinfer {

constexpr int TP_MAX = 8;

struct PeerOut {                 // producer side
  __half* inbox[TP_MAX];         // base of each rank's inbox (peer-mapped), [tp][rows_cap][n]
  int* flag[TP_MAX];             // each rank's flag array for this op, [tp]
  int* sent;                     // local: sequence number of the last completed send
  unsigned int* ticket;          // local: CTA completion counter
  int tp, rank, rows_cap;
};

struct InboxIn {                 // consumer side
  const __half* inbox;           // local inbox, [tp][rows_cap][n]
  const int* flag;               // local flag array, [tp]
  int* seen;                     // local: sequence number consumed so far
  unsigned int* ticket;          // local: CTA completion counter
  int tp, rows_cap;
};

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Called by every thread of a producer CTA after its peer stores.  Returns after the
// last CTA of the grid has published the new sequence number to all peers.
__device__ __forceinline__ void peer_signal_done(const PeerOut& po, unsigned int total_ctas) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(po.ticket, 1u);
    if (t == total_ctas - 1) {
      *po.ticket = 0;
      __threadfence_system();
      const int v = *po.sent + 1;
      *po.sent = v;
      for (int d = 0; d < po.tp; ++d) st_release_sys(po.flag[d] + po.rank, v);
    }
  }
}

// Thread 0 of a consumer CTA waits for every source; false when a wait ran out.
__device__ __forceinline__ bool inbox_wait(const InboxIn& in, int* status) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) {
    const int want = *reinterpret_cast<volatile int*>(in.seen) + 1;
    int ok = 1;
    for (int s = 0; s < in.tp && ok; ++s) {
      if (ld_acquire_sys(in.flag + s) >= want) continue;
      const long long start = clock64();
      while (ld_acquire_sys(in.flag + s) < want) {
        if (clock64() - start > WAIT_LIMIT_CYCLES) {
          report_status(status, STATUS_PEER_WAIT, s);
          ok = 0;
          break;
        }
      }
    }
    ok_flag = ok;
  }
  __syncthreads();
  return ok_flag != 0;
}

__device__ __forceinline__ void inbox_consumed(const InboxIn& in, unsigned int total_ctas) {
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(in.ticket, 1u);
    if (t == total_ctas - 1) {
      *in.ticket = 0;
      __threadfence();
      *in.seen = *in.seen + 1;
    }
  }
}

}  // namespace orinfer
