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
//
// Sequence-parallel form of the same step (prefill packets), bytes over NVLink cut by tp:
//   reduce-scatter: rows are split into contiguous ranges of `rows_per`; the GEMM epilogue
//     stores row m only into the inbox of its owner rank m / rows_per;
//   the owner's norm kernel sums the tp partials of ITS rows, adds its residual slice,
//     normalises, rotates, quantises and
//   all-gathers by push: stores the INT8 row + scale into every rank's activation buffer and
//     publishes a second sequence flag; the next column-parallel GEMM waits (bounded) on the
//     flags of the source ranks covering its M tile before its first TMA load of A.
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
  int rows_per;                  // 0: all-reduce push to every rank; > 0: row m -> rank m / rows_per
};

struct AgOut {                   // all-gather by push (producer: the owner's norm kernel)
  int8_t* q[TP_MAX];             // every rank's activation buffer, int8 [rows_cap][K]
  float* scale[TP_MAX];          // every rank's row scales, fp32 [rows_cap]
  int* flag[TP_MAX];             // every rank's all-gather flag array, [tp]
  int* sent;                     // local sequence counter
  unsigned int* ticket;          // local CTA counter
  int tp, rank, rows_per;        // tp == 0: not sequence-parallel
};

struct AgIn {                    // consumer: the column-parallel GEMM
  const int* flag;               // local all-gather flag array, [tp]
  const int* sent;               // local counter written by the norm kernel that ran just
                                 // before on this stream: the sequence number to wait for
  int tp, rows_per;              // tp == 0: operand is local, no wait
};

struct InboxIn {                 // consumer side
  const __half* inbox;           // local inbox, [tp][rows_cap][n]
  const int* flag;               // local flag array, [tp]
  int* seen;                     // local: sequence number consumed so far
  unsigned int* ticket;          // local: CTA completion counter
  int tp, rows_cap;
  const uint2* ll;               // non-null: low-latency form, [tp][LL_ROWS][n / 2] units;
                                 // `seen` / `ticket` are then the LL counters
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
__device__ __forceinline__ void signal_done(int* const* flag, int* sent, unsigned int* ticket,
                                            int tp, int rank, unsigned int total_ctas) {
  // The barrier orders every thread's peer stores before thread 0; its system-scope fence
  // is cumulative over them, so one fence per CTA is enough (a fence per thread costs
  // microseconds on a grid of hundreds of CTAs).
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int t = atomicAdd(ticket, 1u);
    if (t == total_ctas - 1) {
      *ticket = 0;
      __threadfence_system();
      const int v = *sent + 1;
      *sent = v;
      for (int d = 0; d < tp; ++d) st_release_sys(flag[d] + rank, v);
    }
  }
}
__device__ __forceinline__ void peer_signal_done(const PeerOut& po, unsigned int total_ctas) {
  signal_done(po.flag, po.sent, po.ticket, po.tp, po.rank, total_ctas);
}
__device__ __forceinline__ void ag_signal_done(const AgOut& ag, unsigned int total_ctas) {
  signal_done(ag.flag, ag.sent, ag.ticket, ag.tp, ag.rank, total_ctas);
}

// One thread: wait (bounded) until the source ranks owning rows [m_lo, m_hi] have published
// the current all-gather; false when a wait ran out.
__device__ __forceinline__ bool ag_wait(const AgIn& in, int m_lo, int m_hi, int* status) {
  const int want = *reinterpret_cast<const volatile int*>(in.sent);
  const int s_hi = min(m_hi / in.rows_per, in.tp - 1);
  for (int s = m_lo / in.rows_per; s <= s_hi; ++s) {
    if (ld_acquire_sys(in.flag + s) >= want) continue;
    const long long start = clock64(), limit = wait_limit(status);
    while (ld_acquire_sys(in.flag + s) < want) {
      if (clock64() - start > limit) {
        report_status(status, STATUS_PEER_WAIT, 0x100 | s);
        return false;
      }
    }
  }
  return true;
}

// ---- low-latency form for decode-sized packets (<= 8 rows): no flag, no fence.  Every
// 8-byte unit carries two FP16 values and the sequence number of the step, so data and
// "ready" arrive in the same NVLink store; the consumer spins (bounded) on the units it needs.
// PeerOut.rows_per == LL_MODE selects it; PeerOut.inbox[] then point at the LL regions
// (uint2 [tp][LL_ROWS][n / 2], zero-initialised, sequence numbers only ever grow) and
// `sent` / `ticket` are the LL counters.
constexpr int LL_MODE = -1;
constexpr int LL_ROWS = 8;

__device__ __forceinline__ void ll_store8(const PeerOut& po, int seq, int m, int n, int N,
                                          const __half* h) {
  const uint32_t* w = reinterpret_cast<const uint32_t*>(h);
  const uint4 lo = make_uint4(w[0], static_cast<uint32_t>(seq), w[1], static_cast<uint32_t>(seq));
  const uint4 hi = make_uint4(w[2], static_cast<uint32_t>(seq), w[3], static_cast<uint32_t>(seq));
  const size_t unit = (static_cast<size_t>(po.rank) * LL_ROWS + m) * (N / 2) + n / 2;
  for (int d = 0; d < po.tp; ++d) {
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint2*>(po.inbox[d]) + unit);
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(lo.x),
                 "r"(lo.y), "r"(lo.z), "r"(lo.w) : "memory");
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 1), "r"(hi.x),
                 "r"(hi.y), "r"(hi.z), "r"(hi.w) : "memory");
  }
}

// Last CTA of the producer grid records the sequence number it used (local, no fence: the
// consumer learns readiness from the data itself).
__device__ __forceinline__ void ll_done(const PeerOut& po, int seq, unsigned int total_ctas) {
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(po.ticket, 1u);
    if (t == total_ctas - 1) {
      *po.ticket = 0;
      *po.sent = seq;
    }
  }
}

// Two units (four FP16 values) of source s; spins until both carry `seq` (bounded).
__device__ __forceinline__ bool ll_load4(const uint2* base, int seq, uint32_t& a, uint32_t& b,
                                         int* status, int s) {
  long long start = 0, limit = 0;
  for (uint32_t spins = 1;; ++spins) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(base) : "memory");
    if (static_cast<int>(v.y) == seq && static_cast<int>(v.w) == seq) {
      a = v.x;
      b = v.z;
      return true;
    }
    if ((spins & 63u) == 0) {             // clock and limit only once the wait is a long one
      if (limit == 0) {
        limit = wait_limit(status);
        start = clock64();
      } else if (clock64() - start > limit) {
        report_status(status, STATUS_PEER_WAIT, 0x400 | s);
        a = b = 0;
        return false;
      }
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
      const long long start = clock64(), limit = wait_limit(status);
      while (ld_acquire_sys(in.flag + s) < want) {
        if (clock64() - start > limit) {
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
