// Expert-parallel MoE with sharded tokens: the dispatch and combine all-to-alls as push
// kernels over NVLink peer memory, around the grouped expert GEMM.
//
//   token owner (rank s)                                expert owner (rank d)
//   router top-k, sort assignments by destination rank
//   a2a_dispatch_push: INT8 row + scale + expert id  -> recv[d][s][j]   (+ count, base, flag)
//                                                       a2a_recv_prepare: wait flags, void tail
//                                                       dispatch by expert, grouped gate_up GEMM,
//                                                       SwiGLU+rotate+quantise, grouped down GEMM
//   ret[s][base + j]                                 <- a2a_return_push: FP16 result rows (+ flag)
//   moe_combine (waits flags): sum_k prob * ret[slot] + gated shared expert
//
// Every region is sized for the worst case (all assignments of a rank to one destination:
// cap = owned rows x top_k), so no size negotiation precedes the payload; counts travel with
// the flag.  All waits are bounded and report through the status word.  Peers are written
// with plain stores; nothing here uses TMA multicast.
// Replaces collective call sites C2 / C6 of the reference's TP8 plans (routed transport
// gathers before the grouped expert matmul, FP32 all-reduce after the combine:
// python/orinfer_build/models/deepseek_v41/fuse_ffn_collectives.py:25-80, build.py:1355-1364)
// with true all-to-alls.
#include "api.h"
#include "common.cuh"
#include "tp_comm.cuh"

namespace orinfer {

struct A2aDispatch {
  int8_t* rows[TP_MAX];        // every rank's receive buffer: int8 [tp][cap][K]
  float* scale[TP_MAX];        // fp32 [tp][cap]
  int* expert[TP_MAX];         // int32 [tp][cap] global expert id of each received row
  int* header[TP_MAX];         // int32 [tp][2] = (count, base slot at the sender)
  int* flag[TP_MAX];           // int32 [tp]
  int* sent;
  unsigned int* ticket;
  int tp, rank, cap;
};

struct A2aReturn {
  __half* ret[TP_MAX];         // every rank's return buffer: fp16 [cap][H]
  int* flag[TP_MAX];           // int32 [tp]
  int* sent;
  unsigned int* ticket;
  int tp, rank, cap;
};

// One CTA per assignment (row, k) of the owned rows.  slots[] / offsets[] come from the local
// dispatch of the assignments by destination rank (stable in (row, k) order).
__global__ void __launch_bounds__(128) a2a_dispatch_push_kernel(
    const int* __restrict__ ids, const int* __restrict__ slots, const int* __restrict__ offsets,
    const int8_t* __restrict__ q8, const float* __restrict__ scale, int top_k, int K,
    int experts_per_rank, A2aDispatch a) {
  const int i = blockIdx.x;
  const int e = ids[i];
  const int dst = min(e / experts_per_rank, a.tp - 1);
  const int j = slots[i] - offsets[dst];
  const size_t at = static_cast<size_t>(a.rank) * a.cap + j;
  const int4* src = reinterpret_cast<const int4*>(q8 + static_cast<size_t>(i / top_k) * K);
  int4* out = reinterpret_cast<int4*>(a.rows[dst] + at * K);
  for (int c = threadIdx.x; c < K / 16; c += blockDim.x) out[c] = src[c];
  if (threadIdx.x == 0) {
    a.scale[dst][at] = scale[i / top_k];
    a.expert[dst][at] = e;
  }
  if (blockIdx.x == 0 && threadIdx.x < a.tp) {
    const int d = threadIdx.x;
    a.header[d][a.rank * 2 + 0] = offsets[d + 1] - offsets[d];
    a.header[d][a.rank * 2 + 1] = offsets[d];
  }
  signal_done(a.flag, a.sent, a.ticket, a.tp, a.rank, gridDim.x);
}

// Expert owner: wait (bounded) for every sender, then mark the unused tail of each sender's
// region as "no expert" so that the following dispatch-by-expert skips it.
__global__ void __launch_bounds__(256) a2a_recv_prepare_kernel(
    const int* __restrict__ flag, const int* __restrict__ sent, const int* __restrict__ header,
    int* __restrict__ expert, int tp, int cap, int* status) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    const int want = *reinterpret_cast<const volatile int*>(sent);
    int good = 1;
    for (int s = 0; s < tp && good; ++s) {
      const long long start = clock64(), limit = wait_limit(status);
      while (ld_acquire_sys(flag + s) < want) {
        if (clock64() - start > limit) {
          report_status(status, STATUS_PEER_WAIT, 0x200 | s);
          good = 0;
          break;
        }
      }
    }
    ok = good;
  }
  __syncthreads();
  const int total = tp * cap;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int s = i / cap, j = i % cap;
    const int count = ok ? __ldcg(header + s * 2) : 0;
    if (j >= count) expert[i] = -1;
  }
}

// Expert owner: one CTA per receive position; sends the FP16 result row of a valid position
// back to its sender, at the sender's own slot index.
__global__ void __launch_bounds__(128) a2a_return_push_kernel(
    const __half* __restrict__ down, const int* __restrict__ slots,
    const int* __restrict__ header, int H, A2aReturn a) {
  const int i = blockIdx.x;
  const int s = i / a.cap, j = i % a.cap;
  const int count = __ldcg(header + s * 2), base = __ldcg(header + s * 2 + 1);
  if (j < count) {
    const int slot = slots[i];
    if (slot >= 0) {
      const int4* src = reinterpret_cast<const int4*>(down + static_cast<size_t>(slot) * H);
      int4* out = reinterpret_cast<int4*>(a.ret[s] + static_cast<size_t>(base + j) * H);
      for (int c = threadIdx.x; c < H / 8; c += blockDim.x) out[c] = src[c];
    }
  }
  signal_done(a.flag, a.sent, a.ticket, a.tp, a.rank, gridDim.x);
}

// Token owner: waits (bounded) until every expert owner has returned its rows.
__global__ void a2a_wait_kernel(const int* __restrict__ flag, const int* __restrict__ sent,
                                int tp, int* status) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const int want = *reinterpret_cast<const volatile int*>(sent);
  for (int s = 0; s < tp; ++s) {
    const long long start = clock64(), limit = wait_limit(status);
    while (ld_acquire_sys(flag + s) < want) {
      if (clock64() - start > limit) {
        report_status(status, STATUS_PEER_WAIT, 0x300 | s);
        return;
      }
    }
  }
}

}  // namespace orinfer

using namespace orinfer;

extern "C" {

int orinfer_a2a_dispatch_push(const int* ids, const int* slots, const int* offsets,
                              const int8_t* q8, const float* scale, int rows, int top_k, int K,
                              int experts_per_rank, const OrinferA2aDispatch* d,
                              cudaStream_t stream) {
  if (d == nullptr || d->tp < 1 || d->tp > TP_MAX || rows <= 0 || rows * top_k > d->cap ||
      K % 16 || experts_per_rank < 1)
    return -1;
  A2aDispatch a;
  for (int i = 0; i < TP_MAX; ++i) {
    a.rows[i] = reinterpret_cast<int8_t*>(d->rows[i]);
    a.scale[i] = d->scale[i];
    a.expert[i] = d->expert[i];
    a.header[i] = d->header[i];
    a.flag[i] = d->flag[i];
  }
  a.sent = d->sent;
  a.ticket = d->ticket;
  a.tp = d->tp;
  a.rank = d->rank;
  a.cap = d->cap;
  a2a_dispatch_push_kernel<<<rows * top_k, 128, 0, stream>>>(ids, slots, offsets, q8, scale,
                                                            top_k, K, experts_per_rank, a);
  return static_cast<int>(cudaGetLastError());
}

// flag / sent / header / expert are this rank's own receive-side arrays.
int orinfer_a2a_recv_prepare(const int* flag, const int* sent, const int* header, int* expert,
                             int tp, int cap, cudaStream_t stream) {
  if (tp < 1 || tp > TP_MAX || cap < 1) return -1;
  if (runtime_ensure_init() != cudaSuccess) return -2;
  a2a_recv_prepare_kernel<<<64, 256, 0, stream>>>(flag, sent, header, expert, tp, cap,
                                                  runtime_status_ptr());
  return static_cast<int>(cudaGetLastError());
}

int orinfer_a2a_return_push(const __half* down, const int* slots, const int* header, int H,
                            const OrinferA2aReturn* r, cudaStream_t stream) {
  if (r == nullptr || r->tp < 1 || r->tp > TP_MAX || H % 8) return -1;
  A2aReturn a;
  for (int i = 0; i < TP_MAX; ++i) {
    a.ret[i] = reinterpret_cast<__half*>(r->ret[i]);
    a.flag[i] = r->flag[i];
  }
  a.sent = r->sent;
  a.ticket = r->ticket;
  a.tp = r->tp;
  a.rank = r->rank;
  a.cap = r->cap;
  a2a_return_push_kernel<<<r->tp * r->cap, 128, 0, stream>>>(down, slots, header, H, a);
  return static_cast<int>(cudaGetLastError());
}

int orinfer_a2a_wait(const int* flag, const int* sent, int tp, cudaStream_t stream) {
  if (tp < 1 || tp > TP_MAX) return -1;
  if (runtime_ensure_init() != cudaSuccess) return -2;
  a2a_wait_kernel<<<1, 32, 0, stream>>>(flag, sent, tp, runtime_status_ptr());
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
