// Greedy token of a vocabulary-sharded head without a collective call: every rank pushes
// (local maximum, global token id) of each row into slot [rank] of every peer's table with
// one 16-byte store that also carries the step's sequence number, then reads the tp slots of
// its own table as they arrive and keeps the largest value, the lowest id on ties; a rank
// whose row was invalid (non-finite logits) invalidates the row everywhere.  Every rank
// computes the same token, so nothing is sent back.  Replaces the per-step all_gather +
// tensor ops of the NCCL arm; role of the reference's cross-rank best reduction
// (kernels/ascend/topk.py:74-100 reduce_rank_best).
#include "api.h"
#include "common.cuh"
#include "tp_comm.cuh"

namespace orinfer {

struct HeadMerge {
  uint4* table[TP_MAX];        // every rank's table (peer-mapped): uint4 [tp][cap]
  int* seq;                    // local: sequence number of the last completed merge
  int tp, rank, cap;
};

__global__ void __launch_bounds__(128) tp_head_merge_kernel(
    const float* __restrict__ logits, const int* __restrict__ local_tok, int rows, int vocab_local,
    int vocab0, HeadMerge hm, int* __restrict__ token_out, int* status) {
  const int seq = *reinterpret_cast<volatile int*>(hm.seq) + 1;
  for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < rows;
       row += gridDim.x * blockDim.x) {
    const int lt = local_tok[row];
    float val = -INFINITY;
    int gid = -1;
    if (lt >= 0 && lt < vocab_local) {
      val = logits[static_cast<size_t>(row) * vocab_local + lt];
      gid = lt + vocab0;
    }
    const uint32_t bits = __float_as_uint(val);
    for (int d = 0; d < hm.tp; ++d) {
      uint4* dst = hm.table[d] + static_cast<size_t>(hm.rank) * hm.cap + row;
      asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(bits),
                   "r"(static_cast<uint32_t>(gid)), "r"(static_cast<uint32_t>(seq)),
                   "r"(static_cast<uint32_t>(seq))
                   : "memory");
    }
    float best = -INFINITY;
    int best_id = 0x7fffffff;
    bool bad = false;
    for (int s = 0; s < hm.tp; ++s) {
      const uint4* src = hm.table[hm.rank] + static_cast<size_t>(s) * hm.cap + row;
      uint4 v;
      long long start = 0, limit = 0;
      for (uint32_t spins = 1;; ++spins) {
        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src) : "memory");
        if (static_cast<int>(v.z) == seq && static_cast<int>(v.w) == seq) break;
        if ((spins & 63u) == 0) {
          if (limit == 0) {
            limit = wait_limit(status);
            start = clock64();
          } else if (clock64() - start > limit) {
            report_status(status, STATUS_PEER_WAIT, 0x500 | s);
            v = make_uint4(0, 0xffffffffu, 0, 0);
            break;
          }
        }
      }
      const float ov = __uint_as_float(v.x);
      const int oi = static_cast<int>(v.y);
      if (oi < 0) bad = true;
      else if (ov > best || (ov == best && oi < best_id)) {
        best = ov;
        best_id = oi;
      }
    }
    token_out[row] = bad ? -1 : best_id;
  }
  // one CTA grid-strides over the rows: its last thread to finish publishes the sequence
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x == 0) *hm.seq = seq;
}

}  // namespace orinfer

using namespace orinfer;

extern "C" int orinfer_tp_head_merge(const float* logits, const int* local_tok, int rows,
                                     int vocab_local, int vocab0, const OrinferHeadMerge* h,
                                     int* token_out, cudaStream_t stream) {
  if (h == nullptr || h->tp < 1 || h->tp > TP_MAX || rows < 0 || rows > h->cap) return -1;
  if (rows == 0) return 0;
  if (runtime_ensure_init() != cudaSuccess) return -2;
  HeadMerge hm;
  for (int i = 0; i < TP_MAX; ++i) hm.table[i] = reinterpret_cast<uint4*>(h->table[i]);
  hm.seq = h->seq;
  hm.tp = h->tp;
  hm.rank = h->rank;
  hm.cap = h->cap;
  // a single CTA: the sequence counter is bumped once, after every row has been merged
  tp_head_merge_kernel<<<1, 128, 0, stream>>>(logits, local_tok, rows, vocab_local, vocab0, hm,
                                              token_out, runtime_status_ptr());
  return static_cast<int>(cudaGetLastError());
}
